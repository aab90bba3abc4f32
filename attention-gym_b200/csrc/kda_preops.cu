// Bandwidth-bound pre-ops of the KDA path: packed-chunk offsets, the bounded gate with its
// chunk-local prefix sum (forward and backward), and the L2 row normalisation.
//
// Replaces (reference files):
//   attn_gym/linear/kda/chunk_scheduler.py:279          chunk offsets prefix kernel
//   attn_gym/linear/kda/fwd/triton/gate_fwd.py:59,220   gate + chunk-local cumsum
//   attn_gym/linear/kda/bwd/cute/gate_bwd_fused.py:153, bwd/triton/gate_bwd.py:141  gate backward
//   attn_gym/linear/kda/fwd/triton/l2norm_fwd.py:22, bwd/triton/l2norm_bwd.py:37    l2norm
//
// All of them stream each element once: a thread owns 4 adjacent channels (8-byte bf16 loads,
// 16-byte fp32 stores), a warp covers a contiguous 256/512-byte row segment.
#include "kda_common.cuh"
#include "kda_timing.cuh"

namespace kda {

// ------------------------------------------------------------------------------------------
// chunk_offsets[i+1] = sum_{s<=i} ceil(len_s / chunk)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) chunk_offsets_kernel(const int32_t* __restrict__ cu,
                                                             int nseq, int chunk,
                                                             int32_t* __restrict__ out) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { s_carry = 0; out[0] = 0; }
  __syncthreads();
  for (int base = 0; base < nseq; base += 1024) {
    int i = base + tid;
    int cnt = 0;
    if (i < nseq) {
      int len = cu[i + 1] - cu[i];
      cnt = len > 0 ? (len + chunk - 1) / chunk : 0;
    }
    int x = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    int incl = x + (warp > 0 ? s_warp[warp - 1] : 0) + s_carry;
    if (i < nseq) out[i + 1] = incl;
    __syncthreads();
    if (tid == 1023) s_carry = incl;
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------
// bounded gate + chunk-local inclusive prefix sum (log2 units)
// ------------------------------------------------------------------------------------------
struct GateParams {
  const void* raw; int dt_raw;
  const float* A_log; const float* dt_bias;
  float* out;                 // forward: cumulative gate, fp32
  const float* d_cum;         // backward: gradient of the cumulative gate
  void* d_raw;                // backward: gradient of the raw gate (dtype of raw)
  float* dA_part; float* dbias_part;  // backward: per-chunk partials [chunks, H*K]
  const int32_t* cu_seqlens; const int32_t* chunk_offsets; int nseq;
  int batch, T, H, K, chunk;
  float lower_bound;
  int* error;                 // device error word of the gate kernels
};

static __device__ int g_gate_error = 0;

__device__ __forceinline__ bool gate_locate(const GateParams& p, int gc, int64_t& token0,
                                            int& valid) {
  if (p.cu_seqlens) {
    if (gc >= p.chunk_offsets[p.nseq]) return false;
    int lo = 0, hi = p.nseq;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (p.chunk_offsets[mid] <= gc) lo = mid; else hi = mid - 1;
    }
    int64_t bos = p.cu_seqlens[lo], eos = p.cu_seqlens[lo + 1];
    token0 = bos + (int64_t)(gc - p.chunk_offsets[lo]) * p.chunk;
    int64_t rem = eos - token0;
    valid = rem >= p.chunk ? p.chunk : (int)rem;
    if (valid > 0 && (bos < 0 || eos > (int64_t)p.batch * p.T)) {
      // a sequence that leaves the packed buffer: skipped and reported, never read or written
      if (threadIdx.x == 0 && p.error) atomicExch(p.error, kOffsetsOutOfRange);
      return false;
    }
    return valid > 0;
  }
  int cpr = (p.T + p.chunk - 1) / p.chunk;
  int row = gc / cpr, lc = gc % cpr;
  if (row >= p.batch) return false;
  int64_t t0 = (int64_t)lc * p.chunk;
  token0 = (int64_t)row * p.T + t0;
  int64_t rem = p.T - t0;
  valid = rem >= p.chunk ? p.chunk : (int)rem;
  return true;
}

__device__ __forceinline__ void load4(const void* p, int dt, int64_t i, float (&x)[4]) {
  if (dt == KDA_BF16) {
    uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  } else if (dt == KDA_F16) {
    const __half* h = reinterpret_cast<const __half*>(p) + i;
    uint2 u = *reinterpret_cast<const uint2*>(h);
    __half2 a = *reinterpret_cast<__half2*>(&u.x), b = *reinterpret_cast<__half2*>(&u.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  } else {
    float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    x[0] = f.x; x[1] = f.y; x[2] = f.z; x[3] = f.w;
  }
}
__device__ __forceinline__ void store4(void* p, int dt, int64_t i, const float (&x)[4]) {
  if (dt == KDA_BF16) {
    uint2 u; u.x = pack_bf16(x[0], x[1]); u.y = pack_bf16(x[2], x[3]);
    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p) + i) = u;
  } else if (dt == KDA_F16) {
    __half2 a = __floats2half2_rn(x[0], x[1]), b = __floats2half2_rn(x[2], x[3]);
    uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p) + i) = u;
  } else {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) =
        make_float4(x[0], x[1], x[2], x[3]);
  }
}

// load4 split in two for software prefetch: raw bits now (8 bytes for 16-bit types, 16 for fp32),
// floats when they are needed, so the warp does not wait on the load in between
__device__ __forceinline__ uint4 load4_raw(const void* p, int dt, int64_t i) {
  if (dt == KDA_F32) return *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned short*>(p) + i);
  return make_uint4(u.x, u.y, 0u, 0u);
}
__device__ __forceinline__ void raw4_to_float(const uint4& r, int dt, float (&x)[4]) {
  if (dt == KDA_BF16) {
    float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  } else if (dt == KDA_F16) {
    __half2 a = *reinterpret_cast<const __half2*>(&r.x), b = *reinterpret_cast<const __half2*>(&r.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  } else {
    x[0] = __uint_as_float(r.x); x[1] = __uint_as_float(r.y);
    x[2] = __uint_as_float(r.z); x[3] = __uint_as_float(r.w);
  }
}

__global__ void __launch_bounds__(128) gate_cumsum_fwd_kernel(const GateParams p) {
  const int HK = p.H * p.K;
  const int f0 = (blockIdx.y * 128 + threadIdx.x) * 4;
  if (f0 >= HK) return;
  int64_t token0; int valid;
  if (!gate_locate(p, blockIdx.x, token0, valid)) return;
  const float a = expf(p.A_log[f0 / p.K]);
  const float4 b4 = *reinterpret_cast<const float4*>(p.dt_bias + f0);
  const float bias[4] = {b4.x, b4.y, b4.z, b4.w};
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  // rows are fetched eight ahead as raw bits (converted when used): the prefix sum is serial over
  // the rows, the loads are not
  constexpr int B = 8;
  uint4 nxt[B];
#pragma unroll
  for (int b = 0; b < B; ++b)
    if (b < valid) nxt[b] = load4_raw(p.raw, p.dt_raw, (token0 + b) * HK + f0);
  for (int r0 = 0; r0 < valid; r0 += B) {
    uint4 cur[B];
#pragma unroll
    for (int b = 0; b < B; ++b) cur[b] = nxt[b];
#pragma unroll
    for (int b = 0; b < B; ++b)
      if (r0 + B + b < valid) nxt[b] = load4_raw(p.raw, p.dt_raw, (token0 + r0 + B + b) * HK + f0);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (r0 + b < valid) {
        float x[4], o[4];
        raw4_to_float(cur[b], p.dt_raw, x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float z = a * (x[j] + bias[j]);
          acc[j] += __fdividef(p.lower_bound, 1.f + __expf(-z));   // 2-ulp intrinsics: 1e-6 relative
          o[j] = acc[j] * kLog2e;
        }
        store4(p.out, KDA_F32, (token0 + r0 + b) * HK + f0, o);
      }
    }
  }
}

constexpr int kGateBwdGroup = 4;   // chunks per block of the backward kernel = chunks per partial row

__global__ void __launch_bounds__(128) gate_cumsum_bwd_kernel(const GateParams p, int num_chunks) {
  const int HK = p.H * p.K;
  const int f0 = (blockIdx.y * 128 + threadIdx.x) * 4;
  if (f0 >= HK) return;
  float pa[4] = {0.f, 0.f, 0.f, 0.f}, pb[4] = {0.f, 0.f, 0.f, 0.f};
  for (int gc = blockIdx.x * kGateBwdGroup; gc < min(num_chunks, (int)(blockIdx.x + 1) * kGateBwdGroup); ++gc) {
  int64_t token0; int valid;
  if (gate_locate(p, gc, token0, valid)) {
    const float a = expf(p.A_log[f0 / p.K]);
    const float4 b4 = *reinterpret_cast<const float4*>(p.dt_bias + f0);
    const float bias[4] = {b4.x, b4.y, b4.z, b4.w};
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // reverse walk, rows fetched four ahead as raw bits (see the forward kernel)
    constexpr int B = 4;
    uint4 nx[B], nd[B];
#pragma unroll
    for (int b = 0; b < B; ++b)
      if (valid - 1 - b >= 0) {
        const int64_t idx = (token0 + valid - 1 - b) * HK + f0;
        nx[b] = load4_raw(p.raw, p.dt_raw, idx);
        nd[b] = load4_raw(p.d_cum, KDA_F32, idx);
      }
    for (int r0 = valid - 1; r0 >= 0; r0 -= B) {
      uint4 cx[B], cd[B];
#pragma unroll
      for (int b = 0; b < B; ++b) { cx[b] = nx[b]; cd[b] = nd[b]; }
#pragma unroll
      for (int b = 0; b < B; ++b)
        if (r0 - B - b >= 0) {
          const int64_t idx = (token0 + r0 - B - b) * HK + f0;
          nx[b] = load4_raw(p.raw, p.dt_raw, idx);
          nd[b] = load4_raw(p.d_cum, KDA_F32, idx);
        }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (r0 - b >= 0) {
          float x[4], d[4], o[4];
          raw4_to_float(cx[b], p.dt_raw, x);
          raw4_to_float(cd[b], KDA_F32, d);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[j] += d[j];
            float z = x[j] + bias[j];
            float s = __fdividef(1.f, 1.f + __expf(-a * z));
            o[j] = acc[j] * kLog2e * p.lower_bound * a * s * (1.f - s);
            pa[j] += o[j] * z;
            pb[j] += o[j];
          }
          store4(p.d_raw, p.dt_raw, (token0 + r0 - b) * HK + f0, o);
        }
      }
    }
  }
  }
  int64_t pidx = (int64_t)blockIdx.x * HK + f0;
  store4(p.dA_part, KDA_F32, pidx, pa);
  store4(p.dbias_part, KDA_F32, pidx, pb);
}

// ------------------------------------------------------------------------------------------
// L2 row normalisation: one warp per row (any width and dtype); vector kernels for 16-bit rows of
// 64 / 128 / 256 elements further down
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) l2norm_fwd_kernel(const void* x, int dt, void* y,
                                                         float* rstd, int64_t rows, int D,
                                                         float eps) {
  const int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float ss = 0.f;
  for (int c = lane * 4; c < D; c += 128) {
    float v[4];
    load4(x, dt, row * D + c, v);
    ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  float r = rsqrtf(ss + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  for (int c = lane * 4; c < D; c += 128) {
    float v[4];
    load4(x, dt, row * D + c, v);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] *= r;
    store4(y, dt, row * D + c, v);
  }
}

__global__ void __launch_bounds__(256) l2norm_bwd_kernel(const void* y, const float* rstd,
                                                         const void* dy, int dt, void* dx,
                                                         int64_t rows, int D) {
  const int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float dot = 0.f;
  for (int c = lane * 4; c < D; c += 128) {
    float a[4], b[4];
    load4(y, dt, row * D + c, a);
    load4(dy, dt, row * D + c, b);
    dot += a[0] * b[0] + a[1] * b[1] + a[2] * b[2] + a[3] * b[3];
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
  float r = rstd[row];
  for (int c = lane * 4; c < D; c += 128) {
    float a[4], b[4], o[4];
    load4(y, dt, row * D + c, a);
    load4(dy, dt, row * D + c, b);
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = r * (b[j] - a[j] * dot);
    store4(dx, dt, row * D + c, o);
  }
}

// 16-bit rows of 64 / 128 / 256 elements: LPR = D / 8 lanes share a row (one 16-byte vector each), a
// warp holds 32 / LPR rows per slot and four slots in flight; every element is read once and stays
// in registers between the reduction and the scaling.
template <int LPR>
__global__ void __launch_bounds__(256) l2norm_fwd_vec_kernel(const uint4* __restrict__ x, int dt,
                                                             uint4* __restrict__ y, float* rstd,
                                                             int64_t rows, float eps) {
  constexpr int RPS = 32 / LPR, SLOTS = 4;
  const int lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * (RPS * SLOTS) + lane / LPR;
  uint4 v[SLOTS];
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int64_t row = row0 + s * RPS;
    if (row < rows) v[s] = x[row * LPR + lane % LPR];
  }
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int64_t row = row0 + s * RPS;
    float f[8];
    float ss = 0.f;
    if (row < rows) {
      raw8_to_float(v[s], dt, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
#pragma unroll
    for (int d = LPR / 2; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if (row < rows) {
      const float r = rsqrtf(ss + eps);
      if (lane % LPR == 0 && rstd) rstd[row] = r;
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= r;
      y[row * LPR + lane % LPR] = float8_to_raw(f, dt);
    }
  }
}

template <int LPR>
__global__ void __launch_bounds__(256) l2norm_bwd_vec_kernel(const uint4* __restrict__ y,
                                                             const float* __restrict__ rstd,
                                                             const uint4* __restrict__ dy, int dt,
                                                             uint4* __restrict__ dx, int64_t rows) {
  constexpr int RPS = 32 / LPR, SLOTS = 4;
  const int lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * (RPS * SLOTS) + lane / LPR;
  uint4 a[SLOTS], b[SLOTS];
  float rs[SLOTS];
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int64_t row = row0 + s * RPS;
    if (row < rows) {
      a[s] = y[row * LPR + lane % LPR];
      b[s] = dy[row * LPR + lane % LPR];
      rs[s] = rstd[row];
    }
  }
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int64_t row = row0 + s * RPS;
    float fy[8], fd[8];
    float dot = 0.f;
    if (row < rows) {
      raw8_to_float(a[s], dt, fy);
      raw8_to_float(b[s], dt, fd);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot = fmaf(fy[j], fd[j], dot);
    }
#pragma unroll
    for (int d = LPR / 2; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
    if (row < rows) {
#pragma unroll
      for (int j = 0; j < 8; ++j) fd[j] = rs[s] * (fd[j] - fy[j] * dot);
      dx[row * LPR + lane % LPR] = float8_to_raw(fd, dt);
    }
  }
}

// dA_log[h] = sum over partial rows and channels, d_dt_bias[h, c] = sum over partial rows; every sum
// in a fixed order.  Blocks 0 .. ceil(HK / 32) - 1 own 32 channels of d_dt_bias each: eight row groups
// side by side, sixteen rows of loads in flight per thread.  The H blocks after them own one head of
// dA_log: the head's rows x K slice is walked by the whole block, sixteen loads in flight per thread.
__global__ void __launch_bounds__(256) gate_bwd_reduce_kernel(const float* __restrict__ pa,
                                                              const float* __restrict__ pb, int64_t rows,
                                                              int H, int K, float* __restrict__ dA,
                                                              float* __restrict__ dbias) {
  __shared__ float s_part[256];
  const int tid = threadIdx.x, lane = tid & 31, grp = tid >> 5;
  const int64_t HK = (int64_t)H * K;
  const int col_blocks = (int)((HK + 31) / 32);
  if ((int)blockIdx.x < col_blocks) {
    const int64_t ch = (int64_t)blockIdx.x * 32 + lane;
    float b = 0.f;
    if (ch < HK) {
      const float* q = pb + ch;
      int64_t r = grp;
      for (; r + 15 * 8 < rows; r += 16 * 8) {
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = q[(r + 8 * u) * HK];
#pragma unroll
        for (int u = 0; u < 16; ++u) b += v[u];
      }
      for (; r < rows; r += 8) b += q[r * HK];
    }
    s_part[tid] = b;
    __syncthreads();
    if (grp == 0 && ch < HK) {
      float t = 0.f;
#pragma unroll
      for (int g = 0; g < 8; ++g) t += s_part[32 * g + lane];
      dbias[ch] = t;
    }
    return;
  }
  const int h = (int)blockIdx.x - col_blocks;
  const float* q = pa + (int64_t)h * K;
  const int64_t n = rows * K;
  float a = 0.f;
  int64_t e = tid;
  for (; e + 15 * 256 < n; e += 16 * 256) {
    float v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int64_t i = e + 256 * u, r = i / K;
      v[u] = q[r * HK + (i - r * K)];
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) a += v[u];
  }
  for (; e < n; e += 256) {
    const int64_t r = e / K;
    a += q[r * HK + (e - r * K)];
  }
  s_part[tid] = a;
  __syncthreads();
  if (tid < 32) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) t += s_part[32 * g + tid];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
    if (tid == 0) dA[h] = t;
  }
}

static int check_launch() { return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH; }

int gate_error_word() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gate_error, sizeof(int)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(g_gate_error, &zero, sizeof(int));
  return v;
}

}  // namespace kda

extern "C" int kda_prepare_chunk_offsets(const int32_t* cu_seqlens, int nseq, int chunk_size,
                                         int32_t* chunk_offsets, void* stream) {
  if (!cu_seqlens || !chunk_offsets || nseq < 1 || chunk_size < 1) return KDA_ERR_ARG;
  kda::chunk_offsets_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(cu_seqlens, nseq, chunk_size,
                                                                  chunk_offsets);
  return kda::check_launch();
}

static int gate_common(kda::GateParams& p, const int32_t* cu, const int32_t* co, int nseq,
                       int batch, int tokens, int heads, int dim, int chunk, int64_t chunks) {
  if (heads <= 0 || dim <= 0 || dim % 4 || chunk < 1 || batch < 1 || tokens < 1) return KDA_ERR_ARG;
  if ((cu != nullptr) != (co != nullptr)) return KDA_ERR_ARG;
  if (cu && batch != 1) return KDA_ERR_ARG;
  if (chunks > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.nseq = nseq;
  p.batch = batch; p.T = tokens; p.H = heads; p.K = dim; p.chunk = chunk;
  p.error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), kda::g_gate_error) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  return KDA_OK;
}

extern "C" int kda_gate_cumsum_fwd(const void* raw_gate, int dt_raw, const float* A_log,
                                   const float* dt_bias, float* out, const int32_t* cu_seqlens,
                                   const int32_t* chunk_offsets, int nseq, int batch, int tokens,
                                   int heads, int dim, int chunk_size, float lower_bound,
                                   int64_t num_chunks, void* stream) {
  if (!raw_gate || !A_log || !dt_bias || !out) return KDA_ERR_ARG;
  kda::GateParams p{};
  int rc = gate_common(p, cu_seqlens, chunk_offsets, nseq, batch, tokens, heads, dim, chunk_size,
                       num_chunks);
  if (rc) return rc;
  if (num_chunks == 0) return KDA_OK;
  p.raw = raw_gate; p.dt_raw = dt_raw; p.A_log = A_log; p.dt_bias = dt_bias; p.out = out;
  p.lower_bound = lower_bound;
  dim3 grid((unsigned)num_chunks, (unsigned)((heads * dim / 4 + 127) / 128));
  kda::StageScope timing(kda::kStageGateFwd, (cudaStream_t)stream);
  kda::gate_cumsum_fwd_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(p);
  return kda::check_launch();
}

extern "C" int64_t kda_gate_bwd_partial_rows(int64_t num_chunks) {
  return (num_chunks + kda::kGateBwdGroup - 1) / kda::kGateBwdGroup;
}

extern "C" int kda_gate_cumsum_bwd(const void* raw_gate, int dt_raw, const float* A_log,
                                   const float* dt_bias, const float* d_cumulative, void* d_raw,
                                   float* dA_partial, float* dbias_partial,
                                   const int32_t* cu_seqlens, const int32_t* chunk_offsets,
                                   int nseq, int batch, int tokens, int heads, int dim,
                                   int chunk_size, float lower_bound, int64_t num_chunks,
                                   void* stream) {
  if (!raw_gate || !A_log || !dt_bias || !d_cumulative || !d_raw || !dA_partial || !dbias_partial)
    return KDA_ERR_ARG;
  kda::GateParams p{};
  int rc = gate_common(p, cu_seqlens, chunk_offsets, nseq, batch, tokens, heads, dim, chunk_size,
                       num_chunks);
  if (rc) return rc;
  if (num_chunks == 0) return KDA_OK;
  p.raw = raw_gate; p.dt_raw = dt_raw; p.A_log = A_log; p.dt_bias = dt_bias;
  p.d_cum = d_cumulative; p.d_raw = d_raw; p.dA_part = dA_partial; p.dbias_part = dbias_partial;
  p.lower_bound = lower_bound;
  dim3 grid((unsigned)kda_gate_bwd_partial_rows(num_chunks), (unsigned)((heads * dim / 4 + 127) / 128));
  kda::StageScope timing(kda::kStageGateBwd, (cudaStream_t)stream);
  kda::gate_cumsum_bwd_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(p, (int)num_chunks);
  return kda::check_launch();
}

// Sums the partial rows kda_gate_cumsum_bwd wrote: dA_log [heads], d_dt_bias [heads, dim] (fp32).
extern "C" int kda_gate_bwd_reduce(const float* dA_partial, const float* dbias_partial, int64_t rows,
                                   int heads, int dim, float* dA_log, float* d_dt_bias, void* stream) {
  if (!dA_partial || !dbias_partial || !dA_log || !d_dt_bias || rows < 0 || heads < 1 || dim < 1)
    return KDA_ERR_ARG;
  const unsigned blocks = (unsigned)(((int64_t)heads * dim + 31) / 32 + heads);
  kda::gate_bwd_reduce_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      dA_partial, dbias_partial, rows, heads, dim, dA_log, d_dt_bias);
  return kda::check_launch();
}

extern "C" int kda_l2norm_fwd(const void* x, int dtype, void* y, float* rstd, int64_t rows,
                              int dim, float eps, void* stream) {
  if (!x || !y || rows < 0 || dim <= 0 || dim % 4) return KDA_ERR_ARG;
  if (rows == 0) return KDA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = dtype != KDA_F32 && (dim == 64 || dim == 128 || dim == 256) &&
                   ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0;
  if (vec) {
    const int lpr = dim / 8, rows_per_block = 8 * (32 / lpr) * 4;
    const unsigned blocks = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    uint4* yv = reinterpret_cast<uint4*>(y);
    if (lpr == 8) kda::l2norm_fwd_vec_kernel<8><<<blocks, 256, 0, s>>>(xv, dtype, yv, rstd, rows, eps);
    else if (lpr == 16) kda::l2norm_fwd_vec_kernel<16><<<blocks, 256, 0, s>>>(xv, dtype, yv, rstd, rows, eps);
    else kda::l2norm_fwd_vec_kernel<32><<<blocks, 256, 0, s>>>(xv, dtype, yv, rstd, rows, eps);
    return kda::check_launch();
  }
  kda::l2norm_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(x, dtype, y, rstd, rows, dim, eps);
  return kda::check_launch();
}

extern "C" int kda_l2norm_bwd(const void* y, const float* rstd, const void* dy, int dtype, void* dx,
                              int64_t rows, int dim, void* stream) {
  if (!y || !rstd || !dy || !dx || rows < 0 || dim <= 0 || dim % 4) return KDA_ERR_ARG;
  if (rows == 0) return KDA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = dtype != KDA_F32 && (dim == 64 || dim == 128 || dim == 256) &&
                   ((uintptr_t)y & 15) == 0 && ((uintptr_t)dy & 15) == 0 && ((uintptr_t)dx & 15) == 0;
  if (vec) {
    const int lpr = dim / 8, rows_per_block = 8 * (32 / lpr) * 4;
    const unsigned blocks = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    const uint4* yv = reinterpret_cast<const uint4*>(y);
    const uint4* dv = reinterpret_cast<const uint4*>(dy);
    uint4* xv = reinterpret_cast<uint4*>(dx);
    if (lpr == 8) kda::l2norm_bwd_vec_kernel<8><<<blocks, 256, 0, s>>>(yv, rstd, dv, dtype, xv, rows);
    else if (lpr == 16) kda::l2norm_bwd_vec_kernel<16><<<blocks, 256, 0, s>>>(yv, rstd, dv, dtype, xv, rows);
    else kda::l2norm_bwd_vec_kernel<32><<<blocks, 256, 0, s>>>(yv, rstd, dv, dtype, xv, rows);
    return kda::check_launch();
  }
  kda::l2norm_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(y, rstd, dy, dtype, dx, rows, dim);
  return kda::check_launch();
}
