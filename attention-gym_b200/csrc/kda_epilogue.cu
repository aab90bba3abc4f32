// Output epilogue of the KDA layer in one pass:  y = rms_norm(o) * weight * sigmoid(gate_logits)
// with rms_norm(o) = o * rsqrt(mean(o^2) + eps) over the head dimension, and its backward.
//
// The reference module runs this as three elementwise launches on the output of chunk_kda
// (examples/kda_training.py:507-517 F.rms_norm, :519-532 sigmoid of the gate projection,
// :535-539 their product), i.e. 14 bytes per element in bf16; fused it is 6 (forward) and 10
// (backward: o, logits, dy in; d_o, d_logits out), both streamed once.
//
// 16-bit rows of 64 / 128 / 256 elements: LPR = D / 8 lanes share a row, one 16-byte vector each,
// four row slots in flight per warp, raw bits prefetched and converted when they are used.  The
// weight gradient is accumulated in registers over a grid-stride loop and leaves the kernel as one
// partial row per block (summed by the caller): deterministic, no atomics.
// Any other width (multiple of 4, at most 512) or fp32 goes through the warp-per-row kernels.
#include "kda_common.cuh"
#include "kda_timing.cuh"

namespace kda {

__device__ __forceinline__ float sigmoid_fast(float z) { return __fdividef(1.f, 1.f + __expf(-z)); }

template <int LPR>
__global__ void __launch_bounds__(256) out_gate_fwd_vec_kernel(const uint4* __restrict__ x,
                                                               const uint4* __restrict__ z,
                                                               const float* __restrict__ weight,
                                                               int dt, uint4* __restrict__ y,
                                                               int64_t rows, float eps) {
  constexpr int RPS = 32 / LPR, SLOTS = 4;
  const int lane = threadIdx.x & 31, sub = lane % LPR;
  const int64_t row0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * (RPS * SLOTS) + lane / LPR;
  uint4 vx[SLOTS], vz[SLOTS];
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int64_t row = row0 + s * RPS;
    if (row < rows) { vx[s] = x[row * LPR + sub]; vz[s] = z[row * LPR + sub]; }
  }
  float w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = weight[sub * 8 + j];
  constexpr float inv_d = 1.f / (LPR * 8);
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int64_t row = row0 + s * RPS;
    float f[8], g[8];
    float ss = 0.f;
    if (row < rows) {
      raw8_to_float(vx[s], dt, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
#pragma unroll
    for (int d = LPR / 2; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if (row < rows) {
      const float r = rsqrtf(ss * inv_d + eps);
      raw8_to_float(vz[s], dt, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * r * w[j] * sigmoid_fast(g[j]);
      y[row * LPR + sub] = float8_to_raw(f, dt);
    }
  }
}

// Backward.  With n = o * rstd, s = sigmoid(z), a = dy * w:
//   d_z = a * n * s * (1 - s);   d_n = a * s;   d_o = rstd * (d_n - n * mean(d_n * n));
//   d_w[c] = sum over rows of dy * n * s.
template <int LPR>
__global__ void __launch_bounds__(256) out_gate_bwd_vec_kernel(const uint4* __restrict__ x,
                                                               const uint4* __restrict__ z,
                                                               const uint4* __restrict__ dy,
                                                               const float* __restrict__ weight,
                                                               int dt, uint4* __restrict__ dx,
                                                               uint4* __restrict__ dz,
                                                               float* __restrict__ dw_partial,
                                                               int64_t rows, float eps) {
  constexpr int RPS = 32 / LPR, SLOTS = 2, D = LPR * 8;
  __shared__ float s_dw[8 * RPS][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane % LPR;
  float w[8], dw[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { w[j] = weight[sub * 8 + j]; dw[j] = 0.f; }
  constexpr float inv_d = 1.f / D;
  const int64_t stride = (int64_t)gridDim.x * 8 * (RPS * SLOTS);
  int64_t row0 = ((int64_t)blockIdx.x * 8 + warp) * (RPS * SLOTS) + lane / LPR;
  uint4 vx[SLOTS], vz[SLOTS], vd[SLOTS];
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int64_t row = row0 + s * RPS;
    if (row < rows) { vx[s] = x[row * LPR + sub]; vz[s] = z[row * LPR + sub]; vd[s] = dy[row * LPR + sub]; }
  }
  for (; row0 - lane / LPR < rows; row0 += stride) {
    uint4 cx[SLOTS], cz[SLOTS], cd[SLOTS];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) { cx[s] = vx[s]; cz[s] = vz[s]; cd[s] = vd[s]; }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {      // raw bits of the next group: in flight during the math
      const int64_t row = row0 + stride + s * RPS;
      if (row < rows) { vx[s] = x[row * LPR + sub]; vz[s] = z[row * LPR + sub]; vd[s] = dy[row * LPR + sub]; }
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int64_t row = row0 + s * RPS;
      const bool live = row < rows;
      float f[8], g[8], a[8];
      float ss = 0.f, dot = 0.f;
      if (live) {
        raw8_to_float(cx[s], dt, f);
        raw8_to_float(cz[s], dt, g);
        raw8_to_float(cd[s], dt, a);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          g[j] = sigmoid_fast(g[j]);
          ss = fmaf(f[j], f[j], ss);
          dot = fmaf(a[j] * w[j] * g[j], f[j], dot);       // sum of d_n * o  (= sum d_n * n / rstd)
        }
      }
#pragma unroll
      for (int d = LPR / 2; d > 0; d >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, d);
        dot += __shfl_xor_sync(0xffffffffu, dot, d);
      }
      if (live) {
        const float r = rsqrtf(ss * inv_d + eps);
        const float c = dot * r * r * inv_d;                // mean(d_n * n) * rstd, per unit of o
        float ox[8], oz[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = f[j] * r, dyn = a[j] * n;          // dy * n
          dw[j] = fmaf(dyn, g[j], dw[j]);
          oz[j] = dyn * w[j] * g[j] * (1.f - g[j]);
          ox[j] = r * (a[j] * w[j] * g[j] - f[j] * c);
        }
        dx[row * LPR + sub] = float8_to_raw(ox, dt);
        dz[row * LPR + sub] = float8_to_raw(oz, dt);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_dw[warp * RPS + lane / LPR][sub * 8 + j] = dw[j];
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += 256) {
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < 8 * RPS; ++r) acc += s_dw[r][c];
    dw_partial[(int64_t)blockIdx.x * D + c] = acc;
  }
}

// Any dtype, any width that is a multiple of 4 up to 512: one warp per row.
constexpr int kEpiMaxD = 512;

__global__ void __launch_bounds__(256) out_gate_fwd_kernel(const void* x, const void* z,
                                                           const float* __restrict__ weight, int dt,
                                                           void* y, int64_t rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) { const float v = load_as_float(x, dt, row * D + c); ss = fmaf(v, v, ss); }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  const float r = rsqrtf(ss / D + eps);
  for (int c = lane; c < D; c += 32) {
    const float v = load_as_float(x, dt, row * D + c), g = load_as_float(z, dt, row * D + c);
    store_from_float(y, dt, row * D + c, v * r * weight[c] / (1.f + expf(-g)));
  }
}

__global__ void __launch_bounds__(256) out_gate_bwd_kernel(const void* x, const void* z, const void* dy,
                                                           const float* __restrict__ weight, int dt,
                                                           void* dx, void* dz, float* dw_partial,
                                                           int64_t rows, int D, float eps) {
  __shared__ float s_dw[8][kEpiMaxD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float dw[kEpiMaxD / 32];
#pragma unroll
  for (int i = 0; i < kEpiMaxD / 32; ++i) dw[i] = 0.f;
  for (int64_t row = (int64_t)blockIdx.x * 8 + warp; row < rows; row += (int64_t)gridDim.x * 8) {
    float ss = 0.f, dot = 0.f;
    for (int c = lane; c < D; c += 32) {
      const float v = load_as_float(x, dt, row * D + c);
      const float s = 1.f / (1.f + expf(-load_as_float(z, dt, row * D + c)));
      ss = fmaf(v, v, ss);
      dot = fmaf(load_as_float(dy, dt, row * D + c) * weight[c] * s, v, dot);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, d);
      dot += __shfl_xor_sync(0xffffffffu, dot, d);
    }
    const float r = rsqrtf(ss / D + eps), cc = dot * r * r / D;
#pragma unroll
    for (int i = 0; i < kEpiMaxD / 32; ++i) {
      const int c = lane + 32 * i;
      if (c < D) {
        const float v = load_as_float(x, dt, row * D + c);
        const float s = 1.f / (1.f + expf(-load_as_float(z, dt, row * D + c)));
        const float a = load_as_float(dy, dt, row * D + c), dyn = a * v * r;
        dw[i] = fmaf(dyn, s, dw[i]);
        store_from_float(dz, dt, row * D + c, dyn * weight[c] * s * (1.f - s));
        store_from_float(dx, dt, row * D + c, r * (a * weight[c] * s - v * cc));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kEpiMaxD / 32; ++i) s_dw[warp][lane + 32 * i] = dw[i];
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += 256) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) acc += s_dw[w][c];
    dw_partial[(int64_t)blockIdx.x * D + c] = acc;
  }
}

static bool epilogue_vec_ok(int dtype, int dim, const void* a, const void* b, const void* c,
                            const void* d, const void* e) {
  const uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d | (uintptr_t)e;
  return dtype != KDA_F32 && (dim == 64 || dim == 128 || dim == 256) && (bits & 15) == 0;
}

}  // namespace kda

extern "C" int kda_output_gate_fwd(const void* o, const void* gate_logits, const float* weight,
                                   int dtype, void* y, int64_t rows, int dim, float eps,
                                   void* stream) {
  if (!o || !gate_logits || !weight || !y || rows < 0 || dim <= 0 || dim % 4) return KDA_ERR_ARG;
  if (dim > kda::kEpiMaxD) return KDA_ERR_UNSUPPORTED;
  if (rows == 0) return KDA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  kda::StageScope timing(kda::kStageEpilogue, s);
  if (kda::epilogue_vec_ok(dtype, dim, o, gate_logits, y, nullptr, nullptr)) {
    const int lpr = dim / 8, rows_per_block = 8 * (32 / lpr) * 4;
    const unsigned blocks = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    const uint4 *xv = reinterpret_cast<const uint4*>(o), *zv = reinterpret_cast<const uint4*>(gate_logits);
    uint4* yv = reinterpret_cast<uint4*>(y);
    if (lpr == 8) kda::out_gate_fwd_vec_kernel<8><<<blocks, 256, 0, s>>>(xv, zv, weight, dtype, yv, rows, eps);
    else if (lpr == 16) kda::out_gate_fwd_vec_kernel<16><<<blocks, 256, 0, s>>>(xv, zv, weight, dtype, yv, rows, eps);
    else kda::out_gate_fwd_vec_kernel<32><<<blocks, 256, 0, s>>>(xv, zv, weight, dtype, yv, rows, eps);
  } else {
    kda::out_gate_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(o, gate_logits, weight, dtype, y,
                                                                        rows, dim, eps);
  }
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

// Rows of the weight-gradient partial buffer ([rows, dim] fp32) that kda_output_gate_bwd fills.
extern "C" int64_t kda_output_gate_bwd_partial_rows(int64_t rows) {
  const int64_t want = (rows + 63) / 64;
  return want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want);
}

extern "C" int kda_output_gate_bwd(const void* o, const void* gate_logits, const void* dy,
                                   const float* weight, int dtype, void* d_o, void* d_logits,
                                   float* dw_partial, int64_t rows, int dim, float eps,
                                   void* stream) {
  if (!o || !gate_logits || !dy || !weight || !d_o || !d_logits || !dw_partial || rows < 0 ||
      dim <= 0 || dim % 4)
    return KDA_ERR_ARG;
  if (dim > kda::kEpiMaxD) return KDA_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)kda_output_gate_bwd_partial_rows(rows);
  kda::StageScope timing(kda::kStageEpilogue, s);
  if (kda::epilogue_vec_ok(dtype, dim, o, gate_logits, dy, d_o, d_logits)) {
    const int lpr = dim / 8;
    const uint4 *xv = reinterpret_cast<const uint4*>(o), *zv = reinterpret_cast<const uint4*>(gate_logits),
                *dv = reinterpret_cast<const uint4*>(dy);
    uint4 *ox = reinterpret_cast<uint4*>(d_o), *oz = reinterpret_cast<uint4*>(d_logits);
    if (lpr == 8) kda::out_gate_bwd_vec_kernel<8><<<blocks, 256, 0, s>>>(xv, zv, dv, weight, dtype, ox, oz, dw_partial, rows, eps);
    else if (lpr == 16) kda::out_gate_bwd_vec_kernel<16><<<blocks, 256, 0, s>>>(xv, zv, dv, weight, dtype, ox, oz, dw_partial, rows, eps);
    else kda::out_gate_bwd_vec_kernel<32><<<blocks, 256, 0, s>>>(xv, zv, dv, weight, dtype, ox, oz, dw_partial, rows, eps);
  } else {
    kda::out_gate_bwd_kernel<<<blocks, 256, 0, s>>>(o, gate_logits, dy, weight, dtype, d_o, d_logits,
                                                    dw_partial, rows, dim, eps);
  }
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}
