// Causal depthwise short convolution with optional fused SiLU: forward, decode step, backward.
//
//   y[t, c] = act( sum_{j < W} w[c, j] * x[t - (W-1) + j, c] ),  positions before the start of a
//   sequence read the [W-1, C] history (oldest first) or zero.
//
// Replaces the reference's CuTeDSL kernels in attn_gym/linear/kda/short_conv/cute.py:
//   CausalConv1dSiluForward :296, ...Decode :470, ...InputGradient :582,
//   ...WeightGradientPartials :791, ...InitialStateGradient :1960.
// HBM-bound streaming kernels: a thread owns 16 bytes of adjacent channels and walks a run of
// consecutive tokens with a W-wide register window, so every element is read once per pass
// (plus a W-1 halo per run).
#include "kda_common.cuh"

namespace kda {

constexpr int WMAX = 8;     // widest supported filter
constexpr int CONV_TT = 32; // tokens per thread run

template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename T, int N>
__device__ __forceinline__ void ldv(const T* p, float (&x)[N]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) x[i] = (float)e[i];
}
template <typename T, int N>
__device__ __forceinline__ void stv(T* p, const float (&x)[N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = (T)x[i];
  *reinterpret_cast<uint4*>(p) = raw;
}

struct ConvParams {
  const void* x; const void* w; void* y;
  const void* state;            // [nseq, W-1, C] initial history or NULL
  const void* dy; void* dx; float* dpre;   // backward
  float* dw_part; float* dstate;           // backward: [blocks, C, W] partials; fp32 [nseq, W-1, C]
  const int32_t* cu_seqlens; int nseq;
  int batch, T, C, W, act;      // act: 0 none, 1 silu
};

// sequence that holds token t (packed) -- upper_bound(cu, t) - 1
__device__ __forceinline__ int find_seq(const int32_t* cu, int nseq, int64_t t) {
  int lo = 0, hi = nseq;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Walks tokens [t0, t1) of one thread run, maintaining the window win[j] = x[t-(W-1)+j].
// `body(t, seq, bos, eos, win)` is called once per active token with the full window loaded.
template <typename T, typename F>
__device__ __forceinline__ void conv_walk(const ConvParams& p, int64_t t0, int64_t t1, int c0,
                                          F&& body) {
  constexpr int N = VecOf<T>::N;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* st = reinterpret_cast<const T*>(p.state);
  const int W = p.W, C = p.C;
  float win[WMAX][N];
  int seq; int64_t bos, eos;
  if (p.cu_seqlens) {
    if (t0 >= p.cu_seqlens[p.nseq]) return;
    seq = find_seq(p.cu_seqlens, p.nseq, t0);
    bos = p.cu_seqlens[seq]; eos = p.cu_seqlens[seq + 1];
    if (t1 > p.cu_seqlens[p.nseq]) t1 = p.cu_seqlens[p.nseq];
  } else {
    seq = (int)(t0 / p.T); bos = (int64_t)seq * p.T; eos = bos + p.T;
  }
  bool fresh = true;
  for (int64_t t = t0; t < t1; ++t) {
    while (t >= eos) { ++seq; bos = eos; eos = p.cu_seqlens ? p.cu_seqlens[seq + 1] : bos + p.T; fresh = true; }
    if (fresh) {
#pragma unroll
      for (int j = 0; j < WMAX - 1; ++j) {
        if (j < W - 1) {
          int64_t pos = t - (W - 1) + j;
          if (pos >= bos) ldv<T, N>(x + pos * C + c0, win[j]);
          else if (st) ldv<T, N>(st + ((int64_t)seq * (W - 1) + (pos - bos + W - 1)) * C + c0, win[j]);
          else {
#pragma unroll
            for (int i = 0; i < N; ++i) win[j][i] = 0.f;
          }
        }
      }
      fresh = false;
    }
#pragma unroll
    for (int j = 0; j < WMAX; ++j)
      if (j == W - 1) ldv<T, N>(x + t * C + c0, win[j]);
    body(t, seq, bos, eos, win);
#pragma unroll
    for (int j = 0; j < WMAX - 1; ++j)
      if (j < W - 1) {
#pragma unroll
        for (int i = 0; i < N; ++i) win[j][i] = win[j + 1][i];
      }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) conv_fwd_kernel(const ConvParams p) {
  constexpr int N = VecOf<T>::N;
  const int c0 = (blockIdx.y * 128 + threadIdx.x) * N;
  if (c0 >= p.C) return;
  const int64_t total = (int64_t)p.batch * p.T;
  int64_t t0, t1;
  if (p.cu_seqlens) { t0 = (int64_t)blockIdx.x * CONV_TT; t1 = min(t0 + CONV_TT, total); }
  else {  // runs never straddle dense rows
    int rpr = (p.T + CONV_TT - 1) / CONV_TT;
    int row = blockIdx.x / rpr, rb = blockIdx.x % rpr;
    t0 = (int64_t)row * p.T + (int64_t)rb * CONV_TT;
    t1 = min(t0 + CONV_TT, (int64_t)(row + 1) * p.T);
  }
  const T* w = reinterpret_cast<const T*>(p.w);
  float wr[N][WMAX];
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j < WMAX; ++j) wr[i][j] = j < p.W ? (float)w[(int64_t)(c0 + i) * p.W + j] : 0.f;
  T* y = reinterpret_cast<T*>(p.y);
  conv_walk<T>(p, t0, t1, c0, [&](int64_t t, int, int64_t, int64_t, float (&win)[WMAX][N]) {
    float o[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < WMAX; ++j)
        if (j < p.W) s += wr[i][j] * win[j][i];
      o[i] = p.act ? s / (1.f + expf(-s)) : s;
    }
    stv<T, N>(y + t * p.C + c0, o);
  });
}

// backward pass A: dpre = dy * act'(pre) (fp32 scratch), weight-gradient partials, history gradient
template <typename T>
__global__ void __launch_bounds__(256) conv_bwd_pre_kernel(const ConvParams p) {
  constexpr int N = VecOf<T>::N;
  __shared__ float s_red[8][32][N];
  const int cx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = (blockIdx.y * 32 + cx) * N;
  const bool live = c0 < p.C;
  const int64_t total = (int64_t)p.batch * p.T;
  int64_t t0, t1;
  if (p.cu_seqlens) { t0 = ((int64_t)blockIdx.x * 8 + ty) * CONV_TT; t1 = min(t0 + CONV_TT, total); }
  else {
    int rpr = (p.T + 8 * CONV_TT - 1) / (8 * CONV_TT);
    int row = blockIdx.x / rpr, rb = blockIdx.x % rpr;
    t0 = (int64_t)row * p.T + ((int64_t)rb * 8 + ty) * CONV_TT;
    t1 = min(t0 + CONV_TT, (int64_t)(row + 1) * p.T);
  }
  float dwacc[N][WMAX];
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j < WMAX; ++j) dwacc[i][j] = 0.f;
  if (live && t0 < t1) {
    const T* w = reinterpret_cast<const T*>(p.w);
    const T* dy = reinterpret_cast<const T*>(p.dy);
    float wr[N][WMAX];
#pragma unroll
    for (int i = 0; i < N; ++i)
#pragma unroll
      for (int j = 0; j < WMAX; ++j) wr[i][j] = j < p.W ? (float)w[(int64_t)(c0 + i) * p.W + j] : 0.f;
    conv_walk<T>(p, t0, t1, c0, [&](int64_t t, int seq, int64_t bos, int64_t, float (&win)[WMAX][N]) {
      float g[N], d[N];
      ldv<T, N>(dy + t * p.C + c0, g);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < WMAX; ++j)
          if (j < p.W) s += wr[i][j] * win[j][i];
        float dact = 1.f;
        if (p.act) { float sg = 1.f / (1.f + expf(-s)); dact = sg * (1.f + s * (1.f - sg)); }
        d[i] = g[i] * dact;
#pragma unroll
        for (int j = 0; j < WMAX; ++j)
          if (j < p.W) dwacc[i][j] += d[i] * win[j][i];
      }
#pragma unroll
      for (int i = 0; i < N; i += 4)
        *reinterpret_cast<float4*>(p.dpre + t * p.C + c0 + i) = make_float4(d[i], d[i + 1], d[i + 2], d[i + 3]);
      if (p.dstate && t - bos < p.W - 1) {  // window slots that fall before the sequence start
#pragma unroll
        for (int j = 0; j < WMAX - 1; ++j) {
          int64_t pos = t - (p.W - 1) + j;
          if (j < p.W - 1 && pos < bos) {
#pragma unroll
            for (int i = 0; i < N; ++i)
              atomicAdd(p.dstate + ((int64_t)seq * (p.W - 1) + (pos - bos + p.W - 1)) * p.C + c0 + i,
                        wr[i][j] * d[i]);
          }
        }
      }
    });
  }
  // reduce the 8 time slices of the block, then one partial per (block, channel, tap)
  for (int j = 0; j < p.W; ++j) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float val = 0.f;
#pragma unroll
      for (int jj = 0; jj < WMAX; ++jj) if (jj == j) val = dwacc[i][jj];
      s_red[ty][cx][i] = val;
    }
    __syncthreads();
    if (ty == 0 && live) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        float s = 0.f;
#pragma unroll
        for (int y = 0; y < 8; ++y) s += s_red[y][cx][i];
        p.dw_part[((int64_t)blockIdx.x * p.C + c0 + i) * p.W + j] = s;
      }
    }
    __syncthreads();
  }
}

// backward pass B: dx[t] = sum_j w[j] dpre[t + (W-1) - j] over tokens of the same sequence
template <typename T>
__global__ void __launch_bounds__(128) conv_bwd_dx_kernel(const ConvParams p) {
  constexpr int N = VecOf<T>::N;
  const int c0 = (blockIdx.y * 128 + threadIdx.x) * N;
  if (c0 >= p.C) return;
  int64_t total = (int64_t)p.batch * p.T;
  if (p.cu_seqlens) total = min(total, (int64_t)p.cu_seqlens[p.nseq]);
  int64_t t0 = (int64_t)blockIdx.x * CONV_TT, t1 = min(t0 + CONV_TT, total);
  if (t0 >= t1) return;
  const T* w = reinterpret_cast<const T*>(p.w);
  float wr[N][WMAX];
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j < WMAX; ++j) wr[i][j] = j < p.W ? (float)w[(int64_t)(c0 + i) * p.W + j] : 0.f;
  int seq; int64_t eos;
  if (p.cu_seqlens) { seq = find_seq(p.cu_seqlens, p.nseq, t0); eos = p.cu_seqlens[seq + 1]; }
  else { seq = (int)(t0 / p.T); eos = (int64_t)(seq + 1) * p.T; }
  T* dx = reinterpret_cast<T*>(p.dx);
  for (int64_t t = t0; t < t1; ++t) {
    while (t >= eos) { ++seq; eos = p.cu_seqlens ? p.cu_seqlens[seq + 1] : eos + p.T; }
    float o[N];
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] = 0.f;
    for (int j = 0; j < p.W; ++j) {
      int64_t src = t + (p.W - 1) - j;
      if (src < eos) {
#pragma unroll
        for (int i = 0; i < N; i += 4) {
          float4 d = *reinterpret_cast<const float4*>(p.dpre + src * p.C + c0 + i);
          float dd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int jj = 0; jj < WMAX; ++jj) if (jj == j) o[i + e] += wr[i + e][jj] * dd[e];
        }
      }
    }
    stv<T, N>(dx + t * p.C + c0, o);
  }
}

// decode: one token per sequence over a paged [slots, W-1, C] history advanced in place
template <typename T>
__global__ void __launch_bounds__(128) conv_decode_kernel(const void* x_, const void* w_,
                                                          void* state_, const int32_t* indices,
                                                          void* y_, int nseq, int num_slots, int C,
                                                          int W, int act) {
  constexpr int N = VecOf<T>::N;
  const int c0 = (blockIdx.y * 128 + threadIdx.x) * N;
  const int seq = blockIdx.x;
  if (c0 >= C) return;
  const T* x = reinterpret_cast<const T*>(x_);
  const T* w = reinterpret_cast<const T*>(w_);
  T* st = reinterpret_cast<T*>(state_);
  T* y = reinterpret_cast<T*>(y_);
  int slot = seq;
  float o[N];
  if (indices) {
    slot = indices[seq];
    if (slot <= 0 || slot >= num_slots) {  // padding: zero output, pool untouched
#pragma unroll
      for (int i = 0; i < N; ++i) o[i] = 0.f;
      stv<T, N>(y + (int64_t)seq * C + c0, o);
      return;
    }
  }
  float xn[N];
  ldv<T, N>(x + (int64_t)seq * C + c0, xn);
#pragma unroll
  for (int i = 0; i < N; ++i) o[i] = (float)w[(int64_t)(c0 + i) * W + (W - 1)] * xn[i];
  T* base = st + (int64_t)slot * (W - 1) * C + c0;
  for (int j = 0; j < W - 1; ++j) {
    float h[N];
    ldv<T, N>(base + (int64_t)j * C, h);
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] += (float)w[(int64_t)(c0 + i) * W + j] * h[i];
    if (j > 0) stv<T, N>(base + (int64_t)(j - 1) * C, h);  // shift left (same thread owns the column)
  }
  if (W > 1) stv<T, N>(base + (int64_t)(W - 2) * C, xn);
  if (act) {
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] = o[i] / (1.f + expf(-o[i]));
  }
  stv<T, N>(y + (int64_t)seq * C + c0, o);
}

static int conv_check(const ConvParams& p) {
  if (!p.x || !p.w || p.C <= 0 || p.W < 1 || p.W > WMAX || p.batch < 1 || p.T < 1) return KDA_ERR_ARG;
  if (p.cu_seqlens && p.batch != 1) return KDA_ERR_ARG;
  return KDA_OK;
}

template <typename T>
static int conv_fwd_launch(const ConvParams& p, cudaStream_t s) {
  constexpr int N = VecOf<T>::N;
  if (p.C % N) return KDA_ERR_UNSUPPORTED;
  int64_t total = (int64_t)p.batch * p.T;
  int64_t runs = p.cu_seqlens ? (total + CONV_TT - 1) / CONV_TT
                              : (int64_t)p.batch * ((p.T + CONV_TT - 1) / CONV_TT);
  dim3 grid((unsigned)runs, (unsigned)((p.C / N + 127) / 128));
  conv_fwd_kernel<T><<<grid, 128, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

template <typename T>
static int conv_bwd_launch(const ConvParams& p, int64_t blocks, cudaStream_t s) {
  constexpr int N = VecOf<T>::N;
  if (p.C % N) return KDA_ERR_UNSUPPORTED;
  dim3 grid((unsigned)blocks, (unsigned)((p.C / N + 31) / 32));
  conv_bwd_pre_kernel<T><<<grid, 256, 0, s>>>(p);
  if (cudaGetLastError() != cudaSuccess) return KDA_ERR_LAUNCH;
  int64_t total = (int64_t)p.batch * p.T;
  dim3 grid2((unsigned)((total + CONV_TT - 1) / CONV_TT), (unsigned)((p.C / N + 127) / 128));
  conv_bwd_dx_kernel<T><<<grid2, 128, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

}  // namespace kda

extern "C" int kda_conv1d_fwd(const void* x, const void* weight, const void* initial_state, void* y,
                              int dtype, const int32_t* cu_seqlens, int nseq, int batch, int tokens,
                              int channels, int width, int activation, void* stream) {
  kda::ConvParams p{};
  p.x = x; p.w = weight; p.y = y; p.state = initial_state; p.cu_seqlens = cu_seqlens; p.nseq = nseq;
  p.batch = batch; p.T = tokens; p.C = channels; p.W = width; p.act = activation;
  if (!y) return KDA_ERR_ARG;
  int rc = kda::conv_check(p);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == KDA_BF16) return kda::conv_fwd_launch<__nv_bfloat16>(p, s);
  if (dtype == KDA_F16) return kda::conv_fwd_launch<__half>(p, s);
  return kda::conv_fwd_launch<float>(p, s);
}

extern "C" int64_t kda_conv1d_bwd_blocks(int batch, int tokens, int packed) {
  const int64_t span = 8 * kda::CONV_TT;
  if (packed) return ((int64_t)batch * tokens + span - 1) / span;
  return (int64_t)batch * ((tokens + span - 1) / span);
}

extern "C" int kda_conv1d_bwd(const void* x, const void* weight, const void* initial_state,
                              const void* dy, void* dx, float* dw_partial, float* dstate,
                              float* dpre_scratch, int dtype, const int32_t* cu_seqlens, int nseq,
                              int batch, int tokens, int channels, int width, int activation,
                              void* stream) {
  kda::ConvParams p{};
  p.x = x; p.w = weight; p.state = initial_state; p.dy = dy; p.dx = dx; p.dpre = dpre_scratch;
  p.dw_part = dw_partial; p.dstate = dstate; p.cu_seqlens = cu_seqlens; p.nseq = nseq;
  p.batch = batch; p.T = tokens; p.C = channels; p.W = width; p.act = activation;
  if (!dy || !dx || !dw_partial || !dpre_scratch) return KDA_ERR_ARG;
  int rc = kda::conv_check(p);
  if (rc) return rc;
  int64_t blocks = kda_conv1d_bwd_blocks(batch, tokens, cu_seqlens != nullptr);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == KDA_BF16) return kda::conv_bwd_launch<__nv_bfloat16>(p, blocks, s);
  if (dtype == KDA_F16) return kda::conv_bwd_launch<__half>(p, blocks, s);
  return kda::conv_bwd_launch<float>(p, blocks, s);
}

extern "C" int kda_conv1d_decode(const void* x, const void* weight, void* state,
                                 const int32_t* state_indices, void* y, int dtype, int nseq,
                                 int num_slots, int channels, int width, int activation,
                                 void* stream) {
  if (!x || !weight || !state || !y || nseq < 0 || channels <= 0 || width < 2 || width > kda::WMAX)
    return KDA_ERR_ARG;
  if (nseq == 0) return KDA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  int n = dtype == KDA_F32 ? 4 : 8;
  if (channels % n) return KDA_ERR_UNSUPPORTED;
  dim3 grid((unsigned)nseq, (unsigned)((channels / n + 127) / 128));
  if (dtype == KDA_BF16)
    kda::conv_decode_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(x, weight, state, state_indices, y, nseq, num_slots, channels, width, activation);
  else if (dtype == KDA_F16)
    kda::conv_decode_kernel<__half><<<grid, 128, 0, s>>>(x, weight, state, state_indices, y, nseq, num_slots, channels, width, activation);
  else
    kda::conv_decode_kernel<float><<<grid, 128, 0, s>>>(x, weight, state, state_indices, y, nseq, num_slots, channels, width, activation);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}
