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
constexpr int CONV_TT = 64; // tokens per thread run

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

// raw 16-byte vector of adjacent channels (converted only when used, so loads can be issued ahead)
template <typename T, int N>
__device__ __forceinline__ void cvt_raw(const uint4& raw, float (&x)[N]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) x[i] = (float)e[i];
}
// the same for N adjacent channels of any vector width (8 or 16 bytes)
// two adjacent channels of a shared-memory tile / of the output
template <typename T>
__device__ __forceinline__ float2 unpack2(const T* p) {
  if constexpr (sizeof(T) == 4) return *reinterpret_cast<const float2*>(p);
  else return make_float2((float)p[0], (float)p[1]);
}
template <typename T>
__device__ __forceinline__ void pack2(T* p, float a, float b) {
  if constexpr (sizeof(T) == 4) *reinterpret_cast<float2*>(p) = make_float2(a, b);
  else {
    T v[2] = {(T)a, (T)b};
    *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<uint32_t*>(v);
  }
}
template <typename T, int N> struct RawVec { uint32_t w[N * sizeof(T) / 4]; };
template <typename T, int N>
__device__ __forceinline__ RawVec<T, N> ld_raw(const T* p) {
  RawVec<T, N> r;
  if constexpr (N * sizeof(T) == 16) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    r.w[0] = u.x; r.w[1] = u.y; r.w[2] = u.z; r.w[3] = u.w;
  } else if constexpr (N * sizeof(T) == 8) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    r.w[0] = u.x; r.w[1] = u.y;
  } else {
    static_assert(N * sizeof(T) == 4, "4-, 8- or 16-byte vectors");
    r.w[0] = *reinterpret_cast<const uint32_t*>(p);
  }
  return r;
}
template <typename T, int N>
__device__ __forceinline__ void cvt_rawv(const RawVec<T, N>& raw, float (&x)[N]) {
  const T* e = reinterpret_cast<const T*>(raw.w);
#pragma unroll
  for (int i = 0; i < N; ++i) x[i] = (float)e[i];
}
template <typename T, int N>
__device__ __forceinline__ void st_vec(T* p, const float (&x)[N]) {
  RawVec<T, N> r;
  T* e = reinterpret_cast<T*>(r.w);
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = (T)x[i];
  if constexpr (N * sizeof(T) == 16) *reinterpret_cast<uint4*>(p) = make_uint4(r.w[0], r.w[1], r.w[2], r.w[3]);
  else if constexpr (N * sizeof(T) == 8) *reinterpret_cast<uint2*>(p) = make_uint2(r.w[0], r.w[1]);
  else *reinterpret_cast<uint32_t*>(p) = r.w[0];
}

// Sequence that holds a run starting at token t0.  Returns true when the whole run [t0, t1) lies in
// that sequence: the fast kernels then handle it, reading the history (or zeros) before the sequence
// start and nothing past its end.  Runs that straddle a packed sequence boundary, and first runs
// when the history gradient is wanted, go to the general kernels.
__device__ __forceinline__ bool conv_run_simple(const ConvParams& p, int64_t t0, int64_t t1, int& seq,
                                                int64_t& bos, int64_t& eos) {
  if (p.cu_seqlens) {
    if (t0 >= p.cu_seqlens[p.nseq]) return false;
    seq = find_seq(p.cu_seqlens, p.nseq, t0);
    bos = p.cu_seqlens[seq]; eos = p.cu_seqlens[seq + 1];
  } else {
    seq = (int)(t0 / p.T); bos = (int64_t)seq * p.T; eos = bos + p.T;
  }
  if (t1 > eos) return false;
  return !(p.dstate && t0 - (p.W - 1) < bos);
}

// y for tokens [t0, t1) of a run inside one sequence, filter width W known at compile time: the
// inputs are fetched four tokens ahead as raw vectors, the window slides through registers.
template <typename T, int W, int N, int B>
__device__ __forceinline__ void conv_fwd_run(const ConvParams& p, int64_t t0, int64_t t1, int c0, int seq,
                                             int64_t bos) {
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* w = reinterpret_cast<const T*>(p.w);
  const T* st = reinterpret_cast<const T*>(p.state);
  T* y = reinterpret_cast<T*>(p.y);
  const int64_t C = p.C;
  float wr[N][W], win[W][N];
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j < W; ++j) wr[i][j] = (float)w[(int64_t)(c0 + i) * W + j];
#pragma unroll
  for (int j = 0; j < W - 1; ++j) {
    const int64_t pos = t0 - (W - 1) + j;
    if (pos >= bos) cvt_rawv<T, N>(ld_raw<T, N>(x + pos * C + c0), win[j]);
    else if (st) cvt_rawv<T, N>(ld_raw<T, N>(st + ((int64_t)seq * (W - 1) + (pos - bos + W - 1)) * C + c0), win[j]);
    else {
#pragma unroll
      for (int i = 0; i < N; ++i) win[j][i] = 0.f;
    }
  }
  const int n = (int)(t1 - t0);
  const T* xl = x + t0 * C + c0;       // next token to fetch
  T* yp = y + t0 * C + c0;             // next token to write
  RawVec<T, N> nxt[B];
#pragma unroll
  for (int b = 0; b < B; ++b)
    if (b < n) { nxt[b] = ld_raw<T, N>(xl); xl += C; }
  for (int tb = 0; tb < n; tb += B) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (tb + b < n) {
        cvt_rawv<T, N>(nxt[b], win[W - 1]);
        if (tb + B + b < n) { nxt[b] = ld_raw<T, N>(xl); xl += C; }   // B tokens ahead
        float o[N];
#pragma unroll
        for (int i = 0; i < N; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < W; ++j) acc = fmaf(wr[i][j], win[j][i], acc);
          o[i] = p.act ? __fdividef(acc, 1.f + __expf(-acc)) : acc;
        }
        st_vec<T, N>(yp, o);
        yp += C;
#pragma unroll
        for (int j = 0; j < W - 1; ++j)
#pragma unroll
          for (int i = 0; i < N; ++i) win[j][i] = win[j + 1][i];
      }
    }
  }
}

// token run of block bx: CONV_TT tokens; runs never straddle dense rows
__device__ __forceinline__ void conv_run_of(const ConvParams& p, int bx, int64_t& t0, int64_t& t1) {
  const int64_t total = (int64_t)p.batch * p.T;
  if (p.cu_seqlens) { t0 = (int64_t)bx * CONV_TT; t1 = min(t0 + CONV_TT, total); }
  else {
    int rpr = (p.T + CONV_TT - 1) / CONV_TT;
    int row = bx / rpr, rb = bx % rpr;
    t0 = (int64_t)row * p.T + (int64_t)rb * CONV_TT;
    t1 = min(t0 + CONV_TT, (int64_t)(row + 1) * p.T);
  }
}

// width-4 filter, every run that lies inside one sequence.  A thread owns kFwdN adjacent channels
// (8-byte vectors for 16-bit types) and keeps kFwdB tokens of loads in flight: few registers, so
// that the resident threads together hold enough bytes in flight to cover the DRAM latency.
constexpr int kFwdN = 4, kFwdB = 8;
template <typename T>
__global__ void __launch_bounds__(128, 8) conv_fwd_fast_kernel(const ConvParams p) {
  const int c0 = (blockIdx.y * 128 + threadIdx.x) * kFwdN;
  if (c0 >= p.C) return;
  int64_t t0, t1, bos, eos;
  int seq;
  conv_run_of(p, blockIdx.x, t0, t1);
  if (t0 < t1 && conv_run_simple(p, t0, t1, seq, bos, eos))
    conv_fwd_run<T, 4, kFwdN, (sizeof(T) == 4 ? kFwdB / 2 : kFwdB)>(p, t0, t1, c0, seq, bos);
}

// any width, sequence starts, histories; with skip_interior != 0 only the runs the fast kernel left
template <typename T>
__global__ void __launch_bounds__(128) conv_fwd_kernel(const ConvParams p, int skip_interior) {
  constexpr int N = VecOf<T>::N;
  const int c0 = (blockIdx.y * 128 + threadIdx.x) * N;
  if (c0 >= p.C) return;
  int64_t t0, t1;
  conv_run_of(p, blockIdx.x, t0, t1);
  {
    int seq; int64_t bos, eos;
    if (skip_interior && (t0 >= t1 || conv_run_simple(p, t0, t1, seq, bos, eos))) return;
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
// With edge_only != 0 (width-4 filters) only the runs the fast kernel left are processed, nothing is
// written to the fp32 scratch, and the partials go to the second half of dw_part.
template <typename T>
__global__ void __launch_bounds__(256) conv_bwd_pre_kernel(const ConvParams p, int edge_only) {
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
  int seq_; int64_t bos_, eos_;
  if (live && t0 < t1 && !(edge_only && conv_run_simple(p, t0, t1, seq_, bos_, eos_))) {
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
      if (!edge_only) {
#pragma unroll
        for (int i = 0; i < N; i += 4)
          *reinterpret_cast<float4*>(p.dpre + t * p.C + c0 + i) = make_float4(d[i], d[i + 1], d[i + 2], d[i + 3]);
      }
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
        p.dw_part[((int64_t)(blockIdx.x + (edge_only ? gridDim.x : 0)) * p.C + c0 + i) * p.W + j] = s;
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

// ------------------------------------------------------------------------------------------
// Width-4 backward in one pass for every run that lies inside one sequence:
//   pre[s] = sum_j w[j] x[s-3+j];  dpre[s] = dy[s] act'(pre[s]);  dx[t] = sum_j w[j] dpre[t+3-j]
//   dw[j] += dpre[s] x[s-3+j]
// A block covers a 512-token span and 64 channels: warp r walks run r of the span, lane l owns the
// channel pair 2l, 2l+1 (a warp reads one 128-byte row segment per token).  The x and dy words are
// fetched eight tokens ahead as raw bits; the x and dpre windows slide through registers over the
// run's 64 tokens plus 3 recomputed ones past them, so no dpre ever goes to memory.  Tokens before
// the sequence start read the history (or zeros), tokens past its end contribute nothing.  Few
// registers per thread, no shared-memory staging and no barriers in the loop: 1024 threads per SM
// keep 64 KB of loads in flight.
// ------------------------------------------------------------------------------------------
constexpr int kBwdCh = 64;                  // channels per block
constexpr int kBwdAhead = 8;                // tokens of loads in flight per thread
template <typename T>
__global__ void __launch_bounds__(256, 3) conv_bwd_fast_kernel(const ConvParams p) {
  constexpr int W = 4, HALO = W - 1, B = kBwdAhead;
  static_assert(sizeof(T) == 2, "channel pairs travel as one 32-bit word");
  __shared__ float s_dw[8][kBwdCh][W];
  const int tid = threadIdx.x, lane = tid & 31, r = tid >> 5;
  const int64_t C = p.C, total = (int64_t)p.batch * p.T;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* dy = reinterpret_cast<const T*>(p.dy);
  const T* st = reinterpret_cast<const T*>(p.state);
  const T* w = reinterpret_cast<const T*>(p.w);
  T* dx = reinterpret_cast<T*>(p.dx);
  const int c0 = blockIdx.y * kBwdCh + 2 * lane;   // this thread's two channels
  const bool live = c0 < p.C;                      // C is even
  float wr[2][W], dwacc[2][W];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < W; ++j) {
      wr[i][j] = live ? (float)w[(int64_t)(c0 + i) * W + j] : 0.f;
      dwacc[i][j] = 0.f;
    }
  int64_t t0, t1;
  if (p.cu_seqlens) { t0 = ((int64_t)blockIdx.x * 8 + r) * CONV_TT; t1 = min(t0 + CONV_TT, total); }
  else {
    int rpr = (p.T + 8 * CONV_TT - 1) / (8 * CONV_TT);
    int row = blockIdx.x / rpr, rb = blockIdx.x % rpr;
    t0 = (int64_t)row * p.T + ((int64_t)rb * 8 + r) * CONV_TT;
    t1 = min(t0 + CONV_TT, (int64_t)(row + 1) * p.T);
  }
  int seq; int64_t bos, eos;
  if (live && t0 < t1 && conv_run_simple(p, t0, t1, seq, bos, eos)) {     // uniform over the warp
    const int owned = (int)(t1 - t0);                                    // tokens whose dx is written
    const int avail = (int)(min(t1 + HALO, eos) - t0);                   // tokens that have a dpre
    const int steps = owned + HALO;
    float xw[W][2], dp[W][2];                        // circular: slot = (token - t0) & 3
#pragma unroll
    for (int j = 0; j < HALO; ++j) {                 // tokens t0-3 .. t0-1 -> slots 1, 2, 3
      const int64_t pos = t0 - HALO + j;
      uint32_t raw = 0u;
      if (pos >= bos) raw = *reinterpret_cast<const uint32_t*>(x + pos * C + c0);
      else if (st) raw = *reinterpret_cast<const uint32_t*>(st + ((int64_t)seq * HALO + (pos - bos + HALO)) * C + c0);
      const float2 v = unpack2<T>(reinterpret_cast<const T*>(&raw));
      xw[j + 1][0] = v.x; xw[j + 1][1] = v.y;
      dp[j + 1][0] = 0.f; dp[j + 1][1] = 0.f;
    }
    const T* xl = x + t0 * C + c0;                   // next token to fetch
    const T* gl = dy + t0 * C + c0;
    T* dxp = dx + t0 * C + c0;                       // next dx row to write
    uint32_t nx[B], ng[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      nx[b] = 0u; ng[b] = 0u;
      if (b < avail) {
        nx[b] = *reinterpret_cast<const uint32_t*>(xl); ng[b] = *reinterpret_cast<const uint32_t*>(gl);
        xl += C; gl += C;
      }
    }
    for (int kb = 0; kb < steps; kb += B) {
#pragma unroll
      for (int b8 = 0; b8 < B; ++b8) {
        const int k = kb + b8, b = b8 & 3;
        if (k < steps) {
          const float2 xv = unpack2<T>(reinterpret_cast<const T*>(&nx[b8]));
          const float2 gv = unpack2<T>(reinterpret_cast<const T*>(&ng[b8]));   // zero past `avail`
          nx[b8] = 0u; ng[b8] = 0u;
          if (k + B < avail) {
            nx[b8] = *reinterpret_cast<const uint32_t*>(xl); ng[b8] = *reinterpret_cast<const uint32_t*>(gl);
            xl += C; gl += C;
          }
          xw[b][0] = xv.x; xw[b][1] = xv.y;
          const float g[2] = {gv.x, gv.y};
          const bool own = k < owned;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            float pre = 0.f;
#pragma unroll
            for (int j = 0; j < W; ++j) pre = fmaf(wr[i][j], xw[(b + 1 + j) & 3][i], pre);
            float dact = 1.f;
            if (p.act) {
              const float sg = __fdividef(1.f, 1.f + __expf(-pre));
              dact = sg * fmaf(pre, 1.f - sg, 1.f);
            }
            const float d = g[i] * dact;
            dp[b][i] = d;
            if (own) {
#pragma unroll
              for (int j = 0; j < W; ++j) dwacc[i][j] = fmaf(d, xw[(b + 1 + j) & 3][i], dwacc[i][j]);
            }
          }
          if (k >= HALO) {                           // dx[k-3] = w0 dpre[k] + ... + w3 dpre[k-3]
            float o[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              float acc = 0.f;
#pragma unroll
              for (int j = 0; j < W; ++j) acc = fmaf(wr[i][j], dp[(b + 4 - j) & 3][i], acc);
              o[i] = acc;
            }
            pack2<T>(dxp, o[0], o[1]);
            dxp += C;
          }
        }
      }
    }
  }
  // reduce the eight runs, then one partial per (block, channel, tap)
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < W; ++j) s_dw[r][2 * lane + i][j] = dwacc[i][j];
  __syncthreads();
  for (int e = tid; e < kBwdCh * W; e += 256) {
    const int ch = e / W, j = e % W;
    if (blockIdx.y * kBwdCh + ch < p.C) {
      float acc = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) acc += s_dw[q][ch][j];
      p.dw_part[((int64_t)blockIdx.x * C + blockIdx.y * kBwdCh + ch) * W + j] = acc;
    }
  }
}

// dx for the runs the fast kernel left (first and last run of a sequence): dpre is rebuilt on the
// fly from x and dy, with the history or zeros before the sequence start.  Any width.
template <typename T>
__global__ void __launch_bounds__(128) conv_bwd_dx_edge_kernel(const ConvParams p) {
  constexpr int N = VecOf<T>::N;
  const int c0 = (blockIdx.y * 128 + threadIdx.x) * N;
  if (c0 >= p.C) return;
  int64_t t0, t1;
  conv_run_of(p, blockIdx.x, t0, t1);
  if (p.cu_seqlens) t1 = min(t1, (int64_t)p.cu_seqlens[p.nseq]);
  {
    int seq_; int64_t bos_, eos_;
    if (t0 >= t1 || conv_run_simple(p, t0, t1, seq_, bos_, eos_)) return;
  }
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* w = reinterpret_cast<const T*>(p.w);
  const T* dy = reinterpret_cast<const T*>(p.dy);
  const T* st = reinterpret_cast<const T*>(p.state);
  T* dx = reinterpret_cast<T*>(p.dx);
  const int W = p.W;
  const int64_t C = p.C;
  float wr[N][WMAX];
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j < WMAX; ++j) wr[i][j] = j < W ? (float)w[(int64_t)(c0 + i) * W + j] : 0.f;
  int seq; int64_t bos, eos;
  if (p.cu_seqlens) { seq = find_seq(p.cu_seqlens, p.nseq, t0); bos = p.cu_seqlens[seq]; eos = p.cu_seqlens[seq + 1]; }
  else { seq = (int)(t0 / p.T); bos = (int64_t)seq * p.T; eos = bos + p.T; }
  for (int64_t t = t0; t < t1; ++t) {
    while (t >= eos) { ++seq; bos = eos; eos = p.cu_seqlens ? p.cu_seqlens[seq + 1] : bos + p.T; }
    float o[N];
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] = 0.f;
    for (int j = 0; j < W; ++j) {
      const int64_t src = t + (W - 1) - j;
      if (src >= eos) continue;
      float pre[N], g[N];
#pragma unroll
      for (int i = 0; i < N; ++i) pre[i] = 0.f;
      for (int jj = 0; jj < W; ++jj) {
        const int64_t pos = src - (W - 1) + jj;
        float xv[N];
        if (pos >= bos) ldv<T, N>(x + pos * C + c0, xv);
        else if (st) ldv<T, N>(st + ((int64_t)seq * (W - 1) + (pos - bos + W - 1)) * C + c0, xv);
        else {
#pragma unroll
          for (int i = 0; i < N; ++i) xv[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < N; ++i)
#pragma unroll
          for (int q = 0; q < WMAX; ++q) if (q == jj) pre[i] += wr[i][q] * xv[i];
      }
      ldv<T, N>(dy + src * C + c0, g);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        float dact = 1.f;
        if (p.act) { const float sg = 1.f / (1.f + expf(-pre[i])); dact = sg * (1.f + pre[i] * (1.f - sg)); }
#pragma unroll
        for (int q = 0; q < WMAX; ++q) if (q == j) o[i] += wr[i][q] * g[i] * dact;
      }
    }
    stv<T, N>(dx + t * C + c0, o);
  }
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
  const int fast = p.W == 4;
  if (fast) {
    dim3 gridf((unsigned)runs, (unsigned)((p.C / kFwdN + 127) / 128));
    conv_fwd_fast_kernel<T><<<gridf, 128, 0, s>>>(p);
  }
  conv_fwd_kernel<T><<<grid, 128, 0, s>>>(p, fast);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

template <typename T>
static int conv_bwd_launch(const ConvParams& p, int64_t blocks, cudaStream_t s) {
  constexpr int N = VecOf<T>::N;
  if (p.C % N) return KDA_ERR_UNSUPPORTED;
  // dw_part holds 2 * blocks partial slots: [0, blocks) and [blocks, 2 blocks)
  dim3 grid((unsigned)blocks, (unsigned)((p.C / N + 31) / 32));
  int64_t total = (int64_t)p.batch * p.T;
  if constexpr (sizeof(T) == 2) if (p.W == 4) {
    // one-pass kernel for the runs inside one sequence, the general kernels for the other runs
    if (p.C % 8) return KDA_ERR_UNSUPPORTED;
    dim3 gridf((unsigned)blocks, (unsigned)((p.C + kBwdCh - 1) / kBwdCh));
    conv_bwd_fast_kernel<T><<<gridf, 256, 0, s>>>(p);
    conv_bwd_pre_kernel<T><<<grid, 256, 0, s>>>(p, 1);
    int64_t runs = p.cu_seqlens ? (total + CONV_TT - 1) / CONV_TT
                                : (int64_t)p.batch * ((p.T + CONV_TT - 1) / CONV_TT);
    dim3 grid3((unsigned)runs, (unsigned)((p.C / N + 127) / 128));
    conv_bwd_dx_edge_kernel<T><<<grid3, 128, 0, s>>>(p);
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
  }
  if (!p.dpre) return KDA_ERR_ARG;
  if (cudaMemsetAsync(p.dw_part + blocks * p.C * p.W, 0, sizeof(float) * blocks * p.C * p.W, s) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  conv_bwd_pre_kernel<T><<<grid, 256, 0, s>>>(p, 0);
  if (cudaGetLastError() != cudaSuccess) return KDA_ERR_LAUNCH;
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

// launch blocks of the backward kernels (each covers 8 runs of CONV_TT tokens)
static int64_t conv_bwd_launch_blocks(int batch, int tokens, int packed) {
  const int64_t span = 8 * kda::CONV_TT;
  if (packed) return ((int64_t)batch * tokens + span - 1) / span;
  return (int64_t)batch * ((tokens + span - 1) / span);
}
// partial slots of dw_partial: two per launch block (interior runs, sequence-edge runs)
extern "C" int64_t kda_conv1d_bwd_blocks(int batch, int tokens, int packed) {
  return 2 * conv_bwd_launch_blocks(batch, tokens, packed);
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
  if (!dy || !dx || !dw_partial) return KDA_ERR_ARG;     // dpre_scratch is needed only when width != 4
  int rc = kda::conv_check(p);
  if (rc) return rc;
  int64_t blocks = conv_bwd_launch_blocks(batch, tokens, cu_seqlens != nullptr);
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
