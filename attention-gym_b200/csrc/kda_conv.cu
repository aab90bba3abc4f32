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
#include <type_traits>
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

// two 16-bit values in one register word <-> two floats (bf16: a shift and a mask; no memory trip)
template <typename T>
__device__ __forceinline__ float2 word_to_float2(uint32_t u) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value)
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  else return __half22float2(*reinterpret_cast<const __half2*>(&u));
}
template <typename T>
__device__ __forceinline__ uint32_t float2_to_word(float a, float b) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}
template <typename T, int N>
__device__ __forceinline__ void words_to_float(const RawVec<T, N>& raw, float (&x)[N]) {
  static_assert(sizeof(T) == 2, "16-bit types");
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const float2 v = word_to_float2<T>(raw.w[i]);
    x[2 * i] = v.x; x[2 * i + 1] = v.y;
  }
}
template <typename T, int N>
__device__ __forceinline__ void st_words(T* p, const float (&x)[N]) {
  static_assert(sizeof(T) == 2, "16-bit types");
  uint32_t w[N / 2];
#pragma unroll
  for (int i = 0; i < N / 2; ++i) w[i] = float2_to_word<T>(x[2 * i], x[2 * i + 1]);
  if constexpr (N == 8) *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  else if constexpr (N == 4) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
  else *reinterpret_cast<uint32_t*>(p) = w[0];
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

// The same for 16-bit types and the width-4 filter, written for few instructions per element: the
// window is circular (token k lives in slot k & 3, so nothing is moved), words are converted in
// registers, and groups of B tokens that need no bounds checks run without any.
template <typename T, int N, int B, bool ACT>
__device__ __forceinline__ void conv_fwd_run16(const ConvParams& p, int64_t t0, int64_t t1, int c0, int seq,
                                               int64_t bos) {
  constexpr int W = 4;
  static_assert(B % 4 == 0, "the window slot of a token is its position in the group");
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* w = reinterpret_cast<const T*>(p.w);
  const T* st = reinterpret_cast<const T*>(p.state);
  T* y = reinterpret_cast<T*>(p.y);
  const int64_t C = p.C;
  float wr[N][W], win[W][N];
#pragma unroll
  for (int i = 0; i < N; ++i) {          // the four taps of a channel are one 8-byte word pair
    RawVec<T, 4> taps = ld_raw<T, 4>(w + (int64_t)(c0 + i) * W);
    words_to_float<T, 4>(taps, wr[i]);
  }
#pragma unroll
  for (int j = 0; j < W - 1; ++j) {      // tokens t0-3 .. t0-1 -> slots 1, 2, 3
    const int64_t pos = t0 - (W - 1) + j;
    if (pos >= bos) words_to_float<T, N>(ld_raw<T, N>(x + pos * C + c0), win[j + 1]);
    else if (st) words_to_float<T, N>(ld_raw<T, N>(st + ((int64_t)seq * (W - 1) + (pos - bos + W - 1)) * C + c0), win[j + 1]);
    else {
#pragma unroll
      for (int i = 0; i < N; ++i) win[j + 1][i] = 0.f;
    }
  }
  // Channel pairs go through the packed fp32 instructions (two lanes per issue slot); the results are
  // the same correctly rounded products and sums as the scalar forms.
  auto token = [&](const RawVec<T, N>& raw, int slot, T* out) {    // slot: constant after unrolling
    words_to_float<T, N>(raw, win[slot]);
    const int s1 = (slot + 1) & 3, s2 = (slot + 2) & 3, s3 = (slot + 3) & 3;
    float o[N];
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      float2 acc = __fmul2_rn(make_float2(wr[i][0], wr[i + 1][0]), make_float2(win[s1][i], win[s1][i + 1]));
      acc = __ffma2_rn(make_float2(wr[i][1], wr[i + 1][1]), make_float2(win[s2][i], win[s2][i + 1]), acc);
      acc = __ffma2_rn(make_float2(wr[i][2], wr[i + 1][2]), make_float2(win[s3][i], win[s3][i + 1]), acc);
      acc = __ffma2_rn(make_float2(wr[i][3], wr[i + 1][3]), make_float2(win[slot][i], win[slot][i + 1]), acc);
      if (ACT) {                                   // acc / (1 + e^-acc)
        const float2 e = __fmul2_rn(acc, make_float2(-kLog2e, -kLog2e));
        const float2 den = __fadd2_rn(make_float2(fexp2(e.x), fexp2(e.y)), make_float2(1.f, 1.f));
        acc = __fmul2_rn(acc, make_float2(__fdividef(1.f, den.x), __fdividef(1.f, den.y)));
      }
      o[i] = acc.x; o[i + 1] = acc.y;
    }
    st_words<T, N>(out, o);
  };
  const int n = (int)(t1 - t0);
  const T* xrow = x + t0 * C + c0;
  T* yrow = y + t0 * C + c0;
  const uint32_t Cu = (uint32_t)p.C;     // element offsets inside a run fit 32 bits (checked at launch)
  RawVec<T, N> nxt[B];
#pragma unroll
  for (int b = 0; b < B; ++b)
    if (b < n) nxt[b] = ld_raw<T, N>(xrow + b * Cu);
  int k = 0;
  for (; k + 2 * B <= n; k += B) {       // B tokens and the B after them all exist
    const uint32_t off = (uint32_t)k * Cu;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const RawVec<T, N> cur = nxt[b];
      nxt[b] = ld_raw<T, N>(xrow + (off + (B + b) * Cu));
      token(cur, b & 3, yrow + (off + b * Cu));
    }
  }
  for (; k < n; k += B) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (k + b < n) {
        const RawVec<T, N> cur = nxt[b];
        if (k + B + b < n) nxt[b] = ld_raw<T, N>(xrow + (uint32_t)(k + B + b) * Cu);
        token(cur, b & 3, yrow + (uint32_t)(k + b) * Cu);
      }
    }
  }
}

// width-4 filter, every run that lies inside one sequence.  A thread owns kFwdN adjacent channels
// (one 8-byte vector of a 16-bit type) and keeps kFwdB tokens of loads in flight; 72 registers, so
// seven blocks per SM hold about 57 KB of loads in flight.
constexpr int kFwdN = 4, kFwdB = 8, kFwdMinBlocks = 7;
template <typename T, int N16, int B, int MINB>
__global__ void __launch_bounds__(128, MINB) conv_fwd_fast_kernel(const ConvParams p, int chan_blocks) {
  constexpr int N = sizeof(T) == 2 ? N16 : N16 / 2;
  // channel block fastest: the blocks resident at one time cover whole token rows
  const int cblk = blockIdx.x % chan_blocks, run = blockIdx.x / chan_blocks;
  const int c0 = (cblk * 128 + threadIdx.x) * N;
  if (c0 >= p.C) return;
  int64_t t0, t1, bos, eos;
  int seq;
  conv_run_of(p, run, t0, t1);
  if (t0 < t1 && conv_run_simple(p, t0, t1, seq, bos, eos)) {
    if constexpr (sizeof(T) == 2) {
      if (p.act) conv_fwd_run16<T, N, B, true>(p, t0, t1, c0, seq, bos);
      else conv_fwd_run16<T, N, B, false>(p, t0, t1, c0, seq, bos);
    } else {
      conv_fwd_run<T, 4, N, 4>(p, t0, t1, c0, seq, bos);
    }
  }
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
constexpr int kBwdN = 4;                    // adjacent channels per thread (one 8-byte vector)
constexpr int kBwdCh = 32 * kBwdN;          // channels per block
constexpr int kBwdAhead = 4;                // tokens of loads in flight per thread
template <typename T, int B, bool ACT>
__global__ void __launch_bounds__(256, 2) conv_bwd_fast_kernel(const ConvParams p, int chan_blocks) {
  constexpr int W = 4, HALO = W - 1, N = kBwdN;
  static_assert(sizeof(T) == 2 && B % 4 == 0, "16-bit types; a token's window slot is its position in the group");
  __shared__ float s_dw[8][kBwdCh][W];
  const int tid = threadIdx.x, lane = tid & 31, r = tid >> 5;
  // channel block fastest, so that the resident blocks cover whole token rows
  const int cblk = blockIdx.x % chan_blocks, span = blockIdx.x / chan_blocks;
  const int64_t C = p.C, total = (int64_t)p.batch * p.T;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* dy = reinterpret_cast<const T*>(p.dy);
  const T* st = reinterpret_cast<const T*>(p.state);
  const T* w = reinterpret_cast<const T*>(p.w);
  T* dx = reinterpret_cast<T*>(p.dx);
  const int c0 = cblk * kBwdCh + N * lane;         // this thread's channels
  const bool live = c0 < p.C;                      // C is a multiple of 8
  float wr[N][W], dwacc[N][W];
#pragma unroll
  for (int i = 0; i < N; ++i) {
#pragma unroll
    for (int j = 0; j < W; ++j) { wr[i][j] = 0.f; dwacc[i][j] = 0.f; }
    if (live) words_to_float<T, 4>(ld_raw<T, 4>(w + (int64_t)(c0 + i) * W), wr[i]);
  }
  int64_t t0, t1;
  if (p.cu_seqlens) { t0 = ((int64_t)span * 8 + r) * CONV_TT; t1 = min(t0 + CONV_TT, total); }
  else {
    int rpr = (p.T + 8 * CONV_TT - 1) / (8 * CONV_TT);
    int row = span / rpr, rb = span % rpr;
    t0 = (int64_t)row * p.T + ((int64_t)rb * 8 + r) * CONV_TT;
    t1 = min(t0 + CONV_TT, (int64_t)(row + 1) * p.T);
  }
  int seq; int64_t bos, eos;
  if (live && t0 < t1 && conv_run_simple(p, t0, t1, seq, bos, eos)) {     // uniform over the warp
    const int owned = (int)(t1 - t0);                                    // tokens whose dx is written
    const int avail = (int)(min(t1 + HALO, eos) - t0);                   // tokens that have a dpre
    const int steps = owned + HALO;
    float xw[W][N], dp[W][N];                        // circular: slot = (token - t0) & 3
#pragma unroll
    for (int j = 0; j < HALO; ++j) {                 // tokens t0-3 .. t0-1 -> slots 1, 2, 3
      const int64_t pos = t0 - HALO + j;
      RawVec<T, N> raw;
#pragma unroll
      for (int q = 0; q < N / 2; ++q) raw.w[q] = 0u;
      if (pos >= bos) raw = ld_raw<T, N>(x + pos * C + c0);
      else if (st) raw = ld_raw<T, N>(st + ((int64_t)seq * HALO + (pos - bos + HALO)) * C + c0);
      words_to_float<T, N>(raw, xw[j + 1]);
#pragma unroll
      for (int i = 0; i < N; ++i) dp[j + 1][i] = 0.f;
    }
    const T* xrow = x + t0 * C + c0;
    const T* grow = dy + t0 * C + c0;
    T* dxrow = dx + t0 * C + c0;
    const uint32_t Cu = (uint32_t)p.C;               // element offsets inside a run fit 32 bits
    RawVec<T, N> nx[B], ng[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
#pragma unroll
      for (int q = 0; q < N / 2; ++q) { nx[b].w[q] = 0u; ng[b].w[q] = 0u; }
      if (b < avail) { nx[b] = ld_raw<T, N>(xrow + b * Cu); ng[b] = ld_raw<T, N>(grow + b * Cu); }
    }
    // One token: slot is constant after unrolling; OWN / OUT say whether the token adds to dw and
    // whether a dx row (three tokens back) is complete.
    auto token = [&](const RawVec<T, N>& rx, const RawVec<T, N>& rg, int slot, bool own, bool out, T* dxp) {
      float g[N];
      words_to_float<T, N>(rx, xw[slot]);
      words_to_float<T, N>(rg, g);                   // zero past `avail`
      const int s1 = (slot + 1) & 3, s2 = (slot + 2) & 3, s3 = (slot + 3) & 3;
      const float2 one = make_float2(1.f, 1.f);
      float o[N];
#pragma unroll
      for (int i = 0; i < N; i += 2) {               // channel pairs on the packed fp32 instructions
        const float2 w0 = make_float2(wr[i][0], wr[i + 1][0]), w1 = make_float2(wr[i][1], wr[i + 1][1]),
                     w2 = make_float2(wr[i][2], wr[i + 1][2]), w3 = make_float2(wr[i][3], wr[i + 1][3]);
        const float2 x1 = make_float2(xw[s1][i], xw[s1][i + 1]), x2 = make_float2(xw[s2][i], xw[s2][i + 1]),
                     x3 = make_float2(xw[s3][i], xw[s3][i + 1]), x0 = make_float2(xw[slot][i], xw[slot][i + 1]);
        float2 pre = __fmul2_rn(w0, x1);
        pre = __ffma2_rn(w1, x2, pre);
        pre = __ffma2_rn(w2, x3, pre);
        pre = __ffma2_rn(w3, x0, pre);
        float2 d = make_float2(g[i], g[i + 1]);
        if (ACT) {                                   // act'(pre) = s (1 + pre (1 - s)),  s = sigmoid(pre)
          const float2 e = __fmul2_rn(pre, make_float2(-kLog2e, -kLog2e));
          const float2 den = __fadd2_rn(make_float2(fexp2(e.x), fexp2(e.y)), one);
          const float2 sg = make_float2(__fdividef(1.f, den.x), __fdividef(1.f, den.y));
          const float2 om = __ffma2_rn(sg, make_float2(-1.f, -1.f), one);
          d = __fmul2_rn(d, __fmul2_rn(sg, __ffma2_rn(pre, om, one)));
        }
        dp[slot][i] = d.x; dp[slot][i + 1] = d.y;
        if (own) {
          float2 a0 = __ffma2_rn(d, x1, make_float2(dwacc[i][0], dwacc[i + 1][0]));
          float2 a1 = __ffma2_rn(d, x2, make_float2(dwacc[i][1], dwacc[i + 1][1]));
          float2 a2 = __ffma2_rn(d, x3, make_float2(dwacc[i][2], dwacc[i + 1][2]));
          float2 a3 = __ffma2_rn(d, x0, make_float2(dwacc[i][3], dwacc[i + 1][3]));
          dwacc[i][0] = a0.x; dwacc[i + 1][0] = a0.y; dwacc[i][1] = a1.x; dwacc[i + 1][1] = a1.y;
          dwacc[i][2] = a2.x; dwacc[i + 1][2] = a2.y; dwacc[i][3] = a3.x; dwacc[i + 1][3] = a3.y;
        }
        // dx[k-3] = w0 dpre[k] + w1 dpre[k-1] + w2 dpre[k-2] + w3 dpre[k-3]
        float2 acc = __fmul2_rn(w0, d);
        acc = __ffma2_rn(w1, make_float2(dp[s3][i], dp[s3][i + 1]), acc);
        acc = __ffma2_rn(w2, make_float2(dp[s2][i], dp[s2][i + 1]), acc);
        acc = __ffma2_rn(w3, make_float2(dp[s1][i], dp[s1][i + 1]), acc);
        o[i] = acc.x; o[i + 1] = acc.y;
      }
      if (out) st_words<T, N>(dxp, o);
    };
    const RawVec<T, N> zero = [] { RawVec<T, N> z;
#pragma unroll
      for (int q = 0; q < N / 2; ++q) z.w[q] = 0u;
      return z; }();
    int k = 0;
    if (owned >= B && 2 * B <= avail) {              // first group: no dx rows for its first three tokens
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const RawVec<T, N> cx = nx[b], cg = ng[b];
        nx[b] = ld_raw<T, N>(xrow + (B + b) * Cu);
        ng[b] = ld_raw<T, N>(grow + (B + b) * Cu);
        token(cx, cg, b & 3, true, b >= HALO, dxrow + (b >= HALO ? (b - HALO) * Cu : 0u));
      }
      k = B;
    }
    for (; k > 0 && k + B <= owned && k + 2 * B <= avail; k += B) {   // interior: nothing to check
      const uint32_t off = (uint32_t)k * Cu;
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const RawVec<T, N> cx = nx[b], cg = ng[b];
        nx[b] = ld_raw<T, N>(xrow + (off + (B + b) * Cu));
        ng[b] = ld_raw<T, N>(grow + (off + (B + b) * Cu));
        token(cx, cg, b & 3, true, true, dxrow + (off + b * Cu - HALO * Cu));
      }
    }
    for (; k < steps; k += B) {                      // the rest, every condition checked
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (k + b < steps) {
          const RawVec<T, N> cx = nx[b], cg = ng[b];
          nx[b] = zero; ng[b] = zero;
          if (k + B + b < avail) {
            nx[b] = ld_raw<T, N>(xrow + (uint32_t)(k + B + b) * Cu);
            ng[b] = ld_raw<T, N>(grow + (uint32_t)(k + B + b) * Cu);
          }
          token(cx, cg, b & 3, k + b < owned, k + b >= HALO,
                dxrow + (k + b >= HALO ? (uint32_t)(k + b - HALO) * Cu : 0u));
        }
      }
    }
  }
  // reduce the eight runs, then one partial per (block, channel, tap)
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j < W; ++j) s_dw[r][N * lane + i][j] = dwacc[i][j];
  __syncthreads();
  for (int e = tid; e < kBwdCh * W; e += 256) {
    const int ch = e / W, j = e % W;
    if (cblk * kBwdCh + ch < p.C) {
      float acc = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) acc += s_dw[q][ch][j];
      p.dw_part[((int64_t)span * C + cblk * kBwdCh + ch) * W + j] = acc;
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
  {
    // the same test, on the same unclamped run, that made the one-pass kernel take or leave this
    // run; clamping to the packed end first would make a run that ends in the unused tail of a
    // fixed-capacity buffer look "simple" here although the one-pass kernel left it
    int seq_; int64_t bos_, eos_;
    if (t0 >= t1 || conv_run_simple(p, t0, t1, seq_, bos_, eos_)) return;
  }
  if (p.cu_seqlens) t1 = min(t1, (int64_t)p.cu_seqlens[p.nseq]);
  if (t0 >= t1) return;
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
    if ((int64_t)(CONV_TT + 8) * p.C > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
    const int chan_blocks = (p.C / (sizeof(T) == 2 ? kFwdN : kFwdN / 2) + 127) / 128;
    if (runs * chan_blocks > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
    conv_fwd_fast_kernel<T, kFwdN, kFwdB, kFwdMinBlocks><<<(unsigned)(runs * chan_blocks), 128, 0, s>>>(p, chan_blocks);
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
    const int chan_blocks = (int)((p.C + kBwdCh - 1) / kBwdCh);
    if (blocks * chan_blocks > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
    if ((int64_t)(CONV_TT + 16) * p.C > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
    const unsigned nb = (unsigned)(blocks * chan_blocks);
    if (p.act) conv_bwd_fast_kernel<T, kBwdAhead, true><<<nb, 256, 0, s>>>(p, chan_blocks);
    else conv_bwd_fast_kernel<T, kBwdAhead, false><<<nb, 256, 0, s>>>(p, chan_blocks);
    if (!p.cu_seqlens && !p.dstate) {
      // dense rows without a history gradient: every run went through the one-pass kernel
      if (cudaMemsetAsync(p.dw_part + blocks * p.C * p.W, 0, sizeof(float) * blocks * p.C * p.W, s) != cudaSuccess)
        return KDA_ERR_LAUNCH;
      return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
    }
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

// dw[e] = sum over the partial rows, written in the weight's dtype
__global__ void __launch_bounds__(256) conv_dw_reduce_kernel(const float* __restrict__ part, int64_t rows,
                                                             int64_t n, void* dw, int dt) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= n) return;
  float acc = 0.f;
  for (int64_t r = 0; r < rows; ++r) acc += part[r * n + e];
  store_from_float(dw, dt, e, acc);
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

// dw [C, W] in `dtype` = the sum of the `rows` fp32 partial rows kda_conv1d_bwd wrote (fixed order).
extern "C" int kda_conv1d_dw_reduce(const float* dw_partial, int64_t rows, int64_t channels_times_width,
                                    void* dw, int dtype, void* stream) {
  if (!dw_partial || !dw || rows < 0 || channels_times_width < 0) return KDA_ERR_ARG;
  if (channels_times_width == 0) return KDA_OK;
  const unsigned blocks = (unsigned)((channels_times_width + 255) / 256);
  kda::conv_dw_reduce_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(dw_partial, rows, channels_times_width, dw, dtype);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}
