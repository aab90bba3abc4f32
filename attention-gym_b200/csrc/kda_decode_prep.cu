// Decode-step preprocessing in one launch: for every (sequence, head)
//   y = SiLU(causal depthwise conv of the new token over the paged history)   for the q, k, v channels,
//   the history pool advanced in place;
//   q = y_q / ||y_q||,  k = y_k / ||y_k||  (rsqrt(sum y^2 + eps));  v = y_v;
//   g = log2(e) * lower_bound * sigmoid(exp(A_log[h]) * (raw_gate + dt_bias[h]))   (per-token gate).
// The reference runs these as separate launches -- causal_conv1d_decode (short_conv/cute.py:3569),
// l2norm twice (fwd/triton/l2norm_fwd.py:231) and the bounded gate with chunk size 1
// (fwd/triton/gate_fwd.py:716) -- and names "decode preprocessing and scan are separate launches"
// as a serving limitation (kda/api.py:210-212).  Here the preprocessing is one kernel and the
// state update (kda_recurrent_fwd) the second.
//
// x and the history are [.., 3 * H * 128] with the q channels first, then k, then v.  Two kernels:
// the vector kernel further down for 16-bit tensors, and this scalar one (any dtype, W <= 8): one
// block of 128 threads per (sequence, head), thread c owns channel c of the head's q, k and v blocks.
#include "kda_common.cuh"
#include "kda_timing.cuh"

namespace kda {

struct PrepDecodeParams {
  const void* x; const void* w; void* conv_state;          // [N, 3HD], [3HD, W], [slots, W-1, 3HD]
  const void* raw_gate; const float* A_log; const float* dt_bias;   // [N, H, D], [H], [H, D]
  void* q; void* k; void* v; float* g;                     // [N, H, D] each (q, k, v in the dtype of x)
  const int32_t* state_indices;                            // conv pool slots or NULL (slot = sequence)
  int dt, dt_gate, nseq, H, W, num_slots, act;
  float lower_bound, eps;
};

__device__ __forceinline__ float block_sum128(float v, float* scratch, int tid) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  if ((tid & 31) == 0) scratch[tid >> 5] = v;
  __syncthreads();
  const float s = scratch[0] + scratch[1] + scratch[2] + scratch[3];
  __syncthreads();
  return s;
}

__global__ void __launch_bounds__(128) kda_decode_prep_kernel(const PrepDecodeParams p) {
  __shared__ float scratch[4];
  const int tid = threadIdx.x, head = blockIdx.x % p.H, seq = blockIdx.x / p.H;
  const int HD = p.H * 128, C = 3 * HD, W = p.W;
  const int64_t orow = ((int64_t)seq * p.H + head) * 128 + tid;
  int64_t slot = seq;
  bool active = true;
  if (p.state_indices) {
    const int si = p.state_indices[seq];
    active = si > 0 && si < p.num_slots;         // non-positive (or out of range) slots are padding
    slot = si;
  }
  if (!active) {      // padding rows: zero operands (the scan skips them as well), pool untouched
    store_from_float(p.q, p.dt, orow, 0.f);
    store_from_float(p.k, p.dt, orow, 0.f);
    store_from_float(p.v, p.dt, orow, 0.f);
    p.g[orow] = 0.f;
    return;
  }
  float y[3];
#pragma unroll
  for (int part = 0; part < 3; ++part) {
    const int ch = part * HD + head * 128 + tid;
    const float xn = load_as_float(p.x, p.dt, (int64_t)seq * C + ch);
    float acc = load_as_float(p.w, p.dt, (int64_t)ch * W + (W - 1)) * xn;
    const int64_t hbase = slot * (int64_t)(W - 1) * C + ch;
    for (int j = 0; j < W - 1; ++j) {
      const float h = load_as_float(p.conv_state, p.dt, hbase + (int64_t)j * C);
      acc = fmaf(load_as_float(p.w, p.dt, (int64_t)ch * W + j), h, acc);
      if (j > 0) store_from_float(p.conv_state, p.dt, hbase + (int64_t)(j - 1) * C, h);   // shift left
    }
    if (W > 1) store_from_float(p.conv_state, p.dt, hbase + (int64_t)(W - 2) * C, xn);
    y[part] = p.act ? acc / (1.f + expf(-acc)) : acc;
  }
  const float rq = rsqrtf(block_sum128(y[0] * y[0], scratch, tid) + p.eps);
  const float rk = rsqrtf(block_sum128(y[1] * y[1], scratch, tid) + p.eps);
  store_from_float(p.q, p.dt, orow, y[0] * rq);
  store_from_float(p.k, p.dt, orow, y[1] * rk);
  store_from_float(p.v, p.dt, orow, y[2]);
  const float z = expf(p.A_log[head]) * (load_as_float(p.raw_gate, p.dt_gate, orow) + p.dt_bias[head * 128 + tid]);
  p.g[orow] = p.lower_bound / (1.f + expf(-z)) * kLog2e;
}

// 16-bit tensors: a thread owns one 16-byte vector of 8 adjacent channels.  Vector v covers channels
// 8 v .. 8 v + 7 of the q | k | v row, i.e. part v / (16 H), head (v / 16) % H; the 16 threads of a
// (part, head) group are adjacent lanes, so the L2 norms are half-warp shuffles and every global
// access is a coalesced 16-byte vector.  Threads of the q part also evaluate the gate of their
// eight (head, channel) pairs.
template <int W>
__global__ void __launch_bounds__(256) kda_decode_prep_vec_kernel(const PrepDecodeParams p) {
  const int seq = blockIdx.y, vec = blockIdx.x * 256 + threadIdx.x;
  const int HD = p.H * 128, C = 3 * HD, nvec = C / 8;
  const bool in_range = vec < nvec;
  const int part = in_range ? vec / (p.H * 16) : 3, hv = vec - part * (p.H * 16);   // hv: vector inside the part
  int64_t slot = seq;
  bool active = true;
  if (p.state_indices) {
    const int si = p.state_indices[seq];
    active = si > 0 && si < p.num_slots;
    slot = si;
  }
  const int dt = p.dt;
  float y[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = 0.f;
  if (in_range && active) {
    const uint4* xr = reinterpret_cast<const uint4*>(p.x) + (int64_t)seq * nvec + vec;
    uint4* hist = reinterpret_cast<uint4*>(p.conv_state) + slot * (int64_t)(W - 1) * nvec + vec;
    const uint4* wv = reinterpret_cast<const uint4*>(p.w) + (int64_t)vec * W;    // 8 channels x W taps
    uint4 raw[W];                                  // history rows 0 .. W-2, then the new token
#pragma unroll
    for (int j = 0; j < W - 1; ++j) raw[j] = hist[(int64_t)j * nvec];
    raw[W - 1] = *xr;
    uint4 wraw[W];                                 // 8 W weights = W vectors; element i * W + j
#pragma unroll
    for (int j = 0; j < W; ++j) wraw[j] = wv[j];
    const unsigned short* wh = reinterpret_cast<const unsigned short*>(wraw);
#pragma unroll
    for (int j = 0; j < W; ++j) {
      float f[8];
      raw8_to_float(raw[j], dt, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = fmaf(raw_to_float(wh[i * W + j], dt), f[i], y[i]);
    }
#pragma unroll
    for (int j = 0; j < W - 1; ++j) hist[(int64_t)j * nvec] = raw[j + 1];      // shift left, append x
    if (p.act) {
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = y[i] / (1.f + expf(-y[i]));
    }
  }
  // q, k: L2 norm over the 128 channels of the head = 16 adjacent lanes (all lanes take part)
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(y[i], y[i], ss);
#pragma unroll
  for (int d = 8; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  if (!in_range) return;
  if (part < 2) {
    const float r = rsqrtf(ss + p.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] *= r;
  }
  void* dst = part == 0 ? p.q : (part == 1 ? p.k : p.v);
  reinterpret_cast<uint4*>(dst)[(int64_t)seq * (p.H * 16) + hv] = float8_to_raw(y, dt);   // zeros for padding
  if (part == 0) {                                 // the gate of the same (head, 8 channels)
    const int head = hv >> 4, c0 = (hv & 15) * 8;
    float g[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = 0.f;
    if (active) {
      const float a = expf(p.A_log[head]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float z = a * (load_as_float(p.raw_gate, p.dt_gate, ((int64_t)seq * p.H + head) * 128 + c0 + i) +
                             p.dt_bias[head * 128 + c0 + i]);
        g[i] = p.lower_bound / (1.f + expf(-z)) * kLog2e;
      }
    }
    float4* go = reinterpret_cast<float4*>(p.g + ((int64_t)seq * p.H + head) * 128 + c0);
    go[0] = make_float4(g[0], g[1], g[2], g[3]);
    go[1] = make_float4(g[4], g[5], g[6], g[7]);
  }
}

}  // namespace kda

extern "C" int kda_decode_prep(const void* x, const void* conv_weight, void* conv_state,
                               const int32_t* conv_state_indices, const void* raw_gate, int dt_gate,
                               const float* A_log, const float* dt_bias, void* q, void* k, void* v,
                               float* gate, int dtype, int nseq, int heads, int head_dim, int width,
                               int num_slots, int activation, float lower_bound, float eps,
                               void* stream) {
  if (!x || !conv_weight || !conv_state || !raw_gate || !A_log || !dt_bias || !q || !k || !v || !gate)
    return KDA_ERR_ARG;
  if (head_dim != 128) return KDA_ERR_UNSUPPORTED;
  if (nseq < 0 || heads < 1 || width < 1 || width > 8 || num_slots < 1) return KDA_ERR_ARG;
  if (nseq == 0) return KDA_OK;
  if ((int64_t)nseq * heads > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  kda::PrepDecodeParams p;
  p.x = x; p.w = conv_weight; p.conv_state = conv_state; p.raw_gate = raw_gate; p.A_log = A_log;
  p.dt_bias = dt_bias; p.q = q; p.k = k; p.v = v; p.g = gate; p.state_indices = conv_state_indices;
  p.dt = dtype; p.dt_gate = dt_gate; p.nseq = nseq; p.H = heads; p.W = width; p.num_slots = num_slots;
  p.act = activation; p.lower_bound = lower_bound; p.eps = eps;
  kda::StageScope timing(kda::kStageConv, (cudaStream_t)stream);
  const uintptr_t bits = (uintptr_t)x | (uintptr_t)conv_weight | (uintptr_t)conv_state | (uintptr_t)q |
                         (uintptr_t)k | (uintptr_t)v | (uintptr_t)gate;
  if (dtype != KDA_F32 && (width == 4 || width == 2 || width == 3) && (bits & 15) == 0 && nseq <= 65535) {
    dim3 grid((unsigned)((3 * heads * 16 + 255) / 256), (unsigned)nseq);
    if (width == 4) kda::kda_decode_prep_vec_kernel<4><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    else if (width == 3) kda::kda_decode_prep_vec_kernel<3><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    else kda::kda_decode_prep_vec_kernel<2><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
  }
  kda::kda_decode_prep_kernel<<<(unsigned)(nseq * heads), 128, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}
