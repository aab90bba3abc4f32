// Token-sequential KDA scan: the decode step (T = 1) and inference prefill.
//
// Replaces the reference's Triton scan `_kda_recurrent_fwd_kernel`
// (attn_gym/linear/kda/fwd/triton/recurrent.py:41-153).  Per token, per (sequence, head):
//     S <- diag(2^g) S ;  d = beta (v - S^T k) ;  S <- S + k d^T ;  o = scale S^T q
// One CTA owns a [K x 32*VEC] column slab of the fp32 state and keeps it in registers for
// the whole scan: warp w holds rows w, w+8, ...; lane l holds VEC adjacent columns, so a
// warp touches one contiguous 128*VEC-byte row segment per load (VEC = 4: 512 B, LDG.128).
// The two K-reductions of a step (S^T k and S^T q, both taken on the decayed state) share
// one shared-memory exchange:  o = scale (S_d^T q + (q.k) d).
// The decode step is pure state streaming: 2*K*V*4 bytes per (sequence, head) per step.
#include "kda_common.cuh"
#include "kda_timing.cuh"

namespace kda {

struct ScanParams {
  const void* q; const void* k; const void* v; const void* g; const void* beta;
  int dt_q, dt_k, dt_v, dt_g, dt_beta;
  const float* h0;        // initial state / paged pool (may be null)
  float* ht;              // final state (may be null); the pool itself when paged
  void* out; int dt_out;
  const int32_t* cu_seqlens;     // null = dense [B, T]
  const int32_t* state_indices;  // null = sequence i uses row i
  int64_t slot_stride;           // elements between pool slots
  int num_slots;
  int nseq, T, H, K, V;
  float scale;
};

template <int KR, int VEC, int MINB>
__global__ void __launch_bounds__(256, MINB) kda_scan_kernel(const ScanParams p) {
  constexpr int BV = 32 * VEC;
  constexpr int NW = 8;
  __shared__ float s_q[2][256], s_k[2][256], s_d[2][256];
  __shared__ float s_red[2][2][NW][BV];
  __shared__ float s_qk[2][NW];
  __shared__ float s_beta[2];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vtiles = (p.V + BV - 1) / BV;
  const int vt = blockIdx.x % vtiles;
  const int sh = blockIdx.x / vtiles;
  const int head = sh % p.H, seq = sh / p.H;
  const int K = p.K, V = p.V, H = p.H;
  int64_t bos, eos;
  if (p.cu_seqlens) { bos = p.cu_seqlens[seq]; eos = p.cu_seqlens[seq + 1]; }
  else { bos = (int64_t)seq * p.T; eos = bos + p.T; }
  const int c0 = vt * BV + lane * VEC;

  int64_t slot = seq;
  bool active = true;
  if (p.state_indices) {
    int si = p.state_indices[seq];
    active = si > 0 && si < p.num_slots;   // non-positive (or out of range) slots are padding
    slot = si;
  }
  if (!active) {  // padding rows produce zero output and leave the pool untouched
    if (warp == 0)
      for (int64_t t = bos; t < eos; ++t)
        for (int j = 0; j < VEC; ++j)
          if (c0 + j < V) store_from_float(p.out, p.dt_out, (t * H + head) * V + c0 + j, 0.f);
    return;
  }
  const bool paged = p.state_indices != nullptr;
  const float* sin = p.h0 ? p.h0 + (paged ? slot * p.slot_stride : (int64_t)seq * H * K * V) +
                                (int64_t)head * K * V : nullptr;
  float* sout = paged ? const_cast<float*>(sin)
                      : (p.ht ? p.ht + ((int64_t)seq * H + head) * K * V : nullptr);

  float S[KR][VEC];
#pragma unroll
  for (int i = 0; i < KR; ++i) {
    int r = i * NW + warp;
#pragma unroll
    for (int j = 0; j < VEC; ++j) S[i][j] = 0.f;
    if (sin && r < K) {
      if (VEC == 4 && c0 + 3 < V) {
        float4 x = *reinterpret_cast<const float4*>(sin + (int64_t)r * V + c0);
        S[i][0] = x.x; S[i][1] = x.y; S[i][2] = x.z; S[i][3] = x.w;
      } else if (VEC == 2 && c0 + 1 < V) {
        float2 x = *reinterpret_cast<const float2*>(sin + (int64_t)r * V + c0);
        S[i][0] = x.x; S[i][1] = x.y;
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j)
          if (c0 + j < V) S[i][j] = sin[(int64_t)r * V + c0 + j];
      }
    }
  }

  // stage token `t` into parity buffer `b`: q*scale, k, 2^g, beta
  auto stage = [&](int64_t t, int b) {
    int64_t base = (t * H + head) * K;
    for (int r = tid; r < K; r += 256) {
      s_q[b][r] = load_as_float(p.q, p.dt_q, base + r) * p.scale;
      s_k[b][r] = load_as_float(p.k, p.dt_k, base + r);
      s_d[b][r] = exp2f(load_as_float(p.g, p.dt_g, base + r));
    }
    if (tid == 0) s_beta[b] = load_as_float(p.beta, p.dt_beta, t * H + head);
  };

  if (bos < eos) stage(bos, 0);
  for (int64_t t = bos; t < eos; ++t) {
    const int b = (int)((t - bos) & 1);
    float vv[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      vv[j] = (c0 + j < V) ? load_as_float(p.v, p.dt_v, (t * H + head) * V + c0 + j) : 0.f;
    __syncthreads();  // staged token visible; previous step's readers are done
    float pk[VEC], pq[VEC], pqk = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) { pk[j] = 0.f; pq[j] = 0.f; }
#pragma unroll
    for (int i = 0; i < KR; ++i) {
      int r = i * NW + warp;
      if (r < K) {
        float d = s_d[b][r], kk = s_k[b][r], qq = s_q[b][r];
        pqk += qq * kk;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          float s = S[i][j] * d;
          S[i][j] = s;
          pk[j] += kk * s;
          pq[j] += qq * s;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      s_red[b][0][warp][lane * VEC + j] = pk[j];
      s_red[b][1][warp][lane * VEC + j] = pq[j];
    }
    if (lane == 0) s_qk[b][warp] = pqk;
    if (t + 1 < eos) stage(t + 1, b ^ 1);  // overlaps the exchange below
    __syncthreads();
    float qk = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) qk += s_qk[b][w];
    const float bt = s_beta[b];
    float delta[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float a = 0.f, o = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        a += s_red[b][0][w][lane * VEC + j];
        o += s_red[b][1][w][lane * VEC + j];
      }
      delta[j] = bt * (vv[j] - a);
      o += qk * delta[j];
      if (warp == 0 && c0 + j < V)
        store_from_float(p.out, p.dt_out, (t * H + head) * V + c0 + j, o);
    }
#pragma unroll
    for (int i = 0; i < KR; ++i) {
      int r = i * NW + warp;
      if (r < K) {
        float kk = s_k[b][r];
#pragma unroll
        for (int j = 0; j < VEC; ++j) S[i][j] += kk * delta[j];
      }
    }
  }

  if (sout) {
#pragma unroll
    for (int i = 0; i < KR; ++i) {
      int r = i * NW + warp;
      if (r < K) {
        if (VEC == 4 && c0 + 3 < V) {
          *reinterpret_cast<float4*>(sout + (int64_t)r * V + c0) =
              make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
        } else if (VEC == 2 && c0 + 1 < V) {
          *reinterpret_cast<float2*>(sout + (int64_t)r * V + c0) = make_float2(S[i][0], S[i][1]);
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j)
            if (c0 + j < V) sout[(int64_t)r * V + c0 + j] = S[i][j];
        }
      }
    }
  }
}

template <int KR, int VEC, int MINB = 1>
static int launch_scan(const ScanParams& p, cudaStream_t stream) {
  constexpr int BV = 32 * VEC;
  int64_t blocks = (int64_t)p.nseq * p.H * ((p.V + BV - 1) / BV);
  if (blocks <= 0) return KDA_OK;
  if (blocks > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  StageScope timing(kStageRecurrent, stream);
  kda_scan_kernel<KR, VEC, MINB><<<(unsigned)blocks, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

}  // namespace kda

extern "C" int kda_recurrent_fwd(const void* q, const void* k, const void* v, const void* gate,
                                 const void* beta, int dt_q, int dt_k, int dt_v, int dt_gate,
                                 int dt_beta, const float* initial_state, float* final_state,
                                 void* out, int dt_out, const int32_t* cu_seqlens,
                                 const int32_t* state_indices, int64_t slot_stride, int num_slots,
                                 int nseq, int tokens_per_row, int heads, int key_dim,
                                 int value_dim, float scale, void* stream) {
  using namespace kda;
  if (!q || !k || !v || !gate || !beta || !out) return KDA_ERR_ARG;
  if (nseq < 0 || heads <= 0 || key_dim <= 0 || key_dim > 256 || value_dim <= 0)
    return KDA_ERR_ARG;
  if (state_indices && !initial_state) return KDA_ERR_ARG;
  ScanParams p;
  p.q = q; p.k = k; p.v = v; p.g = gate; p.beta = beta;
  p.dt_q = dt_q; p.dt_k = dt_k; p.dt_v = dt_v; p.dt_g = dt_gate; p.dt_beta = dt_beta;
  p.h0 = initial_state; p.ht = final_state; p.out = out; p.dt_out = dt_out;
  p.cu_seqlens = cu_seqlens; p.state_indices = state_indices;
  p.slot_stride = slot_stride; p.num_slots = num_slots;
  p.nseq = nseq; p.T = tokens_per_row; p.H = heads; p.K = key_dim; p.V = value_dim;
  p.scale = scale;
  cudaStream_t s = (cudaStream_t)stream;
  // Wide column slabs (float4 rows) when the state rows allow 16-byte accesses and there are
  // enough (sequence, head) pairs to fill the machine; otherwise 32-column slabs for parallelism.
  bool vec4 = (value_dim % 4 == 0) && (slot_stride % 4 == 0) &&
              ((int64_t)nseq * heads * ((value_dim + 127) / 128) >= 296 || value_dim > 1024);
  int kr = (key_dim + 7) / 8;
  if (vec4) {
    if (kr <= 4) return launch_scan<4, 4>(p, s);
    if (kr <= 8) return launch_scan<8, 4>(p, s);
    if (kr <= 16) return launch_scan<16, 4, 2>(p, s);  // two CTAs per SM: loads overlap stores
    return launch_scan<32, 1>(p, s);
  }
  if (kr <= 4) return launch_scan<4, 1>(p, s);
  if (kr <= 8) return launch_scan<8, 1>(p, s);
  if (kr <= 16) return launch_scan<16, 1>(p, s);
  return launch_scan<32, 1>(p, s);
}
