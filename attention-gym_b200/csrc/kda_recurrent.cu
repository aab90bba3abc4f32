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
#include "kda_sm100.cuh"
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

// ------------------------------------------------------------------------------------------------
// Decode step (one token per sequence) for K = V = 128 with an fp32 state: pure state streaming,
// 2 x 64 KiB per (sequence, head).  Persistent CTAs move the states as [128 x 32] column slabs (TMA
// tiles) through four independent three-stage shared-memory rings, one per column group -- a slab
// arriving, one being updated in place, one leaving -- so loads, stores and arithmetic overlap.
// 16 arithmetic warps: thread (group = tid / 128, warp-in-group w, lane) owns column 32 group + lane
// and the key rows 32 w .. 32 w + 31 of it; the two K-reductions cross the four warps of a group
// through shared memory and a 128-thread named barrier.  Four more warps are the producers: one
// thread per column group issues its loads and stores, paced by a full / done mbarrier pair per
// stage.
// ------------------------------------------------------------------------------------------------
constexpr int kDecStages = 3;            // per column group
constexpr int kDecSlabBytes = 128 * 32 * 4;   // one [128 x 32] fp32 column slab of a state
constexpr int kDecRingBytes = 4 * kDecStages * kDecSlabBytes;
constexpr int kDecOpsFloats = 448;       // one operand slot (418 floats used)
constexpr int kDecTailBytes = 20480;     // barriers, token operands, reduction scratch (18.3 KiB used)
constexpr int kDecSmemBytes = kDecRingBytes + kDecTailBytes;
constexpr int kDecConsumers = 512;       // 16 arithmetic warps; warps 16..19 move the slabs

struct DecodeMaps { CUtensorMap src, dst; };   // [state rows, 128] fp32, box 32 columns x 128 rows

long long* debug_profile_buffer();
// Debugging aid: timestamps of the 20th item of the first 64 CTAs (one thread per role).
__device__ __forceinline__ void dec_mark(long long* prof, int i, int slot) {
#ifdef KDA_PHASE_PROFILE
  if (prof && (i & 7) == 4 && blockIdx.x < 8 && slot < 4) {     // items 4, 12, 20, ... of the first 8 CTAs
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    prof[blockIdx.x * 32 + (i >> 3) * 4 + slot] = t;
  }
#endif
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sm100::saddr(bar)) : "memory");
}

__global__ void __launch_bounds__(kDecConsumers + 128, 1)
kda_decode_kernel(const ScanParams p, const __grid_constant__ DecodeMaps maps, int* error, long long* prof) {
  using namespace sm100;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* sm = smem_dyn + ((1024u - (saddr(smem_dyn) & 1023u)) & 1023u);
  unsigned char* tail = sm + kDecRingBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(tail);                  // [4 groups][3] slab has arrived
  uint64_t* done = full + 12;                                          // [4 groups][3] slab has been updated
  // token operands: per group two slots of [q 128 (pre-scaled) | k 128 | 2^g 128 | v 32 | beta | active]
  float* s_ops = reinterpret_cast<float*>(tail + 256);                 // [4 groups][2][kDecOpsFloats]
  float* s_red = s_ops + 4 * 2 * kDecOpsFloats;                        // [4 groups][2][4 warps][32]
  float* s_qk = s_red + 1024;                                          // [4][4]
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_qk + 16);
  static_assert(256 + (4 * 2 * kDecOpsFloats + 1024 + 16 + 1) * 4 <= kDecTailBytes, "tail region too small");

  const int tid = threadIdx.x, lane = tid & 31;
  const int H = p.H, items = p.nseq * H;
  const bool paged = p.state_indices != nullptr;
  const int stride = (int)gridDim.x;

  // slot of sequence `seq`: >= 0 active, -1 padding (non-positive or out-of-range pool index)
  auto slot_of = [&](int seq) -> int64_t {
    if (!paged) return seq;
    const int si = p.state_indices[seq];
    return (si > 0 && si < p.num_slots) ? si : -1;
  };

  if (tid == 0) {
    for (int s = 0; s < 4 * kDecStages; ++s) { mbar_init(&full[s], 1); mbar_init(&done[s], 4); }
    mbar_init_fence();
    *s_abort = 0;
  }
  __syncthreads();

  if (tid >= kDecConsumers) {
    // ---- producer warps: one thread per column group moves its slabs in and out ------------------------
    // A stage cycles load -> (consumers) -> store -> load of the slab three items on.  Pool slots are
    // looked up one item before they are needed, so no copy waits for a plain global load.
    if (lane != 0) return;
    const int g = (tid - kDecConsumers) >> 5;
    unsigned char* ring = sm + g * kDecStages * kDecSlabBytes;
    uint64_t* gfull = full + g * kDecStages;
    uint64_t* gdone = done + g * kDecStages;
    const int rows_per_slot = paged ? (int)(p.slot_stride / 128) : H * 128;
    auto row_of = [&](int n, int64_t slot) {       // first tensor-map row of the state of item n
      const int seq = n / H, head = n - seq * H;
      return (int)((paged ? slot : (int64_t)seq) * rows_per_slot) + head * 128;
    };
    int64_t held[kDecStages];                      // slot of the slab each stage holds (-1 = none)
    auto load = [&](int n, int s, int64_t slot) {
      if (n >= items || slot < 0) return;
      mbar_expect_tx(&gfull[s], kDecSlabBytes);
      tma_load_2d(ring + s * kDecSlabBytes, &maps.src, 32 * g, row_of(n, slot), &gfull[s]);
    };
    auto lookup = [&](int n) -> int64_t { return n < items ? slot_of(n / H) : -1; };
#pragma unroll
    for (int j = 0; j < kDecStages; ++j) {
      held[j] = lookup(blockIdx.x + j * stride);
      load(blockIdx.x + j * stride, j, held[j]);
    }
    int64_t slot_pre = lookup(blockIdx.x + kDecStages * stride);
    uint32_t phases = 0;
    int i = 0;
    for (int n = blockIdx.x; n < items; n += stride, ++i) {
      const int st = i % kDecStages;
      const int64_t slot = st == 0 ? held[0] : (st == 1 ? held[1] : held[2]);
      if (slot >= 0) {
        if (g == 0) dec_mark(prof, i, 8);
        if (!mbar_wait(&gdone[st], (phases >> st) & 1u)) { *s_abort = 1; break; }
        if (g == 0) dec_mark(prof, i, 9);
        phases ^= 1u << st;
        tma_store_2d(&maps.dst, ring + st * kDecSlabBytes, 32 * g, row_of(n, slot));
        tma_store_commit();
        tma_store_wait_read();            // the stage has been read: it takes the slab three items on
        if (g == 0) dec_mark(prof, i, 10);
      }
      load(n + kDecStages * stride, st, slot_pre);
      if (st == 0) held[0] = slot_pre; else if (st == 1) held[1] = slot_pre; else held[2] = slot_pre;
      slot_pre = lookup(n + (kDecStages + 1) * stride);
    }
    tma_store_wait_read();
    return;
  }

  // ---- consumers: four independent groups of 128 threads, one per column slab ---------------------------
  const int grp = tid >> 7, wj = (tid >> 5) & 3, ft = tid & 127;
  const int col = 32 * grp + lane;
  unsigned char* ring = sm + grp * kDecStages * kDecSlabBytes;
  uint64_t* gfull = full + grp * kDecStages;
  uint64_t* gdone = done + grp * kDecStages;
  float* gops = s_ops + grp * 2 * kDecOpsFloats;          // the group's two operand slots
  float* red = s_red + grp * 256;
  // Token operands (T = 1: token index = sequence index) are fetched three items ahead, because a
  // plain global load takes microseconds while the copies saturate the memory system.  Every group
  // fetches its own copy (thread t: q, k, gate of channel t; v of its column), so the groups never
  // wait for one another.  Three register sets rotate: set (item mod 3) holds the item's operands.
  // The register sets hold raw bits: converting at fetch time would stall on the load at once.
  struct Ops { uint32_t q, k, g, v, beta; int si; };
  auto fetch = [&](int n, Ops& r) {
    if (n < items) {
      const int seq = n / H, head = n - seq * H;
      const int64_t base = ((int64_t)seq * H + head) * 128;
      r.q = load_raw(p.q, p.dt_q, base + ft);
      r.k = load_raw(p.k, p.dt_k, base + ft);
      r.g = load_raw(p.g, p.dt_g, base + ft);
      if (ft < 32) r.v = load_raw(p.v, p.dt_v, base + 32 * grp + ft);
      if (ft == 0) {
        r.beta = load_raw(p.beta, p.dt_beta, (int64_t)seq * H + head);
        r.si = paged ? p.state_indices[seq] : 1;
      }
    }
  };
  auto publish = [&](int slot, const Ops& r) {
    float* o = gops + slot * kDecOpsFloats;
    o[ft] = raw_to_float(r.q, p.dt_q) * p.scale;
    o[128 + ft] = raw_to_float(r.k, p.dt_k);
    o[256 + ft] = exp2f(raw_to_float(r.g, p.dt_g));
    if (ft < 32) o[384 + ft] = raw_to_float(r.v, p.dt_v);
    if (ft == 0) {
      o[416] = raw_to_float(r.beta, p.dt_beta);
      o[417] = __int_as_float((!paged || (r.si > 0 && r.si < p.num_slots)) ? 1 : 0);
    }
  };
  const int lane_hi = lane >> 2, lane_lo = (lane & 3) * 4;
  uint32_t phases = 0;          // bit s = parity of the next phase of full[s] (padding items load nothing)

  // one item: `next` (item i + 1) is published at the end, `far` receives item i + 3
  auto step = [&](int i, int n, Ops& far, const Ops& next) {
    const int st = i % kDecStages;
    const float* o = gops + (i & 1) * kDecOpsFloats;
    const int seq = n / H, head = n - seq * H;
    const bool active = __float_as_int(o[417]) != 0;
    fetch(n + 3 * stride, far);
    if (tid == 0) dec_mark(prof, i, 0);
    if (active) {
      if (!mbar_wait(&gfull[st], (phases >> st) & 1u)) *s_abort = 1;   // bounded: give up, do not hang
      if (tid == 0) dec_mark(prof, i, 1);
      phases ^= 1u << st;
      // element (kappa, lane) of a slab: rows of 128 bytes, 16-byte chunks XOR-swizzled with (kappa & 7)
      unsigned char* S = ring + st * kDecSlabBytes + (32 * wj) * 128 + lane_lo;
      const float* dq = o + 32 * wj;
      const float* dk = o + 128 + 32 * wj;
      const float* dd = o + 256 + 32 * wj;
      float sr[32], pk = 0.f, pq = 0.f, pqk = 0.f;
#pragma unroll
      for (int kk = 0; kk < 32; kk += 4) {
        const float4 d4 = *reinterpret_cast<const float4*>(dd + kk);
        const float4 k4 = *reinterpret_cast<const float4*>(dk + kk);
        const float4 q4 = *reinterpret_cast<const float4*>(dq + kk);
        const float dv[4] = {d4.x, d4.y, d4.z, d4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w},
                    qv[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = kk + e;           // 32 wj is a multiple of 8: (kappa & 7) = (r & 7)
          const float s = *reinterpret_cast<const float*>(S + r * 128 + ((lane_hi ^ (r & 7)) << 4)) * dv[e];
          sr[r] = s;
          pk = fmaf(kv[e], s, pk);
          pq = fmaf(qv[e], s, pq);
          pqk = fmaf(qv[e], kv[e], pqk);
        }
      }
      red[wj * 32 + lane] = pk;
      red[128 + wj * 32 + lane] = pq;
      if (lane == 0) s_qk[grp * 4 + wj] = pqk;
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
      const float a = red[lane] + red[32 + lane] + red[64 + lane] + red[96 + lane];
      float out = red[128 + lane] + red[160 + lane] + red[192 + lane] + red[224 + lane];
      const float qk = s_qk[grp * 4] + s_qk[grp * 4 + 1] + s_qk[grp * 4 + 2] + s_qk[grp * 4 + 3];
      const float delta = o[416] * (o[384 + lane] - a);
      out = fmaf(qk, delta, out);
      if (wj == 0) store_from_float(p.out, p.dt_out, ((int64_t)seq * H + head) * 128 + col, out);
#pragma unroll
      for (int kk = 0; kk < 32; kk += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(dk + kk);
        const float kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = kk + e;
          *reinterpret_cast<float*>(S + r * 128 + ((lane_hi ^ (r & 7)) << 4)) = fmaf(kv[e], delta, sr[r]);
        }
      }
      fence_async_smem();
      __syncwarp();
      if (tid == 0) dec_mark(prof, i, 2);
      if (lane == 0) mbar_arrive(&gdone[st]);     // 4 arrivals hand the slab to the group's producer
    } else if (wj == 0) {                 // padding rows produce zero output and leave the pool untouched
      store_from_float(p.out, p.dt_out, ((int64_t)seq * H + head) * 128 + col, 0.f);
    }
    publish((i + 1) & 1, next);           // the other slot was last read one item ago
    asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");   // operands visible; scratch reusable
    if (tid == 0) dec_mark(prof, i, 3);
  };

  Ops f0{}, f1{}, f2{};                   // set (item counter mod 3)
  fetch(blockIdx.x, f0);
  publish(0, f0);
  fetch(blockIdx.x + stride, f1);
  fetch(blockIdx.x + 2 * stride, f2);
  asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
  int i = 0;
  for (int n = blockIdx.x; n < items; ) {
    step(i, n, f0, f1); ++i; n += stride;
    if (n >= items || *s_abort) break;
    step(i, n, f1, f2); ++i; n += stride;
    if (n >= items || *s_abort) break;
    step(i, n, f2, f0); ++i; n += stride;
    if (*s_abort) break;
  }
  if (*s_abort && tid == 0 && error) atomicExch(error, 64);
}

static __device__ int g_decode_error = 0;

static int launch_decode(const ScanParams& p, cudaStream_t stream) {
  const int64_t items = (int64_t)p.nseq * p.H;
  if (items <= 0) return KDA_OK;
  const bool paged = p.state_indices != nullptr;
  DecodeMaps maps;
  const int64_t rows = paged ? (int64_t)p.num_slots * (p.slot_stride / 128) : items * 128;
  if (!sm100::make_tensor_map(&maps.src, p.h0, rows, 128, 128, true) ||
      !sm100::make_tensor_map(&maps.dst, paged ? p.h0 : p.ht, rows, 128, 128, true))
    return KDA_ERR_LAUNCH;
  int dev = 0, sms = 0;
  int* error = nullptr;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1 ||
      cudaGetSymbolAddress(reinterpret_cast<void**>(&error), g_decode_error) != cudaSuccess ||
      cudaFuncSetAttribute(kda_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kDecSmemBytes + 1024) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  StageScope timing(kStageRecurrent, stream);
  kda_decode_kernel<<<(unsigned)(items < sms ? items : sms), kDecConsumers + 128, kDecSmemBytes + 1024, stream>>>(
      p, maps, error, debug_profile_buffer());
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
  // the decode step proper: one token per sequence, K = V = 128, state in and out
  const bool decode = tokens_per_row == 1 && !cu_seqlens && key_dim == 128 && value_dim == 128 &&
                      initial_state && (state_indices || final_state) && nseq * (int64_t)heads < (1 << 24) &&
                      ((uintptr_t)initial_state & 15) == 0 && ((uintptr_t)final_state & 15) == 0 &&
                      (!state_indices || (slot_stride % 128 == 0 && slot_stride >= (int64_t)heads * 16384 &&
                                          (int64_t)num_slots * (slot_stride / 128) < (1LL << 31)));
  if (decode) return launch_decode(p, s);
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
