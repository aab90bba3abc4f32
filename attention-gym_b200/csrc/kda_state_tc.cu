// Inter-chunk state recurrence on the 5th-generation tensor cores (tcgen05 / UMMA), forward.
//
//   v_new = u - w h ;  o = qg h + Aqk v_new ;  h <- diag(2^{G_last}) h + kg^T v_new
//
// One CTA (128 threads) walks the chunks of one (sequence, head).  The fp32 state h [128 x 128]
// lives in tensor memory for the whole walk (128 lanes x 128 columns) and never goes to HBM in
// the forward pass; a second 128-column accumulator holds [w h ; qg h + Aqk v_new].
// Per chunk:
//   a. every thread (= state row kappa = TMEM lane) reads its row of h, writes it as bf16 into the
//      swizzled MN-major B tile, multiplies by the chunk decay and stores it back to TMEM;
//   b. UMMA 128x128x128:  D1 = [w ; qg] h          (A: TMA tile, K-major; B: the h tile)
//   c. threads 0..63 read D1 rows 0..63, form v_new = u - w h, write it as the bf16 B tile;
//   d. UMMA 128x128x64:   D1 += [0 ; Aqk] v_new    and   h += kg^T v_new  (A: kg, MN-major)
//   e. threads 64..127 read D1 rows 64..127 and store o.
// w, qg, kg, u, Aqk tiles arrive by TMA (128-byte swizzle) into a two-stage ring, one chunk ahead.
// Replaces the reference's fwd/triton/chunk_delta_h.py:40-162 + fwd/triton/chunk_gla_fwd_o.py:202-226.
// Every barrier wait is bounded; a wait that runs out raises the error word and the CTA leaves.
#include "kda_common.cuh"
#include "kda_sm100.cuh"
#include "kda_timing.cuh"

namespace kda {

using namespace sm100;
constexpr int D = 128;

struct StateTcParams {
  CUtensorMap tm_w, tm_qg, tm_kg, tm_u, tm_aqk;
  const float* g; const float* h0; float* ht;
  bf16* o; bf16* h_out; bf16* vnew_out;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int* error;
  int nseq, H;
  int use_u, use_o;
};

constexpr int kStageBytes = 32768 + 16384 + 16384 + 16384;   // A1, KG, U, A2
struct StateTcLayout {
  static constexpr int A1 = 0, KG = 32768, U = 49152, A2 = 65536;
  static constexpr int H = 2 * kStageBytes;              // 163840
  static constexpr int VN = H + 32768;                   // 196608
  static constexpr int BAR = VN + 16384;                 // 212992
  static constexpr int TOTAL = BAR + 1024;
};

__device__ __forceinline__ void pack8(const float* x, uint4& o) {
  o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]);
  o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
}

__global__ void __launch_bounds__(128) kda_state_fwd_tc_kernel(const __grid_constant__ StateTcParams p) {
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment by offset, so the compiler still knows this is shared memory
  unsigned char* smem = smem_dyn + ((1024u - (saddr(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + StateTcLayout::BAR);        // [2]
  uint64_t* bar_mma1 = bar_full + 2;
  uint64_t* bar_mma2 = bar_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_full + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bar_full + 5);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int H = p.H;
  const int head = blockIdx.x % H, seq = blockIdx.x / H;
  const int64_t bos = p.cu_seqlens[seq], eos = p.cu_seqlens[seq + 1];
  const int chunk0 = p.chunk_offsets[seq];
  const int nchunks = p.chunk_offsets[seq + 1] - chunk0;
  const int64_t sbase = ((int64_t)seq * H + head) * D * D;

  if (warp == 0) tmem_alloc(tmem_slot, 256);
  if (tid == 0) {
    mbar_init(&bar_full[0], 1); mbar_init(&bar_full[1], 1);
    mbar_init(bar_mma1, 1); mbar_init(bar_mma2, 1);
    mbar_init_fence();
    *s_abort = 0;
    tma_prefetch_desc(&p.tm_w); tma_prefetch_desc(&p.tm_qg); tma_prefetch_desc(&p.tm_kg);
    tma_prefetch_desc(&p.tm_u); tma_prefetch_desc(&p.tm_aqk);
  }
  // rows 0..63 of both A2 tiles stay zero: [0 ; Aqk] keeps the UMMA at M = 128
  for (int idx = tid; idx < 2 * 512; idx += 128) {
    int st = idx >> 9, off = (idx & 511) * 16;
    *reinterpret_cast<uint4*>(smem + st * kStageBytes + StateTcLayout::A2 + off) = make_uint4(0, 0, 0, 0);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = (uint32_t)(32 * warp) << 16;
  const uint32_t tDh = tmem + lane_off, tD1 = tmem + 128 + lane_off;

  auto chunk_valid = [&](int c) {
    int64_t rem = eos - (bos + (int64_t)c * 64);
    return rem >= 64 ? 64 : (int)rem;
  };
  auto issue_stage = [&](int c) {   // thread 0 only
    unsigned char* st = smem + (c & 1) * kStageBytes;
    uint64_t* bar = &bar_full[c & 1];
    const int y = (int)(bos + (int64_t)c * 64);
    const int x = head * D;
    uint32_t bytes = 2 * 8192 + 2 * 8192;                       // w, kg
    if (p.use_u) bytes += 2 * 8192;
    if (p.use_o) bytes += 2 * 8192 + 8192;                       // qg, Aqk
    mbar_expect_tx(bar, bytes);
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(st + StateTcLayout::A1 + b * 16384, &p.tm_w, x + 64 * b, y, bar);
      tma_load_2d(st + StateTcLayout::KG + b * 8192, &p.tm_kg, x + 64 * b, y, bar);
      if (p.use_u) tma_load_2d(st + StateTcLayout::U + b * 8192, &p.tm_u, x + 64 * b, y, bar);
      if (p.use_o) tma_load_2d(st + StateTcLayout::A1 + b * 16384 + 8192, &p.tm_qg, x + 64 * b, y, bar);
    }
    if (p.use_o) tma_load_2d(st + StateTcLayout::A2 + 8192, &p.tm_aqk, head * 64, y, bar);
  };

  if (tid == 0) {
    if (nchunks > 0) issue_stage(0);
    if (nchunks > 1) issue_stage(1);
  }
  // initial state -> tensor memory (this thread owns state row `tid`)
  {
    float x[32];
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.h0) v4 = *reinterpret_cast<const float4*>(p.h0 + sbase + (int64_t)tid * D + 32 * cb + i);
        x[i] = v4.x; x[i + 1] = v4.y; x[i + 2] = v4.z; x[i + 3] = v4.w;
      }
      tmem_st32(tDh + 32 * cb, x);
    }
    tmem_st_wait();
  }
  const uint32_t idesc_kmn = instr_desc(128, 128, 0, 1);
  const uint32_t idesc_mnmn = instr_desc(128, 128, 1, 1);
  const uint32_t sH = saddr(smem + StateTcLayout::H), sVN = saddr(smem + StateTcLayout::VN);
  bool failed = false;

  float glast = 0.f;
  if (nchunks > 0)
    glast = p.g[((bos + chunk_valid(0) - 1) * H + head) * D + tid];

  for (int c = 0; c < nchunks; ++c) {
    unsigned char* st = smem + (c & 1) * kStageBytes;
    const int64_t token0 = bos + (int64_t)c * 64;
    const int valid = chunk_valid(c);
    const float dec = exp2f(glast);
    if (c + 1 < nchunks)
      glast = p.g[((token0 + 64 + chunk_valid(c + 1) - 1) * H + head) * D + tid];

    // ---- a. h row -> bf16 B tile (MN-major: rows kappa, boxes = 64-wide v halves); decay in place
    {
      float x[32];
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        tmem_ld32(tDh + 32 * cb, x);
        unsigned char* box = smem + StateTcLayout::H + (cb >> 1) * 16384;
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          uint4 v;
          pack8(x + 8 * qd, v);
          *reinterpret_cast<uint4*>(box + sw128_chunk(tid, (cb & 1) * 4 + qd)) = v;
          if (p.h_out)
            *reinterpret_cast<uint4*>(p.h_out + (((int64_t)(chunk0 + c) * H + head) * D + tid) * D +
                                      32 * cb + 8 * qd) = v;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] *= dec;
        tmem_st32(tDh + 32 * cb, x);
      }
      tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) { failed = true; break; }

    // ---- b. D1 = [w ; qg] h ----------------------------------------------------------------
    if (tid == 0) {
      if (!mbar_wait(&bar_full[c & 1], (c >> 1) & 1)) *s_abort = 1;
      tc_fence_after();
      const uint32_t a1 = saddr(st + StateTcLayout::A1);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + 128, desc_kmajor(a1, ks, 16384), desc_mnmajor(sH, ks, 16384), idesc_kmn, ks > 0);
      umma_commit(bar_mma1);
    }

    // ---- c. v_new = u - w h (threads 0..63); zero the kg rows past a partial chunk (64..127) ---
    if (!mbar_wait(&bar_full[c & 1], (c >> 1) & 1)) *s_abort = 1;
    if (tid < 64) {
      if (!mbar_wait(bar_mma1, c & 1)) *s_abort = 1;
      tc_fence_after();
      float x[32];
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        tmem_ld32(tD1 + 32 * cb, x);
        const unsigned char* ubox = st + StateTcLayout::U + (cb >> 1) * 8192;
        unsigned char* vbox = smem + StateTcLayout::VN + (cb >> 1) * 8192;
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          const int off = sw128_chunk(tid, (cb & 1) * 4 + qd);
          float y[8];
          if (p.use_u) {
            uint4 u4 = *reinterpret_cast<const uint4*>(ubox + off);
            float2 a = unpack_bf16(u4.x), b = unpack_bf16(u4.y), cc = unpack_bf16(u4.z),
                   d = unpack_bf16(u4.w);
            y[0] = a.x; y[1] = a.y; y[2] = b.x; y[3] = b.y; y[4] = cc.x; y[5] = cc.y; y[6] = d.x; y[7] = d.y;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] = tid < valid ? y[i] - x[8 * qd + i] : 0.f;
          uint4 v;
          pack8(y, v);
          *reinterpret_cast<uint4*>(vbox + off) = v;
          if (p.vnew_out && tid < valid)
            *reinterpret_cast<uint4*>(p.vnew_out + ((token0 + tid) * H + head) * D + 32 * cb + 8 * qd) = v;
        }
      }
    } else if (valid < 64) {
      // rows >= valid of the kg tile hold another sequence's tokens (or unwritten memory)
      for (int idx = tid - 64; idx < (64 - valid) * 16; idx += 64) {
        int r = valid + (idx >> 4), ch = idx & 15;
        *reinterpret_cast<uint4*>(st + StateTcLayout::KG + (ch >> 3) * 8192 + sw128_chunk(r, ch & 7)) =
            make_uint4(0, 0, 0, 0);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) { failed = true; break; }

    // ---- d. D1 += [0 ; Aqk] v_new ;  h += kg^T v_new ----------------------------------------
    if (tid == 0) {
      tc_fence_after();
      const uint32_t a2 = saddr(st + StateTcLayout::A2), kg = saddr(st + StateTcLayout::KG);
      if (p.use_o) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma(tmem + 128, desc_kmajor(a2, ks, 0), desc_mnmajor(sVN, ks, 8192), idesc_kmn, 1);
      }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem, desc_mnmajor(kg, ks, 8192), desc_mnmajor(sVN, ks, 8192), idesc_mnmn, 1);
      umma_commit(bar_mma2);
    }
    if (!mbar_wait(bar_mma2, c & 1)) *s_abort = 1;
    tc_fence_after();
    if (tid == 0 && c + 2 < nchunks) issue_stage(c + 2);

    // ---- e. o rows (threads 64..127) ----------------------------------------------------------
    if (p.use_o && tid >= 64) {   // warp-uniform: tensor-memory loads are whole-warp operations
      float x[32];
      const bool live = tid - 64 < valid;
      bf16* orow = p.o + ((token0 + (live ? tid - 64 : 0)) * H + head) * D;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        tmem_ld32(tD1 + 32 * cb, x);
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          uint4 v;
          pack8(x + 8 * qd, v);
          if (live) *reinterpret_cast<uint4*>(orow + 32 * cb + 8 * qd) = v;
        }
      }
    }
  }

  if (!failed && p.ht) {
    float x[32];
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
      tmem_ld32(tDh + 32 * cb, x);
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(p.ht + sbase + (int64_t)tid * D + 32 * cb + i) =
            make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    }
  }
  if (failed && tid == 0 && p.error) atomicExch(p.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

static __device__ int g_state_tc_error = 0;

// ---- host side: tensor maps --------------------------------------------------------------------
int launch_state_fwd_tc(const bf16* w, const bf16* u, const bf16* kg, const bf16* qg, const bf16* aqk,
                        const float* g, const float* h0, float* ht, bf16* o, bf16* h_out,
                        bf16* vnew_out, const int32_t* cu, const int32_t* co, int nseq, int H,
                        int64_t tokens, cudaStream_t s) {
  if (nseq == 0) return KDA_OK;
  StateTcParams p;
  int* error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&error), g_state_tc_error) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  const int64_t cols = (int64_t)H * D;
  if (!make_tensor_map(&p.tm_w, w, tokens, cols, 64) || !make_tensor_map(&p.tm_kg, kg, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_qg, qg, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_u, u ? u : w, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_aqk, aqk, tokens, (int64_t)H * 64, 64))
    return KDA_ERR_LAUNCH;
  p.g = g; p.h0 = h0; p.ht = ht; p.o = o; p.h_out = h_out; p.vnew_out = vnew_out;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.error = error; p.nseq = nseq; p.H = H;
  p.use_u = u != nullptr; p.use_o = o != nullptr;
  const int smem = StateTcLayout::TOTAL + 1024;
  if (cudaFuncSetAttribute(kda_state_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
      cudaSuccess)
    return KDA_ERR_LAUNCH;
  StageScope timing(kStageStateFwd, s);
  kda_state_fwd_tc_kernel<<<(unsigned)(nseq * H), 128, smem, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}


// ------------------------------------------------------------------------------------------------
// Reverse state-gradient recurrence on tcgen05:
//   dv2 = kg dh + Aqk^T dO ;  dh <- diag(2^{G_last}) dh + qg^T dO - w^T dv2 ;  dh0 at the end.
// Same structure as the forward walk: dh [128 x 128] fp32 lives in tensor memory, one CTA per
// (sequence, head), chunks in reverse order, TMA two-stage ring.  Replaces the reference's
// bwd/triton/chunk_kda_bwd_dav.py:73-93 + bwd/cute/chunk_delta_h_bwd_v1.py:1147-1276.
// ------------------------------------------------------------------------------------------------
struct StateBwdTcParams {
  CUtensorMap tm_w, tm_qg, tm_kg, tm_do, tm_aqk;
  const float* g; const float* dht; float* dh0;
  bf16* dh_out; bf16* dv2_out;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int* error;
  int nseq, H;
};

constexpr int kBStageBytes = 4 * 16384 + 8192;   // KG, W, QG, DO, AQK
struct StateBwdLayout {
  static constexpr int KG = 0, W = 16384, QG = 32768, DO = 49152, AQK = 65536;
  static constexpr int DH = 2 * kBStageBytes;            // 147456
  static constexpr int DV2 = DH + 32768;                 // 180224
  static constexpr int BAR = DV2 + 16384;                // 196608
  static constexpr int TOTAL = BAR + 1024;
};

__global__ void __launch_bounds__(128) kda_state_bwd_tc_kernel(const __grid_constant__ StateBwdTcParams p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = smem_dyn + ((1024u - (saddr(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + StateBwdLayout::BAR);
  uint64_t* bar_mma1 = bar_full + 2;
  uint64_t* bar_mma2 = bar_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_full + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bar_full + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lid = tid & 31;
  const int H = p.H;
  const int head = blockIdx.x % H, seq = blockIdx.x / H;
  const int64_t bos = p.cu_seqlens[seq], eos = p.cu_seqlens[seq + 1];
  const int chunk0 = p.chunk_offsets[seq];
  const int nchunks = p.chunk_offsets[seq + 1] - chunk0;
  const int64_t sbase = ((int64_t)seq * H + head) * D * D;

  if (warp == 0) tmem_alloc(tmem_slot, 256);
  if (tid == 0) {
    mbar_init(&bar_full[0], 1); mbar_init(&bar_full[1], 1);
    mbar_init(bar_mma1, 1); mbar_init(bar_mma2, 1);
    mbar_init_fence();
    *s_abort = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = (uint32_t)(32 * warp) << 16;
  const uint32_t tDh = tmem + lane_off, tDv = tmem + 128 + lane_off;

  auto chunk_valid = [&](int c) {
    int64_t rem = eos - (bos + (int64_t)c * 64);
    return rem >= 64 ? 64 : (int)rem;
  };
  auto issue_stage = [&](int it) {   // thread 0 only; iteration `it` handles chunk nchunks-1-it
    const int c = nchunks - 1 - it;
    unsigned char* st = smem + (it & 1) * kBStageBytes;
    uint64_t* bar = &bar_full[it & 1];
    const int y = (int)(bos + (int64_t)c * 64);
    const int x = head * D;
    mbar_expect_tx(bar, kBStageBytes);
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(st + StateBwdLayout::KG + b * 8192, &p.tm_kg, x + 64 * b, y, bar);
      tma_load_2d(st + StateBwdLayout::W + b * 8192, &p.tm_w, x + 64 * b, y, bar);
      tma_load_2d(st + StateBwdLayout::QG + b * 8192, &p.tm_qg, x + 64 * b, y, bar);
      tma_load_2d(st + StateBwdLayout::DO + b * 8192, &p.tm_do, x + 64 * b, y, bar);
    }
    tma_load_2d(st + StateBwdLayout::AQK, &p.tm_aqk, head * 64, y, bar);
  };
  if (tid == 0) {
    if (nchunks > 0) issue_stage(0);
    if (nchunks > 1) issue_stage(1);
  }
  {
    float x[32];
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.dht) v4 = *reinterpret_cast<const float4*>(p.dht + sbase + (int64_t)tid * D + 32 * cb + i);
        x[i] = v4.x; x[i + 1] = v4.y; x[i + 2] = v4.z; x[i + 3] = v4.w;
      }
      tmem_st32(tDh + 32 * cb, x);
    }
    tmem_st_wait();
  }
  const uint32_t sDH = saddr(smem + StateBwdLayout::DH), sDV2 = saddr(smem + StateBwdLayout::DV2);
  bool failed = false;

  float glast = 0.f;
  if (nchunks > 0)
    glast = p.g[((bos + (int64_t)(nchunks - 1) * 64 + chunk_valid(nchunks - 1) - 1) * H + head) * D + tid];

  for (int it = 0; it < nchunks; ++it) {
    const int c = nchunks - 1 - it;
    unsigned char* st = smem + (it & 1) * kBStageBytes;
    const int64_t token0 = bos + (int64_t)c * 64;
    const int valid = chunk_valid(c);
    const float dec = exp2f(glast);
    if (c > 0) glast = p.g[((token0 - 1) * H + head) * D + tid];   // last row of the previous chunk

    if (!mbar_wait(&bar_full[it & 1], (it >> 1) & 1)) *s_abort = 1;
    if (valid < 64) {
      // rows past the tail hold another sequence's tokens or unwritten memory: they are contraction
      // rows of w, qg, dO and Aqk
      for (int idx = tid; idx < (64 - valid) * 16; idx += 128) {
        const int r = valid + (idx >> 4), ch = idx & 15;
        const int off = (ch >> 3) * 8192 + sw128_chunk(r, ch & 7);
        *reinterpret_cast<uint4*>(st + StateBwdLayout::W + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(st + StateBwdLayout::QG + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(st + StateBwdLayout::DO + off) = make_uint4(0, 0, 0, 0);
        if (ch < 8)
          *reinterpret_cast<uint4*>(st + StateBwdLayout::AQK + sw128_chunk(r, ch)) = make_uint4(0, 0, 0, 0);
      }
    }
    // ---- a. dh row -> bf16 B tile + global copy; decay in place ---------------------------------
    {
      float x[32];
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        tmem_ld32(tDh + 32 * cb, x);
        unsigned char* box = smem + StateBwdLayout::DH + (cb >> 1) * 16384;
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          uint4 v;
          pack8(x + 8 * qd, v);
          *reinterpret_cast<uint4*>(box + sw128_chunk(tid, (cb & 1) * 4 + qd)) = v;
          *reinterpret_cast<uint4*>(p.dh_out + (((int64_t)(chunk0 + c) * H + head) * D + tid) * D +
                                    32 * cb + 8 * qd) = v;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] *= dec;
        tmem_st32(tDh + 32 * cb, x);
      }
      tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) { failed = true; break; }

    // ---- b. dv2 = kg dh + Aqk^T dO ;  dh += qg^T dO ------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      const uint32_t kg = saddr(st + StateBwdLayout::KG), qg = saddr(st + StateBwdLayout::QG),
                     dO = saddr(st + StateBwdLayout::DO), aqk = saddr(st + StateBwdLayout::AQK);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + 128, desc_kmajor(kg, ks, 8192), desc_mnmajor(sDH, ks, 16384),
             instr_desc(64, 128, 0, 1), ks > 0);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem + 128, desc_mnmajor(aqk, ks, 0), desc_mnmajor(dO, ks, 8192), instr_desc(64, 128, 1, 1), 1);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem, desc_mnmajor(qg, ks, 8192), desc_mnmajor(dO, ks, 8192), instr_desc(128, 128, 1, 1), 1);
      umma_commit(bar_mma1);
    }
    if (!mbar_wait(bar_mma1, it & 1)) *s_abort = 1;
    tc_fence_after();
    // ---- c. dv2 rows (M = 64 accumulator: row j on lane 32 (j / 16) + j % 16) -----------------------
    {
      float x[32];
      const int j = warp * 16 + lid;
      const bool row = lid < 16;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        tmem_ld32(tDv + 32 * cb, x);
        if (row) {
          unsigned char* box = smem + StateBwdLayout::DV2 + (cb >> 1) * 8192;
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j < valid) pack8(x + 8 * qd, v);
            *reinterpret_cast<uint4*>(box + sw128_chunk(j, (cb & 1) * 4 + qd)) = v;
            if (j < valid)
              *reinterpret_cast<uint4*>(p.dv2_out + ((token0 + j) * H + head) * D + 32 * cb + 8 * qd) = v;
          }
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) { failed = true; break; }

    // ---- d. dh -= w^T dv2 ------------------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      const uint32_t w = saddr(st + StateBwdLayout::W);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem, desc_mnmajor(w, ks, 8192), desc_mnmajor(sDV2, ks, 8192), instr_desc(128, 128, 1, 1, 1), 1);
      umma_commit(bar_mma2);
    }
    if (!mbar_wait(bar_mma2, it & 1)) *s_abort = 1;
    tc_fence_after();
    if (tid == 0 && it + 2 < nchunks) issue_stage(it + 2);
  }

  if (!failed && p.dh0) {
    float x[32];
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
      tmem_ld32(tDh + 32 * cb, x);
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(p.dh0 + sbase + (int64_t)tid * D + 32 * cb + i) =
            make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    }
  }
  if (failed && tid == 0 && p.error) atomicExch(p.error, 16);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

int launch_state_bwd_tc(const bf16* w, const bf16* kg, const bf16* qg, const bf16* aqk, const bf16* dout,
                        const float* g, const float* dht, float* dh0, bf16* dh_out, bf16* dv2_out,
                        const int32_t* cu, const int32_t* co, int nseq, int H, int64_t tokens,
                        cudaStream_t s) {
  if (nseq == 0) return KDA_OK;
  StateBwdTcParams p;
  const int64_t cols = (int64_t)H * D;
  if (!make_tensor_map(&p.tm_w, w, tokens, cols, 64) || !make_tensor_map(&p.tm_kg, kg, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_qg, qg, tokens, cols, 64) || !make_tensor_map(&p.tm_do, dout, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_aqk, aqk, tokens, (int64_t)H * 64, 64))
    return KDA_ERR_LAUNCH;
  p.g = g; p.dht = dht; p.dh0 = dh0; p.dh_out = dh_out; p.dv2_out = dv2_out;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.nseq = nseq; p.H = H;
  p.error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), g_state_tc_error) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  const int smem = StateBwdLayout::TOTAL + 1024;
  if (cudaFuncSetAttribute(kda_state_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
      cudaSuccess)
    return KDA_ERR_LAUNCH;
  StageScope timing(kStageStateBwd, s);
  kda_state_bwd_tc_kernel<<<(unsigned)(nseq * H), 128, smem, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

}  // namespace kda

// 1 if a tensor-memory kernel gave up on a barrier wait since the last call (clears the flag).
// Synchronises the device; meant for tests and debugging.
namespace kda { int bwd_chunk_tc_error_word(); }

extern "C" int kda_device_error_word(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, kda::g_state_tc_error, sizeof(int)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(kda::g_state_tc_error, &zero, sizeof(int));
  return v | (kda::bwd_chunk_tc_error_word() << 8);
}
