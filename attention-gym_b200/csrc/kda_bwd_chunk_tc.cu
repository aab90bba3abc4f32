// Per-chunk backward of the chunked KDA path on tcgen05 tensor cores: one kernel replaces the
// reference's WY/dqkg stage (bwd/cute/chunk_kda_bwd_wy_dqkg_fused.py:2623, oracle
// attn_gym/testing/kda.py:144-240) and its intra-chunk stage (bwd/cute/chunk_kda_bwd_intra.py:931,
// oracle attn_gym/testing/kda.py:67-141).
//
// Everything is computed transposed, with the channel (kappa or v) on the 128 tensor-memory lanes
// and the 64 chunk rows on the columns, so every large product is a full-rate M = 128 UMMA and
// every thread owns one channel: elementwise work is "thread = channel, loop over rows", the
// per-channel reductions over rows are thread-local, and global stores are coalesced.
//
//   phase 0  TMA: h, dh, dO, v_new, dv2, v, k, q, A, G.
//            UMMA: dq^T = h dO^T, dks^T = dh v_new^T, dw^T = -h dv2^T, dAqk = dO v_new^T
//   phase 1  epilogue: dq, dk, dG partial sums in registers; dw^T and k 2^G as bf16 tiles; dAqk tile
//            UMMA: dvb^T = dv2^T A, dkgb^T = dw^T A, X = dv2 v^T + dw (k 2^G)^T
//   phase 2  epilogue: dv, dk, dG, dbeta terms; X tile
//            UMMA: Y = A^T X;  dL = -Y A^T  (two short serial products)
//   phase 3  gated operand tiles for the pairwise products (16-row gate rebasing, as in the
//            forward), UMMAs with N = 16 per row block:
//              dq_intra^T, X1^T [kappa][i in block ri] = Kn_ri^T {dAqk, dL}[i, j <= 16 ri + 15]
//              dk2^T [kappa][j in block cj] = Qn_cj^T dAqk[i >= 16 cj, j] + Kn'_cj^T dL[i >= 16 cj, j]
//   phase 4  epilogue: combine, last-row gate terms, ln 2; dbeta by a warp butterfly.
//
// 512 threads: warp w owns tensor-memory lanes 32 (w % 4) .. +31 (channels) and the 16 chunk rows
// 16 (w / 4) .. +15.  Outputs are staged in shared memory as swizzled tiles and leave with TMA
// stores (full chunks) or coalesced 16-byte stores (the partial tail chunk of a sequence).
//
// All barrier waits are bounded (error word + early exit instead of a hang).
#include "kda_common.cuh"
#include "kda_sm100.cuh"
#include "kda_timing.cuh"

namespace kda {

using namespace sm100;

struct BwdTcParams {
  CUtensorMap tm_h, tm_dh, tm_do, tm_vn, tm_dv2, tm_v, tm_k, tm_q, tm_a, tm_g;
  CUtensorMap tm_dq, tm_dk, tm_dv, tm_dg;
  const float* beta;
  bf16* dq; bf16* dk; bf16* dv; float* dg; float* db;
  // NORM kernels: q and k are the unnormalised rows, rstd_* their reciprocal norms [tokens, H]
  const bf16* q; const bf16* k; const float* rstd_q; const float* rstd_k;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int* error;
  int nseq, H, total;          // total = chunk capacity x heads work items
  int64_t tokens;              // rows of the packed buffers
  float scale;
  long long* prof;
};

// Debugging aid: phase timestamps of the 20th work item of the first 64 CTAs (steady state) into
// the buffer set with kda_debug_set_profile_buffer.
__device__ __forceinline__ void tc_mark(const BwdTcParams& p, int it, int slot) {
#ifdef KDA_PHASE_PROFILE
#ifndef KDA_PROFILE_THREAD
#define KDA_PROFILE_THREAD 0
#endif
  if (p.prof && it == 20 && threadIdx.x == KDA_PROFILE_THREAD && blockIdx.x < 64) {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.prof[blockIdx.x * 32 + slot] = t;
  }
#endif
}

namespace bl {  // shared-memory layout (bytes)
constexpr int HH = 0, DHH = 32768, VN = 65536, DO = 81920, DV2 = 90112, V = 114688, K = 131072,
              Q = 147456, AK = 163840, G = 172032, MISC = 204800, TOTAL = 212992;
constexpr int OFFS = TOTAL, kOffCache = 256;                 // cu_seqlens / chunk_offsets entries kept in shared memory
constexpr int NORMX = OFFS + 2048, TOTAL_PLAIN = NORMX;      // row norms and row dots of the NORM kernels
constexpr int TOTAL_NORM = NORMX + 4096;
// overlays (valid once their host tiles are dead)
constexpr int DWT = HH, KGM = HH + 16384;                       // after phase 0
constexpr int X = DHH, Y = DHH + 8192, DA = DHH + 16384, DL = DHH + 24576;
// dO and dv2 are interleaved by 64-channel box (dO box b at DO + 16384 b, dv2 box b right behind it),
// so that [dO; dv2] is one 128-row operand: h dO and h dv2 are one N = 128 product per k step.
constexpr int KN0 = VN;                                         // row-type tiles: 40960 bytes from v_new (tiles 0..2 end where dv2 box 0 begins)
constexpr int QN0 = HH, KP0 = HH + 16384;                       // column block 0 (64 rows)
constexpr int QN1 = 106496, KP1 = 118784;                       // column block 1 (48 rows): dv2 box 1 and v, dead by then
constexpr int QN2 = 65536, KP2 = 65536 + 8192;                  // column block 2 (32 rows), after R1
constexpr int QN3 = 65536 + 16384, KP3 = 65536 + 20480;         // column block 3 (16 rows)
constexpr int DVO = HH;                                         // dv staging (phase 2, h tile is dead)
}  // namespace bl
namespace tc {  // tensor-memory columns
constexpr int DQ = 0, DW = 64, DKS = 128, DVB = 192, DKG = 256, X = 320, Y = 384, DAQK = 448, DL = 448;   // DQ, DW adjacent: one N = 128 product
}

__device__ __forceinline__ float ld_bf(const unsigned char* tile, int box_bytes, int row, int col) {
  return __bfloat162float(*reinterpret_cast<const bf16*>(tile + (col >> 6) * box_bytes + sw128(row, col & 63)));
}
__device__ __forceinline__ void st_bf(unsigned char* tile, int box_bytes, int row, int col, float x) {
  *reinterpret_cast<bf16*>(tile + (col >> 6) * box_bytes + sw128(row, col & 63)) = __float2bfloat16(x);
}
// fp32 gate tile: 4 boxes of [64 rows x 32 floats], 128-byte swizzle
__device__ __forceinline__ float ld_g(const unsigned char* g, int row, int c) {
  return *reinterpret_cast<const float*>(g + (c >> 5) * 8192 + row * 128 +
                                         (((((c & 31) >> 2) ^ (row & 7)) << 4) | ((c & 3) << 2)));
}
// 8 consecutive channels kappa0 .. kappa0+7 (kappa0 % 8 == 0) of one row
__device__ __forceinline__ void ld_g8(const unsigned char* g, int row, int kappa0, float (&o)[8]) {
  // The eight lanes of a quarter-warp hold kappa0 = 0, 8, .., 56 (+64): two 32-float boxes, the same
  // four even chunks in each.  Lanes of the odd box fetch their second chunk first, so each 16-byte
  // load touches eight different chunks (no bank conflict).
  const unsigned char* base = g + (kappa0 >> 5) * 8192 + row * 128;
  const int c = (kappa0 & 31) >> 2, sw = row & 7, odd = (kappa0 >> 5) & 1;
  const float4 a = *reinterpret_cast<const float4*>(base + (((c + odd) ^ sw) << 4));
  const float4 b = *reinterpret_cast<const float4*>(base + (((c + 1 - odd) ^ sw) << 4));
  const float4 lo = odd ? b : a, hi = odd ? a : b;
  o[0] = lo.x; o[1] = lo.y; o[2] = lo.z; o[3] = lo.w; o[4] = hi.x; o[5] = hi.y; o[6] = hi.z; o[7] = hi.w;
}
__device__ __forceinline__ void ld_bf8(const unsigned char* tile, int box_bytes, int row, int c16,
                                       float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(tile + (c16 >> 3) * box_bytes + sw128_chunk(row, c16 & 7));
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y; o[4] = c.x; o[5] = c.y; o[6] = d.x; o[7] = d.y;
}
__device__ __forceinline__ uint4 ld_raw8(const unsigned char* tile, int box_bytes, int row, int c16) {
  return *reinterpret_cast<const uint4*>(tile + (c16 >> 3) * box_bytes + sw128_chunk(row, c16 & 7));
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&o)[8]) {
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y; o[4] = c.x; o[5] = c.y; o[6] = d.x; o[7] = d.y;
}
__device__ __forceinline__ void st_bf8(unsigned char* tile, int box_bytes, int row, int c16,
                                       const float (&x)[8]) {
  uint4 u;
  u.x = pack_bf16(x[0], x[1]); u.y = pack_bf16(x[2], x[3]);
  u.z = pack_bf16(x[4], x[5]); u.w = pack_bf16(x[6], x[7]);
  *reinterpret_cast<uint4*>(tile + (c16 >> 3) * box_bytes + sw128_chunk(row, c16 & 7)) = u;
}
__device__ __forceinline__ void pack8v(const float* x, uint4& o) {
  o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]);
  o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
}

// Sum pb[0..31] over the 32 lanes of the warp: afterwards lane l holds the total of entry l (in pb[0]).
__device__ __forceinline__ float warp_transpose_reduce(float (&pb)[32], int lid) {
#pragma unroll
  for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j < n / 2) {
        const bool up = (lid & off) != 0;
        const float send = up ? pb[j] : pb[j + n / 2];
        const float keep = up ? pb[j + n / 2] : pb[j];
        pb[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
  }
  return pb[0];
}

// Sum pb[0..15] over the 32 lanes: afterwards lanes 2e and 2e+1 both hold the total of entry e.
__device__ __forceinline__ float warp_transpose_reduce16(float (&pb)[16], int lid) {
#pragma unroll
  for (int off = 16, n = 16; off >= 2; off >>= 1, n >>= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < n / 2) {
        const bool up = (lid & off) != 0;
        const float send = up ? pb[j] : pb[j + n / 2];
        const float keep = up ? pb[j + n / 2] : pb[j];
        pb[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
  }
  return pb[0] + __shfl_xor_sync(0xffffffffu, pb[0], 1);
}

// Sum pb[0..7] over the 32 lanes: afterwards lanes 4e .. 4e+3 all hold the total of entry e.
__device__ __forceinline__ float warp_transpose_reduce8(float (&pb)[8], int lid) {
#pragma unroll
  for (int off = 16, n = 8; off >= 4; off >>= 1, n >>= 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < n / 2) {
        const bool up = (lid & off) != 0;
        const float send = up ? pb[j] : pb[j + n / 2];
        const float keep = up ? pb[j + n / 2] : pb[j];
        pb[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
  }
  float v = pb[0] + __shfl_xor_sync(0xffffffffu, pb[0], 2);
  return v + __shfl_xor_sync(0xffffffffu, v, 1);
}

constexpr int NT = 512;

// NORM: the forward pass normalised q and k inside its first kernel; this kernel receives the
// unnormalised rows with their reciprocal norms, normalises the q and k tiles as they land (to the
// same bf16 values), and turns dq, dk into gradients of the unnormalised rows before they leave:
// dx = rstd (dy - y <dy, y>)  (reference stage: bwd/triton/l2norm_bwd.py:37).
template <bool NORM>
__global__ void __launch_bounds__(NT, 1) kda_bwd_chunk_tc_kernel(const __grid_constant__ BwdTcParams p) {
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment by offset, so the compiler still knows this is shared memory
  unsigned char* sm = smem_dyn + ((1024u - (saddr(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + bl::MISC);    // [0], [7] TMA; [1..6] UMMA groups
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + bl::MISC + 64);
  volatile int* s_abort = reinterpret_cast<volatile int*>(sm + bl::MISC + 72);
  float* s_beta = reinterpret_cast<float*>(sm + bl::MISC + 128);          // [64]
  float* s_db = s_beta + 64;                                              // [2 terms][4 quadrants][64]
  float* s_hd = s_db + 512;                                               // [4][128]
  float* s_kdk = s_hd + 512;                                              // [4][128]
  int* s_next = reinterpret_cast<int*>(s_kdk + 512);                      // next item: token0 (two words), valid
  // reciprocal norms [2 = q, k][64], one copy per item parity: an item's copy is written while the
  // item before it runs, so barriers lie between that write and its first read
  float* s_rs2 = reinterpret_cast<float*>(sm + bl::NORMX);
  float* s_dot = s_rs2 + 256;                                             // [2][64 rows][4 quadrants] <dy, y>

  const int tid = threadIdx.x, warp = tid >> 5, lid = tid & 31;
  const int quad = warp & 3, rq = warp >> 2;
  const int L = quad * 32 + lid;                 // channel owned by this thread (TMEM lane)
  const int r0 = 16 * rq;                        // first of the 16 chunk rows it handles
  const int H = p.H;

  // Work items are located by a binary search over the sequence offsets: from shared memory when
  // they fit (a chain of dependent global loads per item would sit on the critical path).
  int32_t* s_cu = reinterpret_cast<int32_t*>(sm + bl::OFFS);
  int32_t* s_co = s_cu + bl::kOffCache;
  const bool cached = p.nseq + 1 <= bl::kOffCache;
  if (cached)
    for (int i = tid; i <= p.nseq; i += NT) { s_cu[i] = p.cu_seqlens[i]; s_co[i] = p.chunk_offsets[i]; }
  const int32_t* cu_off = cached ? s_cu : p.cu_seqlens;
  const int32_t* ch_off = cached ? s_co : p.chunk_offsets;
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  if (tid == 0) {
    // arrival counts = number of threads that issue (and commit) products of that group
    const int counts[8] = {1, 3, 3, 1, 1, 2, 4, 3};
    for (int i = 0; i < 8; ++i) mbar_init(&bar[i], counts[i]);
    mbar_init_fence();
    *s_abort = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * quad) << 16);    // this warp's lane quadrant
  const unsigned char* sG = sm + bl::G;

  // Loads of one work item, in two parts so that the next item's tiles start arriving as soon as
  // their shared-memory regions die.  Part 0 (barrier 0): h, dh, dO, v_new, dv2, v, A -- dead once
  // the last products of the current item have completed.  Part 1 (barrier 7): k, q, G, whose
  // tiles stage dk, dq, dG until the current item's stores have read them.  Part 0 is issued by thread 0.
  // (Part 0 spread over lane 0 of 13 warps, one tile each, was measured: 1.40 against 1.366 ms.)
  auto issue_loads = [&](int chunk, int head, int64_t token0) {
    const int ty = (int)token0, tx = head * 128;
    {
      const int yh = (chunk * H + head) * 128;
      mbar_expect_tx(&bar[0], 2 * 32768 + 4 * 16384 + 8192);
      for (int b = 0; b < 2; ++b) {
        tma_load_2d(sm + bl::HH + b * 16384, &p.tm_h, 64 * b, yh, &bar[0]);
        tma_load_2d(sm + bl::DO + b * 16384, &p.tm_do, tx + 64 * b, ty, &bar[0]);
        tma_load_2d(sm + bl::DV2 + b * 16384, &p.tm_dv2, tx + 64 * b, ty, &bar[0]);
        tma_load_2d(sm + bl::DHH + b * 16384, &p.tm_dh, 64 * b, yh, &bar[0]);
        tma_load_2d(sm + bl::VN + b * 8192, &p.tm_vn, tx + 64 * b, ty, &bar[0]);
      }
      for (int b = 0; b < 2; ++b) tma_load_2d(sm + bl::V + b * 8192, &p.tm_v, tx + 64 * b, ty, &bar[0]);
      tma_load_2d(sm + bl::AK, &p.tm_a, head * 64, ty, &bar[0]);
    }
  };
  // Part 1 is issued by lane 0 of warps 4, 5, 6 (q, k, G): each of them also issued the bulk stores
  // out of the tiles it reloads (dq, dk, dG of the previous item), so each waits for its own stores
  // only and the three drain, and reload, side by side (measured on one GPU against one thread doing
  // all stores and eight lanes the loads: 1.351 against 1.366 ms).
  auto reload_piece = [&](int which, int head, int64_t token0) {
    const int ty = (int)token0, tx = head * 128;
    tma_store_wait_read();
    if (which == 0) {
      mbar_expect_tx(&bar[7], 16384);
      for (int b = 0; b < 2; ++b) tma_load_2d(sm + bl::Q + b * 8192, &p.tm_q, tx + 64 * b, ty, &bar[7]);
    } else if (which == 1) {
      mbar_expect_tx(&bar[7], 16384);
      for (int b = 0; b < 2; ++b) tma_load_2d(sm + bl::K + b * 8192, &p.tm_k, tx + 64 * b, ty, &bar[7]);
    } else {
      mbar_expect_tx(&bar[7], 32768);
      for (int b = 0; b < 4; ++b) tma_load_2d(sm + bl::G + b * 8192, &p.tm_g, tx + 32 * b, ty, &bar[7]);
    }
  };

  // Phase-0 products: one issuing thread per accumulator (lane 0 of warps 0..3).  A product's time is
  // about its shared-memory operand bytes / 128 B per clock (4 KB + 2 KB for M = 128, N = 64, K = 16),
  // and the issuing thread is held while the queue is full: issuing them from the end of the
  // previous item was measured and gained 1 % (the stores and reloads compete for the same bandwidth).
  auto issue_phase0 = [&]() {
    tc_fence_after();
    const uint32_t hh = saddr(sm + bl::HH), dhh = saddr(sm + bl::DHH), dO = saddr(sm + bl::DO),
                   vn = saddr(sm + bl::VN);
    if (warp == 0) {         // dq_inter^T and dw^T: h [dO; dv2], N = 128 (the sign of dw is applied where it is read)
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + tc::DQ, desc_kmajor(hh, ks, 16384), desc_kmajor(dO, ks, 16384),
             instr_desc(128, 128, 0, 0), ks > 0);
    } else if (warp == 1) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + tc::DAQK, desc_kmajor(dO, ks, 16384), desc_kmajor(vn, ks, 8192),
             instr_desc(64, 64, 0, 0), ks > 0);
    } else {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + tc::DKS, desc_kmajor(dhh, ks, 16384), desc_kmajor(vn, ks, 8192),
             instr_desc(128, 64, 0, 0), ks > 0);
    }
    umma_commit(&bar[1]);
  };

  // persistent walk over the (chunk, head) work items
  uint32_t ph = 0;              // parity of this item's barrier phases
  int it = 0, rc = 0;
  bool pre = false;             // part 0 of this item's loads was issued by the previous item
  bool prev_full = false;       // the previous item was a full chunk (its results left through bulk stores)
  ChunkWork cw_next{};
  float beta_next = 0.f;
  for (int w = blockIdx.x; w < p.total; w += gridDim.x) {
  tc_mark(p, it, 15);
  const int chunk = w / H, head = w - chunk * H;
  const ChunkWork cw = pre ? cw_next : locate_chunk(cu_off, ch_off, p.nseq, chunk);
  if (cw.valid == 0) continue;              // capacity slot past the last active chunk
  if (!pre && !chunk_in_range(cw, p.tokens)) {     // (with pre the previous item checked it)
    if (tid == 0 && p.error) atomicExch(p.error, kOffsetsOutOfRange);
    continue;
  }
  const int valid = cw.valid;
  const int ty = (int)cw.token0, tx = head * 128;
  if (tid < 64)
    s_beta[tid] = pre ? beta_next : (tid < valid ? p.beta[(cw.token0 + tid) * H + head] : 0.f);
  float* s_rs = s_rs2 + 128 * (it & 1);
  if constexpr (NORM) {
    if (!pre && tid >= 64 && tid < 192) {      // (with pre the item before this one wrote them)
      const int row = (tid - 64) & 63;
      const float* rs = tid < 128 ? p.rstd_q : p.rstd_k;
      s_rs[tid - 64] = row < valid ? rs[(cw.token0 + row) * H + head] : 0.f;
    }
  }
  // Between two full chunks nothing that is written before the next barrier (beta, hd) is read
  // before it or is still read by the previous item, whose accumulators were read before its last barrier
  // and whose bulk stores are drained by the thread that reloads their tiles: no barrier.
  const bool chained = valid == 64 && prev_full && pre;
  if (!chained) __syncthreads();     // the previous item's staging tiles have been read
  tc_mark(p, it, 16);
  if (tid == 0 && !pre) issue_loads(chunk, head, cw.token0);
  if (lid == 0 && warp >= 4 && warp < 7 && valid < 64) reload_piece(warp - 4, head, cw.token0);   // the fix-up of a partial chunk needs every tile before the first product
  int chunk_n = 0, head_n = 0;
  bool next_ok = false;
  tc_mark(p, it, 17);
  auto body = [&]() -> int {
  tc_mark(p, it, 0);
  if (!mbar_wait(&bar[0], ph)) *s_abort = 1;
  if (valid < 64 && !mbar_wait(&bar[7], ph)) *s_abort = 1;     // the fix-up below touches every tile
  tc_mark(p, it, 1);

  // partial tail chunk: rows >= valid hold another sequence's tokens or unwritten memory.  Zero them
  // in every token tile and repeat the last gate row, so no later step needs a row guard.
  if (valid < 64) {
    const int tiles[6] = {bl::DO, bl::VN, bl::DV2, bl::V, bl::K, bl::Q};
    const int boxes[6] = {16384, 8192, 16384, 8192, 8192, 8192};
    for (int idx = tid; idx < (64 - valid) * 16; idx += NT) {
      const int r = valid + (idx >> 4), ch = idx & 15;
#pragma unroll
      for (int t = 0; t < 6; ++t)
        *reinterpret_cast<uint4*>(sm + tiles[t] + (ch >> 3) * boxes[t] + sw128_chunk(r, ch & 7)) = make_uint4(0, 0, 0, 0);
      if (ch < 8) *reinterpret_cast<uint4*>(sm + bl::AK + sw128_chunk(r, ch)) = make_uint4(0, 0, 0, 0);
    }
    for (int idx = tid; idx < (64 - valid) * 32; idx += NT) {
      const int r = valid + (idx >> 5), ch = idx & 31;        // 32 chunks of 4 floats per row
      const int off = (ch >> 3) * 8192, c = ch & 7;
      *reinterpret_cast<float4*>(sm + bl::G + off + r * 128 + ((c ^ (r & 7)) << 4)) =
          *reinterpret_cast<const float4*>(sm + bl::G + off + (valid - 1) * 128 + ((c ^ ((valid - 1) & 7)) << 4));
    }
    fence_async_smem();
  }
  if (!chained) {
    __syncthreads();
    if (*s_abort) return 2;
  }

  // ---- phase 0 UMMAs ---------------------------------------------------------------------------------
  if (lid == 0 && warp < 3) issue_phase0();
  if (lid == 0 && warp >= 4 && warp < 7 && valid == 64) reload_piece(warp - 4, head, cw.token0);   // k, q, G: their tiles staged the previous item's dk, dq, dG
  // meanwhile: hd[kappa] = sum_v h dh over this thread's quarter of v (giving the quarter of the
  // issuing warps 0..3 to warps 4..7 as well was measured: slower, 1.383 against 1.364 ms)
  {
    float s = 0.f;
    const unsigned char* hb = sm + bl::HH + (rq >> 1) * 16384;
    const unsigned char* db = sm + bl::DHH + (rq >> 1) * 16384;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      const int ch = 4 * (rq & 1) + c4;
      uint4 a = *reinterpret_cast<const uint4*>(hb + sw128_chunk(L, ch));
      uint4 b = *reinterpret_cast<const uint4*>(db + sw128_chunk(L, ch));
      float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
      float2 b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y), b2 = unpack_bf16(b.z), b3 = unpack_bf16(b.w);
      s += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y +
           a3.x * b3.x + a3.y * b3.y;
    }
    s_hd[rq * 128 + L] = s;
  }
  // the next work item is located by one thread of a warp that issues nothing while the first
  // products run (the search is a chain of dependent loads: done by every thread it sat on the
  // path of the issuing warps); everybody reads the result after the barrier below
  if (tid == 160) {
    const int wn = w + (int)gridDim.x;
    ChunkWork nx{};
    if (wn < p.total) nx = locate_chunk(cu_off, ch_off, p.nseq, wn / H);
    if (!chunk_in_range(nx, p.tokens)) nx.valid = 0;     // not prefetched; the item itself reports and skips
    s_next[0] = (int)(nx.token0 & 0xffffffffLL);
    s_next[1] = (int)(nx.token0 >> 32);
    s_next[2] = nx.valid;
  }
  tc_mark(p, it, 2);
  if (!mbar_wait(&bar[7], ph)) *s_abort = 1;       // k, q, A, G, v have landed
  if constexpr (NORM) {
    // q and k rows to unit norm, rounded to bf16 as the forward pass rounded them: every later read
    // of these tiles (by threads only) comes after the barrier below
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int i = (tid >> 4) + 32 * n, c16 = tid & 15;
      float x[8];
      ld_bf8(sm + bl::Q, 8192, i, c16, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] *= s_rs[i];
      st_bf8(sm + bl::Q, 8192, i, c16, x);
      ld_bf8(sm + bl::K, 8192, i, c16, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] *= s_rs[64 + i];
      st_bf8(sm + bl::K, 8192, i, c16, x);
    }
  }
  const float glast = ld_g(sG, valid - 1, L);
  if (!mbar_wait(&bar[1], ph)) *s_abort = 1;
  tc_fence_after();
  __syncthreads();
  tc_mark(p, it, 3);      // every thread is done with the raw h / dh tiles
  if (*s_abort) return 3;
  {   // the next item, and what this thread carries over to it
    const int wn = w + (int)gridDim.x;
    chunk_n = wn / H;
    head_n = wn - chunk_n * H;
    cw_next.token0 = (int64_t)(((uint64_t)(uint32_t)s_next[1] << 32) | (uint32_t)s_next[0]);
    cw_next.valid = s_next[2];
    next_ok = cw_next.valid > 0;        // 0 also when there is no further item
    if (tid < 64)
      beta_next = (next_ok && tid < cw_next.valid) ? p.beta[(cw_next.token0 + tid) * H + head_n] : 0.f;
    if constexpr (NORM) {
      if (tid >= 64 && tid < 192) {
        const int row = (tid - 64) & 63;
        const float* rs = tid < 128 ? p.rstd_q : p.rstd_k;
        s_rs2[128 * ((it + 1) & 1) + tid - 64] =
            (next_ok && row < cw_next.valid) ? rs[(cw_next.token0 + row) * H + head_n] : 0.f;
      }
    }
  }

  // This thread's two (row, 8-channel) pieces -- rows tid / 16 and tid / 16 + 32, channels 8 (tid % 16) --
  // are the same in every pass that builds gated k tiles: their k (raw bf16) and gate values are read
  // once and stay in registers.
  float gkeep[2][8];
  uint4 kkeep[2];
  // ---- phase 1 epilogue: operand tiles for the next products; dq^T and dks^T stay in tensor memory
  {
    float a[16];
    tmem_ld16(tl + tc::DW + r0, a);      // h dv2: dw^T = -(h dv2)
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) a[jj] = -a[jj];
#pragma unroll
    for (int qd = 0; qd < 2; ++qd) {
      uint4 v;
      pack8v(a + 8 * qd, v);
      *reinterpret_cast<uint4*>(sm + bl::DWT + sw128_chunk(L, 2 * rq + qd)) = v;
    }
    // k 2^G as a K-major tile [s][kappa]
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int i = (tid >> 4) + 32 * n, c16 = tid & 15;
      float kk[8];
      kkeep[n] = ld_raw8(sm + bl::K, 8192, i, c16);
      unpack8(kkeep[n], kk);
      ld_g8(sG, i, 8 * c16, gkeep[n]);
#pragma unroll
      for (int e = 0; e < 8; ++e) kk[e] *= fexp2(gkeep[n][e]);
      st_bf8(sm + bl::KGM, 8192, i, c16, kk);
    }
    // dAqk (M = 64 accumulator: row r lives on lane 32 (r / 16) + r % 16)
    tmem_ld16(tl + tc::DAQK + r0, a);
    if (lid < 16) {
      const int r = quad * 16 + lid;
      float y[16];
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) y[jj] = (r >= r0 + jj && r < valid) ? a[jj] * p.scale : 0.f;
#pragma unroll
      for (int qd = 0; qd < 2; ++qd) {
        uint4 v;
        pack8v(y + 8 * qd, v);
        *reinterpret_cast<uint4*>(sm + bl::DA + sw128_chunk(r, 2 * rq + qd)) = v;
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  tc_mark(p, it, 4);
  // ---- phase 1 UMMAs: dvb^T, dkgb^T, X (three issuing threads) ------------------------------------
  if (lid == 0 && warp < 3) {
    tc_fence_after();
    const uint32_t dv2 = saddr(sm + bl::DV2), ak = saddr(sm + bl::AK), dwt = saddr(sm + bl::DWT),
                   v = saddr(sm + bl::V), kgm = saddr(sm + bl::KGM);
    if (warp == 0) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem + tc::DVB, desc_mnmajor(dv2, ks, 16384), desc_mnmajor(ak, ks, 0),
             instr_desc(128, 64, 1, 1), ks > 0);
    } else if (warp == 1) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem + tc::DKG, desc_kmajor(dwt, ks, 0), desc_mnmajor(ak, ks, 0),
             instr_desc(128, 64, 0, 1), ks > 0);
    } else {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + tc::X, desc_kmajor(dv2, ks, 16384), desc_kmajor(v, ks, 8192),
             instr_desc(64, 64, 0, 0), ks > 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + tc::X, desc_mnmajor(dwt, ks, 0), desc_kmajor(kgm, ks, 8192),
             instr_desc(64, 64, 1, 0), 1);
    }
    umma_commit(&bar[2]);
  }
  // Row-type gated tiles  Kn_ri[j][kappa] = k_j 2^{R_ri - G_j},  j < 16 (ri + 1): the four tiles
  // (16, 32, 48, 64 rows) are one flat list of 2560 eight-channel tasks.  The first three tiles
  // overlay v_new and box 0 of dO (dead) and are built while the phase 1 products run; the last one
  // covers box 0 of dv2 and waits for them.
  auto build_row_tiles = [&](int begin, int end) {
    // (only the last tile, ri = 3, is built here: tasks 1536 .. 2559; its reference row depends on
    // the channel piece only, which is the same for a thread's tasks)
    float rr[8];
    ld_g8(sG, 48, 8 * (tid & 15), rr);
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int j = (tid >> 4) + 32 * n, c16 = tid & 15;
      float kk[8];
      unpack8(kkeep[n], kk);
#pragma unroll
      for (int e = 0; e < 8; ++e) kk[e] *= fexp2(fminf(rr[e] - gkeep[n][e], 126.f));
      st_bf8(sm + bl::KN0 + 1536 * 16, 64 * 128, j, c16, kk);
    }
  };
  // Tiles 0..2 in one pass over the rows j < 48: k_j and G_j are read once for all the tiles that
  // hold row j (tiles ri >= j / 16).  Threads 0..255 take a row of block 0 (three tiles), the others a
  // row of block 1 and one of block 2 (two tiles + one): three tile rows per thread either way.
  {
    const int c16 = tid & 15;
    auto fused_row = [&](int j, const uint4& kraw, const float (&gj)[8]) {
      float kk[8];
      unpack8(kraw, kk);
#pragma unroll
      for (int ri = 0; ri < 3; ++ri) {
        if (ri >= (j >> 4)) {
          float rr[8], o[8];
          ld_g8(sG, 16 * ri, 8 * c16, rr);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = kk[e] * fexp2(fminf(rr[e] - gj[e], 126.f));
          st_bf8(sm + bl::KN0 + (ri == 0 ? 0 : (ri == 1 ? 4096 : 12288)), 2048 * (ri + 1), j, c16, o);
        }
      }
    };
    fused_row(tid >> 4, kkeep[0], gkeep[0]);           // rows 0..31: the first kept piece
    if (tid >= 256) {                                  // rows 32..47: not one of this thread's kept rows
      const int j = 16 + (tid >> 4);
      float g2[8];
      const uint4 k2 = ld_raw8(sm + bl::K, 8192, j, c16);
      ld_g8(sG, j, 8 * c16, g2);
      fused_row(j, k2, g2);
    }
  }
  // sum_i k dks 2^{G_last - G_i} over this thread's rows: the last row of dG needs the block-wide sum
  {
    float a[16], kdk = 0.f;
    tmem_ld16(tl + tc::DKS + r0, a);
#pragma unroll
    for (int ii = 0; ii < 16; ++ii)
      kdk += ld_bf(sm + bl::K, 8192, r0 + ii, L) * a[ii] * fexp2(glast - ld_g(sG, r0 + ii, L));
    s_kdk[rq * 128 + L] = kdk;
  }
  tc_mark(p, it, 22);
  if (!mbar_wait(&bar[2], ph)) *s_abort = 1;
  tc_fence_after();
  tc_mark(p, it, 5);

  // ---- phase 2 epilogue: dv (staged) and its dbeta term; X tile (dkgb^T stays in tensor memory) ----
  {
    float a[16], pb[16], bt[16];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const float4 b4 = *reinterpret_cast<const float4*>(s_beta + r0 + 4 * q4);
      bt[4 * q4] = b4.x; bt[4 * q4 + 1] = b4.y; bt[4 * q4 + 2] = b4.z; bt[4 * q4 + 3] = b4.w;
    }
    tmem_ld16(tl + tc::DVB + r0, a);      // this thread = value channel v = L
#pragma unroll
    for (int ii = 0; ii < 16; ++ii) {
      const int s = r0 + ii;
      st_bf(sm + bl::DVO, 8192, s, L, a[ii] * bt[ii]);
      pb[ii] = a[ii] * ld_bf(sm + bl::V, 8192, s, L);
    }
    {   // dbeta term 0: one slot per (channel quadrant, row), summed in a fixed order at the end
      const float tot = warp_transpose_reduce16(pb, lid);
      if ((lid & 1) == 0) s_db[quad * 64 + r0 + (lid >> 1)] = tot;
    }
    tmem_ld16(tl + tc::X + r0, a);
    if (lid < 16) {
      const int t = quad * 16 + lid;
      float y[16];
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const int s = r0 + jj;
        y[jj] = (t > s && t < valid) ? a[jj] * bt[jj] : 0.f;
      }
#pragma unroll
      for (int qd = 0; qd < 2; ++qd) {
        uint4 v;
        pack8v(y + 8 * qd, v);
        *reinterpret_cast<uint4*>(sm + bl::X + sw128_chunk(t, 2 * rq + qd)) = v;
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (*s_abort) return 4;

  tc_mark(p, it, 6);
  // ---- Y = A^T X; dv leaves -------------------------------------------------------------------------
  if (tid == 0) {
    tc_fence_after();
    const uint32_t ak = saddr(sm + bl::AK), x = saddr(sm + bl::X);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      umma(tmem + tc::Y, desc_mnmajor(ak, ks, 0), desc_mnmajor(x, ks, 0), instr_desc(64, 64, 1, 1), ks > 0);
    umma_commit(&bar[3]);
    if (valid == 64) {
      tma_store_2d(&p.tm_dv, sm + bl::DVO, tx, ty);
      tma_store_2d(&p.tm_dv, sm + bl::DVO + 8192, tx + 64, ty);
      tma_store_commit();
    }
  }
  if (valid < 64) {
    for (int idx = tid; idx < valid * 16; idx += NT) {
      const int r = idx >> 4, ch = idx & 15;
      *reinterpret_cast<uint4*>(p.dv + ((cw.token0 + r) * H + head) * 128 + ch * 8) =
          *reinterpret_cast<const uint4*>(sm + bl::DVO + (ch >> 3) * 8192 + sw128_chunk(r, ch & 7));
    }
  }
  build_row_tiles(1536, 2560);
  tc_mark(p, it, 7);
  tc_mark(p, it, 23);
  if (!mbar_wait(&bar[3], ph)) *s_abort = 1;
  tc_fence_after();
  {
    float a[16];
    tmem_ld16(tl + tc::Y + r0, a);
    if (lid < 16) {
      const int r = quad * 16 + lid;
#pragma unroll
      for (int qd = 0; qd < 2; ++qd) {
        uint4 v;
        pack8v(a + 8 * qd, v);
        *reinterpret_cast<uint4*>(sm + bl::Y + sw128_chunk(r, 2 * rq + qd)) = v;
      }
    }
  }
  if (tid == 0) tma_store_wait_read();      // the dv staging tile is rewritten after the next barrier
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (*s_abort) return 5;

  tc_mark(p, it, 8);
  // ---- dL = -(Y A^T) (warp 0), and the dAqk half of the row-type products (warp 1) --------------------
  if (lid == 0 && warp < 2) {
    tc_fence_after();
    if (warp == 0) {
      const uint32_t ak = saddr(sm + bl::AK), y = saddr(sm + bl::Y);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem + tc::DL, desc_kmajor(y, ks, 0), desc_kmajor(ak, ks, 0), instr_desc(64, 64, 0, 0, 1), ks > 0);
      umma_commit(&bar[4]);
    } else {      // committed together with the dL half, on barrier 5
      const uint32_t da = saddr(sm + bl::DA);
      int off = 0;
#pragma unroll
      for (int ri = 0; ri < 4; ++ri) {
        const int rows = 16 * (ri + 1);
        const uint32_t kn = saddr(sm + bl::KN0 + off);
#pragma unroll
        for (int ks = 0; ks <= ri; ++ks)
          umma(tmem + tc::DVB + 16 * ri, desc_mnmajor(kn, ks, rows * 128), desc_kmajor(da + 2048 * ri, ks, 0),
               instr_desc(128, 16, 1, 0), ks > 0);
        off += rows * 256;
      }
    }
  }
  // meanwhile: column-type gated tiles.  Block cj holds rows 16 cj .. 63 of
  //   Qn[i][kappa] = q_i 2^{G_i - R'_cj},  Kp[i][kappa] = beta_i k_i 2^{G_i - R'_cj},  R'_cj = G[16 cj + 15]
  // Column blocks cjA and cjA + 1 in one pass: q_i, k_i, G_i are read once for both tiles (block
  // cjA + 1 holds the rows i >= 16 (cjA + 1) only).
  auto fused_col = [&](int i, int c16, int cjA, int q0, int k0, int q1, int k1, const float (&ref0)[8],
                       const float (&ref1)[8], const uint4& kraw, const float (&gi)[8]) {
    float qq[8], kk[8];
    ld_bf8(sm + bl::Q, 8192, i, c16, qq);
    unpack8(kraw, kk);
    const float b = s_beta[i];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int cj = cjA + t;
      if (i >= 16 * cj) {
        float oq[8], ok[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float ex = fexp2(fminf(gi[e] - (t == 0 ? ref0[e] : ref1[e]), 126.f));
          oq[e] = qq[e] * ex;
          ok[e] = kk[e] * (ex * b);
        }
        st_bf8(sm + (t == 0 ? q0 : q1), (64 - 16 * cj) * 128, i - 16 * cj, c16, oq);
        st_bf8(sm + (t == 0 ? k0 : k1), (64 - 16 * cj) * 128, i - 16 * cj, c16, ok);
      }
    }
  };
  {   // the reference rows R'_cj depend on the channel piece only, which is the same for a thread's tasks
    float ref0[8], ref1[8];
    ld_g8(sG, 15, 8 * (tid & 15), ref0);
    ld_g8(sG, 31, 8 * (tid & 15), ref1);
#pragma unroll
    for (int n = 0; n < 2; ++n)                           // blocks 0 (64 rows) and 1 (48 rows)
      fused_col((tid >> 4) + 32 * n, tid & 15, 0, bl::QN0, bl::KP0, bl::QN1, bl::KP1, ref0, ref1, kkeep[n],
                gkeep[n]);
  }
  tc_mark(p, it, 9);
  tc_mark(p, it, 24);
  if (!mbar_wait(&bar[4], ph)) *s_abort = 1;
  tc_fence_after();
  {
    float a[16];
    tmem_ld16(tl + tc::DL + r0, a);
    if (lid < 16) {
      const int r = quad * 16 + lid;
      float y[16];
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) y[jj] = (r > r0 + jj && r < valid) ? a[jj] : 0.f;
#pragma unroll
      for (int qd = 0; qd < 2; ++qd) {
        uint4 v;
        pack8v(y + 8 * qd, v);
        *reinterpret_cast<uint4*>(sm + bl::DL + sw128_chunk(r, 2 * rq + qd)) = v;
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (*s_abort) return 6;

  auto issue_col = [&](int cj, int qoff, int koff) {   // one issuing thread per column block
    const int rows = 64 - 16 * cj;
    const uint32_t qn = saddr(sm + qoff), kp = saddr(sm + koff);
    const uint32_t da = saddr(sm + bl::DA) + 2048 * cj + 32 * cj;
    const uint32_t dl = saddr(sm + bl::DL) + 2048 * cj + 32 * cj;
    const uint32_t id = instr_desc(128, 16, 1, 1);
    for (int ks = 0; ks < 4 - cj; ++ks)
      umma(tmem + tc::DW + 16 * cj, desc_mnmajor(qn, ks, rows * 128), smem_desc(da + ks * 2048, 0, 1024), id, ks > 0);
    for (int ks = 0; ks < 4 - cj; ++ks)
      umma(tmem + tc::DW + 16 * cj, desc_mnmajor(kp, ks, rows * 128), smem_desc(dl + ks * 2048, 0, 1024), id, 1);
    umma_commit(&bar[6]);
  };
  if (lid == 0 && warp < 4) {
    tc_fence_after();
    if (warp == 0) {     // the dL half of the row-type products
      const uint32_t dl = saddr(sm + bl::DL);
      int off = 0;
#pragma unroll
      for (int ri = 0; ri < 4; ++ri) {
        const int rows = 16 * (ri + 1);
        const uint32_t kn = saddr(sm + bl::KN0 + off);
#pragma unroll
        for (int ks = 0; ks <= ri; ++ks)
          umma(tmem + tc::X + 16 * ri, desc_mnmajor(kn, ks, rows * 128), desc_kmajor(dl + 2048 * ri, ks, 0),
               instr_desc(128, 16, 1, 0), ks > 0);
        off += rows * 256;
      }
      umma_commit(&bar[5]);
    } else if (warp == 1) {
      umma_commit(&bar[5]);          // its dAqk half, issued one step earlier
    } else if (warp == 2) {
      issue_col(0, bl::QN0, bl::KP0);
    } else {
      issue_col(1, bl::QN1, bl::KP1);
    }
  }
  tc_mark(p, it, 10);
  // the next item's k, q, G tiles are asked into L2 for the reload that follows this item's stores (without
  // the request the kernel takes 7 % longer; asked for here, two phases before the end, rather than with
  // the other tiles' loads: 1 % faster; earlier still: slower)
  if (warp == 5 && lid < 8 && next_ok) {
    const int ty = (int)cw_next.token0, tx = head_n * 128;
    if (lid < 2) tma_prefetch_2d(&p.tm_k, tx + 64 * lid, ty);
    else if (lid < 6) tma_prefetch_2d(&p.tm_g, tx + 32 * (lid - 2), ty);
    else tma_prefetch_2d(&p.tm_q, tx + 64 * (lid - 6), ty);
  }
  tc_mark(p, it, 25);
  if (!mbar_wait(&bar[5], ph)) *s_abort = 1;   // row-type tiles are free again
  tc_fence_after();
  {
    float ref0[8], ref1[8];
    ld_g8(sG, 47, 8 * (tid & 15), ref0);
    ld_g8(sG, 63, 8 * (tid & 15), ref1);
    fused_col(32 + (tid >> 4), tid & 15, 2, bl::QN2, bl::KP2, bl::QN3, bl::KP3, ref0, ref1, kkeep[1],
              gkeep[1]);                                   // blocks 2 and 3
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (*s_abort) return 7;
  if (lid == 0 && warp < 2) {
    tc_fence_after();
    if (warp == 0) issue_col(2, bl::QN2, bl::KP2);
    else issue_col(3, bl::QN3, bl::KP3);
  }
  tc_mark(p, it, 11);
  tc_mark(p, it, 26);
  if (!mbar_wait(&bar[6], ph)) *s_abort = 1;
  tc_fence_after();
  tc_mark(p, it, 12);
  // every tile but k, q, G is dead from here on: the next item's tiles start arriving
  if (tid == 0 && next_ok) issue_loads(chunk_n, head_n, cw_next.token0);
  // NORM: the unnormalised q, k pieces this thread turns into y again once the epilogue below is
  // through; fetched now so that their latency hides behind the epilogue instead of ending the item
  uint4 raw_q[2], raw_k[2];
  if constexpr (NORM) {
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int i = (tid >> 4) + 32 * n;
      raw_q[n] = raw_k[n] = make_uint4(0, 0, 0, 0);
      if (i < valid) {
        const int64_t at = ((cw.token0 + i) * H + head) * 128 + 8 * (tid & 15);
        raw_q[n] = *reinterpret_cast<const uint4*>(p.q + at);
        raw_k[n] = *reinterpret_cast<const uint4*>(p.k + at);
      }
    }
  }

  // ---- final epilogue: six accumulators, 8 rows at a time; thread = channel L, rows r0 .. r0 + 15 ------
  //   DQ: dq_inter^T   DVB: dq_intra^T   DKS: dks^T   DKG: dkgb^T   X: X1^T   DW: dk2^T
  //   dq = e (scale 2^R dq_inter + dq_intra)              e = 2^{G_i - R},  R  = G[r0]
  //   dk = 2^{G_last - G_i} dks + beta (2^G dkgb + e X1) + f dk2      f = 2^{R' - G_i}, R' = G[r0 + 15]
  //   dG = q dq - k (dk - 2 beta (...))  assembled term by term below; dbeta_i = sum_kappa k (2^G dkgb + e X1)
  // Results are staged in place: dq over the q tile, dk over the k tile, dG over the G tile (every
  // element of those tiles is read only by the thread that overwrites it).
  {
    const int constB = (L >> 6) * 8192 + (L & 7) * 2, cB = (L & 63) >> 3;
    const int constG = (L >> 5) * 8192 + (L & 3) * 4, cG = (L & 31) >> 2;
    const float gfirst = ld_g(sG, r0, L), rlast = ld_g(sG, r0 + 15, L);
    const float E0 = fexp2(gfirst), F0 = fexp2(glast - rlast), sE0 = p.scale * E0;
    // last valid row of dG: + (sum_v h dh) 2^{G_last} + sum_i k dks 2^{G_last - G_i}
    float hdv = 0.f;
    if (rq == ((valid - 1) >> 4))
      hdv = ((s_hd[L] + s_hd[128 + L] + s_hd[256 + L] + s_hd[384 + L]) * fexp2(glast) +
             s_kdk[L] + s_kdk[128 + L] + s_kdk[256 + L] + s_kdk[384 + L]) * kLn2;
    float pb[16];
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
      const int rb = r0 + 8 * grp;
      unsigned char* rowB = sm + constB + rb * 128;
      unsigned char* rowG = sm + constG + rb * 128;
      float a[8], a2[8], e[8], f[8], kr[8], dkr[8], dgr[8];
      float ydq[8], ydk[8];       // NORM: y dy per row, summed over the channels below
      int oB[8], oG[8];
      const float4 b0 = *reinterpret_cast<const float4*>(s_beta + rb), b1 = *reinterpret_cast<const float4*>(s_beta + rb + 4);
      const float bt[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int ii = 0; ii < 8; ++ii) {
        oB[ii] = ii * 128 + ((cB ^ ii) << 4);
        oG[ii] = ii * 128 + ((cG ^ ii) << 4);
        const float g = *reinterpret_cast<const float*>(rowG + bl::G + oG[ii]);
        e[ii] = fexp2(g - gfirst);
        f[ii] = fexp2(rlast - g);
        kr[ii] = __bfloat162float(*reinterpret_cast<const bf16*>(rowB + bl::K + oB[ii]));
      }
      tmem_ld8(tl + tc::DQ + rb, a);
      tmem_ld8(tl + tc::DVB + rb, a2);
#pragma unroll
      for (int ii = 0; ii < 8; ++ii) {
        const float dqv = e[ii] * fmaf(a[ii], sE0, a2[ii]);
        bf16* cell = reinterpret_cast<bf16*>(rowB + bl::Q + oB[ii]);
        dgr[ii] = __bfloat162float(*cell) * dqv;
        if constexpr (NORM) ydq[ii] = dgr[ii];
        *cell = __float2bfloat16(dqv);
      }
      tmem_ld8(tl + tc::DKS + rb, a);
#pragma unroll
      for (int ii = 0; ii < 8; ++ii) {
        const float x = a[ii] * (f[ii] * F0);
        dkr[ii] = x;
        dgr[ii] = fmaf(-kr[ii], x, dgr[ii]);
      }
      tmem_ld8(tl + tc::DKG + rb, a);
      tmem_ld8(tl + tc::X + rb, a2);
#pragma unroll
      for (int ii = 0; ii < 8; ++ii) {
        const float gam = e[ii] * E0;                     // 2^{G_i}
        const float y = fmaf(a[ii], gam, a2[ii] * e[ii]); // 2^G dkgb + e X1
        const float ky = kr[ii] * y;
        pb[8 * grp + ii] = ky;
        dkr[ii] = fmaf(bt[ii], y, dkr[ii]);
        dgr[ii] = fmaf(bt[ii], ky, dgr[ii]);
      }
      tmem_ld8(tl + tc::DW + rb, a);
#pragma unroll
      for (int ii = 0; ii < 8; ++ii) {
        const float x = a[ii] * f[ii];
        *reinterpret_cast<bf16*>(rowB + bl::K + oB[ii]) = __float2bfloat16(dkr[ii] + x);
        if constexpr (NORM) ydk[ii] = kr[ii] * (dkr[ii] + x);
        float dgv = fmaf(-kr[ii], x, dgr[ii]) * kLn2;
        if (rb + ii == valid - 1) dgv += hdv;
        *reinterpret_cast<float*>(rowG + bl::G + oG[ii]) = dgv;
      }
      if constexpr (NORM) {      // one slot per (row, channel quadrant), summed in a fixed order later
        const float tq = warp_transpose_reduce8(ydq, lid), tk = warp_transpose_reduce8(ydk, lid);
        if ((lid & 3) == 0) {
          s_dot[(rb + (lid >> 2)) * 4 + quad] = tq;
          s_dot[256 + (rb + (lid >> 2)) * 4 + quad] = tk;
        }
      }
    }
    {
      const float tot = warp_transpose_reduce16(pb, lid);
      if ((lid & 1) == 0) s_db[256 + quad * 64 + r0 + (lid >> 1)] = tot;
    }
  }
  tc_mark(p, it, 13);
  if constexpr (NORM) {
    // dq, dk (staged, bf16) -> gradients of the unnormalised rows, one (row, 8 channels) piece per task;
    // y is rebuilt from the unnormalised row exactly as it was when the tile landed
    __syncthreads();
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int i = (tid >> 4) + 32 * n, c16 = tid & 15;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const float4 d4 = *reinterpret_cast<const float4*>(s_dot + 256 * t + 4 * i);
        const float dot = (d4.x + d4.y) + (d4.z + d4.w), rs = s_rs[64 * t + i];
        uint4 raw = t == 0 ? raw_q[n] : raw_k[n];
        float y[8], d[8];
        unpack8(raw, y);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] *= rs;
        pack8v(y, raw);
        unpack8(raw, y);
        unsigned char* tile = sm + (t == 0 ? bl::Q : bl::K);
        ld_bf8(tile, 8192, i, c16, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) d[e] = rs * (d[e] - y[e] * dot);
        st_bf8(tile, 8192, i, c16, d);
      }
    }
  }
  fence_async_smem();
  tc_fence_before();     // every accumulator has been read: the next item's first products may overwrite them
  __syncthreads();
  if (valid == 64) {
    if (lid == 0 && warp >= 4 && warp < 7) {
      if (warp == 4) { for (int b = 0; b < 2; ++b) tma_store_2d(&p.tm_dq, sm + bl::Q + b * 8192, tx + 64 * b, ty); }
      else if (warp == 5) { for (int b = 0; b < 2; ++b) tma_store_2d(&p.tm_dk, sm + bl::K + b * 8192, tx + 64 * b, ty); }
      else { for (int b = 0; b < 4; ++b) tma_store_2d(&p.tm_dg, sm + bl::G + b * 8192, tx + 32 * b, ty); }
      tma_store_commit();
    }
  } else {
    for (int idx = tid; idx < valid * 16; idx += NT) {
      const int r = idx >> 4, ch = idx & 15;
      const int64_t gi = ((cw.token0 + r) * H + head) * 128 + ch * 8;
      const int so = (ch >> 3) * 8192 + sw128_chunk(r, ch & 7);
      *reinterpret_cast<uint4*>(p.dq + gi) = *reinterpret_cast<const uint4*>(sm + bl::Q + so);
      *reinterpret_cast<uint4*>(p.dk + gi) = *reinterpret_cast<const uint4*>(sm + bl::K + so);
    }
    for (int idx = tid; idx < valid * 32; idx += NT) {
      const int r = idx >> 5, ch = idx & 31;
      *reinterpret_cast<float4*>(p.dg + ((cw.token0 + r) * H + head) * 128 + ch * 4) =
          *reinterpret_cast<const float4*>(sm + bl::G + (ch >> 3) * 8192 + r * 128 + (((ch & 7) ^ (r & 7)) << 4));
    }
  }
  if (tid < valid) {
    float t = 0.f;
#pragma unroll
    for (int part = 0; part < 8; ++part) t += s_db[part * 64 + tid];
    p.db[(cw.token0 + tid) * H + head] = t;
  }
  tc_mark(p, it, 14);
  return 0;
  };
  rc = body();
  tc_mark(p, it, 18);
  if (rc) break;
  pre = next_ok;
  prev_full = valid == 64;
  ph ^= 1;
  ++it;
  }  // work items
  if (lid == 0 && (warp == 0 || (warp >= 4 && warp < 7))) tma_store_wait_read();      // staged tiles must outlive the bulk stores' reads
  if (rc && tid == 0 && p.error) atomicExch(p.error, rc);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_slot[0], 512);
}

static __device__ int g_bwd_tc_error = 0;

int launch_bwd_chunk_tc(const bf16* q, const bf16* k, const bf16* v, const float* g, const float* beta,
                        const bf16* akk, const bf16* h, const bf16* dh, const bf16* vnew,
                        const bf16* dv2, const bf16* dout, bf16* dq, bf16* dk, bf16* dv, float* dg,
                        float* db, const float* rstd_q, const float* rstd_k, const int32_t* cu,
                        const int32_t* co, int nseq, int H, int64_t tokens, int chunks, long long* prof,
                        cudaStream_t s) {
  if (chunks == 0) return KDA_OK;
  if ((rstd_q == nullptr) != (rstd_k == nullptr)) return KDA_ERR_ARG;
  BwdTcParams p;
  p.prof = prof;
  p.q = q; p.k = k; p.rstd_q = rstd_q; p.rstd_k = rstd_k;
  const int64_t cols = (int64_t)H * 128, hrows = (int64_t)chunks * H * 128;
  bool ok = make_tensor_map(&p.tm_h, h, hrows, 128, 128) && make_tensor_map(&p.tm_dh, dh, hrows, 128, 128) &&
            make_tensor_map(&p.tm_do, dout, tokens, cols, 64) && make_tensor_map(&p.tm_vn, vnew, tokens, cols, 64) &&
            make_tensor_map(&p.tm_dv2, dv2, tokens, cols, 64) && make_tensor_map(&p.tm_v, v, tokens, cols, 64) &&
            make_tensor_map(&p.tm_k, k, tokens, cols, 64) && make_tensor_map(&p.tm_q, q, tokens, cols, 64) &&
            make_tensor_map(&p.tm_a, akk, tokens, (int64_t)H * 64, 64) &&
            make_tensor_map(&p.tm_g, g, tokens, cols, 64, true) &&
            make_tensor_map(&p.tm_dq, dq, tokens, cols, 64) && make_tensor_map(&p.tm_dk, dk, tokens, cols, 64) &&
            make_tensor_map(&p.tm_dv, dv, tokens, cols, 64) && make_tensor_map(&p.tm_dg, dg, tokens, cols, 64, true);
  if (!ok) return KDA_ERR_LAUNCH;
  p.beta = beta; p.dq = dq; p.dk = dk; p.dv = dv; p.dg = dg; p.db = db;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.nseq = nseq; p.H = H;
  p.total = chunks * H;
  p.tokens = tokens;
  p.scale = 0.08838834764831845f;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    return KDA_ERR_LAUNCH;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), g_bwd_tc_error) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  const int smem = (rstd_q ? bl::TOTAL_NORM : bl::TOTAL_PLAIN) + 1024;
  auto kernel = rstd_q ? kda_bwd_chunk_tc_kernel<true> : kda_bwd_chunk_tc_kernel<false>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  StageScope timing(kStageBwdChunk, s);
  kernel<<<(unsigned)(p.total < sms ? p.total : sms), NT, smem, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

int bwd_chunk_tc_error_word() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_bwd_tc_error, sizeof(int)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(g_bwd_tc_error, &zero, sizeof(int));
  return v;
}

}  // namespace kda
