// Chunk-parallel half of the forward pass on tcgen05 tensor cores: per (chunk, head), one persistent
// kernel computes the gated pairwise products, the WY solve and the WY products
//
//   Aqk = scale tril(Q~ K~^T),  L = stril(diag(beta) K~ K~^T),  A = (I + L)^-1,
//   w = A (beta k 2^G),  u = A (beta v),  kg = k 2^{G_last - G},  qg = scale q 2^G
//
// (reference stages: fwd/triton/chunk_kda_fwd_intra_sub_chunk_forloop.py:66,
//  fwd/cute/chunk_kda_k3b_offdiag_cutedsl.py:177, fwd/cute/chunk_kda_k4b_inverse_cutedsl.py:188,
//  fwd/triton/recompute_w_u.py:257).
//
//   phase 0  TMA: q, k, v, G (the next item's tiles are requested as their regions die).
//   phase 1  every (row, 8 channels) piece once: Qr = q 2^{G - R_b}, Kr = k 2^{G - R_b} (R_b = gate of
//            the first row of the 16-row block b of the row), the column operands
//            Kn_r = k 2^{R_r - G} for r >= b, the WY operands beta k 2^G, beta v (in place), and the
//            results kg, qg.  Per element two exponentials; everything else comes from a small
//            per-(block, channel) table.
//   phase 2  UMMA, transposed, N = 16 per row block r:  Aqk^T[j][i], P^T[j][i] = Kn_r {Qr, Kr}_r^T
//   phase 3  epilogue: masked, scaled Aqk tile (bf16); L in fp32; A = (I + L)^-1 by 16 x 16 blocks on
//            the CUDA cores in fp32; A as a bf16 operand tile (which is also the stored tape)
//   phase 4  UMMA M = 64, N = 128:  w = A (beta k 2^G),  u = A (beta v);  epilogue; TMA stores.
//
// Gate rebasing and its range contract are those of the reference (fwd/triton/gate_fwd.py:619-631):
// exponents are clamped at 126, so masked entries cannot produce NaN.
// All barrier waits are bounded (error word + early exit instead of a hang).
#include "kda_common.cuh"
#include "kda_sm100.cuh"
#include "kda_timing.cuh"

#include <type_traits>

namespace kda {
namespace {

using namespace sm100;

struct PrepParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_g;                       // inputs
  CUtensorMap tm_qg, tm_kg, tm_w, tm_u, tm_aqk, tm_akk;     // results
  const float* beta;
  bf16* qg; bf16* kg; bf16* w; bf16* u; bf16* aqk; bf16* akk;
  float* rstd_q; float* rstd_k;    // NORM kernels: 1 / sqrt(sum x^2 + eps) of every q and k row, [tokens, H]
  float eps;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int* error;
  int nseq, H, total;          // total = chunk capacity x heads work items
  int64_t tokens;              // rows of the packed buffers
  float scale;
  long long* prof;             // debugging aid: phase timestamps of the 20th item of the first 64 CTAs
};

__device__ __forceinline__ void pr_mark(const PrepParams& p, int it, int slot) {
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

namespace pl {  // shared-memory layout (bytes)
constexpr int Q = 0, K = 16384, V = 32768, G = 49152, QKR = 81920, KN = 114688,
              KG = 155648, AT = 172032, AQK = 180224, LF = 188416, AF = 205824, MISC = 223232,
              OFFS = 228352, TOTAL = 230400;
constexpr int kOffCache = 256;          // cu_seqlens / chunk_offsets entries kept in shared memory
constexpr int TAB = AT;                 // phase 1 table (3 KiB) over the A / Aqk tiles, dead until phase 3
constexpr int QG = Q;                   // qg is staged in place over q
constexpr int W = QKR, U = QKR + 16384; // result staging over the Qr / Kr tile, dead after phase 2
constexpr int LP = 68;                  // pitch of the fp32 matrices L and A
}  // namespace pl
namespace pt {  // tensor-memory columns
constexpr int AQ = 0, W = 128, U = 256;   // AQ: 32 columns per row block, Aqk^T then P^T
}

constexpr int NT = 512;

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
// byte offset of Kn_r inside the KN region: the tiles have 16, 32, 48, 64 rows of 256 bytes
__device__ __forceinline__ int kn_off(int r) { return 4096 * (r * (r + 1) / 2); }

// NORM: q and k arrive unnormalised; every row is scaled to unit L2 norm (and rounded to bf16, as a
// separate l2norm launch would leave it) while its pieces pass through the registers of phase 1a,
// and the two reciprocal norms are kept for the backward pass
// (reference stages: fwd/triton/l2norm_fwd.py:22, applied right before the core in
// examples/kda_training.py:412-421).
template <bool NORM>
__global__ void __launch_bounds__(NT, 1) kda_prepare_tc_kernel(const __grid_constant__ PrepParams p) {
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment by offset, so the compiler still knows this is shared memory
  unsigned char* sm = smem_dyn + ((1024u - (saddr(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + pl::MISC);     // [0] TMA, [1] pairwise, [2] w / u
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + pl::MISC + 64);
  volatile int* s_abort = reinterpret_cast<volatile int*>(sm + pl::MISC + 72);
  float* s_beta = reinterpret_cast<float*>(sm + pl::MISC + 128);           // [64]
  int* s_next = reinterpret_cast<int*>(sm + pl::MISC + 96);                // next item: token0 (two words), valid
  float* Lf = reinterpret_cast<float*>(sm + pl::LF);
  float* Af = reinterpret_cast<float*>(sm + pl::AF);
  float* Bf = reinterpret_cast<float*>(sm + pl::KN);     // A[r][r] L[r][m] blocks: the column-operand tiles are dead by then
  float* tab = reinterpret_cast<float*>(sm + pl::TAB);   // [14][128], see phase 1
  const unsigned char* sG = sm + pl::G;

  const int tid = threadIdx.x, warp = tid >> 5, lid = tid & 31;
  const int quad = warp & 3, wq = warp >> 2;       // TMEM lane quadrant; which of its four warps
  const int H = p.H;

  // Work items are located by a binary search over the sequence offsets: from shared memory when
  // they fit (a chain of dependent global loads per item would sit on the critical path).
  int32_t* s_cu = reinterpret_cast<int32_t*>(sm + pl::OFFS);
  int32_t* s_co = s_cu + pl::kOffCache;
  const bool cached = p.nseq + 1 <= pl::kOffCache;
  if (cached)
    for (int i = tid; i <= p.nseq; i += NT) { s_cu[i] = p.cu_seqlens[i]; s_co[i] = p.chunk_offsets[i]; }
  const int32_t* cu_off = cached ? s_cu : p.cu_seqlens;
  const int32_t* ch_off = cached ? s_co : p.chunk_offsets;
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 4);       // one arrival per issuing thread
    mbar_init(&bar[2], 2);
    mbar_init_fence();
    *s_abort = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * quad) << 16);

  // Loads of one work item in three parts, issued as the regions of the previous item die:
  // 0 = G (arms the barrier for all parts), 1 = q, 2 = k and v.  Thread 0 only.
  auto issue_loads = [&](int part, int head, int64_t token0) {
    const int ty = (int)token0, tx = head * 128;
    if (part == 0) {
      mbar_expect_tx(&bar[0], 3 * 16384 + 32768);
      for (int b = 0; b < 4; ++b) tma_load_2d(sm + pl::G + b * 8192, &p.tm_g, tx + 32 * b, ty, &bar[0]);
    } else if (part == 1) {
      for (int b = 0; b < 2; ++b) tma_load_2d(sm + pl::Q + b * 8192, &p.tm_q, tx + 64 * b, ty, &bar[0]);
    } else {
      for (int b = 0; b < 2; ++b) {
        tma_load_2d(sm + pl::K + b * 8192, &p.tm_k, tx + 64 * b, ty, &bar[0]);
        tma_load_2d(sm + pl::V + b * 8192, &p.tm_v, tx + 64 * b, ty, &bar[0]);
      }
    }
  };

  // The 16 x 16 blocks above the diagonal of A are zero.  No work item writes them (the solve fills the
  // diagonal and lower blocks only) and the fp32 matrix has a region of its own, so once is enough.
  for (int idx = tid; idx < 6 * 256; idx += NT) {
    const int blk = idx >> 8, i = (idx >> 4) & 15, j = idx & 15;
    const int br = blk >= 5 ? 2 : (blk >= 3 ? 1 : 0);          // (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
    const int bc = br == 0 ? blk + 1 : (br == 1 ? blk - 1 : 3);
    Af[(16 * br + i) * pl::LP + 16 * bc + j] = 0.f;
  }
  uint32_t ph = 0;
  int rc = 0, it = 0;
  bool pre = false;              // this item's loads were issued by the previous item
  ChunkWork cw_next{};
  float beta_next = 0.f;
  for (int wi = blockIdx.x; wi < p.total; wi += gridDim.x) {
  const int chunk = wi / H, head = wi - chunk * H;
  const ChunkWork cw = pre ? cw_next : locate_chunk(cu_off, ch_off, p.nseq, chunk);
  if (cw.valid == 0) continue;               // capacity slot past the last active chunk
  if (!pre && !chunk_in_range(cw, p.tokens)) {     // (with pre the previous item checked it)
    if (tid == 0 && p.error) atomicExch(p.error, kOffsetsOutOfRange);
    continue;
  }
  const int valid = cw.valid;
  const int ty = (int)cw.token0, tx = head * 128;
  if (tid < 64)
    s_beta[tid] = pre ? beta_next : (tid < valid ? p.beta[(cw.token0 + tid) * H + head] : 0.f);
  // No CTA barrier here: everything written before the barrier that ends the table step (beta, the
  // table over the A tile, tiles loaded for an item without prefetch) was last read before the
  // previous item's final barrier, where thread 0 had also drained every store group but w, u.
  if (tid == 0 && !pre) { issue_loads(0, head, cw.token0); issue_loads(1, head, cw.token0); issue_loads(2, head, cw.token0); }
  // the next item is located by one thread while this item's tiles arrive (the search is a chain of
  // dependent loads); everybody reads the result after the barrier that ends the table step
  int head_n = 0;
  bool next_ok = false;
  if (tid == 160) {
    const int wn = wi + (int)gridDim.x;
    ChunkWork nx{};
    if (wn < p.total) nx = locate_chunk(cu_off, ch_off, p.nseq, wn / H);
    if (!chunk_in_range(nx, p.tokens)) {     // not prefetched; the item itself reports and skips
      nx.valid = 0;
    }
    s_next[0] = (int)(nx.token0 & 0xffffffffLL);
    s_next[1] = (int)(nx.token0 >> 32);
    s_next[2] = nx.valid;
  }
  auto body = [&]() -> int {
  pr_mark(p, it, 0);
  if (!mbar_wait(&bar[0], ph)) *s_abort = 1;
  pr_mark(p, it, 1);
  // partial tail chunk: rows >= valid hold another sequence's tokens or unwritten memory.  Zero them
  // in every token tile and repeat the last gate row, so no later step needs a row guard.
  if (valid < 64) {
    const int tiles[3] = {pl::Q, pl::K, pl::V};
    for (int idx = tid; idx < (64 - valid) * 16; idx += NT) {
      const int r = valid + (idx >> 4), ch = idx & 15;
#pragma unroll
      for (int t = 0; t < 3; ++t)
        *reinterpret_cast<uint4*>(sm + tiles[t] + (ch >> 3) * 8192 + sw128_chunk(r, ch & 7)) = make_uint4(0, 0, 0, 0);
    }
    for (int idx = tid; idx < (64 - valid) * 32; idx += NT) {
      const int r = valid + (idx >> 5), ch = idx & 31;
      const int off = (ch >> 3) * 8192, c = ch & 7;
      *reinterpret_cast<float4*>(sm + pl::G + off + r * 128 + ((c ^ (r & 7)) << 4)) =
          *reinterpret_cast<const float4*>(sm + pl::G + off + (valid - 1) * 128 + ((c ^ ((valid - 1) & 7)) << 4));
    }
    __syncthreads();
  }

  // ---- table, per (block pair, channel): 2^{R_r - R_b} for (r, b) = (1,0) (2,0) (3,0) (2,1) (3,1) (3,2)
  for (int e = tid; e < 6 * 128; e += NT) {
    const int k6 = e >> 7, ch = e & 127;
    auto gate = [&](int row) {
      return *reinterpret_cast<const float*>(sG + (ch >> 5) * 8192 + row * 128 +
                                             (((((ch & 31) >> 2) ^ (row & 7)) << 4) | ((ch & 3) << 2)));
    };
    const int bb = k6 >= 5 ? 2 : (k6 >= 3 ? 1 : 0);
    const int rr = bb == 0 ? k6 + 1 : (bb == 1 ? k6 - 1 : 3);
    tab[e] = fexp2(gate(16 * rr) - gate(16 * bb));
  }
  if (tid == 0) tma_store_wait_read();       // the w, u staging tiles (over Kr / Kn) of the previous item have been read
  __syncthreads();
  pr_mark(p, it, 2);
  if (*s_abort) return 2;
  {   // the next item, and the beta value this thread carries over to it
    const int wn = wi + (int)gridDim.x;
    head_n = wn - (wn / H) * H;
    cw_next.token0 = (int64_t)(((uint64_t)(uint32_t)s_next[1] << 32) | (uint32_t)s_next[0]);
    cw_next.valid = s_next[2];
    next_ok = cw_next.valid > 0;        // 0 also when there is no further item
    if (tid < 64)
      beta_next = (next_ok && tid < cw_next.valid) ? p.beta[(cw_next.token0 + tid) * H + head_n] : 0.f;
  }

  // ---- phase 1a: the operands of the pairwise products; one (row, 8 channels) piece per task ---------
  float gkeep[2][8];                 // the gate rows of this thread's two tasks, reused by phase 1b
  uint4 qkeep[2], kkeep[2];          // and their q, k pieces as raw bf16 vectors
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int task = tid + n * NT;
    const int i = task >> 4, c16 = task & 15, b = i >> 4, c0 = 8 * c16;
    float qq[8], kk[8], r[8], ei[8], o[8];
    float (&g)[8] = gkeep[n];
    qkeep[n] = ld_raw8(sm + pl::Q, 8192, i, c16);
    kkeep[n] = ld_raw8(sm + pl::K, 8192, i, c16);
    unpack8(qkeep[n], qq);
    unpack8(kkeep[n], kk);
    if constexpr (NORM) {
      // the 16 lanes of a half-warp hold one row: sum of squares in the order of the stand-alone
      // kernel (eight fused multiply-adds per lane, then a butterfly over the lanes)
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) { sq = fmaf(qq[e], qq[e], sq); sk = fmaf(kk[e], kk[e], sk); }
#pragma unroll
      for (int d = 8; d > 0; d >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, d);
        sk += __shfl_xor_sync(0xffffffffu, sk, d);
      }
      const float rq = rsqrtf(sq + p.eps), rk = rsqrtf(sk + p.eps);
      if (c16 == 0 && i < valid) {
        p.rstd_q[(cw.token0 + i) * H + head] = rq;
        p.rstd_k[(cw.token0 + i) * H + head] = rk;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) { qq[e] *= rq; kk[e] *= rk; }
      pack8v(qq, qkeep[n]);        // the bf16 rows are what every later step works with
      pack8v(kk, kkeep[n]);
      unpack8(qkeep[n], qq);
      unpack8(kkeep[n], kk);
    }
    ld_g8(sG, i, c0, g);
    ld_g8(sG, 16 * b, c0, r);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float er = fexp2(g[e] - r[e]);              // 2^{G_i - R_b} <= 1
      ei[e] = fexp2(fminf(r[e] - g[e], 126.f));         // 2^{R_b - G_i}
      qq[e] *= er;
      o[e] = kk[e] * er;
    }
    // one row-operand tile for both sides: rows 32 b .. 32 b + 15 hold Qr of block b, the next 16 Kr,
    // so that one N = 32 product per row block and k step gives Aqk^T and P^T side by side
    st_bf8(sm + pl::QKR, 16384, 32 * b + (i & 15), c16, qq);
    st_bf8(sm + pl::QKR, 16384, 32 * b + 16 + (i & 15), c16, o);
    // column operands Kn_r[i] = k_i 2^{R_r - G_i} for the row blocks r >= b
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = kk[e] * ei[e];
    st_bf8(sm + pl::KN + kn_off(b), 16 * (b + 1) * 128, i, c16, o);
    for (int rr = b + 1; rr < 4; ++rr) {
      const int slot = b == 0 ? rr - 1 : (b == 1 ? rr + 1 : 5);
      // lanes 32 bytes apart: the upper four of a quarter-warp read their halves in the other order
      const int odd = (c16 >> 2) & 1;
      const float4 ta = *reinterpret_cast<const float4*>(tab + slot * 128 + c0 + 4 * odd);
      const float4 tb = *reinterpret_cast<const float4*>(tab + slot * 128 + c0 + 4 - 4 * odd);
      const float4 t0 = odd ? tb : ta, t1 = odd ? ta : tb;
      const float f[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};     // 2^{R_r - R_b} <= 1
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = kk[e] * (ei[e] * f[e]);
      st_bf8(sm + pl::KN + kn_off(rr), 16 * (rr + 1) * 128, i, c16, o);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  pr_mark(p, it, 3);

  // ---- phase 2: pairwise products, one issuing thread per row block (lane 0 of warps 0..3) ---------
  //   (issuing the products of row blocks 0, 1 half way through phase 1a, behind one more barrier,
  //   was measured: 0.887 against 0.850 ms)
  //   Aqk^T[j][i in block r] = sum_kappa Kn_r[j] Qr[i],   P^T[j][i] = sum_kappa Kn_r[j] Kr[i]
  //   (M = 64 rows j of which the first 16 (r + 1) are meaningful; the rest are masked below)
  if (lid == 0 && warp < 4) {
    tc_fence_after();
    const int r = warp;
    const uint32_t kn = saddr(sm + pl::KN + kn_off(r)), box = 16 * (r + 1) * 128;
    const uint32_t rows = saddr(sm + pl::QKR) + 4096 * r;
    const uint32_t acc = tmem + pt::AQ + 32 * r;       // columns 32 r .. +15: Aqk^T, +16 .. +31: P^T
    const uint32_t id = instr_desc(64, 32, 0, 0);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) umma(acc, desc_kmajor(kn, ks, box), desc_kmajor(rows, ks, 16384), id, ks > 0);
    umma_commit(&bar[1]);
  }
  // ---- phase 1b, while the products run: the WY operands beta k 2^G, beta v and the results kg, qg,
  //      each in place or into its staging tile -----------------------------------------------------------
  float gl[8];                       // last gate row: depends on the channel piece only
  ld_g8(sG, valid - 1, 8 * (tid & 15), gl);
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int task = tid + n * NT;
    const int i = task >> 4, c16 = task & 15;
    float qq[8], kk[8], vv[8], o[8];
    const float (&g)[8] = gkeep[n];
    unpack8(qkeep[n], qq);
    unpack8(kkeep[n], kk);
    ld_bf8(sm + pl::V, 8192, i, c16, vv);
    const float bt = s_beta[i];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gam = fexp2(g[e]);
      qq[e] = qq[e] * gam * p.scale;                    // qg = scale q 2^G
      o[e] = kk[e] * fexp2(gl[e] - g[e]);               // kg = k 2^{G_last - G}
      kk[e] = kk[e] * gam * bt;                         // beta k 2^G
      vv[e] *= bt;                                      // beta v
    }
    st_bf8(sm + pl::QG, 8192, i, c16, qq);
    st_bf8(sm + pl::KG, 8192, i, c16, o);
    st_bf8(sm + pl::K, 8192, i, c16, kk);
    st_bf8(sm + pl::V, 8192, i, c16, vv);
  }
  fence_async_smem();
  pr_mark(p, it, 12);
  __syncthreads();
  pr_mark(p, it, 13);
  if (tid == 0) {
    // kg and qg leave; G is dead: the next item's gates start arriving
    if (valid == 64) {
      for (int b = 0; b < 2; ++b) {
        tma_store_2d(&p.tm_qg, sm + pl::QG + b * 8192, tx + 64 * b, ty);
        tma_store_2d(&p.tm_kg, sm + pl::KG + b * 8192, tx + 64 * b, ty);
      }
      tma_store_commit();
    }
    if (next_ok) issue_loads(0, head_n, cw_next.token0);
  }
  if (valid < 64) {        // partial chunk: rows < valid only, plain 16-byte stores
    for (int idx = tid; idx < valid * 16; idx += NT) {
      const int r = idx >> 4, ch = idx & 15;
      const int64_t gi = ((cw.token0 + r) * H + head) * 128 + ch * 8;
      const int so = (ch >> 3) * 8192 + sw128_chunk(r, ch & 7);
      *reinterpret_cast<uint4*>(p.qg + gi) = *reinterpret_cast<const uint4*>(sm + pl::QG + so);
      *reinterpret_cast<uint4*>(p.kg + gi) = *reinterpret_cast<const uint4*>(sm + pl::KG + so);
    }
  }
  if (!mbar_wait(&bar[1], ph)) *s_abort = 1;
  tc_fence_after();
  pr_mark(p, it, 4);

  // ---- phase 3a: this warp reads columns i = 16 wq .. 16 wq + 15 of both accumulators; lanes 0..15
  //      of a quadrant hold the rows j = 16 quad + lane (M = 64 layout)
  {
    float a[16], pk[16], bt[16];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const float4 b4 = *reinterpret_cast<const float4*>(s_beta + 16 * wq + 4 * q4);
      bt[4 * q4] = b4.x; bt[4 * q4 + 1] = b4.y; bt[4 * q4 + 2] = b4.z; bt[4 * q4 + 3] = b4.w;
    }
    tmem_ld16(tl + pt::AQ + 32 * wq, a);
    tmem_ld16(tl + pt::AQ + 32 * wq + 16, pk);
    if (lid < 16) {
      const int j = 16 * quad + lid;
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) {
        const int i = 16 * wq + ii;
        const float x = (j <= i && i < valid) ? a[ii] * p.scale : 0.f;
        *reinterpret_cast<bf16*>(sm + pl::AQK + sw128(i, j)) = __float2bfloat16(x);
        if (quad <= wq) Lf[i * pl::LP + j] = (j < i) ? pk[ii] * bt[ii] : 0.f;    // blocks above the diagonal are never read
      }
    }
  }
  __syncthreads();
  pr_mark(p, it, 5);
  if (*s_abort) return 3;

  // ---- phase 3b: A = (I + L)^-1 by 16 x 16 blocks, fp32 ---------------------------------------------------
  if (tid < 64) {  // diagonal blocks: column c of block b by forward substitution
    const int b = tid >> 4, c = tid & 15;
    const float* L = Lf + (16 * b) * pl::LP + 16 * b;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = (i == c) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s -= L[i * pl::LP + j] * x[j];
      x[i] = s;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) Af[(16 * b + i) * pl::LP + 16 * b + c] = x[i];
  }
  __syncthreads();
  pr_mark(p, it, 6);
  // B[r][m] = A[r][r] L[r][m] for the six blocks below the diagonal, all at once (they only need the
  // diagonal blocks): with them every block of the inverse is ONE product,
  //   A[r][c] = -sum_{c <= m < r} B[r][m] A[m][c],
  // so the block diagonals at distance 1, 2, 3 cost one barrier each instead of two.
  if (tid < 384) {
    const int blk = tid >> 6, tile = tid & 63, i = 2 * (tile >> 3), j = 2 * (tile & 7);
    const int r = blk < 3 ? blk + 1 : (blk < 5 ? blk - 1 : 3);     // (1,0) (2,0) (3,0) (2,1) (3,1) (3,2)
    const int m = blk < 3 ? 0 : (blk < 5 ? 1 : 2);
    const float* A0 = Af + (16 * r + i) * pl::LP + 16 * r;          // A[r][r], rows i, i + 1
    const float* B_ = Lf + (16 * r) * pl::LP + 16 * m + j;          // L[r][m], columns j, j + 1
    float s00 = 0.f, s01 = 0.f, s10 = 0.f, s11 = 0.f;
#pragma unroll
    for (int k = 0; k < 16; k += 4) {
      const float4 a0 = *reinterpret_cast<const float4*>(A0 + k);
      const float4 a1 = *reinterpret_cast<const float4*>(A0 + pl::LP + k);
      const float av0[4] = {a0.x, a0.y, a0.z, a0.w}, av1[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float2 bv = *reinterpret_cast<const float2*>(B_ + (k + kk) * pl::LP);
        s00 = fmaf(av0[kk], bv.x, s00); s01 = fmaf(av0[kk], bv.y, s01);
        s10 = fmaf(av1[kk], bv.x, s10); s11 = fmaf(av1[kk], bv.y, s11);
      }
    }
    float* dst = Bf + (16 * r + i) * pl::LP + 16 * m + j;
    *reinterpret_cast<float2*>(dst) = make_float2(s00, s01);
    *reinterpret_cast<float2*>(dst + pl::LP) = make_float2(s10, s11);
  }
  __syncthreads();
  // A pair of adjacent lanes owns a 2 x 2 tile of a 16 x 16 result block and splits the inner
  // dimension between its lanes in interleaved groups of four (16-byte loads along k for the row
  // operand, 8-byte loads for the column operand; the two lanes' column rows sit 16 banks apart);
  // one shuffle per accumulator joins the halves and each lane then stores one row of the tile.
  auto round = [&](auto dist_tag) {
    constexpr int DIST = decltype(dist_tag)::value;
    constexpr int pairs = 4 - DIST;
    const int ks = tid & 1, rest = tid >> 1;
    const bool act = tid < pairs * 128;                           // whole warps
    const int c = rest >> 6, r = c + DIST, i = 2 * ((rest >> 3) & 7), j = 2 * (rest & 7);
    if (act) {
      const float* A0 = Bf + (16 * r + i) * pl::LP + 16 * c;      // B[r][c .. r-1], rows i, i + 1
      const float* B_ = Af + (16 * c) * pl::LP + 16 * c + j;      // A[c .. r-1][c], columns j, j + 1
      float s00 = 0.f, s01 = 0.f, s10 = 0.f, s11 = 0.f;
#pragma unroll
      for (int m = 0; m < 2 * DIST; ++m) {
        const int k = 4 * (ks + 2 * m);
        const float4 a0 = *reinterpret_cast<const float4*>(A0 + k);
        const float4 a1 = *reinterpret_cast<const float4*>(A0 + pl::LP + k);
        const float av0[4] = {a0.x, a0.y, a0.z, a0.w}, av1[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float2 bv = *reinterpret_cast<const float2*>(B_ + (k + kk) * pl::LP);
          s00 = fmaf(av0[kk], bv.x, s00); s01 = fmaf(av0[kk], bv.y, s01);
          s10 = fmaf(av1[kk], bv.x, s10); s11 = fmaf(av1[kk], bv.y, s11);
        }
      }
      s00 += __shfl_xor_sync(0xffffffffu, s00, 1); s01 += __shfl_xor_sync(0xffffffffu, s01, 1);
      s10 += __shfl_xor_sync(0xffffffffu, s10, 1); s11 += __shfl_xor_sync(0xffffffffu, s11, 1);
      float* dst = Af + (16 * r + i + ks) * pl::LP + 16 * c + j;
      *reinterpret_cast<float2*>(dst) = ks ? make_float2(-s10, -s11) : make_float2(-s00, -s01);
    }
    __syncthreads();
  };
  round(std::integral_constant<int, 1>{});
  round(std::integral_constant<int, 2>{});
  round(std::integral_constant<int, 3>{});
  pr_mark(p, it, 7);
  // A as a bf16 operand tile [i][j] (K-major, one 128-byte-swizzled box): also the stored tape
  for (int idx = tid; idx < 64 * 8; idx += NT) {
    const int r = idx >> 3, c = idx & 7, odd = (c >> 2) & 1;
    // lanes 32 bytes apart: the upper four of a quarter-warp read their halves in the other order
    const float4 fa = *reinterpret_cast<const float4*>(Af + r * pl::LP + 8 * c + 4 * odd);
    const float4 fb = *reinterpret_cast<const float4*>(Af + r * pl::LP + 8 * c + 4 - 4 * odd);
    const float4 lo = odd ? fb : fa, hi = odd ? fa : fb;
    const float f8[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    uint4 v;
    pack8v(f8, v);
    *reinterpret_cast<uint4*>(sm + pl::AT + sw128_chunk(r, c)) = v;
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  pr_mark(p, it, 8);
  // ---- phase 4: w = A (beta k 2^G) (thread 0), u = A (beta v) (thread 32); the tapes leave ---------------
  if (lid == 0 && warp < 2) {
    tc_fence_after();
    const uint32_t at = saddr(sm + pl::AT);
    const uint32_t bop = saddr(sm + (warp == 0 ? pl::K : pl::V));
    const uint32_t id = instr_desc(64, 128, 0, 1);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      umma(tmem + (warp == 0 ? pt::W : pt::U), desc_kmajor(at, ks, 0), desc_mnmajor(bop, ks, 8192), id, ks > 0);
    umma_commit(&bar[2]);
    if (warp == 0 && next_ok) {       // the q tile staged qg: reload it once that store has read it
      tma_store_wait_read();
      issue_loads(1, head_n, cw_next.token0);
    }
    if (warp == 0 && valid == 64) {
      tma_store_2d(&p.tm_aqk, sm + pl::AQK, head * 64, ty);
      tma_store_2d(&p.tm_akk, sm + pl::AT, head * 64, ty);
      tma_store_commit();
    }
  }
  if (valid < 64) {
    for (int idx = tid; idx < valid * 8; idx += NT) {
      const int r = idx >> 3, c = idx & 7;
      const int64_t gi = ((cw.token0 + r) * H + head) * 64 + c * 8;
      *reinterpret_cast<uint4*>(p.aqk + gi) = *reinterpret_cast<const uint4*>(sm + pl::AQK + sw128_chunk(r, c));
      *reinterpret_cast<uint4*>(p.akk + gi) = *reinterpret_cast<const uint4*>(sm + pl::AT + sw128_chunk(r, c));
    }
  }
  if (!mbar_wait(&bar[2], ph)) *s_abort = 1;
  tc_fence_after();
  pr_mark(p, it, 9);
  if (warp == 0 && lid < 4 && next_ok) {      // the k and v tiles are dead: one lane per 64-channel tile
    // (a thread spends about 50 ns per bulk copy it issues, and this warp's share of the epilogue
    // below is what the barrier after it waits for)
    const int b = lid >> 1, tyn = (int)cw_next.token0, txn = head_n * 128 + 64 * b;
    if (lid & 1) tma_load_2d(sm + pl::V + b * 8192, &p.tm_v, txn, tyn, &bar[0]);
    else tma_load_2d(sm + pl::K + b * 8192, &p.tm_k, txn, tyn, &bar[0]);
  }

  // ---- epilogue: rows i = 16 quad + lane (lanes 0..15), columns 32 wq .. 32 wq + 31 of w and u -----------
  {
    float a[32];
    const int i = 16 * quad + lid;
    tmem_ld32(tl + pt::W + 32 * wq, a);
    if (lid < 16) {
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        uint4 v;
        pack8v(a + 8 * qd, v);
        *reinterpret_cast<uint4*>(sm + pl::W + (wq >> 1) * 8192 + sw128_chunk(i, 4 * (wq & 1) + qd)) = v;
      }
    }
    tmem_ld32(tl + pt::U + 32 * wq, a);
    if (lid < 16) {
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        uint4 v;
        pack8v(a + 8 * qd, v);
        *reinterpret_cast<uint4*>(sm + pl::U + (wq >> 1) * 8192 + sw128_chunk(i, 4 * (wq & 1) + qd)) = v;
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  if (tid == 0) tma_store_wait_read();       // qg, kg, Aqk, A have left their tiles (issued long ago)
  __syncthreads();
  pr_mark(p, it, 10);
  if (*s_abort) return 4;
  if (valid == 64) {
    if (tid == 0) {
      for (int b = 0; b < 2; ++b) {
        tma_store_2d(&p.tm_w, sm + pl::W + b * 8192, tx + 64 * b, ty);
        tma_store_2d(&p.tm_u, sm + pl::U + b * 8192, tx + 64 * b, ty);
      }
      tma_store_commit();
    }
  } else {
    for (int idx = tid; idx < valid * 16; idx += NT) {
      const int r = idx >> 4, ch = idx & 15;
      const int64_t gi = ((cw.token0 + r) * H + head) * 128 + ch * 8;
      const int so = (ch >> 3) * 8192 + sw128_chunk(r, ch & 7);
      *reinterpret_cast<uint4*>(p.w + gi) = *reinterpret_cast<const uint4*>(sm + pl::W + so);
      *reinterpret_cast<uint4*>(p.u + gi) = *reinterpret_cast<const uint4*>(sm + pl::U + so);
    }
  }
  pr_mark(p, it, 11);
  return 0;
  };
  rc = body();
  if (rc) break;
  pre = next_ok;
  ph ^= 1;
  ++it;
  }  // work items
  if (tid == 0) tma_store_wait_read();      // staged tiles must outlive the bulk stores' reads
  if (rc && tid == 0 && p.error) atomicExch(p.error, 32 + rc);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_slot[0], 512);
}

static __device__ int g_prepare_error = 0;

}  // namespace

long long* debug_profile_buffer();

int launch_prepare_tc(const bf16* q, const bf16* k, const bf16* v, const float* g, const float* beta,
                      bf16* aqk, bf16* akk, bf16* w, bf16* u, bf16* kg, bf16* qg, float* rstd_q,
                      float* rstd_k, float eps, const int32_t* cu, const int32_t* co, int nseq, int H,
                      int64_t tokens, int chunks, cudaStream_t s) {
  if (chunks == 0) return KDA_OK;
  PrepParams p;
  const int64_t cols = (int64_t)H * 128, acols = (int64_t)H * 64;
  bool ok = make_tensor_map(&p.tm_q, q, tokens, cols, 64) && make_tensor_map(&p.tm_k, k, tokens, cols, 64) &&
            make_tensor_map(&p.tm_v, v, tokens, cols, 64) && make_tensor_map(&p.tm_g, g, tokens, cols, 64, true) &&
            make_tensor_map(&p.tm_qg, qg, tokens, cols, 64) && make_tensor_map(&p.tm_kg, kg, tokens, cols, 64) &&
            make_tensor_map(&p.tm_w, w, tokens, cols, 64) && make_tensor_map(&p.tm_u, u, tokens, cols, 64) &&
            make_tensor_map(&p.tm_aqk, aqk, tokens, acols, 64) && make_tensor_map(&p.tm_akk, akk, tokens, acols, 64);
  if (!ok) return KDA_ERR_LAUNCH;
  p.beta = beta; p.qg = qg; p.kg = kg; p.w = w; p.u = u; p.aqk = aqk; p.akk = akk;
  p.rstd_q = rstd_q; p.rstd_k = rstd_k; p.eps = eps;
  if ((rstd_q == nullptr) != (rstd_k == nullptr)) return KDA_ERR_ARG;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.nseq = nseq; p.H = H;
  p.total = chunks * H;
  p.tokens = tokens;
  p.scale = 0.08838834764831845f;  // 128^-0.5
  p.prof = debug_profile_buffer();
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1 ||
      cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), g_prepare_error) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  const int smem = pl::TOTAL + 1024;
  auto kernel = rstd_q ? kda_prepare_tc_kernel<true> : kda_prepare_tc_kernel<false>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  StageScope timing(kStagePrepare, s);
  kernel<<<(unsigned)(p.total < sms ? p.total : sms), NT, smem, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

int prepare_tc_error_word() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_prepare_error, sizeof(int)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(g_prepare_error, &zero, sizeof(int));
  return v;
}

}  // namespace kda
