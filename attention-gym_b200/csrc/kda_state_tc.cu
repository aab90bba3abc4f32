// Inter-chunk state recurrence on the 5th-generation tensor cores (tcgen05 / UMMA), forward.
//
//   v_new = u - w h ;  o = qg h + Aqk v_new ;  h <- diag(2^{G_last}) h + kg^T v_new
//
// NS = 1, 2 or 4 CTAs (256 threads each) walk the chunks of one (sequence, head); each owns
// N = 128 / NS value columns of the state (every product below is separable along v), so a few long
// chains still fill the SMs.  The fp32 state slice h [128 x N] lives in tensor memory for the whole
// walk (128 lanes x N columns) and never goes to HBM in the forward pass; two more accumulators
// alternate as D1 = [w h ; qg h + Aqk v_new].  Warp w works on tensor-memory lanes 32 (w % 4) .. +31
// and on the half w / 4 of the slice's columns.
// Per chunk:
//   a. every thread reads its half row of h, writes it as bf16 into the swizzled MN-major B tile,
//      multiplies by the chunk decay and stores it back to tensor memory;
//   b. UMMA 128x128x128:  D1 = [w ; qg] h          (A: TMA tile, K-major; B: the h tile)
//   c. lane quadrants 0, 1 read D1 rows 0..63, form v_new = u - w h and write it as the bf16 B
//      tile; meanwhile quadrants 2, 3 store the output rows (D1 rows 64..127) of the previous chunk;
//   d. UMMA 128x128x64:   D1 += [0 ; Aqk] v_new    and   h += kg^T v_new  (A: kg, MN-major).
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
  CUtensorMap tm_hout, tm_vnew, tm_o;      // result tiles leave shared memory with TMA stores
  const float* g; const float* h0; float* ht; float* trans_out;
  const int32_t* limit_in;   // per (sequence, head): walk only this many leading chunks (NULL = all)
  int32_t* limit_out;        // per (sequence, head): chunks after which the transition is exactly zero
  bf16* o; bf16* h_out; bf16* vnew_out;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int* error;
  int nseq, H;
  int64_t tokens;            // rows of the packed buffers
  int use_u, use_o;
  long long* prof;      // debugging aid: phase timestamps of chunk 10 of the first 64 CTAs (rows 32..63)
};

long long* debug_profile_buffer();

__device__ __forceinline__ void st_mark(long long* prof, int c, int slot) {
#ifdef KDA_PHASE_PROFILE
  if (prof && c == 10 && threadIdx.x == 0 && blockIdx.x < 64) {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    prof[blockIdx.x * 32 + 20 + slot] = t;
  }
#endif
}

constexpr int kStageBytes = 32768 + 16384 + 16384 + 16384;   // A1, KG, U, A2
struct StateTcLayout {
  static constexpr int A1 = 0, KG = 32768, U = 49152, A2 = 65536;
  static constexpr int H = 2 * kStageBytes;              // 163840
  static constexpr int VN = H + 32768;                   // 196608
  static constexpr int OST = VN + 16384;                 // 212992: staging of one chunk's output rows
  static constexpr int BAR = OST + 16384;                // 229376
  static constexpr int TOTAL = BAR + 1024;
};

__device__ __forceinline__ void pack8(const float* x, uint4& o) {
  o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]);
  o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
}

constexpr int kStateThreads = 256;

// Value split of a chain: 128 / NS state columns per CTA.  Chosen from the number of chains against
// the number of SMs (the reference tiles the same dimension: fwd/triton/chunk_delta_h.py:166 BV = 64,
// bwd/cute/chunk_delta_h_bwd_v1_dispatch.py:53-55 BV = 16 / 32 by tile count); 0 = automatic.
static int g_value_split = 0;
static int pick_value_split(int64_t chains) {
  if (g_value_split == 1 || g_value_split == 2 || g_value_split == 4) return g_value_split;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (chains * 4 <= sms) return 4;
  if (chains * 2 <= sms) return 2;
  return 1;
}

// Byte offset of the 16-byte piece holding columns c .. c + 7 of row r in a tile made of 64-column
// boxes `box_bytes` apart.
__device__ __forceinline__ int tile_off(int r, int c, int box_bytes) {
  return (c >> 6) * box_bytes + sw128_chunk(r, (c & 63) >> 3);
}

// NS = number of CTAs that share one (sequence, head) chain; each owns N = 128 / NS value columns of
// the state and of every [.., v] product (all of them are separable along v).  The operand tiles
// w, qg, kg, Aqk are the same for the NS CTAs of a chain (the second to read them hits L2).
// CTAs with blockIdx.x >= NS * nseq * H (present when trans_out != NULL) walk the same chains with
// u = 0 from an identity state and write the slice transition instead of outputs.  Such a walk stops
// as soon as the running transition is exactly zero in fp32 (every later one is then zero too) and
// reports how many chunks that took (limit_out): past them an entering state cannot change any
// output or state bit that fp32 can hold, so the corrective pass with the true entering state
// (limit_in) only needs those leading chunks.  This is measured on the data, never assumed.
template <int NS>
__global__ void __launch_bounds__(kStateThreads) kda_state_fwd_tc_kernel(const __grid_constant__ StateTcParams p) {
  constexpr int N = D / NS;            // state columns of this CTA
  constexpr int NC = N / 2;            // columns per thread (two warps share a lane quadrant)
  constexpr int NB = (N + 63) / 64;    // 64-column boxes of a slice-shaped tile
  constexpr bool kTileStore = N >= 64; // results leave by TMA tile stores (whole boxes) or directly
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment by offset, so the compiler still knows this is shared memory
  unsigned char* smem = smem_dyn + ((1024u - (saddr(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + StateTcLayout::BAR);        // [2]
  uint64_t* bar_mma1 = bar_full + 2;
  uint64_t* bar_mma2 = bar_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_full + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bar_full + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lid = tid & 31;
  const int quad = warp & 3, sub = warp >> 2;      // TMEM lane quadrant; which half of the slice columns
  const int row = 32 * quad + lid;                 // TMEM lane = state row kappa / D1 row
  const int H = p.H;
  const int chains = p.nseq * H;
  int item = blockIdx.x / NS;
  const int slice = blockIdx.x % NS;
  const bool trans = item >= chains;               // transition CTA: identity state, u = 0, no outputs
  if (trans) item -= chains;
  const int head = item % H, seq = item / H;
  const int v0 = slice * N;                        // first value column of the slice
  const int col0 = sub * NC;                       // this thread's first column inside the slice
  const int ucol0 = N < 64 ? (v0 & 63) : 0;        // where the slice starts inside the loaded u box
  const bool use_u = p.use_u && !trans, use_o = p.use_o && !trans;
  bf16* const h_out = trans ? nullptr : p.h_out;
  bf16* const vnew_out = trans ? nullptr : p.vnew_out;
  float* const ht = trans ? p.trans_out : p.ht;
  const int64_t bos = p.cu_seqlens[seq], eos = p.cu_seqlens[seq + 1];
  const int chunk0 = p.chunk_offsets[seq];
  int nchunks = p.chunk_offsets[seq + 1] - chunk0;
  if (bos < 0 || eos < bos || eos > p.tokens || chunk0 < 0 || (int64_t)nchunks * 64 < eos - bos) {
    // offsets that do not describe a run inside the packed buffer: the sequence is treated as empty
    if (tid == 0 && p.error) atomicExch(p.error, kOffsetsOutOfRange);
    nchunks = 0;
  }
  if (p.limit_in && !trans) nchunks = min(nchunks, p.limit_in[item]);
  const int64_t sbase = ((int64_t)seq * H + head) * D * D;

  if (warp == 0) tmem_alloc(tmem_slot, 512);
  if (tid == 0) {
    mbar_init(&bar_full[0], 1); mbar_init(&bar_full[1], 1);
    mbar_init(bar_mma1, 1);
    mbar_init(bar_mma2, use_o ? 2 : 1);            // one arrival per issuing thread
    mbar_init_fence();
    *s_abort = 0;
    tma_prefetch_desc(&p.tm_w); tma_prefetch_desc(&p.tm_qg); tma_prefetch_desc(&p.tm_kg);
    tma_prefetch_desc(&p.tm_u); tma_prefetch_desc(&p.tm_aqk);
  }
  // rows 0..63 of both A2 tiles stay zero: [0 ; Aqk] keeps the UMMA at M = 128
  for (int idx = tid; idx < 2 * 512; idx += kStateThreads) {
    int st = idx >> 9, off = (idx & 511) * 16;
    *reinterpret_cast<uint4*>(smem + st * kStageBytes + StateTcLayout::A2 + off) = make_uint4(0, 0, 0, 0);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = (uint32_t)(32 * quad) << 16;
  // state: columns 0..N-1; D1 = [w h ; qg h + Aqk v_new]: two buffers at columns 128 and 256, so the
  // output rows of chunk c leave while the products of chunk c + 1 run
  const uint32_t tDh = tmem + lane_off + col0;
  auto tD1 = [&](int c) { return tmem + 128 + 128 * (c & 1) + lane_off + col0; };

  auto chunk_valid = [&](int c) {
    int64_t rem = eos - (bos + (int64_t)c * 64);
    return rem >= 64 ? 64 : (int)rem;
  };
  auto issue_stage = [&](int c) {   // one thread
    unsigned char* st = smem + (c & 1) * kStageBytes;
    uint64_t* bar = &bar_full[c & 1];
    const int y = (int)(bos + (int64_t)c * 64);
    const int x = head * D;
    uint32_t bytes = 2 * 8192 + 2 * 8192;                       // w, kg
    if (use_u) bytes += NB * 8192;
    if (use_o) bytes += 2 * 8192 + 8192;                         // qg, Aqk
    mbar_expect_tx(bar, bytes);
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(st + StateTcLayout::A1 + b * 16384, &p.tm_w, x + 64 * b, y, bar);
      tma_load_2d(st + StateTcLayout::KG + b * 8192, &p.tm_kg, x + 64 * b, y, bar);
      if (use_o) tma_load_2d(st + StateTcLayout::A1 + b * 16384 + 8192, &p.tm_qg, x + 64 * b, y, bar);
    }
    if (use_u)
      for (int b = 0; b < NB; ++b)     // the 64-column box(es) that hold the slice
        tma_load_2d(st + StateTcLayout::U + b * 8192, &p.tm_u, x + 64 * ((v0 >> 6) + b), y, bar);
    if (use_o) tma_load_2d(st + StateTcLayout::A2 + 8192, &p.tm_aqk, head * 64, y, bar);
  };

  if (tid == 64) {      // the TMA producer: lane 0 of a warp that is off the critical v_new path
    if (nchunks > 0) issue_stage(0);
    if (nchunks > 1) issue_stage(1);
  }
  // initial state -> tensor memory (this thread owns NC columns of state row `row`)
  {
    float x[16];
#pragma unroll 1
    for (int cb = 0; cb < NC / 16; ++cb) {
      const int vcol = v0 + col0 + 16 * cb;
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (trans) {
          v4.x = row == vcol + i ? 1.f : 0.f; v4.y = row == vcol + i + 1 ? 1.f : 0.f;
          v4.z = row == vcol + i + 2 ? 1.f : 0.f; v4.w = row == vcol + i + 3 ? 1.f : 0.f;
        } else if (p.h0) {
          v4 = *reinterpret_cast<const float4*>(p.h0 + sbase + (int64_t)row * D + vcol + i);
        }
        x[i] = v4.x; x[i + 1] = v4.y; x[i + 2] = v4.z; x[i + 3] = v4.w;
      }
      tmem_st16(tDh + 16 * cb, x);
    }
    tmem_st_wait();
  }
  const uint32_t idesc_kmn = instr_desc(128, N, 0, 1);
  const uint32_t idesc_mnmn = instr_desc(128, N, 1, 1);
  const uint32_t sH = saddr(smem + StateTcLayout::H), sVN = saddr(smem + StateTcLayout::VN);
  bool failed = false;

  // Output rows of chunk c (threads of lane quadrants 2, 3 = D1 rows 64..127), NC columns each:
  // into the staging tile (a full chunk, which then leaves with a TMA store) or straight to global
  // memory (the last chunk of the sequence, which may be partial; every chunk of a narrow slice).
  auto store_o = [&](int c, bool staged) {
    const int64_t token0 = bos + (int64_t)c * 64;
    const bool live = row - 64 < chunk_valid(c);
    bf16* orow = p.o + ((token0 + (live ? row - 64 : 0)) * H + head) * D + v0 + col0;
    float x[NC];
    tmem_ld_n<NC>(tD1(c), x);
#pragma unroll
    for (int qd = 0; qd < NC / 8; ++qd) {
      uint4 v;
      pack8(x + 8 * qd, v);
      if (staged && kTileStore)
        *reinterpret_cast<uint4*>(smem + StateTcLayout::OST + tile_off(row - 64, col0 + 8 * qd, 8192)) = v;
      else if (live) *reinterpret_cast<uint4*>(orow + 8 * qd) = v;
    }
  };

  float glast = 0.f;
  if (nchunks > 0)
    glast = p.g[((bos + chunk_valid(0) - 1) * H + head) * D + row];
  int zero_from = nchunks;     // transition walk: first chunk that the (all-zero) running transition enters

  for (int c = 0; c < nchunks; ++c) {
    unsigned char* st = smem + (c & 1) * kStageBytes;
    const int64_t token0 = bos + (int64_t)c * 64;
    const int valid = chunk_valid(c);
    const float dec = exp2f(glast);
    if (c + 1 < nchunks)
      glast = p.g[((token0 + 64 + chunk_valid(c + 1) - 1) * H + head) * D + row];

    st_mark(p.prof, c, 0);
    bool nonzero = false;
    // ---- a. h row -> bf16 B tile (MN-major: rows kappa, 64-wide v boxes); decay in place
    {
      float x[NC];
      tmem_ld_n<NC>(tDh, x);
      if (trans) {
#pragma unroll
        for (int i = 0; i < NC; ++i) nonzero |= x[i] != 0.f;
      }
#pragma unroll
      for (int qd = 0; qd < NC / 8; ++qd) {
        uint4 v;
        pack8(x + 8 * qd, v);
        *reinterpret_cast<uint4*>(smem + StateTcLayout::H + tile_off(row, col0 + 8 * qd, 16384)) = v;
        if (!kTileStore && h_out)
          *reinterpret_cast<uint4*>(h_out + (((int64_t)(chunk0 + c) * H + head) * D + row) * D + v0 + col0 +
                                    8 * qd) = v;
      }
#pragma unroll
      for (int i = 0; i < NC; ++i) x[i] *= dec;
      tmem_st_n<NC>(tDh, x);
      tmem_st_wait();
    }
    st_mark(p.prof, c, 1);
    if (tid == 0) tma_store_wait_read();    // v_new / output staging of the previous chunk are free again
    fence_async_smem();
    tc_fence_before();
    int any = 1;
    if (trans) any = __syncthreads_or(nonzero); else __syncthreads();
    st_mark(p.prof, c, 2);
    if (*s_abort) { failed = true; break; }
    if (!any) {
      // the transition is exactly zero from here on; let the tile loads in flight land before leaving
      zero_from = c;
      if (!mbar_wait(&bar_full[c & 1], (c >> 1) & 1)) failed = true;
      if (c + 1 < nchunks && !mbar_wait(&bar_full[(c + 1) & 1], ((c + 1) >> 1) & 1)) failed = true;
      break;
    }

    // ---- b. D1 = [w ; qg] h ;  the bf16 state tile also leaves as h[c] (kept for the backward pass)
    // (the products first: they are on the chain from chunk to chunk, and a thread spends about
    //  50 ns on every bulk store it issues; the store only reads the tile the products read)
    if (tid == 0) {
      st_mark(p.prof, c, 10);
      if (!mbar_wait(&bar_full[c & 1], (c >> 1) & 1)) *s_abort = 1;
      tc_fence_after();
      st_mark(p.prof, c, 11);
      const uint32_t a1 = saddr(st + StateTcLayout::A1);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + 128 + 128 * (c & 1), desc_kmajor(a1, ks, 16384), desc_mnmajor(sH, ks, 16384),
             idesc_kmn, ks > 0);
      umma_commit(bar_mma1);
      if (kTileStore && h_out) {
        const int yh = ((chunk0 + c) * H + head) * D;
        for (int b = 0; b < NB; ++b)
          tma_store_2d(&p.tm_hout, smem + StateTcLayout::H + b * 16384, v0 + 64 * b, yh);
        tma_store_commit();
      }
    }
    st_mark(p.prof, c, 3);

    // ---- c. v_new = u - w h (lane quadrants 0, 1);  meanwhile quadrants 2, 3 store the output rows of
    //         the previous chunk and zero the kg rows past a partial chunk
    if (!mbar_wait(&bar_full[c & 1], (c >> 1) & 1)) *s_abort = 1;
    if (quad < 2) {
      if (!mbar_wait(bar_mma1, c & 1)) *s_abort = 1;
      tc_fence_after();
      st_mark(p.prof, c, 4);
      float x[NC];
      tmem_ld_n<NC>(tD1(c), x);
#pragma unroll
      for (int qd = 0; qd < NC / 8; ++qd) {
        const int col = col0 + 8 * qd;
        float y[8];
        if (use_u) {
          uint4 u4 = *reinterpret_cast<const uint4*>(st + StateTcLayout::U + tile_off(row, ucol0 + col, 8192));
          float2 a = unpack_bf16(u4.x), b = unpack_bf16(u4.y), cc = unpack_bf16(u4.z),
                 d = unpack_bf16(u4.w);
          y[0] = a.x; y[1] = a.y; y[2] = b.x; y[3] = b.y; y[4] = cc.x; y[5] = cc.y; y[6] = d.x; y[7] = d.y;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = row < valid ? y[i] - x[8 * qd + i] : 0.f;
        uint4 v;
        pack8(y, v);
        *reinterpret_cast<uint4*>(smem + StateTcLayout::VN + tile_off(row, col, 8192)) = v;
        // a partial chunk and a narrow slice cannot use the tile store
        if (vnew_out && (!kTileStore || valid < 64) && row < valid)
          *reinterpret_cast<uint4*>(vnew_out + ((token0 + row) * H + head) * D + v0 + col) = v;
      }
    } else {
      if (valid < 64) {
        // rows >= valid of the kg tile hold another sequence's tokens (or unwritten memory)
        for (int idx = (quad - 2) * 32 + lid + 64 * sub; idx < (64 - valid) * 16; idx += 128) {
          int r = valid + (idx >> 4), ch = idx & 15;
          *reinterpret_cast<uint4*>(st + StateTcLayout::KG + (ch >> 3) * 8192 + sw128_chunk(r, ch & 7)) =
              make_uint4(0, 0, 0, 0);
        }
      }
      if (use_o && c > 0) store_o(c - 1, true);
    }
    st_mark(p.prof, c, 5);
    if (tid == 0) tma_store_wait_read();    // the state tile is rewritten after the next barrier
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    st_mark(p.prof, c, 6);
    if (*s_abort) { failed = true; break; }

    // ---- d. h += kg^T v_new (thread 0);  D1 += [0 ; Aqk] v_new (thread 32); v_new and the previous
    //         chunk's output rows leave
    if (tid == 0) {
      tc_fence_after();
      const uint32_t kg = saddr(st + StateTcLayout::KG);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem, desc_mnmajor(kg, ks, 8192), desc_mnmajor(sVN, ks, 8192), idesc_mnmn, 1);
      umma_commit(bar_mma2);
      st_mark(p.prof, c, 7);
      const int x0 = head * D + v0;
      if (kTileStore) {
        if (vnew_out && valid == 64)
          for (int b = 0; b < NB; ++b)
            tma_store_2d(&p.tm_vnew, smem + StateTcLayout::VN + b * 8192, x0 + 64 * b, (int)token0);
        if (use_o && c > 0)
          for (int b = 0; b < NB; ++b)
            tma_store_2d(&p.tm_o, smem + StateTcLayout::OST + b * 8192, x0 + 64 * b, (int)token0 - 64);
        tma_store_commit();
      }
    } else if (tid == 32 && use_o) {
      tc_fence_after();
      const uint32_t a2 = saddr(st + StateTcLayout::A2);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem + 128 + 128 * (c & 1), desc_kmajor(a2, ks, 0), desc_mnmajor(sVN, ks, 8192), idesc_kmn, 1);
      umma_commit(bar_mma2);
    }
    if (!mbar_wait(bar_mma2, c & 1)) *s_abort = 1;
    tc_fence_after();
    st_mark(p.prof, c, 8);
    if (tid == 64 && c + 2 < nchunks) issue_stage(c + 2);
    st_mark(p.prof, c, 9);
  }
  if (!failed && use_o && nchunks > 0 && quad >= 2) store_o(nchunks - 1, false);
  if (tid == 0) tma_store_wait_read();
  if (!failed && trans && p.limit_out && tid == 0) atomicMax(p.limit_out + item, zero_from);

  if (!failed && ht) {
    float x[16];
#pragma unroll 1
    for (int cb = 0; cb < NC / 16; ++cb) {
      tmem_ld16(tDh + 16 * cb, x);
#pragma unroll
      for (int i = 0; i < 16; i += 4)
        *reinterpret_cast<float4*>(ht + sbase + (int64_t)row * D + v0 + col0 + 16 * cb + i) =
            make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    }
  }
  if (failed && tid == 0 && p.error) atomicExch(p.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

static __device__ int g_state_tc_error = 0;

template <int NS>
static int launch_state_fwd_split(const StateTcParams& p, int64_t ctas, cudaStream_t s) {
  const int smem = StateTcLayout::TOTAL + 1024;
  if (cudaFuncSetAttribute(kda_state_fwd_tc_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
      cudaSuccess)
    return KDA_ERR_LAUNCH;
  StageScope timing(kStageStateFwd, s);
  kda_state_fwd_tc_kernel<NS><<<(unsigned)(ctas * NS), kStateThreads, smem, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

// ---- host side: tensor maps --------------------------------------------------------------------
// trans_out != NULL adds a second set of CTAs that walk the same chains with u = 0 from an identity
// state and write the dense slice transition [nseq, H, 128, 128] there, in the same launch.
int launch_state_fwd_tc(const bf16* w, const bf16* u, const bf16* kg, const bf16* qg, const bf16* aqk,
                        const float* g, const float* h0, float* ht, float* trans_out,
                        const int32_t* limit_in, int32_t* limit_out, bf16* o, bf16* h_out,
                        bf16* vnew_out, const int32_t* cu, const int32_t* co, int nseq, int H,
                        int64_t tokens, int chunks, cudaStream_t s) {
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
  // tensor maps of absent results are built over `w` and never used
  if (!make_tensor_map(&p.tm_vnew, vnew_out ? vnew_out : w, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_o, o ? o : w, tokens, cols, 64))
    return KDA_ERR_LAUNCH;
  if (!make_tensor_map(&p.tm_hout, h_out ? h_out : w, h_out ? (int64_t)chunks * H * D : tokens,
                       h_out ? D : cols, 128))
    return KDA_ERR_LAUNCH;
  p.g = g; p.h0 = h0; p.ht = ht; p.trans_out = trans_out; p.limit_in = limit_in; p.limit_out = limit_out;
  p.o = o; p.h_out = h_out; p.vnew_out = vnew_out;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.error = error; p.nseq = nseq; p.H = H; p.tokens = tokens;
  p.use_u = u != nullptr; p.use_o = o != nullptr;
  p.prof = debug_profile_buffer();
  const int64_t ctas = (int64_t)nseq * H * (trans_out ? 2 : 1);
  switch (pick_value_split(ctas)) {
    case 4: return launch_state_fwd_split<4>(p, ctas, s);
    case 2: return launch_state_fwd_split<2>(p, ctas, s);
    default: return launch_state_fwd_split<1>(p, ctas, s);
  }
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
  CUtensorMap tm_dhout, tm_dv2out;          // result tiles leave shared memory with TMA stores
  const float* g; const float* dht; float* dh0;
  bf16* dh_out; bf16* dv2_out;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int* error;
  int nseq, H;
  int64_t tokens;            // rows of the packed buffers
};

constexpr int kBStageBytes = 4 * 16384 + 8192;   // KG, W, QG, DO, AQK
struct StateBwdLayout {
  static constexpr int KG = 0, W = 16384, QG = 32768, DO = 49152, AQK = 65536;
  static constexpr int DH = 2 * kBStageBytes;            // 147456
  static constexpr int DV2 = DH + 32768;                 // 180224
  static constexpr int BAR = DV2 + 16384;                // 196608
  static constexpr int TOTAL = BAR + 1024;
};

// NS CTAs share a chain, each owning N = 128 / NS value columns of dh, dO and dv2 (see the forward kernel).
template <int NS>
__global__ void __launch_bounds__(kStateThreads) kda_state_bwd_tc_kernel(const __grid_constant__ StateBwdTcParams p) {
  constexpr int N = D / NS;
  constexpr int NC = N / 2;
  constexpr int NB = (N + 63) / 64;
  constexpr bool kTileStore = N >= 64;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = smem_dyn + ((1024u - (saddr(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + StateBwdLayout::BAR);
  uint64_t* bar_mma1 = bar_full + 2;
  uint64_t* bar_mma2 = bar_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_full + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bar_full + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lid = tid & 31;
  const int quad = warp & 3, sub = warp >> 2;      // TMEM lane quadrant; which half of the slice columns
  const int row = 32 * quad + lid;                 // TMEM lane = state row kappa
  const int H = p.H;
  const int item = blockIdx.x / NS, slice = blockIdx.x % NS;
  const int head = item % H, seq = item / H;
  const int v0 = slice * N, col0 = sub * NC;
  const int dcol0 = N < 64 ? (v0 & 63) : 0;        // where the slice starts inside the loaded dO box
  const int64_t bos = p.cu_seqlens[seq], eos = p.cu_seqlens[seq + 1];
  const int chunk0 = p.chunk_offsets[seq];
  int nchunks = p.chunk_offsets[seq + 1] - chunk0;
  if (bos < 0 || eos < bos || eos > p.tokens || chunk0 < 0 || (int64_t)nchunks * 64 < eos - bos) {
    if (tid == 0 && p.error) atomicExch(p.error, kOffsetsOutOfRange);     // treated as an empty sequence
    nchunks = 0;
  }
  const int64_t sbase = ((int64_t)seq * H + head) * D * D;

  if (warp == 0) tmem_alloc(tmem_slot, 256);
  if (tid == 0) {
    mbar_init(&bar_full[0], 1); mbar_init(&bar_full[1], 1);
    mbar_init(bar_mma1, 2); mbar_init(bar_mma2, 1);      // one arrival per issuing thread
    mbar_init_fence();
    *s_abort = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = (uint32_t)(32 * quad) << 16;
  const uint32_t tDh = tmem + lane_off + col0, tDv = tmem + 128 + lane_off + col0;

  auto chunk_valid = [&](int c) {
    int64_t rem = eos - (bos + (int64_t)c * 64);
    return rem >= 64 ? 64 : (int)rem;
  };
  auto issue_stage = [&](int it) {   // one thread; iteration `it` handles chunk nchunks-1-it
    const int c = nchunks - 1 - it;
    unsigned char* st = smem + (it & 1) * kBStageBytes;
    uint64_t* bar = &bar_full[it & 1];
    const int y = (int)(bos + (int64_t)c * 64);
    const int x = head * D;
    mbar_expect_tx(bar, 3 * 16384 + NB * 8192 + 8192);
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(st + StateBwdLayout::KG + b * 8192, &p.tm_kg, x + 64 * b, y, bar);
      tma_load_2d(st + StateBwdLayout::W + b * 8192, &p.tm_w, x + 64 * b, y, bar);
      tma_load_2d(st + StateBwdLayout::QG + b * 8192, &p.tm_qg, x + 64 * b, y, bar);
    }
    for (int b = 0; b < NB; ++b)     // the 64-column box(es) of dO that hold the slice
      tma_load_2d(st + StateBwdLayout::DO + b * 8192, &p.tm_do, x + 64 * ((v0 >> 6) + b), y, bar);
    tma_load_2d(st + StateBwdLayout::AQK, &p.tm_aqk, head * 64, y, bar);
  };
  if (tid == 64) {      // the TMA producer: lane 0 of a warp of its own
    if (nchunks > 0) issue_stage(0);
    if (nchunks > 1) issue_stage(1);
  }
  {
    float x[16];
#pragma unroll 1
    for (int cb = 0; cb < NC / 16; ++cb) {
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.dht)
          v4 = *reinterpret_cast<const float4*>(p.dht + sbase + (int64_t)row * D + v0 + col0 + 16 * cb + i);
        x[i] = v4.x; x[i + 1] = v4.y; x[i + 2] = v4.z; x[i + 3] = v4.w;
      }
      tmem_st16(tDh + 16 * cb, x);
    }
    tmem_st_wait();
  }
  const uint32_t sDH = saddr(smem + StateBwdLayout::DH), sDV2 = saddr(smem + StateBwdLayout::DV2);
  bool failed = false;

  float glast = 0.f;
  if (nchunks > 0)
    glast = p.g[((bos + (int64_t)(nchunks - 1) * 64 + chunk_valid(nchunks - 1) - 1) * H + head) * D + row];

  for (int it = 0; it < nchunks; ++it) {
    const int c = nchunks - 1 - it;
    unsigned char* st = smem + (it & 1) * kBStageBytes;
    const int64_t token0 = bos + (int64_t)c * 64;
    const int valid = chunk_valid(c);
    const float dec = exp2f(glast);
    if (c > 0) glast = p.g[((token0 - 1) * H + head) * D + row];   // last row of the previous chunk

    if (!mbar_wait(&bar_full[it & 1], (it >> 1) & 1)) *s_abort = 1;
    if (valid < 64) {
      // rows past the tail hold another sequence's tokens or unwritten memory: they are contraction
      // rows of w, qg, dO and Aqk
      for (int idx = tid; idx < (64 - valid) * 16; idx += kStateThreads) {
        const int r = valid + (idx >> 4), ch = idx & 15;
        const int off = (ch >> 3) * 8192 + sw128_chunk(r, ch & 7);
        *reinterpret_cast<uint4*>(st + StateBwdLayout::W + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(st + StateBwdLayout::QG + off) = make_uint4(0, 0, 0, 0);
        if (ch < 8 * NB)
          *reinterpret_cast<uint4*>(st + StateBwdLayout::DO + off) = make_uint4(0, 0, 0, 0);
        if (ch < 8)
          *reinterpret_cast<uint4*>(st + StateBwdLayout::AQK + sw128_chunk(r, ch)) = make_uint4(0, 0, 0, 0);
      }
    }
    // ---- a. dh row -> bf16 B tile; decay in place ------------------------------------------------
    {
      float x[NC];
      tmem_ld_n<NC>(tDh, x);
#pragma unroll
      for (int qd = 0; qd < NC / 8; ++qd) {
        uint4 v;
        pack8(x + 8 * qd, v);
        *reinterpret_cast<uint4*>(smem + StateBwdLayout::DH + tile_off(row, col0 + 8 * qd, 16384)) = v;
        if (!kTileStore)     // a narrow slice cannot use the tile store
          *reinterpret_cast<uint4*>(p.dh_out + (((int64_t)(chunk0 + c) * H + head) * D + row) * D + v0 +
                                    col0 + 8 * qd) = v;
      }
#pragma unroll
      for (int i = 0; i < NC; ++i) x[i] *= dec;
      tmem_st_n<NC>(tDh, x);
      tmem_st_wait();
    }
    if (tid == 0) tma_store_wait_read();    // the dv2 tile of the previous step is free again
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) { failed = true; break; }

    // ---- b. dv2 = kg dh + Aqk^T dO ;  dh += qg^T dO ;  the bf16 dh tile leaves as dh[c] ------------------
    // (the slice's dO columns start dcol0 columns into the loaded box: the operand descriptor starts there)
    // (products before the bulk stores, as in the forward walk)
    if (tid == 0) {
      tc_fence_after();
      const uint32_t kg = saddr(st + StateBwdLayout::KG), dO = saddr(st + StateBwdLayout::DO) + 2 * dcol0,
                     aqk = saddr(st + StateBwdLayout::AQK);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma(tmem + 128, desc_kmajor(kg, ks, 8192), desc_mnmajor(sDH, ks, 16384),
             instr_desc(64, N, 0, 1), ks > 0);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem + 128, desc_mnmajor(aqk, ks, 0), desc_mnmajor(dO, ks, 8192), instr_desc(64, N, 1, 1), 1);
      umma_commit(bar_mma1);
      if (kTileStore) {
        const int yh = ((chunk0 + c) * H + head) * D;
        for (int b = 0; b < NB; ++b)
          tma_store_2d(&p.tm_dhout, smem + StateBwdLayout::DH + b * 16384, v0 + 64 * b, yh);
        tma_store_commit();
      }
    } else if (tid == 32) {
      tc_fence_after();
      const uint32_t qg = saddr(st + StateBwdLayout::QG), dO = saddr(st + StateBwdLayout::DO) + 2 * dcol0;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem, desc_mnmajor(qg, ks, 8192), desc_mnmajor(dO, ks, 8192), instr_desc(128, N, 1, 1), 1);
      umma_commit(bar_mma1);
    }
    if (!mbar_wait(bar_mma1, it & 1)) *s_abort = 1;
    tc_fence_after();
    // ---- c. dv2 rows (M = 64 accumulator: row j on lane 32 (j / 16) + j % 16) -----------------------
    {
      float x[NC];
      const int j = quad * 16 + lid;
      tmem_ld_n<NC>(tDv, x);
      if (lid < 16) {
#pragma unroll
        for (int qd = 0; qd < NC / 8; ++qd) {
          const int col = col0 + 8 * qd;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (j < valid) pack8(x + 8 * qd, v);
          *reinterpret_cast<uint4*>(smem + StateBwdLayout::DV2 + tile_off(j, col, 8192)) = v;
          if ((!kTileStore || valid < 64) && j < valid)   // a partial chunk / narrow slice cannot use the tile store
            *reinterpret_cast<uint4*>(p.dv2_out + ((token0 + j) * H + head) * D + v0 + col) = v;
        }
      }
    }
    if (tid == 0) tma_store_wait_read();    // the dh tile is rewritten after the next barrier
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) { failed = true; break; }

    // ---- d. dh -= w^T dv2 ;  dv2 leaves -----------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      const uint32_t w = saddr(st + StateBwdLayout::W);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma(tmem, desc_mnmajor(w, ks, 8192), desc_mnmajor(sDV2, ks, 8192), instr_desc(128, N, 1, 1, 1), 1);
      umma_commit(bar_mma2);
      if (kTileStore && valid == 64) {
        for (int b = 0; b < NB; ++b)
          tma_store_2d(&p.tm_dv2out, smem + StateBwdLayout::DV2 + b * 8192, head * D + v0 + 64 * b, (int)token0);
        tma_store_commit();
      }
    }
    if (!mbar_wait(bar_mma2, it & 1)) *s_abort = 1;
    tc_fence_after();
    if (tid == 64 && it + 2 < nchunks) issue_stage(it + 2);
  }
  if (tid == 0) tma_store_wait_read();

  if (!failed && p.dh0) {
    float x[16];
#pragma unroll 1
    for (int cb = 0; cb < NC / 16; ++cb) {
      tmem_ld16(tDh + 16 * cb, x);
#pragma unroll
      for (int i = 0; i < 16; i += 4)
        *reinterpret_cast<float4*>(p.dh0 + sbase + (int64_t)row * D + v0 + col0 + 16 * cb + i) =
            make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    }
  }
  if (failed && tid == 0 && p.error) atomicExch(p.error, 16);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

template <int NS>
static int launch_state_bwd_split(const StateBwdTcParams& p, int64_t chains, cudaStream_t s) {
  const int smem = StateBwdLayout::TOTAL + 1024;
  if (cudaFuncSetAttribute(kda_state_bwd_tc_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
      cudaSuccess)
    return KDA_ERR_LAUNCH;
  StageScope timing(kStageStateBwd, s);
  kda_state_bwd_tc_kernel<NS><<<(unsigned)(chains * NS), kStateThreads, smem, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

int launch_state_bwd_tc(const bf16* w, const bf16* kg, const bf16* qg, const bf16* aqk, const bf16* dout,
                        const float* g, const float* dht, float* dh0, bf16* dh_out, bf16* dv2_out,
                        const int32_t* cu, const int32_t* co, int nseq, int H, int64_t tokens,
                        int chunks, cudaStream_t s) {
  if (nseq == 0) return KDA_OK;
  StateBwdTcParams p;
  const int64_t cols = (int64_t)H * D;
  if (!make_tensor_map(&p.tm_w, w, tokens, cols, 64) || !make_tensor_map(&p.tm_kg, kg, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_qg, qg, tokens, cols, 64) || !make_tensor_map(&p.tm_do, dout, tokens, cols, 64) ||
      !make_tensor_map(&p.tm_aqk, aqk, tokens, (int64_t)H * 64, 64) ||
      !make_tensor_map(&p.tm_dhout, dh_out, (int64_t)chunks * H * D, D, 128) ||
      !make_tensor_map(&p.tm_dv2out, dv2_out, tokens, cols, 64))
    return KDA_ERR_LAUNCH;
  p.g = g; p.dht = dht; p.dh0 = dh0; p.dh_out = dh_out; p.dv2_out = dv2_out;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.nseq = nseq; p.H = H; p.tokens = tokens;
  p.error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p.error), g_state_tc_error) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  const int64_t chains = (int64_t)nseq * H;
  switch (pick_value_split(chains)) {
    case 4: return launch_state_bwd_split<4>(p, chains, s);
    case 2: return launch_state_bwd_split<2>(p, chains, s);
    default: return launch_state_bwd_split<1>(p, chains, s);
  }
}

}  // namespace kda

// Self-test of the bounded waits: one warp waits, with a small poll limit, on a barrier that nothing
// ever arrives on.  The wait must run out, raise the error word (code 2) and let the kernel return
// normally, leaving the context usable.  Nothing faults, traps or spins without bound.
namespace kda {
__global__ void bounded_wait_selftest_kernel(int* error, int limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    sm100::mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !sm100::mbar_wait(&bar, 0, limit)) atomicExch(error, 2);
}
}  // namespace kda

extern "C" int kda_selftest_bounded_wait(int poll_limit, void* stream) {
  if (poll_limit < 1 || poll_limit > (1 << 20)) return KDA_ERR_ARG;
  int* error = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&error), kda::g_state_tc_error) != cudaSuccess)
    return KDA_ERR_LAUNCH;
  kda::bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(error, poll_limit);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

// 1 if a tensor-memory kernel gave up on a barrier wait since the last call (clears the flag).
// Synchronises the device; meant for tests and debugging.
namespace kda { int bwd_chunk_tc_error_word(); int prepare_tc_error_word(); int gate_error_word(); }

extern "C" int kda_device_error_word(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, kda::g_state_tc_error, sizeof(int)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(kda::g_state_tc_error, &zero, sizeof(int));
  return v | (kda::bwd_chunk_tc_error_word() << 8) | (kda::prepare_tc_error_word() << 16) |
         (kda::gate_error_word() << 24);
}

// Forces the value split of the state recurrences (1, 2 or 4 CTAs per chain; 0 = choose from the
// number of chains and SMs).  Every split gives the same bits; tests and tuning use this.
extern "C" int kda_set_state_value_split(int split) {
  if (split != 0 && split != 1 && split != 2 && split != 4) return KDA_ERR_ARG;
  kda::g_value_split = split;
  return KDA_OK;
}
