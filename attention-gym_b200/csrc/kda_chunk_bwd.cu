// Chunked KDA backward for K = V = 128, chunk = 64 (bf16 operands, fp32 accumulation).
//
// Stages (reference orchestration: attn_gym/linear/kda/bwd/cute/chunk_kda_bwd.py:21-147):
//   wu            recompute w, u, kg, qg from the stored A           (kda_chunk_fwd.cu)
//   state_fwd     recompute the chunk-entry states h[c] and v_new     (kda_chunk_fwd.cu)
//   state_bwd     reverse chunk loop, fp32 dh in registers:
//                 dv2 = kg dh + Aqk^T do ;  dh <- diag(2^{G_last}) dh + qg^T do - w^T dv2
//                 (reference: bwd/triton/chunk_kda_bwd_dav.py:73-93 fused with
//                  bwd/cute/chunk_delta_h_bwd_v1.py:1147-1276)
//   wy            per (chunk, head): dq/dk/dG partials, dv, dbeta partial, dAqk, dL
//                 (reference: bwd/cute/chunk_kda_bwd_wy_dqkg_fused.py:2623; oracle
//                  attn_gym/testing/kda.py:144-240)
//   intra         per (chunk, head): gradients through the gated pairwise products
//                 (reference: bwd/cute/chunk_kda_bwd_intra.py:931; oracle attn_gym/testing/kda.py:67-141)
//
// dG is the gradient with respect to the cumulative log2 gate and is multiplied by ln 2 once,
// in the last stage.
#include "kda_common.cuh"
#include "kda_timing.cuh"
#include <cstdlib>

namespace kda {

constexpr int D = 128;
constexpr int LDD = 136;
constexpr int LD64 = 72;

struct BwdParams {
  const bf16* q; const bf16* k; const bf16* v; const float* g; const float* beta;
  const bf16* aqk; const bf16* akk;
  const bf16* w; const bf16* kg; const bf16* qg;      // recomputed
  const bf16* h; const bf16* vnew;                    // recomputed [chunks,H,128,128], [N,H,128]
  const bf16* dout;                                   // [N,H,128]
  const float* dht; float* dh0;
  bf16* dh; bf16* dv2;                                // state_bwd outputs
  float* daqk; float* dl;                             // [N,H,64] fp32
  float* dq_p; float* dk_p; float* dg_p; float* db_p; // wy partials
  bf16* dq; bf16* dk; bf16* dv; float* dg; float* db; // final outputs
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int nseq, H;
  float scale;
  long long* prof;   // optional per-phase timestamps (debugging aid), null in normal use
};

__device__ __forceinline__ void prof_mark(const BwdParams& p, int slot) {
  if (p.prof && threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.x < 64) {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.prof[blockIdx.x * 32 + slot] = t;
  }
}

// ------------------------------------------------------------------------------------------
// state_bwd
// ------------------------------------------------------------------------------------------
struct BStage {
  bf16 w[64 * LDD];
  bf16 qg[64 * LDD];
  bf16 kg[64 * LDD];
  bf16 dO[64 * LD64];
  bf16 aqk[64 * LD64];
  float dec[D];
};
struct BStateSmem {
  BStage st[2];
  bf16 dh[D * LD64];
  bf16 dv2[64 * LD64];
};

__device__ __forceinline__ void bstate_load_stage(BStage& s, const BwdParams& p, int64_t token0,
                                                  int valid, int head, int vh, int tid) {
  const int H = p.H;
  const int64_t rowD = (token0 * H + head) * D;
  const int64_t gld = (int64_t)H * D;
  load_tile_b16<64, D, LDD, 256>(s.w, p.w + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, 256>(s.qg, p.qg + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, 256>(s.kg, p.kg + rowD, gld, valid, tid);
  load_tile_b16<64, 64, LD64, 256>(s.dO, p.dout + rowD + 64 * vh, gld, valid, tid);
  load_tile_b16<64, 64, LD64, 256>(s.aqk, p.aqk + (token0 * H + head) * 64, (int64_t)H * 64, valid,
                                   tid);
  if (tid < D / 4)
    cp_async16(s.dec + tid * 4, p.g + rowD + (int64_t)(valid - 1) * gld + tid * 4, true);
}

__global__ void __launch_bounds__(256) kda_state_bwd_kernel(const BwdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  BStateSmem& sm = *reinterpret_cast<BStateSmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = p.H;
  const int vh = blockIdx.x & 1;
  const int head = (blockIdx.x >> 1) % H;
  const int seq = (blockIdx.x >> 1) / H;
  const int64_t bos = p.cu_seqlens[seq], eos = p.cu_seqlens[seq + 1];
  const int chunk0 = p.chunk_offsets[seq];
  const int nchunks = p.chunk_offsets[seq + 1] - chunk0;
  const int g8 = lane >> 2, t2 = 2 * (lane & 3);

  float dh[1][8][4];
  const int64_t sbase = ((int64_t)seq * H + head) * D * D + 64 * vh;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * warp + g8 + 8 * hh, c = 8 * nt + t2;
      float2 x = make_float2(0.f, 0.f);
      if (p.dht) x = *reinterpret_cast<const float2*>(p.dht + sbase + (int64_t)r * D + c);
      dh[0][nt][2 * hh] = x.x;
      dh[0][nt][2 * hh + 1] = x.y;
    }
  auto chunk_valid = [&](int c) {
    int64_t rem = eos - (bos + (int64_t)c * 64);
    return rem >= 64 ? 64 : (int)rem;
  };
  if (nchunks > 0)
    bstate_load_stage(sm.st[0], p, bos + (int64_t)(nchunks - 1) * 64, chunk_valid(nchunks - 1),
                      head, vh, tid);
  cp_async_commit();
  if (nchunks > 1)
    bstate_load_stage(sm.st[1], p, bos + (int64_t)(nchunks - 2) * 64, chunk_valid(nchunks - 2),
                      head, vh, tid);
  cp_async_commit();

  const int mt = warp & 3, nq = warp >> 2;
  for (int it = 0; it < nchunks; ++it) {
    const int c = nchunks - 1 - it;
    BStage& st = sm.st[it & 1];
    const int64_t token0 = bos + (int64_t)c * 64;
    const int valid = chunk_valid(c);
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *reinterpret_cast<uint32_t*>(&sm.dh[(16 * warp + g8 + 8 * hh) * LD64 + 8 * nt + t2]) =
            pack_bf16(dh[0][nt][2 * hh], dh[0][nt][2 * hh + 1]);
    __syncthreads();
    store_tile_b16<D, 64, LD64, 256>(
        p.dh + (((int64_t)(chunk0 + c) * H + head) * D) * D + 64 * vh, D, sm.dh, D, tid);

    float acc[1][4][4];
    zero_acc<1, 4>(acc);
    warp_gemm<1, 2, false, true>(acc, st.kg, LDD, 16 * mt, 0, sm.dh, LD64, 0, 32 * nq, 8, lane);
    warp_gemm<1, 2, true, true>(acc, st.aqk, LD64, 16 * mt, 0, st.dO, LD64, 0, 32 * nq, 4, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = 16 * mt + g8 + 8 * hh, cc = 32 * nq + 8 * nt + t2;
        *reinterpret_cast<uint32_t*>(&sm.dv2[r * LD64 + cc]) =
            pack_bf16(acc[0][nt][2 * hh], acc[0][nt][2 * hh + 1]);
      }
    __syncthreads();
    store_tile_b16<64, 64, LD64, 256>(p.dv2 + (token0 * H + head) * D + 64 * vh, (int64_t)H * D,
                                      sm.dv2, valid, tid);
    {
      float d0 = fexp2(st.dec[16 * warp + g8]), d1 = fexp2(st.dec[16 * warp + g8 + 8]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        dh[0][nt][0] *= d0; dh[0][nt][1] *= d0; dh[0][nt][2] *= d1; dh[0][nt][3] *= d1;
      }
    }
    warp_gemm<1, 4, true, true>(dh, st.qg, LDD, 16 * warp, 0, st.dO, LD64, 0, 0, 4, lane);
    warp_gemm<1, 4, true, true, true>(dh, st.w, LDD, 16 * warp, 0, sm.dv2, LD64, 0, 0, 4, lane);
    __syncthreads();
    if (it + 2 < nchunks)
      bstate_load_stage(st, p, token0 - 128, chunk_valid(c - 2), head, vh, tid);
    cp_async_commit();
  }
  cp_async_wait<0>();
  if (p.dh0) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = 16 * warp + g8 + 8 * hh, c = 8 * nt + t2;
        *reinterpret_cast<float2*>(p.dh0 + sbase + (int64_t)r * D + c) =
            make_float2(dh[0][nt][2 * hh], dh[0][nt][2 * hh + 1]);
      }
  }
}

// ------------------------------------------------------------------------------------------
// wy
// ------------------------------------------------------------------------------------------
struct WySmem {
  bf16 hh[D * LDD];    // h[kappa][v]; later dw [64][LDD]
  bf16 dh[D * LDD];    // dh[kappa][v]; later X, Y [64][LD64] each
  bf16 dO[64 * LDD];
  bf16 vn[64 * LDD];
  bf16 dv2[64 * LDD];
  bf16 v[64 * LDD];
  bf16 k[64 * LDD];    // raw k, then k 2^G in place
  float g[64 * D];
  bf16 a[64 * LD64];
  float beta[64];
  float db[64];
  float hd[D];         // sum_v h dh
  float kdk[D];        // sum_t k dk_s
};

template <int NW>
__global__ void __launch_bounds__(32 * NW) kda_bwd_wy_kernel(const BwdParams p) {
  constexpr int THREADS = 32 * NW;
  constexpr int NH = NW / 4;        // column groups of the warp grid (4 row tiles x NH)
  constexpr int CW = D / NH;        // columns per warp in the [64 x 128] products
  constexpr int NTN = CW / 8;
  constexpr int CQ = 64 / NH;       // columns per warp in the [64 x 64] products
  constexpr int NTQ = CQ / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  WySmem& sm = *reinterpret_cast<WySmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.y, H = p.H;
  const ChunkWork cw = locate_chunk(p.cu_seqlens, p.chunk_offsets, p.nseq, blockIdx.x);
  if (cw.valid == 0) return;
  const int valid = cw.valid;
  const int64_t rowD = (cw.token0 * H + head) * D;
  const int64_t gld = (int64_t)H * D;
  const int64_t row64 = (cw.token0 * H + head) * 64;
  const int64_t gld64 = (int64_t)H * 64;
  const int64_t hbase = (((int64_t)blockIdx.x * H + head) * D) * D;
  const int g8 = lane >> 2, t2 = 2 * (lane & 3);

  prof_mark(p, 0);
  load_tile_b16<D, D, LDD, THREADS>(sm.hh, p.h + hbase, D, D, tid);
  load_tile_b16<D, D, LDD, THREADS>(sm.dh, p.dh + hbase, D, D, tid);
  load_tile_b16<64, D, LDD, THREADS>(sm.dO, p.dout + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, THREADS>(sm.vn, p.vnew + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, THREADS>(sm.dv2, p.dv2 + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, THREADS>(sm.v, p.v + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, THREADS>(sm.k, p.k + rowD, gld, valid, tid);
  load_tile_f32<64, D, D, THREADS>(sm.g, p.g + rowD, gld, valid, tid);
  load_tile_b16<64, 64, LD64, THREADS>(sm.a, p.akk + row64, gld64, valid, tid);
  cp_async_commit();
  if (tid < 64) {
    sm.beta[tid] = tid < valid ? p.beta[(cw.token0 + tid) * H + head] : 0.f;
    sm.db[tid] = 0.f;
  }
  if (tid < D) sm.kdk[tid] = 0.f;
  cp_async_wait<0>();
  __syncthreads();
  prof_mark(p, 1);

  // this thread's q and raw-k elements of its (mt, nh) accumulator tile, fetched before any global
  // store so the loads overlap instead of serialising behind possibly-aliasing stores
  uint32_t qreg[NTN][2], kreg[NTN][2];
  {
    const int mt_ = warp & 3, nh_ = warp >> 2;
#pragma unroll
    for (int nt = 0; nt < NTN; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = 16 * mt_ + g8 + 8 * hh, c = CW * nh_ + 8 * nt + t2;
        qreg[nt][hh] = r < valid
            ? *reinterpret_cast<const uint32_t*>(p.q + rowD + (int64_t)r * gld + c) : 0u;
        kreg[nt][hh] = *reinterpret_cast<uint32_t*>(&sm.k[r * LDD + c]);
      }
  }
  __syncthreads();  // raw k captured by every thread before it is gated in place
  // hd[kappa] = sum_v h dh ; k <- k 2^G
  for (int r = warp; r < D; r += NW) {
    float s = 0.f;
    for (int c = lane * 4; c < D; c += 128) {
      float2 a0 = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.hh[r * LDD + c]));
      float2 a1 = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.hh[r * LDD + c + 2]));
      float2 b0 = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.dh[r * LDD + c]));
      float2 b1 = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.dh[r * LDD + c + 2]));
      s += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    if (lane == 0) sm.hd[r] = s;
  }
  for (int idx = tid; idx < 64 * (D / 2); idx += THREADS) {
    int r = idx / (D / 2), c = (idx % (D / 2)) * 2;
    float2 kv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.k[r * LDD + c]));
    *reinterpret_cast<uint32_t*>(&sm.k[r * LDD + c]) =
        pack_bf16(kv.x * fexp2(sm.g[r * D + c]), kv.y * fexp2(sm.g[r * D + c + 1]));
  }
  __syncthreads();

  prof_mark(p, 2);
  const float* glast = sm.g + (valid - 1) * D;
  const int mt = warp & 3, nh = warp >> 2;
  float dgacc[NTN][4], dkacc[NTN][4];
  float acc[1][NTN][4];

  // ---- dq_inter = scale 2^G (do h^T) ---------------------------------------------------------
  zero_acc<1, NTN>(acc);
  warp_gemm<1, NTN / 2, false, false>(acc, sm.dO, LDD, 16 * mt, 0, sm.hh, LDD, 0, CW * nh, 8, lane);
#pragma unroll
  for (int nt = 0; nt < NTN; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + g8 + 8 * hh, c = CW * nh + 8 * nt + t2;
      float x0 = acc[0][nt][2 * hh] * p.scale * fexp2(sm.g[r * D + c]);
      float x1 = acc[0][nt][2 * hh + 1] * p.scale * fexp2(sm.g[r * D + c + 1]);
      float2 qv = unpack_bf16(qreg[nt][hh]);
      if (r < valid) {
        int64_t gi = rowD + (int64_t)r * gld + c;
        *reinterpret_cast<float2*>(p.dq_p + gi) = make_float2(x0, x1);
      }
      dgacc[nt][2 * hh] = qv.x * x0;
      dgacc[nt][2 * hh + 1] = qv.y * x1;
    }
  prof_mark(p, 3);
  // ---- dk_s = (v_new dh^T) 2^{G_last - G} -----------------------------------------------------
  zero_acc<1, NTN>(acc);
  warp_gemm<1, NTN / 2, false, false>(acc, sm.vn, LDD, 16 * mt, 0, sm.dh, LDD, 0, CW * nh, 8, lane);
#pragma unroll
  for (int nt = 0; nt < NTN; ++nt) {
    float cs0 = 0.f, cs1 = 0.f;
    int c = CW * nh + 8 * nt + t2;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + g8 + 8 * hh;
      float x0 = acc[0][nt][2 * hh] * fexp2(glast[c] - sm.g[r * D + c]);
      float x1 = acc[0][nt][2 * hh + 1] * fexp2(glast[c + 1] - sm.g[r * D + c + 1]);
      float2 kv = unpack_bf16(kreg[nt][hh]);
      dkacc[nt][2 * hh] = x0;
      dkacc[nt][2 * hh + 1] = x1;
      dgacc[nt][2 * hh] -= kv.x * x0;
      dgacc[nt][2 * hh + 1] -= kv.y * x1;
      cs0 += kv.x * x0;
      cs1 += kv.y * x1;
    }
#pragma unroll
    for (int d = 4; d < 32; d <<= 1) {
      cs0 += __shfl_xor_sync(0xffffffffu, cs0, d);
      cs1 += __shfl_xor_sync(0xffffffffu, cs1, d);
    }
    if (g8 == 0) {
      atomicAdd(&sm.kdk[c], cs0);
      atomicAdd(&sm.kdk[c + 1], cs1);
    }
  }
  prof_mark(p, 4);
  // ---- dw = -(dv2 h^T) ------------------------------------------------------------------------
  zero_acc<1, NTN>(acc);
  warp_gemm<1, NTN / 2, false, false>(acc, sm.dv2, LDD, 16 * mt, 0, sm.hh, LDD, 0, CW * nh, 8, lane);
  __syncthreads();  // every warp is done with h and dh
  bf16* s_dw = sm.hh;
  bf16* s_x = sm.dh;
  bf16* s_y = sm.dh + 64 * LD64;
#pragma unroll
  for (int nt = 0; nt < NTN; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + g8 + 8 * hh, c = CW * nh + 8 * nt + t2;
      *reinterpret_cast<uint32_t*>(&s_dw[r * LDD + c]) =
          pack_bf16(-acc[0][nt][2 * hh], -acc[0][nt][2 * hh + 1]);
    }
  __syncthreads();

  prof_mark(p, 5);
  // ---- dvb = A^T dv2 ; dv = beta dvb ; dbeta += <dvb, v> --------------------------------------
  zero_acc<1, NTN>(acc);
  warp_gemm<1, NTN / 2, true, true>(acc, sm.a, LD64, 16 * mt, 0, sm.dv2, LDD, 0, CW * nh, 4, lane);
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    int r = 16 * mt + g8 + 8 * hh;
    float b = sm.beta[r], dbp = 0.f;
#pragma unroll
    for (int nt = 0; nt < NTN; ++nt) {
      int c = CW * nh + 8 * nt + t2;
      float x0 = acc[0][nt][2 * hh], x1 = acc[0][nt][2 * hh + 1];
      float2 vv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.v[r * LDD + c]));
      dbp += x0 * vv.x + x1 * vv.y;
      if (r < valid)
        *reinterpret_cast<uint32_t*>(p.dv + rowD + (int64_t)r * gld + c) = pack_bf16(x0 * b, x1 * b);
    }
    dbp += __shfl_xor_sync(0xffffffffu, dbp, 1);
    dbp += __shfl_xor_sync(0xffffffffu, dbp, 2);
    if ((lane & 3) == 0) atomicAdd(&sm.db[r], dbp);
  }
  prof_mark(p, 6);
  // ---- dkgb = A^T dw ; dk += beta 2^G dkgb ; dG += beta k 2^G dkgb ; dbeta += <dkgb, k 2^G> ----
  zero_acc<1, NTN>(acc);
  warp_gemm<1, NTN / 2, true, true>(acc, sm.a, LD64, 16 * mt, 0, s_dw, LDD, 0, CW * nh, 4, lane);
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    int r = 16 * mt + g8 + 8 * hh;
    float b = sm.beta[r], dbp = 0.f;
#pragma unroll
    for (int nt = 0; nt < NTN; ++nt) {
      int c = CW * nh + 8 * nt + t2;
      float x0 = acc[0][nt][2 * hh], x1 = acc[0][nt][2 * hh + 1];
      float2 kgm = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.k[r * LDD + c]));  // k 2^G
      dbp += x0 * kgm.x + x1 * kgm.y;
      float dk0 = dkacc[nt][2 * hh] + b * fexp2(sm.g[r * D + c]) * x0;
      float dk1 = dkacc[nt][2 * hh + 1] + b * fexp2(sm.g[r * D + c + 1]) * x1;
      float dg0 = dgacc[nt][2 * hh] + b * kgm.x * x0;
      float dg1 = dgacc[nt][2 * hh + 1] + b * kgm.y * x1;
      if (r == valid - 1) {
        dg0 += sm.hd[c] * fexp2(glast[c]) + sm.kdk[c];
        dg1 += sm.hd[c + 1] * fexp2(glast[c + 1]) + sm.kdk[c + 1];
      }
      if (r < valid) {
        int64_t gi = rowD + (int64_t)r * gld + c;
        *reinterpret_cast<float2*>(p.dk_p + gi) = make_float2(dk0, dk1);
        *reinterpret_cast<float2*>(p.dg_p + gi) = make_float2(dg0, dg1);
      }
    }
    dbp += __shfl_xor_sync(0xffffffffu, dbp, 1);
    dbp += __shfl_xor_sync(0xffffffffu, dbp, 2);
    if ((lane & 3) == 0) atomicAdd(&sm.db[r], dbp);
  }

  prof_mark(p, 7);
  // ---- X = stril(dv2 v^T + dw (k 2^G)^T) diag(beta) -------------------------------------------
  const int nq = warp >> 2;
  float acs[1][NTQ][4];
  zero_acc<1, NTQ>(acs);
  warp_gemm<1, NTQ / 2, false, false>(acs, sm.dv2, LDD, 16 * mt, 0, sm.v, LDD, 0, CQ * nq, 8, lane);
  warp_gemm<1, NTQ / 2, false, false>(acs, s_dw, LDD, 16 * mt, 0, sm.k, LDD, 0, CQ * nq, 8, lane);
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + g8 + 8 * hh, c = CQ * nq + 8 * nt + t2;
      float x0 = (r > c) ? acs[0][nt][2 * hh] * sm.beta[c] : 0.f;
      float x1 = (r > c + 1) ? acs[0][nt][2 * hh + 1] * sm.beta[c + 1] : 0.f;
      *reinterpret_cast<uint32_t*>(&s_x[r * LD64 + c]) = pack_bf16(x0, x1);
    }
  __syncthreads();
  prof_mark(p, 8);
  // ---- Y = A^T X ------------------------------------------------------------------------------
  zero_acc<1, NTQ>(acs);
  warp_gemm<1, NTQ / 2, true, true>(acs, sm.a, LD64, 16 * mt, 0, s_x, LD64, 0, CQ * nq, 4, lane);
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + g8 + 8 * hh, c = CQ * nq + 8 * nt + t2;
      *reinterpret_cast<uint32_t*>(&s_y[r * LD64 + c]) =
          pack_bf16(acs[0][nt][2 * hh], acs[0][nt][2 * hh + 1]);
    }
  __syncthreads();
  prof_mark(p, 9);
  // ---- dL = -stril(Y A^T) ---------------------------------------------------------------------
  zero_acc<1, NTQ>(acs);
  warp_gemm<1, NTQ / 2, false, false>(acs, s_y, LD64, 16 * mt, 0, sm.a, LD64, 0, CQ * nq, 4, lane);
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + g8 + 8 * hh, c = CQ * nq + 8 * nt + t2;
      if (r < valid)
        *reinterpret_cast<float2*>(p.dl + row64 + (int64_t)r * gld64 + c) =
            make_float2((r > c) ? -acs[0][nt][2 * hh] : 0.f,
                        (r > c + 1) ? -acs[0][nt][2 * hh + 1] : 0.f);
    }
  prof_mark(p, 10);
  // ---- dAqk = scale tril(do v_new^T) ----------------------------------------------------------
  zero_acc<1, NTQ>(acs);
  warp_gemm<1, NTQ / 2, false, false>(acs, sm.dO, LDD, 16 * mt, 0, sm.vn, LDD, 0, CQ * nq, 8, lane);
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + g8 + 8 * hh, c = CQ * nq + 8 * nt + t2;
      if (r < valid)
        *reinterpret_cast<float2*>(p.daqk + row64 + (int64_t)r * gld64 + c) =
            make_float2((r >= c) ? acs[0][nt][2 * hh] * p.scale : 0.f,
                        (r >= c + 1) ? acs[0][nt][2 * hh + 1] * p.scale : 0.f);
    }
  if (tid < valid) p.db_p[(cw.token0 + tid) * H + head] = sm.db[tid];
  prof_mark(p, 11);
}

// ------------------------------------------------------------------------------------------
// intra: gradients through Aqk and L.
// 16 warps in two groups of 8.  A group owns two 16-row blocks ({0,3} or {1,2}: equal work) and
// computes everything that lands on those rows; inside a group warp w owns channels
// [16 w, 16 w + 16), so every output element has exactly one owner and lives in registers.
// ------------------------------------------------------------------------------------------
struct IntraBwdSmem {
  bf16 q[64 * LDD];
  bf16 k[64 * LDD];
  float g[64 * D];
  bf16 da[64 * LD64];    // dAqk
  bf16 dl[64 * LD64];    // dL
  bf16 kn[2][64 * LDD];  // per group: gated k (row phase: columns; column phase: beta-scaled rows)
  bf16 qn[2][64 * LDD];  // per group: gated q (column phase)
  float beta[64];
  float db[64];
};

__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(256) : "memory");
}

__global__ void __launch_bounds__(512) kda_bwd_intra_kernel(const BwdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  IntraBwdSmem& sm = *reinterpret_cast<IntraBwdSmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp >> 3, gtid = tid & 255;
  const int head = blockIdx.y, H = p.H;
  const ChunkWork cw = locate_chunk(p.cu_seqlens, p.chunk_offsets, p.nseq, blockIdx.x);
  if (cw.valid == 0) return;
  const int valid = cw.valid;
  const int64_t rowD = (cw.token0 * H + head) * D;
  const int64_t gld = (int64_t)H * D;
  const int64_t row64 = (cw.token0 * H + head) * 64;
  const int64_t gld64 = (int64_t)H * 64;
  const int g8 = lane >> 2, t2 = 2 * (lane & 3);
  const int n0 = 16 * (warp & 7);
  bf16* kn = sm.kn[group];
  bf16* qn = sm.qn[group];

  prof_mark(p, 16);
  load_tile_b16<64, D, LDD, 512>(sm.q, p.q + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, 512>(sm.k, p.k + rowD, gld, valid, tid);
  load_tile_f32<64, D, D, 512>(sm.g, p.g + rowD, gld, valid, tid);
  cp_async_commit();
  if (tid < 64) {
    sm.beta[tid] = tid < valid ? p.beta[(cw.token0 + tid) * H + head] : 0.f;
    sm.db[tid] = 0.f;
  }
  for (int idx = tid; idx < 64 * 16; idx += 512) {
    int r = idx >> 4, c = (idx & 15) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), l = a;
    if (r < valid) {
      a = __ldg(reinterpret_cast<const float4*>(p.daqk + row64 + (int64_t)r * gld64 + c));
      l = __ldg(reinterpret_cast<const float4*>(p.dl + row64 + (int64_t)r * gld64 + c));
    }
    uint2 ua, ul;
    ua.x = pack_bf16(a.x, a.y); ua.y = pack_bf16(a.z, a.w);
    ul.x = pack_bf16(l.x, l.y); ul.y = pack_bf16(l.z, l.w);
    *reinterpret_cast<uint2*>(&sm.da[r * LD64 + c]) = ua;
    *reinterpret_cast<uint2*>(&sm.dl[r * LD64 + c]) = ul;
  }
  cp_async_wait<0>();
  __syncthreads();
  if (valid < 64) {
    for (int idx = tid; idx < (64 - valid) * D; idx += 512) {
      int r = valid + idx / D, c = idx % D;
      sm.g[r * D + c] = sm.g[(valid - 1) * D + c];
    }
    __syncthreads();
  }

  float dq[2][2][4], dk[2][2][4], dg[2][2][4];
  prof_mark(p, 17);

  // ---- row phase: dq_i, dk_i, dbeta_i from sum_j (.)_ij 2^{G_i - G_j} k_j ----------------------
#pragma unroll
  for (int bi = 0; bi < 2; ++bi) {
    const int ri = group == 0 ? (bi == 0 ? 0 : 3) : (bi == 0 ? 1 : 2);
    const int ncol = 16 * (ri + 1);
    const float* R = sm.g + (16 * ri) * D;
    for (int idx = gtid; idx < ncol * (D / 2); idx += 256) {
      int j = idx / (D / 2), c = (idx % (D / 2)) * 2;
      float e0 = fexp2(fminf(R[c] - sm.g[j * D + c], 126.f));
      float e1 = fexp2(fminf(R[c + 1] - sm.g[j * D + c + 1], 126.f));
      float2 kv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.k[j * LDD + c]));
      *reinterpret_cast<uint32_t*>(&kn[j * LDD + c]) = pack_bf16(kv.x * e0, kv.y * e1);
    }
    group_sync(group);
    float aq[1][2][4], ax[1][2][4];
    zero_acc<1, 2>(aq);
    zero_acc<1, 2>(ax);
    warp_gemm<1, 1, false, true>(aq, sm.da, LD64, 16 * ri, 0, kn, LDD, 0, n0, ri + 1, lane);
    warp_gemm<1, 1, false, true>(ax, sm.dl, LD64, 16 * ri, 0, kn, LDD, 0, n0, ri + 1, lane);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int i = 16 * ri + g8 + 8 * hh;
      float b = sm.beta[i], dbp = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        int c = n0 + 8 * nt + t2;
        float e0 = fexp2(sm.g[i * D + c] - R[c]), e1 = fexp2(sm.g[i * D + c + 1] - R[c + 1]);
        float2 qv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.q[i * LDD + c]));
        float2 kv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.k[i * LDD + c]));
        float q0 = aq[0][nt][2 * hh] * e0, q1 = aq[0][nt][2 * hh + 1] * e1;
        float x0 = ax[0][nt][2 * hh] * e0, x1 = ax[0][nt][2 * hh + 1] * e1;
        dq[bi][nt][2 * hh] = q0;
        dq[bi][nt][2 * hh + 1] = q1;
        dk[bi][nt][2 * hh] = b * x0;
        dk[bi][nt][2 * hh + 1] = b * x1;
        dg[bi][nt][2 * hh] = qv.x * q0 + kv.x * b * x0;
        dg[bi][nt][2 * hh + 1] = qv.y * q1 + kv.y * b * x1;
        dbp += kv.x * x0 + kv.y * x1;
      }
      dbp += __shfl_xor_sync(0xffffffffu, dbp, 1);
      dbp += __shfl_xor_sync(0xffffffffu, dbp, 2);
      if ((lane & 3) == 0) atomicAdd(&sm.db[i], dbp);
    }
    group_sync(group);
  }

  prof_mark(p, 18);
  // ---- column phase: dk_j from sum_i (.)_ij 2^{G_i - G_j} {q_i, beta_i k_i} --------------------
#pragma unroll
  for (int bi = 0; bi < 2; ++bi) {
    const int cj = group == 0 ? (bi == 0 ? 0 : 3) : (bi == 0 ? 1 : 2);
    const float* R = sm.g + (16 * cj + 15) * D;
    const int r0 = 16 * cj;
    for (int idx = gtid; idx < (64 - r0) * (D / 2); idx += 256) {
      int i = r0 + idx / (D / 2), c = (idx % (D / 2)) * 2;
      float e0 = fexp2(fminf(sm.g[i * D + c] - R[c], 126.f));
      float e1 = fexp2(fminf(sm.g[i * D + c + 1] - R[c + 1], 126.f));
      float2 qv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.q[i * LDD + c]));
      float2 kv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.k[i * LDD + c]));
      float b = sm.beta[i];
      *reinterpret_cast<uint32_t*>(&qn[i * LDD + c]) = pack_bf16(qv.x * e0, qv.y * e1);
      *reinterpret_cast<uint32_t*>(&kn[i * LDD + c]) = pack_bf16(kv.x * e0 * b, kv.y * e1 * b);
    }
    group_sync(group);
    float ac[1][2][4];
    zero_acc<1, 2>(ac);
    warp_gemm<1, 1, true, true>(ac, sm.da, LD64, r0, r0, qn, LDD, r0, n0, 4 - cj, lane);
    warp_gemm<1, 1, true, true>(ac, sm.dl, LD64, r0, r0, kn, LDD, r0, n0, 4 - cj, lane);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int j = r0 + g8 + 8 * hh;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        int c = n0 + 8 * nt + t2;
        float f0 = fexp2(R[c] - sm.g[j * D + c]), f1 = fexp2(R[c + 1] - sm.g[j * D + c + 1]);
        float2 kv = unpack_bf16(*reinterpret_cast<uint32_t*>(&sm.k[j * LDD + c]));
        float x0 = ac[0][nt][2 * hh] * f0, x1 = ac[0][nt][2 * hh + 1] * f1;
        dk[bi][nt][2 * hh] += x0;
        dk[bi][nt][2 * hh + 1] += x1;
        dg[bi][nt][2 * hh] -= kv.x * x0;
        dg[bi][nt][2 * hh + 1] -= kv.y * x1;
      }
    }
    group_sync(group);
  }

  prof_mark(p, 19);
  // ---- combine with the wy partials: all loads first, then the stores -------------------------
  float2 pa[2][2][2], pb[2][2][2], pc[2][2][2];
#pragma unroll
  for (int bi = 0; bi < 2; ++bi)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int rb = group == 0 ? (bi == 0 ? 0 : 3) : (bi == 0 ? 1 : 2);
        int r = 16 * rb + g8 + 8 * hh;
        int64_t gi = rowD + (int64_t)r * gld + n0 + 8 * nt + t2;
        float2 z = make_float2(0.f, 0.f);
        pa[bi][hh][nt] = r < valid ? __ldg(reinterpret_cast<const float2*>(p.dq_p + gi)) : z;
        pb[bi][hh][nt] = r < valid ? __ldg(reinterpret_cast<const float2*>(p.dk_p + gi)) : z;
        pc[bi][hh][nt] = r < valid ? __ldg(reinterpret_cast<const float2*>(p.dg_p + gi)) : z;
      }
#pragma unroll
  for (int bi = 0; bi < 2; ++bi)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int rb = group == 0 ? (bi == 0 ? 0 : 3) : (bi == 0 ? 1 : 2);
      int r = 16 * rb + g8 + 8 * hh;
      if (r < valid) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          int64_t gi = rowD + (int64_t)r * gld + n0 + 8 * nt + t2;
          float2 a = pa[bi][hh][nt], b = pb[bi][hh][nt], c = pc[bi][hh][nt];
          *reinterpret_cast<uint32_t*>(p.dq + gi) =
              pack_bf16(a.x + dq[bi][nt][2 * hh], a.y + dq[bi][nt][2 * hh + 1]);
          *reinterpret_cast<uint32_t*>(p.dk + gi) =
              pack_bf16(b.x + dk[bi][nt][2 * hh], b.y + dk[bi][nt][2 * hh + 1]);
          *reinterpret_cast<float2*>(p.dg + gi) = make_float2(
              (c.x + dg[bi][nt][2 * hh]) * kLn2, (c.y + dg[bi][nt][2 * hh + 1]) * kLn2);
        }
      }
    }
  __syncthreads();  // every dbeta contribution is in
  if (tid < valid) {
    int64_t bi = (cw.token0 + tid) * H + head;
    p.db[bi] = p.db_p[bi] + sm.db[tid];
  }
  prof_mark(p, 20);
}

int launch_bwd_chunk_tc(const bf16* q, const bf16* k, const bf16* v, const float* g, const float* beta,
                        const bf16* akk, const bf16* h, const bf16* dh, const bf16* vnew,
                        const bf16* dv2, const bf16* dout, bf16* dq, bf16* dk, bf16* dv, float* dg,
                        float* db, const int32_t* cu, const int32_t* co, int nseq, int H,
                        int64_t tokens, int chunks, long long* prof, cudaStream_t s);

static int check_launch() { return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH; }
template <typename Kern>
static int set_smem(Kern kern, size_t bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) ==
                 cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

// forward-stage launchers (kda_chunk_fwd.cu) driven through a parameter block built there
int launch_recompute(const void* q, const void* k, const void* v, const float* g, const float* beta,
                     const void* aqk, const void* akk, const float* h0, void* w, void* u, void* kg,
                     void* qg, void* h_out, void* vnew_out, const int32_t* cu, const int32_t* co,
                     int nseq, int H, int chunks, int64_t tokens, cudaStream_t s);

}  // namespace kda

using kda::bf16;

static long long* g_prof_buffer = nullptr;
// Debugging aid: device buffer of 64 x 32 int64 that receives per-phase timestamps of the first
// 64 chunks of head 0 from the backward chunk kernels (NULL switches it off).
extern "C" int kda_debug_set_profile_buffer(void* buffer) {
  g_prof_buffer = reinterpret_cast<long long*>(buffer);
  return KDA_OK;
}

extern "C" int64_t kda_chunk_bwd_workspace_bytes(int64_t tokens, int heads, int64_t num_chunks) {
  const int64_t nd = tokens * heads * 128;
  const int64_t hs = num_chunks * heads * 128 * 128;
  int64_t bytes = 0;
  bytes += 6 * nd * 2;            // w, u, kg, qg, v_new, dv2 (bf16)
  bytes += 2 * hs * 2;            // h, dh (bf16)
  bytes += 2 * tokens * heads * 64 * 4;  // dAqk, dL (fp32)
  bytes += 3 * nd * 4;            // dq, dk, dG partials (fp32)
  bytes += tokens * heads * 4;    // dbeta partial
  return bytes + 256;
}

extern "C" int kda_chunk_bwd(const void* q, const void* k, const void* v, const float* cum_gate,
                             const float* beta, const void* aqk, const void* akk,
                             const float* initial_state, const void* d_out,
                             const float* d_final_state, void* dq, void* dk, void* dv, float* dg,
                             float* dbeta, float* d_initial_state, const int32_t* cu_seqlens,
                             const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                             int key_dim, int value_dim, int num_chunks, void* workspace,
                             int64_t workspace_bytes, void* stream) {
  if (!q || !k || !v || !cum_gate || !beta || !aqk || !akk || !d_out || !dq || !dk || !dv || !dg ||
      !dbeta || !cu_seqlens || !chunk_offsets || !workspace)
    return KDA_ERR_ARG;
  if (key_dim != 128 || value_dim != 128) return KDA_ERR_UNSUPPORTED;
  if (nseq < 1 || heads < 1 || tokens < 1 || num_chunks < 0) return KDA_ERR_ARG;
  if (workspace_bytes < kda_chunk_bwd_workspace_bytes(tokens, heads, num_chunks)) return KDA_ERR_ARG;
  if (((uintptr_t)workspace & 15) != 0) return KDA_ERR_ARG;
  const int64_t nd = tokens * heads * 128;
  const int64_t hs = (int64_t)num_chunks * heads * 128 * 128;
  const int64_t n64 = tokens * heads * 64;
  bf16* b = reinterpret_cast<bf16*>(workspace);
  bf16 *w = b, *u = b + nd, *kg = b + 2 * nd, *qg = b + 3 * nd, *vnew = b + 4 * nd,
       *dv2 = b + 5 * nd, *hbuf = b + 6 * nd, *dhbuf = b + 6 * nd + hs;
  float* f = reinterpret_cast<float*>(b + 6 * nd + 2 * hs);
  float *daqk = f, *dl = f + n64, *dq_p = f + 2 * n64, *dk_p = dq_p + nd, *dg_p = dk_p + nd,
        *db_p = dg_p + nd;
  cudaStream_t s = (cudaStream_t)stream;

  int rc = kda::launch_recompute(q, k, v, cum_gate, beta, aqk, akk, initial_state, w, u, kg, qg,
                                 hbuf, vnew, cu_seqlens, chunk_offsets, nseq, heads, num_chunks, tokens, s);
  if (rc) return rc;

  kda::BwdParams p{};
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.g = cum_gate; p.beta = beta;
  p.aqk = (const bf16*)aqk; p.akk = (const bf16*)akk;
  p.w = w; p.kg = kg; p.qg = qg; p.h = hbuf; p.vnew = vnew; p.dout = (const bf16*)d_out;
  p.dht = d_final_state; p.dh0 = d_initial_state; p.dh = dhbuf; p.dv2 = dv2;
  p.daqk = daqk; p.dl = dl; p.dq_p = dq_p; p.dk_p = dk_p; p.dg_p = dg_p; p.db_p = db_p;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.dg = dg; p.db = dbeta;
  p.cu_seqlens = cu_seqlens; p.chunk_offsets = chunk_offsets; p.nseq = nseq; p.H = heads;
  p.scale = 0.08838834764831845f;
  p.prof = g_prof_buffer;

  if (kda::set_smem(kda::kda_state_bwd_kernel, sizeof(kda::BStateSmem))) return KDA_ERR_LAUNCH;
  {
    kda::StageScope timing(kda::kStageStateBwd, s);
    kda::kda_state_bwd_kernel<<<(unsigned)(nseq * heads * 2), 256, sizeof(kda::BStateSmem), s>>>(p);
  }
  if ((rc = kda::check_launch())) return rc;
  if (num_chunks == 0) return KDA_OK;
  if (const char* e = getenv("KDA_BWD_TC")) {
    if (e[0] == '1')
      return kda::launch_bwd_chunk_tc(p.q, p.k, p.v, p.g, p.beta, p.akk, p.h, p.dh, p.vnew, p.dv2,
                                      p.dout, p.dq, p.dk, p.dv, p.dg, p.db, cu_seqlens, chunk_offsets,
                                      nseq, heads, tokens, num_chunks, g_prof_buffer, s);
  }
  if (kda::set_smem(kda::kda_bwd_wy_kernel<16>, sizeof(kda::WySmem))) return KDA_ERR_LAUNCH;
  {
    kda::StageScope timing(kda::kStageBwdWy, s);
    kda::kda_bwd_wy_kernel<16><<<dim3(num_chunks, heads), 512, sizeof(kda::WySmem), s>>>(p);
  }
  if ((rc = kda::check_launch())) return rc;
  if (kda::set_smem(kda::kda_bwd_intra_kernel, sizeof(kda::IntraBwdSmem))) return KDA_ERR_LAUNCH;
  {
    kda::StageScope timing(kda::kStageBwdIntra, s);
    kda::kda_bwd_intra_kernel<<<dim3(num_chunks, heads), 512, sizeof(kda::IntraBwdSmem), s>>>(p);
  }
  return kda::check_launch();
}
