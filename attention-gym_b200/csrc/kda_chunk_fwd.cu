// Chunked KDA forward for K = V = 128, chunk = 64, bf16 operands, fp32 state and accumulation.
//
// Three kernels (two here, the state walk in kda_state_tc.cu) replace the reference's seven forward launches
// (attn_gym/linear/kda/fwd/cute/chunk_kda_fwd.py:79-131):
//
//  intra_solve  per (chunk, head): the gated pairwise products and the WY solve
//               Aqk = scale tril(Q~ K~^T),  A = (I + stril(diag(beta) K~ K~^T))^-1
//               (reference stages: fwd/triton/chunk_kda_fwd_intra_sub_chunk_forloop.py:66,
//                fwd/cute/chunk_kda_k3b_offdiag_cutedsl.py:177, fwd/cute/chunk_kda_k4b_inverse_cutedsl.py:188)
//  wu           per (chunk, head): w = A (beta k 2^G), u = A (beta v), kg = k 2^{G_last-G},
//               qg = scale q 2^G   (reference: fwd/triton/recompute_w_u.py:257); reused by backward
//  state_fwd    per (sequence, head), serial over chunks with the fp32 state in tensor memory
//               (kda_state_tc.cu): v_new = u - w h;  o = qg h + Aqk v_new;
//               h <- diag(2^{G_last}) h + kg^T v_new
//
// Gate rebasing: 2^{G_i - G_j} is split as 2^{G_i - R} * 2^{R - G_j} with R the gate of the first
// row of the 16-row block that holds i, so the row factor is <= 1 and the column factor is <= 1
// for every earlier block; inside the diagonal block the column factor spans at most 15 tokens,
// the same exponent budget as the reference (fwd/triton/gate_fwd.py:619-631).
#include "kda_common.cuh"
#include "kda_timing.cuh"

namespace kda {

constexpr int D = 128;     // K = V
constexpr int LDD = 136;   // padded row stride of a [*, 128] bf16 tile (272 B: conflict-free ldmatrix)
constexpr int LD64 = 72;   // padded row stride of a [*, 64] bf16 tile
constexpr int LDP = 68;    // padded row stride of a [64, 64] fp32 tile

struct ChunkParams {
  const bf16* q; const bf16* k; const bf16* v; const float* g; const float* beta;
  bf16* aqk; bf16* akk;                 // tape [N, H, 64]
  bf16* w; bf16* u; bf16* kg; bf16* qg;  // [N, H, 128]
  const float* h0; float* ht;
  bf16* o; bf16* h_out; bf16* vnew_out;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int nseq, H;
  float scale;
  int64_t tokens;   // rows of the token-major buffers (bounds of the TMA tensor maps)
  int chunks;       // chunk capacity: h_out holds chunks * H states (needed only with h_out)
};

int launch_state_fwd_tc(const bf16* w, const bf16* u, const bf16* kg, const bf16* qg, const bf16* aqk,
                        const float* g, const float* h0, float* ht, bf16* o, bf16* h_out,
                        bf16* vnew_out, const int32_t* cu, const int32_t* co, int nseq, int H,
                        int64_t tokens, int chunks, cudaStream_t s);

// ------------------------------------------------------------------------------------------
// intra_solve
// ------------------------------------------------------------------------------------------
struct IntraSmem {
  bf16 q[64 * LDD];
  bf16 k[64 * LDD];
  float g[64 * D];
  bf16 kn[64 * LDD];     // column operand of the current row block; later holds A (fp32 [64][LDP])
  bf16 rk[16 * LDD];     // gated k rows of the current row block
  float pk[64 * LDP];    // L = stril(beta_i P_ij)
  float beta[64];
  float tmp[3 * 256];
};
static_assert(sizeof(bf16) * 64 * LDD >= sizeof(float) * 64 * LDP, "A overlay must fit");

// dst[i][j] = sign * sum_{k<kk} A[i][k] B[k][j] for a 16x16 tile; thread t -> (t >> 4, t & 15)
__device__ __forceinline__ void block_mm16(float* dst, int ldd, const float* A, int lda,
                                           const float* B, int ldb, int kk, float sign, int tid) {
  int i = tid >> 4, j = tid & 15;
  float s = 0.f;
  for (int k = 0; k < kk; ++k) s += A[i * lda + k] * B[k * ldb + j];
  dst[i * ldd + j] = sign * s;
}

// eight adjacent bf16 / fp32 values of a row-major shared-memory tile (16-byte accesses)
__device__ __forceinline__ void ld8_bf(const bf16* p, float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y; o[4] = c.x; o[5] = c.y; o[6] = d.x; o[7] = d.y;
}
__device__ __forceinline__ uint4 pack8_bf(const float (&x)[8]) {
  uint4 u;
  u.x = pack_bf16(x[0], x[1]); u.y = pack_bf16(x[2], x[3]);
  u.z = pack_bf16(x[4], x[5]); u.w = pack_bf16(x[6], x[7]);
  return u;
}
__device__ __forceinline__ void ld8_f(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

__global__ void __launch_bounds__(256) kda_intra_solve_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  IntraSmem& sm = *reinterpret_cast<IntraSmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.y, H = p.H;
  const ChunkWork cw = locate_chunk(p.cu_seqlens, p.chunk_offsets, p.nseq, blockIdx.x);
  if (cw.valid == 0) return;
  const int valid = cw.valid;
  const int64_t rowD = (cw.token0 * H + head) * D;
  const int64_t gld = (int64_t)H * D;

  load_tile_b16<64, D, LDD, 256>(sm.q, p.q + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, 256>(sm.k, p.k + rowD, gld, valid, tid);
  load_tile_f32<64, D, D, 256>(sm.g, p.g + rowD, gld, valid, tid);
  cp_async_commit();
  if (tid < 64) sm.beta[tid] = tid < valid ? p.beta[(cw.token0 + tid) * H + head] : 0.f;
  cp_async_wait<0>();
  __syncthreads();
  // rows past the tail repeat the last cumulative gate, so they neither decay nor overflow
  if (valid < 64) {
    for (int idx = tid; idx < (64 - valid) * D; idx += 256) {
      int r = valid + idx / D, c = idx % D;
      sm.g[r * D + c] = sm.g[(valid - 1) * D + c];
    }
    __syncthreads();
  }

  for (int ri = 0; ri < 4; ++ri) {
    const int ncol = 16 * (ri + 1);
    const float* R = sm.g + (16 * ri) * D;
    // row operands (in place for q, separate for k): x_i 2^{G_i - R}; one 8-channel piece per thread
    {
      const int r = tid >> 4, c = (tid & 15) * 8, i = 16 * ri + r;
      float gi[8], rr[8], qq[8], kk[8];
      ld8_f(sm.g + i * D + c, gi);
      ld8_f(R + c, rr);
      ld8_bf(sm.q + i * LDD + c, qq);
      ld8_bf(sm.k + i * LDD + c, kk);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float ex = fexp2(gi[e] - rr[e]);
        qq[e] *= ex;
        kk[e] *= ex;
      }
      *reinterpret_cast<uint4*>(sm.q + i * LDD + c) = pack8_bf(qq);
      *reinterpret_cast<uint4*>(sm.rk + r * LDD + c) = pack8_bf(kk);
    }
    // column operand: k_j 2^{R - G_j}, j < ncol (entries with j > i are masked after the product)
    for (int task = tid; task < ncol * 16; task += 256) {
      const int j = task >> 4, c = (task & 15) * 8;
      float gj[8], rr[8], kk[8];
      ld8_f(sm.g + j * D + c, gj);
      ld8_f(R + c, rr);
      ld8_bf(sm.k + j * LDD + c, kk);
#pragma unroll
      for (int e = 0; e < 8; ++e) kk[e] *= fexp2(fminf(rr[e] - gj[e], 126.f));
      *reinterpret_cast<uint4*>(sm.kn + j * LDD + c) = pack8_bf(kk);
    }
    __syncthreads();
    {
      const int which = warp & 1, nb = warp >> 1;
      float acc[1][2][4];
      zero_acc<1, 2>(acc);
      if (nb <= ri) {
        if (which == 0)
          warp_gemm<1, 1, false, false>(acc, sm.q, LDD, 16 * ri, 0, sm.kn, LDD, 0, 16 * nb, 8, lane);
        else
          warp_gemm<1, 1, false, false>(acc, sm.rk, LDD, 0, 0, sm.kn, LDD, 0, 16 * nb, 8, lane);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int i = 16 * ri + (lane >> 2) + 8 * hh;
          int j = 16 * nb + 8 * nt + 2 * (lane & 3);
          float a0 = acc[0][nt][2 * hh], a1 = acc[0][nt][2 * hh + 1];
          if (which == 0) {
            float x0 = (j <= i) ? a0 * p.scale : 0.f;
            float x1 = (j + 1 <= i) ? a1 * p.scale : 0.f;
            if (i < valid)
              *reinterpret_cast<uint32_t*>(p.aqk + ((cw.token0 + i) * H + head) * 64 + j) =
                  pack_bf16(x0, x1);
          } else {
            float b = sm.beta[i];
            sm.pk[i * LDP + j] = (j < i) ? a0 * b : 0.f;
            sm.pk[i * LDP + j + 1] = (j + 1 < i) ? a1 * b : 0.f;
          }
        }
    }
    __syncthreads();
  }

  // ---- A = (I + L)^-1 by 16x16 blocks, fp32 -------------------------------------------------
  float* A = reinterpret_cast<float*>(sm.kn);
  for (int idx = tid; idx < 64 * LDP; idx += 256) A[idx] = 0.f;
  __syncthreads();
  if (tid < 64) {  // diagonal blocks: column c of block b by forward substitution
    const int b = tid >> 4, c = tid & 15;
    const float* L = sm.pk + (16 * b) * LDP + 16 * b;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = (i == c) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s -= L[i * LDP + j] * x[j];
      x[i] = s;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) A[(16 * b + i) * LDP + 16 * b + c] = x[i];
  }
  __syncthreads();
  // A[r][c] = -A[r][r] * sum_{c<=m<r} L[r][m] A[m][c], one block diagonal at a time
  for (int dist = 1; dist < 4; ++dist) {
    for (int c = 0; c + dist < 4; ++c) {
      int r = c + dist;
      block_mm16(sm.tmp + 256 * c, 16, sm.pk + (16 * r) * LDP + 16 * c, LDP,
                 A + (16 * c) * LDP + 16 * c, LDP, 16 * dist, 1.f, tid);
    }
    __syncthreads();
    for (int c = 0; c + dist < 4; ++c) {
      int r = c + dist;
      block_mm16(A + (16 * r) * LDP + 16 * c, LDP, A + (16 * r) * LDP + 16 * r, LDP,
                 sm.tmp + 256 * c, 16, 16, -1.f, tid);
    }
    __syncthreads();
  }
  for (int idx = tid; idx < 64 * 8; idx += 256) {
    int r = idx >> 3, c = (idx & 7) * 8;
    if (r < valid) {
      const float* a = A + r * LDP + c;
      uint4 o;
      o.x = pack_bf16(a[0], a[1]); o.y = pack_bf16(a[2], a[3]);
      o.z = pack_bf16(a[4], a[5]); o.w = pack_bf16(a[6], a[7]);
      *reinterpret_cast<uint4*>(p.akk + ((cw.token0 + r) * H + head) * 64 + c) = o;
    }
  }
}

// ------------------------------------------------------------------------------------------
// wu: w, u, kg, qg from k, v, q, G, beta and the stored A
// ------------------------------------------------------------------------------------------
struct WuSmem {
  bf16 k[64 * LDD];
  bf16 v[64 * LDD];
  bf16 q[64 * LDD];
  float g[64 * D];
  bf16 a[64 * LD64];
  float beta[64];
};

__global__ void __launch_bounds__(256) kda_wu_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  WuSmem& sm = *reinterpret_cast<WuSmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.y, H = p.H;
  const ChunkWork cw = locate_chunk(p.cu_seqlens, p.chunk_offsets, p.nseq, blockIdx.x);
  if (cw.valid == 0) return;
  const int valid = cw.valid;
  const int64_t rowD = (cw.token0 * H + head) * D;
  const int64_t gld = (int64_t)H * D;

  load_tile_b16<64, D, LDD, 256>(sm.k, p.k + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, 256>(sm.v, p.v + rowD, gld, valid, tid);
  load_tile_b16<64, D, LDD, 256>(sm.q, p.q + rowD, gld, valid, tid);
  load_tile_f32<64, D, D, 256>(sm.g, p.g + rowD, gld, valid, tid);
  load_tile_b16<64, 64, LD64, 256>(sm.a, p.akk + (cw.token0 * H + head) * 64, (int64_t)H * 64,
                                   valid, tid);
  cp_async_commit();
  if (tid < 64) sm.beta[tid] = tid < valid ? p.beta[(cw.token0 + tid) * H + head] : 0.f;
  cp_async_wait<0>();
  __syncthreads();

  const float* glast = sm.g + (valid - 1) * D;
  for (int task = tid; task < 64 * 16; task += 256) {      // one 8-channel piece of one row per task
    const int r = task >> 4, c = (task & 15) * 8;
    float g[8], gl[8], kk[8], vv[8], qq[8], kgv[8];
    ld8_f(sm.g + r * D + c, g);
    ld8_f(glast + c, gl);
    ld8_bf(sm.k + r * LDD + c, kk);
    ld8_bf(sm.v + r * LDD + c, vv);
    ld8_bf(sm.q + r * LDD + c, qq);
    const float b = sm.beta[r];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ex = fexp2(g[e]);
      qq[e] = qq[e] * ex * p.scale;
      kgv[e] = kk[e] * fexp2(gl[e] - g[e]);
      kk[e] = kk[e] * ex * b;
      vv[e] *= b;
    }
    if (r < valid) {
      const int64_t gi = rowD + (int64_t)r * gld + c;
      *reinterpret_cast<uint4*>(p.qg + gi) = pack8_bf(qq);
      *reinterpret_cast<uint4*>(p.kg + gi) = pack8_bf(kgv);
    }
    *reinterpret_cast<uint4*>(sm.k + r * LDD + c) = pack8_bf(kk);
    *reinterpret_cast<uint4*>(sm.v + r * LDD + c) = pack8_bf(vv);
  }
  __syncthreads();
  const int mt = warp & 3, nh = warp >> 2;
  float accw[1][8][4], accu[1][8][4];
  zero_acc<1, 8>(accw);
  zero_acc<1, 8>(accu);
  warp_gemm<1, 4, false, true>(accw, sm.a, LD64, 16 * mt, 0, sm.k, LDD, 0, 64 * nh, 4, lane);
  warp_gemm<1, 4, false, true>(accu, sm.a, LD64, 16 * mt, 0, sm.v, LDD, 0, 64 * nh, 4, lane);
  __syncthreads();
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = 16 * mt + (lane >> 2) + 8 * hh, c = 64 * nh + 8 * nt + 2 * (lane & 3);
      *reinterpret_cast<uint32_t*>(&sm.k[r * LDD + c]) =
          pack_bf16(accw[0][nt][2 * hh], accw[0][nt][2 * hh + 1]);
      *reinterpret_cast<uint32_t*>(&sm.v[r * LDD + c]) =
          pack_bf16(accu[0][nt][2 * hh], accu[0][nt][2 * hh + 1]);
    }
  __syncthreads();
  store_tile_b16<64, D, LDD, 256>(p.w + rowD, gld, sm.k, valid, tid);
  store_tile_b16<64, D, LDD, 256>(p.u + rowD, gld, sm.v, valid, tid);
}

static int check_launch() { return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH; }

template <typename Kern>
static int set_smem(Kern kern, size_t bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) ==
                 cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

int launch_intra_solve(const ChunkParams& p, int chunks, cudaStream_t s) {
  if (chunks == 0) return KDA_OK;
  if (set_smem(kda_intra_solve_kernel, sizeof(IntraSmem))) return KDA_ERR_LAUNCH;
  StageScope timing(kStageIntraSolve, s);
  kda_intra_solve_kernel<<<dim3(chunks, p.H), 256, sizeof(IntraSmem), s>>>(p);
  return check_launch();
}
int launch_wu(const ChunkParams& p, int chunks, cudaStream_t s) {
  if (chunks == 0) return KDA_OK;
  if (set_smem(kda_wu_kernel, sizeof(WuSmem))) return KDA_ERR_LAUNCH;
  StageScope timing(kStageWu, s);
  kda_wu_kernel<<<dim3(chunks, p.H), 256, sizeof(WuSmem), s>>>(p);
  return check_launch();
}
int launch_state_fwd(const ChunkParams& p, cudaStream_t s) {
  return launch_state_fwd_tc(p.w, p.u, p.kg, p.qg, p.aqk, p.g, p.h0, p.ht, p.o, p.h_out, p.vnew_out,
                             p.cu_seqlens, p.chunk_offsets, p.nseq, p.H, p.tokens, p.chunks, s);
}

// Backward's recompute leg: w, u, kg, qg from the stored A, then the chunk-entry states h[c]
// and v_new (no output, no final state).
int launch_recompute(const void* q, const void* k, const void* v, const float* g, const float* beta,
                     const void* aqk, const void* akk, const float* h0, void* w, void* u, void* kg,
                     void* qg, void* h_out, void* vnew_out, const int32_t* cu, const int32_t* co,
                     int nseq, int H, int chunks, int64_t tokens, cudaStream_t s) {
  ChunkParams p{};
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.g = g; p.beta = beta;
  p.aqk = (bf16*)aqk; p.akk = (bf16*)akk;
  p.w = (bf16*)w; p.u = (bf16*)u; p.kg = (bf16*)kg; p.qg = (bf16*)qg;
  p.h0 = h0; p.ht = nullptr; p.o = nullptr;
  p.h_out = (bf16*)h_out; p.vnew_out = (bf16*)vnew_out;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.nseq = nseq; p.H = H;
  p.scale = 0.08838834764831845f;
  p.tokens = tokens;
  p.chunks = chunks;
  int rc = launch_wu(p, chunks, s);
  if (rc) return rc;
  return launch_state_fwd(p, s);
}

}  // namespace kda

using kda::bf16;

static int chunk_fwd_impl(bool keep, const void* q, const void* k, const void* v, const float* cum_gate,
                             const float* beta, const float* initial_state, float* final_state,
                             void* out, void* aqk, void* akk, const int32_t* cu_seqlens,
                             const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                             int key_dim, int value_dim, int num_chunks, void* workspace,
                             int64_t workspace_bytes, void* stream) {
  if (!q || !k || !v || !cum_gate || !beta || !out || !aqk || !akk || !cu_seqlens ||
      !chunk_offsets || !workspace)
    return KDA_ERR_ARG;
  if (key_dim != 128 || value_dim != 128) return KDA_ERR_UNSUPPORTED;
  if (nseq < 1 || heads < 1 || tokens < 1 || num_chunks < 0) return KDA_ERR_ARG;
  if ((int64_t)nseq * heads * 2 > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  if (workspace_bytes < (keep ? kda_chunk_bwd_workspace_bytes(tokens, heads, num_chunks)
                              : kda_chunk_fwd_workspace_bytes(tokens, heads)))
    return KDA_ERR_ARG;
  if (((uintptr_t)workspace & 15) != 0) return KDA_ERR_ARG;
  kda::ChunkParams p{};
  const int64_t nd = tokens * heads * 128;
  bf16* ws = reinterpret_cast<bf16*>(workspace);
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.g = cum_gate; p.beta = beta;
  p.aqk = (bf16*)aqk; p.akk = (bf16*)akk;
  p.w = ws; p.u = ws + nd; p.kg = ws + 2 * nd; p.qg = ws + 3 * nd;
  p.h0 = initial_state; p.ht = final_state; p.o = (bf16*)out;
  // keep: the workspace has the backward layout (w, u, kg, qg, v_new, dv2, h, dh) and the state
  // walk also leaves v_new and the chunk-entry states there
  p.vnew_out = keep ? ws + 4 * nd : nullptr;
  p.h_out = keep ? ws + 6 * nd : nullptr;
  p.chunks = num_chunks;
  p.cu_seqlens = cu_seqlens; p.chunk_offsets = chunk_offsets; p.nseq = nseq; p.H = heads;
  p.scale = 0.08838834764831845f;  // 128^-0.5
  p.tokens = tokens;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = kda::launch_intra_solve(p, num_chunks, s);
  if (rc) return rc;
  rc = kda::launch_wu(p, num_chunks, s);
  if (rc) return rc;
  return kda::launch_state_fwd(p, s);
}

extern "C" int kda_chunk_fwd(const void* q, const void* k, const void* v, const float* cum_gate,
                             const float* beta, const float* initial_state, float* final_state,
                             void* out, void* aqk, void* akk, const int32_t* cu_seqlens,
                             const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                             int key_dim, int value_dim, int num_chunks, void* workspace,
                             int64_t workspace_bytes, void* stream) {
  return chunk_fwd_impl(false, q, k, v, cum_gate, beta, initial_state, final_state, out, aqk, akk,
                        cu_seqlens, chunk_offsets, nseq, tokens, heads, key_dim, value_dim,
                        num_chunks, workspace, workspace_bytes, stream);
}

extern "C" int kda_chunk_fwd_save(const void* q, const void* k, const void* v, const float* cum_gate,
                                  const float* beta, const float* initial_state, float* final_state,
                                  void* out, void* aqk, void* akk, const int32_t* cu_seqlens,
                                  const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                                  int key_dim, int value_dim, int num_chunks, void* saved,
                                  int64_t saved_bytes, void* stream) {
  return chunk_fwd_impl(true, q, k, v, cum_gate, beta, initial_state, final_state, out, aqk, akk,
                        cu_seqlens, chunk_offsets, nseq, tokens, heads, key_dim, value_dim,
                        num_chunks, saved, saved_bytes, stream);
}

extern "C" int64_t kda_chunk_fwd_workspace_bytes(int64_t tokens, int heads) {
  return 4 * tokens * heads * 128 * (int64_t)sizeof(bf16);
}

// The two halves of kda_chunk_fwd as separate entry points: `prepare` is the chunk-parallel part
// (pairwise products, solve, w/u/kg/qg into the workspace), `state` the serial recurrence that
// consumes the workspace.  Context parallelism runs `prepare` once per slice and `state` several
// times (zero entering state, identity state for the slice transition, true entering state).
extern "C" int kda_chunk_fwd_prepare(const void* q, const void* k, const void* v,
                                     const float* cum_gate, const float* beta, void* aqk, void* akk,
                                     const int32_t* cu_seqlens, const int32_t* chunk_offsets,
                                     int nseq, int64_t tokens, int heads, int num_chunks,
                                     void* workspace, int64_t workspace_bytes, void* stream) {
  if (!q || !k || !v || !cum_gate || !beta || !aqk || !akk || !cu_seqlens || !chunk_offsets ||
      !workspace)
    return KDA_ERR_ARG;
  if (nseq < 1 || heads < 1 || tokens < 1 || num_chunks < 0) return KDA_ERR_ARG;
  if (workspace_bytes < kda_chunk_fwd_workspace_bytes(tokens, heads)) return KDA_ERR_ARG;
  kda::ChunkParams p{};
  const int64_t nd = tokens * heads * 128;
  bf16* ws = reinterpret_cast<bf16*>(workspace);
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.g = cum_gate; p.beta = beta;
  p.aqk = (bf16*)aqk; p.akk = (bf16*)akk;
  p.w = ws; p.u = ws + nd; p.kg = ws + 2 * nd; p.qg = ws + 3 * nd;
  p.cu_seqlens = cu_seqlens; p.chunk_offsets = chunk_offsets; p.nseq = nseq; p.H = heads;
  p.scale = 0.08838834764831845f;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = kda::launch_intra_solve(p, num_chunks, s);
  if (rc) return rc;
  return kda::launch_wu(p, num_chunks, s);
}

// use_u == 0 runs the homogeneous recurrence (u = 0): with identity matrices as initial_state the
// final state is the slice transition M = prod_t (I - beta_t k_t k_t^T) diag(2^{g_t}), so that the
// state leaving the slice is M h_in + b.  out may be NULL.
extern "C" int kda_chunk_fwd_state(const float* cum_gate, const float* initial_state,
                                   float* final_state, void* out, const void* aqk,
                                   const int32_t* cu_seqlens, const int32_t* chunk_offsets, int nseq,
                                   int64_t tokens, int heads, void* workspace, int use_u,
                                   void* stream) {
  if (!cum_gate || !aqk || !cu_seqlens || !chunk_offsets || !workspace) return KDA_ERR_ARG;
  if (nseq < 1 || heads < 1 || tokens < 1) return KDA_ERR_ARG;
  if ((int64_t)nseq * heads * 2 > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  kda::ChunkParams p{};
  const int64_t nd = tokens * heads * 128;
  bf16* ws = reinterpret_cast<bf16*>(workspace);
  p.g = cum_gate;
  p.aqk = (bf16*)aqk;
  p.w = ws; p.u = use_u ? ws + nd : nullptr; p.kg = ws + 2 * nd; p.qg = ws + 3 * nd;
  p.h0 = initial_state; p.ht = final_state; p.o = (bf16*)out;
  p.cu_seqlens = cu_seqlens; p.chunk_offsets = chunk_offsets; p.nseq = nseq; p.H = heads;
  p.tokens = tokens;
  return kda::launch_state_fwd(p, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------------
// Chunked forward for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc: a serving engine that has handed every free
// byte of the device to its own paged pool, or a plugin running under a runtime that forbids
// allocation once the model is loaded.  For them the w/u/kg/qg scratch of the forward lives in the
// file-scope device array below instead of a caller workspace.  Every GPU that loads the library
// holds the array (KDA_NOALLOC_SCRATCH_BYTES) until the process exits.
// ------------------------------------------------------------------------------------------------
namespace kda {
static __device__ __align__(256) unsigned char g_noalloc_scratch[KDA_NOALLOC_SCRATCH_BYTES];
static void* g_noalloc_ptr[64] = {nullptr};
}  // namespace kda

extern "C" int kda_chunk_fwd_noalloc(const void* q, const void* k, const void* v,
                                     const float* cum_gate, const float* beta,
                                     const float* initial_state, float* final_state, void* out,
                                     void* aqk, void* akk, const int32_t* cu_seqlens,
                                     const int32_t* chunk_offsets, int nseq, int64_t tokens,
                                     int heads, int key_dim, int value_dim, int num_chunks,
                                     void* stream) {
  if (tokens < 1 || heads < 1) return KDA_ERR_ARG;
  const int64_t need = kda_chunk_fwd_workspace_bytes(tokens, heads);
  if (need > (int64_t)KDA_NOALLOC_SCRATCH_BYTES) return KDA_ERR_SCRATCH;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KDA_ERR_LAUNCH;
  // In host code the array's name is only a handle; the device address comes from the runtime,
  // once per device, with that device current.
  void* scratch = kda::g_noalloc_ptr[dev];
  if (!scratch) {
    if (cudaGetSymbolAddress(&scratch, kda::g_noalloc_scratch) != cudaSuccess || !scratch)
      return KDA_ERR_LAUNCH;
    kda::g_noalloc_ptr[dev] = scratch;
  }
  // Nothing in the scratch has to start at zero: every row a kernel reads was written earlier in
  // the same call, rows past a sequence tail are masked on load.
  return kda_chunk_fwd(q, k, v, cum_gate, beta, initial_state, final_state, out, aqk, akk,
                       cu_seqlens, chunk_offsets, nseq, tokens, heads, key_dim, value_dim,
                       num_chunks, scratch, need, stream);
}
