// Chunked KDA backward for K = V = 128, chunk = 64 (bf16 operands, fp32 accumulation): orchestration.
//
// Stages (reference orchestration: attn_gym/linear/kda/bwd/cute/chunk_kda_bwd.py:21-147):
//   wu            recompute w, u, kg, qg from the stored A                  (kda_chunk_fwd.cu)
//   state_fwd     recompute the chunk-entry states h[c] and v_new            (kda_state_tc.cu)
//   state_bwd     reverse chunk walk, fp32 dh in tensor memory: dv2, dh[c], dh0  (kda_state_tc.cu)
//   bwd_chunk     per (chunk, head): everything else, one tcgen05 kernel     (kda_bwd_chunk_tc.cu)
//
// dG is the gradient with respect to the cumulative log2 gate and is multiplied by ln 2 once,
// in the last stage.
#include "kda_common.cuh"
#include "kda_timing.cuh"

namespace kda {

int launch_state_bwd_tc(const bf16* w, const bf16* kg, const bf16* qg, const bf16* aqk, const bf16* dout,
                        const float* g, const float* dht, float* dh0, bf16* dh_out, bf16* dv2_out,
                        const int32_t* cu, const int32_t* co, int nseq, int H, int64_t tokens,
                        int chunks, cudaStream_t s);
int launch_bwd_chunk_tc(const bf16* q, const bf16* k, const bf16* v, const float* g, const float* beta,
                        const bf16* akk, const bf16* h, const bf16* dh, const bf16* vnew,
                        const bf16* dv2, const bf16* dout, bf16* dq, bf16* dk, bf16* dv, float* dg,
                        float* db, const float* rstd_q, const float* rstd_k, const int32_t* cu,
                        const int32_t* co, int nseq, int H, int64_t tokens, int chunks, long long* prof,
                        cudaStream_t s);
int launch_recompute(const void* q, const void* k, const void* v, const float* g, const float* beta,
                     const void* aqk, const void* akk, const float* h0, void* w, void* u, void* kg,
                     void* qg, void* h_out, void* vnew_out, const int32_t* cu, const int32_t* co,
                     int nseq, int H, int chunks, int64_t tokens, cudaStream_t s);

}  // namespace kda

using kda::bf16;

// Development builds (-DKDA_PHASE_PROFILE) can hand the persistent kernels a device buffer of
// 64 x 32 int64 that receives %globaltimer stamps of their phases; the shipped library has neither
// the setter nor the stamps.
static long long* g_prof_buffer = nullptr;
namespace kda { long long* debug_profile_buffer() { return g_prof_buffer; } }
#ifdef KDA_PHASE_PROFILE
extern "C" int kda_debug_set_profile_buffer(void* buffer) {
  g_prof_buffer = reinterpret_cast<long long*>(buffer);
  return KDA_OK;
}
#endif

extern "C" int64_t kda_chunk_bwd_workspace_bytes(int64_t tokens, int heads, int64_t num_chunks) {
  const int64_t nd = tokens * heads * 128;
  const int64_t hs = num_chunks * heads * 128 * 128;
  // w, u, kg, qg, v_new, dv2 and h, dh (all bf16); a scratch tape [2][tokens, H, 64] for the rebuild
  return (6 * nd + 2 * hs + nd) * 2 + 256;
}

static int chunk_bwd_impl(bool saved, const float* rstd_q, const float* rstd_k, const void* q, const void* k, const void* v, const float* cum_gate,
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
  bf16* b = reinterpret_cast<bf16*>(workspace);
  bf16 *w = b, *u = b + nd, *kg = b + 2 * nd, *qg = b + 3 * nd, *vnew = b + 4 * nd,
       *dv2 = b + 5 * nd, *hbuf = b + 6 * nd, *dhbuf = b + 6 * nd + hs, *tape = b + 6 * nd + 2 * hs;
  cudaStream_t s = (cudaStream_t)stream;

  int rc = KDA_OK;
  if (!saved) {   // reference behaviour: rebuild w, u, kg, qg, h[c], v_new from the stored A
    rc = kda::launch_recompute(q, k, v, cum_gate, beta, tape, tape + nd / 2, initial_state, w, u, kg, qg,
                               hbuf, vnew, cu_seqlens, chunk_offsets, nseq, heads, num_chunks, tokens, s);
    if (rc) return rc;
  }

  const bf16* qb = (const bf16*)q; const bf16* kb = (const bf16*)k; const bf16* vb = (const bf16*)v;
  rc = kda::launch_state_bwd_tc(w, kg, qg, (const bf16*)aqk, (const bf16*)d_out, cum_gate,
                                d_final_state, d_initial_state, dhbuf, dv2, cu_seqlens, chunk_offsets,
                                nseq, heads, tokens, num_chunks, s);
  if (rc) return rc;
  return kda::launch_bwd_chunk_tc(qb, kb, vb, cum_gate, beta, (const bf16*)akk, hbuf, dhbuf, vnew, dv2,
                                  (const bf16*)d_out, (bf16*)dq, (bf16*)dk, (bf16*)dv, dg, dbeta,
                                  rstd_q, rstd_k, cu_seqlens, chunk_offsets, nseq, heads, tokens,
                                  num_chunks, g_prof_buffer, s);
}

#define KDA_BWD_ARGS                                                                              \
  const void *q, const void *k, const void *v, const float *cum_gate, const float *beta,           \
      const void *aqk, const void *akk, const float *initial_state, const void *d_out,             \
      const float *d_final_state, void *dq, void *dk, void *dv, float *dg, float *dbeta,           \
      float *d_initial_state, const int32_t *cu_seqlens, const int32_t *chunk_offsets, int nseq,   \
      int64_t tokens, int heads, int key_dim, int value_dim, int num_chunks
#define KDA_BWD_PASS                                                                              \
  q, k, v, cum_gate, beta, aqk, akk, initial_state, d_out, d_final_state, dq, dk, dv, dg, dbeta,   \
      d_initial_state, cu_seqlens, chunk_offsets, nseq, tokens, heads, key_dim, value_dim, num_chunks

extern "C" int kda_chunk_bwd(KDA_BWD_ARGS, void* workspace, int64_t workspace_bytes, void* stream) {
  return chunk_bwd_impl(false, nullptr, nullptr, KDA_BWD_PASS, workspace, workspace_bytes, stream);
}

// The state-gradient walk of kda_chunk_bwd_saved alone: d_initial_state for the cotangents
// (d_out, d_final_state), from the tapes in `saved` (w, kg, qg; read only) -- the part of the backward
// pass that a context-parallel slice needs before the state gradient of the next slice has arrived.
extern "C" int kda_chunk_bwd_state_saved(const float* cum_gate, const void* aqk, const void* d_out,
                                         const float* d_final_state, float* d_initial_state,
                                         const int32_t* cu_seqlens, const int32_t* chunk_offsets,
                                         int nseq, int64_t tokens, int heads, int key_dim,
                                         int value_dim, int num_chunks, void* saved,
                                         int64_t saved_bytes, void* stream) {
  if (!cum_gate || !aqk || !d_out || !d_initial_state || !cu_seqlens || !chunk_offsets || !saved)
    return KDA_ERR_ARG;
  if (key_dim != 128 || value_dim != 128) return KDA_ERR_UNSUPPORTED;
  if (nseq < 1 || heads < 1 || tokens < 1 || num_chunks < 0) return KDA_ERR_ARG;
  if (saved_bytes < kda_chunk_bwd_workspace_bytes(tokens, heads, num_chunks)) return KDA_ERR_ARG;
  if (((uintptr_t)saved & 15) != 0) return KDA_ERR_ARG;
  const int64_t nd = tokens * heads * 128;
  const int64_t hs = (int64_t)num_chunks * heads * 128 * 128;
  bf16* b = reinterpret_cast<bf16*>(saved);
  bf16 *w = b, *kg = b + 2 * nd, *qg = b + 3 * nd, *dv2 = b + 5 * nd, *dhbuf = b + 6 * nd + hs;
  return kda::launch_state_bwd_tc(w, kg, qg, (const bf16*)aqk, (const bf16*)d_out, cum_gate,
                                  d_final_state, d_initial_state, dhbuf, dv2, cu_seqlens,
                                  chunk_offsets, nseq, heads, tokens, num_chunks, (cudaStream_t)stream);
}

extern "C" int kda_chunk_bwd_saved(KDA_BWD_ARGS, void* saved, int64_t saved_bytes, void* stream) {
  return chunk_bwd_impl(true, nullptr, nullptr, KDA_BWD_PASS, saved, saved_bytes, stream);
}

// Backward of kda_chunk_fwd_qknorm(keep = 1): q and k are the unnormalised rows, rstd_q / rstd_k the
// reciprocal norms the forward pass wrote; dq and dk come back as gradients of the unnormalised rows.
extern "C" int kda_chunk_bwd_qknorm_saved(KDA_BWD_ARGS, const float* rstd_q, const float* rstd_k,
                                          void* saved, int64_t saved_bytes, void* stream) {
  if (!rstd_q || !rstd_k) return KDA_ERR_ARG;
  return chunk_bwd_impl(true, rstd_q, rstd_k, KDA_BWD_PASS, saved, saved_bytes, stream);
}
