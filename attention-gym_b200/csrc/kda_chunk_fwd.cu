// Chunked KDA forward for K = V = 128, chunk = 64, bf16 operands, fp32 state and accumulation:
// entry points and orchestration.
//
// Two kernels replace the reference's seven forward launches
// (attn_gym/linear/kda/fwd/cute/chunk_kda_fwd.py:79-131):
//
//  prepare      per (chunk, head), tcgen05 (kda_prepare_tc.cu): the gated pairwise products, the WY
//               solve A = (I + stril(diag(beta) K~ K~^T))^-1, Aqk = scale tril(Q~ K~^T) and
//               w = A (beta k 2^G), u = A (beta v), kg = k 2^{G_last-G}, qg = scale q 2^G
//  state_fwd    per (sequence, head), serial over chunks with the fp32 state in tensor memory
//               (kda_state_tc.cu): v_new = u - w h;  o = qg h + Aqk v_new;
//               h <- diag(2^{G_last}) h + kg^T v_new
//
// The backward pass with recompute=True rebuilds w, u, kg, qg, h[c], v_new with the same two kernels
// (the tape they rewrite goes to scratch), so both modes give bit-identical results.
#include "kda_common.cuh"
#include "kda_timing.cuh"

namespace kda {

constexpr int D = 128;     // K = V
struct ChunkParams {
  const bf16* q; const bf16* k; const bf16* v; const float* g; const float* beta;
  bf16* aqk; bf16* akk;                 // tape [N, H, 64]
  bf16* w; bf16* u; bf16* kg; bf16* qg;  // [N, H, 128]
  float* rstd_q; float* rstd_k; float eps;   // q / k arrive unnormalised when these are set
  const float* h0; float* ht;
  float* trans_out;                     // slice transition [nseq, H, 128, 128], or NULL
  const int32_t* limit_in; int32_t* limit_out;   // per (sequence, head) chunk limits of the state walk, or NULL
  bf16* o; bf16* h_out; bf16* vnew_out;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int nseq, H;
  float scale;
  int64_t tokens;   // rows of the token-major buffers (bounds of the TMA tensor maps)
  int chunks;       // chunk capacity: h_out holds chunks * H states (needed only with h_out)
};

int launch_prepare_tc(const bf16* q, const bf16* k, const bf16* v, const float* g, const float* beta,
                      bf16* aqk, bf16* akk, bf16* w, bf16* u, bf16* kg, bf16* qg, float* rstd_q,
                      float* rstd_k, float eps, const int32_t* cu, const int32_t* co, int nseq, int H,
                      int64_t tokens, int chunks, cudaStream_t s);
int launch_state_fwd_tc(const bf16* w, const bf16* u, const bf16* kg, const bf16* qg, const bf16* aqk,
                        const float* g, const float* h0, float* ht, float* trans_out,
                        const int32_t* limit_in, int32_t* limit_out, bf16* o, bf16* h_out,
                        bf16* vnew_out, const int32_t* cu, const int32_t* co, int nseq, int H,
                        int64_t tokens, int chunks, cudaStream_t s);

// forward: the whole chunk-parallel part (tape, w, u, kg, qg) in one tcgen05 kernel
int launch_prepare(const ChunkParams& p, int chunks, cudaStream_t s) {
  return launch_prepare_tc(p.q, p.k, p.v, p.g, p.beta, p.aqk, p.akk, p.w, p.u, p.kg, p.qg, p.rstd_q,
                           p.rstd_k, p.eps, p.cu_seqlens, p.chunk_offsets, p.nseq, p.H, p.tokens, chunks, s);
}
int launch_state_fwd(const ChunkParams& p, cudaStream_t s) {
  return launch_state_fwd_tc(p.w, p.u, p.kg, p.qg, p.aqk, p.g, p.h0, p.ht, p.trans_out, p.limit_in,
                             p.limit_out, p.o, p.h_out, p.vnew_out, p.cu_seqlens, p.chunk_offsets, p.nseq, p.H, p.tokens, p.chunks, s);
}

// Backward's recompute leg: w, u, kg, qg (and a scratch copy of the tape), then the chunk-entry states
// h[c] and v_new (no output, no final state).
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
  int rc = launch_prepare(p, chunks, s);
  if (rc) return rc;
  return launch_state_fwd(p, s);
}

}  // namespace kda

using kda::bf16;

static int chunk_fwd_impl(bool keep, float* rstd_q, float* rstd_k, float eps, const void* q, const void* k, const void* v, const float* cum_gate,
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
  if ((int64_t)nseq * heads * 8 > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
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
  p.rstd_q = rstd_q; p.rstd_k = rstd_k; p.eps = eps;
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
  int rc = kda::launch_prepare(p, num_chunks, s);
  if (rc) return rc;
  return kda::launch_state_fwd(p, s);
}

extern "C" int kda_chunk_fwd(const void* q, const void* k, const void* v, const float* cum_gate,
                             const float* beta, const float* initial_state, float* final_state,
                             void* out, void* aqk, void* akk, const int32_t* cu_seqlens,
                             const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                             int key_dim, int value_dim, int num_chunks, void* workspace,
                             int64_t workspace_bytes, void* stream) {
  return chunk_fwd_impl(false, nullptr, nullptr, 0.f, q, k, v, cum_gate, beta, initial_state, final_state,
                        out, aqk, akk, cu_seqlens, chunk_offsets, nseq, tokens, heads, key_dim, value_dim,
                        num_chunks, workspace, workspace_bytes, stream);
}

// kda_chunk_fwd / kda_chunk_fwd_save (keep != 0) for unnormalised q and k: every q and k row is scaled
// to unit L2 norm, x * rsqrt(sum x^2 + eps), inside the first kernel, and the reciprocal norms go to
// rstd_q / rstd_k (fp32 [tokens, heads]) for kda_chunk_bwd_qknorm_saved.
extern "C" int kda_chunk_fwd_qknorm(const void* q, const void* k, const void* v, const float* cum_gate,
                                    const float* beta, const float* initial_state, float* final_state,
                                    void* out, void* aqk, void* akk, float* rstd_q, float* rstd_k,
                                    float eps, const int32_t* cu_seqlens, const int32_t* chunk_offsets,
                                    int nseq, int64_t tokens, int heads, int key_dim, int value_dim,
                                    int num_chunks, void* workspace, int64_t workspace_bytes, int keep,
                                    void* stream) {
  if (!rstd_q || !rstd_k || !(eps >= 0.f)) return KDA_ERR_ARG;
  return chunk_fwd_impl(keep != 0, rstd_q, rstd_k, eps, q, k, v, cum_gate, beta, initial_state,
                        final_state, out, aqk, akk, cu_seqlens, chunk_offsets, nseq, tokens, heads,
                        key_dim, value_dim, num_chunks, workspace, workspace_bytes, stream);
}

extern "C" int kda_chunk_fwd_save(const void* q, const void* k, const void* v, const float* cum_gate,
                                  const float* beta, const float* initial_state, float* final_state,
                                  void* out, void* aqk, void* akk, const int32_t* cu_seqlens,
                                  const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                                  int key_dim, int value_dim, int num_chunks, void* saved,
                                  int64_t saved_bytes, void* stream) {
  return chunk_fwd_impl(true, nullptr, nullptr, 0.f, q, k, v, cum_gate, beta, initial_state, final_state,
                        out, aqk, akk, cu_seqlens, chunk_offsets, nseq, tokens, heads, key_dim, value_dim,
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
  p.tokens = tokens;
  cudaStream_t s = (cudaStream_t)stream;
  return kda::launch_prepare(p, num_chunks, s);
}

// use_u == 0 runs the homogeneous recurrence (u = 0): with identity matrices as initial_state the
// final state is the slice transition M = prod_t (I - beta_t k_t k_t^T) diag(2^{g_t}), so that the
// state leaving the slice is M h_in + b.  out may be NULL.
extern "C" int kda_chunk_fwd_state(const float* cum_gate, const float* initial_state,
                                   float* final_state, void* out, const void* aqk,
                                   const int32_t* cu_seqlens, const int32_t* chunk_offsets, int nseq,
                                   int64_t tokens, int heads, void* workspace, int use_u,
                                   const int32_t* chunk_limit, void* stream) {
  if (!cum_gate || !aqk || !cu_seqlens || !chunk_offsets || !workspace) return KDA_ERR_ARG;
  if (nseq < 1 || heads < 1 || tokens < 1) return KDA_ERR_ARG;
  if ((int64_t)nseq * heads * 8 > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  kda::ChunkParams p{};
  const int64_t nd = tokens * heads * 128;
  bf16* ws = reinterpret_cast<bf16*>(workspace);
  p.g = cum_gate;
  p.aqk = (bf16*)aqk;
  p.w = ws; p.u = use_u ? ws + nd : nullptr; p.kg = ws + 2 * nd; p.qg = ws + 3 * nd;
  p.h0 = initial_state; p.ht = final_state; p.o = (bf16*)out;
  p.limit_in = chunk_limit;
  p.cu_seqlens = cu_seqlens; p.chunk_offsets = chunk_offsets; p.nseq = nseq; p.H = heads;
  p.tokens = tokens;
  return kda::launch_state_fwd(p, (cudaStream_t)stream);
}

// One launch for what a context-parallel rank needs before the boundary-state chain can pass through
// it: b = the state leaving the slice for a zero entering state, and M = the dense slice transition,
// so that the leaving state for any entering state is M h_in + b.  Half of the CTAs walk the chains
// with u from a zero state, the other half with u = 0 from an identity state.
extern "C" int kda_chunk_slice_map(const float* cum_gate, float* b_out, float* transition_out,
                                   void* out, int32_t* chunk_limit_out, const void* aqk,
                                   const int32_t* cu_seqlens,
                                   const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                                   void* workspace, void* stream) {
  if (!cum_gate || !b_out || !transition_out || !aqk || !cu_seqlens || !chunk_offsets || !workspace)
    return KDA_ERR_ARG;
  if (nseq < 1 || heads < 1 || tokens < 1) return KDA_ERR_ARG;
  if ((int64_t)nseq * heads * 8 > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  kda::ChunkParams p{};
  const int64_t nd = tokens * heads * 128;
  bf16* ws = reinterpret_cast<bf16*>(workspace);
  p.g = cum_gate;
  p.aqk = (bf16*)aqk;
  p.w = ws; p.u = ws + nd; p.kg = ws + 2 * nd; p.qg = ws + 3 * nd;
  p.ht = b_out; p.trans_out = transition_out;
  p.o = (bf16*)out; p.limit_out = chunk_limit_out;
  p.cu_seqlens = cu_seqlens; p.chunk_offsets = chunk_offsets; p.nseq = nseq; p.H = heads;
  p.tokens = tokens;
  return kda::launch_state_fwd(p, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------------
// Dense batches: `batch` rows of `tokens_per_row` tokens each.
//
// The offsets are built on the device from the two sizes.  When the batch has fewer (row, head)
// chains than half the SMs and the rows are long, every row is cut into segments of whole chunks
// that are walked in parallel, exactly as the ranks of a context-parallel chain would:
//   pass A  every segment from a zero state (outputs, b = its leaving state), and on further CTAs the
//           segment transition M together with the number of chunks after which it is exactly zero;
//   chain   h_in(s + 1) = M_s h_in(s) + b_s along each row (fp32, tiny);
//   pass B  every segment again with its true entering state, over the leading chunks that state
//           can still reach (all of them when the gates never forget completely).
// With gates that forget within a few chunks the serial walk shrinks by the number of segments;
// with gates that never forget it costs about what the unsegmented walk costs.  The results agree
// with the unsegmented walk to fp32 resolution of the state, not bit for bit.
// ------------------------------------------------------------------------------------------------
namespace kda {

int launch_state_affine(const float* M, const float* hin, const float* b, float* hout, int groups,
                        int group, int64_t in_stride, int64_t out_stride, int K, int V, cudaStream_t s);

static int g_row_segments = 0;   // 0 = choose; otherwise the forced number of segments per row (tests, tuning)

struct DensePlan {
  int segs;         // segments per row (1 = plain walk)
  int seg_chunks;   // chunks per segment (the last one of a row may be shorter)
  int row_chunks;
  int64_t count;    // batch * segs
};

static DensePlan plan_dense(int batch, int64_t tokens_per_row, int heads) {
  DensePlan pl;
  pl.row_chunks = (int)((tokens_per_row + kChunk - 1) / kChunk);
  int segs = 1;
  if (g_row_segments > 0) {
    segs = g_row_segments;
  } else {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t chains = (int64_t)batch * heads;
    if (chains * 2 <= sms) segs = (int)(sms / chains < 8 ? sms / chains : 8);
    if (segs > pl.row_chunks / 64) segs = pl.row_chunks / 64;     // at least 64 chunks per segment
  }
  if (segs > pl.row_chunks) segs = pl.row_chunks;
  if (segs < 1) segs = 1;
  pl.seg_chunks = (pl.row_chunks + segs - 1) / segs;
  pl.segs = (pl.row_chunks + pl.seg_chunks - 1) / pl.seg_chunks;
  pl.count = (int64_t)batch * pl.segs;
  return pl;
}

// sequence i = (row i / segs, segment i % segs)
__global__ void dense_offsets_kernel(int32_t* cu, int32_t* co, int count, int segs, int tokens_per_row,
                                     int row_chunks, int seg_chunks) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > count) return;
  const int row = i / segs, s = i % segs;
  const int chunks = min(s * seg_chunks, row_chunks);
  cu[i] = row * tokens_per_row + min(chunks * kChunk, tokens_per_row);
  co[i] = row * row_chunks + chunks;
}

static int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

struct DenseScratch {   // byte offsets from the start of the scratch region
  int64_t cu, co, limit, b, trans, hin, total;
};
static DenseScratch dense_scratch(int64_t count, int heads) {
  DenseScratch d;
  int64_t at = 0;
  d.cu = at; at = align256(at + (count + 1) * 4);
  d.co = at; at = align256(at + (count + 1) * 4);
  d.limit = at; at = align256(at + count * heads * 4);
  const int64_t states = count * heads * (int64_t)D * D * 4;
  d.b = at; at += states;
  d.trans = at; at += states;
  d.hin = at; at += states;
  d.total = at;
  return d;
}

}  // namespace kda

extern "C" int kda_set_row_segments(int segments) {
  if (segments < 0 || segments > 64) return KDA_ERR_ARG;
  kda::g_row_segments = segments;
  return KDA_OK;
}

extern "C" int64_t kda_chunk_fwd_dense_workspace_bytes(int batch, int64_t tokens_per_row, int heads,
                                                       int keep) {
  if (batch < 1 || tokens_per_row < 1 || heads < 1) return 0;
  const int64_t total = (int64_t)batch * tokens_per_row;
  const kda::DensePlan pl = kda::plan_dense(batch, tokens_per_row, heads);
  const int64_t base = keep ? kda_chunk_bwd_workspace_bytes(total, heads, (int64_t)batch * pl.row_chunks)
                            : kda_chunk_fwd_workspace_bytes(total, heads);
  // the plan may change with kda_set_row_segments between this call and the launch: size for the
  // largest scratch either can ask for (segments only matter through count = batch * segs)
  const int64_t worst = (int64_t)batch * (pl.segs > 8 ? pl.segs : 8);
  return kda::align256(base) + kda::dense_scratch(worst, heads).total;
}

static int chunk_fwd_dense_impl(bool keep, const void* q, const void* k, const void* v,
                                const float* cum_gate, const float* beta, const float* initial_state,
                                float* final_state, void* out, void* aqk, void* akk, int batch,
                                int64_t tokens_per_row, int heads, int key_dim, int value_dim,
                                void* workspace, int64_t workspace_bytes, void* stream) {
  if (!q || !k || !v || !cum_gate || !beta || !out || !aqk || !akk || !workspace) return KDA_ERR_ARG;
  if (key_dim != 128 || value_dim != 128) return KDA_ERR_UNSUPPORTED;
  if (batch < 1 || heads < 1 || tokens_per_row < 1) return KDA_ERR_ARG;
  const int64_t total = (int64_t)batch * tokens_per_row;
  if (total > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  const kda::DensePlan pl = kda::plan_dense(batch, tokens_per_row, heads);
  if (pl.count * heads * 8 > 0x7fffffffLL) return KDA_ERR_UNSUPPORTED;
  const int chunks = batch * pl.row_chunks;
  const int64_t base = kda::align256(keep ? kda_chunk_bwd_workspace_bytes(total, heads, chunks)
                                          : kda_chunk_fwd_workspace_bytes(total, heads));
  const kda::DenseScratch sc = kda::dense_scratch(pl.count, heads);
  if (workspace_bytes < base + sc.total || ((uintptr_t)workspace & 15) != 0) return KDA_ERR_ARG;
  unsigned char* scratch = reinterpret_cast<unsigned char*>(workspace) + base;
  int32_t* cu = reinterpret_cast<int32_t*>(scratch + sc.cu);
  int32_t* co = reinterpret_cast<int32_t*>(scratch + sc.co);
  cudaStream_t s = (cudaStream_t)stream;
  const int count = (int)pl.count;
  kda::dense_offsets_kernel<<<(count + 256) / 256, 256, 0, s>>>(cu, co, count, pl.segs, (int)tokens_per_row,
                                                              pl.row_chunks, pl.seg_chunks);
  if (cudaGetLastError() != cudaSuccess) return KDA_ERR_LAUNCH;

  kda::ChunkParams p{};
  const int64_t nd = total * heads * 128;
  bf16* ws = reinterpret_cast<bf16*>(workspace);
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.g = cum_gate; p.beta = beta;
  p.aqk = (bf16*)aqk; p.akk = (bf16*)akk;
  p.w = ws; p.u = ws + nd; p.kg = ws + 2 * nd; p.qg = ws + 3 * nd;
  p.o = (bf16*)out;
  p.vnew_out = keep ? ws + 4 * nd : nullptr;
  p.h_out = keep ? ws + 6 * nd : nullptr;
  p.chunks = chunks;
  p.cu_seqlens = cu; p.chunk_offsets = co; p.nseq = count; p.H = heads;
  p.scale = 0.08838834764831845f;
  p.tokens = total;
  int rc = kda::launch_prepare(p, chunks, s);
  if (rc) return rc;
  if (pl.segs == 1) {
    p.h0 = initial_state; p.ht = final_state;
    return kda::launch_state_fwd(p, s);
  }
  // ---- pass A: zero-state walk of every segment + transitions with their measured reach
  float* b = reinterpret_cast<float*>(scratch + sc.b);
  float* trans = reinterpret_cast<float*>(scratch + sc.trans);
  float* hin = reinterpret_cast<float*>(scratch + sc.hin);
  int32_t* limit = reinterpret_cast<int32_t*>(scratch + sc.limit);
  if (cudaMemsetAsync(limit, 0, (size_t)count * heads * 4, s) != cudaSuccess) return KDA_ERR_LAUNCH;
  p.h0 = nullptr; p.ht = b; p.trans_out = trans; p.limit_out = limit;
  rc = kda::launch_state_fwd(p, s);
  if (rc) return rc;
  // ---- chain along each row: h_in(0) = the row's initial state, h_in(s + 1) = M_s h_in(s) + b_s
  const size_t row_bytes = (size_t)heads * 128 * 128 * 4;
  cudaError_t e = initial_state
      ? cudaMemcpy2DAsync(hin, row_bytes * pl.segs, initial_state, row_bytes, row_bytes, batch,
                          cudaMemcpyDeviceToDevice, s)
      : cudaMemset2DAsync(hin, row_bytes * pl.segs, 0, row_bytes, batch, s);
  if (e != cudaSuccess) return KDA_ERR_LAUNCH;
  const int64_t per_seg = (int64_t)heads * 128 * 128;
  for (int sg = 0; sg + 1 < pl.segs; ++sg) {
    rc = kda::launch_state_affine(trans + sg * per_seg, hin + sg * per_seg, b + sg * per_seg,
                                  hin + (sg + 1) * per_seg, batch, heads, (int64_t)pl.segs * heads,
                                  (int64_t)pl.segs * heads, 128, 128, s);
    if (rc) return rc;
  }
  if (final_state) {
    const int last = pl.segs - 1;
    rc = kda::launch_state_affine(trans + last * per_seg, hin + last * per_seg, b + last * per_seg,
                                  final_state, batch, heads, (int64_t)pl.segs * heads, heads, 128, 128, s);
    if (rc) return rc;
  }
  // ---- pass B: the leading chunks of every segment with its true entering state
  p.h0 = hin; p.ht = nullptr; p.trans_out = nullptr; p.limit_out = nullptr; p.limit_in = limit;
  return kda::launch_state_fwd(p, s);
}

extern "C" int kda_chunk_fwd_dense(const void* q, const void* k, const void* v, const float* cum_gate,
                                   const float* beta, const float* initial_state, float* final_state,
                                   void* out, void* aqk, void* akk, int batch, int64_t tokens_per_row,
                                   int heads, int key_dim, int value_dim, void* workspace,
                                   int64_t workspace_bytes, void* stream) {
  return chunk_fwd_dense_impl(false, q, k, v, cum_gate, beta, initial_state, final_state, out, aqk, akk,
                              batch, tokens_per_row, heads, key_dim, value_dim, workspace,
                              workspace_bytes, stream);
}

extern "C" int kda_chunk_fwd_dense_save(const void* q, const void* k, const void* v,
                                        const float* cum_gate, const float* beta,
                                        const float* initial_state, float* final_state, void* out,
                                        void* aqk, void* akk, int batch, int64_t tokens_per_row,
                                        int heads, int key_dim, int value_dim, void* saved,
                                        int64_t saved_bytes, void* stream) {
  return chunk_fwd_dense_impl(true, q, k, v, cum_gate, beta, initial_state, final_state, out, aqk, akk,
                              batch, tokens_per_row, heads, key_dim, value_dim, saved, saved_bytes,
                              stream);
}

// ------------------------------------------------------------------------------------------------
// Chunked forward for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc: a serving engine that has handed every free
// byte of the device to its own paged pool, or a plugin running under a runtime that forbids
// allocation once the model is loaded.  For them the w/u/kg/qg scratch of the forward lives in the
// file-scope device array below instead of a caller workspace.  CUDA loads device code lazily, so
// a GPU starts to hold the array (KDA_NOALLOC_SCRATCH_BYTES, until the process exits) when the first
// call on it looks the array's address up, not when the library is opened: that first call belongs
// in the host's start-up phase, before its own pool claims the rest of the device.
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
    if (cudaGetSymbolAddress(&scratch, kda::g_noalloc_scratch) != cudaSuccess || !scratch) {
      cudaGetLastError();   // leave no stale error behind for the next entry point's launch check
      return KDA_ERR_LAUNCH;
    }
    kda::g_noalloc_ptr[dev] = scratch;
  }
  // Nothing in the scratch has to start at zero: every row a kernel reads was written earlier in
  // the same call, rows past a sequence tail are masked on load.
  return kda_chunk_fwd(q, k, v, cum_gate, beta, initial_state, final_state, out, aqk, akk,
                       cu_seqlens, chunk_offsets, nseq, tokens, heads, key_dim, value_dim,
                       num_chunks, scratch, need, stream);
}
