// Context-parallel boundary-state composition: h_out = M h_in + b per (sequence, head).
//
// A slice of a long sequence maps its entering state affinely to its leaving state; M [K, K] is the
// slice transition (kda_chunk_transition) and b [K, V] the leaving state for a zero entering state.
// Only h crosses GPUs; this kernel applies the local correction.  fp32 throughout: the product is
// tiny (K = V = 128 per head) and its rounding would otherwise accumulate along the rank chain.
// The reference has no context parallelism (docs/linear.md:220-222).
#include "kda_common.cuh"

namespace kda {

// 64 x 64 output tile per CTA, 4 x 4 per thread, K stepped in slabs of 16 through shared memory
__global__ void __launch_bounds__(256) state_affine_kernel(const float* __restrict__ M,
                                                           const float* __restrict__ hin,
                                                           const float* __restrict__ b,
                                                           float* __restrict__ hout, int K, int V) {
  __shared__ float sA[16][64 + 4];
  __shared__ float sB[16][64 + 4];
  const int n = blockIdx.z, r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const float* Mn = M + (int64_t)n * K * K;
  const float* Hn = hin + (int64_t)n * K * V;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int idx = threadIdx.x; idx < 16 * 64; idx += 256) {
      int kk = idx & 15, rr = idx >> 4;      // M[r0+rr][k0+kk], transposed into sA[kk][rr]
      sA[kk][rr] = Mn[(int64_t)(r0 + rr) * K + k0 + kk];
      int cc = idx & 63, k2 = idx >> 6;
      sB[k2][cc] = Hn[(int64_t)(k0 + k2) * V + c0 + cc];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = sB[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * bb[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t o = (int64_t)n * K * V + (int64_t)(r0 + ty * 4 + i) * V + c0 + tx * 4;
    float4 bv = *reinterpret_cast<const float4*>(b + o);
    *reinterpret_cast<float4*>(hout + o) =
        make_float4(acc[i][0] + bv.x, acc[i][1] + bv.y, acc[i][2] + bv.z, acc[i][3] + bv.w);
  }
}

}  // namespace kda

extern "C" int kda_state_affine(const float* transition, const float* h_in, const float* b,
                                float* h_out, int count, int key_dim, int value_dim, void* stream) {
  if (!transition || !h_in || !b || !h_out || count < 0) return KDA_ERR_ARG;
  if (key_dim % 64 || value_dim % 64 || key_dim <= 0 || value_dim <= 0) return KDA_ERR_UNSUPPORTED;
  if (count == 0) return KDA_OK;
  dim3 grid(value_dim / 64, key_dim / 64, count);
  kda::state_affine_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(transition, h_in, b, h_out,
                                                                  key_dim, value_dim);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}
