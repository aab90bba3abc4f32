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
                                                           float* __restrict__ hout, int K, int V,
                                                           int group, int64_t in_stride,
                                                           int64_t out_stride) {
  __shared__ float sA[16][64 + 4];
  __shared__ float sB[16][64 + 4];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  // matrix blockIdx.z = (g, i) with i < group: inputs at g * in_stride + i, output at g * out_stride + i
  const int64_t n = (int64_t)(blockIdx.z / group) * in_stride + blockIdx.z % group;
  const int64_t no = (int64_t)(blockIdx.z / group) * out_stride + blockIdx.z % group;
  const float* Mn = M + n * K * K;
  const float* Hn = hin + n * K * V;
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
    const int64_t e = (int64_t)(r0 + ty * 4 + i) * V + c0 + tx * 4;
    float4 bv = *reinterpret_cast<const float4*>(b + n * K * V + e);
    *reinterpret_cast<float4*>(hout + no * K * V + e) =
        make_float4(acc[i][0] + bv.x, acc[i][1] + bv.y, acc[i][2] + bv.z, acc[i][3] + bv.w);
  }
}

// `groups` x `group` products; the matrices of group g start at index g * in_stride (inputs) and
// g * out_stride (output).
int launch_state_affine(const float* M, const float* hin, const float* b, float* hout, int groups,
                        int group, int64_t in_stride, int64_t out_stride, int K, int V, cudaStream_t s) {
  if (groups <= 0 || group <= 0) return KDA_OK;
  dim3 grid(V / 64, K / 64, groups * group);
  state_affine_kernel<<<grid, 256, 0, s>>>(M, hin, b, hout, K, V, group, in_stride, out_stride);
  return cudaGetLastError() == cudaSuccess ? KDA_OK : KDA_ERR_LAUNCH;
}

}  // namespace kda

extern "C" int kda_state_affine(const float* transition, const float* h_in, const float* b,
                                float* h_out, int count, int key_dim, int value_dim, void* stream) {
  if (!transition || !h_in || !b || !h_out || count < 0) return KDA_ERR_ARG;
  if (key_dim % 64 || value_dim % 64 || key_dim <= 0 || value_dim <= 0) return KDA_ERR_UNSUPPORTED;
  if (count == 0) return KDA_OK;
  return kda::launch_state_affine(transition, h_in, b, h_out, 1, count, 0, 0, key_dim, value_dim,
                                  (cudaStream_t)stream);
}
