// Shared device helpers for the KDA kernels (sm_100a).
//
// Conventions used by every kernel in this directory:
//   * gates are log2 decays, a = 2^g (reference: attn_gym/linear/kda/naive.py:26-27);
//   * token-major activations [N, H, D] with D contiguous, state [seq, H, K, V] fp32;
//   * packed sequences are described by int32 cu_seqlens[nseq+1] and chunk_offsets[nseq+1]
//     (exclusive prefix of ceil(len/64), reference: attn_gym/linear/kda/chunk_schedule.py:49-91);
//   * every global index is computed in 64-bit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kda_b200.h"

namespace kda {

constexpr int kChunk = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// ------------------------------------------------------------------------------------------
// dtype-erased scalar access (codes: KDA_F32 / KDA_BF16 / KDA_F16)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
  if (dtype == KDA_BF16) return __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
  if (dtype == KDA_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}
// The same access split in two, for software prefetch: the raw bits are loaded now and turned into
// a float only when they are needed, so the warp does not stall on the load in between.
__device__ __forceinline__ uint32_t load_raw(const void* p, int dtype, int64_t i) {
  if (dtype == KDA_F32) return reinterpret_cast<const uint32_t*>(p)[i];
  return reinterpret_cast<const unsigned short*>(p)[i];
}
__device__ __forceinline__ float raw_to_float(uint32_t raw, int dtype) {
  if (dtype == KDA_BF16) return __uint_as_float(raw << 16);
  if (dtype == KDA_F16) return __half2float(__ushort_as_half((unsigned short)raw));
  return __uint_as_float(raw);
}
__device__ __forceinline__ void store_from_float(void* p, int dtype, int64_t i, float x) {
  if (dtype == KDA_BF16) reinterpret_cast<bf16*>(p)[i] = __float2bfloat16(x);
  else if (dtype == KDA_F16) reinterpret_cast<__half*>(p)[i] = __float2half(x);
  else reinterpret_cast<float*>(p)[i] = x;
}
__host__ __device__ __forceinline__ int dtype_size(int dtype) { return dtype == KDA_F32 ? 4 : 2; }

// 2^x on the SFU (ex2.approx, flush-to-zero): the gated operands are rounded to bf16 anyway
__device__ __forceinline__ float fexp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  bf162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  bf162 v = *reinterpret_cast<bf162*>(&u);
  return __bfloat1622float2(v);
}

// ------------------------------------------------------------------------------------------
// packed-sequence routing: global chunk -> (sequence, first token, valid rows)
// reference: attn_gym/linear/kda/chunk_scheduler.py:341 (upper_bound over chunk_offsets)
// ------------------------------------------------------------------------------------------
struct ChunkWork {
  int seq;
  int local_chunk;
  int64_t token0;  // first token of the chunk in the packed buffer
  int valid;       // rows of the chunk that hold tokens (1..64); 0 = inactive capacity slot
  int64_t seq_end; // end of the chunk's sequence in the packed buffer
};

// Device-side check of the offsets a chunk was located with: the chunks of a sequence that does not
// lie inside the packed buffer (inconsistent cu_seqlens / chunk_offsets) are skipped by the kernels and
// reported through their error word (code kOffsetsOutOfRange) instead of being read or written.  The
// reference asserts its offsets on the device in its scheduler kernel (kda/chunk_scheduler.py:278-293); the
// host-side validation cannot see the values without a device synchronisation.
constexpr int kOffsetsOutOfRange = 9;

__device__ __forceinline__ ChunkWork locate_chunk(const int32_t* __restrict__ cu_seqlens,
                                                  const int32_t* __restrict__ chunk_offsets,
                                                  int nseq, int global_chunk) {
  ChunkWork w;
  w.valid = 0;
  w.seq = 0;
  w.local_chunk = 0;
  w.token0 = 0;
  w.seq_end = 0;
  if (global_chunk >= chunk_offsets[nseq]) return w;
  // upper_bound(chunk_offsets, global_chunk) - 1; repeated offsets (empty sequences) are skipped
  int lo = 0, hi = nseq;  // answer in [0, nseq)
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (chunk_offsets[mid] <= global_chunk) lo = mid; else hi = mid - 1;
  }
  w.seq = lo;
  w.local_chunk = global_chunk - chunk_offsets[lo];
  int64_t bos = cu_seqlens[lo], eos = cu_seqlens[lo + 1];
  w.token0 = bos + (int64_t)w.local_chunk * kChunk;
  int64_t rem = eos - w.token0;
  w.valid = rem >= kChunk ? kChunk : (rem > 0 ? (int)rem : 0);
  w.seq_end = eos;
  return w;
}

__device__ __forceinline__ bool chunk_in_range(const ChunkWork& w, int64_t tokens) {
  return w.token0 >= 0 && w.seq_end <= tokens && w.token0 + w.valid <= w.seq_end;
}

// ------------------------------------------------------------------------------------------
// cp.async (16-byte, zero-fill when !pred)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  uint32_t s = smem_u32(smem);
  int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// eight 16-bit values <-> floats
__device__ __forceinline__ void raw8_to_float(const uint4& r, int dt, float (&x)[8]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dt == KDA_BF16) { float2 a = unpack_bf16(w[i]); x[2 * i] = a.x; x[2 * i + 1] = a.y; }
    else { __half2 h = *reinterpret_cast<const __half2*>(&w[i]); x[2 * i] = __low2float(h); x[2 * i + 1] = __high2float(h); }
  }
}
__device__ __forceinline__ uint4 float8_to_raw(const float (&x)[8], int dt) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dt == KDA_BF16) w[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
    else { __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]); w[i] = *reinterpret_cast<uint32_t*>(&h); }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

}  // namespace kda
