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
};

__device__ __forceinline__ ChunkWork locate_chunk(const int32_t* __restrict__ cu_seqlens,
                                                  const int32_t* __restrict__ chunk_offsets,
                                                  int nseq, int global_chunk) {
  ChunkWork w;
  w.valid = 0;
  w.seq = 0;
  w.local_chunk = 0;
  w.token0 = 0;
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
  return w;
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

// Copy a [rows x COLS] tile of 2-byte elements (row stride `gld` elements in global memory) into
// shared memory with row stride LDS elements; rows >= valid_rows are zero-filled.
template <int ROWS, int COLS, int LDS, int THREADS>
__device__ __forceinline__ void load_tile_b16(bf16* smem, const bf16* gmem, int64_t gld,
                                              int valid_rows, int tid) {
  constexpr int VPR = COLS / 8;  // 16-byte vectors per row
  for (int idx = tid; idx < ROWS * VPR; idx += THREADS) {
    int r = idx / VPR, c = (idx % VPR) * 8;
    bool ok = r < valid_rows;
    const bf16* src = gmem + (ok ? (int64_t)r * gld + c : 0);
    cp_async16(smem + r * LDS + c, src, ok);
  }
}
// Same for fp32 tiles.
template <int ROWS, int COLS, int LDS, int THREADS>
__device__ __forceinline__ void load_tile_f32(float* smem, const float* gmem, int64_t gld,
                                              int valid_rows, int tid) {
  constexpr int VPR = COLS / 4;
  for (int idx = tid; idx < ROWS * VPR; idx += THREADS) {
    int r = idx / VPR, c = (idx % VPR) * 4;
    bool ok = r < valid_rows;
    const float* src = gmem + (ok ? (int64_t)r * gld + c : 0);
    cp_async16(smem + r * LDS + c, src, ok);
  }
}
// Coalesced copy of a [rows x COLS] 2-byte tile from shared to global memory (rows < valid_rows).
template <int ROWS, int COLS, int LDS, int THREADS>
__device__ __forceinline__ void store_tile_b16(bf16* gmem, int64_t gld, const bf16* smem,
                                               int valid_rows, int tid) {
  constexpr int VPR = COLS / 8;
  for (int idx = tid; idx < ROWS * VPR; idx += THREADS) {
    int r = idx / VPR, c = (idx % VPR) * 8;
    if (r < valid_rows)
      *reinterpret_cast<uint4*>(gmem + (int64_t)r * gld + c) =
          *reinterpret_cast<const uint4*>(smem + r * LDS + c);
  }
}

// ------------------------------------------------------------------------------------------
// warp-level bf16 tensor-core tiles (mma.sync m16n8k16, fp32 accumulate) fed by ldmatrix
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  uint32_t a = smem_u32(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a) : "memory");
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  uint32_t a = smem_u32(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fragment (16 x 16) of the logical matrix A[m][k].
//   AT == false: shared memory holds A[m][k] with k contiguous (row stride lda)
//   AT == true : shared memory holds A^T, i.e. element (m, k) lives at smem[k * lda + m]
template <bool AT>
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const bf16* A, int lda, int m0,
                                            int k0, int lane) {
  if (!AT) {
    ldsm_x4(a, A + (m0 + (lane & 15)) * lda + k0 + (lane >> 4) * 8);
  } else {
    ldsm_x4_t(a, A + (k0 + (lane & 7) + ((lane >> 4) & 1) * 8) * lda + m0 + ((lane >> 3) & 1) * 8);
  }
}
// B fragments for two adjacent n-tiles (16 k x 16 n) of the logical matrix B[k][n].
//   BT == false: shared memory holds element (k, n) at smem[n * ldb + k]  (k contiguous)
//   BT == true : shared memory holds element (k, n) at smem[k * ldb + n]  (n contiguous)
// b[0], b[1] feed n-tile n0..n0+7; b[2], b[3] feed n-tile n0+8..n0+15.
template <bool BT>
__device__ __forceinline__ void load_b_frag(uint32_t (&b)[4], const bf16* B, int ldb, int k0,
                                            int n0, int lane) {
  if (!BT) {
    ldsm_x4(b, B + (n0 + (lane & 7) + ((lane >> 4) & 1) * 8) * ldb + k0 + ((lane >> 3) & 1) * 8);
  } else {
    ldsm_x4_t(b, B + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldb + n0 + ((lane >> 4) & 1) * 8);
  }
}

// acc[mt][nt][4] += A[m0 + 16 mt .., ka0 ..] * B[kb0 .., n0 + 8 nt ..] over KS k-steps of 16.
// NEG negates the A operand (flips the sign bits of the packed bf16 pairs).
template <int MT, int NT2, bool AT, bool BT, bool NEG = false>
__device__ __forceinline__ void warp_gemm(float (&acc)[MT][NT2 * 2][4], const bf16* A, int lda,
                                          int m0, int ka0, const bf16* B, int ldb, int kb0, int n0,
                                          int ksteps, int lane) {
  for (int ks = 0; ks < ksteps; ++ks) {
    uint32_t a[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      load_a_frag<AT>(a[mt], A, lda, m0 + 16 * mt, ka0 + 16 * ks, lane);
      if (NEG) {
#pragma unroll
        for (int i = 0; i < 4; ++i) a[mt][i] ^= 0x80008000u;
      }
    }
#pragma unroll
    for (int np = 0; np < NT2; ++np) {
      uint32_t b[4];
      load_b_frag<BT>(b, B, ldb, kb0 + 16 * ks, n0 + 16 * np, lane);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma16816(acc[mt][2 * np], a[mt], b[0], b[1]);
        mma16816(acc[mt][2 * np + 1], a[mt], b[2], b[3]);
      }
    }
  }
}

template <int MT, int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[MT][NT][4]) {
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
}

// Accumulator element (mt, nt, i) of a warp tile anchored at (m0, n0) sits at
//   row = m0 + 16 mt + (lane >> 2) + 8 (i >> 1),  col = n0 + 8 nt + 2 (lane & 3) + (i & 1).
__device__ __forceinline__ int acc_row(int m0, int mt, int i, int lane) {
  return m0 + 16 * mt + (lane >> 2) + 8 * (i >> 1);
}
__device__ __forceinline__ int acc_col(int n0, int nt, int i, int lane) {
  return n0 + 8 * nt + 2 * (lane & 3) + (i & 1);
}

}  // namespace kda
