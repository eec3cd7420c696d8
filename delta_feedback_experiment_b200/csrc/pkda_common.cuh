// Shared device helpers for the PKDA kernels (sm_100a).
//
// Layout conventions used by every kernel in this directory:
//   * activations are token-major: x[token][head][channel], channel contiguous,
//     with tokens of all rows / packed sequences on one flat axis;
//   * a "sequence" n owns tokens [bos, bos+len) and chunks [chunk0, chunk0+nchunks)
//     of 64 tokens; dense input has bos = n*T, packed input reads cu_seqlens;
//   * recurrent states are key-major fp32: S[n][head][k][v], A[n][head][k].
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pkda_b200.h"


namespace pkda {

constexpr int kChunk = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------- geometry
struct Geo {
  int n_seqs;
  int seq_len;       // dense: T; packed: 0
  int total_tokens;
  int heads;
  int chunks_per_seq;  // dense only
  int total_chunks;    // dense: exact; packed: upper bound
  const int* cu_seqlens;     // packed only (device)
  const int* chunk_offsets;  // packed only (device, n_seqs+1)
};

struct SeqInfo {
  int bos;
  int len;
  int chunk0;
  int nchunks;
};

__device__ __forceinline__ SeqInfo seq_info(const Geo& g, int n) {
  SeqInfo s;
  if (g.cu_seqlens) {
    s.bos = g.cu_seqlens[n];
    s.len = g.cu_seqlens[n + 1] - s.bos;
    s.chunk0 = g.chunk_offsets ? g.chunk_offsets[n] : 0;
    s.nchunks = (s.len + kChunk - 1) / kChunk;
  } else {
    s.bos = n * g.seq_len;
    s.len = g.seq_len;
    s.chunk0 = n * g.chunks_per_seq;
    s.nchunks = g.chunks_per_seq;
  }
  return s;
}

// Maps a global chunk index to (sequence, first token, valid tokens).  Returns
// false for indices past the last real chunk (packed grids are sized by an
// upper bound).
__device__ __forceinline__ bool chunk_lookup(const Geo& g, int c, int& n, int& tok0, int& valid) {
  if (g.cu_seqlens) {
    if (c >= g.chunk_offsets[g.n_seqs]) return false;
    int lo = 0, hi = g.n_seqs - 1;
    while (lo < hi) {  // last n with chunk_offsets[n] <= c
      int mid = (lo + hi + 1) >> 1;
      if (g.chunk_offsets[mid] <= c) lo = mid; else hi = mid - 1;
    }
    n = lo;
    int local = c - g.chunk_offsets[n];
    int bos = g.cu_seqlens[n];
    int len = g.cu_seqlens[n + 1] - bos;
    tok0 = bos + local * kChunk;
    valid = min(kChunk, len - local * kChunk);
    return true;
  }
  if (c >= g.total_chunks) return false;
  n = c / g.chunks_per_seq;
  int local = c - n * g.chunks_per_seq;
  tok0 = n * g.seq_len + local * kChunk;
  valid = min(kChunk, g.seq_len - local * kChunk);
  return true;
}

// ---------------------------------------------------------------- scalar math
__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16(x); }

// softplus(x) = max(x,0) + log(1 + exp(-|x|)); accurate variant for the fp32 path.
__device__ __forceinline__ float softplus_acc(float x) {
  return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
}
__device__ __forceinline__ float softplus_fast(float x) {
  return fmaxf(x, 0.f) + __logf(1.f + __expf(-fabsf(x)));
}
__device__ __forceinline__ float sigmoid_fast(float x) { return 1.f / (1.f + __expf(-x)); }

// Write-key factor of the diagonal preconditioner:
//   dev = log(A + eps) - centre;  B = exp(-ln(x) * dev / (1 + |dev|)).
__device__ __forceinline__ float precond_factor(float A, float eps, float centre, float ln_x) {
  float dev = logf(A + eps) - centre;
  return expf(-ln_x * dev / (1.f + fabsf(dev)));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

// ---------------------------------------------------------------- warp MMA (bf16, fp32 accumulate)
// Row stride padding (in bf16 elements) that makes 8 consecutive rows of an
// ldmatrix land on distinct 16-byte bank groups.
constexpr int kPad = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fragment (16 x 16) of the logical matrix A[m][k].
//   kATrans = false: smem holds A as [m][k] (k contiguous), element (m,k) at base[m*ld + k]
//   kATrans = true : smem holds A as [k][m] (m contiguous), element (m,k) at base[k*ld + m]
template <bool kATrans>
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const bf16* base, int ld, int m0, int k0) {
  const int lane = threadIdx.x & 31;
  if (!kATrans) {
    // matrices: (m0..+7,k0..+7) (m0+8..,k0..) (m0..,k0+8..) (m0+8..,k0+8..)
    const bf16* p = base + (m0 + (lane & 15)) * ld + k0 + ((lane >> 4) << 3);
    ldsm_x4(a, smem_u32(p));
  } else {
    // stored rows are k; matrices: (k0..+7, m0..+7) (k0.., m0+8..) (k0+8.., m0..) (k0+8.., m0+8..)
    const bf16* p = base + (k0 + (lane & 7) + ((lane >> 4) << 3)) * ld + m0 + (((lane >> 3) & 1) << 3);
    ldsm_x4_t(a, smem_u32(p));
  }
}

// Two B fragments (k16 x n8 each, n0 and n0+8) of the logical matrix B[k][n].
//   kBKN = false: smem holds B as [n][k] (k contiguous), element (k,n) at base[n*ld + k]
//   kBKN = true : smem holds B as [k][n] (n contiguous), element (k,n) at base[k*ld + n]
// r[0],r[1] = fragment for n0..n0+7, r[2],r[3] = fragment for n0+8..n0+15.
template <bool kBKN>
__device__ __forceinline__ void load_b_frag2(uint32_t (&r)[4], const bf16* base, int ld, int k0, int n0) {
  const int lane = threadIdx.x & 31;
  if (!kBKN) {
    // matrices: (n0..+7,k0..+7) (n0..+7,k0+8..) (n0+8..,k0..) (n0+8..,k0+8..)
    const bf16* p = base + (n0 + (lane & 7) + ((lane >> 4) << 3)) * ld + k0 + (((lane >> 3) & 1) << 3);
    ldsm_x4(r, smem_u32(p));
  } else {
    // matrices: (k0..+7,n0..+7) (k0+8..,n0..+7) (k0..+7,n0+8..) (k0+8..,n0+8..)
    const bf16* p = base + (k0 + (lane & 7) + (((lane >> 3) & 1) << 3)) * ld + n0 + ((lane >> 4) << 3);
    ldsm_x4_t(r, smem_u32(p));
  }
}

// acc[mt][nt][4] += A[m0 + 16*mt .., kbeg..kend) * B[kbeg..kend, n0 + 8*nt ..)
// for one warp; kNT must be even.  Accumulator element mapping (g = lane/4,
// t = lane%4): [0],[1] -> row g, cols 2t,2t+1; [2],[3] -> row g+8.
template <int kMT, int kNT, bool kATrans, bool kBKN>
__device__ __forceinline__ void warp_gemm(float (&acc)[kMT][kNT][4], const bf16* A, int lda, int m0,
                                          const bf16* B, int ldb, int n0, int kbeg, int kend) {
  static_assert(kNT % 2 == 0, "n tiles come in pairs");
#pragma unroll 1
  for (int k0 = kbeg; k0 < kend; k0 += 16) {
    uint32_t a[kMT][4];
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt) load_a_frag<kATrans>(a[mt], A, lda, m0 + 16 * mt, k0);
#pragma unroll
    for (int np = 0; np < kNT / 2; ++np) {
      uint32_t b[4];
      load_b_frag2<kBKN>(b, B, ldb, k0, n0 + 16 * np);
#pragma unroll
      for (int mt = 0; mt < kMT; ++mt) {
        mma_bf16(acc[mt][2 * np], a[mt], b[0], b[1]);
        mma_bf16(acc[mt][2 * np + 1], a[mt], b[2], b[3]);
      }
    }
  }
}

template <int kMT, int kNT>
__device__ __forceinline__ void zero_acc(float (&acc)[kMT][kNT][4]) {
#pragma unroll
  for (int i = 0; i < kMT; ++i)
#pragma unroll
    for (int j = 0; j < kNT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
}

// ---------------------------------------------------------------- async copies
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  uint32_t s = smem_u32(smem);
  int bytes = pred ? 16 : 0;  // src-size 0 => zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem, bool pred) {
  uint32_t s = smem_u32(smem);
  int bytes = pred ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" :: "r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" :: "n"(N));
}

// Copies a [rows x cols] bf16 tile (cols a multiple of 8) from global memory
// with row stride gld (elements) into shared memory with row stride sld; rows
// >= valid_rows are zero filled.  All threads of the CTA take part.
__device__ __forceinline__ void tile_load_async(bf16* s, int sld, const bf16* g, long gld, int rows,
                                                int cols, int valid_rows, int nthreads) {
  const int cpr = cols >> 3;  // 16-byte pieces per row
  for (int i = threadIdx.x; i < rows * cpr; i += nthreads) {
    int r = i / cpr, c = (i - r * cpr) << 3;
    bool ok = r < valid_rows;
    cp_async16(s + r * sld + c, g + (ok ? (long)r * gld + c : 0), ok);
  }
}

}  // namespace pkda
