// Pieces shared by the chunked forward and backward kernels (D = 128, chunk 64).
#pragma once

#include "pkda_common.cuh"
#include "pkda_launch.h"

namespace pkda {

constexpr int kD = 128;                       // head width handled by the chunked kernels
constexpr int kLdD = kD + kPad;               // smem row stride of a [*][128] bf16 tile
constexpr int kLdC = kChunk + kPad;           // smem row stride of a [*][64] bf16 tile
constexpr int kTileBytes = kChunk * kLdD * 2; // one [64][128] bf16 tile

// Level `lvl` (a power of two < 64) pairs row i (bit lvl set) with row j (bit
// lvl clear) of the same 2*lvl block.
__device__ __forceinline__ bool level_pair_ok(int i, int j, int lvl) {
  return (((i ^ j) & ~(2 * lvl - 1)) == 0) && (i & lvl) && !(j & lvl);
}

constexpr int kLdG = kD + 8;                  // smem row stride of a [64][128] fp32 array

// "Direct" pairing: inside a block of b rows (b a power of two) all pairs j < i
// use ONE reference row, the block's first: row factor 2^(G_i - G_ref) <= 1,
// column factor 2^(G_ref - G_j) >= 1.  That is only safe while the decay across a
// b-block stays far inside the fp32 / bf16 exponent range, so each (chunk, head)
// picks the largest b whose worst block decay is below kDirectLimit (log2 units)
// and covers the remaining pairs with hierarchy levels >= b.  lvl == 0 denotes the
// direct level everywhere below.
// With the limit at 112 the column operand kt 2^112 (|kt| <= 1.5 |k|) and the fp32 sums of up to 128
// masked products of that size stay below 2^127, and the row operand k 2^-112 only loses (to the
// flush of denormals) channels with |k| < 2^-14, whose products are below the bf16 rounding of the
// others; chunks of the benchmark's gate distribution (about 75 +- 6 log2 units of decay per 64
// tokens) then practically always form one block.
constexpr float kDirectLimit = 112.f;

__device__ __forceinline__ bool pair_ok(int i, int j, int lvl, int b) {
  if (lvl) return level_pair_ok(i, j, lvl);
  return (((i ^ j) & ~(b - 1)) == 0) && (j < i);
}

// Per-channel worst block decay for b = 2,4,...,64 (dmax[0..5]) from the cumulative
// log2-decay column c of sG.
__device__ __forceinline__ void block_decay_max(const float* sG, int c, float (&dmax)[6]) {
#pragma unroll
  for (int e = 0; e < 6; ++e) {
    const int b = 2 << e;
    float m = 0.f;
    for (int bs = 0; bs < kChunk; bs += b) m = fmaxf(m, sG[bs * kLdG + c] - sG[(bs + b - 1) * kLdG + c]);
    dmax[e] = m;
  }
}

// Largest admissible direct block size given the per-warp maxima (nw warps x 6).
__device__ __forceinline__ int pick_direct_block(const float* sWarpMax, int nw, int cap) {
  int b = 1;
#pragma unroll
  for (int e = 0; e < 6; ++e) {
    float m = 0.f;
    for (int w = 0; w < nw; ++w) m = fmaxf(m, sWarpMax[w * 6 + e]);
    if (m <= kDirectLimit && (2 << e) <= cap) b = 2 << e;
    else break;
  }
  return b;
}

// 2^x by the hardware approximation (flushes denormal results to zero, which is
// what the gating factors want: every argument here is <= 0).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void scale8(uint4& x, const float (&f)[8]) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = unpack_bf16(w[j]);
    w[j] = pack_bf16(v.x * f[2 * j], v.y * f[2 * j + 1]);
  }
}

// Builds the gated operands of one level from the log2-domain cumulative decay
// sG [64][kLdG]: rows with bit lvl set get X * 2^(G_r - G_ref) (into sXq from sQ
// and sXk from sK), the others get Y * 2^(G_ref - G_r) (into sY from sKt), where
// ref is the first row of the upper half of the row's 2*lvl block.  Rows of the
// other kind are left untouched (their products are masked out).  Null
// destinations are skipped.  sFac (optional, fp32 [64][kLdG]) receives the factor
// each row used.  Eight channels per thread and step (128-bit accesses).
__device__ __forceinline__ void stage_level(bf16* sXq, bf16* sXk, bf16* sY, const bf16* sQ, const bf16* sK,
                                            const bf16* sKt, const float* sG, int lvl, int b, int tid,
                                            int nthreads, float* sFac = nullptr) {
  for (int idx = tid; idx < kChunk * kD / 8; idx += nthreads) {
    const int r = idx >> 4, c8 = (idx & 15) << 3;
    const int ref = lvl ? (r & ~(2 * lvl - 1)) + lvl : (r & ~(b - 1));
    const bool upper = lvl ? (r & lvl) != 0 : true;
    const float4 a0 = *reinterpret_cast<const float4*>(sG + r * kLdG + c8);
    const float4 a1 = *reinterpret_cast<const float4*>(sG + r * kLdG + c8 + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(sG + ref * kLdG + c8);
    const float4 b1 = *reinterpret_cast<const float4*>(sG + ref * kLdG + c8 + 4);
    const float sgn = upper ? 1.f : -1.f;
    float f[8];
    f[0] = ex2(sgn * (a0.x - b0.x)); f[1] = ex2(sgn * (a0.y - b0.y));
    f[2] = ex2(sgn * (a0.z - b0.z)); f[3] = ex2(sgn * (a0.w - b0.w));
    f[4] = ex2(sgn * (a1.x - b1.x)); f[5] = ex2(sgn * (a1.y - b1.y));
    f[6] = ex2(sgn * (a1.z - b1.z)); f[7] = ex2(sgn * (a1.w - b1.w));
    if (sFac) {
      *reinterpret_cast<float4*>(sFac + r * kLdG + c8) = make_float4(f[0], f[1], f[2], f[3]);
      *reinterpret_cast<float4*>(sFac + r * kLdG + c8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
    if (upper) {
      if (sXq) {
        uint4 x = *reinterpret_cast<const uint4*>(sQ + r * kLdD + c8);
        scale8(x, f);
        *reinterpret_cast<uint4*>(sXq + r * kLdD + c8) = x;
      }
      if (sXk) {
        uint4 x = *reinterpret_cast<const uint4*>(sK + r * kLdD + c8);
        scale8(x, f);
        *reinterpret_cast<uint4*>(sXk + r * kLdD + c8) = x;
      }
      if (!lvl && sY) {  // direct level: the same row is also a column operand, factor 1/f
        float fi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) fi[j] = __fdividef(1.f, f[j]);
        uint4 x = *reinterpret_cast<const uint4*>(sKt + r * kLdD + c8);
        scale8(x, fi);
        *reinterpret_cast<uint4*>(sY + r * kLdD + c8) = x;
      }
    } else if (sY) {
      uint4 x = *reinterpret_cast<const uint4*>(sKt + r * kLdD + c8);
      scale8(x, f);
      *reinterpret_cast<uint4*>(sY + r * kLdD + c8) = x;
    }
  }
}

// Elementwise part of the decay gate for one chunk, all kNThreads threads: log2-domain
// per-token log-decay  -exp(A_log) log2(e) softplus(raw + bias)  into sG (zero for
// rows past the sequence end).  The cumulative sum over rows follows separately.
// The raw gate of the tile is fetched first (gate_load, at the top of a kernel, so
// that the loads fly while other data is set up) and converted later (gate_apply).
template <int kNThreads>
struct GateRaw {
  static constexpr int kIter = kChunk * kD / 8 / kNThreads;
  static_assert(kIter * kNThreads * 8 == kChunk * kD, "tile must divide evenly");
  uint4 raw[kIter];
};

template <int kNThreads>
__device__ __forceinline__ void gate_load(GateRaw<kNThreads>& gr, const bf16* g_row0, long gld, int valid, int tid) {
#pragma unroll
  for (int it = 0; it < GateRaw<kNThreads>::kIter; ++it) {
    const int idx = tid + it * kNThreads, r = idx >> 4, c8 = (idx & 15) << 3;
    gr.raw[it] = make_uint4(0, 0, 0, 0);
    if (r < valid) gr.raw[it] = *reinterpret_cast<const uint4*>(g_row0 + (size_t)r * gld + c8);
  }
}

template <int kNThreads>
__device__ __forceinline__ void gate_apply(const GateRaw<kNThreads>& gr, float* sG, int valid, const float* bias_h,
                                           float ea2, int tid) {
#pragma unroll
  for (int it = 0; it < GateRaw<kNThreads>::kIter; ++it) {
    const int idx = tid + it * kNThreads, r = idx >> 4, c8 = (idx & 15) << 3;
    float o[8];
    if (r < valid) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&gr.raw[it]);
      const float4 bA = *reinterpret_cast<const float4*>(bias_h + c8);
      const float4 bB = *reinterpret_cast<const float4*>(bias_h + c8 + 4);
      const float bb[8] = {bA.x, bA.y, bA.z, bA.w, bB.x, bB.y, bB.z, bB.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = unpack_bf16(w[j]);
        o[2 * j] = -ea2 * softplus_fast(v.x + bb[2 * j]);
        o[2 * j + 1] = -ea2 * softplus_fast(v.y + bb[2 * j + 1]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = 0.f;
    }
    *reinterpret_cast<float4*>(sG + r * kLdG + c8) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4*>(sG + r * kLdG + c8 + 4) = make_float4(o[4], o[5], o[6], o[7]);
  }
}

template <int kNThreads>
__device__ __forceinline__ void gate_elementwise(float* sG, const bf16* g_row0, long gld, int valid,
                                                 const float* bias_h, float ea2, int tid) {
  GateRaw<kNThreads> gr;
  gate_load(gr, g_row0, gld, valid, tid);
  gate_apply(gr, sG, valid, bias_h, ea2, tid);
}

// In-place cumulative sum over the 64 rows of sG, one channel per thread (tid < 128).
__device__ __forceinline__ void gate_cumsum(float* sG, int c) {
  float run = 0.f;
#pragma unroll 8
  for (int r = 0; r < kChunk; ++r) {
    run += sG[r * kLdG + c];
    sG[r * kLdG + c] = run;
  }
}

// warp_gemm for one m-tile whose A operand is a [64][64] pair-weight matrix
// restricted to the pairs of one level.  With mask = true every A element
// (i, j) that is not a valid pair of `lvl` is zeroed in registers after the
// load; kATrans means the logical A is the transpose (A[m=j][k=i]).
template <int kNT, bool kATrans, bool kBKN>
__device__ __forceinline__ void warp_gemm_lvl(float (&acc)[1][kNT][4], const bf16* A, int lda, int m0,
                                              const bf16* B, int ldb, int n0, int kbeg, int kend, int lvl,
                                              int b, bool mask) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll 1
  for (int k0 = kbeg; k0 < kend; k0 += 16) {
    uint32_t a[4];
    load_a_frag<kATrans>(a, A, lda, m0, k0);
    if (mask) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int m = m0 + g + 8 * (r & 1);
        const int kk = k0 + 2 * t + 8 * (r >> 1);
        const bool ok0 = kATrans ? pair_ok(kk, m, lvl, b) : pair_ok(m, kk, lvl, b);
        const bool ok1 = kATrans ? pair_ok(kk + 1, m, lvl, b) : pair_ok(m, kk + 1, lvl, b);
        a[r] &= (ok0 ? 0x0000ffffu : 0u) | (ok1 ? 0xffff0000u : 0u);
      }
    }
#pragma unroll
    for (int np = 0; np < kNT / 2; ++np) {
      uint32_t bf[4];
      load_b_frag2<kBKN>(bf, B, ldb, k0, n0 + 16 * np);
      mma_bf16(acc[0][2 * np], a, bf[0], bf[1]);
      mma_bf16(acc[0][2 * np + 1], a, bf[2], bf[3]);
    }
  }
}

// One doubling step of the triangular inverse: for every pair of inverted diagonal
// blocks T11, T22 of size N and their coupling block L21, T21 = -T22 (L21 T11).
// Loops run over full N (the blocks' upper triangles are zero) so they unroll.
template <int N>
__device__ __forceinline__ void inverse_merge(const float* sL, float* sT, float* sY2, int ldl, int ldt, int tid,
                                              int nthreads) {
  constexpr int SH = N == 4 ? 2 : (N == 8 ? 3 : (N == 16 ? 4 : 5));
  for (int o = tid; o < 32 * N; o += nthreads) {
    const int pr = o >> (2 * SH), r = (o >> SH) & (N - 1), c = o & (N - 1);
    const int base = pr * 2 * N;
    const float* Lrow = sL + (base + N + r) * ldl + base;
    const float* Tcol = sT + base * ldt + base + c;
    float s = 0.f;
#pragma unroll
    for (int m = 0; m < N; ++m) s += Lrow[m] * Tcol[m * ldt];
    sY2[o] = s;
  }
  __syncthreads();
  for (int o = tid; o < 32 * N; o += nthreads) {
    const int pr = o >> (2 * SH), r = (o >> SH) & (N - 1), c = o & (N - 1);
    const int base = pr * 2 * N;
    const float* Trow = sT + (base + N + r) * ldt + base + N;
    const float* Ycol = sY2 + (pr << (2 * SH)) + c;
    float t = 0.f;
#pragma unroll
    for (int m = 0; m < N; ++m) t -= Trow[m] * Ycol[m << SH];
    sT[(base + N + r) * ldt + base + c] = t;
  }
  __syncthreads();
}

// The same merge on the tensor cores for N = 16 and 32: both products as
// mma.sync m16n8k8 TF32 with every fp32 operand split into a high and a low TF32
// part (three MMAs per step: lo*hi + hi*lo + hi*hi), which keeps fp32-level
// accuracy (the dropped lo*lo term is 2^-22 relative).  One warp per 16 x 8
// output tile; operands come straight from the fp32 arrays in shared memory.
//
// Rounding to TF32 (nearest, ties away from zero: what cvt.rna.tf32.f32 returns for
// finite values and infinities) is an integer add and a mask on the bit pattern; both
// run at full rate, the conversion instruction does not.
__device__ __forceinline__ uint32_t tf32_rna(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }

__device__ __forceinline__ void tf32_split(float x, uint32_t& hi, uint32_t& lo) {
  hi = tf32_rna(x);
  lo = tf32_rna(x - __uint_as_float(hi));
}

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// d[16 x 8] += A[16 x K] B[K x 8] over the k range [kbeg, kend) (multiples of 8),
// A(r, m) = Ap[r * lda + m],  B(m, c) = Bp[m * ldb + c].  The fragment loads of A are
// free of bank conflicts when lda = 4 (mod 8), those of B when ldb = 8 (mod 16); with an
// odd stride (65) every one of them is a 4-way conflict, and the merge is bound by them.
template <int K>
__device__ __forceinline__ void tile_mma_3xtf32(float (&d)[4], const float* Ap, int lda, const float* Bp, int ldb,
                                                int lane, int kbeg = 0, int kend = K) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int k0 = 0; k0 < K; k0 += 8) {
    if (k0 < kbeg || k0 >= kend) continue;
    const float a[4] = {Ap[g * lda + k0 + t], Ap[(g + 8) * lda + k0 + t], Ap[g * lda + k0 + t + 4],
                        Ap[(g + 8) * lda + k0 + t + 4]};
    const float b[2] = {Bp[(k0 + t) * ldb + g], Bp[(k0 + t + 4) * ldb + g]};
    uint32_t ah[4], al[4], bh[2], bl[2];
#pragma unroll
    for (int e = 0; e < 4; ++e) tf32_split(a[e], ah[e], al[e]);
#pragma unroll
    for (int e = 0; e < 2; ++e) tf32_split(b[e], bh[e], bl[e]);
    mma_tf32(d, al, bh);
    mma_tf32(d, ah, bl);
    mma_tf32(d, ah, bh);
  }
}

// kYPad widens the rows of the scratch Y to N + kYPad floats (8 makes the second
// product's B loads conflict-free; the scratch then holds 2 * 16 * 24 or 32 * 40 floats).
// kSkip leaves out the k-steps in which a triangular factor is all zero (the rows of
// T11 above the output tile's columns, the columns of T22 right of the output tile's
// rows): the sums lose only exact zeros.
template <int N, int kYPad, bool kSkip>
__device__ __forceinline__ void inverse_merge_tc(const float* sL, float* sT, float* sY2, int ldl, int ldt, int tid) {
  constexpr int kMT = N / 16, kNT = N / 8, kTiles = (32 / N) * kMT * kNT;  // N = 32: 8 tiles, N = 16: 4 tiles
  constexpr int ldy = N + kYPad;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int pr = warp / (kMT * kNT), mt = (warp / kNT) % kMT, nt = warp % kNT;
  const int base = pr * 2 * N;
  if (warp < kTiles) {  // Y = L21 T11
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    tile_mma_3xtf32<N>(d, sL + (base + N + 16 * mt) * ldl + base, ldl, sT + base * ldt + base + 8 * nt, ldt, lane,
                       kSkip ? 8 * nt : 0, N);
    float* y = sY2 + pr * N * ldy + (16 * mt + g) * ldy + 8 * nt + 2 * t;
    *reinterpret_cast<float2*>(y) = make_float2(d[0], d[1]);
    *reinterpret_cast<float2*>(y + 8 * ldy) = make_float2(d[2], d[3]);
  }
  __syncthreads();
  if (warp < kTiles) {  // T21 = -T22 Y
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    tile_mma_3xtf32<N>(d, sT + (base + N + 16 * mt) * ldt + base + N, ldt, sY2 + pr * N * ldy + 8 * nt, ldy, lane, 0,
                       kSkip ? 16 * mt + 16 : N);
    float* o = sT + (base + N + 16 * mt + g) * ldt + base + 8 * nt + 2 * t;
    o[0] = -d[0];
    o[1] = -d[1];
    o[8 * ldt] = -d[2];
    o[8 * ldt + 1] = -d[3];
  }
  __syncthreads();
}

// T = (I + L)^-1 for a 64 x 64 strictly lower triangular L (fp32; row strides ldl of L
// and ldt of T), all nthreads threads of the CTA (at least 256): 4 x 4 diagonal blocks by
// forward substitution, then four doubling steps, the last two on the tensor cores.  sY2 is
// a scratch of 1024 floats (kYPad = 0) or 1280 (kYPad = 8).  The result does not depend on
// the strides or on kYPad.  L must be visible to every thread on entry (a barrier after its
// last write); ends with a __syncthreads().
template <int kYPad = 0>
__device__ __forceinline__ void unit_lower_inverse_64(const float* sL, float* sT, float* sY2, int ldl, int ldt, int tid,
                                                      int nthreads) {
  for (int i = tid; i < kChunk * kChunk; i += nthreads) sT[(i >> 6) * ldt + (i & 63)] = 0.f;
  __syncthreads();
  if (tid < 64) {
    const int base = (tid >> 2) << 2, col = tid & 3;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float s = (i == col) ? 1.f : 0.f;
#pragma unroll
      for (int m = 0; m < i; ++m) s -= sL[(base + i) * ldl + base + m] * x[m];
      x[i] = s;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) sT[(base + i) * ldt + base + col] = x[i];
  }
  __syncthreads();
  inverse_merge<4>(sL, sT, sY2, ldl, ldt, tid, nthreads);
  inverse_merge<8>(sL, sT, sY2, ldl, ldt, tid, nthreads);
  inverse_merge_tc<16, kYPad, true>(sL, sT, sY2, ldl, ldt, tid);
  inverse_merge_tc<32, kYPad, true>(sL, sT, sY2, ldl, ldt, tid);
}

// Sums each of v[0..7] over the 32 lanes.  On return lane l holds in v[0] the
// total of entry ((l >> 4) & 1) * 4 + ((l >> 3) & 1) * 2 + ((l >> 2) & 1).
__device__ __forceinline__ void row_sums8(float (&v)[8], int lane) {
  const bool hi16 = lane & 16, hi8 = lane & 8, hi4 = lane & 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float keep = hi16 ? v[j + 4] : v[j], send = hi16 ? v[j] : v[j + 4];
    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float keep = hi8 ? v[j + 2] : v[j], send = hi8 ? v[j] : v[j + 2];
    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  {
    const float keep = hi4 ? v[1] : v[0], send = hi4 ? v[0] : v[1];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

// Tail of the classifier kernels: a CTA of 256 threads has put the kind of its 64 items into sKind
// (-1: none, 0: tensor-memory kernel, 1: mma.sync kernel) and appends them to the two work lists with
// one atomic per list, keeping their order.
__device__ __forceinline__ void append_work_items(const int* sKind, int* sBase, int* fast_list, int* slow_list,
                                                  int* counts, int first_item, int tid) {
  __syncthreads();
  if (tid < 2) {
    int cnt = 0;
    for (int i = 0; i < 64; ++i) cnt += sKind[i] == tid;
    sBase[tid] = cnt ? atomicAdd(counts + tid, cnt) : 0;
  }
  __syncthreads();
  if (tid < 2) {
    int* list = tid ? slow_list : fast_list;
    int pos = sBase[tid];
    for (int i = 0; i < 64; ++i)
      if (sKind[i] == tid) list[pos++] = first_item + i;
  }
}

// Arguments of the intra-chunk forward stage (both implementations).
struct IntraParams {
  Geo geo;
  const bf16 *q, *k, *v, *g;
  const float* g_atk;
  const bf16* beta_atk;
  const float *A_log, *dt_bias, *log_atk_scale;
  const float* beta_c;
  const float* a_start;
  bf16 *Aqk, *Akk, *kt;
  float* gc;  // [chunks][H][D] exp of the chunk's total log-decay
  bf16 *w, *u, *kg, *qg;
  float scale, ln_x, eps;
  int direct_cap;  // upper limit for the direct block size (64 = no limit, 1 = hierarchy only)
  int* status;     // device status word (tcgen05 kernel): set to 1 when a bounded wait gives up
  // Work list of (chunk * heads + head) items the tensor-memory kernel leaves to the mma.sync kernel;
  // counts[1] is its length, counts[0] and counts[2] the cursors the CTAs of the two kernels draw their
  // items with (all zeroed before every call).  slow_list == NULL: the mma.sync kernel takes every chunk, one CTA per item.
  int *slow_list, *counts;
  // Preconditioner state across chunks inside the tensor-memory kernel (dense batches; chain != 0):
  // every item computes its chunk's local scan anyway, so it takes its chunk-entry state from the item
  // of the chunk before (a_chain, which is the saved "state at chunk starts" tensor; chain_flags counts
  // the four warps that have published an entry), and publishes the next chunk's.  The items are
  // then drawn chunk level by chunk level across all (row, head) units, so that an item's predecessor
  // started long before it.  beta (raw) is packed to beta_c_w on the way; sa takes the chunk's summed
  // preconditioner log-decay, A0 / AT are the initial / final preconditioner states (may be NULL).
  int chain;
  const bf16* beta;
  float *beta_c_w, *a_chain, *sa, *AT;
  const float* A0;
  int* chain_flags;
};

// tcgen05 / tensor-memory intra-chunk forward stage (pkda_intra_fwd_tc.cu).
int launch_intra_fwd_tc(const IntraParams& ip, bool recompute, cudaStream_t st);

// Arguments of the chunk-parallel backward stage (both implementations).
struct IntraBwdParams {
  Geo geo;
  const bf16 *q, *k, *kt, *g;
  const float *A_log, *dt_bias;
  const float *beta_c, *gc;
  const bf16 *Akk, *v_new, *h, *dh, *dF, *d_o;
  bf16 *dq, *dv, *dg, *dbeta;
  float *dk_read, *dkt;
  float *partA, *partB;
  float scale;
  int direct_cap;
  int use_tma;   // the five phase-A tiles of full chunks arrive by TMA (tensor maps valid)
  int out_tma;   // dq, dv, dk_read and dkt of full chunks leave by TMA from padded shared-memory tiles
  int* status;   // set to 1 if a bounded wait gives up
  // The local part of the preconditioner's backward runs inside the tensor-memory kernel (the mma.sync
  // kernel leaves it to pkda_atk_bwd_kernel<false>): with B the write-key factor kt = k B(A_t),
  //   dkt buffer <- dA_local = d(loss)/dA_t through B alone,  dk_read buffer <- dk_read + dkt B,
  //   c_loc[chunk] = sum_r (prod_{j<=r} decay_j) dA_local_r,  partC[chunk] = d(loss)/d(centre).
  const float* g_atk;
  const bf16* beta_atk;
  const float* log_atk_scale;
  const float* a_start;
  float *c_loc, *partC;
  float ln_x, eps;
  // Work lists of (chunk * heads + head) items written by pkda_bwd_classify_kernel: fast_list for the
  // tensor-memory kernel, slow_list for the mma.sync kernel; fast_count[0] / fast_count[1] are their
  // lengths and fast_count[2] the cursor the mma.sync CTAs draw items with (all zeroed before every
  // call).  slow_list == NULL: the mma.sync kernel takes every chunk, one CTA per (chunk, head).
  int *fast_list, *slow_list, *fast_count;
};

// tcgen05 / tensor-memory chunk-parallel backward stage (pkda_intra_bwd_tc.cu).
int launch_intra_bwd_tc(const IntraBwdParams& ip, cudaStream_t st);
// The backward's first kernel on the default path: sorts the items into the two work lists (counts zeroed
// before) and packs beta chunk-major.
int launch_bwd_classify(const Geo& geo, const float* gc, int direct_cap, int* fast_list, int* slow_list, int* counts,
                        const bf16* beta, float* beta_c, cudaStream_t st);

// tcgen05 / TMA output stage (pkda_out_tc.cu).
int launch_out_fwd_tc(const Geo& geo, int total_tokens, const bf16* qg, const bf16* h, const bf16* Aqk,
                      const bf16* v_new, const float* beta_c, bf16* o, int* status, cudaStream_t st);

// tcgen05 / TMA forward state scan (pkda_scan_tc.cu): one CTA per (sequence, head).
int launch_scan_fwd_tc(const Geo& geo, int total_tokens, int units, const bf16* w, const bf16* kg, const bf16* u,
                       const float* beta_c, const float* gc, const float* S0, bf16* h, bf16* v_new, float* ST,
                       int* status, bool recompute, const bf16* qg, const bf16* Aqk, bf16* o, cudaStream_t st);

// tcgen05 / TMA reverse state scan of the backward (pkda_scan_bwd_tc.cu): one CTA per (sequence, head).
int launch_scan_bwd_tc(const Geo& geo, int total_tokens, int units, const bf16* kg, const bf16* w, const bf16* qg,
                       const bf16* d_o, const bf16* Aqk, const float* beta_c, const float* gc, const float* dST,
                       bf16* dh, bf16* dF, float* dS0, int* status, cudaStream_t st);

// Host-side pieces defined in pkda_chunk_fwd.cu and reused by the backward.
int check_chunk_problem(const pkda_problem& p);
int run_prologue(const pkda_problem& p, int* chunk_offsets, float* beta_c, Geo* geo, cudaStream_t st);
// lists: room for chunks * heads ints (the forward's work list); counts: three zeroed ints.
// o / o_done: the forward's output tensor; *o_done says whether the state scan has already written it.
// What the tensor-memory intra kernel needs to carry the preconditioner state across chunks itself
// (dense batches): see IntraParams::chain.
struct ChainArgs {
  float *beta_c_w, *a_chain, *sa, *AT;
  int* flags;
};
// True when the forward can run in chained mode (no preconditioner kernels in front of the intra stage).
bool forward_chain_possible(const pkda_problem& p);
int run_forward_stages(const pkda_problem& p, const Geo& geo, const float* beta_c, bf16* u_ws, bf16* Aqk,
                       bf16* Akk, bf16* kt, float* gc, const float* a_start, bf16* w, bf16* kg, bf16* v_new,
                       bf16* h, bf16* qg, float* ST, bool recompute, int* status, int* lists, int* counts,
                       cudaStream_t st, bf16* o = nullptr, bool* o_done = nullptr, const ChainArgs* chain = nullptr);

}  // namespace pkda
