// Intra-chunk stage of the chunked forward on tcgen05 / tensor memory (D = 128, chunk 64).
//
// Persistent CTAs of 256 threads, two per SM (about 105 KB of shared memory and 256 tensor-memory
// columns each), walk the (chunk, head) items.  The kernel finishes the chunks whose decay lets
// the whole chunk be ONE direct block (pkda_chunk.cuh): the gated operands are then k 2^G, q 2^G
// and kt 2^-G with G the cumulative log2-decay from the chunk start, one set for all pairs, and
// k 2^G is at the same time the operand Kd of W.  A chunk that turns out (once its cumulative
// decay is known) to decay by more than kDirectLimit is put on a work list and left to the
// mma.sync kernel of pkda_chunk_fwd.cu, which runs right after this one and pairs such chunks
// level by level.  The decision depends on the inputs only, so the recompute pass of a lean
// backward sends every chunk to the kernel that built it.  What the stage computes is described
// at the top of pkda_chunk_fwd.cu; this file differs from the kernel there in how:
//
//  * Elementwise work runs on registers in a "strip" layout: warp w owns rows 8w..8w+7 of the
//    chunk, lane l owns channels 4l..4l+3, so a warp reads or writes whole 256-byte token rows.
//    The two sequential passes over the rows (cumulative log-decay, the preconditioner
//    recurrence A_t) are blocked scans: eight rows in registers, one exchange of (block total,
//    block decay) through shared memory, then each block continues from the prefix it is owed.
//  * q, k and the raw gate arrive by cp.async straight into the places of the operand tiles
//    their gated values will take (128-byte-swizzled canonical layout); the gating happens in
//    place, each thread touching only its own 8-byte pieces.  The rows of k and q are stacked
//    to one 128-row A operand, the write keys are the B operand: eight tcgen05.mma (M = 128,
//    N = 64, K = 16) give M = k kt^T in accumulator rows 0..63 and P = q kt^T in rows 64..127.
//    All eight warps read the accumulator back (one tensor-memory lane = one row per thread)
//    and write L = tril(M, -1) diag(beta) in fp32 and scale tril(P) in bf16.
//  * T = (I + L)^-1 stays on the CUDA cores and 3xTF32 mma.sync (pkda_chunk.cuh): it needs
//    fp32-level accuracy and its products are at most 32 x 32.
//  * W^T = Kd^T T^T and U^T = V^T T^T are two more accumulators (M = 128 channels, N = 64
//    tokens, K = 64 tokens); V and the outputs of full chunks move by TMA.
//
// Every mbarrier wait is bounded; a CTA whose wait gives up sets the status word.
#include "pkda_chunk.cuh"
#include "pkda_tc.cuh"


namespace pkda {

namespace intratc {
constexpr int kThreads = 256;
constexpr int kLdL = 68;                    // row stride of L and T: float4 rows, and conflict-free MMA fragments
constexpr int oA = 0;                       // 2 blocks [128 rows][64 ch]: rows 0..63 k 2^G (= Kd, the MN-major A of
                                            // W^T), rows 64..127 q 2^G (together the K-major A of the pair products)
constexpr int oY = oA + 32768;              // 2 blocks [64 rows][64 ch]: kt 2^-G (K-major B); + 1 KB so that T fits
constexpr int oV = oY + 16384 + 1024;       // 2 blocks [64 tok][64 ch]: V (MN-major A of U^T)
constexpr int oTm = oV + 16384;             // [64 i][64 j] bf16 T (K-major B)
constexpr int oP = oTm + 8192;              // [64 i][64 j] bf16 scale * P
constexpr int oL = oP + 8192;               // f32 [64][68] L; before the products: the scan exchange arrays
constexpr int oBeta = oL + 64 * kLdL * 4;   // f32 [64]
constexpr int oDiag = oBeta + 256;          // f32 [64] q_i . kt_i
constexpr int oBar = oDiag + 256;           // TMA barrier, MMA barrier, tensor-memory base address
constexpr int kSmem = oBar + 64 + 1024;     // + slack to align the tiles to 1024 bytes
// inside the L region before the products
constexpr int oTot = oL;                    // f32 [8][128] per-strip decay totals
constexpr int oEnd = oL + 4096;             // f32 [8][128] per-strip end value of the zero-start A scan
constexpr int oDec = oL + 8192;             // f32 [8] per-strip product of preconditioner decays
constexpr int oSum = oDec + 32;             // f32 [8] per-strip sum of the preconditioner's log-decays
constexpr int oA0 = oSum + 32;              // f32 [128] the chunk-entry preconditioner state (chained mode)
// while the inverse runs: T in the (dead) write-key operand, its scratch in the (dead) q rows of block 0
constexpr int oT = oY;                      // f32 [64][68]
constexpr int oY2 = oA + 8192;              // f32 [1280]
static_assert(oA0 + 512 <= oBeta && oT + 64 * kLdL * 4 <= oV && oY2 + 5120 <= oA + 16384, "aliases must fit");
constexpr uint32_t kCols = 256;             // pair accumulator 0..63, W^T 64..127, U^T 128..191
}  // namespace intratc

__device__ __forceinline__ void unpack4(uint2 r, float (&f)[4]) {
  const float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 scale4(uint2 r, const float (&f)[4]) {
  float x[4];
  unpack4(r, x);
  return make_uint2(pack_bf16(x[0] * f[0], x[1] * f[1]), pack_bf16(x[2] * f[2], x[3] * f[3]));
}

// Acquire load / release add at device scope: the hand-over of the preconditioner state between items.
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <bool kRecompute>
__global__ void __launch_bounds__(intratc::kThreads, 2)
pkda_intra_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_akk,
                         const __grid_constant__ CUtensorMap tm_aqk, const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_u, const IntraParams p) {
  using namespace intratc;
  extern __shared__ unsigned char smem_raw[];
  const int H = p.geo.heads;
  const int n_items = p.geo.total_chunks * H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long gld = (long)H * kD;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_tma = base + oBar, bar_mma = base + oBar + 8, tmem_slot = base + oBar + 16;
  float* sL = reinterpret_cast<float*>(tiles + oL);
  float* sBeta = reinterpret_cast<float*>(tiles + oBeta);
  float* sDiag = reinterpret_cast<float*>(tiles + oDiag);
  float* sTot = reinterpret_cast<float*>(tiles + oTot);
  float* sEnd = reinterpret_cast<float*>(tiles + oEnd);
  float* sDec = reinterpret_cast<float*>(tiles + oDec);
  float* sSum = reinterpret_cast<float*>(tiles + oSum);
  float* sA0 = reinterpret_cast<float*>(tiles + oA0);
  const bool chain = !kRecompute && p.chain;
  const int units = p.geo.n_seqs * H;  // (chained mode: items are drawn level by level over all units)

  // strip layout: this thread's rows r0..r0+7, channels c4..c4+3
  const int r0 = warp * 8, c4 = lane << 2;
  // byte offset of the thread's 8-byte half piece inside a swizzled row is ((piece ^ row%8) << 4) + half * 8
  const int blk = lane >> 4, piece = (lane & 15) >> 1, half8 = (lane & 1) << 3;
  // The slot of strip row i is the very place its gated value goes later: row r0 + i of the
  // stacked operand for k (rows 0..63) and q (rows 64..127), of the write-key operand for g (and,
  // once g is consumed, for the write key kt).  A thread only ever touches its own 8-byte pieces
  // there until the operands are complete, so the in-place updates need no barrier.
  unsigned char* aBase = tiles + oA + blk * 16384 + half8;  // + slot_off(i): k; + 8192: q
  unsigned char* yBase = tiles + oY + blk * 8192 + half8;   // + slot_off(i): g, then kt
  auto slot_off = [&](int i) { return (r0 + i) * 128 + ((piece ^ i) << 4); };
  auto ld_k = [&](int i) { return *reinterpret_cast<const uint2*>(aBase + slot_off(i)); };
  auto ld_q = [&](int i) { return *reinterpret_cast<const uint2*>(aBase + 8192 + slot_off(i)); };
  auto ld_y = [&](int i) { return *reinterpret_cast<const uint2*>(yBase + slot_off(i)); };

  if (tid == 0) {
    tc::mbar_init(bar_tma, 1);
    tc::mbar_init(bar_mma, 1);
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, kCols);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tiles + oBar + 16);
  bool ok = true;
  uint32_t mma_phase = 0, tma_phase = 0;
  const int R = 32 * (warp & 3) + lane;     // this thread's accumulator row in the pair products
  const int ei = R & 63, j0 = 32 * (warp >> 2);
  const bool isP = (warp & 3) >= 2;

  // Items differ in cost (a chunk that is handed over costs a fraction of one that is finished), so
  // the CTAs draw them one at a time from a cursor instead of striding through them.
  __shared__ int s_next;
  if (tid == 0) s_next = atomicAdd(p.counts, 1);
  __syncthreads();
  int draw = s_next;
#pragma unroll 1
  while (draw < n_items) {
  // the draw-th item: in chained mode chunk level draw / units of unit draw % units (a dense batch)
  const int level = chain ? draw / units : 0;
  const int item = chain ? ((draw % units) / H * p.geo.chunks_per_seq + level) * H + (draw % units) % H : draw;
  const int h = item % H;
  int n, tok0, valid;
  if (!chunk_lookup(p.geo, item / H, n, tok0, valid)) break;  // past the last real chunk of a packed batch (items ascend)
  const size_t chh = (size_t)item;
  const size_t row0 = ((size_t)tok0 * H + h) * kD;
  const bool full = valid == kChunk;
  // The operand descriptors depend on the tile base only; keeping the base opaque per item stops the
  // compiler from computing all of them ahead of the loop and holding them in registers.
  uint32_t dbase = base;
  asm volatile("" : "+r"(dbase));

  // ---- 0. V (and T when recomputing) by TMA; this thread's strips of g, k and q by cp.async
  if (tid == 0) {
    tc::mbar_expect_tx(bar_tma, kRecompute ? 16384 + 8192 : 16384);
    tc::tma_load_3d(base + oV, &tm_v, bar_tma, 0, h, tok0);
    tc::tma_load_3d(base + oV + 8192, &tm_v, bar_tma, 64, h, tok0);
    if (kRecompute) tc::tma_load_3d(base + oTm, &tm_akk, bar_tma, 0, h, tok0);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool okr = r0 + i < valid;
    const size_t off = row0 + (size_t)(okr ? r0 + i : 0) * gld + c4;
    const int nb = okr ? 8 : 0;  // rows past the sequence end read as zero
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_u32(yBase + slot_off(i))), "l"(p.g + off), "r"(nb));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_u32(aBase + slot_off(i))), "l"(p.k + off), "r"(nb));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_u32(aBase + 8192 + slot_off(i))), "l"(p.q + off), "r"(nb));
  }
  cp_async_commit();
  uint2 ktraw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ktraw[i] = make_uint2(0, 0);
    if (kRecompute && r0 + i < valid)
      ktraw[i] = *reinterpret_cast<const uint2*>(p.kt + row0 + (size_t)(r0 + i) * gld + c4);
  }
  float sc_beta = 0.f, sc_pd = 0.f, sc_bp = 0.f;  // lane i < 8: scalars of row r0 + i
  if (lane < 8) {
    const int r = r0 + lane;
    if (chain) {  // beta is packed chunk-major on the way (the later stages read that copy)
      sc_beta = r < valid ? to_f(p.beta[(size_t)(tok0 + r) * H + h]) : 0.f;
      p.beta_c_w[chh * kChunk + r] = sc_beta;
    } else {
      sc_beta = p.beta_c[chh * kChunk + r];
    }
    if (!kRecompute && r < valid) {
      const size_t s = (size_t)(tok0 + r) * H + h;
      sc_pd = p.g_atk[s];
      sc_bp = to_f(p.beta_atk[s]);
    }
  }
  const float4 bias4 = *reinterpret_cast<const float4*>(p.dt_bias + h * kD + c4);
  const float ea2 = __expf(p.A_log[h]) * kLog2e;
  float4 a_first = make_float4(0.f, 0.f, 0.f, 0.f);
  float centre = 0.f;
  // Chained mode: the chunk-entry state of the preconditioner was normally published long ago by the
  // item of the chunk before; it is asked for now, so that the two dependent loads (counter, then
  // value) are back when the strips are.
  int chain_seen = 4;
  float chain_a0 = 0.f;
  if (!kRecompute) {
    if (!chain) {
      a_first = *reinterpret_cast<const float4*>(p.a_start + chh * kD + c4);
    } else if (tid < kD) {
      if (level == 0) {
        if (p.A0) chain_a0 = p.A0[((size_t)n * H + h) * kD + tid];
      } else {
        chain_seen = ld_acquire(p.chain_flags + item);
        if (chain_seen >= 4) chain_a0 = __ldcg(p.a_chain + chh * kD + tid);
      }
    }
    centre = p.log_atk_scale[h];
  }
  cp_async_wait<0>();

  // ---- 1. decay gate, strip-local cumulative sum; strip-local preconditioner scan from zero
  float G[8][4];
  {
    const float bias[4] = {bias4.x, bias4.y, bias4.z, bias4.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float x[4];
      unpack4(ld_y(i), x);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float gv = (r0 + i < valid) ? -ea2 * softplus_fast(x[e] + bias[e]) : 0.f;
        G[i][e] = i ? G[i - 1][e] + gv : gv;
      }
    }
  }
  if (!kRecompute) {
    if (chain) {  // the strip's summed log-decay, added in row order
      float gsum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) gsum += __shfl_sync(0xffffffffu, sc_pd, i);
      if (lane == 0) sSum[warp] = gsum;
    }
    sc_pd = __expf(sc_pd);  // rows past the end: exp(0) = 1, beta 0
    float a[4] = {0.f, 0.f, 0.f, 0.f}, dblk = 1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float pd = __shfl_sync(0xffffffffu, sc_pd, i), bp = __shfl_sync(0xffffffffu, sc_bp, i);
      float kc[4];
      unpack4(ld_k(i), kc);
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] = pd * a[e] + bp * kc[e] * kc[e];
      dblk *= pd;
    }
    *reinterpret_cast<float4*>(sEnd + warp * kD + c4) = make_float4(a[0], a[1], a[2], a[3]);
    if (lane == 0) sDec[warp] = dblk;
  }
  *reinterpret_cast<float4*>(sTot + warp * kD + c4) = make_float4(G[7][0], G[7][1], G[7][2], G[7][3]);
  if (lane < 8) sBeta[r0 + lane] = sc_beta;
  __syncthreads();

  // ---- 2. prefixes over the strips: cumulative decay of every row, and of the chunk's last row
  float Glast[4];
  {
    float P[4] = {0.f, 0.f, 0.f, 0.f}, pre[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int wp = 0; wp < 8; ++wp) {
      const float4 to = *reinterpret_cast<const float4*>(sTot + wp * kD + c4);
      if (wp == warp) {
#pragma unroll
        for (int e = 0; e < 4; ++e) pre[e] = P[e];
      }
      P[0] += to.x; P[1] += to.y; P[2] += to.z; P[3] += to.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) Glast[e] = P[e];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) G[i][e] += pre[e];
  }
  // Chained mode: this chunk's entry state of the preconditioner comes from the item of the chunk
  // before it (or the initial state), the next chunk's goes out.  Four warps, one channel per thread;
  // a warp publishes with a fence and one count on the successor's flag, which the successor's four
  // warps poll (bounded) until all four counts are in.
  if (chain && tid < kD) {
    float loc = 0.f, gs = 0.f;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      loc = sDec[b] * loc + sEnd[b * kD + tid];
      gs += sSum[b];
    }
    float a0 = chain_a0;
    if (level == 0) {
      p.a_chain[chh * kD + tid] = a0;
    } else if (chain_seen < 4) {  // not there yet when the item began: poll (bounded)
      uint32_t it = 0;
      while ((chain_seen = ld_acquire(p.chain_flags + item)) < 4 && ++it < tc::kSpinLimit) {}
      ok = ok && chain_seen >= 4;
      a0 = __ldcg(p.a_chain + chh * kD + tid);
    }
    sA0[tid] = a0;
    const float an = __expf(gs) * a0 + loc;
    if (level + 1 < p.geo.chunks_per_seq) {
      p.a_chain[(chh + H) * kD + tid] = an;
      __syncwarp();
      if (lane == 0) red_release_add(p.chain_flags + item + H, 1);  // (orders the warp's stores before the count)
    } else if (p.AT) {
      p.AT[((size_t)n * H + h) * kD + tid] = an;
    }
    if (tid == 0) p.sa[chh] = gs;
  }
  // A chunk that decays too much for one direct block goes to the mma.sync kernel (the decision is
  // the same for all threads: every thread holds the totals of its four channels, the CTA all 128).
  {
    const float worst = -fminf(fminf(Glast[0], Glast[1]), fminf(Glast[2], Glast[3]));
    if (__syncthreads_or(worst > kDirectLimit)) {
      if (tid == 0) p.slow_list[atomicAdd(p.counts + 1, 1)] = item;
      ok = tc::mbar_wait(bar_tma, tma_phase) && ok;  // the V tile in flight must land before the tile is reused
      tma_phase ^= 1;
      if (tid == 0) s_next = atomicAdd(p.counts, 1);
      __syncthreads();
      draw = s_next;
      continue;
    }
  }

  // ---- 3. one pass over the strip: preconditioner states of its rows -> write keys kt = k * B(A_t)
  // (to global memory), kg = kt * decay to the chunk end, the diagonal q_i . kt_i, and the gated operands
  // in place: Kd = k 2^G (rows 0..63 of the stacked operand, later the operand of W^T), q 2^G (rows
  // 64..127), kt 2^-G (into the slots g has left); qg goes to global memory.  The decay to the chunk
  // end is 2^G_last times the 2^-G the operand needs anyway.  Nothing of the strip is needed afterwards.
  {
    if (chain) a_first = *reinterpret_cast<const float4*>(sA0 + c4);  // (written before the barrier of the decision)
    float A[4] = {a_first.x, a_first.y, a_first.z, a_first.w};
    if (!kRecompute) {
      for (int b = 0; b < warp; ++b) {
        const float d = sDec[b];
        const float4 e4 = *reinterpret_cast<const float4*>(sEnd + b * kD + c4);
        A[0] = d * A[0] + e4.x; A[1] = d * A[1] + e4.y; A[2] = d * A[2] + e4.z; A[3] = d * A[3] + e4.w;
      }
    }
    const float glE[4] = {ex2(Glast[0]), ex2(Glast[1]), ex2(Glast[2]), ex2(Glast[3])};
    float dg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int off = slot_off(i);
      const uint2 kr = ld_k(i), qr = ld_q(i);
      uint2 kt = ktraw[i];
      if (!kRecompute) {
        const float pd = __shfl_sync(0xffffffffu, sc_pd, i), bp = __shfl_sync(0xffffffffu, sc_bp, i);
        float kc[4], f[4];
        unpack4(kr, kc);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          A[e] = pd * A[e] + bp * kc[e] * kc[e];
          const float dev = __logf(A[e] + p.eps) - centre;
          f[e] = __expf(-p.ln_x * __fdividef(dev, 1.f + fabsf(dev)));
        }
        kt = scale4(kr, f);
        if (r0 + i < valid) *reinterpret_cast<uint2*>(p.kt + row0 + (size_t)(r0 + i) * gld + c4) = kt;
        float kc2[4], qc[4];
        unpack4(kt, kc2);
        unpack4(qr, qc);
        dg[i] = qc[0] * kc2[0] + qc[1] * kc2[1] + qc[2] * kc2[2] + qc[3] * kc2[3];
      }
      float e[4], es[4], fi[4], tl[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        e[c] = ex2(G[i][c]);
        es[c] = e[c] * p.scale;
        fi[c] = __fdividef(1.f, e[c]);
        tl[c] = glE[c] * fi[c];
      }
      *reinterpret_cast<uint2*>(aBase + off) = scale4(kr, e);
      if (!kRecompute) {
        *reinterpret_cast<uint2*>(aBase + 8192 + off) = scale4(qr, e);
        *reinterpret_cast<uint2*>(yBase + off) = scale4(kt, fi);
      }
      if (r0 + i < valid) {
        *reinterpret_cast<uint2*>(p.kg + row0 + (size_t)(r0 + i) * gld + c4) = scale4(kt, tl);
        *reinterpret_cast<uint2*>(p.qg + row0 + (size_t)(r0 + i) * gld + c4) = scale4(qr, es);
      }
    }
    if (!kRecompute) {
      row_sums8(dg, lane);
      if ((lane & 3) == 0) sDiag[r0 + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)] = dg[0];
      if (warp == 0)
        *reinterpret_cast<float4*>(p.gc + chh * kD + c4) = make_float4(glE[0], glE[1], glE[2], glE[3]);
    }
  }
  tc::fence_proxy_async();
  tc::tc_fence_before();
  __syncthreads();  // (the strip exchange arrays are dead from here on: L takes their place)
  if (!kRecompute) {
    if (tid == 0) {
      tc::tc_fence_after();
      constexpr uint32_t idesc_pair = tc::idesc_bf16(128, 64, false, false);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t a = tc::desc_kmajor(dbase + oA + (kk >> 2) * 16384 + (kk & 3) * 32);
        const uint64_t b = tc::desc_kmajor(dbase + oY + (kk >> 2) * 8192 + (kk & 3) * 32);
        tc::umma_bf16(tmem, a, b, idesc_pair, kk > 0);
      }
      tc::umma_commit(bar_mma);
    }
    ok = tc::mbar_wait(bar_mma, mma_phase) && ok;
    mma_phase ^= 1;
    tc::tc_fence_after();
    {
      float acc[32];
      tc::tmem_ld32(tmem + ((uint32_t)(32 * (warp & 3)) << 16) + j0, acc);
      tc::tmem_ld_wait();
      if (!isP) {  // L = tril(M, -1) diag(beta)
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          float4 x;
          x.x = (j0 + t < ei) ? acc[t] * sBeta[j0 + t] : 0.f;
          x.y = (j0 + t + 1 < ei) ? acc[t + 1] * sBeta[j0 + t + 1] : 0.f;
          x.z = (j0 + t + 2 < ei) ? acc[t + 2] * sBeta[j0 + t + 2] : 0.f;
          x.w = (j0 + t + 3 < ei) ? acc[t + 3] * sBeta[j0 + t + 3] : 0.f;
          *reinterpret_cast<float4*>(sL + ei * kLdL + j0 + t) = x;
        }
      } else {     // scale * tril(P) with the ungated diagonal
        unsigned char* prow = tiles + oP + ei * 128;
        const float dv = sDiag[ei];
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          float x[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int j = j0 + 8 * pc + t;
            x[t] = (j < ei ? acc[8 * pc + t] : (j == ei ? dv : 0.f)) * p.scale;
          }
          *reinterpret_cast<uint4*>(prow + ((((j0 >> 3) + pc) ^ (ei & 7)) << 4)) =
              make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
        }
      }
    }
    tc::tc_fence_before();
  }
  ok = tc::mbar_wait(bar_tma, tma_phase) && ok;  // V (and T) landed long ago
  tma_phase ^= 1;
  if (!full) {  // rows past the sequence end hold another sequence's data: they must not reach the product
    for (int idx = tid; idx < kChunk * 16; idx += kThreads) {
      const int r = idx >> 4, pc = idx & 15;
      if (r >= valid)
        *reinterpret_cast<uint4*>(tiles + oV + (pc >> 3) * 8192 + r * 128 + ((pc & 7) << 4)) = make_uint4(0, 0, 0, 0);
    }
  }
  tc::fence_proxy_async();
  __syncthreads();

  if (!kRecompute) {
    // ---- 5. scaled P -> Aqk;  T = (I + L)^-1 -> bf16 operand tile and Akk
    if (full) {
      if (tid == 0) {
        tc::tma_store_3d(&tm_aqk, base + oP, 0, h, tok0);
        tc::bulk_commit();
      }
    } else {
      for (int idx = tid; idx < kChunk * 8; idx += kThreads) {
        const int r = idx >> 3, pc = idx & 7;
        if (r < valid)
          *reinterpret_cast<uint4*>(p.Aqk + ((size_t)(tok0 + r) * H + h) * kChunk + 8 * pc) =
              *reinterpret_cast<const uint4*>(tiles + oP + r * 128 + ((pc ^ (r & 7)) << 4));
      }
    }
    float* sT = reinterpret_cast<float*>(tiles + oT);
    unit_lower_inverse_64<8>(sL, sT, reinterpret_cast<float*>(tiles + oY2), kLdL, kLdL, tid, kThreads);  // ends with a barrier
    for (int idx = tid; idx < kChunk * 8; idx += kThreads) {
      const int r = idx >> 3, pc = idx & 7;
      const float4 s0 = *reinterpret_cast<const float4*>(sT + r * kLdL + 8 * pc);
      const float4 s1 = *reinterpret_cast<const float4*>(sT + r * kLdL + 8 * pc + 4);
      const uint4 pk = make_uint4(pack_bf16(s0.x, s0.y), pack_bf16(s0.z, s0.w), pack_bf16(s1.x, s1.y),
                                  pack_bf16(s1.z, s1.w));
      *reinterpret_cast<uint4*>(tiles + oTm + r * 128 + ((pc ^ (r & 7)) << 4)) = pk;
      if (!full && r < valid)
        *reinterpret_cast<uint4*>(p.Akk + ((size_t)(tok0 + r) * H + h) * kChunk + 8 * pc) = pk;
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
  }

  // ---- 6. W^T = Kd^T T^T, U^T = V^T T^T
  if (tid == 0) {
    tc::tc_fence_after();
    if (!kRecompute && full) {
      tc::tma_store_3d(&tm_akk, base + oTm, 0, h, tok0);
      tc::bulk_commit();
    }
    constexpr uint32_t idesc = tc::idesc_bf16(128, 64, /*a_mn_major=*/true, /*b_mn_major=*/false);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      tc::umma_bf16(tmem + 64, tc::desc_mnmajor(dbase + oA + kk * 2048, 16384), tc::desc_kmajor(dbase + oTm + kk * 32),
                    idesc, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      tc::umma_bf16(tmem + 128, tc::desc_mnmajor(dbase + oV + kk * 2048, 8192), tc::desc_kmajor(dbase + oTm + kk * 32),
                    idesc, kk > 0);
    tc::umma_commit(bar_mma);
  }
  ok = tc::mbar_wait(bar_mma, mma_phase) && ok;
  mma_phase ^= 1;
  tc::tc_fence_after();
  {
    const int ch = 32 * (warp & 3) + lane, t0 = 32 * (warp >> 2);  // accumulator row = channel; this warp's tokens
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      float acc[32];
      tc::tmem_ld32(tmem + ((uint32_t)(32 * (warp & 3)) << 16) + 64 + 64 * m + t0, acc);
      tc::tmem_ld_wait();
      if (full) {  // transposed into a swizzled [token][channel] tile for the TMA store
        unsigned char* out = tiles + oA + m * 16384;
#pragma unroll
        for (int t = 0; t < 32; ++t)
          *reinterpret_cast<bf16*>(out + sw128_offset(t0 + t, ch, 8192)) = __float2bfloat16(acc[t]);
      } else {
        bf16* dst = m ? p.u : p.w;
#pragma unroll
        for (int t = 0; t < 32; ++t)
          if (t0 + t < valid) dst[row0 + (size_t)(t0 + t) * gld + ch] = __float2bfloat16(acc[t]);
      }
    }
  }
  tc::fence_proxy_async();
  tc::tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    if (full) {
      tc::tma_store_3d(&tm_w, base + oA, 0, h, tok0);
      tc::tma_store_3d(&tm_w, base + oA + 8192, 64, h, tok0);
      tc::tma_store_3d(&tm_u, base + oA + 16384, 0, h, tok0);
      tc::tma_store_3d(&tm_u, base + oA + 16384 + 8192, 64, h, tok0);
      tc::bulk_commit();
    }
    tc::bulk_wait_read();  // the tiles stay in place until every store of this item has read them
    s_next = atomicAdd(p.counts, 1);
  }
  __syncthreads();  // the next item's copies overwrite the tiles
  draw = s_next;
  }  // item loop
  if (__syncthreads_or(!ok) && tid == 0) atomicExch(p.status, 1);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) tc::tmem_dealloc(tmem, kCols);
}

// ------------------------------------------------------------------ host side
int launch_intra_fwd_tc(const IntraParams& ip, bool recompute, cudaStream_t st) {
  const uint64_t H = ip.geo.heads, tok = ip.geo.total_tokens;
  CUtensorMap tm_v, tm_akk, tm_aqk, tm_w, tm_u;
  {
    const uint64_t dims[3] = {kD, H, tok}, str[2] = {kD * 2, H * kD * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_v, ip.v, 3, dims, str, box) || !encode_bf16_map(&tm_w, ip.w, 3, dims, str, box) ||
        !encode_bf16_map(&tm_u, ip.u, 3, dims, str, box))
      return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {kChunk, H, tok}, str[2] = {kChunk * 2, H * kChunk * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_akk, ip.Akk, 3, dims, str, box) || !encode_bf16_map(&tm_aqk, ip.Aqk, 3, dims, str, box))
      return PKDA_ERR_LAUNCH;
  }
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int items = ip.geo.total_chunks * ip.geo.heads;
  const int grid = items < 2 * sms ? items : 2 * sms;  // persistent: two CTAs per SM
  // two CTAs per SM need the largest shared-memory carve-out
  if (recompute) {
    if (!ensure_dynamic_smem(pkda_intra_fwd_tc_kernel<true>, intratc::kSmem, 100))
      return PKDA_ERR_LAUNCH;
    pkda_intra_fwd_tc_kernel<true><<<grid, intratc::kThreads, intratc::kSmem, st>>>(tm_v, tm_akk, tm_aqk, tm_w, tm_u, ip);
  } else {
    if (!ensure_dynamic_smem(pkda_intra_fwd_tc_kernel<false>, intratc::kSmem, 100))
      return PKDA_ERR_LAUNCH;
    pkda_intra_fwd_tc_kernel<false><<<grid, intratc::kThreads, intratc::kSmem, st>>>(tm_v, tm_akk, tm_aqk, tm_w, tm_u, ip);
  }
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda

