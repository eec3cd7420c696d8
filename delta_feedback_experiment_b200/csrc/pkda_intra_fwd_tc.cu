// Intra-chunk stage of the chunked forward on tcgen05 / tensor memory (D = 128, chunk 64).
//
// One CTA of 256 threads per (chunk, head), two CTAs per SM (about 105 KB of shared memory
// and 256 tensor-memory columns each).  What the stage computes is described at the top of
// pkda_chunk_fwd.cu; this file differs from the mma.sync kernel there in how:
//
//  * Elementwise work runs on registers in a "strip" layout: warp w owns rows 8w..8w+7 of
//    the chunk, lane l owns channels 4l..4l+3, so a thread holds an 8 x 4 patch of q, k, the
//    gate and the write keys for the whole kernel and a warp reads or writes whole 256-byte
//    token rows.  The two sequential passes over the rows (cumulative log-decay, the
//    preconditioner recurrence A_t) are blocked scans: eight rows in registers, one exchange
//    of (block total, block decay) through shared memory, then each block continues from
//    the prefix it is owed.  Reference rows of the pair hierarchy are either one of a
//    thread's own rows (levels below 8) or the first row of a warp's strip (levels 8 and
//    up), so the full cumulative-decay tile never goes to shared memory.
//  * The gated operands of a level are written once, as bf16, straight into the
//    128-byte-swizzled canonical tiles tcgen05 reads: the rows of k and q stacked to a
//    128-row A operand, the write keys as the B operand.  One thread issues eight
//    tcgen05.mma (M = 128, N = 64, K = 16) per level; rows 0..63 of the accumulator are the
//    key-key products M, rows 64..127 the query-key products P.  All eight warps read the
//    accumulator back (one tensor-memory lane = one row per thread), keep the pairs that
//    belong to the level and write L = tril(M) diag(beta) in fp32 and P in bf16.
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
constexpr int kLdL = 65;
constexpr int oA = 0;                       // 2 blocks [128 rows][64 ch]: rows 0..63 gated k (in the end Kd, the
                                            // MN-major A of W^T), rows 64..127 gated q (K-major A of the pairs)
constexpr int oY = oA + 32768;              // 2 blocks [64 rows][64 ch]: gated write keys (K-major B); + 1 KB: T fits
constexpr int oV = oY + 16384 + 1024;       // 2 blocks [64 tok][64 ch]: V (MN-major A of U^T)
constexpr int oTm = oV + 16384;             // [64 i][64 j] bf16 T (K-major B)
constexpr int oP = oTm + 8192;              // [64 i][64 j] bf16 scale * P
constexpr int oL = oP + 8192;               // f32 [64][65] L; before the levels: the scan exchange arrays
constexpr int oGf = oL + 64 * kLdL * 4;     // f32 [8][128] cumulative decay of the first row of each warp strip
constexpr int oBeta = oGf + 4096;           // f32 [64]
constexpr int oDiag = oBeta + 256;          // f32 [64] q_i . kt_i
constexpr int oWmax = oDiag + 256;          // f32 [8][6]
constexpr int oBar = oWmax + 256;           // TMA barrier, MMA barrier, tensor-memory base address
constexpr int kSmem = oBar + 64 + 1024;     // + slack to align the tiles to 1024 bytes
// inside the L region before the levels
constexpr int oTot = oL;                    // f32 [8][128] per-strip decay totals
constexpr int oFirst = oL + 4096;           // f32 [8][128] per-strip first-row gate
constexpr int oEnd = oL + 8192;             // f32 [8][128] per-strip end value of the zero-start A scan
constexpr int oDec = oL + 12288;            // f32 [8] per-strip product of preconditioner decays
// while the inverse runs: T in the (dead) write-key operand, its scratch in the (dead) q rows of block 0
constexpr int oT = oY;                      // f32 [64][65]
constexpr int oY2 = oA + 8192;              // f32 [1024]
static_assert(oDec + 32 <= oGf && oT + 64 * kLdL * 4 <= oV && oY2 + 4096 <= oA + 16384, "aliases must fit");
constexpr uint32_t kCols = 256;             // level accumulator 0..63, W^T 64..127, U^T 128..191
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

template <bool kRecompute>
__global__ void __launch_bounds__(intratc::kThreads, 2)
pkda_intra_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_akk,
                         const __grid_constant__ CUtensorMap tm_aqk, const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_u, const IntraParams p) {
  using namespace intratc;
  extern __shared__ unsigned char smem_raw[];
  int n, tok0, valid;
  if (!chunk_lookup(p.geo, blockIdx.x, n, tok0, valid)) return;
  PKDA_PHASE(0);
  const int h = blockIdx.y, H = p.geo.heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t chh = (size_t)blockIdx.x * H + h;
  const size_t row0 = ((size_t)tok0 * H + h) * kD;
  const long gld = (long)H * kD;
  const bool full = valid == kChunk;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_tma = base + oBar, bar_mma = base + oBar + 8, tmem_slot = base + oBar + 16;
  float* sL = reinterpret_cast<float*>(tiles + oL);
  float* sGf = reinterpret_cast<float*>(tiles + oGf);
  float* sBeta = reinterpret_cast<float*>(tiles + oBeta);
  float* sDiag = reinterpret_cast<float*>(tiles + oDiag);
  float* sWmax = reinterpret_cast<float*>(tiles + oWmax);
  float* sTot = reinterpret_cast<float*>(tiles + oTot);
  float* sFirst = reinterpret_cast<float*>(tiles + oFirst);
  float* sEnd = reinterpret_cast<float*>(tiles + oEnd);
  float* sDec = reinterpret_cast<float*>(tiles + oDec);

  // strip layout: this thread's rows r0..r0+7, channels c4..c4+3
  const int r0 = warp * 8, c4 = lane << 2;
  // byte offset of the thread's 8-byte half piece inside a swizzled row is ((piece ^ row%8) << 4) + half * 8
  const int blk = lane >> 4, piece = (lane & 15) >> 1, half8 = (lane & 1) << 3;

  // ---- 0. set-up: barriers + V (and T when recomputing) by TMA, tensor memory; this thread's strips of
  // g, k and q by cp.async into private slots of the (still unused) operand tiles, so that all of
  // them are in flight at once without holding registers
  if (tid == 0) {
    tc::mbar_init(bar_tma, 1);
    tc::mbar_init(bar_mma, 1);
    tc::fence_barrier_init();
    tc::mbar_expect_tx(bar_tma, kRecompute ? 16384 + 8192 : 16384);
    tc::tma_load_3d(base + oV, &tm_v, bar_tma, 0, h, tok0);
    tc::tma_load_3d(base + oV + 8192, &tm_v, bar_tma, 64, h, tok0);
    if (kRecompute) tc::tma_load_3d(base + oTm, &tm_akk, bar_tma, 0, h, tok0);
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, kCols);
  // The slot of strip row i is the very place its gated value goes later: row r0 + i of the
  // stacked operand for k (rows 0..63) and q (rows 64..127), of the write-key operand for g (and,
  // once g is consumed, for the write key kt).  A thread only ever touches its own 8-byte pieces
  // there until the operands are complete, so the in-place updates need no barrier.
  unsigned char* aBase = tiles + oA + blk * 16384 + half8;  // + slot_off(i): k; + 8192: q
  unsigned char* yBase = tiles + oY + blk * 8192 + half8;   // + slot_off(i): g, then kt
  auto slot_off = [&](int i) { return (r0 + i) * 128 + ((piece ^ i) << 4); };
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
  auto ld_k = [&](int i) { return *reinterpret_cast<const uint2*>(aBase + slot_off(i)); };
  auto ld_q = [&](int i) { return *reinterpret_cast<const uint2*>(aBase + 8192 + slot_off(i)); };
  auto ld_y = [&](int i) { return *reinterpret_cast<const uint2*>(yBase + slot_off(i)); };
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
    sc_beta = p.beta_c[chh * kChunk + r];
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
  if (!kRecompute) {
    a_first = *reinterpret_cast<const float4*>(p.a_start + chh * kD + c4);
    centre = p.log_atk_scale[h];
  }
  PKDA_PHASE(20);
  cp_async_wait<0>();
  PKDA_PHASE(21);

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
  PKDA_PHASE(22);
  if (!kRecompute) {
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
  *reinterpret_cast<float4*>(sFirst + warp * kD + c4) = make_float4(G[0][0], G[0][1], G[0][2], G[0][3]);
  if (lane < 8) sBeta[r0 + lane] = sc_beta;
  tc::tc_fence_before();
  PKDA_PHASE(23);
  __syncthreads(); PKDA_PHASE(1);
  tc::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tiles + oBar + 16);

  // ---- 2. prefixes over the strips: cumulative decay of every row; worst block decays.  A block of b
  // rows is paired through one reference row when the decay from that row to the block's last row
  // stays under kDirectLimit; for b = 64 the reference is the chunk start (decay total of the chunk),
  // which makes the gated read keys of that case the operand Kd of W as well.
  float Glast[4];
  {
    float P[4] = {0.f, 0.f, 0.f, 0.f}, pre[4] = {0.f, 0.f, 0.f, 0.f};
    float f16[4], f32[4], dm16 = 0.f, dm32 = 0.f;
#pragma unroll
    for (int wp = 0; wp < 8; ++wp) {
      const float4 fr = *reinterpret_cast<const float4*>(sFirst + wp * kD + c4);
      const float4 to = *reinterpret_cast<const float4*>(sTot + wp * kD + c4);
      const float first[4] = {P[0] + fr.x, P[1] + fr.y, P[2] + fr.z, P[3] + fr.w};
      if (wp == warp) {
#pragma unroll
        for (int e = 0; e < 4; ++e) pre[e] = P[e];
        if (!kRecompute)
          *reinterpret_cast<float4*>(sGf + wp * kD + c4) = make_float4(first[0], first[1], first[2], first[3]);
      }
      P[0] += to.x; P[1] += to.y; P[2] += to.z; P[3] += to.w;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if ((wp & 1) == 0) f16[e] = first[e];
        if ((wp & 3) == 0) f32[e] = first[e];
        if ((wp & 1) == 1) dm16 = fmaxf(dm16, f16[e] - P[e]);
        if ((wp & 3) == 3) dm32 = fmaxf(dm32, f32[e] - P[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) Glast[e] = P[e];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) G[i][e] += pre[e];
    if (!kRecompute) {
      float dm[6] = {0.f, 0.f, 0.f, dm16, dm32, 0.f};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) dm[0] = fmaxf(dm[0], G[i][e] - G[i + 1][e]);
        dm[1] = fmaxf(dm[1], fmaxf(G[0][e] - G[3][e], G[4][e] - G[7][e]));
        dm[2] = fmaxf(dm[2], G[0][e] - G[7][e]);
        dm[5] = fmaxf(dm[5], -Glast[e]);
      }
#pragma unroll
      for (int k6 = 0; k6 < 6; ++k6) {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) dm[k6] = fmaxf(dm[k6], __shfl_xor_sync(0xffffffffu, dm[k6], o));
        if (lane == 0) sWmax[warp * 6 + k6] = dm[k6];
      }
    }
  }

  PKDA_PHASE(24);
  // ---- 3. preconditioner states of this strip's rows -> write keys kt = k * B(A_t) (into the slots g
  // has left, and to global memory), kg = kt * decay to the chunk end; diagonal q_i . kt_i
  {
    float A[4] = {a_first.x, a_first.y, a_first.z, a_first.w};
    if (!kRecompute) {
      for (int b = 0; b < warp; ++b) {
        const float d = sDec[b];
        const float4 e4 = *reinterpret_cast<const float4*>(sEnd + b * kD + c4);
        A[0] = d * A[0] + e4.x; A[1] = d * A[1] + e4.y; A[2] = d * A[2] + e4.z; A[3] = d * A[3] + e4.w;
      }
    }
    float dg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint2 kt = ktraw[i];
      if (!kRecompute) {
        const float pd = __shfl_sync(0xffffffffu, sc_pd, i), bp = __shfl_sync(0xffffffffu, sc_bp, i);
        const uint2 kr = ld_k(i);
        float kc[4], f[4];
        unpack4(kr, kc);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          A[e] = pd * A[e] + bp * kc[e] * kc[e];
          const float dev = __logf(A[e] + p.eps) - centre;
          f[e] = __expf(-p.ln_x * __fdividef(dev, 1.f + fabsf(dev)));
        }
        kt = scale4(kr, f);
        *reinterpret_cast<uint2*>(yBase + slot_off(i)) = kt;
        if (r0 + i < valid) *reinterpret_cast<uint2*>(p.kt + row0 + (size_t)(r0 + i) * gld + c4) = kt;
        float kc2[4], qc[4];
        unpack4(kt, kc2);
        unpack4(ld_q(i), qc);
        dg[i] = qc[0] * kc2[0] + qc[1] * kc2[1] + qc[2] * kc2[2] + qc[3] * kc2[3];
      }
      float tl[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) tl[e] = ex2(Glast[e] - G[i][e]);
      if (r0 + i < valid) *reinterpret_cast<uint2*>(p.kg + row0 + (size_t)(r0 + i) * gld + c4) = scale4(kt, tl);
    }
    if (!kRecompute) {
      row_sums8(dg, lane);
      if ((lane & 3) == 0) sDiag[r0 + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)] = dg[0];
      if (warp == 0)
        *reinterpret_cast<float4*>(p.gc + chh * kD + c4) =
            make_float4(ex2(Glast[0]), ex2(Glast[1]), ex2(Glast[2]), ex2(Glast[3]));
    }
  }
  PKDA_PHASE(25);
  __syncthreads(); PKDA_PHASE(2);  // the strip exchange arrays are dead: L takes their place

  bool ok = true;
  uint32_t mma_phase = 0;
  const int R = 32 * (warp & 3) + lane;     // this thread's accumulator row in the pair products
  const int ei = R & 63, j0 = 32 * (warp >> 2);
  const bool isP = (warp & 3) >= 2;
  constexpr uint32_t idesc_pair = tc::idesc_bf16(128, 64, false, false);
  const int bdir = kRecompute ? 0 : pick_direct_block(sWmax, 8, p.direct_cap);
  if (!kRecompute && bdir == 64) {
    // ---- 4a. the whole chunk is one direct block: reference = chunk start.  One pass writes
    // Kd = k 2^G (rows 0..63 of the stacked operand, and later the operand of W^T), q 2^G
    // (rows 64..127), the write keys times 2^-G, and qg; nothing of the strip is needed afterwards.
    {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float e[4], es[4], fi[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          e[c] = ex2(G[i][c]);
          es[c] = e[c] * p.scale;
          fi[c] = __fdividef(1.f, e[c]);
        }
        const int off = slot_off(i);
        const uint2 qr = ld_q(i);
        *reinterpret_cast<uint2*>(aBase + off) = scale4(ld_k(i), e);
        *reinterpret_cast<uint2*>(aBase + 8192 + off) = scale4(qr, e);
        *reinterpret_cast<uint2*>(yBase + off) = scale4(ld_y(i), fi);
        if (r0 + i < valid) *reinterpret_cast<uint2*>(p.qg + row0 + (size_t)(r0 + i) * gld + c4) = scale4(qr, es);
      }
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads(); PKDA_PHASE(3);
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t a = tc::desc_kmajor(base + oA + (kk >> 2) * 16384 + (kk & 3) * 32);
        const uint64_t b = tc::desc_kmajor(base + oY + (kk >> 2) * 8192 + (kk & 3) * 32);
        tc::umma_bf16(tmem, a, b, idesc_pair, kk > 0);
      }
      tc::umma_commit(bar_mma);
    }
    ok = tc::mbar_wait(bar_mma, mma_phase) && ok;
    mma_phase ^= 1;
    tc::tc_fence_after();
    PKDA_PHASE(4);
    {
      float acc[32];
      tc::tmem_ld32(tmem + ((uint32_t)(32 * (warp & 3)) << 16) + j0, acc);
      tc::tmem_ld_wait();
      if (!isP) {  // L = tril(M, -1) diag(beta)
#pragma unroll
        for (int t = 0; t < 32; ++t) sL[ei * kLdL + j0 + t] = (j0 + t < ei) ? acc[t] * sBeta[j0 + t] : 0.f;
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
    PKDA_PHASE(5);
  } else {
  // ---- 4b. gated pair products, level by level.  Every level gates the raw rows anew, so this path
  // takes them out of their slots into registers first.
  uint2 kraw[8], qraw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    kraw[i] = ld_k(i);
    qraw[i] = ld_q(i);
    if (!kRecompute) ktraw[i] = ld_y(i);
  }
  if (!kRecompute) {
    bool first_level = true;
#pragma unroll 1
    for (int it = (bdir > 1 ? 0 : 1); it <= 6; ++it) {
      const int lvl = it ? (64 >> it) : 0;  // 0 (direct), 32, 16, 8, 4, 2, 1
      if (lvl && lvl < bdir) break;
      // -- stage this level's operands
      {
        const bool own_ref = lvl ? (lvl < 8) : (bdir <= 8);
        float gbig[4] = {0.f, 0.f, 0.f, 0.f};
        if (!own_ref) {
          const int refrow = lvl ? ((r0 & ~(2 * lvl - 1)) + lvl) : (r0 & ~(bdir - 1));
          const float4 g4 = *reinterpret_cast<const float4*>(sGf + (refrow >> 3) * kD + c4);
          gbig[0] = g4.x; gbig[1] = g4.y; gbig[2] = g4.z; gbig[3] = g4.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float gref[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float own;
            if (lvl == 0) own = bdir == 8 ? G[0][e] : (bdir == 4 ? G[i & ~3][e] : G[i & ~1][e]);
            else own = lvl == 4 ? G[4][e] : (lvl == 2 ? G[(i & ~3) + 2][e] : G[(i & ~1) + 1][e]);
            gref[e] = own_ref ? own : gbig[e];
          }
          const bool upper = lvl ? (((r0 + i) & lvl) != 0) : true;
          const float sgn = upper ? 1.f : -1.f;
          float f[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) f[e] = ex2(sgn * (G[i][e] - gref[e]));
          const int off = slot_off(i);
          if (upper) {
            *reinterpret_cast<uint2*>(aBase + off) = scale4(kraw[i], f);
            *reinterpret_cast<uint2*>(aBase + 8192 + off) = scale4(qraw[i], f);
            if (!lvl) {  // direct level: the same row is also a column operand, factor 1/f
              float fi[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) fi[e] = __fdividef(1.f, f[e]);
              *reinterpret_cast<uint2*>(yBase + off) = scale4(ktraw[i], fi);
            }
          } else {
            *reinterpret_cast<uint2*>(yBase + off) = scale4(ktraw[i], f);
          }
        }
      }
      tc::fence_proxy_async();
      tc::tc_fence_before();
      __syncthreads(); PKDA_PHASE(3);
      if (tid == 0) {
        tc::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a = tc::desc_kmajor(base + oA + (kk >> 2) * 16384 + (kk & 3) * 32);
          const uint64_t b = tc::desc_kmajor(base + oY + (kk >> 2) * 8192 + (kk & 3) * 32);
          tc::umma_bf16(tmem, a, b, idesc_pair, kk > 0);
        }
        tc::umma_commit(bar_mma);
      }
      ok = tc::mbar_wait(bar_mma, mma_phase) && ok;
      mma_phase ^= 1;
      tc::tc_fence_after();
      PKDA_PHASE(4);
      // -- read the accumulator back: row ei of M (L = M diag(beta), strictly lower) or of P,
      // sixteen columns at a time (the strip registers stay live through the level loop)
#pragma unroll
      for (int hq = 0; hq < 2; ++hq) {
        float acc[16];
        const int jq = j0 + 16 * hq;
        tc::tmem_ld16(tmem + ((uint32_t)(32 * (warp & 3)) << 16) + jq, acc);
        tc::tmem_ld_wait();
        if (!isP) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const int j = jq + t;
            const bool pok = pair_ok(ei, j, lvl, bdir);
            if (pok) sL[ei * kLdL + j] = acc[t] * sBeta[j];
            else if (first_level) sL[ei * kLdL + j] = 0.f;
          }
        } else {
          unsigned char* prow = tiles + oP + ei * 128;
          if (first_level) {
            const float dv = sDiag[ei];
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
              float x[8];
#pragma unroll
              for (int t = 0; t < 8; ++t) {
                const int j = jq + 8 * pc + t;
                x[t] = pair_ok(ei, j, lvl, bdir) ? acc[8 * pc + t] * p.scale : (j == ei ? dv * p.scale : 0.f);
              }
              *reinterpret_cast<uint4*>(prow + ((((jq >> 3) + pc) ^ (ei & 7)) << 4)) =
                  make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
            }
          } else {
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              const int j = jq + t;
              if (pair_ok(ei, j, lvl, bdir))
                *reinterpret_cast<bf16*>(prow + (((j >> 3) ^ (ei & 7)) << 4) + (j & 7) * 2) =
                    __float2bfloat16(acc[t] * p.scale);
            }
          }
        }
      }
      first_level = false;
      tc::tc_fence_before();
      PKDA_PHASE(5);
    }
  }

  // ---- 5. decayed operands: Kd -> rows 0..63 of the stacked operand (operand of W^T); qg -> global
  {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float e[4], es[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        e[c] = ex2(G[i][c]);
        es[c] = e[c] * p.scale;
      }
      *reinterpret_cast<uint2*>(aBase + slot_off(i)) = scale4(kraw[i], e);
      if (r0 + i < valid) *reinterpret_cast<uint2*>(p.qg + row0 + (size_t)(r0 + i) * gld + c4) = scale4(qraw[i], es);
    }
  }
  }
  ok = tc::mbar_wait(bar_tma, 0) && ok;  // V (and T) landed long ago
  if (!full) {  // rows past the sequence end hold another sequence's data: they must not reach the product
    for (int idx = tid; idx < kChunk * 16; idx += kThreads) {
      const int r = idx >> 4, pc = idx & 15;
      if (r >= valid)
        *reinterpret_cast<uint4*>(tiles + oV + (pc >> 3) * 8192 + r * 128 + ((pc & 7) << 4)) = make_uint4(0, 0, 0, 0);
    }
  }
  tc::fence_proxy_async();
  __syncthreads(); PKDA_PHASE(6);

  if (!kRecompute) {
    // ---- 6. scaled P -> Aqk;  T = (I + L)^-1 -> bf16 operand tile and Akk
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
    unit_lower_inverse_64(sL, sT, reinterpret_cast<float*>(tiles + oY2), kLdL, tid, kThreads);  // ends with a barrier
    PKDA_PHASE(7);
    for (int idx = tid; idx < kChunk * 8; idx += kThreads) {
      const int r = idx >> 3, pc = idx & 7;
      const float* src = sT + r * kLdL + 8 * pc;
      const uint4 pk = make_uint4(pack_bf16(src[0], src[1]), pack_bf16(src[2], src[3]), pack_bf16(src[4], src[5]),
                                  pack_bf16(src[6], src[7]));
      *reinterpret_cast<uint4*>(tiles + oTm + r * 128 + ((pc ^ (r & 7)) << 4)) = pk;
      if (!full && r < valid)
        *reinterpret_cast<uint4*>(p.Akk + ((size_t)(tok0 + r) * H + h) * kChunk + 8 * pc) = pk;
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads(); PKDA_PHASE(8);
  }

  // ---- 7. W^T = Kd^T T^T, U^T = V^T T^T
  if (tid == 0) {
    tc::tc_fence_after();
    if (!kRecompute && full) {
      tc::tma_store_3d(&tm_akk, base + oTm, 0, h, tok0);
      tc::bulk_commit();
    }
    constexpr uint32_t idesc = tc::idesc_bf16(128, 64, /*a_mn_major=*/true, /*b_mn_major=*/false);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      tc::umma_bf16(tmem + 64, tc::desc_mnmajor(base + oA + kk * 2048, 16384), tc::desc_kmajor(base + oTm + kk * 32),
                    idesc, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      tc::umma_bf16(tmem + 128, tc::desc_mnmajor(base + oV + kk * 2048, 8192), tc::desc_kmajor(base + oTm + kk * 32),
                    idesc, kk > 0);
    tc::umma_commit(bar_mma);
  }
  ok = tc::mbar_wait(bar_mma, mma_phase) && ok;
  tc::tc_fence_after();
  PKDA_PHASE(9);
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
  const bool all_ok = !__syncthreads_or(!ok);
  PKDA_PHASE(10);
  if (tid == 0) {
    if (!all_ok) atomicExch(p.status, 1);
    if (full && all_ok) {
      tc::tma_store_3d(&tm_w, base + oA, 0, h, tok0);
      tc::tma_store_3d(&tm_w, base + oA + 8192, 64, h, tok0);
      tc::tma_store_3d(&tm_u, base + oA + 16384, 0, h, tok0);
      tc::tma_store_3d(&tm_u, base + oA + 16384 + 8192, 64, h, tok0);
      tc::bulk_commit();
    }
    tc::bulk_wait_read();  // the tiles stay in place until every store of this CTA has read them
  }
  if (warp == 1) tc::tmem_dealloc(tmem, kCols);
  PKDA_PHASE(11);
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
  const dim3 grid(ip.geo.total_chunks, ip.geo.heads);
  // two CTAs per SM need the largest shared-memory carve-out
  cudaFuncSetAttribute(pkda_intra_fwd_tc_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
  cudaFuncSetAttribute(pkda_intra_fwd_tc_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
  if (recompute) {
    if (cudaFuncSetAttribute(pkda_intra_fwd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             intratc::kSmem) != cudaSuccess)
      return PKDA_ERR_LAUNCH;
    pkda_intra_fwd_tc_kernel<true><<<grid, intratc::kThreads, intratc::kSmem, st>>>(tm_v, tm_akk, tm_aqk, tm_w, tm_u, ip);
  } else {
    if (cudaFuncSetAttribute(pkda_intra_fwd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             intratc::kSmem) != cudaSuccess)
      return PKDA_ERR_LAUNCH;
    pkda_intra_fwd_tc_kernel<false><<<grid, intratc::kThreads, intratc::kSmem, st>>>(tm_v, tm_akk, tm_aqk, tm_w, tm_u, ip);
  }
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda

#ifdef PKDA_PHASE_PROFILE
extern "C" int pkda_phase_prof_intratc(long long* out) {
  return cudaMemcpyFromSymbol(out, g_phase_prof, sizeof(long long) * 64) == cudaSuccess ? 0 : 1;
}
#endif
