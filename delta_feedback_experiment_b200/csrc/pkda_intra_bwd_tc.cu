// Chunk-parallel stage of the chunked backward on tcgen05 / tensor memory (D = 128, chunk 64).
//
// Persistent CTAs of 512 threads (one per SM) walk a list of (chunk, head) items; all operand
// tiles of an item (about 216 KB) sit in shared memory at once, every one of them placed by TMA
// in the 128-byte-swizzled layout the tensor core reads, and every dense product is a
// tcgen05.mma chain into tensor memory.  The tiles of the next item are requested as soon as the
// current item's last read of them is over, so they land while the gate's backward runs.  The
// list holds the chunks that are full (64 tokens) and whose decay lets the whole chunk be ONE
// direct block (pkda_chunk.cuh): there the gated operands are q 2^G, k 2^G and kt 2^-G with G the
// cumulative log2-decay from the chunk start, one set for all pairs.  A small kernel in front
// (pkda_bwd_classify_kernel) sorts the chunks: every other chunk (a ragged last chunk, a chunk
// that decays by more than kDirectLimit, a capped direct block) goes on a second list, which the
// mma.sync kernel of pkda_chunk_bwd.cu works off right after this one.
//
// Accumulators are laid out with one value / key channel per tensor-memory lane and tokens along
// the columns (M = 128 channels everywhere, N = 64 tokens), so a thread owns one channel and 16
// consecutive tokens for all elementwise work: the gate and its cumulative sum, the gating of the
// operands (in place in the tiles), the gradient epilogue, the reverse cumulative sum of the
// log-decay gradient and the gate's own backward need no transposition, only one exchange
// between the four token slices of a channel.
//
//   (1) dR^T  = dF^T (diag(beta) T)                      K = 64    -> dv, and rows 0..63 of the stack
//   (2) [dR; dO] E^T                                     K = 128   -> dM = -tril(.,-1) diag(beta),
//                                                                     dP = scale tril(.) diag(beta)
//       Qs = S0 dO^T, Ks = -S0 dR^T, Kts = dS1 E^T       K = 128   (state-coupled parts)
//   (3) Qp = Y^T dP^T, Kp = Y^T dM^T, KtM = Xk^T dM, KtP = Xq^T dP   K = 64 (pair parts)
//   dq  = 2^G (scale Qs + Qp)      dk_read = 2^G (Ks + Kp)
//   dkt = 2^-G (2^G_last beta Kts + KtM + KtP)
//   dG  = Xq (scale Qs + Qp) + Xk (Ks + Kp) - Y (2^G_last beta Kts + KtM + KtP)
// with Xq = bf16(q 2^G), Xk = bf16(k 2^G), Y = bf16(kt 2^-G) the very operands of the products, so
// that the two sides of every pair cancel under the reverse cumulative sum.
//
// The kernel also takes the local part of the preconditioner's backward along (kt = k B(A_t) with the
// diagonal state A_t = decay_t A_(t-1) + gain_t k_t^2): it has dkt in registers, reloads the raw k
// tile into the dead state tile and recomputes A_t per channel, so the gradient buffers leave as
// dA_local (in the dkt buffer) and dk_read + dkt B, and the chunk-parallel reverse scan that follows
// (pkda_atk_bwd_kernel<true>) needs no transcendental.
//
// Every mbarrier wait is bounded; a CTA whose wait gives up sets the status word.
#include "pkda_chunk.cuh"
#include "pkda_tc.cuh"


namespace pkda {

namespace ibtc {
constexpr int kThreads = 512;
constexpr int oS0 = 0;                  // [128 c][128 v] chunk-entry state           (K-major A)
constexpr int oDS = oS0 + 32768;        // [128 c][128 v] cotangent of the exit state (K-major A)
constexpr int oStk = oDS + 32768;       // [128][128 v]: rows 0..63 dR, rows 64..127 dO (K-major A, and K-major B by halves)
constexpr int oDF = oStk + 32768;       // [64 j][128 v] dF                            (MN-major A)
constexpr int oE = oDF + 16384;         // [64 j][128 v] E                             (K-major B)
constexpr int oQ = oE + 16384;          // [64 i][128 c] q, then Xq                    (MN-major A)
constexpr int oK = oQ + 16384;          // [64 i][128 c] k, then Xk                    (MN-major A)
constexpr int oKt = oK + 16384;         // [64 j][128 c] kt, then Y                    (MN-major A)
constexpr int oG = oKt + 16384;         // [64][128 c] raw gate
constexpr int oTm = oG + 16384;         // [64 j][64 i] T, then diag(beta) T           (MN-major B)
constexpr int oDM = oTm + 8192;         // [64 i][64 j] dM                             (K-major / MN-major B)
constexpr int oDP = oDM + 8192;         // [64 i][64 j] dP
constexpr int oSmall = oDP + 8192;      // f32: beta[64] | x1[4][128] | x2[4][128] | red[32] | pd[64] | bp[64] | 1/beta[64] | slice decays[4]
constexpr int oBar = oSmall + 256 + 2048 + 2048 + 128 + 512 + 256 + 64;  // barriers A, B, C, M, K and the tensor-memory address
constexpr int kSmem = oBar + 64 + 1024;
static_assert(kSmem <= 232448, "shared memory of one SM");
// after the last product: exchange arrays in the (dead) pair-gradient tiles
constexpr int oX3 = oDM;                // f32 [4][128] slice sums of dG
constexpr int oX4 = oDM + 2048;         // f32 [4][128] slice sums of kt dkt (state part)
constexpr int oX5 = oDM + 4096;         // f32 [4][128] slice sums of the raw-gate gradient
constexpr int oDb = oDM + 6144;         // f32 [4][64] per lane-quarter partial sums of dbeta
constexpr int oX6 = oDP;                // f32 [4][128] slice sums of the preconditioner's outgoing carry
constexpr uint32_t kCols = 512;
constexpr uint32_t cR = 0, cStk = 64, cQs = 128, cKs = 192, cKts = 256, cKtM = 320, cKtP = 384;  // cR / cStk later Qp / Kp
}  // namespace ibtc

// Sums each of v[0..15] over the 32 lanes.  On return lane l holds in v[0] the total of entry
// ((l >> 4) & 1) * 8 + ((l >> 3) & 1) * 4 + ((l >> 2) & 1) * 2 + ((l >> 1) & 1).
__device__ __forceinline__ void row_sums16(float (&v)[16], int lane) {
  const bool b16 = lane & 16, b8 = lane & 8, b4 = lane & 4, b2 = lane & 2;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float keep = b16 ? v[j + 8] : v[j], send = b16 ? v[j] : v[j + 8];
    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float keep = b8 ? v[j + 4] : v[j], send = b8 ? v[j] : v[j + 4];
    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float keep = b4 ? v[j + 2] : v[j], send = b4 ? v[j] : v[j + 2];
    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
  {
    const float keep = b2 ? v[1] : v[0], send = b2 ? v[0] : v[1];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

// One bf16 element of shared memory by its 32-bit shared address (register + immediate addressing).
__device__ __forceinline__ float lds_bf16(uint32_t addr) {
  unsigned short u;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(u) : "r"(addr));
  return __uint_as_float((uint32_t)u << 16);
}
__device__ __forceinline__ void sts_bf16(uint32_t addr, float x) {
  const bf16 b = __float2bfloat16(x);
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<const unsigned short*>(&b)) : "memory");
}

struct IntraBwdTcMaps {
  CUtensorMap h, dh, d_o, dF, E, q, k, kt, g, Akk, dv;
};

// Sorts the (chunk, head) items of a backward call into the two work lists.  One warp per item
// reads the chunk's decay totals (128 floats); a CTA appends its items with one atomic per list.
// It is the backward's first kernel and also packs beta chunk-major.
__global__ void __launch_bounds__(256)
pkda_bwd_classify_kernel(Geo geo, const float* gc, int direct_cap, int* fast_list, int* slow_list, int* counts,
                         const bf16* beta, float* beta_c) {
  __shared__ int sKind[64];
  __shared__ int sBase[2];
  const int H = geo.heads, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int items = geo.total_chunks * H;
  // a warp's eight items: every load of all eight is issued before the first is used
  float4 x[8];
  float bv[8][2];
  int tok0s[8], valids[8];
  bool live[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int chh = blockIdx.x * 64 + warp * 8 + k;
    int n;
    live[k] = chh < items && chunk_lookup(geo, chh / H, n, tok0s[k], valids[k]);
    x[k] = make_float4(1.f, 1.f, 1.f, 1.f);
    bv[k][0] = bv[k][1] = 0.f;
    if (live[k]) {
      x[k] = *reinterpret_cast<const float4*>(gc + (size_t)chh * kD + 4 * lane);
      const int h = chh % H;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int r = lane + 32 * j;
        if (r < valids[k]) bv[k][j] = to_f(beta[(size_t)(tok0s[k] + r) * H + h]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int local = warp * 8 + k, chh = blockIdx.x * 64 + local;
    int kind = -1;  // -1: not an item, 0: tensor-memory kernel, 1: mma.sync kernel
    if (live[k]) {
      float m = fminf(fminf(x[k].x, x[k].y), fminf(x[k].z, x[k].w));
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) m = fminf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const bool fast = valids[k] == kChunk && direct_cap >= 64 && m > 0.f && -__log2f(m) <= kDirectLimit;
      kind = fast ? 0 : 1;
      // the chunk-major fp32 copy of beta that every later stage reads (saves the packing launch)
      beta_c[(size_t)chh * kChunk + lane] = bv[k][0];
      beta_c[(size_t)chh * kChunk + lane + 32] = bv[k][1];
    }
    if (lane == 0) sKind[local] = kind;
  }
  append_work_items(sKind, sBase, fast_list, slow_list, counts, blockIdx.x * 64, tid);
}

__global__ void __launch_bounds__(ibtc::kThreads, 1)
pkda_intra_bwd_tc_kernel(const IntraBwdParams p, const __grid_constant__ IntraBwdTcMaps maps) {
  using namespace ibtc;
  extern __shared__ unsigned char smem_raw[];
  const int n_items = *p.fast_count;
  if ((int)blockIdx.x >= n_items) return;
  const int H = p.geo.heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, sl = warp >> 2;      // lane quarter of tensor memory; token slice
  const int c = 32 * q4 + lane;                 // this thread's channel (= tensor-memory lane)
  const int j0 = 16 * sl;                       // first of its 16 tokens
  const uint32_t lane_addr = (uint32_t)(32 * q4) << 16;
  const size_t gld = (size_t)H * kD;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t barA = base + oBar, barB = barA + 8, barC = barA + 16, barM = barA + 24, barK = barA + 32;
  const uint32_t tmem_slot = barA + 48;
  // Shared address of element (token j0 + t, channel c) of a [64][128] tile at offset o: sa[t & 7] + o + 128 t
  // (the 16-byte pieces of a row are permuted by the row index modulo 8).
  uint32_t sa[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) sa[k] = base + sw128_offset(k, c, 8192) - 128 * k + j0 * 128;
  float* sBeta = reinterpret_cast<float*>(tiles + oSmall);
  float* sX1 = sBeta + 64;     // [4][128] slice totals of the gate
  float* sX2 = sX1 + 512;      // [4][128] slice partials of sum_v S0 dS1
  float* sRed = sX2 + 512;     // [32]: 16 warp sums of dA_log, 16 of the centre gradient
  float* sPd = sRed + 32;      // [64] preconditioner decay exp(g_atk) per token
  float* sBp = sPd + 64;       // [64] preconditioner gain beta_atk per token
  float* sBinv = sBp + 64;     // [64] 1 / beta (0 where beta is 0)
  float* sDsl = sBinv + 64;    // [4] product of the preconditioner decays of each 16-token slice
  float* sX3 = reinterpret_cast<float*>(tiles + oX3);
  float* sX4 = reinterpret_cast<float*>(tiles + oX4);
  float* sX5 = reinterpret_cast<float*>(tiles + oX5);
  float* sDb = reinterpret_cast<float*>(tiles + oDb);
  float* sX6 = reinterpret_cast<float*>(tiles + oX6);

  // All tiles of one item by TMA.  Thread 0 arms the three barriers with the byte counts (arm), a
  // CTA-wide barrier later the 20 copies are issued by the first lanes of the 16 warps (request), so
  // that no single thread spends a thousand cycles issuing them.
  auto arm = [&]() {
    tc::mbar_expect_tx(barB, 8192 + 3 * 16384 + 256);
    tc::mbar_expect_tx(barA, 4 * 16384);
    tc::mbar_expect_tx(barC, 2 * 32768);
  };
  auto request = [&](int item) {
    if (lane != 0) return;  // (the barriers were armed by arm() before the preceding CTA-wide barrier)
    const int chh = p.fast_list[item];
    const int h = chh % H;
    int n, tok0, valid;
    chunk_lookup(p.geo, chh / H, n, tok0, valid);
    const int srow = chh * kD;
    if (warp == 0) {
      tc::tma_load_3d(base + oTm, &maps.Akk, barB, 0, h, tok0);
      tc::bulk_load(base + oSmall, p.beta_c + (size_t)chh * kChunk, 256, barB);
    }
    const int kb = warp & 1;
    switch (warp >> 1) {
      case 0: tc::tma_load_3d(base + oDF + kb * 8192, &maps.dF, barB, 64 * kb, h, tok0); break;
      case 1: tc::tma_load_3d(base + oE + kb * 8192, &maps.E, barB, 64 * kb, h, tok0); break;
      case 2: tc::tma_load_3d(base + oStk + kb * 16384 + 8192, &maps.d_o, barB, 64 * kb, h, tok0); break;
      case 3: tc::tma_load_3d(base + oG + kb * 8192, &maps.g, barA, 64 * kb, h, tok0); break;
      case 4: tc::tma_load_3d(base + oQ + kb * 8192, &maps.q, barA, 64 * kb, h, tok0); break;
      case 5: tc::tma_load_3d(base + oK + kb * 8192, &maps.k, barA, 64 * kb, h, tok0); break;
      case 6: tc::tma_load_3d(base + oKt + kb * 8192, &maps.kt, barA, 64 * kb, h, tok0); break;
      default:
        tc::tma_load_2d(base + oS0 + kb * 16384, &maps.h, barC, 64 * kb, srow);
        tc::tma_load_2d(base + oDS + kb * 16384, &maps.dh, barC, 64 * kb, srow);
        break;
    }
  };

  if (tid == 0) {
    tc::mbar_init(barA, 1);
    tc::mbar_init(barB, 1);
    tc::mbar_init(barC, 1);
    tc::mbar_init(barM, 1);
    tc::mbar_init(barK, 1);
    tc::fence_barrier_init();
    arm();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, kCols);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  request(blockIdx.x);
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tiles + oBar + 48);
  bool ok = true;
  uint32_t m_phase = 0, ld_phase = 0;
  // per-item scalars of this thread, fetched one item ahead: 2^G_last of its channel, the gate bias, A_log
  float gl_n, bias_n, alog_n, astart_n, centre_n, gatk_n = 0.f, batk_n = 0.f;
  int chh_n;
  auto fetch_scalars = [&](int item) {
    const int chh = p.fast_list[item], h = chh % H;
    chh_n = chh;
    gl_n = p.gc[(size_t)chh * kD + c];
    bias_n = p.dt_bias[h * kD + c];
    alog_n = p.A_log[h];
    astart_n = p.a_start[(size_t)chh * kD + c];
    centre_n = p.log_atk_scale[h];
    if (tid < kChunk) {  // the preconditioner's per-token controls
      int n, tok0, valid;
      chunk_lookup(p.geo, chh / H, n, tok0, valid);
      const size_t s = (size_t)(tok0 + tid) * H + h;
      gatk_n = p.g_atk[s];
      batk_n = to_f(p.beta_atk[s]);
    }
  };
  fetch_scalars(blockIdx.x);

#pragma unroll 1
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
  const int chh = chh_n;
  const int h = chh % H;
  int n, tok0, valid;
  chunk_lookup(p.geo, chh / H, n, tok0, valid);  // a full chunk (the classifier checked)
  const float gl = gl_n, bias = bias_n, ea = __expf(alog_n), a_start = astart_n, centre = centre_n;
  if (tid < kChunk) {
    sPd[tid] = __expf(gatk_n);
    sBp[tid] = batk_n;
  }
  // The operand descriptors are functions of the tile base only; keeping the base opaque per item
  // stops the compiler from computing all sixty of them ahead of the loop and holding them in registers.
  uint32_t dbase = base;
  asm volatile("" : "+r"(dbase));

  // ---- 1. T <- diag(beta) T (row j scaled by beta_j: the beta of dE = beta dF moves onto T), then dR^T
  ok = tc::mbar_wait(barB, ld_phase) && ok;
  if (tid < kChunk) {
    const float b = sBeta[tid];
    sBinv[tid] = b != 0.f ? __fdividef(1.f, b) : 0.f;
  }
  {
    const int j = tid >> 3, pc = tid & 7;
    uint4* piece = reinterpret_cast<uint4*>(tiles + oTm + j * 128 + (pc << 4));  // a whole row takes one factor
    const float b = sBeta[j];
    const float f[8] = {b, b, b, b, b, b, b, b};
    uint4 x = *piece;
    scale8(x, f);
    *piece = x;
  }
  tc::fence_proxy_async();
  __syncthreads();
  if (tid == 0) {
    tc::tc_fence_after();
    constexpr uint32_t idesc = tc::idesc_bf16(128, 64, true, true);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      tc::umma_bf16(tmem + cR, tc::desc_mnmajor(dbase + oDF + kk * 2048, 8192), tc::desc_mnmajor(dbase + oTm + kk * 2048, 8192),
                    idesc, kk > 0);
    tc::umma_commit(barM);
  }
  if (warp == 15 && lane < 4) {  // (multiplied in token order, once, instead of by every thread)
    float d = 1.f;
#pragma unroll
    for (int t = 0; t < 16; ++t) d *= sPd[16 * lane + t];
    sDsl[lane] = d;
  }

  // ---- 2. while that runs: the gate, its cumulative sum over the tokens, the operands gated in place
  ok = tc::mbar_wait(barA, ld_phase) && ok;
  float G[16], G_before;  // cumulative log2-decay of the 16 tokens, and of the token before them
  {
    const float ea2 = ea * kLog2e;
    float run = 0.f;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      run += -ea2 * softplus_fast(lds_bf16(sa[t & 7] + oG + 128 * t) + bias);
      G[t] = run;
    }
    sX1[sl * kD + c] = run;
  }
  __syncthreads();
  {
    float pre = 0.f;
#pragma unroll
    for (int s = 0; s < 3; ++s) pre += (s < sl) ? sX1[s * kD + c] : 0.f;
#pragma unroll
    for (int t = 0; t < 16; ++t) G[t] += pre;
    G_before = pre;
  }
  // the state-coupled products that need nothing but landed tiles
  ok = tc::mbar_wait(barC, ld_phase) && ok;
  ld_phase ^= 1;
  if (tid == 0) {
    tc::tc_fence_after();
    constexpr uint32_t idesc = tc::idesc_bf16(128, 64, false, false);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t ko = (kk >> 2) * 16384 + (kk & 3) * 32;
      tc::umma_bf16(tmem + cQs, tc::desc_kmajor(dbase + oS0 + ko), tc::desc_kmajor(dbase + oStk + 8192 + ko), idesc, kk > 0);
    }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t ko = (kk >> 2) * 16384 + (kk & 3) * 32, ke = (kk >> 2) * 8192 + (kk & 3) * 32;
      tc::umma_bf16(tmem + cKts, tc::desc_kmajor(dbase + oDS + ko), tc::desc_kmajor(dbase + oE + ke), idesc, kk > 0);
    }
  }

  // ---- 3. dR^T -> bf16 -> rows 0..63 of the stack (it is dv as it stands)
  ok = tc::mbar_wait(barM, m_phase) && ok;
  m_phase ^= 1;
  tc::tc_fence_after();
  {
    float acc[16];
    tc::tmem_ld16(tmem + lane_addr + cR + j0, acc);
    tc::tmem_ld_wait();
#pragma unroll
    for (int t = 0; t < 16; ++t) sts_bf16(sa[t & 7] + oStk + (c >> 6) * 8192 + 128 * t, acc[t]);  // K blocks 16 KB apart
  }
  tc::fence_proxy_async();
  tc::tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc::tc_fence_after();
    tc::tma_store_3d(&maps.dv, base + oStk, 0, h, tok0);
    tc::tma_store_3d(&maps.dv, base + oStk + 16384, 64, h, tok0);
    tc::bulk_commit();
    constexpr uint32_t idesc = tc::idesc_bf16(128, 64, false, false);
    constexpr uint32_t idesc_neg = idesc | (1u << 13);  // A negated
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {  // [dR; dO] E^T
      const uint32_t ko = (kk >> 2) * 16384 + (kk & 3) * 32, ke = (kk >> 2) * 8192 + (kk & 3) * 32;
      tc::umma_bf16(tmem + cStk, tc::desc_kmajor(dbase + oStk + ko), tc::desc_kmajor(dbase + oE + ke), idesc, kk > 0);
    }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {  // -S0 dR^T
      const uint32_t ko = (kk >> 2) * 16384 + (kk & 3) * 32;
      tc::umma_bf16(tmem + cKs, tc::desc_kmajor(dbase + oS0 + ko), tc::desc_kmajor(dbase + oStk + ko), idesc_neg, kk > 0);
    }
    tc::umma_commit(barM);
  }

  // ---- 3b. while those run: the operands gated in place; sum_v S0 dS1 per channel
  {
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const float e = ex2(G[t]), ei = __fdividef(1.f, e);
      const uint32_t a0 = sa[t & 7] + 128 * t;
      sts_bf16(a0 + oQ, lds_bf16(a0 + oQ) * e);
      sts_bf16(a0 + oK, lds_bf16(a0 + oK) * e);
      sts_bf16(a0 + oKt, lds_bf16(a0 + oKt) * ei);
    }
    // channel c's row of both state tiles, values 32 sl .. 32 sl + 31 (four 16-byte pieces of one K block)
    const unsigned char* rs = tiles + oS0 + (sl >> 1) * 16384 + c * 128;
    const unsigned char* rd = tiles + oDS + (sl >> 1) * 16384 + c * 128;
    float acc = 0.f;
    // (unrolled by two on purpose: fully unrolled, the schedule the compiler picks for this kernel at its
    // register limit costs 7 % of its time, with movable or with pinned loads; rolled up, 1 %.  Measured.)
#pragma unroll 2
    for (int pc = 0; pc < 4; ++pc) {
      const int po = (((4 * (sl & 1) + pc) ^ (c & 7)) << 4);
      const uint4 a = *reinterpret_cast<const uint4*>(rs + po), b = *reinterpret_cast<const uint4*>(rd + po);
      const uint32_t* a32 = reinterpret_cast<const uint32_t*>(&a);
      const uint32_t* b32 = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = unpack_bf16(a32[e]), y = unpack_bf16(b32[e]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
    sX2[sl * kD + c] = acc;
  }

  // ---- 4. pair-weight gradients: row i of dM = -tril(dR E^T, -1) diag(beta), of dP = scale tril(dO E^T) diag(beta)
  ok = tc::mbar_wait(barM, m_phase) && ok;
  m_phase ^= 1;
  tc::tc_fence_after();
  {
    float acc[16];
    tc::tmem_ld16(tmem + lane_addr + cStk + j0, acc);
    tc::tmem_ld_wait();
    const bool isP = c >= 64;
    const int i = c & 63;
    float x[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const int j = j0 + t;
      const float b = sBeta[j];
      x[t] = isP ? (j <= i ? acc[t] * b * p.scale : 0.f) : (j < i ? -acc[t] * b : 0.f);
    }
    unsigned char* row = tiles + (isP ? oDP : oDM) + i * 128;
    *reinterpret_cast<uint4*>(row + (((2 * sl) ^ (i & 7)) << 4)) =
        make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
    *reinterpret_cast<uint4*>(row + (((2 * sl + 1) ^ (i & 7)) << 4)) =
        make_uint4(pack_bf16(x[8], x[9]), pack_bf16(x[10], x[11]), pack_bf16(x[12], x[13]), pack_bf16(x[14], x[15]));
  }
  tc::fence_proxy_async();  // also covers the gated operands written in step 2
  tc::tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc::tc_fence_after();
    // the raw k tile comes back into the (dead) entry-state tile for the preconditioner's backward
    tc::mbar_expect_tx(barK, 16384);
    tc::tma_load_3d(base + oS0, &maps.k, barK, 0, h, tok0);
    tc::tma_load_3d(base + oS0 + 8192, &maps.k, barK, 64, h, tok0);
    constexpr uint32_t idesc_k = tc::idesc_bf16(128, 64, true, false);  // B = pair gradient as [i][j], K = j
    constexpr uint32_t idesc_m = tc::idesc_bf16(128, 64, true, true);   // B = pair gradient read as [j][i], K = i
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint64_t ay = tc::desc_mnmajor(dbase + oKt + kk * 2048, 8192);
      tc::umma_bf16(tmem + cR, ay, tc::desc_kmajor(dbase + oDP + kk * 32), idesc_k, kk > 0);    // Qp = Y^T dP^T
      tc::umma_bf16(tmem + cStk, ay, tc::desc_kmajor(dbase + oDM + kk * 32), idesc_k, kk > 0);  // Kp = Y^T dM^T
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      tc::umma_bf16(tmem + cKtM, tc::desc_mnmajor(dbase + oK + kk * 2048, 8192), tc::desc_mnmajor(dbase + oDM + kk * 2048, 8192),
                    idesc_m, kk > 0);  // Xk^T dM
      tc::umma_bf16(tmem + cKtP, tc::desc_mnmajor(dbase + oQ + kk * 2048, 8192), tc::desc_mnmajor(dbase + oDP + kk * 2048, 8192),
                    idesc_m, kk > 0);  // Xq^T dP
    }
    tc::umma_commit(barM);
  }

  // ---- 5a. preconditioner state at the start of this thread's token slice: zero-start scan of the slice,
  // one exchange, then the slices before it folded in (a slice's decay product is the same for all channels)
  ok = tc::mbar_wait(barK, ld_phase ^ 1) && ok;  // (ld_phase was flipped after this item's tile waits)
  float A_in, w_in = 1.f;  // state before the slice's first token; product of the decays before it
  {
    float a = 0.f;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const float kc = lds_bf16(sa[t & 7] + oS0 + 128 * t);
      a = sPd[j0 + t] * a + sBp[j0 + t] * kc * kc;
    }
    sX1[sl * kD + c] = a;  // (the gate totals that lived here were consumed in step 2)
    __syncthreads();
    A_in = a_start;
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const float d = sDsl[s];
      if (s < sl) {
        A_in = d * A_in + sX1[s * kD + c];
        w_in *= d;
      }
    }
  }

  // the four pair products ran while the slice states were formed
  ok = tc::mbar_wait(barM, m_phase) && ok;
  m_phase ^= 1;
  tc::tc_fence_after();

  // ---- 5b. gradients of this thread's channel and 16 tokens, four tokens at a time (the accumulator
  // pieces stay small next to the per-token state)
  const size_t out0 = ((size_t)(tok0 + j0) * H + h) * kD + c;  // element (first token of the slice, h, c)
  float dGv[16], kdsum = 0.f, cloc = 0.f, dcen = 0.f;
  {
    bf16* pq = p.dq + out0;  // walked row by row (running pointers keep the row offsets out of registers)
    float* pk = p.dk_read + out0;
    float* pkt = p.dkt + out0;
    float A = A_in, w = w_in;
    float dbv[8];
#pragma unroll
    for (int qq = 0; qq < 4; ++qq) {  // four tokens at a time: all seven accumulator pieces of a token in one pass
      const uint32_t ta = tmem + lane_addr + j0 + 4 * qq;
      float aQ[4], bR[4], aK[4], bS[4], m[4], bP[4], aT[4];
      tc::tmem_ld4(ta + cQs, aQ);
      tc::tmem_ld4(ta + cR, bR);
      tc::tmem_ld4(ta + cKs, aK);
      tc::tmem_ld4(ta + cStk, bS);
      tc::tmem_ld4(ta + cKtM, m);
      tc::tmem_ld4(ta + cKtP, bP);
      tc::tmem_ld4(ta + cKts, aT);
      tc::tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int t = 4 * qq + u;
        const uint32_t a0 = sa[t & 7] + 128 * t;
        const float e = ex2(G[t]);
        const float totq = p.scale * aQ[u] + bR[u];
        const float xq = lds_bf16(a0 + oQ);
        *pq = __float2bfloat16(e * totq);
        pq += gld;
        const float totk = aK[u] + bS[u];
        const float xk = lds_bf16(a0 + oK);
        const float dkr = e * totk;
        // write-key gradient; the part of dbeta that flows through M (rows of KtM against Y)
        const float bj = sBeta[j0 + t];
        const float y = lds_bf16(a0 + oKt);
        const float df = lds_bf16(a0 + oDF);
        const float ev = lds_bf16(a0 + oE);
        dbv[4 * (qq & 1) + u] = df * ev + y * m[u] * sBinv[j0 + t];
        const float st = gl * bj * aT[u], pr = m[u] + bP[u];
        const float dkt = __fdividef(st + pr, e);
        const float kd = y * st;
        dGv[t] = xq * totq + xk * totk - (y * pr + kd);
        kdsum += kd;
        // the preconditioner: A_t, the factor B(A_t) and its derivative (pkda_atk_bwd_kernel has the same math)
        const float kc = lds_bf16(a0 + oS0);
        const float pd = sPd[j0 + t];
        A = pd * A + sBp[j0 + t] * kc * kc;
        w *= pd;
        const float dev = __logf(A + p.eps) - centre;
        const float rden = __fdividef(1.f, 1.f + fabsf(dev));
        const float Bf = __expf(-p.ln_x * dev * rden);
        const float ddev = -p.ln_x * dkt * kc * Bf * rden * rden;
        const float dA = __fdividef(ddev, A + p.eps);
        *pkt = dA;
        pkt += gld;
        *pk = dkr + dkt * Bf;
        pk += gld;
        dcen -= ddev;
        cloc += w * dA;
      }
      if (qq & 1) {
        row_sums8(dbv, lane);
        if ((lane & 3) == 0)
          sDb[q4 * kChunk + j0 + 8 * (qq >> 1) + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)] = dbv[0];
      }
    }
    float tot = 0.f;
#pragma unroll
    for (int t = 0; t < 16; ++t) tot += dGv[t];
    sX3[sl * kD + c] = tot;     // the pair-gradient tiles are dead: every product has finished
    sX4[sl * kD + c] = kdsum;
    sX6[sl * kD + c] = cloc;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) dcen += __shfl_xor_sync(0xffffffffu, dcen, o);
    if (lane == 0) sRed[16 + warp] = dcen;
  }
  tc::tc_fence_before();
  tc::fence_proxy_async();  // this item's last reads of the operand tiles come before the next item's copies
  if (tid == 0 && item + (int)gridDim.x < n_items) arm();
  __syncthreads();
  // every tile except the stack rows the dv store is reading is free: the next item's tiles start to
  // arrive while the gate's backward runs
  if (item + (int)gridDim.x < n_items) {
    request(item + gridDim.x);
    fetch_scalars(item + gridDim.x);
  }
  // reverse cumulative sum over the tokens (the chunk's last row also takes the decay-total terms),
  // then the gate's own backward:  g = -exp(A_log) softplus(raw + bias)
  {
    float run = gl * (sX2[c] + sX2[kD + c] + sX2[2 * kD + c] + sX2[3 * kD + c]) + sX4[c] + sX4[kD + c] + sX4[2 * kD + c] +
                sX4[3 * kD + c];
#pragma unroll
    for (int s = 1; s < 4; ++s) run += (s > sl) ? sX3[s * kD + c] : 0.f;
    // softplus and sigmoid of (raw + bias) come back from the per-token decay the forward part of this
    // kernel summed up: G_t - G_(t-1) = -exp(A_log) log2(e) softplus, and sigmoid = 1 - exp(-softplus)
    float pa = 0.f, pb = 0.f;
    bf16* pg = p.dg + out0 + 15 * gld;
    const float inv_ea = __fdividef(1.f, ea), inv_ea2 = inv_ea * kLn2;
#pragma unroll
    for (int t = 15; t >= 0; --t) {
      run += dGv[t];
      const float dlog2 = G[t] - (t ? G[t - 1] : G_before);  // <= 0
      const float sp = -dlog2 * inv_ea2;
      const float sg = 1.f - ex2(dlog2 * inv_ea);
      const float dr = run * (-ea) * sg;
      pa += run * (-ea * sp);
      pb += dr;
      *pg = __float2bfloat16(dr);
      pg -= gld;
    }
    sX5[sl * kD + c] = pb;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) pa += __shfl_xor_sync(0xffffffffu, pa, o);
    if (lane == 0) sRed[warp] = pa;
  }
  if (tid < kChunk)
    p.dbeta[(size_t)(tok0 + tid) * H + h] =
        __float2bfloat16(sDb[tid] + sDb[kChunk + tid] + sDb[2 * kChunk + tid] + sDb[3 * kChunk + tid]);
  __syncthreads();
  if (tid < kD) {
    p.partB[(size_t)chh * kD + tid] = sX5[tid] + sX5[kD + tid] + sX5[2 * kD + tid] + sX5[3 * kD + tid];
    p.c_loc[(size_t)chh * kD + tid] = sX6[tid] + sX6[kD + tid] + sX6[2 * kD + tid] + sX6[3 * kD + tid];
  }
  if (tid == 0) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) acc += sRed[w];
    p.partA[chh] = acc;
    float accc = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) accc += sRed[16 + w];
    p.partC[chh] = accc;
    tc::bulk_wait_read();  // the dv store has read the stack rows the next item's dR overwrites
  }
  __syncthreads();  // the exchange arrays and beta are rewritten by the next item
  }  // item loop
  if (__syncthreads_or(!ok) && tid == 0) atomicExch(p.status, 1);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) tc::tmem_dealloc(tmem, kCols);
}

// ------------------------------------------------------------------ host side
int launch_bwd_classify(const Geo& geo, const float* gc, int direct_cap, int* fast_list, int* slow_list, int* counts,
                        const bf16* beta, float* beta_c, cudaStream_t st) {
  const int items = geo.total_chunks * geo.heads;
  begin_stage(kStageBwdClassify, st);
  pkda_bwd_classify_kernel<<<(items + 63) / 64, 256, 0, st>>>(geo, gc, direct_cap, fast_list, slow_list, counts, beta,
                                                             beta_c);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

int launch_intra_bwd_tc(const IntraBwdParams& ip, cudaStream_t st) {
  const uint64_t H = ip.geo.heads, tok = ip.geo.total_tokens, rows = (uint64_t)ip.geo.total_chunks * H * kD;
  IntraBwdTcMaps maps;
  {
    const uint64_t dims[3] = {kD, H, tok}, str[2] = {kD * 2, H * kD * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&maps.d_o, ip.d_o, 3, dims, str, box) || !encode_bf16_map(&maps.dF, ip.dF, 3, dims, str, box) ||
        !encode_bf16_map(&maps.E, ip.v_new, 3, dims, str, box) || !encode_bf16_map(&maps.q, ip.q, 3, dims, str, box) ||
        !encode_bf16_map(&maps.k, ip.k, 3, dims, str, box) || !encode_bf16_map(&maps.kt, ip.kt, 3, dims, str, box) ||
        !encode_bf16_map(&maps.g, ip.g, 3, dims, str, box) || !encode_bf16_map(&maps.dv, ip.dv, 3, dims, str, box))
      return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {kChunk, H, tok}, str[2] = {kChunk * 2, H * kChunk * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&maps.Akk, ip.Akk, 3, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {kD, rows}, str[1] = {kD * 2};
    const uint32_t box[2] = {64, 128};
    if (!encode_bf16_map(&maps.h, ip.h, 2, dims, str, box) || !encode_bf16_map(&maps.dh, ip.dh, 2, dims, str, box))
      return PKDA_ERR_LAUNCH;
  }
  if (!ensure_dynamic_smem(pkda_intra_bwd_tc_kernel, ibtc::kSmem))
    return PKDA_ERR_LAUNCH;
  const int items = ip.geo.total_chunks * ip.geo.heads;
  begin_stage(kStageIntraBwd, st);
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  pkda_intra_bwd_tc_kernel<<<items < sms ? items : sms, ibtc::kThreads, ibtc::kSmem, st>>>(ip, maps);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda

