// Chunked PKDA backward for D = 128, chunk 64, bf16 activations.
//
// With the forward's per-chunk quantities (see pkda_chunk_fwd.cu)
//   E = Tm (V - Kd S0), F = beta E, O = qg S0 + P F, S1 = Gam_last S0 + kg^T F
// the cotangents are
//   dF = kg dS1 + P^T dO,  dE = beta dF,  dS0 = Gam_last dS1 + qg^T dO - W^T dE
//   dR = Tm^T dE (= dV),  dKd = -dR S0^T,  d(tril M) = -tril(dR E^T) diag(beta)
//   dP = scale tril(dO F^T),  dkg = F dS1^T,  dqg = dO S0^T
// and the gated pair products are differentiated level by level with the same
// rounded operands on both sides, so that each pair's +/- contributions to the
// log-decay gradient cancel exactly under the reverse cumulative sum.
//
// Pipeline:  [recompute forward stages]  scan_bwd (sequential over chunks)
//   -> intra_bwd (per chunk) -> atk_bwd local / carry / final (preconditioner
//   reverse scan, chunk-parallel) -> param_reduce.
#include <algorithm>

#include "pkda_chunk.cuh"
#include "pkda_tc.cuh"

namespace pkda {

// ------------------------------------------------------------------ reverse state scan
struct ScanBwdParams {
  Geo geo;
  const bf16 *kg, *qg, *w, *Aqk, *d_o;
  const float *beta_c, *gc;
  const float* dST;
  bf16 *dh, *dF;
  float* dS0;
};

namespace scanb {
template <int VB> __host__ __device__ constexpr int threads() { return 128 * (VB / 32); }  // 4 warps per 32 value columns
template <int VB> struct L {
  static constexpr int ldv = VB + kPad;
  static constexpr int oKg = 0;
  static constexpr int oP = oKg + kTileBytes;            // bf16 [64][72]
  static constexpr int oBeta = oP + kChunk * kLdC * 2;   // f32 [64]
  static constexpr int oQg = oBeta + kChunk * 4;
  static constexpr int oW = oQg + kTileBytes;
  static constexpr int oGc = oW + kTileBytes;            // f32 [128]
  static constexpr int oDo = oGc + kD * 4;               // 2 x bf16 [64][ldv]
  static constexpr int kDoBytes = kChunk * ldv * 2;
  static constexpr int oD = oDo + 2 * kDoBytes;          // bf16 [128][ldv]
  static constexpr int oDE = oD + kD * ldv * 2;          // bf16 [64][ldv]
  static constexpr int kSmem = oDE + kChunk * ldv * 2;
};
}  // namespace scanb

template <int VB>
__global__ void __launch_bounds__(scanb::threads<VB>())
pkda_scan_bwd_kernel(const ScanBwdParams p) {
  using Lay = scanb::L<VB>;
  constexpr int ldv = Lay::ldv, NT = 4, kT = scanb::threads<VB>();
  extern __shared__ __align__(128) unsigned char smem[];
  const int VS = kD / VB;
  const int vs = blockIdx.x % VS;
  const int nh = blockIdx.x / VS;
  const int n = nh / p.geo.heads, h = nh - n * p.geo.heads, H = p.geo.heads;
  const SeqInfo sq = seq_info(p.geo, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int wr = warp & 3, c0 = 32 * (warp >> 2);  // this warp: rows [32 wr, +32), columns [c0, +32) of the slice
  const int v0 = vs * VB;
  const long gld = (long)H * kD;
  const size_t sbase = ((size_t)n * H + h) * kD * kD;

  bf16* sKg = reinterpret_cast<bf16*>(smem + Lay::oKg);
  bf16* sP = reinterpret_cast<bf16*>(smem + Lay::oP);
  float* sBeta = reinterpret_cast<float*>(smem + Lay::oBeta);
  bf16* sQg = reinterpret_cast<bf16*>(smem + Lay::oQg);
  bf16* sW = reinterpret_cast<bf16*>(smem + Lay::oW);
  float* sGc = reinterpret_cast<float*>(smem + Lay::oGc);
  bf16* sD = reinterpret_cast<bf16*>(smem + Lay::oD);
  bf16* sDE = reinterpret_cast<bf16*>(smem + Lay::oDE);

  auto prefetchA = [&](int i) {
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t row0 = ((size_t)tok0 * H + h) * kD;
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    tile_load_async(sKg, kLdD, p.kg + row0, gld, kChunk, kD, valid, kT);
    tile_load_async(sP, kLdC, p.Aqk + ((size_t)tok0 * H + h) * kChunk, (long)H * kChunk, kChunk, kChunk, valid,
                    kT);
    tile_load_async(reinterpret_cast<bf16*>(smem + Lay::oDo + (i & 1) * Lay::kDoBytes), ldv, p.d_o + row0 + v0, gld,
                    kChunk, VB, valid, kT);
    if (tid < 16) cp_async16(smem + Lay::oBeta + tid * 16, p.beta_c + chh * kChunk + tid * 4, true);
  };
  auto prefetchB = [&](int i) {
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t row0 = ((size_t)tok0 * H + h) * kD;
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    tile_load_async(sQg, kLdD, p.qg + row0, gld, kChunk, kD, valid, kT);
    tile_load_async(sW, kLdD, p.w + row0, gld, kChunk, kD, valid, kT);
    if (tid < 32) cp_async16(smem + Lay::oGc + tid * 16, p.gc + chh * kD + tid * 4, true);
  };

  float dS[2][NT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = 32 * wr + 16 * mt + gq + 8 * half, c = v0 + c0 + 8 * nt + 2 * tq;
        float2 s2 = make_float2(0.f, 0.f);
        if (p.dST) s2 = *reinterpret_cast<const float2*>(p.dST + sbase + (size_t)r * kD + c);
        dS[mt][nt][2 * half] = s2.x;
        dS[mt][nt][2 * half + 1] = s2.y;
      }

  const int last = sq.nchunks - 1;
  if (last >= 0) {
    prefetchA(last);
    cp_async_commit();
    prefetchB(last);
    cp_async_commit();
  }
  for (int i = last; i >= 0; --i) {
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    const bf16* sdO = reinterpret_cast<const bf16*>(smem + Lay::oDo + (i & 1) * Lay::kDoBytes);
    cp_async_wait<1>();  // group A(i) has landed
    // a. chunk-exit state cotangent -> bf16 operand tile (and the saved dh)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 32 * wr + 16 * mt + gq + 8 * half, c = c0 + 8 * nt + 2 * tq;
          *reinterpret_cast<uint32_t*>(sD + r * ldv + c) = pack_bf16(dS[mt][nt][2 * half], dS[mt][nt][2 * half + 1]);
        }
    __syncthreads();
    {
      constexpr int cpr = VB / 8;
      for (int j = tid; j < kD * cpr; j += kT) {
        const int r = j / cpr, c = (j - r * cpr) * 8;
        *reinterpret_cast<uint4*>(p.dh + (chh * kD + r) * kD + v0 + c) =
            *reinterpret_cast<const uint4*>(sD + r * ldv + c);
      }
    }
    // c. dF = kg dS1 + P^T dO ;  -dE = -beta dF
    {
      float f[1][NT][4];
      zero_acc(f);
      warp_gemm<1, NT, false, true>(f, sKg, kLdD, 16 * wr, sD, ldv, c0, 0, kD);
      warp_gemm<1, NT, true, true>(f, sP, kLdC, 16 * wr, sdO, ldv, c0, 16 * wr, kChunk);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 16 * wr + gq + 8 * half, c = c0 + 8 * nt + 2 * tq;
          const uint32_t fk = pack_bf16(f[0][nt][2 * half], f[0][nt][2 * half + 1]);
          if (r < valid) *reinterpret_cast<uint32_t*>(p.dF + ((size_t)(tok0 + r) * H + h) * kD + v0 + c) = fk;
          const float2 fr = unpack_bf16(fk);
          const float b = sBeta[r];
          *reinterpret_cast<uint32_t*>(sDE + r * ldv + c) = pack_bf16(-b * fr.x, -b * fr.y);
        }
    }
    __syncthreads();  // group-A buffers free
    if (i > 0) prefetchA(i - 1);
    cp_async_commit();
    cp_async_wait<1>();  // group B(i) has landed
    __syncthreads();
    // d. dS0 = Gam_last dS1 + qg^T dO - W^T dE
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float gcv = sGc[32 * wr + 16 * mt + gq + 8 * half];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          dS[mt][nt][2 * half] *= gcv;
          dS[mt][nt][2 * half + 1] *= gcv;
        }
      }
    warp_gemm<2, NT, true, true>(dS, sQg, kLdD, 32 * wr, sdO, ldv, c0, 0, kChunk);
    warp_gemm<2, NT, true, true>(dS, sW, kLdD, 32 * wr, sDE, ldv, c0, 0, kChunk);
    __syncthreads();  // group-B buffers, sD and sDE free
    if (i > 0) prefetchB(i - 1);
    cp_async_commit();
  }
  cp_async_wait<0>();
  if (p.dS0) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 32 * wr + 16 * mt + gq + 8 * half, c = v0 + c0 + 8 * nt + 2 * tq;
          *reinterpret_cast<float2*>(p.dS0 + sbase + (size_t)r * kD + c) =
              make_float2(dS[mt][nt][2 * half], dS[mt][nt][2 * half + 1]);
        }
  }
}

// ------------------------------------------------------------------ chunk-parallel backward
// Tensor maps of the phase-A tiles.  Each box is wider than the data it needs (136
// or 72 columns for 128 or 64) so that the rows land in shared memory with the
// padded pitch the ldmatrix reads want; the surplus columns are the neighbouring
// head's data or, past the end of a row, zero fill.
// The four output maps are [token][head][channel] with a box of one head and 136
// columns: a store clips the eight columns past the head, so the padded pitch of
// the shared-memory tile never reaches the neighbouring head.
struct IntraBwdMaps {
  CUtensorMap d_o, dF, h, dh, Akk, E;
  CUtensorMap dq, dv, dk_read, dkt;
};

namespace ib {
constexpr int kThreads = 512;
constexpr int oA0 = 0;                        // dO          | later q
constexpr int oA1 = kTileBytes;               // S0 [128][136] | E | later k, kt
constexpr int oG = oA1 + 2 * kTileBytes;      // f32 [64][kLdG] log2-domain cumulative decay
constexpr int oTm = oG + kChunk * kLdG * 4;   // bf16 [64][72]
constexpr int oDE = oTm + kChunk * kLdC * 2;  // dE | later F = beta E
constexpr int oDR = oDE + kTileBytes;
constexpr int oStage = oTm;                   // three gated operand tiles | later dG f32 [64][128]
constexpr int oDP = oStage + 3 * kTileBytes;  // bf16 [64][72]
constexpr int oDM = oDP + kChunk * kLdC * 2;
constexpr int oFac = oDM + kChunk * kLdC * 2; // f32 [64][kLdG]
constexpr int oSmall = oFac + kChunk * kLdG * 4;
// small: beta[64] db[64] hdh[128] gcv[128] col[4][128] rb[4][64] red[16] bias[128] warpmax[4][6]
constexpr int kSmallFloats = 64 + 64 + 128 + 128 + 512 + 256 + 16 + 128 + 24;
constexpr int oBar = oSmall + kSmallFloats * 4;  // one mbarrier
constexpr int kSmem = oBar + 16;
constexpr uint32_t kTmaBytes = (3 * kChunk + 2 * kD) * kLdD * 2 + kChunk * kLdC * 2;  // dO, dF, E, S0, dS1 and Tm tiles
static_assert(2 * kChunk * kLdC * 2 >= kTileBytes && oDP % 128 == 0, "E waits in the pair-gradient tiles");
static_assert(oBar % 8 == 0 && oA1 % 128 == 0 && oTm % 128 == 0 && oDE % 128 == 0 && oFac % 128 == 0,
              "TMA destinations and the mbarrier must be aligned");
static_assert(oDR + kTileBytes <= oDP, "phase-A tiles must not reach the pair-gradient tiles");
static_assert(oDE + kD * kLdD * 2 <= oDP, "dS1 tile must fit");
}  // namespace ib

// acc += fac * t and dG += sign * x * t on one warp's [16 x 32] fragment
// (i0 = first row + lane/4, c0 = first column + 2*(lane%4)); fac is the fp32
// level factor of each row (kInverse: its reciprocal, the column factor of the
// direct level), x the staged bf16 operand the product was formed with.
template <bool kInverse>
__device__ __forceinline__ void epi_add(float (&acc)[1][4][4], float (&dG)[1][4][4], const float (&t)[1][4][4],
                                        const float* sFac, const bf16* sX, float sign, int i0, int c0) {
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = i0 + 8 * half, c = c0 + 8 * nt;
      float2 f = *reinterpret_cast<const float2*>(sFac + i * kLdG + c);
      if (kInverse) { f.x = __fdividef(1.f, f.x); f.y = __fdividef(1.f, f.y); }
      const float2 x = unpack_bf16(*reinterpret_cast<const uint32_t*>(sX + i * kLdD + c));
      const float t0 = t[0][nt][2 * half], t1 = t[0][nt][2 * half + 1];
      acc[0][nt][2 * half] += f.x * t0;
      acc[0][nt][2 * half + 1] += f.y * t1;
      dG[0][nt][2 * half] += sign * x.x * t0;
      dG[0][nt][2 * half + 1] += sign * x.y * t1;
    }
}

// One (chunk bx, head by) item; every thread of the CTA takes part.
__device__ __forceinline__ void intra_bwd_item(const IntraBwdParams& p, const IntraBwdMaps& maps, int bx, int by) {
  using namespace ib;
  extern __shared__ __align__(128) unsigned char smem[];
  bf16* sdO = reinterpret_cast<bf16*>(smem + oA0);
  bf16* sS0 = reinterpret_cast<bf16*>(smem + oA1);
  bf16* sE = reinterpret_cast<bf16*>(smem + oA1);
  bf16* sF = reinterpret_cast<bf16*>(smem + oDE);  // F = beta E takes the dE tile once that is dead
  float* sG = reinterpret_cast<float*>(smem + oG);
  bf16* sTm = reinterpret_cast<bf16*>(smem + oTm);
  bf16* sdE = reinterpret_cast<bf16*>(smem + oDE);
  bf16* sdR = reinterpret_cast<bf16*>(smem + oDR);
  bf16* sdP = reinterpret_cast<bf16*>(smem + oDP);
  bf16* sdM = reinterpret_cast<bf16*>(smem + oDM);
  float* sFac = reinterpret_cast<float*>(smem + oFac);
  float* sBeta = reinterpret_cast<float*>(smem + oSmall);
  float* sDb = sBeta + 64;
  float* sHdh = sDb + 64;
  float* sGcv = sHdh + 128;
  float* sCol = sGcv + 128;  // [4][128]
  float* sRb = sCol + 512;   // [4][64]
  float* sRed = sRb + 256;   // [16]
  float* sBias = sRed + 16;  // [128]
  float* sWarpMax = sBias + 128;  // [4][6]

  int n, tok0, valid;
  if (!chunk_lookup(p.geo, bx, n, tok0, valid)) return;
  const int h = by, H = p.geo.heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int I = warp & 3, cq = warp >> 2;
  const size_t chh = (size_t)bx * H + h;
  const size_t row0 = ((size_t)tok0 * H + h) * kD;
  const long gld = (long)H * kD;
  const size_t crow0 = ((size_t)tok0 * H + h) * kChunk;
  const long cld = (long)H * kChunk;

  // ================= phase A: state-coupled terms =================
  // The per-row scalars the first barrier waits for are requested before everything else.
  float s_small = 0.f;
  if (tid < kChunk) s_small = p.beta_c[chh * kChunk + tid];
  else if (tid >= 2 * kD && tid < 3 * kD) s_small = p.gc[chh * kD + tid - 2 * kD];
  else if (tid >= kD && tid < 2 * kD) s_small = p.dt_bias[h * kD + tid - kD];
  GateRaw<kThreads> graw;  // the raw gate is needed next
  gate_load(graw, p.g + row0, gld, valid, tid);
  // dS1 waits in the (not yet used) level-factor array until the dkg product, E in the (not yet
  // used) pair-gradient tiles until S0 has left the tile E belongs in
  bf16* sdSC = reinterpret_cast<bf16*>(smem + oFac);
  bf16* sEarly = reinterpret_cast<bf16*>(smem + oDP);
  // Full chunks: one thread starts five TMA tile copies and everybody goes on to the
  // gate computation while they land.  Ragged chunks (rows past the sequence end must
  // read as zero) take 16-byte cp.async copies.
  const bool by_tma = p.use_tma && valid == kChunk;
  const bool out_tma = by_tma && p.out_tma;  // gradients of full chunks leave by TMA from padded tiles
  const uint32_t bar = smem_u32(smem + oBar);
  if (by_tma) {
    if (tid == 0) {
      tc::mbar_init(bar, 1);
      tc::fence_barrier_init();
      tc::mbar_expect_tx(bar, kTmaBytes);
      tc::tma_load_2d(smem_u32(sdO), &maps.d_o, bar, h * kD, tok0);
      tc::tma_load_2d(smem_u32(sS0), &maps.h, bar, 0, (int)(chh * kD));
      tc::tma_load_2d(smem_u32(sTm), &maps.Akk, bar, h * kChunk, tok0);
      tc::tma_load_2d(smem_u32(sdE), &maps.dF, bar, h * kD, tok0);  // raw dF; scaled by beta below
      tc::tma_load_2d(smem_u32(sdSC), &maps.dh, bar, 0, (int)(chh * kD));
      tc::tma_load_2d(smem_u32(sEarly), &maps.E, bar, h * kD, tok0);
    }
  } else {
    tile_load_async(sdO, kLdD, p.d_o + row0, gld, kChunk, kD, valid, kThreads);
    tile_load_async(sS0, kLdD, p.h + chh * kD * kD, kD, kD, kD, kD, kThreads);
    tile_load_async(sTm, kLdC, p.Akk + crow0, cld, kChunk, kChunk, valid, kThreads);
    tile_load_async(sdE, kLdD, p.dF + row0, gld, kChunk, kD, valid, kThreads);
    tile_load_async(sdSC, kLdD, p.dh + chh * kD * kD, kD, kD, kD, kD, kThreads);
    tile_load_async(sEarly, kLdD, p.v_new + row0, gld, kChunk, kD, valid, kThreads);
    cp_async_commit();
  }
  if (tid < kChunk) sBeta[tid] = s_small;
  else if (tid >= 2 * kD && tid < 3 * kD) sGcv[tid - 2 * kD] = s_small;
  else if (tid >= kD && tid < 2 * kD) sBias[tid - kD] = s_small;
  __syncthreads();
  // log2-domain cumulative log-decay, exactly as the forward computes it
  gate_apply(graw, sG, valid, sBias, __expf(p.A_log[h]) * kLog2e, tid);
  __syncthreads();
  if (tid < kD) {
    gate_cumsum(sG, tid);
    float dmax[6];
    block_decay_max(sG, tid, dmax);
#pragma unroll
    for (int e = 0; e < 6; ++e) {
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) dmax[e] = fmaxf(dmax[e], __shfl_xor_sync(0xffffffffu, dmax[e], o));
      if (lane == 0) sWarpMax[warp * 6 + e] = dmax[e];
    }
  }
  if (by_tma) {
    if (!tc::mbar_wait(bar, 0) && tid == 0) atomicExch(p.status, 1);  // gave up: flag it, results are void
  } else {
    cp_async_wait<0>();
  }
  __syncthreads();
  // the direct part of dbeta, rowsum(dF * E), while dF is still unscaled; dE = beta * dF in place;
  // hdh[k] = sum_v S0[k][v] dS1[k][v] (four threads per state row)
  for (int i = tid; i < kChunk * kD / 8; i += kThreads) {
    const int r = i >> 4, c = (i & 15) << 3;
    const float b = sBeta[r];
    const float f[8] = {b, b, b, b, b, b, b, b};
    uint4 x = *reinterpret_cast<const uint4*>(sdE + r * kLdD + c);
    const uint4 ev = *reinterpret_cast<const uint4*>(sEarly + r * kLdD + c);
    const uint32_t* e32 = reinterpret_cast<const uint32_t*>(&ev);
    const uint32_t* f32 = reinterpret_cast<const uint32_t*>(&x);
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xe = unpack_bf16(e32[j]), y = unpack_bf16(f32[j]);
      part += xe.x * y.x + xe.y * y.y;
    }
    part += __shfl_xor_sync(0xffffffffu, part, 8);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    if ((i & 15) == 0) sDb[r] = part;
    scale8(x, f);
    *reinterpret_cast<uint4*>(sdE + r * kLdD + c) = x;
  }
  {
    const int row = tid >> 2, part = tid & 3;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 a = *reinterpret_cast<const uint4*>(sS0 + row * kLdD + part * 32 + 8 * j);
      const uint4 b = *reinterpret_cast<const uint4*>(sdSC + row * kLdD + part * 32 + 8 * j);
      const uint32_t* a32 = reinterpret_cast<const uint32_t*>(&a);
      const uint32_t* b32 = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = unpack_bf16(a32[e]), y = unpack_bf16(b32[e]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (part == 0) sHdh[row] = acc;
  }
  __syncthreads();

  float dQ[1][4][4], dK[1][4][4], dKt[1][4][4], dG[1][4][4];
  float t[1][4][4];
  // dqg = dO S0^T  ->  dq_a = scale * Gam * dqg
  zero_acc(t);
  warp_gemm<1, 4, false, false>(t, sdO, kLdD, 16 * I, sS0, kLdD, 32 * cq, 0, kD);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 16 * I + gq + 8 * (e >> 1), c = 32 * cq + 8 * nt + 2 * tq + (e & 1);
      dQ[0][nt][e] = t[0][nt][e] * p.scale * ex2(sG[i * kLdG + c]);
    }
  // dR = Tm^T dE  (= dV)
  zero_acc(t);
  warp_gemm<1, 4, true, true>(t, sTm, kLdC, 16 * I, sdE, kLdD, 32 * cq, 16 * I, kChunk);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = 16 * I + gq + 8 * half, c = 32 * cq + 8 * nt + 2 * tq;
      const uint32_t pk = pack_bf16(t[0][nt][2 * half], t[0][nt][2 * half + 1]);
      if (!out_tma && r < valid) *reinterpret_cast<uint32_t*>(p.dv + row0 + (size_t)r * gld + c) = pk;
      *reinterpret_cast<uint32_t*>(sdR + r * kLdD + c) = pk;
    }
  if (out_tma) tc::fence_proxy_async();
  __syncthreads();
  if (out_tma && tid == 0) {  // dv is the dR tile as it stands
    tc::tma_store_3d(&maps.dv, smem_u32(sdR), 0, h, tok0);
    tc::bulk_commit();
  }
  // dKd = -dR S0^T  ->  dk_a = Gam * dKd
  zero_acc(t);
  warp_gemm<1, 4, false, false>(t, sdR, kLdD, 16 * I, sS0, kLdD, 32 * cq, 0, kD);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 16 * I + gq + 8 * (e >> 1), c = 32 * cq + 8 * nt + 2 * tq + (e & 1);
      dK[0][nt][e] = -t[0][nt][e] * ex2(sG[i * kLdG + c]);
    }
  __syncthreads();  // S0 no longer needed
  // E moves into its operand tile (S0 has left it) and F = beta E into the dead dE tile
  for (int i = tid; i < kChunk * kD / 8; i += kThreads) {
    const int r = i >> 4, c = (i & 15) << 3;
    const uint4 ev = *reinterpret_cast<const uint4*>(sEarly + r * kLdD + c);
    const float b = sBeta[r];
    const uint32_t* e32 = reinterpret_cast<const uint32_t*>(&ev);
    uint4 bf;
    uint32_t* bf32 = reinterpret_cast<uint32_t*>(&bf);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = unpack_bf16(e32[j]);
      bf32[j] = pack_bf16(b * x.x, b * x.y);
    }
    *reinterpret_cast<uint4*>(sE + r * kLdD + c) = ev;
    *reinterpret_cast<uint4*>(sF + r * kLdD + c) = bf;
  }
  __syncthreads();
  // pair-weight gradients: dM = -tril(dR E^T, -1) diag(beta),  dP = scale tril(dO F^T)
  {
    const int J = cq;
    float t2[1][2][4];
    zero_acc(t2);
    if (J <= I) warp_gemm<1, 2, false, false>(t2, sdR, kLdD, 16 * I, sE, kLdD, 16 * J, 0, kD);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = 16 * I + gq + 8 * half, j = 16 * J + 8 * nt + 2 * tq;
        const float m0 = (j < i) ? -t2[0][nt][2 * half] * sBeta[j] : 0.f;
        const float m1 = (j + 1 < i) ? -t2[0][nt][2 * half + 1] * sBeta[j + 1] : 0.f;
        *reinterpret_cast<uint32_t*>(sdM + i * kLdC + j) = pack_bf16(m0, m1);
      }
    zero_acc(t2);
    if (J <= I) warp_gemm<1, 2, false, false>(t2, sdO, kLdD, 16 * I, sF, kLdD, 16 * J, 0, kD);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = 16 * I + gq + 8 * half, j = 16 * J + 8 * nt + 2 * tq;
        const float p0 = (j <= i) ? t2[0][nt][2 * half] * p.scale : 0.f;
        const float p1 = (j + 1 <= i) ? t2[0][nt][2 * half + 1] * p.scale : 0.f;
        *reinterpret_cast<uint32_t*>(sdP + i * kLdC + j) = pack_bf16(p0, p1);
      }
  }
  if (out_tma && tid == 0) tc::bulk_wait_read();  // the dv store has read the dR tile
  __syncthreads();  // dO, dR, E no longer needed
  // dkg = F dS1^T  ->  dkt_a = exp(G_last - G) * dkg
  // q, k and kt tiles of the pair-product phase land while the dkg product runs
  tile_load_async(reinterpret_cast<bf16*>(smem + oA0), kLdD, p.q + row0, gld, kChunk, kD, valid, kThreads);
  tile_load_async(reinterpret_cast<bf16*>(smem + oA1), kLdD, p.k + row0, gld, kChunk, kD, valid, kThreads);
  tile_load_async(reinterpret_cast<bf16*>(smem + oA1 + kTileBytes), kLdD, p.kt + row0, gld, kChunk, kD, valid, kThreads);
  cp_async_commit();
  zero_acc(t);
  warp_gemm<1, 4, false, false>(t, sF, kLdD, 16 * I, sdSC, kLdD, 32 * cq, 0, kD);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 16 * I + gq + 8 * (e >> 1), c = 32 * cq + 8 * nt + 2 * tq + (e & 1);
      dKt[0][nt][e] = t[0][nt][e] * ex2(sG[(kChunk - 1) * kLdG + c] - sG[i * kLdG + c]);
    }
  __syncthreads();

  // ================= phase B: gated pair products =================
  bf16* sQ = reinterpret_cast<bf16*>(smem + oA0);
  bf16* sK = reinterpret_cast<bf16*>(smem + oA1);
  bf16* sKt = reinterpret_cast<bf16*>(smem + oA1 + kTileBytes);
  bf16* sXq = reinterpret_cast<bf16*>(smem + oStage);
  bf16* sXk = sXq + kChunk * kLdD;
  bf16* sY = sXk + kChunk * kLdD;
  cp_async_wait<0>();
  __syncthreads();
  {
    // dG starts from the state-coupled parts; column sums of kt * dkt_a feed the
    // chunk's last row (d/dG_last of exp(G_last - G_j)).
    float cs[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      cs[nt][0] = cs[nt][1] = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 16 * I + gq + 8 * (e >> 1), c = 32 * cq + 8 * nt + 2 * tq + (e & 1);
        const float qv = to_f(sQ[i * kLdD + c]), kv = to_f(sK[i * kLdD + c]), ktv = to_f(sKt[i * kLdD + c]);
        const float kd = ktv * dKt[0][nt][e];
        dG[0][nt][e] = qv * dQ[0][nt][e] + kv * dK[0][nt][e] - kd;
        cs[nt][e & 1] += kd;
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        float v = cs[nt][b];
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (gq == 0) sCol[I * kD + 32 * cq + 8 * nt + 2 * tq + b] = v;
      }
  }
  // Rows a level does not write keep older contents; their products are removed
  // by zeroed pair weights, which only works on finite data (0 * NaN = NaN), so
  // the staging tiles start from zeros rather than from whatever phase A left.
  for (int i = tid; i < 3 * kTileBytes / 16; i += kThreads)
    reinterpret_cast<uint4*>(smem + oStage)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  float rb[2] = {0.f, 0.f};
  // Direct level (lvl = 0) for pairs inside a b-block, hierarchy levels >= b for the rest.
  const int bdir = pick_direct_block(sWarpMax, 4, p.direct_cap);
#pragma unroll 1
  for (int it = (bdir > 1 ? 0 : 1); it <= 6; ++it) {
    const int lvl = it ? (64 >> it) : 0;
    if (lvl && lvl < bdir) break;
    stage_level(sXq, sXk, sY, sQ, sK, sKt, sG, lvl, bdir, tid, kThreads, sFac);
    __syncthreads();
    const bool big = lvl >= 16;               // whole 16-row tiles are upper or lower: no masking
    const bool wide = !lvl && bdir >= 16;     // direct block made of whole tiles
    const int blk = lvl ? ((16 * I) & ~(2 * lvl - 1)) : ((16 * I) & ~(bdir - 1));
    if (!big || ((16 * I) & lvl)) {  // rows act as the upper ("i") side
      int kb = 16 * I, ke = 16 * I + 16;
      if (big) { kb = blk; ke = blk + lvl; }
      else if (wide) { kb = blk; }
      zero_acc(t);
      warp_gemm_lvl<4, false, true>(t, sdP, kLdC, 16 * I, sY, kLdD, 32 * cq, kb, ke, lvl, bdir, !big);
      epi_add<false>(dQ, dG, t, sFac, sXq, 1.f, 16 * I + gq, 32 * cq + 2 * tq);
      zero_acc(t);
      warp_gemm_lvl<4, false, true>(t, sdM, kLdC, 16 * I, sY, kLdD, 32 * cq, kb, ke, lvl, bdir, !big);
      epi_add<false>(dK, dG, t, sFac, sXk, 1.f, 16 * I + gq, 32 * cq + 2 * tq);
    }
    if (!big || !((16 * I) & lvl)) {  // rows act as the lower ("j") side
      int kb = 16 * I, ke = 16 * I + 16;
      if (big) { kb = blk + lvl; ke = kb + lvl; }
      else if (wide) { ke = blk + bdir; }
      zero_acc(t);
      warp_gemm_lvl<4, true, true>(t, sdM, kLdC, 16 * I, sXk, kLdD, 32 * cq, kb, ke, lvl, bdir, !big);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const float2 y = unpack_bf16(*reinterpret_cast<const uint32_t*>(
              sY + (16 * I + gq + 8 * half) * kLdD + 32 * cq + 8 * nt + 2 * tq));
          rb[half] += y.x * t[0][nt][2 * half] + y.y * t[0][nt][2 * half + 1];
        }
      warp_gemm_lvl<4, true, true>(t, sdP, kLdC, 16 * I, sXq, kLdD, 32 * cq, kb, ke, lvl, bdir, !big);
      if (lvl) epi_add<false>(dKt, dG, t, sFac, sY, -1.f, 16 * I + gq, 32 * cq + 2 * tq);
      else epi_add<true>(dKt, dG, t, sFac, sY, -1.f, 16 * I + gq, 32 * cq + 2 * tq);
    }
    __syncthreads();
  }
  // ungated diagonal of P
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 16 * I + gq + 8 * (e >> 1), c = 32 * cq + 8 * nt + 2 * tq + (e & 1);
      const float d = to_f(sdP[i * kLdC + i]);
      dQ[0][nt][e] += d * to_f(sKt[i * kLdD + c]);
      dKt[0][nt][e] += d * to_f(sQ[i * kLdD + c]);
    }
  // dbeta: direct part + <kt_j, dkt_j(M path)> / beta_j
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float v = rb[half];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    if (tq == 0) sRb[cq * kChunk + 16 * I + gq + 8 * half] = v;
  }
  // outputs of this stage; dG goes through shared memory for the reverse cumulative sum.
  // Full chunks send dq, dk_read and dkt through padded tiles in dead regions (q, k|kt and the
  // decay tile) and TMA stores; the scattered fragment stores of the direct path cost more
  // issue slots than the rest of this phase together.
  float* sdG = reinterpret_cast<float*>(smem + oStage);
  if (out_tma) {
    float* sOutKt = sG;  // the decay tile is dead after the level loop
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = 16 * I + gq + 8 * half, c = 32 * cq + 8 * nt + 2 * tq;
        *reinterpret_cast<float2*>(sOutKt + i * kLdG + c) = make_float2(dKt[0][nt][2 * half], dKt[0][nt][2 * half + 1]);
        *reinterpret_cast<float2*>(sdG + i * kLdG + c) = make_float2(dG[0][nt][2 * half], dG[0][nt][2 * half + 1]);
      }
    tc::fence_proxy_async();
  } else {
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = 16 * I + gq + 8 * half, c = 32 * cq + 8 * nt + 2 * tq;
        if (i < valid) {
          const size_t off = row0 + (size_t)i * gld + c;
          *reinterpret_cast<uint32_t*>(p.dq + off) = pack_bf16(dQ[0][nt][2 * half], dQ[0][nt][2 * half + 1]);
          *reinterpret_cast<float2*>(p.dk_read + off) = make_float2(dK[0][nt][2 * half], dK[0][nt][2 * half + 1]);
          *reinterpret_cast<float2*>(p.dkt + off) = make_float2(dKt[0][nt][2 * half], dKt[0][nt][2 * half + 1]);
        }
        *reinterpret_cast<float2*>(sdG + i * kLdG + c) = make_float2(dG[0][nt][2 * half], dG[0][nt][2 * half + 1]);
      }
  }
  __syncthreads();
  if (out_tma) {
    // every warp is past its reads of q and kt: their tiles take dq and dk_read
    if (tid == 0) {
      tc::tma_store_3d(&maps.dkt, smem_u32(sG), 0, h, tok0);
      tc::bulk_commit();
    }
    float* sOutK = reinterpret_cast<float*>(smem + oA1);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = 16 * I + gq + 8 * half, c = 32 * cq + 8 * nt + 2 * tq;
        *reinterpret_cast<uint32_t*>(sQ + i * kLdD + c) = pack_bf16(dQ[0][nt][2 * half], dQ[0][nt][2 * half + 1]);
        *reinterpret_cast<float2*>(sOutK + i * kLdG + c) = make_float2(dK[0][nt][2 * half], dK[0][nt][2 * half + 1]);
      }
    tc::fence_proxy_async();
  }
  // The raw gate of the tail phase is requested here, with the accumulators gone and the
  // reverse cumulative sum still to run: loaded where it is used, it cost the tail a full
  // memory round trip.
  constexpr int kIter = kChunk * kD / 8 / kThreads;
  uint4 raws[kIter];
#pragma unroll
  for (int it = 0; it < kIter; ++it) {
    const int r = (tid + it * kThreads) >> 4;
    raws[it] = make_uint4(0, 0, 0, 0);
    if (r < valid) raws[it] = *reinterpret_cast<const uint4*>(p.g + row0 + (size_t)r * gld + ((tid & 15) << 3));
  }
  if (tid < kChunk && tid < valid) {
    const float b = sBeta[tid];
    const float s = sRb[tid] + sRb[kChunk + tid] + sRb[2 * kChunk + tid] + sRb[3 * kChunk + tid];
    const float db = sDb[tid] + (b != 0.f ? s / b : 0.f);
    p.dbeta[(size_t)(tok0 + tid) * H + h] = __float2bfloat16(db);
  }
  // reverse cumulative sum over the chunk (one channel per thread, in place) ...
  if (tid < kD) {
    const int c = tid;
    float run = sCol[c] + sCol[kD + c] + sCol[2 * kD + c] + sCol[3 * kD + c] + sGcv[c] * sHdh[c];
#pragma unroll 8
    for (int r = kChunk - 1; r >= 0; --r) {
      run += sdG[r * kLdG + c];
      sdG[r * kLdG + c] = run;
    }
  }
  __syncthreads();
  if (out_tma && tid == 0) {
    tc::tma_store_3d(&maps.dq, smem_u32(sQ), 0, h, tok0);
    tc::tma_store_3d(&maps.dk_read, smem_u32(smem + oA1), 0, h, tok0);
    tc::bulk_commit();
  }
  // ... then the gate's own backward, elementwise over the tile with all threads:
  //   g = -exp(A_log) softplus(raw + bias);  draw = dg * (-exp(A_log)) sigmoid(raw + bias)
  // Per-thread partial sums (dA_log: scalar; ddt_bias: per channel) are reduced in a fixed order.
  float* sPart = sFac;  // [32][kLdG] per-(row group, channel) partials of ddt_bias (the factors are dead)
  {
    const float ea = __expf(p.A_log[h]);
    float pa = 0.f;
    float pb[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) pb[j] = 0.f;
    const int c8 = (tid & 15) << 3;
#pragma unroll
    for (int it = 0; it < kIter; ++it) {
      const int r = (tid + it * kThreads) >> 4;
      if (r < valid) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&raws[it]);
        const float4 d0 = *reinterpret_cast<const float4*>(sdG + r * kLdG + c8);
        const float4 d1 = *reinterpret_cast<const float4*>(sdG + r * kLdG + c8 + 4);
        const float dgv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
        uint4 outv;
        uint32_t* o32 = reinterpret_cast<uint32_t*>(&outv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 x = unpack_bf16(w[j]);
          const float z0 = x.x + sBias[c8 + 2 * j], z1 = x.y + sBias[c8 + 2 * j + 1];
          // sigmoid and softplus from one exp(-|z|): 1/(1+e) (or e/(1+e)) and max(z,0) - log(1/(1+e))
          const float e0 = __expf(-fabsf(z0)), e1 = __expf(-fabsf(z1));
          const float i0 = __fdividef(1.f, 1.f + e0), i1 = __fdividef(1.f, 1.f + e1);
          const float sg0 = z0 >= 0.f ? i0 : e0 * i0, sg1 = z1 >= 0.f ? i1 : e1 * i1;
          const float sp0 = fmaxf(z0, 0.f) - __logf(i0), sp1 = fmaxf(z1, 0.f) - __logf(i1);
          const float dr0 = dgv[2 * j] * (-ea) * sg0, dr1 = dgv[2 * j + 1] * (-ea) * sg1;
          pa += dgv[2 * j] * (-ea * sp0) + dgv[2 * j + 1] * (-ea * sp1);
          pb[2 * j] += dr0;
          pb[2 * j + 1] += dr1;
          o32[j] = pack_bf16(dr0, dr1);
        }
        *reinterpret_cast<uint4*>(p.dg + row0 + (size_t)r * gld + c8) = outv;
      }
    }
    // thread (tid >> 4) in 0..31 covers rows (tid >> 4) and (tid >> 4) + 32 of channel group c8
    *reinterpret_cast<float4*>(sPart + (tid >> 4) * kLdG + c8) = make_float4(pb[0], pb[1], pb[2], pb[3]);
    *reinterpret_cast<float4*>(sPart + (tid >> 4) * kLdG + c8 + 4) = make_float4(pb[4], pb[5], pb[6], pb[7]);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) pa += __shfl_xor_sync(0xffffffffu, pa, o);
    if (lane == 0) sRed[warp] = pa;
  }
  __syncthreads();
  if (tid < kD) {
    float acc = 0.f;
#pragma unroll 8
    for (int g = 0; g < 32; ++g) acc += sPart[g * kLdG + tid];
    p.partB[chh * kD + tid] = acc;
  }
  if (tid == 0) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) acc += sRed[w];
    p.partA[chh] = acc;
    if (out_tma) tc::bulk_wait_read();  // the tiles stay in place until the stores have read them
    if (by_tma) tc::mbar_inval(bar);    // a CTA that walks a work list sets the barrier up anew per item
  }
}

// grid (chunks, heads): one item per CTA; or, with a work list, a few persistent CTAs that walk it.
__global__ void __launch_bounds__(ib::kThreads, 1)
pkda_intra_bwd_kernel(const IntraBwdParams p, const __grid_constant__ IntraBwdMaps maps) {
  if (!p.slow_list) {
    intra_bwd_item(p, maps, blockIdx.x, blockIdx.y);
    return;
  }
  // items differ in cost (the number of pairing levels follows the decay): CTAs draw them one at a time
  __shared__ int s_item;
  const int n_items = p.fast_count[1], H = p.geo.heads;
  for (;;) {
    if (threadIdx.x == 0) s_item = atomicAdd(p.fast_count + 2, 1);
    __syncthreads();
    const int item = s_item;
    if (item >= n_items) break;
    const int chh = p.slow_list[item];
    intra_bwd_item(p, maps, chh / H, chh % H);
    __syncthreads();  // the next item reuses every shared-memory region (and s_item)
  }
}

// ------------------------------------------------------------------ preconditioner backward
struct AtkBwdParams {
  Geo geo;
  const bf16* k;
  const float* g_atk;
  const bf16* beta_atk;
  const float* log_atk_scale;
  const float* a_start;
  float* dkt;      // in: d(loss)/d(kt); after the local pass: dA_local
  float* dk_read;  // in: d(loss)/dk through the read path; after the local pass: + dkt B
  const float* lam_in;
  float* c_loc;
  bf16* dk;
  float* dg_atk;
  bf16* dbeta_atk;
  float* partC;
  float ln_x, eps;
  // local pass only: the (chunk * heads + head) items it works on and their number (NULL: every tile)
  const int* tile_list;
  const int* tile_count;
};

// One (chunk, head) per CTA, 256 threads, everything in registers.  Warp w owns
// rows 8w..8w+7 of the chunk, lane l owns channels 4l..4l+3, so a whole token row
// lives in one warp (128-bit loads of the fp32 gradients, 64-bit loads of k) and a
// thread holds its 8 x 4 elements for the whole kernel; all global loads are
// issued before the first use.  Both first-order scans over the 64 rows (A_t
// forward, lam = dL/dA backward) are blocked: a thread scans its 8 rows, the
// eight row blocks exchange one (decay product, end value) pair through shared
// memory, and each block continues from the carry it is owed -- every factor is a
// product of decays <= 1, so nothing overflows.  The per-row channel sums are
// transposed butterfly reductions (9 shuffles for 8 rows).
//   kFinal = false (local pass): everything that needs the write-key factor B(A_t) -- it turns the
//                   gradient buffers into dA_local (in the dkt buffer) and dk_read + dkt B, and leaves
//                   the chunk's outgoing carry and its share of the centre gradient.  Runs on the
//                   chunks the mma.sync chunk kernel handled; the tensor-memory kernel does the same
//                   for its chunks itself.
//   kFinal = true : incoming carry given; reverse scan of dA_local and all gradients.  No
//                   transcendental per element: the states A_t are rebuilt with multiply-adds.
namespace atkb {
constexpr int kThreads = 256;
constexpr int kRows = 8;  // rows per warp
}  // namespace atkb

// Thread-private prefetch slots in dynamic shared memory (a thread only reads back
// what it copied itself, so they need no barrier): per row k (8 B), dkt (16 B),
// dk_read (16 B); per tile the chunk's entry state and incoming carry (16 B each).
namespace atkb {
template <bool kFinal> __host__ __device__ constexpr int slot_bytes() {
  return kRows * (8 + 16 + 16) + 16 + (kFinal ? 16 : 0);
}
template <bool kFinal> __host__ __device__ constexpr int smem_bytes() { return kThreads * slot_bytes<kFinal>(); }
}  // namespace atkb

template <bool kFinal>
__global__ void __launch_bounds__(atkb::kThreads, 2)
pkda_atk_bwd_kernel(const AtkBwdParams p, int n_tiles) {
  using namespace atkb;
  extern __shared__ __align__(16) unsigned char slots[];
  __shared__ __align__(16) float sEnd[8][kD];  // per row block: end value of its zero-start scan
  __shared__ float sDec[8];                    // per row block: product of its decays
  __shared__ float sRed[8];
  const int H = p.geo.heads, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c4 = lane << 2, r0 = warp * kRows;
  const long gld = (long)H * kD;
  // slot layout: arrays of [kRows][kThreads] (then [kThreads]) so that a warp's accesses are contiguous
  uint2* sK = reinterpret_cast<uint2*>(slots);
  float4* sDkt = reinterpret_cast<float4*>(slots + kThreads * kRows * 8);
  float4* sDkr = sDkt + kThreads * kRows;
  float4* sA0 = sDkr + kThreads * kRows;
  float4* sLin = sA0 + kThreads;

  // A persistent CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; a tile is one (chunk, head).
  // The next tile's data is requested before the current tile is computed.
  int tok0_n = 0, valid_n = 0;
  bool live_n = false;
  // The next tile's beta_atk and log-decay (lane i of a warp holds the values of the warp's row i) and centre,
  // by plain loads that nothing consumes before the next iteration.
  uint32_t bpraw_n = 0;
  float centre_n = 0.f, lg_n = 0.f;  // lg_n: the same for the row's log-decay
  static_assert(kRows <= 32 && (kRows & (kRows - 1)) == 0, "one lane per row");
  if (!kFinal && p.tile_list) n_tiles = *p.tile_count;
  int tile_n = 0;  // the (chunk * heads + head) item behind the next position of the walk
  auto request = [&](int pos) {
    live_n = false;
    int tile = 0;
    if (pos < n_tiles) {
      tile = (!kFinal && p.tile_list) ? p.tile_list[pos] : pos;
      int n;
      live_n = chunk_lookup(p.geo, tile / H, n, tok0_n, valid_n);
    }
    tile_n = tile;
    if (live_n) {
      const int hh = tile % H;
      const size_t col0 = ((size_t)tok0_n * H + hh) * kD + c4;
#pragma unroll
      for (int i = 0; i < kRows; ++i) {
        const int r = r0 + i;
        const bool ok = r < valid_n;
        const size_t off = ok ? col0 + (size_t)r * gld : 0;
        // 8-byte copy as two 4-byte pieces (cp.async sizes are 4, 8 or 16)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_u32(sK + i * kThreads + tid)),
                     "l"(p.k + off), "r"(ok ? 8 : 0));
        cp_async16(sDkt + i * kThreads + tid, p.dkt + off, ok);
        cp_async16(sDkr + i * kThreads + tid, p.dk_read + off, ok);
      }
      {
        const int r = r0 + (lane & (kRows - 1));
        bpraw_n = 0;
        lg_n = 0.f;  // rows past the end: decay 1
        if (r < valid_n) {
          bpraw_n = *reinterpret_cast<const unsigned short*>(p.beta_atk + (size_t)(tok0_n + r) * H + hh);
          lg_n = p.g_atk[(size_t)(tok0_n + r) * H + hh];
        }
        centre_n = p.log_atk_scale[hh];
      }
      cp_async16(sA0 + tid, p.a_start + (size_t)tile * kD + c4, true);
      if (kFinal) cp_async16(sLin + tid, p.lam_in + (size_t)tile * kD + c4, true);
    }
    cp_async_commit();
  };
  request(blockIdx.x);
  for (int pos = blockIdx.x; pos < n_tiles; pos += gridDim.x) {
  const bool live = live_n;
  const int tile = tile_n;
  const int tok0 = tok0_n, valid = valid_n, h = tile % H;
  const size_t chh = (size_t)tile;
  const size_t col0 = ((size_t)tok0 * H + h) * kD + c4;
  cp_async_wait<0>();
  // ---- this tile's data: shared-memory slots -> registers
  uint2 kraw[kRows];
  float4 dkt[kFinal ? kRows : 1], dkr[kFinal ? kRows : 1];  // the local pass takes these from its slots row by row
  float pd[kRows], bp[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    kraw[i] = sK[i * kThreads + tid];
    if (kFinal) {
      dkt[i] = sDkt[i * kThreads + tid];
      dkr[i] = sDkr[i * kThreads + tid];
    }
    pd[i] = __shfl_sync(0xffffffffu, lg_n, i);  // the log-decay for now
    bp[i] = __uint_as_float(__shfl_sync(0xffffffffu, bpraw_n, i) << 16);
  }
  const float4 a0 = sA0[tid];
  float4 lin = make_float4(0.f, 0.f, 0.f, 0.f);
  if (kFinal) lin = sLin[tid];
  const float centre = centre_n;
  // final pass: the slots are free again, the next tile's copies fly during the computation; the local
  // pass still reads its gradient rows from the slots and asks for the next tile after that
  if (kFinal) request(pos + gridDim.x);
  if (!live) {               // (uniform) index past the last real chunk of a packed batch
    if (!kFinal) request(pos + gridDim.x);
    continue;
  }
  float dblk = 1.f;
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    pd[i] = __expf(pd[i]);  // rows past the end: exp(0) = 1, beta 0: the state passes through
    dblk *= pd[i];
  }
  // ---- forward scan, pass 1: the block's end value from a zero start
  {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const float2 x = unpack_bf16(kraw[i].x), y = unpack_bf16(kraw[i].y);
      const float kc[4] = {x.x, x.y, y.x, y.y};
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] = pd[i] * a[e] + bp[i] * kc[e] * kc[e];
    }
    *reinterpret_cast<float4*>(&sEnd[warp][c4]) = make_float4(a[0], a[1], a[2], a[3]);
    if (lane == 0) sDec[warp] = dblk;
  }
  __syncthreads();
  float A[4] = {a0.x, a0.y, a0.z, a0.w};  // state before this block's first row
  for (int b = 0; b < warp; ++b) {
    const float d = sDec[b];
    const float4 e4 = *reinterpret_cast<const float4*>(&sEnd[b][c4]);
    A[0] = d * A[0] + e4.x; A[1] = d * A[1] + e4.y; A[2] = d * A[2] + e4.z; A[3] = d * A[3] + e4.w;
  }
  const float Ain[4] = {A[0], A[1], A[2], A[3]};
  // ---- pass 2 (local pass only): true states; dA_local replaces dkt, dk_read takes the lam-free part
  // of dk; the block's share of the outgoing carry = sum_r (prod_{j<=r} decay_j) dA_local_r
  float dcacc = 0.f;
  if (!kFinal) {
    float w = 1.f, part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const bool ok = r0 + i < valid;
      const float2 x = unpack_bf16(kraw[i].x), y = unpack_bf16(kraw[i].y);
      const float kc[4] = {x.x, x.y, y.x, y.y};
      float4 dkt_i = sDkt[i * kThreads + tid], dkr_i = sDkr[i * kThreads + tid];
      float* dk_t = reinterpret_cast<float*>(&dkt_i);
      float* dk_r = reinterpret_cast<float*>(&dkr_i);
      w *= pd[i];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float An = pd[i] * A[e] + bp[i] * kc[e] * kc[e];
        const float dev = __logf(An + p.eps) - centre;
        const float den = 1.f + fabsf(dev);
        const float rden = __fdividef(1.f, den);
        const float Bf = __expf(-p.ln_x * dev * rden);
        const float ddev = -p.ln_x * dk_t[e] * kc[e] * Bf * rden * rden;
        dk_r[e] += dk_t[e] * Bf;
        dk_t[e] = ok ? __fdividef(ddev, An + p.eps) : 0.f;
        if (ok) dcacc -= ddev;
        part[e] += w * dk_t[e];
        A[e] = An;
      }
      if (ok) {  // the gradient buffers now hold what the final pass reads
        *reinterpret_cast<float4*>(p.dkt + col0 + (size_t)(r0 + i) * gld) = dkt_i;
        *reinterpret_cast<float4*>(p.dk_read + col0 + (size_t)(r0 + i) * gld) = dkr_i;
      }
    }
    request(pos + gridDim.x);  // the slots are free now
    __syncthreads();  // every warp has read the forward end values
    *reinterpret_cast<float4*>(&sEnd[warp][c4]) = make_float4(part[0], part[1], part[2], part[3]);
    __syncthreads();
    if (tid < kD) {
      float acc = 0.f, w2 = 1.f;
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        acc += w2 * sEnd[b][tid];
        w2 *= sDec[b];
      }
      p.c_loc[chh * kD + tid] = acc;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) dcacc += __shfl_xor_sync(0xffffffffu, dcacc, o);
    if (lane == 0) sRed[warp] = dcacc;
    __syncthreads();
    if (tid == 0) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) acc += sRed[w];
      p.partC[chh] = acc;
    }
    __syncthreads();  // the exchange arrays are reused by the next tile
    continue;
  }
  // ---- reverse scan: block-local lam from a zero incoming value (into dkt), outgoing value exchanged
  {
    float l[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = kRows - 1; i >= 0; --i) {
      float* d = reinterpret_cast<float*>(&dkt[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        l[e] += d[e];
        d[e] = l[e];
        l[e] *= pd[i];
      }
    }
    __syncthreads();  // every warp has read the forward end values
    *reinterpret_cast<float4*>(&sEnd[warp][c4]) = make_float4(l[0], l[1], l[2], l[3]);
  }
  __syncthreads();
  float L[4] = {lin.x, lin.y, lin.z, lin.w};  // lam arriving at the end of this block
  for (int b = 7; b > warp; --b) {
    const float d = sDec[b];
    const float4 e4 = *reinterpret_cast<const float4*>(&sEnd[b][c4]);
    L[0] = d * L[0] + e4.x; L[1] = d * L[1] + e4.y; L[2] = d * L[2] + e4.z; L[3] = d * L[3] + e4.w;
  }
  // suffix[i] = product of the decays of rows i+1 .. 7 of this block
  float suf[kRows];
  suf[kRows - 1] = 1.f;
#pragma unroll
  for (int i = kRows - 2; i >= 0; --i) suf[i] = suf[i + 1] * pd[i + 1];
  // ---- pass 3: outputs, walking the rows forward again for the state before each row
  float x1[kRows], x2[kRows];
  A[0] = Ain[0]; A[1] = Ain[1]; A[2] = Ain[2]; A[3] = Ain[3];
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const int r = r0 + i;
    const float2 x = unpack_bf16(kraw[i].x), y = unpack_bf16(kraw[i].y);
    const float kc[4] = {x.x, x.y, y.x, y.y};
    const float* ll = reinterpret_cast<const float*>(&dkt[i]);
    const float* t2 = reinterpret_cast<const float*>(&dkr[i]);
    float o[4];
    x1[i] = 0.f;
    x2[i] = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lam = ll[e] + suf[i] * L[e];
      o[e] = t2[e] + 2.f * lam * bp[i] * kc[e];
      const float k2 = kc[e] * kc[e];
      x1[i] += lam * k2;
      x2[i] += lam * A[e];
      A[e] = pd[i] * A[e] + bp[i] * k2;
    }
    x2[i] *= pd[i];
    if (r < valid)
      *reinterpret_cast<uint2*>(p.dk + col0 + (size_t)r * gld) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
  }
  row_sums8(x1, lane);
  row_sums8(x2, lane);
  if ((lane & 3) == 0) {
    const int r = r0 + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if (r < valid) {
      const size_t s = (size_t)(tok0 + r) * H + h;
      p.dbeta_atk[s] = __float2bfloat16(x1[0]);
      p.dg_atk[s] = x2[0];
    }
  }
  __syncthreads();  // the exchange arrays are reused by the next tile
  }  // tile loop
  cp_async_wait<0>();
}

// Sequential carry over a sequence's chunks, last to first.
__global__ void __launch_bounds__(kD)
pkda_atk_bwd_carry_kernel(Geo geo, const float* c_loc, const float* sa, float* lam_in, float* dA0) {
  const int n = blockIdx.x, h = blockIdx.y, H = geo.heads, c = threadIdx.x;
  const SeqInfo sq = seq_info(geo, n);
  float lam = 0.f;
  constexpr int kBatch = 16;  // loads of 16 chunks in flight before the dependent multiply-adds
  for (int i0 = sq.nchunks - 1; i0 >= 0; i0 -= kBatch) {
    float dec[kBatch], loc[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const bool ok = i0 - j >= 0;
      const size_t ch = (size_t)(sq.chunk0 + (ok ? i0 - j : 0)) * H + h;
      dec[j] = ok ? sa[ch] : 0.f;
      loc[j] = ok ? c_loc[ch * kD + c] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (i0 - j >= 0) {
        lam_in[((size_t)(sq.chunk0 + i0 - j) * H + h) * kD + c] = lam;
        lam = loc[j] + __expf(dec[j]) * lam;
      }
    }
  }
  if (dA0) dA0[((size_t)n * H + h) * kD + c] = lam;
}

// Deterministic reduction of the per-chunk partial sums of the three per-head
// parameter gradients.  grid (H), 1024 threads: eight sub-ranges of the chunk axis are
// summed side by side per channel and then added in order.
constexpr int kReduceSubs = 8;
__global__ void __launch_bounds__(kD * kReduceSubs)
pkda_param_reduce_kernel(Geo geo, const float* partA, const float* partB, const float* partC, float* dA_log,
                         float* ddt_bias, float* dcentre, const int* status, bf16* g0, bf16* g1, bf16* g2, size_t guard_n) {
  // The backward's last kernel: if any kernel of the call gave up, the heads of dq, dk and dv become
  // NaN, so that a caller who never reads the status word cannot take partial gradients for complete ones.
  if (blockIdx.x == 0 && *status != 0) {
    const bf16 nan = __float2bfloat16(__int_as_float(0x7fc00000));
    for (size_t i = threadIdx.x; i < guard_n; i += blockDim.x) {
      g0[i] = nan;
      g1[i] = nan;
      g2[i] = nan;
    }
  }
  __shared__ float sSub[kReduceSubs][kD];
  __shared__ float sR[2][4];
  const int h = blockIdx.x, H = geo.heads, tid = threadIdx.x, c = tid % kD, sub = tid / kD;
  const int warp = tid >> 5, lane = tid & 31;
  const int nreal = geo.cu_seqlens ? geo.chunk_offsets[geo.n_seqs] : geo.total_chunks;
  const int per = (nreal + kReduceSubs - 1) / kReduceSubs;
  const int lo = sub * per, hi = min(nreal, lo + per);
  float b = 0.f;
  for (int ch = lo; ch < hi; ++ch) b += partB[((size_t)ch * H + h) * kD + c];
  sSub[sub][c] = b;
  float a = 0.f, cc = 0.f;
  if (tid < kD) {
    for (int ch = c; ch < nreal; ch += kD) {
      a += partA[(size_t)ch * H + h];
      cc += partC[(size_t)ch * H + h];
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      cc += __shfl_xor_sync(0xffffffffu, cc, o);
    }
    if (lane == 0) { sR[0][warp] = a; sR[1][warp] = cc; }
  }
  __syncthreads();
  if (tid < kD) {
    float t = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < kReduceSubs; ++s2) t += sSub[s2][c];
    ddt_bias[h * kD + c] = t;
  }
  if (tid == 0) {
    dA_log[h] = sR[0][0] + sR[0][1] + sR[0][2] + sR[0][3];
    dcentre[h] = sR[1][0] + sR[1][1] + sR[1][2] + sR[1][3];
  }
}

// ------------------------------------------------------------------ host side
struct BwdWorkspace {
  int* chunk_offsets;
  float* beta_c;
  bf16 *u, *dF, *dh;
  float *dk_read, *dkt, *partA, *partB, *partC, *c_loc, *lam_in;
  int *fast_list, *slow_list, *counts;
  int *fwd_lists, *fwd_counts;  // work lists of the recompute pass (lean backward)
  int* status;
  size_t bytes;
};

static BwdWorkspace carve_bwd(const pkda_problem& p, void* base) {
  BwdWorkspace w;
  const size_t chunks = (size_t)chunk_bound(p), H = p.heads, tok = p.total_tokens;
  size_t off = 0;
  unsigned char* b = static_cast<unsigned char*>(base);
  auto take = [&](size_t bytes) {
    void* ptr = b + off;
    off += align_up(bytes);
    return ptr;
  };
  w.chunk_offsets = static_cast<int*>(take((size_t)(p.n_seqs + 1) * sizeof(int)));
  w.beta_c = static_cast<float*>(take(chunks * H * kChunk * 4));
  w.u = static_cast<bf16*>(take(tok * H * kD * 2));
  w.dF = static_cast<bf16*>(take(tok * H * kD * 2));
  w.dh = static_cast<bf16*>(take(chunks * H * kD * kD * 2));
  w.dk_read = static_cast<float*>(take(tok * H * kD * 4));
  w.dkt = static_cast<float*>(take(tok * H * kD * 4));
  w.partA = static_cast<float*>(take(chunks * H * 4));
  w.partB = static_cast<float*>(take(chunks * H * kD * 4));
  w.partC = static_cast<float*>(take(chunks * H * 4));
  w.c_loc = static_cast<float*>(take(chunks * H * kD * 4));
  w.lam_in = static_cast<float*>(take(chunks * H * kD * 4));
  w.fast_list = static_cast<int*>(take(chunks * H * sizeof(int)));
  w.slow_list = static_cast<int*>(take(chunks * H * sizeof(int)));
  w.fwd_lists = static_cast<int*>(take(chunks * H * sizeof(int)));
  w.status = static_cast<int*>(take(16 * sizeof(int)));  // status word, then lengths and cursors of the work lists
  w.counts = w.status + 1;       // [0] fast, [1] slow, [2] cursor
  w.fwd_counts = w.status + 5;   // [1] slow, [2] cursor
  w.bytes = off;
  return w;
}

size_t chunk_bwd_workspace(const pkda_problem& p) { return carve_bwd(p, nullptr).bytes; }
size_t chunk_bwd_status_offset(const pkda_problem& p) {
  return (size_t)(reinterpret_cast<unsigned char*>(carve_bwd(p, nullptr).status) - static_cast<unsigned char*>(nullptr));
}

#define PKDA_CHECK_LAUNCH()                                        \
  do {                                                             \
    end_stage(st);                                                 \
    if (cudaGetLastError() != cudaSuccess) return PKDA_ERR_LAUNCH; \
  } while (0)

template <typename K>
static bool set_smem(K kernel, int bytes) {
  return ensure_dynamic_smem(kernel, bytes);
}

template <int VB>
static int launch_scan_bwd(const ScanBwdParams& sp, int units, cudaStream_t st) {
  if (!set_smem(pkda_scan_bwd_kernel<VB>, scanb::L<VB>::kSmem)) return PKDA_ERR_LAUNCH;
  pkda_scan_bwd_kernel<VB><<<units * (kD / VB), scanb::threads<VB>(), scanb::L<VB>::kSmem, st>>>(sp);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

int chunk_bwd(const pkda_chunk_bwd_args* a, cudaStream_t st) {
  const pkda_problem& p = a->p;
  int rc = check_chunk_problem(p);
  if (rc != PKDA_OK) return rc;
  if (p.n_seqs == 0 || p.total_tokens == 0) return PKDA_OK;
  if (!a->d_o || !a->Aqk || !a->Akk || !a->k_precond || !a->ac_atk || !a->a_atk || !a->sa_atk || !a->w ||
      !a->kg || !a->v_new || !a->h || !a->qg || !a->dq || !a->dk || !a->dv || !a->dg || !a->dg_atk ||
      !a->dbeta_atk || !a->dbeta || !a->dA_log || !a->ddt_bias || !a->dlog_atk_scale)
    return PKDA_ERR_NULL;
  if (!a->workspace || a->workspace_bytes < chunk_bwd_workspace(p)) return PKDA_ERR_WORKSPACE;
  BwdWorkspace ws = carve_bwd(p, a->workspace);
  Geo geo;
  // On the default path the classifier of the intra stage runs first and packs beta on the way.
  const bool tc_intra = stage_variant(kStageIntraBwd) == 0;
  rc = run_prologue(p, ws.chunk_offsets, tc_intra ? nullptr : ws.beta_c, &geo, st);
  if (rc != PKDA_OK) return rc;

  const bf16* Aqk = static_cast<const bf16*>(a->Aqk);
  const bf16* Akk = static_cast<const bf16*>(a->Akk);
  const bf16* kt = static_cast<const bf16*>(a->k_precond);
  const float* gc = a->ac_atk;
  bf16* w = static_cast<bf16*>(a->w);
  bf16* kg = static_cast<bf16*>(a->kg);
  bf16* v_new = static_cast<bf16*>(a->v_new);
  bf16* h = static_cast<bf16*>(a->h);
  bf16* qg = static_cast<bf16*>(a->qg);
  if (cudaMemsetAsync(ws.status, 0, 16 * sizeof(int), st) != cudaSuccess) return PKDA_ERR_LAUNCH;
  if (tc_intra) {
    rc = launch_bwd_classify(geo, gc, direct_block_cap(), ws.fast_list, ws.slow_list, ws.counts,
                             static_cast<const bf16*>(p.beta), ws.beta_c, st);
    if (rc != PKDA_OK) return rc;
  }
  if (a->recompute) {
    // The recompute kernels only read the products, write keys and decay totals.
    rc = run_forward_stages(p, geo, ws.beta_c, ws.u, const_cast<bf16*>(Aqk), const_cast<bf16*>(Akk),
                            const_cast<bf16*>(kt), const_cast<float*>(gc), a->a_atk, w, kg, v_new, h, qg,
                            nullptr, true, ws.status, ws.fwd_lists, ws.fwd_counts, st);
    if (rc != PKDA_OK) return rc;
  }

  ScanBwdParams sp;
  sp.geo = geo; sp.kg = kg; sp.qg = qg; sp.w = w; sp.Aqk = Aqk; sp.d_o = static_cast<const bf16*>(a->d_o);
  sp.beta_c = ws.beta_c; sp.gc = gc; sp.dST = a->d_final_state; sp.dh = ws.dh; sp.dF = ws.dF;
  sp.dS0 = a->d_initial_state;
  {
    const int units = p.n_seqs * p.heads;
    const int vb = units >= 120 ? 128 : (units >= 60 ? 64 : 32);  // value columns per CTA of the mma.sync kernel
    // tcgen05 / TMEM / TMA at every size unless the mma.sync kernel is pinned (pkda_set_variant).
    const bool scan_mma = stage_variant(kStageScanBwd) == 1;
    begin_stage(kStageScanBwd, st);
    if (!scan_mma)
      rc = launch_scan_bwd_tc(geo, p.total_tokens, units, kg, w, qg, sp.d_o, Aqk, ws.beta_c, gc, a->d_final_state,
                              ws.dh, ws.dF, a->d_initial_state, ws.status, st);
    else if (vb == 128) rc = launch_scan_bwd<128>(sp, units, st);
    else if (vb == 64) rc = launch_scan_bwd<64>(sp, units, st);
    else rc = launch_scan_bwd<32>(sp, units, st);
    end_stage(st);
    if (rc != PKDA_OK) return rc;
  }

  dim3 gridc(geo.total_chunks, p.heads);
  IntraBwdParams ip;
  ip.geo = geo;
  ip.q = static_cast<const bf16*>(p.q); ip.k = static_cast<const bf16*>(p.k); ip.kt = kt;
  ip.g = static_cast<const bf16*>(p.g); ip.A_log = p.A_log; ip.dt_bias = p.dt_bias;
  ip.beta_c = ws.beta_c; ip.gc = gc; ip.Akk = Akk; ip.v_new = v_new; ip.h = h; ip.dh = ws.dh; ip.dF = ws.dF;
  ip.d_o = static_cast<const bf16*>(a->d_o);
  ip.dq = static_cast<bf16*>(a->dq); ip.dk_read = ws.dk_read; ip.dv = static_cast<bf16*>(a->dv);
  ip.dg = static_cast<bf16*>(a->dg); ip.dbeta = static_cast<bf16*>(a->dbeta); ip.dkt = ws.dkt;
  ip.partA = ws.partA; ip.partB = ws.partB; ip.scale = p.scale; ip.direct_cap = direct_block_cap();
  ip.g_atk = p.g_atk; ip.beta_atk = static_cast<const bf16*>(p.beta_atk); ip.log_atk_scale = p.log_atk_scale;
  ip.a_start = a->a_atk; ip.c_loc = ws.c_loc; ip.partC = ws.partC;
  ip.ln_x = logf(p.squash_x); ip.eps = p.squash_eps;
  IntraBwdMaps maps;
  {
    const uint64_t H = p.heads, tok = p.total_tokens, rows = (uint64_t)geo.total_chunks * H * kD;
    const uint64_t act_dims[2] = {H * kD, tok}, act_str[1] = {H * kD * 2};
    const uint32_t act_box[2] = {kLdD, kChunk};
    const uint64_t st_dims[2] = {kD, rows}, st_str[1] = {kD * 2};
    const uint32_t st_box[2] = {kLdD, kD};
    const uint64_t pr_dims[2] = {H * kChunk, tok}, pr_str[1] = {H * kChunk * 2};
    const uint32_t pr_box[2] = {kLdC, kChunk};
    ip.use_tma = tok >= kChunk && encode_bf16_map(&maps.d_o, ip.d_o, 2, act_dims, act_str, act_box, false) &&
                 encode_bf16_map(&maps.dF, ip.dF, 2, act_dims, act_str, act_box, false) &&
                 encode_bf16_map(&maps.E, ip.v_new, 2, act_dims, act_str, act_box, false) &&
                 encode_bf16_map(&maps.h, ip.h, 2, st_dims, st_str, st_box, false) &&
                 encode_bf16_map(&maps.dh, ip.dh, 2, st_dims, st_str, st_box, false) &&
                 encode_bf16_map(&maps.Akk, ip.Akk, 2, pr_dims, pr_str, pr_box, false);
    const uint64_t o_dims[3] = {kD, H, tok}, o_str2[2] = {kD * 2, H * kD * 2}, o_str4[2] = {kD * 4, H * kD * 4};
    const uint32_t o_box[3] = {kLdD, 1, kChunk};
    ip.out_tma = ip.use_tma && encode_bf16_map(&maps.dq, ip.dq, 3, o_dims, o_str2, o_box, false) &&
                 encode_bf16_map(&maps.dv, ip.dv, 3, o_dims, o_str2, o_box, false) &&
                 encode_f32_map(&maps.dk_read, ip.dk_read, 3, o_dims, o_str4, o_box) &&
                 encode_f32_map(&maps.dkt, ip.dkt, 3, o_dims, o_str4, o_box);
    ip.status = ws.status;
  }
  // Full chunks that are one direct block run on tcgen05 / tensor memory; a classifier in front sorts
  // the chunks into two work lists and the mma.sync kernel works off the second one (every chunk, one
  // CTA each, when it is pinned).
  ip.fast_list = ip.slow_list = ip.fast_count = nullptr;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (tc_intra) {
    ip.fast_list = ws.fast_list; ip.slow_list = ws.slow_list; ip.fast_count = ws.counts;
    rc = launch_intra_bwd_tc(ip, st);
    if (rc != PKDA_OK) return rc;
    const int items = geo.total_chunks * p.heads;
    gridc = dim3(items < sms ? items : sms, 1);
  }
  if (!set_smem(pkda_intra_bwd_kernel, ib::kSmem)) return PKDA_ERR_LAUNCH;
  begin_stage(ip.slow_list ? kStageIntraBwdRest : kStageIntraBwd, st);
  pkda_intra_bwd_kernel<<<gridc, ib::kThreads, ib::kSmem, st>>>(ip, maps);
  PKDA_CHECK_LAUNCH();

  AtkBwdParams ap;
  ap.geo = geo; ap.k = static_cast<const bf16*>(p.k); ap.g_atk = p.g_atk;
  ap.beta_atk = static_cast<const bf16*>(p.beta_atk); ap.log_atk_scale = p.log_atk_scale;
  ap.a_start = a->a_atk; ap.dkt = ws.dkt; ap.dk_read = ws.dk_read; ap.lam_in = ws.lam_in; ap.c_loc = ws.c_loc;
  ap.dk = static_cast<bf16*>(a->dk); ap.dg_atk = a->dg_atk; ap.dbeta_atk = static_cast<bf16*>(a->dbeta_atk);
  ap.partC = ws.partC; ap.ln_x = logf(p.squash_x); ap.eps = p.squash_eps;
  // the tensor-memory chunk kernel has done the local pass of its own chunks
  ap.tile_list = ip.slow_list; ap.tile_count = ip.slow_list ? ws.counts + 1 : nullptr;
  begin_stage(kStageAtkBwdLocal, st);
  const int atk_tiles = geo.total_chunks * p.heads;
  const int atk_grid = atk_tiles < 2 * sms ? atk_tiles : 2 * sms;  // persistent: two CTAs per SM
  if (!set_smem(pkda_atk_bwd_kernel<false>, atkb::smem_bytes<false>())) return PKDA_ERR_LAUNCH;
  pkda_atk_bwd_kernel<false><<<atk_grid, atkb::kThreads, atkb::smem_bytes<false>(), st>>>(ap, atk_tiles);
  PKDA_CHECK_LAUNCH();
  begin_stage(kStageAtkBwdCarry, st);
  pkda_atk_bwd_carry_kernel<<<dim3(p.n_seqs, p.heads), kD, 0, st>>>(geo, ws.c_loc, a->sa_atk, ws.lam_in,
                                                                   a->d_initial_A_state);
  PKDA_CHECK_LAUNCH();
  begin_stage(kStageAtkBwdFinal, st);
  if (!set_smem(pkda_atk_bwd_kernel<true>, atkb::smem_bytes<true>())) return PKDA_ERR_LAUNCH;
  pkda_atk_bwd_kernel<true><<<atk_grid, atkb::kThreads, atkb::smem_bytes<true>(), st>>>(ap, atk_tiles);
  PKDA_CHECK_LAUNCH();
  begin_stage(kStageParamReduce, st);
  const size_t guard_n = std::min<size_t>((size_t)p.total_tokens * p.heads * kD, 4096);
  pkda_param_reduce_kernel<<<p.heads, kD * kReduceSubs, 0, st>>>(
      geo, ws.partA, ws.partB, ws.partC, a->dA_log, a->ddt_bias, a->dlog_atk_scale, ws.status,
      static_cast<bf16*>(a->dq), static_cast<bf16*>(a->dk), static_cast<bf16*>(a->dv), guard_n);
  PKDA_CHECK_LAUNCH();
  return PKDA_OK;
}

}  // namespace pkda

