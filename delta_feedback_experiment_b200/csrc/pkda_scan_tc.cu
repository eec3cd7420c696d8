// Forward state scan on tcgen05 / TMEM / TMA (one CTA per (sequence, head), all
// 128 value columns).  The running state S [128 k][128 v] fp32 lives in tensor
// memory for the whole sequence; per 64-token chunk
//   h   = bf16(S)                         TMEM -> registers -> swizzled smem (+ TMA store of the chunk state)
//   S  *= Gam_last (row scale)            registers -> TMEM
//   E^T = U^T I - h^T W^T                 tcgen05.mma  M=128 (v) N=64 (tok) K=128 (k) with A negated, plus
//                                         K=64 against a constant identity tile (adds U^T exactly), in TMEM
//   F   = beta * bf16(E)                  TMEM -> registers -> swizzled smem (K-major: one 64-byte run per thread);
//                                         E is transposed warp-locally (ldmatrix.trans) into a [tok][v]
//                                         tile and leaves by TMA store
//   S  += kg^T F                          tcgen05.mma  M=128 (k) N=128 (v) K=64 (tok), accumulating into S
// W, kg and U tiles (and beta, Gam_last) arrive by TMA / bulk copies one chunk
// ahead (two stages).  Every mbarrier wait is bounded: on a timeout the CTA sets
// the status word, stops working on its sequence, frees its TMEM and exits.
#include "pkda_chunk.cuh"
#include "pkda_tc.cuh"

namespace pkda {

struct ScanTcParams {
  Geo geo;
  const float *beta_c, *gc, *S0;
  bf16* v_new;
  float* ST;
  int* status;
};

namespace scantc {
constexpr int kThreads = 256;
constexpr int oW = 0;                       // 2 blocks [64 tok][64 k]   (B of product 1, K-major)
constexpr int oKg = oW + 16384;             // 2 blocks [64 tok][64 k]   (A of product 2, MN-major)
constexpr int oU = oKg + 16384;             // 2 blocks [64 tok][64 v]
constexpr int oBeta = oU + 16384;           // f32 [64]
constexpr int oGc = oBeta + 256;            // f32 [128]
constexpr int kTx = oGc + 512;              // bytes that land per stage
constexpr int kStage = 50176;               // stage pitch (1024-aligned)
constexpr int kStages = 2;                  // W / kg / U tiles in flight
constexpr int oH = kStages * kStage;              // 2 blocks [128 k][64 v]    (A of product 1, MN-major)
constexpr int oF = oH + 32768;              // [128 v][64 tok]           (B of product 2, K-major)
constexpr int oI = oF + 16384;              // [64 tok][64 tok] identity (B of the U^T pass, K-major)
constexpr int oEt = oI + 8192;              // [128 v][64 tok]           E as the accumulator holds it
constexpr int oE = oEt + 16384;             // 2 blocks [64 tok][64 v]   E as v_new stores it
constexpr int oBar = oE + 16384;            // full[kStages], mma1, mma2, tmem slot
constexpr int kSmem = oBar + 64 + 1024;
constexpr uint32_t kCols = 256;             // S: columns 0..127, E^T accumulator: 128..191
}  // namespace scantc

template <bool kRecompute>
__global__ void __launch_bounds__(scantc::kThreads, 1)
pkda_scan_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_kg,
                        const __grid_constant__ CUtensorMap tm_u, const __grid_constant__ CUtensorMap tm_h,
                        const __grid_constant__ CUtensorMap tm_e, const ScanTcParams p) {
  using namespace scantc;
  extern __shared__ unsigned char smem_raw[];
  const int n = blockIdx.x / p.geo.heads, h = blockIdx.x - n * p.geo.heads, H = p.geo.heads;
  const SeqInfo sq = seq_info(p.geo, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = warp & 3, hf = warp >> 2;
  const int L = 32 * q + lane;  // this thread's TMEM lane: state row k, or value channel v of E^T
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_full0 = base + oBar, bar_mma1 = base + oBar + 32, bar_mma2 = base + oBar + 40;
  const uint32_t tmem_slot = base + oBar + 48;
  const size_t sbase = ((size_t)n * H + h) * kD * kD;

  if (warp == 0) tc::tmem_alloc(tmem_slot, kCols);
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) tc::mbar_init(bar_full0 + 8 * s, 1);
    tc::mbar_init(bar_mma1, 1);
    tc::mbar_init(bar_mma2, 1);
    tc::fence_barrier_init();
  }
  // identity tile: piece jc of row n holds columns 8 jc .. 8 jc + 7
  for (int idx = tid; idx < kChunk * 8; idx += kThreads) {
    const int r = idx >> 3, jc = idx & 7;
    uint4 pk = make_uint4(0, 0, 0, 0);
    if ((r >> 3) == jc) {
      const uint32_t one = (r & 1) ? 0x3F800000u : 0x00003F80u;  // bf16 1.0 in the high or low half
      reinterpret_cast<uint32_t*>(&pk)[(r & 7) >> 1] = one;
    }
    *reinterpret_cast<uint4*>(tiles + oI + r * 128 + ((jc ^ (r & 7)) << 4)) = pk;
  }
  tc::fence_proxy_async();
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tiles + oBar + 48);
  const uint32_t tS = tmem + ((uint32_t)(32 * q) << 16);       // this warp's lanes, S columns
  const uint32_t tE = tS + 128;                                 // E^T accumulator columns

  // ---- initial state -> TMEM
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float v[32];
#pragma unroll
    for (int e = 0; e < 32; e += 4) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p.S0) x = *reinterpret_cast<const float4*>(p.S0 + sbase + (size_t)L * kD + 64 * hf + 32 * j + e);
      v[e] = x.x; v[e + 1] = x.y; v[e + 2] = x.z; v[e + 3] = x.w;
    }
    tc::tmem_st32(tS + 64 * hf + 32 * j, v);
  }
  tc::tmem_st_wait();

  auto prefetch = [&](int i) {  // thread 0 only
    const uint32_t st = base + (i % kStages) * kStage, bar = bar_full0 + 8 * (i % kStages);
    const int tok0 = sq.bos + i * kChunk;
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    tc::mbar_expect_tx(bar, kTx);
    tc::tma_load_3d(st + oW, &tm_w, bar, 0, h, tok0);
    tc::tma_load_3d(st + oW + 8192, &tm_w, bar, 64, h, tok0);
    tc::tma_load_3d(st + oKg, &tm_kg, bar, 0, h, tok0);
    tc::tma_load_3d(st + oKg + 8192, &tm_kg, bar, 64, h, tok0);
    tc::tma_load_3d(st + oU, &tm_u, bar, 0, h, tok0);
    tc::tma_load_3d(st + oU + 8192, &tm_u, bar, 64, h, tok0);
    tc::bulk_load(st + oBeta, p.beta_c + chh * kChunk, 256, bar);
    tc::bulk_load(st + oGc, p.gc + chh * kD, 512, bar);
  };
  if (tid == 0) {
    for (int i = 0; i < kStages - 1 && i < sq.nchunks; ++i) prefetch(i);
  }

  constexpr uint32_t idesc1 = tc::idesc_bf16(128, 64, true, false);
  constexpr uint32_t idesc1n = idesc1 | (1u << 13);  // A negated
  constexpr uint32_t idesc2 = tc::idesc_bf16(128, 128, true, false);
  bool ok = true;
  for (int i = 0; i < sq.nchunks; ++i) {
    const int stg = i % kStages;
    const uint32_t st = base + stg * kStage;
    unsigned char* stp = tiles + stg * kStage;
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    PKDA_SCANTC_PHASE(i, 0);
    if (tid == 0) {
      tc::bulk_wait_read();  // the previous chunk's stores have finished reading sH / sE
      if (i + kStages - 1 < sq.nchunks) prefetch(i + kStages - 1);  // into the stage chunk i-1 used
    }
    ok = tc::mbar_wait(bar_full0 + 8 * stg, (i / kStages) & 1) && ok;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    PKDA_SCANTC_PHASE(i, 1);

    // a. h = bf16(S) -> operand tile; S *= Gam_last
    {
      const float gcv = reinterpret_cast<const float*>(stp + oGc)[L];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float v[32];
        tc::tmem_ld32(tS + 64 * hf + 32 * j, v);
        tc::tmem_ld_wait();
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint4 pk;
          pk.x = pack_bf16(v[8 * pc], v[8 * pc + 1]);
          pk.y = pack_bf16(v[8 * pc + 2], v[8 * pc + 3]);
          pk.z = pack_bf16(v[8 * pc + 4], v[8 * pc + 5]);
          pk.w = pack_bf16(v[8 * pc + 6], v[8 * pc + 7]);
          *reinterpret_cast<uint4*>(tiles + oH + sw128_offset(L, 64 * hf + 32 * j + 8 * pc, 16384)) = pk;
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] *= gcv;
        tc::tmem_st32(tS + 64 * hf + 32 * j, v);
      }
      tc::tmem_st_wait();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    PKDA_SCANTC_PHASE(i, 2);
    if (tid == 0) {
      tc::tc_fence_after();
      const int hrow = (int)(chh * kD);
      tc::tma_store_2d(&tm_h, base + oH, 0, hrow);
      tc::tma_store_2d(&tm_h, base + oH + 16384, 64, hrow);
      tc::bulk_commit();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t a = tc::desc_mnmajor(base + oH + kk * 2048, 16384);
        const uint64_t b = tc::desc_kmajor(st + oW + (kk >> 2) * 8192 + (kk & 3) * 32);
        tc::umma_bf16(tmem + 128, a, b, idesc1n, kk > 0);
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // + U^T I
        const uint64_t a = tc::desc_mnmajor(st + oU + kk * 2048, 8192);
        const uint64_t b = tc::desc_kmajor(base + oI + kk * 32);
        tc::umma_bf16(tmem + 128, a, b, idesc1, 1);
      }
      tc::umma_commit(bar_mma1);
    }
    ok = tc::mbar_wait(bar_mma1, i & 1) && ok;
    tc::tc_fence_after();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    PKDA_SCANTC_PHASE(i, 3);

    // b. E^T sits in the accumulator (lane = value channel, column = token);  F = beta E
    {
      float acc[32];
      tc::tmem_ld32(tE + 32 * hf, acc);
      tc::tmem_ld_wait();
      const float* sBeta = reinterpret_cast<const float*>(stp + oBeta) + 32 * hf;
      uint32_t fpk[16], epk[16];
#pragma unroll
      for (int t = 0; t < 32; t += 2) {
        const bf16 e0 = __float2bfloat16(acc[t]), e1 = __float2bfloat16(acc[t + 1]);
        epk[t >> 1] = pack_bf16(to_f(e0), to_f(e1));
        fpk[t >> 1] = pack_bf16(sBeta[t] * to_f(e0), sBeta[t + 1] * to_f(e1));
      }
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {  // row L of the [v][tok] tiles: tokens 32 hf + 8 pc .. + 7
        const uint32_t off = L * 128 + (((4 * hf + pc) ^ (L & 7)) << 4);
        *reinterpret_cast<uint4*>(tiles + oF + off) = make_uint4(fpk[4 * pc], fpk[4 * pc + 1], fpk[4 * pc + 2], fpk[4 * pc + 3]);
        *reinterpret_cast<uint4*>(tiles + oEt + off) = make_uint4(epk[4 * pc], epk[4 * pc + 1], epk[4 * pc + 2], epk[4 * pc + 3]);
      }
      // Transpose this warp's 32 v x 32 tok block of E into the [tok][v] tile: four 8x8
      // matrices (the four 8-channel groups of one 8-token group) per ldmatrix.trans.
      __syncwarp();
      const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
      for (int tb = 0; tb < 4; ++tb) {
        const int vrow = 32 * q + lane;  // lanes 0-7 / 8-15 / 16-23 / 24-31 address the rows of matrices 0..3
        uint32_t r[4];
        ldsm_x4_t(r, base + oEt + vrow * 128 + (((4 * hf + tb) ^ (vrow & 7)) << 4));
        const int tok = 32 * hf + 8 * tb + gq;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const int v = 32 * q + 8 * m + 2 * tq;
          *reinterpret_cast<uint32_t*>(tiles + oE + sw128_offset(tok, v, 8192)) = r[m];
          if (valid < kChunk && tok < valid)  // ragged last chunk: plain stores of the valid rows only
            *reinterpret_cast<uint32_t*>(p.v_new + ((size_t)(tok0 + tok) * H + h) * kD + v) = r[m];
        }
      }
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    PKDA_SCANTC_PHASE(i, 4);
    if (tid == 0) {
      tc::tc_fence_after();
      if (valid == kChunk) {
        tc::tma_store_3d(&tm_e, base + oE, 0, h, tok0);
        tc::tma_store_3d(&tm_e, base + oE + 8192, 64, h, tok0);
        tc::bulk_commit();
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t a = tc::desc_mnmajor(st + oKg + kk * 2048, 8192);
        const uint64_t b = tc::desc_kmajor(base + oF + kk * 32);
        tc::umma_bf16(tmem, a, b, idesc2, 1);
      }
      tc::umma_commit(bar_mma2);
    }
    ok = tc::mbar_wait(bar_mma2, i & 1) && ok;
    tc::tc_fence_after();
    PKDA_SCANTC_PHASE(i, 5);
  }
  if (__syncthreads_or(!ok)) {
    if (tid == 0) atomicExch(p.status, 1);
  } else if (!kRecompute && p.ST) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float v[32];
      tc::tmem_ld32(tS + 64 * hf + 32 * j, v);
      tc::tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; e += 4)
        *reinterpret_cast<float4*>(p.ST + sbase + (size_t)L * kD + 64 * hf + 32 * j + e) =
            make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
    }
  }
  if (tid == 0) tc::bulk_wait_all();  // our stores must have left shared memory before the CTA exits
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, kCols);
}

int launch_scan_fwd_tc(const Geo& geo, int total_tokens, int units, const bf16* w, const bf16* kg, const bf16* u,
                       const float* beta_c, const float* gc, const float* S0, bf16* h, bf16* v_new, float* ST,
                       int* status, bool recompute, cudaStream_t st) {
  const uint64_t H = geo.heads, chunks = geo.total_chunks, tok = total_tokens;
  CUtensorMap tm_w, tm_kg, tm_u, tm_h, tm_e;
  {
    const uint64_t dims[3] = {kD, H, tok}, str[2] = {kD * 2, H * kD * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_w, w, 3, dims, str, box) || !encode_bf16_map(&tm_kg, kg, 3, dims, str, box) ||
        !encode_bf16_map(&tm_u, u, 3, dims, str, box) || !encode_bf16_map(&tm_e, v_new, 3, dims, str, box))
      return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {kD, chunks * H * kD}, str[1] = {kD * 2};
    const uint32_t box[2] = {64, 128};
    if (!encode_bf16_map(&tm_h, h, 2, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  ScanTcParams sp;
  sp.geo = geo; sp.beta_c = beta_c; sp.gc = gc; sp.S0 = S0; sp.v_new = v_new; sp.ST = ST; sp.status = status;
  if (recompute) {
    if (cudaFuncSetAttribute(pkda_scan_fwd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             scantc::kSmem) != cudaSuccess)
      return PKDA_ERR_LAUNCH;
    pkda_scan_fwd_tc_kernel<true><<<units, scantc::kThreads, scantc::kSmem, st>>>(tm_w, tm_kg, tm_u, tm_h, tm_e, sp);
  } else {
    if (cudaFuncSetAttribute(pkda_scan_fwd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             scantc::kSmem) != cudaSuccess)
      return PKDA_ERR_LAUNCH;
    pkda_scan_fwd_tc_kernel<false><<<units, scantc::kThreads, scantc::kSmem, st>>>(tm_w, tm_kg, tm_u, tm_h, tm_e, sp);
  }
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda

#ifdef PKDA_PHASE_PROFILE
extern "C" int pkda_phase_prof_scantc(long long* out) {
  return cudaMemcpyFromSymbol(out, g_phase_prof, sizeof(long long) * 64) == cudaSuccess ? 0 : 1;
}
#endif
