// Reverse state scan of the backward on tcgen05 / TMEM / TMA (one CTA per
// (sequence, head), all 128 value columns).  The running state cotangent dS
// [128 k][128 v] fp32 lives in tensor memory for the whole sequence; per
// 64-token chunk, last chunk first,
//   d    = bf16(dS)                       TMEM -> registers -> swizzled smem (+ TMA store: the saved dh)
//   dS  *= Gam_last (row scale)           registers -> TMEM
//   dF^T = d^T kg^T + dO^T P              tcgen05.mma  M=128 (v) N=64 (tok), K=128 (k) then K=64 (tok'), in TMEM
//   dS  += qg^T dO                        tcgen05.mma  M=128 (k) N=128 (v) K=64 (tok); runs while the
//                                         threads work on dF
//   dE   = -beta * bf16(dF)               TMEM -> registers -> swizzled smem (K-major: one 64-byte run per
//                                         thread); dF is transposed warp-locally (ldmatrix.trans) into a
//                                         [tok][v] tile and leaves by TMA store
//   dS  += W^T dE                         tcgen05.mma  M=128 (k) N=128 (v) K=64 (tok)
// kg, W, qg, dO and P tiles (and beta, Gam_last) arrive by TMA / bulk copies one
// chunk ahead (two stages).  Every mbarrier wait is bounded: on a timeout the CTA
// sets the status word, stops working on its sequence, frees its TMEM and exits.
// Rows of a ragged last chunk past its end hold the next sequence's tokens (or
// the zero fill past the end of the tensor): dO is zeroed there, beta is zero
// there, and nothing else of those rows reaches a kept result.
#include "pkda_chunk.cuh"
#include "pkda_tc.cuh"

namespace pkda {

struct ScanBwdTcParams {
  Geo geo;
  const float *beta_c, *gc, *dST;
  bf16* dF;
  float* dS0;
  int* status;
};

namespace scanbtc {
constexpr int kThreads = 256;
constexpr int oKg = 0;                      // 2 blocks [64 tok][64 k]   (B of d^T kg^T, K-major)
constexpr int oW = oKg + 16384;             // 2 blocks [64 tok][64 k]   (A of W^T dE, MN-major)
constexpr int oQg = oW + 16384;             // 2 blocks [64 tok][64 k]   (A of qg^T dO, MN-major)
constexpr int oDo = oQg + 16384;            // 2 blocks [64 tok][64 v]   (A of dO^T P and B of qg^T dO, MN-major)
constexpr int oP = oDo + 16384;             // [64 tok'][64 tok]         (B of dO^T P, MN-major)
constexpr int oBeta = oP + 8192;            // f32 [64]
constexpr int oGc = oBeta + 256;            // f32 [128]
constexpr int kTx = oGc + 512;              // bytes that land per stage
constexpr int kStage = 74752;               // stage pitch (1024-aligned)
constexpr int kStages = 2;
constexpr int oD = kStages * kStage;        // 2 blocks [128 k][64 v]    (A of d^T kg^T, MN-major)
constexpr int oDE = oD + 32768;             // [128 v][64 tok]           dF as the accumulator holds it, then dE
constexpr int oF = oDE + 16384;             // 2 blocks [64 tok][64 v]   dF as the output stores it
constexpr int oBar = oF + 16384;            // full[kStages], mma1, mma2, tmem slot
constexpr int kSmem = oBar + 64 + 1024;
constexpr uint32_t kCols = 256;             // dS: columns 0..127, dF^T accumulator: 128..191
static_assert(kTx <= kStage && kStage % 1024 == 0 && oD % 1024 == 0 && oDE % 1024 == 0 && oF % 1024 == 0,
              "operand tiles must be 1024-byte aligned");
static_assert(kSmem <= 232448, "shared memory of one SM");
}  // namespace scanbtc

__global__ void __launch_bounds__(scanbtc::kThreads, 1)
pkda_scan_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_kg, const __grid_constant__ CUtensorMap tm_w,
                        const __grid_constant__ CUtensorMap tm_qg, const __grid_constant__ CUtensorMap tm_do,
                        const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_dh,
                        const __grid_constant__ CUtensorMap tm_df, const ScanBwdTcParams p) {
  using namespace scanbtc;
  extern __shared__ unsigned char smem_raw[];
  const int n = blockIdx.x / p.geo.heads, h = blockIdx.x - n * p.geo.heads, H = p.geo.heads;
  const SeqInfo sq = seq_info(p.geo, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = warp & 3, hf = warp >> 2;
  const int L = 32 * q + lane;  // this thread's TMEM lane: state row k, or value channel v of dF^T
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
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tiles + oBar + 48);
  const uint32_t tS = tmem + ((uint32_t)(32 * q) << 16);       // this warp's lanes, dS columns
  const uint32_t tF = tS + 128;                                 // dF^T accumulator columns

  // ---- cotangent of the final state -> TMEM
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float v[32];
#pragma unroll
    for (int e = 0; e < 32; e += 4) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p.dST) x = *reinterpret_cast<const float4*>(p.dST + sbase + (size_t)L * kD + 64 * hf + 32 * j + e);
      v[e] = x.x; v[e + 1] = x.y; v[e + 2] = x.z; v[e + 3] = x.w;
    }
    tc::tmem_st32(tS + 64 * hf + 32 * j, v);
  }
  tc::tmem_st_wait();

  const int last = sq.nchunks - 1;
  // A TMA instruction costs its thread about a hundred cycles and every thread is on the critical chain
  // (the barriers wait for the slowest), so the copies of a chunk step are spread over the first lanes of
  // the warps: eleven pieces of the next chunk's tiles (warps 5..7 take two), the halves of the d tile
  // stored by warps 1, 2 and those of dF by warps 3, 4.  The bytes may land before thread 0 has armed the
  // barrier: the phase cannot complete without its arrival.
  auto prefetch_piece = [&](int j, int piece) {  // j counts processed chunks, chunk index = last - j
    const int i = last - j;
    const uint32_t st = base + (j % kStages) * kStage, bar = bar_full0 + 8 * (j % kStages);
    const int tok0 = sq.bos + i * kChunk;
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    switch (piece) {
      case 0: tc::mbar_expect_tx(bar, kTx); tc::tma_load_3d(st + oKg, &tm_kg, bar, 0, h, tok0); break;
      case 1: tc::tma_load_3d(st + oKg + 8192, &tm_kg, bar, 64, h, tok0); break;
      case 2: tc::tma_load_3d(st + oDo, &tm_do, bar, 0, h, tok0); break;
      case 3: tc::tma_load_3d(st + oDo + 8192, &tm_do, bar, 64, h, tok0); break;
      case 4: tc::tma_load_3d(st + oP, &tm_p, bar, 0, h, tok0); break;
      case 5: tc::tma_load_3d(st + oQg, &tm_qg, bar, 0, h, tok0);
              tc::bulk_load(st + oBeta, p.beta_c + chh * kChunk, 256, bar); break;
      case 6: tc::tma_load_3d(st + oQg + 8192, &tm_qg, bar, 64, h, tok0);
              tc::bulk_load(st + oGc, p.gc + chh * kD, 512, bar); break;
      default: tc::tma_load_3d(st + oW, &tm_w, bar, 0, h, tok0);
               tc::tma_load_3d(st + oW + 8192, &tm_w, bar, 64, h, tok0); break;
    }
  };
  if (lane == 0) {
    for (int j = 0; j < kStages - 1 && j < sq.nchunks; ++j) prefetch_piece(j, warp);
  }

  constexpr uint32_t idesc_dkg = tc::idesc_bf16(128, 64, true, false);    // d^T (MN) x kg (K)
  constexpr uint32_t idesc_dop = tc::idesc_bf16(128, 64, true, true);     // dO^T (MN) x P (MN)
  constexpr uint32_t idesc_qdo = tc::idesc_bf16(128, 128, true, true);    // qg^T (MN) x dO (MN)
  constexpr uint32_t idesc_wde = tc::idesc_bf16(128, 128, true, false);   // W^T (MN) x dE (K)
  bool ok = true;
  for (int j = 0; j < sq.nchunks; ++j) {
    const int i = last - j;
    const int stg = j % kStages;
    const uint32_t st = base + stg * kStage;
    unsigned char* stp = tiles + stg * kStage;
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    if (lane == 0) {
      if (warp >= 1 && warp <= 4) tc::bulk_wait_read();  // this thread's store of the previous chunk has read its tile
      if (j + kStages - 1 < sq.nchunks) prefetch_piece(j + kStages - 1, warp);  // into the stage the chunk before used
    }
    // (one warp polls each barrier, the others sleep in the barrier that follows: a polling warp takes
    // issue slots and shared-memory bandwidth from whoever shares its scheduler)
    if (warp == 0) ok = tc::mbar_wait(bar_full0 + 8 * stg, (j / kStages) & 1) && ok;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc::tc_fence_after();
    if (valid < kChunk) {  // ragged last chunk: no output cotangent past its end
      for (int idx = tid; idx < (kChunk - valid) * 16; idx += kThreads) {
        const int r = valid + (idx >> 4), pc = idx & 15;
        *reinterpret_cast<uint4*>(stp + oDo + (pc >> 3) * 8192 + r * 128 + ((pc & 7) << 4)) = make_uint4(0, 0, 0, 0);
      }
    }

    // a. d = bf16(dS) -> operand tile; dS *= Gam_last
    {
      const float gcv = reinterpret_cast<const float*>(stp + oGc)[L];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        float v[32];
        tc::tmem_ld32(tS + 64 * hf + 32 * jj, v);
        tc::tmem_ld_wait();
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint4 pk;
          pk.x = pack_bf16(v[8 * pc], v[8 * pc + 1]);
          pk.y = pack_bf16(v[8 * pc + 2], v[8 * pc + 3]);
          pk.z = pack_bf16(v[8 * pc + 4], v[8 * pc + 5]);
          pk.w = pack_bf16(v[8 * pc + 6], v[8 * pc + 7]);
          *reinterpret_cast<uint4*>(tiles + oD + sw128_offset(L, 64 * hf + 32 * jj + 8 * pc, 16384)) = pk;
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] *= gcv;
        tc::tmem_st32(tS + 64 * hf + 32 * jj, v);
      }
      tc::tmem_st_wait();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    if (lane == 0 && (warp == 1 || warp == 2)) {  // the d tile out, one half each
      tc::tma_store_2d(&tm_dh, base + oD + (warp - 1) * 16384, 64 * (warp - 1), (int)(chh * kD));
      tc::bulk_commit();
    }
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {  // d^T kg^T
        const uint64_t a = tc::desc_mnmajor(base + oD + kk * 2048, 16384);
        const uint64_t b = tc::desc_kmajor(st + oKg + (kk >> 2) * 8192 + (kk & 3) * 32);
        tc::umma_bf16(tmem + 128, a, b, idesc_dkg, kk > 0);
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // + dO^T P
        const uint64_t a = tc::desc_mnmajor(st + oDo + kk * 2048, 8192);
        const uint64_t b = tc::desc_mnmajor(st + oP + kk * 2048, 8192);
        tc::umma_bf16(tmem + 128, a, b, idesc_dop, 1);
      }
      tc::umma_commit(bar_mma1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // dS += qg^T dO, behind the threads' work on dF
        const uint64_t a = tc::desc_mnmajor(st + oQg + kk * 2048, 8192);
        const uint64_t b = tc::desc_mnmajor(st + oDo + kk * 2048, 8192);
        tc::umma_bf16(tmem, a, b, idesc_qdo, 1);
      }
    }
    if (warp == 0) ok = tc::mbar_wait(bar_mma1, j & 1) && ok;
    tc::tc_fence_before();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc::tc_fence_after();

    // b. dF^T sits in the accumulator (lane = value channel, column = token);  dE = -beta dF
    {
      float acc[32];
      tc::tmem_ld32(tF + 32 * hf, acc);
      tc::tmem_ld_wait();
      const float* sBeta = reinterpret_cast<const float*>(stp + oBeta) + 32 * hf;
      uint32_t fpk[16], epk[16];
#pragma unroll
      for (int t = 0; t < 32; t += 2) {
        const bf16 f0 = __float2bfloat16(acc[t]), f1 = __float2bfloat16(acc[t + 1]);
        fpk[t >> 1] = pack_bf16(to_f(f0), to_f(f1));
        epk[t >> 1] = pack_bf16(-sBeta[t] * to_f(f0), -sBeta[t + 1] * to_f(f1));
      }
      // row L of the [v][tok] tile: tokens 32 hf + 8 pc .. + 7.  dF goes in first and is transposed
      // warp-locally into the [tok][v] tile (four 8x8 matrices, the four 8-channel groups of one
      // 8-token group, per ldmatrix.trans); then dE takes its place as the operand of the last product.
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        const uint32_t off = L * 128 + (((4 * hf + pc) ^ (L & 7)) << 4);
        *reinterpret_cast<uint4*>(tiles + oDE + off) = make_uint4(fpk[4 * pc], fpk[4 * pc + 1], fpk[4 * pc + 2], fpk[4 * pc + 3]);
      }
      __syncwarp();
      const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
      for (int tb = 0; tb < 4; ++tb) {
        const int vrow = 32 * q + lane;  // lanes 0-7 / 8-15 / 16-23 / 24-31 address the rows of matrices 0..3
        uint32_t r[4];
        ldsm_x4_t(r, base + oDE + vrow * 128 + (((4 * hf + tb) ^ (vrow & 7)) << 4));
        const int tok = 32 * hf + 8 * tb + gq;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const int v = 32 * q + 8 * m + 2 * tq;
          *reinterpret_cast<uint32_t*>(tiles + oF + sw128_offset(tok, v, 8192)) = r[m];
          if (valid < kChunk && tok < valid)  // ragged last chunk: plain stores of the valid rows only
            *reinterpret_cast<uint32_t*>(p.dF + ((size_t)(tok0 + tok) * H + h) * kD + v) = r[m];
        }
      }
      __syncwarp();
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        const uint32_t off = L * 128 + (((4 * hf + pc) ^ (L & 7)) << 4);
        *reinterpret_cast<uint4*>(tiles + oDE + off) = make_uint4(epk[4 * pc], epk[4 * pc + 1], epk[4 * pc + 2], epk[4 * pc + 3]);
      }
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    if (lane == 0 && (warp == 3 || warp == 4) && valid == kChunk) {
      tc::tma_store_3d(&tm_df, base + oF + (warp - 3) * 8192, 64 * (warp - 3), h, tok0);
      tc::bulk_commit();
    }
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // dS += W^T dE
        const uint64_t a = tc::desc_mnmajor(st + oW + kk * 2048, 8192);
        const uint64_t b = tc::desc_kmajor(base + oDE + kk * 32);
        tc::umma_bf16(tmem, a, b, idesc_wde, 1);
      }
      tc::umma_commit(bar_mma2);
    }
    if (warp == 0) ok = tc::mbar_wait(bar_mma2, j & 1) && ok;
    tc::tc_fence_before();  // (the barrier at the top of the next step, or the one after the loop, follows)
  }
  if (__syncthreads_or(!ok)) {
    if (tid == 0) atomicExch(p.status, 1);
  } else if (p.dS0) {
    tc::tc_fence_after();
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      float v[32];
      tc::tmem_ld32(tS + 64 * hf + 32 * jj, v);
      tc::tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; e += 4)
        *reinterpret_cast<float4*>(p.dS0 + sbase + (size_t)L * kD + 64 * hf + 32 * jj + e) =
            make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
    }
  }
  if (lane == 0 && warp >= 1 && warp <= 4) tc::bulk_wait_all();  // our stores must have left shared memory before the CTA exits
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, kCols);
}

int launch_scan_bwd_tc(const Geo& geo, int total_tokens, int units, const bf16* kg, const bf16* w, const bf16* qg,
                       const bf16* d_o, const bf16* Aqk, const float* beta_c, const float* gc, const float* dST,
                       bf16* dh, bf16* dF, float* dS0, int* status, cudaStream_t st) {
  const uint64_t H = geo.heads, chunks = geo.total_chunks, tok = total_tokens;
  CUtensorMap tm_kg, tm_w, tm_qg, tm_do, tm_p, tm_dh, tm_df;
  {
    const uint64_t dims[3] = {kD, H, tok}, str[2] = {kD * 2, H * kD * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_kg, kg, 3, dims, str, box) || !encode_bf16_map(&tm_w, w, 3, dims, str, box) ||
        !encode_bf16_map(&tm_qg, qg, 3, dims, str, box) || !encode_bf16_map(&tm_do, d_o, 3, dims, str, box) ||
        !encode_bf16_map(&tm_df, dF, 3, dims, str, box))
      return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {kChunk, H, tok}, str[2] = {kChunk * 2, H * kChunk * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_p, Aqk, 3, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {kD, chunks * H * kD}, str[1] = {kD * 2};
    const uint32_t box[2] = {64, 128};
    if (!encode_bf16_map(&tm_dh, dh, 2, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  ScanBwdTcParams sp;
  sp.geo = geo; sp.beta_c = beta_c; sp.gc = gc; sp.dST = dST; sp.dF = dF; sp.dS0 = dS0; sp.status = status;
  if (!ensure_dynamic_smem(pkda_scan_bwd_tc_kernel, scanbtc::kSmem))
    return PKDA_ERR_LAUNCH;
  pkda_scan_bwd_tc_kernel<<<units, scanbtc::kThreads, scanbtc::kSmem, st>>>(tm_kg, tm_w, tm_qg, tm_do, tm_p, tm_dh,
                                                                             tm_df, sp);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
