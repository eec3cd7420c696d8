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
//
// With kOut the kernel also produces the chunk's output, which needs exactly the
// two tiles the scan has on chip anyway (the chunk-entry state h and E):
//   O^T = h^T qg^T + E^T (P diag beta)^T   tcgen05.mma  M=128 (v) N=64 (tok), K=128 then K=64
// Four more warps own this: one of their threads fetches qg and P (two buffers,
// one chunk ahead) and issues the twelve products when the scan warps signal that
// h, then E, stand in shared memory; three warps scale P by beta meanwhile; all
// four read the 64-column accumulator back and store o.  The scan warps wait for
// them only before they overwrite a tile the output products read (one warp polls
// the products' barrier; they were issued most of a chunk step earlier).  Same
// operands, same instruction shapes and same accumulation order as the
// stand-alone output kernel: the same bits.  Measured at 128 sequences x heads,
// T = 4096: scan alone 0.158 ms + output kernel 0.122 ms, fused 0.192 ms.
#include "pkda_chunk.cuh"
#include "pkda_tc.cuh"

namespace pkda {

struct ScanTcParams {
  Geo geo;
  const float *beta_c, *gc, *S0;
  bf16* v_new;
  float* ST;
  bf16* o;  // kOut only
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
constexpr int oE = oI + 8192;               // 2 blocks [64 tok][64 v]   E as v_new stores it (A of the output's second product)
constexpr int oBar = oE + 16384;            // full[kStages], mma1, mma2, tmem slot, the output warps' barriers
constexpr int oQP = oBar + 1024;            // kOut: two buffers of qg (2 blocks [64 tok][64 k]) + P ([64 tok][64 j])
constexpr int kQP = 16384 + 8192;
constexpr int kSmem = oBar + 128 + 1024;    // (the barriers sit in the first 128 bytes of their 1 KB slot)
constexpr int kSmemOut = oQP + 2 * kQP + 1024;
constexpr int kOutThreads = 128;
constexpr uint32_t kCols = 256;             // S: columns 0..127, E^T accumulator: 128..191, O^T accumulator: 192..255
}  // namespace scantc

// Barrier of the 256 scan threads (named barrier 1), with an OR reduction of a predicate; the output
// warps of the fused kernel synchronise among themselves on barrier 2.
__device__ __forceinline__ void scan_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ bool scan_sync_or(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r) : "r"((uint32_t)pred) : "memory");
  return r != 0;
}
__device__ __forceinline__ bool out_sync_or(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 2, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r) : "r"((uint32_t)pred) : "memory");
  return r != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <bool kRecompute, bool kOut>
__global__ void __launch_bounds__(scantc::kThreads + (kOut ? scantc::kOutThreads : 0), 1)
pkda_scan_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_kg,
                        const __grid_constant__ CUtensorMap tm_u, const __grid_constant__ CUtensorMap tm_h,
                        const __grid_constant__ CUtensorMap tm_e, const __grid_constant__ CUtensorMap tm_qg,
                        const __grid_constant__ CUtensorMap tm_p, const ScanTcParams p) {
  using namespace scantc;
  extern __shared__ unsigned char smem_raw[];
  const int n = blockIdx.x / p.geo.heads, h = blockIdx.x - n * p.geo.heads, H = p.geo.heads;
  const SeqInfo sq = seq_info(p.geo, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = warp & 3, hf = (warp >> 2) & 1;
  const int L = 32 * q + lane;  // this thread's TMEM lane: state row k, or value channel v of E^T and O^T
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_full0 = base + oBar, bar_qp0 = base + oBar + 16, bar_mma1 = base + oBar + 32,
                 bar_mma2 = base + oBar + 40, tmem_slot = base + oBar + 48, bar_hready = base + oBar + 56,
                 bar_eready = base + oBar + 64, bar_o1 = base + oBar + 72, bar_o = base + oBar + 80;

  const size_t sbase = ((size_t)n * H + h) * kD * kD;

  if (warp == 0) tc::tmem_alloc(tmem_slot, kCols);
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) tc::mbar_init(bar_full0 + 8 * s, 1);
    tc::mbar_init(bar_mma1, 1);
    tc::mbar_init(bar_mma2, 1);
    if (kOut) {
      tc::mbar_init(bar_qp0, 1);
      tc::mbar_init(bar_qp0 + 8, 1);
      tc::mbar_init(bar_hready, 1);
      tc::mbar_init(bar_eready, 1);
      tc::mbar_init(bar_o1, 1);
      tc::mbar_init(bar_o, 1);
    }
    tc::fence_barrier_init();
  }
  // identity tile: piece jc of row n holds columns 8 jc .. 8 jc + 7
  for (int idx = tid; idx < kChunk * 8; idx += (int)blockDim.x) {
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
  bool ok = true;

  if (kOut && warp >= kThreads / 32) {
    // ================= the output warps: O^T of every chunk, one chunk behind nothing but the tiles it needs
    const int e = tid - kThreads;          // 0..127
    const bool issuer = e == 32;  // (not in the scheduler that thread 0, which issues the scan's products, lives in)
    const uint32_t tO = tmem + ((uint32_t)(32 * q) << 16) + 192;
    auto fetch = [&](int i) {  // issuer only: qg and P of chunk i into buffer i & 1
      const uint32_t dst = base + oQP + (i & 1) * kQP, bar = bar_qp0 + 8 * (i & 1);
      const int tok0 = sq.bos + i * kChunk;
      tc::mbar_expect_tx(bar, kQP);
      tc::tma_load_3d(dst, &tm_qg, bar, 0, h, tok0);
      tc::tma_load_3d(dst + 8192, &tm_qg, bar, 64, h, tok0);
      tc::tma_load_3d(dst + 16384, &tm_p, bar, 0, h, tok0);
    };
    if (issuer && sq.nchunks > 0) fetch(0);
    constexpr uint32_t idesc_o = tc::idesc_bf16(128, 64, /*a_mn_major=*/true, /*b_mn_major=*/false);
    // Per chunk: the issuing thread queues the first product as soon as h stands while three warps scale
    // P; it queues the second product when E stands; all four warps read the accumulator and stage o.
    // The issuing thread's own warp does nothing else while it waits (a lane that spins holds up the
    // other lanes of its warp), and nobody but that thread polls the scan's signals.
    const bool issuer_warp = (e >> 5) == 1;
    const int sc = e < 32 ? e : e - 32;  // 0..95 among the threads that scale P
    float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;  // beta of this thread's eight columns of P, one chunk ahead
    if (sq.nchunks > 0 && !issuer_warp) {
      const size_t chh = (size_t)sq.chunk0 * H + h;
      b0 = *reinterpret_cast<const float4*>(p.beta_c + chh * kChunk + 8 * (sc & 7));
      b1 = *reinterpret_cast<const float4*>(p.beta_c + chh * kChunk + 8 * (sc & 7) + 4);
    }
    for (int i = 0; i < sq.nchunks; ++i) {
      const uint32_t qp = base + oQP + (i & 1) * kQP;
      unsigned char* qpp = tiles + oQP + (i & 1) * kQP;
      const int tok0 = sq.bos + i * kChunk;
      const int valid = min(kChunk, sq.len - i * kChunk);
      // qg and P of this chunk were requested a chunk step ago: one poll each
      ok = tc::mbar_wait(bar_qp0 + 8 * (i & 1), (i >> 1) & 1) && ok;
      if (issuer_warp) {
        if (issuer) {
          // the other buffer was last read by the products of chunk i - 1, which this thread saw complete
          if (i + 1 < sq.nchunks) fetch(i + 1);
          ok = tc::mbar_wait(bar_hready, i & 1) && ok;  // h of this chunk stands in its tile
          if (ok) {
            tc::tc_fence_after();  // (the accumulator is free: all four warps read it before the barrier after the read)
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              tc::umma_bf16(tmem + 192, tc::desc_mnmajor(base + oH + kk * 2048, 16384),
                            tc::desc_kmajor(qp + (kk >> 2) * 8192 + (kk & 3) * 32), idesc_o, kk > 0);
            tc::umma_commit(bar_o1);
          }
        }
        __syncwarp();
      } else {
        if (ok) {  // P[tok][j] *= beta[j] in place: 16-byte piece jc of row r sits at r*128 + ((jc ^ (r & 7)) << 4)
          const float f[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
          for (int idx = sc; idx < kChunk * 8; idx += 96) {
            const int r = idx >> 3, jc = idx & 7;
            uint4* piece = reinterpret_cast<uint4*>(qpp + 16384 + r * 128 + ((jc ^ (r & 7)) << 4));
            uint4 x = *piece;
            scale8(x, f);
            *piece = x;
          }
        }
        if (i + 1 < sq.nchunks) {
          const size_t chn = (size_t)(sq.chunk0 + i + 1) * H + h;
          b0 = *reinterpret_cast<const float4*>(p.beta_c + chn * kChunk + 8 * (sc & 7));
          b1 = *reinterpret_cast<const float4*>(p.beta_c + chn * kChunk + 8 * (sc & 7) + 4);
        }
        tc::fence_proxy_async();
      }
      if (out_sync_or(!ok)) { ok = false; break; }
      if (issuer) {
        ok = tc::mbar_wait(bar_eready, i & 1) && ok;  // E of this chunk stands in its tile
        if (ok) {
          tc::tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc::umma_bf16(tmem + 192, tc::desc_mnmajor(base + oE + kk * 2048, 8192),
                          tc::desc_kmajor(qp + 16384 + kk * 32), idesc_o, 1);
          tc::umma_commit(bar_o);
          ok = tc::mbar_wait(bar_o, i & 1) && ok;
        }
      }
      if (out_sync_or(!ok)) { ok = false; break; }
      tc::tc_fence_after();
      float acc0[32], acc1[32];
      tc::tmem_ld32(tO, acc0);
      tc::tmem_ld32(tO + 32, acc1);
      tc::tmem_ld_wait();
      tc::tc_fence_before();
      out_sync_or(false);  // all four warps hold their part: the next chunk's first product may overwrite the accumulator
      bf16* dst = p.o + ((size_t)tok0 * H + h) * kD + L;
      const size_t gld = (size_t)H * kD;
      if (valid == kChunk) {
        // (2-byte stores, 64 contiguous bytes per warp and token.  Staging the tile in shared memory for a
        // TMA store, and trading values between lanes for 8-byte stores, were both measured: no faster,
        // these warps run in the issue slots the scan warps leave them.)
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          *dst = __float2bfloat16(acc0[t]);
          dst += gld;
        }
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          *dst = __float2bfloat16(acc1[t]);
          dst += gld;
        }
      } else {
#pragma unroll
        for (int t = 0; t < 32; ++t)
          if (t < valid) dst[t * gld] = __float2bfloat16(acc0[t]);
#pragma unroll
        for (int t = 0; t < 32; ++t)
          if (32 + t < valid) dst[(32 + t) * gld] = __float2bfloat16(acc1[t]);
      }
    }
    if (!ok && issuer) atomicExch(p.status, 1);
  } else {
  // ================= the scan warps
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

  // A TMA instruction costs the thread that issues it about a hundred cycles, and every scan thread is
  // on the critical chain (the barriers wait for the slowest), so the ten copies of a chunk step are
  // spread over the first lanes of the warps: warp w issues piece w of the next chunk's tiles; warps
  // 1, 2 store the halves of the state tile and warps 3, 4 those of E.  Thread 0 arms the barrier (the
  // bytes may land before it does: the phase cannot complete without its arrival) and issues the products.
  auto prefetch_piece = [&](int i, int piece) {
    const uint32_t st = base + (i % kStages) * kStage, bar = bar_full0 + 8 * (i % kStages);
    const int tok0 = sq.bos + i * kChunk;
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    switch (piece) {
      case 0: tc::mbar_expect_tx(bar, kTx); tc::tma_load_3d(st + oW, &tm_w, bar, 0, h, tok0); break;
      case 1: tc::tma_load_3d(st + oW + 8192, &tm_w, bar, 64, h, tok0); break;
      case 2: tc::tma_load_3d(st + oKg, &tm_kg, bar, 0, h, tok0); break;
      case 3: tc::tma_load_3d(st + oKg + 8192, &tm_kg, bar, 64, h, tok0); break;
      case 4: tc::tma_load_3d(st + oU, &tm_u, bar, 0, h, tok0); break;
      case 5: tc::tma_load_3d(st + oU + 8192, &tm_u, bar, 64, h, tok0); break;
      case 6: tc::bulk_load(st + oBeta, p.beta_c + chh * kChunk, 256, bar); break;
      default: tc::bulk_load(st + oGc, p.gc + chh * kD, 512, bar); break;
    }
  };
  if (lane == 0) {
    for (int i = 0; i < kStages - 1 && i < sq.nchunks; ++i) prefetch_piece(i, warp);
  }

  constexpr uint32_t idesc1 = tc::idesc_bf16(128, 64, true, false);
  constexpr uint32_t idesc1n = idesc1 | (1u << 13);  // A negated
  constexpr uint32_t idesc2 = tc::idesc_bf16(128, 128, true, false);
  for (int i = 0; i < sq.nchunks; ++i) {
    const int stg = i % kStages;
    const uint32_t st = base + stg * kStage;
    unsigned char* stp = tiles + stg * kStage;
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    if (lane == 0) {
      if (warp >= 1 && warp <= 4) tc::bulk_wait_read();  // this thread's store of the previous chunk has read its tile
      if (i + kStages - 1 < sq.nchunks) prefetch_piece(i + kStages - 1, warp);  // into the stage chunk i-1 used
    }
    // (one warp polls each barrier; the others sleep in the named barrier that follows: a polling warp
    // takes issue slots and shared-memory bandwidth from whoever shares its scheduler)
    if (warp == 0) ok = tc::mbar_wait(bar_full0 + 8 * stg, (i / kStages) & 1) && ok;
    // The h tile is rewritten below: the output's first product of the previous chunk, queued most of a
    // chunk step ago, must have read it.
    if (kOut && warp == 0 && i > 0) ok = tc::mbar_wait(bar_o1, (i - 1) & 1) && ok;
    if (scan_sync_or(!ok)) { ok = false; break; }
    tc::tc_fence_after();

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
    scan_sync();
    if (lane == 0 && (warp == 1 || warp == 2)) {  // the state tile out, one half each
      tc::tma_store_2d(&tm_h, base + oH + (warp - 1) * 16384, 64 * (warp - 1), (int)(chh * kD));
      tc::bulk_commit();
    }
    if (tid == 0) {
      tc::tc_fence_after();
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
      if (kOut) mbar_arrive(bar_hready);  // (after this chunk's own product is queued: it goes first)
    }
    if (warp == 0) ok = tc::mbar_wait(bar_mma1, i & 1) && ok;
    tc::tc_fence_before();
    // likewise the E tile, which step b rewrites, and the output's second product of the previous chunk
    if (kOut && warp == 0 && i > 0) ok = tc::mbar_wait(bar_o, (i - 1) & 1) && ok;
    if (scan_sync_or(!ok)) { ok = false; break; }
    tc::tc_fence_after();

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
      // E as the accumulator holds it ([v][tok]) is parked in this stage's W tile, which the first
      // product has finished reading, and transposed from there
      unsigned char* sEt = stp + oW;
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {  // row L of the [v][tok] tiles: tokens 32 hf + 8 pc .. + 7
        const uint32_t off = L * 128 + (((4 * hf + pc) ^ (L & 7)) << 4);
        *reinterpret_cast<uint4*>(tiles + oF + off) = make_uint4(fpk[4 * pc], fpk[4 * pc + 1], fpk[4 * pc + 2], fpk[4 * pc + 3]);
        *reinterpret_cast<uint4*>(sEt + off) = make_uint4(epk[4 * pc], epk[4 * pc + 1], epk[4 * pc + 2], epk[4 * pc + 3]);
      }
      // Transpose this warp's 32 v x 32 tok block of E into the [tok][v] tile: four 8x8
      // matrices (the four 8-channel groups of one 8-token group) per ldmatrix.trans.
      __syncwarp();
      const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
      for (int tb = 0; tb < 4; ++tb) {
        const int vrow = 32 * q + lane;  // lanes 0-7 / 8-15 / 16-23 / 24-31 address the rows of matrices 0..3
        uint32_t r[4];
        ldsm_x4_t(r, st + oW + vrow * 128 + (((4 * hf + tb) ^ (vrow & 7)) << 4));
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
    scan_sync();
    if (lane == 0 && (warp == 3 || warp == 4) && valid == kChunk) {
      tc::tma_store_3d(&tm_e, base + oE + (warp - 3) * 8192, 64 * (warp - 3), h, tok0);
      tc::bulk_commit();
    }
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t a = tc::desc_mnmajor(st + oKg + kk * 2048, 8192);
        const uint64_t b = tc::desc_kmajor(base + oF + kk * 32);
        tc::umma_bf16(tmem, a, b, idesc2, 1);
      }
      tc::umma_commit(bar_mma2);
      if (kOut) mbar_arrive(bar_eready);
    }
    if (warp == 0) ok = tc::mbar_wait(bar_mma2, i & 1) && ok;
    tc::tc_fence_before();  // (the barrier at the top of the next step, or the one after the loop, follows)
  }
  if (scan_sync_or(!ok)) {
    if (tid == 0) atomicExch(p.status, 1);
  } else if (!kRecompute && p.ST) {
    tc::tc_fence_after();
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
  if (lane == 0 && warp >= 1 && warp <= 4) tc::bulk_wait_all();  // our stores must have left shared memory before the CTA exits
  }  // scan warps
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, kCols);
  // This is the forward's last kernel when it forms the output.  If any kernel of the call gave up
  // (this CTA included), the first output row of this (sequence, head) becomes NaN, so that a caller
  // who never reads the status word cannot take a partial result for a complete one.
  if (kOut && warp == 1 && sq.len > 0 && *reinterpret_cast<volatile int*>(p.status) != 0) {
    const bf16 nan = __float2bfloat16(__int_as_float(0x7fc00000));
    bf16* row = p.o + ((size_t)sq.bos * H + h) * kD;
    for (int c = lane; c < kD; c += 32) row[c] = nan;
  }
}

int launch_scan_fwd_tc(const Geo& geo, int total_tokens, int units, const bf16* w, const bf16* kg, const bf16* u,
                       const float* beta_c, const float* gc, const float* S0, bf16* h, bf16* v_new, float* ST,
                       int* status, bool recompute, const bf16* qg, const bf16* Aqk, bf16* o, cudaStream_t st) {
  const uint64_t H = geo.heads, chunks = geo.total_chunks, tok = total_tokens;
  const bool with_out = o != nullptr && !recompute;
  CUtensorMap tm_w, tm_kg, tm_u, tm_h, tm_e, tm_qg, tm_p;
  {
    const uint64_t dims[3] = {kD, H, tok}, str[2] = {kD * 2, H * kD * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_w, w, 3, dims, str, box) || !encode_bf16_map(&tm_kg, kg, 3, dims, str, box) ||
        !encode_bf16_map(&tm_u, u, 3, dims, str, box) || !encode_bf16_map(&tm_e, v_new, 3, dims, str, box) ||
        !encode_bf16_map(&tm_qg, with_out ? qg : w, 3, dims, str, box))
      return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[2] = {kD, chunks * H * kD}, str[1] = {kD * 2};
    const uint32_t box[2] = {64, 128};
    if (!encode_bf16_map(&tm_h, h, 2, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  if (with_out) {
    const uint64_t dims[3] = {kChunk, H, tok}, str[2] = {kChunk * 2, H * kChunk * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_p, Aqk, 3, dims, str, box)) return PKDA_ERR_LAUNCH;
  } else {
    tm_p = tm_qg;  // unused
  }
  ScanTcParams sp;
  sp.geo = geo; sp.beta_c = beta_c; sp.gc = gc; sp.S0 = S0; sp.v_new = v_new; sp.ST = ST; sp.o = o; sp.status = status;
  if (recompute) {
    if (!ensure_dynamic_smem(pkda_scan_fwd_tc_kernel<true, false>, scantc::kSmem))
      return PKDA_ERR_LAUNCH;
    pkda_scan_fwd_tc_kernel<true, false><<<units, scantc::kThreads, scantc::kSmem, st>>>(tm_w, tm_kg, tm_u, tm_h, tm_e,
                                                                                        tm_qg, tm_p, sp);
  } else if (with_out) {
    if (!ensure_dynamic_smem(pkda_scan_fwd_tc_kernel<false, true>, scantc::kSmemOut))
      return PKDA_ERR_LAUNCH;
    pkda_scan_fwd_tc_kernel<false, true><<<units, scantc::kThreads + scantc::kOutThreads, scantc::kSmemOut, st>>>(
        tm_w, tm_kg, tm_u, tm_h, tm_e, tm_qg, tm_p, sp);
  } else {
    if (!ensure_dynamic_smem(pkda_scan_fwd_tc_kernel<false, false>, scantc::kSmem))
      return PKDA_ERR_LAUNCH;
    pkda_scan_fwd_tc_kernel<false, false><<<units, scantc::kThreads, scantc::kSmem, st>>>(tm_w, tm_kg, tm_u, tm_h, tm_e,
                                                                                         tm_qg, tm_p, sp);
  }
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda

