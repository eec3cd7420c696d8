// Chunked PKDA forward for D = 128, chunk 64, bf16 activations.
//
// Pipeline (one launch each, all on the caller's stream):
//   offsets   packed input only: cumulative chunk counts per sequence
//   pack_beta beta -> fp32 [chunks][H][64], zero for rows past a sequence end
//   atk_local chunk-local preconditioner accumulation (from A = 0) and decay sums
//   atk_carry sequential over a sequence's chunks: A at every chunk start
//   intra     per chunk: log-decay cumsum, write keys, gated pair products
//             M (k x kt) and P (q x kt) by a binary hierarchy of reference rows,
//             Tm = (I + tril(M) diag(beta))^-1, W = Tm (k*Gam), U = Tm v,
//             kg = kt * exp(G_last - G), qg = scale q * Gam
//   scan      sequential over chunks, V split across CTAs: h_n, E = U - W h_n,
//             S <- Gam_last * S + kg^T (beta E)
//   out       per chunk: o = qg h_n + P (beta E)
// With per-channel decay exp(G_i - G_j) cannot be factored as exp(G_i)exp(-G_j)
// (overflow after a few tokens); level L of the hierarchy pairs rows whose index
// has bit L set with rows of the same 2L-block whose bit L is clear, both
// expressed relative to the first row of the upper half, so every factor is <= 1.
#include <algorithm>

#include "pkda_chunk.cuh"

namespace pkda {

// ------------------------------------------------------------------ small kernels
__global__ void pkda_chunk_offsets_kernel(const int* cu, int n_seqs, int* offs) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int acc = 0;
    offs[0] = 0;
    for (int n = 0; n < n_seqs; ++n) {
      acc += (cu[n + 1] - cu[n] + kChunk - 1) / kChunk;
      offs[n + 1] = acc;
    }
  }
}

__global__ void pkda_pack_beta_kernel(Geo geo, const bf16* beta, float* beta_c) {
  int n, tok0, valid;
  if (!chunk_lookup(geo, blockIdx.x, n, tok0, valid)) return;
  const int H = geo.heads;
  for (int i = threadIdx.x; i < H * kChunk; i += blockDim.x) {
    int h = i / kChunk, r = i - h * kChunk;
    float b = r < valid ? to_f(beta[(size_t)(tok0 + r) * H + h]) : 0.f;
    beta_c[((size_t)blockIdx.x * H + h) * kChunk + r] = b;
  }
}

// Chunk-local preconditioner scan from A = 0: loc[c] = sum_j (prod_{m>j} d_m) bP_j k_j[c]^2
// and the chunk's summed log-decay; also the chunk-major fp32 copy of beta (when beta_c is
// given), which saves a launch.  grid (chunks, H), 256 threads: warp w scans rows 8w..8w+7 with
// lane l holding channels 4l..4l+3 (64-bit loads, one token row per warp request), then the
// eight row blocks are chained in order through shared memory.
__global__ void __launch_bounds__(256)
pkda_atk_local_kernel(Geo geo, const bf16* k, const float* g_atk, const bf16* beta_atk, const bf16* beta,
                      float* ac_local, float* sa, float* beta_c) {
  __shared__ __align__(16) float sEnd[8][kD];
  __shared__ float sDec[8], sSum[8];
  int n, tok0, valid;
  if (!chunk_lookup(geo, blockIdx.x, n, tok0, valid)) return;
  const int h = blockIdx.y, H = geo.heads, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t chh = (size_t)blockIdx.x * H + h;
  const int c4 = lane << 2, r0 = warp * 8;
  uint2 kraw[8];
  float lg[8], bp[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {  // all loads first
    const int r = r0 + i;
    const bool ok = r < valid;
    const size_t s = (size_t)(tok0 + (ok ? r : 0)) * H + h;
    kraw[i] = ok ? *reinterpret_cast<const uint2*>(k + s * kD + c4) : make_uint2(0, 0);
    lg[i] = ok ? g_atk[s] : 0.f;
    bp[i] = ok ? to_f(beta_atk[s]) : 0.f;
  }
  if (beta_c && tid < kChunk)
    beta_c[chh * kChunk + tid] = tid < valid ? to_f(beta[(size_t)(tok0 + tid) * H + h]) : 0.f;
  float a[4] = {0.f, 0.f, 0.f, 0.f}, dblk = 1.f, gsum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 x = unpack_bf16(kraw[i].x), y = unpack_bf16(kraw[i].y);
    const float pd = __expf(lg[i]);  // rows past the end: decay 1, beta 0
    a[0] = pd * a[0] + bp[i] * x.x * x.x;
    a[1] = pd * a[1] + bp[i] * x.y * x.y;
    a[2] = pd * a[2] + bp[i] * y.x * y.x;
    a[3] = pd * a[3] + bp[i] * y.y * y.y;
    dblk *= pd;
    gsum += lg[i];
  }
  *reinterpret_cast<float4*>(&sEnd[warp][c4]) = make_float4(a[0], a[1], a[2], a[3]);
  if (lane == 0) { sDec[warp] = dblk; sSum[warp] = gsum; }
  __syncthreads();
  if (tid < kD) {
    float acc = 0.f;
#pragma unroll
    for (int b = 0; b < 8; ++b) acc = sDec[b] * acc + sEnd[b][tid];
    ac_local[chh * kD + tid] = acc;
  }
  if (tid == 0) {
    float g = 0.f;
#pragma unroll
    for (int b = 0; b < 8; ++b) g += sSum[b];
    sa[chh] = g;
  }
}

// Sequential carry over the chunks of one (sequence, head): A at each chunk start.
__global__ void __launch_bounds__(kD)
pkda_atk_carry_kernel(Geo geo, const float* ac_local, const float* sa, const float* A0,
                      float* a_start, float* AT) {
  const int n = blockIdx.x, h = blockIdx.y, H = geo.heads, c = threadIdx.x;
  const SeqInfo sq = seq_info(geo, n);
  float A = A0 ? A0[((size_t)n * H + h) * kD + c] : 0.f;
  constexpr int kBatch = 16;  // loads of 16 chunks in flight before the dependent multiply-adds
  for (int i0 = 0; i0 < sq.nchunks; i0 += kBatch) {
    float dec[kBatch], loc[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const bool ok = i0 + j < sq.nchunks;
      const size_t ch = (size_t)(sq.chunk0 + (ok ? i0 + j : 0)) * H + h;
      dec[j] = ok ? sa[ch] : 0.f;
      loc[j] = ok ? ac_local[ch * kD + c] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (i0 + j < sq.nchunks) {
        a_start[((size_t)(sq.chunk0 + i0 + j) * H + h) * kD + c] = A;
        A = __expf(dec[j]) * A + loc[j];
      }
    }
  }
  if (AT) AT[((size_t)n * H + h) * kD + c] = A;
}

// ------------------------------------------------------------------ intra-chunk kernel
namespace intra {
constexpr int kThreads = 512;
constexpr int oQ = 0;
constexpr int oK = oQ + kTileBytes;
constexpr int oKt = oK + kTileBytes;
constexpr int oG = oKt + kTileBytes;              // fp32 [64][kLdG]
constexpr int oStage = oG + kChunk * kLdG * 4;    // 3 bf16 tiles; aliased (see below)
constexpr int oTmb = oStage + 3 * kTileBytes;     // bf16 [64][72]: P staging, then Tm
constexpr int oSmall = oTmb + kChunk * kLdC * 2;  // beta[64] pd[64] bp[64] bias[128]
constexpr int kSmem = oSmall + (3 * kChunk + kD + 24) * 4;  // + per-warp block-decay maxima
// aliases inside the staging area
constexpr int oAt = oStage;                       // fp32 [64][kLdG] preconditioner states (before the levels)
constexpr int kLdL = 68;                          // = 4 (mod 8): the inverse's MMA fragments load without bank conflicts
constexpr int oL = oStage;                        // after the levels: L, T, Y2
constexpr int oT = oL + kChunk * kLdL * 4;
constexpr int oY2 = oT + kChunk * kLdL * 4;       // fp32 [1280]
static_assert(oY2 + 1280 * 4 <= oTmb, "inverse scratch must fit in the staging area");
static_assert(kChunk * kLdG * 4 <= 3 * kTileBytes, "A_t array must fit in the staging area");
}  // namespace intra

// Writes one 16x16 accumulator tile pair (two n8 tiles) through a functor f(i, j, value).
template <typename F>
__device__ __forceinline__ void for_tile(const float (&t)[2][4], int i0, int j0, int gq, int tq, F f) {
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) f(i0 + gq + 8 * (e >> 1), j0 + 8 * nt + 2 * tq + (e & 1), t[nt][e]);
}

// kRecompute: rebuild w,u,kg,qg only (backward's lean mode); the products, the
// write keys and the decay totals already exist and are left untouched.
// One (chunk bx, head by) item; every thread of the CTA takes part.
template <bool kRecompute>
__device__ __forceinline__ void intra_fwd_item(const IntraParams& p, int bx, int by) {
  using namespace intra;
  extern __shared__ __align__(128) unsigned char smem[];
  bf16* sQ = reinterpret_cast<bf16*>(smem + oQ);
  bf16* sK = reinterpret_cast<bf16*>(smem + oK);
  bf16* sKt = reinterpret_cast<bf16*>(smem + oKt);
  float* sG = reinterpret_cast<float*>(smem + oG);
  bf16* sXq = reinterpret_cast<bf16*>(smem + oStage);
  bf16* sXk = sXq + kChunk * kLdD;
  bf16* sY = sXk + kChunk * kLdD;
  bf16* sTmb = reinterpret_cast<bf16*>(smem + oTmb);
  float* sBeta = reinterpret_cast<float*>(smem + oSmall);
  float* sPd = sBeta + kChunk;
  float* sBp = sPd + kChunk;
  float* sBias = sBp + kChunk;
  float* sWarpMax = sBias + kD;  // [4][6]
  float* sAt = reinterpret_cast<float*>(smem + oAt);
  float* sL = reinterpret_cast<float*>(smem + oL);
  float* sT = reinterpret_cast<float*>(smem + oT);
  float* sY2 = reinterpret_cast<float*>(smem + oY2);

  int n, tok0, valid;
  if (!chunk_lookup(p.geo, bx, n, tok0, valid)) return;
  const int h = by, H = p.geo.heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const size_t chh = (size_t)bx * H + h;
  const size_t row0 = ((size_t)tok0 * H + h) * kD;  // element offset of (tok0, h, 0)
  const long gld = (long)H * kD;

  // ---- 1. tiles and per-row scalars.  The per-row scalars are requested first (the first barrier
  // waits for them and they would otherwise queue behind the 48 KB of tile traffic), then the raw
  // gate (needed next), then the q and k tiles.
  float s_beta = 0.f, s_pd = 0.f, s_bp = 0.f, s_bias = 0.f;
  if (tid < kChunk) {
    const size_t s = (size_t)(tok0 + min(tid, valid - 1)) * H + h;
    s_beta = p.beta_c[chh * kChunk + tid];
    s_pd = p.g_atk[s];
    s_bp = to_f(p.beta_atk[s]);
  } else if (tid < kChunk + kD) {
    s_bias = p.dt_bias[h * kD + tid - kChunk];
  }
  GateRaw<kThreads> graw;
  gate_load(graw, p.g + row0, gld, valid, tid);
  // Scalars of later phases are fetched here: a global load issued where it is used costs
  // that phase a full memory round trip with nothing to overlap it.
  const float a_log = p.A_log[h];
  const float centre = kRecompute ? 0.f : p.log_atk_scale[h];
  float a_first = 0.f;
  if (!kRecompute && tid >= kD && tid < 2 * kD) a_first = p.a_start[chh * kD + tid - kD];
  tile_load_async(sQ, kLdD, p.q + row0, gld, kChunk, kD, valid, kThreads);
  tile_load_async(sK, kLdD, p.k + row0, gld, kChunk, kD, valid, kThreads);
  if (kRecompute) tile_load_async(sKt, kLdD, p.kt + row0, gld, kChunk, kD, valid, kThreads);
  cp_async_commit();
  if (tid < kChunk) {
    const bool ok = tid < valid;
    sBeta[tid] = s_beta;
    sPd[tid] = ok ? __expf(s_pd) : 1.f;
    sBp[tid] = ok ? s_bp : 0.f;
  } else if (tid < kChunk + kD) {
    sBias[tid - kChunk] = s_bias;
  }
  // zero the P staging tile (upper triangle must read as zero)
  for (int i = tid; i < kChunk * kLdC / 8; i += kThreads) reinterpret_cast<uint4*>(sTmb)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();

  // ---- 2. decay gate (elementwise, all threads; the q and k tiles are still landing), then
  // the two per-channel sequential passes side by side: cumulative sum | preconditioner recurrence A_t
  gate_apply(graw, sG, valid, sBias, __expf(a_log) * kLog2e, tid);
  cp_async_wait<0>();
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
  } else if (!kRecompute && tid < 2 * kD) {
    const int c = tid - kD;
    float A = a_first;
#pragma unroll 8
    for (int r = 0; r < kChunk; ++r) {
      const float kc = to_f(sK[r * kLdD + c]);
      A = sPd[r] * A + sBp[r] * kc * kc;
      sAt[r * kLdG + c] = A;
    }
  }
  __syncthreads();
  if (!kRecompute) {
    // write keys kt = k * exp(-ln(x) * dev / (1 + |dev|)), dev = log(A + eps) - centre
    for (int idx = tid; idx < kChunk * kD / 8; idx += kThreads) {
      const int r = idx >> 4, c8 = (idx & 15) << 3;
      const float4 A0 = *reinterpret_cast<const float4*>(sAt + r * kLdG + c8);
      const float4 A1 = *reinterpret_cast<const float4*>(sAt + r * kLdG + c8 + 4);
      const float Av[8] = {A0.x, A0.y, A0.z, A0.w, A1.x, A1.y, A1.z, A1.w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float dev = __logf(Av[j] + p.eps) - centre;
        f[j] = __expf(-p.ln_x * __fdividef(dev, 1.f + fabsf(dev)));
      }
      uint4 x = *reinterpret_cast<const uint4*>(sK + r * kLdD + c8);
      scale8(x, f);
      *reinterpret_cast<uint4*>(sKt + r * kLdD + c8) = x;
      if (r < valid) *reinterpret_cast<uint4*>(p.kt + row0 + (size_t)r * gld + c8) = x;
    }
    __syncthreads();
  }

  // ---- 3. gated pair products, level by level.
  // warps 0-7 : (mat, I) own the diagonal 16x16 tile (I,I): levels 8,4,2,1 (and the ungated diagonal of P)
  // warps 8-15: (mat, idx) own one tile of level 32 and (idx < 2) one tile of level 16
  // mat 0 = M (rows k), mat 1 = P (rows q).
  const bool diagw = warp < 8;
  const int mat = (warp >> 2) & 1, I = warp & 3;
  float accA[2][4], accB[2][4];  // diag warps: accA; off warps: accA = level-32 tile, accB = level-16 tile
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int e = 0; e < 4; ++e) accA[a][e] = accB[a][e] = 0.f;
  const int I32 = 2 + (I >> 1), J32 = I & 1;   // level-32 tile of an off warp
  const int I16 = 1 + 2 * I, J16 = 2 * I;      // level-16 tile (I < 2)

  // Pairs inside a b-block go through the direct level (lvl = 0), the rest through
  // hierarchy levels >= b.  Each off-diagonal tile is produced exactly once.
  const int bdir = pick_direct_block(sWarpMax, 4, p.direct_cap);
#pragma unroll 1
  for (int it = (bdir > 1 ? 0 : 1); it <= 6; ++it) {
    const int lvl = it ? (64 >> it) : 0;  // 0 (direct), 32, 16, 8, 4, 2, 1
    if (lvl && lvl < bdir) break;
    stage_level(sXq, sXk, sY, sQ, sK, sKt, sG, lvl, bdir, tid, kThreads);
    __syncthreads();
    const bf16* X = mat ? sXq : sXk;
    float tmp[1][2][4];
    if (!diagw) {
      // level-32 region tile: by hierarchy level 32 unless the direct block covers it (b = 64)
      if ((lvl == 32) || (lvl == 0 && bdir > 32)) {
        zero_acc(tmp);
        warp_gemm<1, 2, false, false>(tmp, X, kLdD, 16 * I32, sY, kLdD, 16 * J32, 0, kD);
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int e = 0; e < 4; ++e) accA[a][e] = tmp[0][a][e];
      }
      // level-16 region tile: by hierarchy level 16 unless the direct block covers it (b >= 32)
      if (I < 2 && ((lvl == 16 && bdir <= 16) || (lvl == 0 && bdir > 16))) {
        zero_acc(tmp);
        warp_gemm<1, 2, false, false>(tmp, X, kLdD, 16 * I16, sY, kLdD, 16 * J16, 0, kD);
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int e = 0; e < 4; ++e) accB[a][e] = tmp[0][a][e];
      }
    } else if (lvl <= 8) {
      zero_acc(tmp);
      warp_gemm<1, 2, false, false>(tmp, X, kLdD, 16 * I, sY, kLdD, 16 * I, 0, kD);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = 16 * I + gq + ((e >> 1) << 3);
          const int j = 16 * I + 8 * nt + 2 * tq + (e & 1);
          if (pair_ok(i, j, lvl, bdir)) accA[nt][e] += tmp[0][nt][e];
        }
    }
    __syncthreads();
  }
  if (diagw && mat == 1) {  // diagonal of P: ungated q_i . kt_i
    float tmp[1][2][4];
    zero_acc(tmp);
    warp_gemm<1, 2, false, false>(tmp, sQ, kLdD, 16 * I, sKt, kLdD, 16 * I, 0, kD);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 16 * I + gq + ((e >> 1) << 3);
        const int j = 16 * I + 8 * nt + 2 * tq + (e & 1);
        if (i == j) accA[nt][e] += tmp[0][nt][e];
      }
  }

  // ---- 4. P -> bf16 staging tile (scaled) ; L = tril(M,-1) diag(beta) -> smem fp32
  for (int i = tid; i < kChunk * kLdL; i += kThreads) sL[i] = 0.f;
  __syncthreads();
  {
    auto putP = [&](int i, int j, float v) { if (j <= i) sTmb[i * kLdC + j] = __float2bfloat16(v * p.scale); };
    auto putL = [&](int i, int j, float v) { if (j < i) sL[i * kLdL + j] = v * sBeta[j]; };
    if (diagw) {
      if (mat) for_tile(accA, 16 * I, 16 * I, gq, tq, putP); else for_tile(accA, 16 * I, 16 * I, gq, tq, putL);
    } else {
      if (mat) for_tile(accA, 16 * I32, 16 * J32, gq, tq, putP); else for_tile(accA, 16 * I32, 16 * J32, gq, tq, putL);
      if (I < 2) {
        if (mat) for_tile(accB, 16 * I16, 16 * J16, gq, tq, putP); else for_tile(accB, 16 * I16, 16 * J16, gq, tq, putL);
      }
    }
  }
  __syncthreads();
  if (!kRecompute) {
    for (int i = tid; i < kChunk * kChunk / 8; i += kThreads) {
      const int r = i >> 3, c8 = (i & 7) << 3;
      if (r < valid)
        *reinterpret_cast<uint4*>(p.Aqk + ((size_t)(tok0 + r) * H + h) * kChunk + c8) =
            *reinterpret_cast<const uint4*>(sTmb + r * kLdC + c8);
    }
  }

  // ---- 5. T = (I + L)^-1 in fp32
  unit_lower_inverse_64<8>(sL, sT, sY2, kLdL, kLdL, tid, kThreads);  // ends with a __syncthreads()
  for (int i = tid; i < kChunk * kChunk / 2; i += kThreads) {
    const int r = i >> 5, c2 = (i & 31) << 1;
    const uint32_t pk = pack_bf16(sT[r * kLdL + c2], sT[r * kLdL + c2 + 1]);
    *reinterpret_cast<uint32_t*>(sTmb + r * kLdC + c2) = pk;
    if (!kRecompute && r < valid)
      *reinterpret_cast<uint32_t*>(p.Akk + ((size_t)(tok0 + r) * H + h) * kChunk + c2) = pk;
  }
  __syncthreads();

  // ---- 6. decayed operands: Kd -> smem; qg, kg, gc -> global; V tile -> smem
  bf16* sKd = sXq;
  bf16* sV = sXk;
  tile_load_async(sV, kLdD, p.v + row0, gld, kChunk, kD, valid, kThreads);
  cp_async_commit();
  for (int idx = tid; idx < kChunk * kD / 8; idx += kThreads) {
    const int r = idx >> 4, c8 = (idx & 15) << 3;
    const float4 g0 = *reinterpret_cast<const float4*>(sG + r * kLdG + c8);
    const float4 g1 = *reinterpret_cast<const float4*>(sG + r * kLdG + c8 + 4);
    const float4 l0 = *reinterpret_cast<const float4*>(sG + (kChunk - 1) * kLdG + c8);
    const float4 l1 = *reinterpret_cast<const float4*>(sG + (kChunk - 1) * kLdG + c8 + 4);
    const float G[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const float Gl[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
    float e[8], es[8], tl[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      e[j] = ex2(G[j]);
      es[j] = e[j] * p.scale;
      tl[j] = ex2(Gl[j] - G[j]);
    }
    uint4 kk = *reinterpret_cast<const uint4*>(sK + r * kLdD + c8);
    scale8(kk, e);
    *reinterpret_cast<uint4*>(sKd + r * kLdD + c8) = kk;
    if (r < valid) {
      uint4 qq = *reinterpret_cast<const uint4*>(sQ + r * kLdD + c8);
      uint4 kt = *reinterpret_cast<const uint4*>(sKt + r * kLdD + c8);
      scale8(qq, es);
      scale8(kt, tl);
      const size_t off = row0 + (size_t)r * gld + c8;
      *reinterpret_cast<uint4*>(p.qg + off) = qq;
      *reinterpret_cast<uint4*>(p.kg + off) = kt;
    }
    if (!kRecompute && r == kChunk - 1) {
      *reinterpret_cast<float4*>(p.gc + chh * kD + c8) = make_float4(e[0], e[1], e[2], e[3]);
      *reinterpret_cast<float4*>(p.gc + chh * kD + c8 + 4) = make_float4(e[4], e[5], e[6], e[7]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- 7. W = Tm Kd, U = Tm V   (warp: matrix = warp>>3, rows 16*((warp>>1)&3), column half warp&1)
  {
    const int m7 = warp >> 3, I7 = (warp >> 1) & 3, n0 = 64 * (warp & 1);
    float acc2[1][8][4];
    zero_acc(acc2);
    warp_gemm<1, 8, false, true>(acc2, sTmb, kLdC, 16 * I7, m7 ? sV : sKd, kLdD, n0, 0, 16 * (I7 + 1));
    bf16* dst = m7 ? p.u : p.w;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = 16 * I7 + gq + 8 * half;
        if (i < valid)
          *reinterpret_cast<uint32_t*>(dst + row0 + (size_t)i * gld + n0 + 8 * nt + 2 * tq) =
              pack_bf16(acc2[0][nt][2 * half], acc2[0][nt][2 * half + 1]);
      }
  }
}

// grid (chunks, heads): one item per CTA; or, with a work list, a few persistent CTAs that walk it.
template <bool kRecompute>
__global__ void __launch_bounds__(intra::kThreads, 1)
pkda_intra_fwd_kernel(const IntraParams p) {
  if (!p.slow_list) {
    intra_fwd_item<kRecompute>(p, blockIdx.x, blockIdx.y);
    return;
  }
  // items differ in cost (the number of pairing levels follows the decay): CTAs draw them one at a time
  __shared__ int s_item;
  const int n_items = p.counts[1], H = p.geo.heads;
  for (;;) {
    if (threadIdx.x == 0) s_item = atomicAdd(p.counts + 2, 1);
    __syncthreads();
    const int item = s_item;
    if (item >= n_items) break;
    const int chh = p.slow_list[item];
    intra_fwd_item<kRecompute>(p, chh / H, chh % H);
    __syncthreads();  // the next item reuses every shared-memory region (and s_item)
  }
}

// ------------------------------------------------------------------ forward state scan
struct ScanParams {
  Geo geo;
  const bf16 *w, *u, *kg;
  const float *beta_c, *gc;
  const float* S0;
  bf16 *h, *v_new;
  float* ST;
};

namespace scan {
template <int VB> __host__ __device__ constexpr int threads() { return 128 * (VB / 32); }  // 4 warps per 32 value columns
template <int VB> struct L {
  static constexpr int ldv = VB + kPad;
  static constexpr int oW = 0;
  static constexpr int oKg = oW + kTileBytes;
  static constexpr int oU = oKg + kTileBytes;            // bf16 [64][ldv]
  static constexpr int oBeta = oU + kChunk * ldv * 2;    // f32 [64]
  static constexpr int oGc = oBeta + kChunk * 4;         // f32 [128]
  static constexpr int kStage = oGc + kD * 4;
  static constexpr int oH = 2 * kStage;                  // bf16 [128][ldv]
  static constexpr int oF = oH + kD * ldv * 2;           // bf16 [64][ldv]
  static constexpr int kSmem = oF + kChunk * ldv * 2;
};
}  // namespace scan

template <int VB, bool kRecompute>
__global__ void __launch_bounds__(scan::threads<VB>())
pkda_scan_fwd_kernel(const ScanParams p) {
  using Lay = scan::L<VB>;
  constexpr int ldv = Lay::ldv, NT = 4, kT = scan::threads<VB>();
  extern __shared__ __align__(128) unsigned char smem[];
  const int VS = kD / VB;
  const int vs = blockIdx.x % VS;
  const int nh = blockIdx.x / VS;
  const int n = nh / p.geo.heads, h = nh - n * p.geo.heads, H = p.geo.heads;
  const SeqInfo sq = seq_info(p.geo, n);
  if (sq.nchunks == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int wr = warp & 3, c0 = 32 * (warp >> 2);  // this warp: state rows [32 wr, +32), columns [c0, +32) of the slice
  const int v0 = vs * VB;
  const long gld = (long)H * kD;
  bf16* sH = reinterpret_cast<bf16*>(smem + Lay::oH);
  bf16* sF = reinterpret_cast<bf16*>(smem + Lay::oF);

  auto prefetch = [&](int i) {
    unsigned char* st = smem + (i & 1) * Lay::kStage;
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t row0 = ((size_t)tok0 * H + h) * kD;
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;
    tile_load_async(reinterpret_cast<bf16*>(st + Lay::oW), kLdD, p.w + row0, gld, kChunk, kD, valid, kT);
    tile_load_async(reinterpret_cast<bf16*>(st + Lay::oKg), kLdD, p.kg + row0, gld, kChunk, kD, valid, kT);
    tile_load_async(reinterpret_cast<bf16*>(st + Lay::oU), ldv, p.u + row0 + v0, gld, kChunk, VB, valid, kT);
    if (tid < 16) cp_async16(st + Lay::oBeta + tid * 16, p.beta_c + chh * kChunk + tid * 4, true);
    else if (tid < 48) cp_async16(st + Lay::oGc + (tid - 16) * 16, p.gc + chh * kD + (tid - 16) * 4, true);
  };

  // state rows [32*warp, +32) x VB columns, fp32 fragments
  float S[2][NT][4];
  const size_t sbase = ((size_t)n * H + h) * kD * kD;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = 32 * wr + 16 * mt + gq + 8 * half, c = v0 + c0 + 8 * nt + 2 * tq;
        float2 s2 = make_float2(0.f, 0.f);
        if (p.S0) s2 = *reinterpret_cast<const float2*>(p.S0 + sbase + (size_t)r * kD + c);
        S[mt][nt][2 * half] = s2.x;
        S[mt][nt][2 * half + 1] = s2.y;
      }

  prefetch(0);
  cp_async_commit();
  for (int i = 0; i < sq.nchunks; ++i) {
    if (i + 1 < sq.nchunks) prefetch(i + 1);
    cp_async_commit();
    cp_async_wait<1>();
    unsigned char* st = smem + (i & 1) * Lay::kStage;
    const bf16* sW = reinterpret_cast<const bf16*>(st + Lay::oW);
    const bf16* sKg = reinterpret_cast<const bf16*>(st + Lay::oKg);
    const bf16* sU = reinterpret_cast<const bf16*>(st + Lay::oU);
    const float* sBeta = reinterpret_cast<const float*>(st + Lay::oBeta);
    const float* sGc = reinterpret_cast<const float*>(st + Lay::oGc);
    const int tok0 = sq.bos + i * kChunk;
    const int valid = min(kChunk, sq.len - i * kChunk);
    const size_t chh = (size_t)(sq.chunk0 + i) * H + h;

    // a. chunk-entry state -> bf16 operand tile (and the saved chunk states)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 32 * wr + 16 * mt + gq + 8 * half, c = c0 + 8 * nt + 2 * tq;
          *reinterpret_cast<uint32_t*>(sH + r * ldv + c) = pack_bf16(S[mt][nt][2 * half], S[mt][nt][2 * half + 1]);
        }
    __syncthreads();  // sH complete; stage i landed for every thread
    {
      constexpr int cpr = VB / 8;
      for (int j = tid; j < kD * cpr; j += kT) {
        const int r = j / cpr, c = (j - r * cpr) * 8;
        *reinterpret_cast<uint4*>(p.h + (chh * kD + r) * kD + v0 + c) =
            *reinterpret_cast<const uint4*>(sH + r * ldv + c);
      }
    }
    // b. E = U - W h ; F = beta * E
    {
      float e[1][NT][4];
      zero_acc(e);
      warp_gemm<1, NT, false, true>(e, sW, kLdD, 16 * wr, sH, ldv, c0, 0, kD);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 16 * wr + gq + 8 * half, c = c0 + 8 * nt + 2 * tq;
          const float2 uu = unpack_bf16(*reinterpret_cast<const uint32_t*>(sU + r * ldv + c));
          const uint32_t ek = pack_bf16(uu.x - e[0][nt][2 * half], uu.y - e[0][nt][2 * half + 1]);
          if (r < valid)
            *reinterpret_cast<uint32_t*>(p.v_new + ((size_t)(tok0 + r) * H + h) * kD + v0 + c) = ek;
          const float2 er = unpack_bf16(ek);
          const float b = sBeta[r];
          *reinterpret_cast<uint32_t*>(sF + r * ldv + c) = pack_bf16(b * er.x, b * er.y);
        }
    }
    __syncthreads();
    // c. S <- Gam_last * S + kg^T F
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float gcv = sGc[32 * wr + 16 * mt + gq + 8 * half];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          S[mt][nt][2 * half] *= gcv;
          S[mt][nt][2 * half + 1] *= gcv;
        }
      }
    warp_gemm<2, NT, true, true>(S, sKg, kLdD, 32 * wr, sF, ldv, c0, 0, kChunk);
    __syncthreads();  // everyone done with stage i and sF before they are refilled
  }
  cp_async_wait<0>();
  if (!kRecompute && p.ST) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 32 * wr + 16 * mt + gq + 8 * half, c = v0 + c0 + 8 * nt + 2 * tq;
          *reinterpret_cast<float2*>(p.ST + sbase + (size_t)r * kD + c) =
              make_float2(S[mt][nt][2 * half], S[mt][nt][2 * half + 1]);
        }
  }
}

// ------------------------------------------------------------------ output kernel
struct OutParams {
  Geo geo;
  const bf16 *qg, *h, *Aqk, *v_new;
  const float* beta_c;
  bf16* o;
};

namespace outk {
constexpr int kThreads = 256;
constexpr int oQg = 0;
constexpr int oH = oQg + kTileBytes;              // bf16 [128][136]
constexpr int oP = oH + kD * kLdD * 2;            // bf16 [64][72]
constexpr int oF = oP + kChunk * kLdC * 2;        // bf16 [64][136]
constexpr int kSmem = oF + kTileBytes;
}  // namespace outk

__global__ void __launch_bounds__(outk::kThreads)
pkda_out_fwd_kernel(const OutParams p) {
  using namespace outk;
  extern __shared__ __align__(128) unsigned char smem[];
  bf16* sQg = reinterpret_cast<bf16*>(smem + oQg);
  bf16* sH = reinterpret_cast<bf16*>(smem + oH);
  bf16* sP = reinterpret_cast<bf16*>(smem + oP);
  bf16* sF = reinterpret_cast<bf16*>(smem + oF);
  int n, tok0, valid;
  if (!chunk_lookup(p.geo, blockIdx.x, n, tok0, valid)) return;
  const int h = blockIdx.y, H = p.geo.heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const size_t chh = (size_t)blockIdx.x * H + h;
  const size_t row0 = ((size_t)tok0 * H + h) * kD;
  const long gld = (long)H * kD;

  tile_load_async(sQg, kLdD, p.qg + row0, gld, kChunk, kD, valid, kThreads);
  tile_load_async(sH, kLdD, p.h + chh * kD * kD, kD, kD, kD, kD, kThreads);
  tile_load_async(sP, kLdC, p.Aqk + ((size_t)tok0 * H + h) * kChunk, (long)H * kChunk, kChunk, kChunk, valid, kThreads);
  cp_async_commit();
  // F = beta * E (E read from global, rounded exactly as the scan rounded it)
  for (int i = tid; i < kChunk * kD / 8; i += kThreads) {
    const int r = i >> 4, c = (i & 15) << 3;
    uint4 ev = make_uint4(0, 0, 0, 0);
    if (r < valid) ev = *reinterpret_cast<const uint4*>(p.v_new + row0 + (size_t)r * gld + c);
    const float b = p.beta_c[chh * kChunk + r];
    uint32_t* e32 = reinterpret_cast<uint32_t*>(&ev);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = unpack_bf16(e32[j]);
      e32[j] = pack_bf16(b * x.x, b * x.y);
    }
    *reinterpret_cast<uint4*>(sF + r * kLdD + c) = ev;
  }
  cp_async_wait<0>();
  __syncthreads();

  const int I = warp & 3, n0 = 64 * (warp >> 2);
  float acc[1][8][4];
  zero_acc(acc);
  warp_gemm<1, 8, false, true>(acc, sQg, kLdD, 16 * I, sH, kLdD, n0, 0, kD);
  warp_gemm<1, 8, false, true>(acc, sP, kLdC, 16 * I, sF, kLdD, n0, 0, 16 * (I + 1));
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = 16 * I + gq + 8 * half;
      if (i < valid)
        *reinterpret_cast<uint32_t*>(p.o + row0 + (size_t)i * gld + n0 + 8 * nt + 2 * tq) =
            pack_bf16(acc[0][nt][2 * half], acc[0][nt][2 * half + 1]);
    }
}

// ------------------------------------------------------------------ host side
struct FwdWorkspace {
  int* chain_flags;  // one counter per (chunk, head) item, right behind the status slot (zeroed with it)
  int* chunk_offsets;
  float* beta_c;
  bf16* u;
  int* lists;   // work list of the intra-chunk stage (chunks * heads ints)
  int* status;  // device status word: 0 = ok, 1 = a bounded wait in a kernel gave up; then the list lengths
  size_t bytes;
};

static FwdWorkspace carve_fwd(const pkda_problem& p, void* base) {
  FwdWorkspace w;
  const size_t chunks = (size_t)chunk_bound(p);
  size_t off = 0;
  unsigned char* b = static_cast<unsigned char*>(base);
  w.chunk_offsets = reinterpret_cast<int*>(b + off);
  off += align_up((size_t)(p.n_seqs + 1) * sizeof(int));
  w.beta_c = reinterpret_cast<float*>(b + off);
  off += align_up(chunks * p.heads * kChunk * sizeof(float));
  w.u = reinterpret_cast<bf16*>(b + off);
  off += align_up((size_t)p.total_tokens * p.heads * kD * sizeof(bf16));
  w.lists = reinterpret_cast<int*>(b + off);
  off += align_up(chunks * p.heads * sizeof(int));
  w.status = reinterpret_cast<int*>(b + off);
  off += 8 * sizeof(int);
  w.chain_flags = reinterpret_cast<int*>(b + off);
  off += align_up(chunks * p.heads * sizeof(int));
  w.bytes = off;
  return w;
}

size_t chunk_fwd_workspace(const pkda_problem& p) { return carve_fwd(p, nullptr).bytes; }

bool forward_chain_possible(const pkda_problem& p) {
  // With few (row, head) units the chains are few and long compared with the number of items in
  // flight, and an item waits for many hand-overs: measured break-even near 32 units (the state it
  // yields is the same bit for bit either way).
  return !p.cu_seqlens && stage_variant(kStageIntraFwd) == 0 && direct_block_cap() >= 64 &&
         (long)p.n_seqs * p.heads >= 32;
}
size_t chunk_fwd_status_offset(const pkda_problem& p) {
  return (size_t)(reinterpret_cast<unsigned char*>(carve_fwd(p, nullptr).status) - static_cast<unsigned char*>(nullptr));
}

template <typename K>
static bool set_smem(K kernel, int bytes) {
  return ensure_dynamic_smem(kernel, bytes);
}

#define PKDA_CHECK_LAUNCH()                                        \
  do {                                                             \
    end_stage(st);                                                 \
    if (cudaGetLastError() != cudaSuccess) return PKDA_ERR_LAUNCH; \
  } while (0)

int check_chunk_problem(const pkda_problem& p) {
  int rc = check_problem(p);
  if (rc != PKDA_OK) return rc;
  if (p.head_dim != kD) return PKDA_ERR_SHAPE;
  if (p.dtype != PKDA_BF16) return PKDA_ERR_DTYPE;
  return PKDA_OK;
}

template <int VB, bool kRecompute>
static int launch_scan_fwd(const ScanParams& sp, int units, cudaStream_t st) {
  if (!set_smem(pkda_scan_fwd_kernel<VB, kRecompute>, scan::L<VB>::kSmem)) return PKDA_ERR_LAUNCH;
  pkda_scan_fwd_kernel<VB, kRecompute><<<units * (kD / VB), scan::threads<VB>(), scan::L<VB>::kSmem, st>>>(sp);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

// Shared by the forward and by the backward's recompute mode.
int run_forward_stages(const pkda_problem& p, const Geo& geo, const float* beta_c, bf16* u_ws,
                       bf16* Aqk, bf16* Akk, bf16* kt, float* gc, const float* a_start,
                       bf16* w, bf16* kg, bf16* v_new, bf16* h, bf16* qg, float* ST,
                       bool recompute, int* status, int* lists, int* counts, cudaStream_t st, bf16* o,
                       bool* o_done, const ChainArgs* chain) {
  const int chunks = geo.total_chunks;
  IntraParams ip;
  ip.geo = geo;
  ip.q = static_cast<const bf16*>(p.q); ip.k = static_cast<const bf16*>(p.k);
  ip.v = static_cast<const bf16*>(p.v); ip.g = static_cast<const bf16*>(p.g);
  ip.g_atk = p.g_atk; ip.beta_atk = static_cast<const bf16*>(p.beta_atk);
  ip.A_log = p.A_log; ip.dt_bias = p.dt_bias; ip.log_atk_scale = p.log_atk_scale;
  ip.beta_c = beta_c; ip.a_start = a_start;
  ip.Aqk = Aqk; ip.Akk = Akk; ip.kt = kt; ip.gc = gc;
  ip.w = w; ip.u = u_ws; ip.kg = kg; ip.qg = qg;
  ip.scale = p.scale; ip.ln_x = logf(p.squash_x); ip.eps = p.squash_eps;
  ip.direct_cap = direct_block_cap();
  ip.status = status;
  ip.slow_list = ip.counts = nullptr;
  ip.chain = 0;
  ip.beta = static_cast<const bf16*>(p.beta); ip.A0 = p.initial_A_state;
  ip.beta_c_w = ip.a_chain = ip.sa = ip.AT = nullptr;
  ip.chain_flags = nullptr;
  if (chain && !recompute && status && lists && forward_chain_possible(p)) {
    ip.chain = 1;
    ip.beta_c_w = chain->beta_c_w; ip.a_chain = chain->a_chain; ip.sa = chain->sa; ip.AT = chain->AT;
    ip.chain_flags = chain->flags;
  }
  dim3 gridc(chunks, p.heads);
  // Chunks that are one direct block run on tcgen05 / tensor memory; that kernel lists the others and
  // the mma.sync kernel works the list off (it takes every chunk, one CTA each, when it is pinned or the
  // direct block is capped).  The recompute pass of a lean backward decides the same way, from the same
  // inputs, so that every chunk is rebuilt by the kernel that built it.
  if (status && lists && stage_variant(kStageIntraFwd) == 0 && ip.direct_cap >= 64) {
    const int items = chunks * p.heads;
    ip.slow_list = lists; ip.counts = counts;
    begin_stage(kStageIntraFwd, st);
    const int rc_tc = launch_intra_fwd_tc(ip, recompute, st);
    end_stage(st);
    if (rc_tc != PKDA_OK) return rc_tc;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    gridc = dim3(items < sms ? items : sms, 1);
  }
  const int rest_stage = ip.slow_list ? kStageIntraFwdRest : kStageIntraFwd;
  if (recompute) {
    if (!set_smem(pkda_intra_fwd_kernel<true>, intra::kSmem)) return PKDA_ERR_LAUNCH;
    begin_stage(rest_stage, st);
    pkda_intra_fwd_kernel<true><<<gridc, intra::kThreads, intra::kSmem, st>>>(ip);
  } else {
    if (!set_smem(pkda_intra_fwd_kernel<false>, intra::kSmem)) return PKDA_ERR_LAUNCH;
    begin_stage(rest_stage, st);
    pkda_intra_fwd_kernel<false><<<gridc, intra::kThreads, intra::kSmem, st>>>(ip);
  }
  PKDA_CHECK_LAUNCH();

  ScanParams sp;
  sp.geo = geo; sp.w = w; sp.u = u_ws; sp.kg = kg; sp.beta_c = beta_c; sp.gc = gc;
  sp.S0 = p.initial_state; sp.h = h; sp.v_new = v_new; sp.ST = ST;
  // The scan runs on tcgen05 / TMEM / TMA, one CTA per (sequence, head), unless the mma.sync kernel is
  // pinned (pkda_set_variant).  That holds for few units too: a chunk step is a latency chain whose
  // length does not depend on how many CTAs run (2 rows x 16 heads, T = 4096: 0.82 ms per
  // forward+backward against 0.87 ms with the value-sliced mma.sync scans).  The mma.sync kernel
  // slices the value columns when there are fewer units than SMs.
  const int units = p.n_seqs * p.heads;
  const int vb = units >= 120 ? 128 : (units >= 60 ? 64 : 32);
  int rc = PKDA_ERR_LAUNCH;
  const bool scan_mma = stage_variant(kStageScanFwd) == 1;
  // The tcgen05 scan also produces the output (it holds h and E of every chunk) unless a separate
  // output kernel is asked for (pkda_set_variant("out_fwd", 1: mma.sync, 2: tcgen05)).
  const bool fuse_out = o && !recompute && stage_variant(kStageOutFwd) == 0;
  if (o_done) *o_done = false;
  begin_stage(kStageScanFwd, st);
  if (status && !scan_mma) {
    rc = launch_scan_fwd_tc(geo, p.total_tokens, units, w, kg, u_ws, beta_c, gc, p.initial_state, h, v_new, ST,
                            status, recompute, qg, Aqk, fuse_out ? o : nullptr, st);
    if (o_done) *o_done = fuse_out;
  }
  else if (vb == 128) rc = recompute ? launch_scan_fwd<128, true>(sp, units, st) : launch_scan_fwd<128, false>(sp, units, st);
  else if (vb == 64) rc = recompute ? launch_scan_fwd<64, true>(sp, units, st) : launch_scan_fwd<64, false>(sp, units, st);
  else rc = recompute ? launch_scan_fwd<32, true>(sp, units, st) : launch_scan_fwd<32, false>(sp, units, st);
  end_stage(st);
  if (rc != PKDA_OK) return rc;
  return PKDA_OK;
}

int run_prologue(const pkda_problem& p, int* chunk_offsets, float* beta_c, Geo* geo, cudaStream_t st) {
  // beta_c == nullptr: the caller fills the chunk-major beta itself (the forward does, in its first kernel)
  if (p.cu_seqlens) {
    begin_stage(kStageOffsets, st);
    pkda_chunk_offsets_kernel<<<1, 32, 0, st>>>(p.cu_seqlens, p.n_seqs, chunk_offsets);
    PKDA_CHECK_LAUNCH();
  }
  *geo = make_geo(p, chunk_offsets);
  if (beta_c) {
    begin_stage(kStagePackBeta, st);
    pkda_pack_beta_kernel<<<geo->total_chunks, 256, 0, st>>>(*geo, static_cast<const bf16*>(p.beta), beta_c);
    PKDA_CHECK_LAUNCH();
  }
  return PKDA_OK;
}

int chunk_fwd(const pkda_chunk_fwd_args* a, cudaStream_t st) {
  const pkda_problem& p = a->p;
  int rc = check_chunk_problem(p);
  if (rc != PKDA_OK) return rc;
  if (p.n_seqs == 0 || p.total_tokens == 0) return PKDA_OK;
  if (!a->o || !a->Aqk || !a->Akk || !a->k_precond || !a->ac_atk || !a->a_atk || !a->sa_atk || !a->w ||
      !a->kg || !a->v_new || !a->h || !a->qg)
    return PKDA_ERR_NULL;
  if (!a->workspace || a->workspace_bytes < chunk_fwd_workspace(p)) return PKDA_ERR_WORKSPACE;
  FwdWorkspace ws = carve_fwd(p, a->workspace);
  Geo geo;
  rc = run_prologue(p, ws.chunk_offsets, nullptr, &geo, st);
  if (rc != PKDA_OK) return rc;

  // Dense batches on the default kernels: the intra stage carries the preconditioner state across
  // chunks itself (and packs beta).  Otherwise two small kernels in front do.
  const bool chained = forward_chain_possible(p);
  if (!chained) {
    dim3 gridc(geo.total_chunks, p.heads);
    begin_stage(kStageAtkLocal, st);
    pkda_atk_local_kernel<<<gridc, 256, 0, st>>>(geo, static_cast<const bf16*>(p.k), p.g_atk,
                                                 static_cast<const bf16*>(p.beta_atk), static_cast<const bf16*>(p.beta),
                                                 a->ac_atk, a->sa_atk, ws.beta_c);
    PKDA_CHECK_LAUNCH();
    begin_stage(kStageAtkCarry, st);
    pkda_atk_carry_kernel<<<dim3(p.n_seqs, p.heads), kD, 0, st>>>(geo, a->ac_atk, a->sa_atk, p.initial_A_state,
                                                                 a->a_atk, a->final_A_state);
    PKDA_CHECK_LAUNCH();
  }

  const size_t zero_ints = 8 + (chained ? (size_t)geo.total_chunks * p.heads : 0);  // status, cursors, chain counters
  if (cudaMemsetAsync(ws.status, 0, zero_ints * sizeof(int), st) != cudaSuccess) return PKDA_ERR_LAUNCH;
  ChainArgs chain_args;
  chain_args.beta_c_w = ws.beta_c; chain_args.a_chain = a->a_atk; chain_args.sa = a->sa_atk;
  chain_args.AT = a->final_A_state; chain_args.flags = ws.chain_flags;
  bool o_done = false;
  rc = run_forward_stages(p, geo, ws.beta_c, ws.u, static_cast<bf16*>(a->Aqk), static_cast<bf16*>(a->Akk),
                          static_cast<bf16*>(a->k_precond), a->ac_atk, a->a_atk, static_cast<bf16*>(a->w),
                          static_cast<bf16*>(a->kg), static_cast<bf16*>(a->v_new), static_cast<bf16*>(a->h),
                          static_cast<bf16*>(a->qg), a->final_state, false, ws.status, ws.lists, ws.status + 1, st,
                          static_cast<bf16*>(a->o), &o_done, chained ? &chain_args : nullptr);
  if (rc != PKDA_OK) return rc;

  // Output stage, when the scan has not produced o already: tcgen05 + TMA unless the mma.sync kernel is
  // pinned (pkda_set_variant).
  const size_t guard_n = std::min<size_t>((size_t)p.total_tokens * p.heads * kD, 4096);
  if (o_done) return PKDA_OK;  // (that kernel also marks the output if any kernel gave up)
  if (stage_variant(kStageOutFwd) != 1) {
    rc = launch_out_fwd_tc(geo, p.total_tokens, static_cast<const bf16*>(a->qg), static_cast<const bf16*>(a->h),
                           static_cast<const bf16*>(a->Aqk), static_cast<const bf16*>(a->v_new), ws.beta_c,
                           static_cast<bf16*>(a->o), ws.status, st);
    if (rc != PKDA_OK) return rc;
    return launch_status_guard(ws.status, a->o, nullptr, nullptr, guard_n, st);
  }
  OutParams op;
  op.geo = geo;
  op.qg = static_cast<const bf16*>(a->qg); op.h = static_cast<const bf16*>(a->h);
  op.Aqk = static_cast<const bf16*>(a->Aqk); op.v_new = static_cast<const bf16*>(a->v_new);
  op.beta_c = ws.beta_c; op.o = static_cast<bf16*>(a->o);
  if (!set_smem(pkda_out_fwd_kernel, outk::kSmem)) return PKDA_ERR_LAUNCH;
  begin_stage(kStageOutFwd, st);
  pkda_out_fwd_kernel<<<dim3(geo.total_chunks, p.heads), outk::kThreads, outk::kSmem, st>>>(op);
  PKDA_CHECK_LAUNCH();
  return launch_status_guard(ws.status, a->o, nullptr, nullptr, guard_n, st);
}

}  // namespace pkda

