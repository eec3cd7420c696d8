// Output stage of the chunked forward on the 5th-generation tensor cores:
//   O = qg h + (P diag(beta)) E        per (chunk, head)
// computed transposed so that the accumulator has 128 rows (one per value
// channel, = one TMEM lane each):
//   D[128 v][64 tok] = h^T[128 v x 128 k] qg^T[128 k x 64 tok] + E^T[128 v x 64 j] (P diag beta)^T[64 j x 64 tok]
// All four operand tiles arrive by TMA (128-byte swizzle) straight from the
// tensors the earlier stages wrote; the products are 12 tcgen05.mma (M=128,
// N=64, K=16) issued by one thread into a 64-column TMEM accumulator, which four
// warps read back with tcgen05.ld.  Every wait is bounded; on a timeout the CTA
// records a status word, skips its stores, frees its TMEM and exits.
#include "pkda_chunk.cuh"
#include "pkda_tc.cuh"

namespace pkda {

struct OutTcParams {
  Geo geo;
  const float* beta_c;
  bf16* o;
  int* status;
};

namespace outtc {
constexpr int kThreads = 128;
constexpr int oH = 0;                  // 2 blocks [128 k][64 v]   (A of product 1, MN-major)
constexpr int oQg = oH + 2 * 16384;    // 2 blocks [64 tok][64 k]  (B of product 1, K-major)
constexpr int oE = oQg + 2 * 8192;     // 2 blocks [64 j][64 v]    (A of product 2, MN-major)
constexpr int oP = oE + 2 * 8192;      // 1 block  [64 tok][64 j]  (B of product 2, K-major)
constexpr int oBar = oP + 8192;        // two mbarriers + the TMEM base address
constexpr int kTxBytes = oBar;
constexpr int kSmem = oBar + 64 + 1024;  // + slack to align the tiles to 1024 bytes
constexpr uint32_t kCols = 64;
}  // namespace outtc

__global__ void __launch_bounds__(outtc::kThreads)
pkda_out_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_qg,
                       const __grid_constant__ CUtensorMap tm_e, const __grid_constant__ CUtensorMap tm_p,
                       const __grid_constant__ CUtensorMap tm_o, const OutTcParams p) {
  using namespace outtc;
  extern __shared__ unsigned char smem_raw[];
  int n, tok0, valid;
  if (!chunk_lookup(p.geo, blockIdx.x, n, tok0, valid)) return;
  const int h = blockIdx.y, H = p.geo.heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t chh = (size_t)blockIdx.x * H + h;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_full = base + oBar, bar_mma = base + oBar + 8, tmem_slot = base + oBar + 16;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tiles + oBar + 16);

  // The tile copies start before the tensor-memory allocation and the CTA-wide barrier: one
  // thread of the second warp sets up the mbarriers and issues them while warp 0 allocates.
  if (warp == 0) tc::tmem_alloc(tmem_slot, kCols);
  if (tid == 32) {
    tc::mbar_init(bar_full, 1);
    tc::mbar_init(bar_mma, 1);
    tc::fence_barrier_init();
    tc::mbar_expect_tx(bar_full, kTxBytes);
    const int hrow = (int)(chh * kD);
    tc::tma_load_2d(base + oH, &tm_h, bar_full, 0, hrow);
    tc::tma_load_2d(base + oH + 16384, &tm_h, bar_full, 64, hrow);
    tc::tma_load_3d(base + oQg, &tm_qg, bar_full, 0, h, tok0);
    tc::tma_load_3d(base + oQg + 8192, &tm_qg, bar_full, 64, h, tok0);
    tc::tma_load_3d(base + oE, &tm_e, bar_full, 0, h, tok0);
    tc::tma_load_3d(base + oE + 8192, &tm_e, bar_full, 64, h, tok0);
    tc::tma_load_3d(base + oP, &tm_p, bar_full, 0, h, tok0);
  }
  // beta of this thread's eight columns of P (the same columns in every row it scales), requested
  // now so that it is back when the tiles are
  const float4 b0 = *reinterpret_cast<const float4*>(p.beta_c + chh * kChunk + 8 * (tid & 7));
  const float4 b1 = *reinterpret_cast<const float4*>(p.beta_c + chh * kChunk + 8 * (tid & 7) + 4);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;

  bool ok = tc::mbar_wait(bar_full, 0);

  // P[tok][j] *= beta[j], in place in the swizzled tile: 16-byte piece jc of row i
  // sits at i*128 + ((jc ^ (i & 7)) << 4).
  if (ok) {
    for (int idx = tid; idx < kChunk * 8; idx += kThreads) {
      const int i = idx >> 3, jc = idx & 7;
      uint4* piece = reinterpret_cast<uint4*>(tiles + oP + i * 128 + ((jc ^ (i & 7)) << 4));
      const float f[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      uint4 x = *piece;
      scale8(x, f);
      *piece = x;
    }
  }
  tc::fence_proxy_async();
  __syncthreads();

  if (tid == 0 && ok) {
    tc::tc_fence_after();
    constexpr uint32_t idesc = tc::idesc_bf16(128, 64, /*a_mn_major=*/true, /*b_mn_major=*/false);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {  // product 1: K = 128 state rows
      const uint64_t a = tc::desc_mnmajor(base + oH + kk * 2048, 16384);
      const uint64_t b = tc::desc_kmajor(base + oQg + (kk >> 2) * 8192 + (kk & 3) * 32);
      tc::umma_bf16(tmem, a, b, idesc, kk > 0);
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {  // product 2: K = 64 tokens j
      const uint64_t a = tc::desc_mnmajor(base + oE + kk * 2048, 8192);
      const uint64_t b = tc::desc_kmajor(base + oP + kk * 32);
      tc::umma_bf16(tmem, a, b, idesc, 1);
    }
    tc::umma_commit(bar_mma);
  }
  if (ok) ok = tc::mbar_wait(bar_mma, 0);
  tc::tc_fence_after();

  // Full chunks leave through a swizzled shared-memory tile (the dead h tile) and two TMA stores;
  // ragged chunks store their valid tokens directly.
  const bool by_tma = valid == kChunk;
  if (ok) {
    const int v = 32 * warp + lane;  // this thread's accumulator row = value channel
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float acc[32];
      tc::tmem_ld32(tmem + ((uint32_t)(32 * warp) << 16) + 32 * half, acc);
      tc::tmem_ld_wait();
      if (by_tma) {
#pragma unroll
        for (int t = 0; t < 32; ++t)
          *reinterpret_cast<bf16*>(tiles + oH + sw128_offset(32 * half + t, v, 8192)) = __float2bfloat16(acc[t]);
      } else {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          const int tok = 32 * half + t;
          if (tok < valid) p.o[((size_t)(tok0 + tok) * H + h) * kD + v] = __float2bfloat16(acc[t]);
        }
      }
    }
  } else if (tid == 0) {
    atomicExch(p.status, 1);
  }
  if (by_tma) {  // uniform over the CTA
    tc::fence_proxy_async();
    __syncthreads();
    if (tid == 0 && ok) {
      tc::tma_store_3d(&tm_o, base + oH, 0, h, tok0);
      tc::tma_store_3d(&tm_o, base + oH + 8192, 64, h, tok0);
      tc::bulk_commit();
      tc::bulk_wait_read();  // the tile must stay in place until the copies have read it
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, kCols);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

static bool encode_map(CUtensorMap* map, CUtensorMapDataType type, CUtensorMapSwizzle swizzle, const void* base,
                       int rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bdim[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides[i - 1];
  }
  return fn(map, type, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_bf16_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                     const uint32_t* box, bool swizzle128) {
  return encode_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, base, rank, dims, strides, box);
}

bool encode_f32_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                    const uint32_t* box) {
  return encode_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, CU_TENSOR_MAP_SWIZZLE_NONE, base, rank, dims, strides, box);
}

int launch_out_fwd_tc(const Geo& geo, int total_tokens, const bf16* qg, const bf16* h, const bf16* Aqk,
                      const bf16* v_new, const float* beta_c, bf16* o, int* status, cudaStream_t st) {
  const uint64_t H = geo.heads, chunks = geo.total_chunks, tok = total_tokens;
  CUtensorMap tm_h, tm_qg, tm_e, tm_p, tm_o;
  {
    const uint64_t dims[2] = {kD, chunks * H * kD}, str[1] = {kD * 2};
    const uint32_t box[2] = {64, 128};
    if (!encode_bf16_map(&tm_h, h, 2, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {kD, H, tok}, str[2] = {kD * 2, H * kD * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_qg, qg, 3, dims, str, box)) return PKDA_ERR_LAUNCH;
    if (!encode_bf16_map(&tm_e, v_new, 3, dims, str, box)) return PKDA_ERR_LAUNCH;
    if (!encode_bf16_map(&tm_o, o, 3, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  {
    const uint64_t dims[3] = {kChunk, H, tok}, str[2] = {kChunk * 2, H * kChunk * 2};
    const uint32_t box[3] = {64, 1, 64};
    if (!encode_bf16_map(&tm_p, Aqk, 3, dims, str, box)) return PKDA_ERR_LAUNCH;
  }
  OutTcParams op;
  op.geo = geo; op.beta_c = beta_c; op.o = o; op.status = status;
  if (!ensure_dynamic_smem(pkda_out_fwd_tc_kernel, outtc::kSmem))
    return PKDA_ERR_LAUNCH;
  begin_stage(kStageOutFwd, st);
  pkda_out_fwd_tc_kernel<<<dim3(geo.total_chunks, geo.heads), outtc::kThreads, outtc::kSmem, st>>>(tm_h, tm_qg, tm_e,
                                                                                                   tm_p, tm_o, op);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
