// Fused Q|K|V short convolution of the PKDA layer, forward and backward:
//   y[t][c] = sum_j w[c][j] * x[t - (taps-1) + j][c]      (causal, depthwise, <= 4 taps)
//   s = silu(y)
//   out = s * rsqrt(sum over the head of s^2 + eps)        for c < norm_channels (Q and K)
//   out = s                                                otherwise (V)
// written as three slabs q, k, v.  Pure streaming work.  A CTA stages a tile of
// tokens x 256 channels (plus the halo rows the filter reaches into) in shared
// memory with 16-byte cp.async copies -- all of a CTA's loads are in flight at
// once and several CTAs share an SM -- and then every thread walks a few tokens of
// 4 adjacent channels with the filter window in registers.  The per-head sums are
// shuffle reductions inside a warp (a head is at most 32 lanes).  The backward
// recomputes the pre-activation instead of saving it: phase A turns the tile of
// output gradients into the gradient of the pre-activation (fp32, in shared
// memory), phase B forms dx (a 4-tap correlation of that tile, no atomics) and the
// weight gradient, which is reduced in a fixed order (registers -> across the
// CTA's token groups -> one partial per CTA -> a small second kernel).
#include "pkda_common.cuh"
#include "pkda_launch.h"

namespace pkda {

namespace conv {
constexpr int kVec = 4;          // channels per thread
constexpr int kThreads = 256;
constexpr int kTileCh = 256;     // channels per CTA = 64 lanes
constexpr int kLanes = kTileCh / kVec;
constexpr int kGroups = kThreads / kLanes;  // token groups per CTA (4)
constexpr int kMaxTaps = 4;
constexpr int kHalo = kMaxTaps - 1;
constexpr int kFwdTokens = 64;   // tokens per forward CTA (16 per group)
constexpr int kBwdTokens = 32;   // tokens per backward tile (8 per group)
constexpr int kBwdTiles = 8;     // tiles one backward CTA walks (one weight-gradient partial per CTA)
constexpr int kBwdDyRows = kBwdTokens + kHalo;             // 35
constexpr int kBwdDyPerGroup = (kBwdDyRows + kGroups - 1) / kGroups;  // 9
template <typename T> constexpr int fwd_smem() { return (kFwdTokens + kHalo) * kTileCh * (int)sizeof(T); }
template <typename T> constexpr int bwd_smem() {
  return (kBwdTokens + 2 * kHalo) * kTileCh * (int)sizeof(T) + kBwdDyRows * kTileCh * (int)sizeof(T) +
         kBwdDyRows * kTileCh * 4;
}
}  // namespace conv

struct ConvParams {
  int batch, seq_len, channels, slab, taps, head_lanes, norm_channels, spans_per_row;
  float eps;
  const void* x;
  const float* w;
  void *q, *k, *v;
  const void *dq, *dk, *dv;
  void* dx;
  float* part;  // [gridDim.y][channels][taps]
};

template <typename T> struct Vec4;
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&f)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  static __device__ __forceinline__ void store(bf16* p, const float (&f)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
  }
  // 0.5 * (1 + tanh(y / 2)) with the single-instruction tanh: relative error 2^-11,
  // below the bf16 rounding of the result.
  static __device__ __forceinline__ float sigmoid(float y) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * y));
    return fmaf(0.5f, t, 0.5f);
  }
};
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  static __device__ __forceinline__ float sigmoid(float y) { return 1.f / (1.f + expf(-y)); }
};

// Sum over the kHeadLanes adjacent lanes of one head (a power of two <= 32; a
// template parameter so that the token loops around it unroll without control flow).
template <int kHeadLanes>
__device__ __forceinline__ float head_sum(float v) {
#pragma unroll
  for (int o = kHeadLanes >> 1; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Stages rows [t_first, t_first + rows) x 256 channels of a [seq_len][row_channels]
// matrix into shared memory; rows outside [0, seq_len) and channels past the end
// read as zero.
template <typename T>
__device__ __forceinline__ void stage_rows(T* s, const T* g, int t_first, int rows, int seq_len, int c_first,
                                           int row_channels) {
  constexpr int kPiece = 16 / (int)sizeof(T), kPerRow = conv::kTileCh / kPiece;
  constexpr int kRowStep = conv::kThreads / kPerRow;  // a thread keeps its column piece, rows advance
  const int pc = (threadIdx.x % kPerRow) * kPiece, c = c_first + pc;
  const bool col_ok = c < row_channels;
  const T* gcol = g + (col_ok ? c : 0);
  for (int r = threadIdx.x / kPerRow; r < rows; r += kRowStep) {
    const int t = t_first + r;
    const bool ok = col_ok && t >= 0 && t < seq_len;
    cp_async16(s + r * conv::kTileCh + pc, gcol + (ok ? (size_t)t * row_channels : 0), ok);
  }
}

// The same for the output gradients, which live in three slabs [seq_len][slab]:
// channel c of the concatenated axis is channel c % slab of slab c / slab (a
// 16-byte piece never straddles slabs because the slab width is a multiple of 8).
template <typename T>
__device__ __forceinline__ void stage_grad_rows(T* s, const T* g0, const T* g1, const T* g2, int t_first, int rows,
                                                int seq_len, int c_first, int channels, int slab) {
  constexpr int kPiece = 16 / (int)sizeof(T), kPerRow = conv::kTileCh / kPiece;
  constexpr int kRowStep = conv::kThreads / kPerRow;
  const int pc = (threadIdx.x % kPerRow) * kPiece, c = c_first + pc;
  const bool col_ok = c < channels;
  const int id = col_ok ? c / slab : 0;
  const T* gcol = (id == 0 ? g0 : id == 1 ? g1 : g2) + (col_ok ? c - id * slab : 0);
  for (int r = threadIdx.x / kPerRow; r < rows; r += kRowStep) {
    const int t = t_first + r;
    const bool ok = col_ok && t >= 0 && t < seq_len;
    cp_async16(s + r * conv::kTileCh + pc, gcol + (ok ? (size_t)t * slab : 0), ok);
  }
}

__device__ __forceinline__ void load_taps(const ConvParams& p, int c, bool active, float (&w)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int jj = j - (conv::kMaxTaps - p.taps);  // tap j of the filter padded to four taps
      w[i][j] = (active && jj >= 0) ? p.w[(size_t)(c + i) * p.taps + jj] : 0.f;
    }
}

template <typename T, int kHeadLanes>
__global__ void __launch_bounds__(conv::kThreads)
pkda_qkv_conv_fwd_kernel(const ConvParams p) {
  using namespace conv;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sx = reinterpret_cast<T*>(smem_raw);
  const int b = blockIdx.y / p.spans_per_row;
  const int t0 = (blockIdx.y - b * p.spans_per_row) * kFwdTokens;
  const int cb = blockIdx.x * kTileCh;
  const int lane = threadIdx.x % kLanes, grp = threadIdx.x / kLanes;
  const int c = cb + kVec * lane;
  const bool active = c < p.channels;
  stage_rows(sx, static_cast<const T*>(p.x) + (size_t)b * p.seq_len * p.channels, t0 - kHalo, kFwdTokens + kHalo,
             p.seq_len, cb, p.channels);
  cp_async_commit();
  float w[4][4];
  load_taps(p, c, active, w);
  const int cc = active ? c : 0;
  const int slab_id = cc / p.slab, cs = cc - slab_id * p.slab;
  const bool normed = active && c < p.norm_channels;
  T* out = static_cast<T*>(slab_id == 0 ? p.q : slab_id == 1 ? p.k : p.v) + (size_t)b * p.seq_len * p.slab + cs;
  cp_async_wait<0>();
  __syncthreads();
  constexpr int kPer = kFwdTokens / kGroups;  // 16 tokens per thread
  const T* col = sx + kVec * lane;
  float win[3][4];
#pragma unroll
  for (int j = 0; j < 3; ++j) Vec4<T>::load(col + (kPer * grp + j) * kTileCh, win[j]);
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    const int t = t0 + kPer * grp + u;
    float xa[4], s[4], ss = 0.f;
    Vec4<T>::load(col + (kPer * grp + kHalo + u) * kTileCh, xa);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float y = w[i][0] * win[0][i] + w[i][1] * win[1][i] + w[i][2] * win[2][i] + w[i][3] * xa[i];
      s[i] = y * Vec4<T>::sigmoid(y);
      ss += s[i] * s[i];
      win[0][i] = win[1][i]; win[1][i] = win[2][i]; win[2][i] = xa[i];
    }
    ss = head_sum<kHeadLanes>(ss);
    const float r = normed ? rsqrtf(ss + p.eps) : 1.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] *= r;
    if (active && t < p.seq_len) Vec4<T>::store(out + (size_t)t * p.slab, s);
  }
}

template <typename T, int kHeadLanes>
__global__ void __launch_bounds__(conv::kThreads)
pkda_qkv_conv_bwd_kernel(const ConvParams p) {
  using namespace conv;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sx = reinterpret_cast<T*>(smem_raw);                      // tokens t0-3 .. t0+34
  T* sd = sx + (kBwdTokens + 2 * kHalo) * kTileCh;             // tokens t0 .. t0+34
  float* sdy = reinterpret_cast<float*>(sd + kBwdDyRows * kTileCh);  // tokens t0 .. t0+34; later the dw exchange
  const int b = blockIdx.y / p.spans_per_row;
  const int span0 = (blockIdx.y - b * p.spans_per_row) * (kBwdTokens * kBwdTiles);
  const int cb = blockIdx.x * kTileCh;
  const int lane = threadIdx.x % kLanes, grp = threadIdx.x / kLanes;
  const int c = cb + kVec * lane;
  const bool active = c < p.channels;
  const int cc = active ? c : 0;
  const bool normed = active && c < p.norm_channels;
  float w[4][4], dwacc[4][4];
  load_taps(p, c, active, w);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dwacc[i][j] = 0.f;
  const T* xrow = static_cast<const T*>(p.x) + (size_t)b * p.seq_len * p.channels;
  const size_t doff = (size_t)b * p.seq_len * p.slab;
  const T *dq = static_cast<const T*>(p.dq) + doff, *dk = static_cast<const T*>(p.dk) + doff,
          *dv = static_cast<const T*>(p.dv) + doff;
  T* dxrow = static_cast<T*>(p.dx) + (size_t)b * p.seq_len * p.channels + cc;
  for (int tile = 0; tile < kBwdTiles; ++tile) {
    const int t0 = span0 + tile * kBwdTokens;
    if (t0 >= p.seq_len) break;
    stage_rows(sx, xrow, t0 - kHalo, kBwdTokens + 2 * kHalo, p.seq_len, cb, p.channels);
    stage_grad_rows(sd, dq, dk, dv, t0, kBwdDyRows, p.seq_len, cb, p.channels, p.slab);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    // ---- phase A: gradient of the pre-activation for tokens t0 .. t0+34
    {
      const int i0 = kBwdDyPerGroup * grp;
      const T* xc = sx + kVec * lane;
      float win[3][4];
#pragma unroll
      for (int j = 0; j < 3; ++j) Vec4<T>::load(xc + (i0 + j) * kTileCh, win[j]);
#pragma unroll
      for (int u = 0; u < kBwdDyPerGroup; ++u) {
        const int i = i0 + u;  // token t0 + i; its filter window is rows i .. i+3 of sx
        if (i < kBwdDyRows) {
          float xa[4], da[4], y[4], sg[4], s[4], ss = 0.f, sdot = 0.f;
          Vec4<T>::load(xc + (i + kHalo) * kTileCh, xa);
          Vec4<T>::load(sd + i * kTileCh + kVec * lane, da);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            y[e] = w[e][0] * win[0][e] + w[e][1] * win[1][e] + w[e][2] * win[2][e] + w[e][3] * xa[e];
            sg[e] = Vec4<T>::sigmoid(y[e]);
            s[e] = y[e] * sg[e];
            ss += s[e] * s[e];
            sdot += s[e] * da[e];
            win[0][e] = win[1][e]; win[1][e] = win[2][e]; win[2][e] = xa[e];
          }
          ss = head_sum<kHeadLanes>(ss);
          sdot = head_sum<kHeadLanes>(sdot);
          const float r = normed ? rsqrtf(ss + p.eps) : 1.f;
          const float back = normed ? r * r * r * sdot : 0.f;
          float dy[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float ds = r * da[e] - s[e] * back;
            dy[e] = ds * (sg[e] + s[e] * (1.f - sg[e]));  // silu'(y) = sig + y sig (1 - sig)
          }
          *reinterpret_cast<float4*>(sdy + i * kTileCh + kVec * lane) = make_float4(dy[0], dy[1], dy[2], dy[3]);
        }
      }
    }
    __syncthreads();
    // ---- phase B: dx and the weight gradient for the tile's own 32 tokens
    {
      constexpr int kPer = kBwdTokens / kGroups;  // 8
      const int j0 = kPer * grp;
      const T* xc = sx + kVec * lane;
      const float* dc = sdy + kVec * lane;
      float xw[3][4], dw3[3][4];  // x rows j..j+2 (tokens t-3..t-1), dy rows j..j+2 (tokens t..t+2)
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        Vec4<T>::load(xc + (j0 + j) * kTileCh, xw[j]);
        const float4 d4 = *reinterpret_cast<const float4*>(dc + (j0 + j) * kTileCh);
        dw3[j][0] = d4.x; dw3[j][1] = d4.y; dw3[j][2] = d4.z; dw3[j][3] = d4.w;
      }
#pragma unroll
      for (int u = 0; u < kPer; ++u) {
        const int j = j0 + u, t = t0 + j;
        float xa[4], dn[4], dxv[4];
        Vec4<T>::load(xc + (j + kHalo) * kTileCh, xa);  // x[t]
        const float4 d4 = *reinterpret_cast<const float4*>(dc + (j + kHalo) * kTileCh);  // dy[t+3]
        dn[0] = d4.x; dn[1] = d4.y; dn[2] = d4.z; dn[3] = d4.w;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float dyt = dw3[0][e];
          dxv[e] = w[e][3] * dyt + w[e][2] * dw3[1][e] + w[e][1] * dw3[2][e] + w[e][0] * dn[e];
          dwacc[e][0] += dyt * xw[0][e];
          dwacc[e][1] += dyt * xw[1][e];
          dwacc[e][2] += dyt * xw[2][e];
          dwacc[e][3] += dyt * xa[e];
          xw[0][e] = xw[1][e]; xw[1][e] = xw[2][e]; xw[2][e] = xa[e];
          dw3[0][e] = dw3[1][e]; dw3[1][e] = dw3[2][e]; dw3[2][e] = dn[e];
        }
        if (active && t < p.seq_len) Vec4<T>::store(dxrow + (size_t)t * p.channels, dxv);
      }
    }
    __syncthreads();
  }
  // ---- weight gradient: the four token groups in a fixed order, one partial per CTA
  float* sPart = sdy;  // [kGroups][kLanes][16]
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) sPart[(grp * kLanes + lane) * 16 + 4 * i + j] = dwacc[i][j];
  __syncthreads();
  if (grp == 0 && active) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      for (int j = 0; j < p.taps; ++j) {
        const int e = 4 * i + j + (kMaxTaps - p.taps);
        float a = 0.f;
#pragma unroll
        for (int g = 0; g < kGroups; ++g) a += sPart[(g * kLanes + lane) * 16 + e];
        p.part[((size_t)blockIdx.y * p.channels + c + i) * p.taps + j] = a;
      }
  }
}

__global__ void pkda_qkv_conv_dw_kernel(const float* part, float* dw, int n, int groups) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  float a = 0.f;
  for (int g = 0; g < groups; ++g) a += part[(size_t)g * n + idx];
  dw[idx] = a;
}

// ------------------------------------------------------------------ host side
static int conv_check(const pkda_qkv_conv_args& a, ConvParams& p) {
  if (a.batch < 0 || a.seq_len < 0 || a.channels <= 0 || a.channels % 3) return PKDA_ERR_SHAPE;
  if (a.taps < 1 || a.taps > conv::kMaxTaps) return PKDA_ERR_SHAPE;
  const int slab = a.channels / 3, hd = a.head_dim;
  if (hd < 8 || hd > 128 || (hd & (hd - 1)) || slab % hd) return PKDA_ERR_SHAPE;
  if (a.norm_channels < 0 || a.norm_channels > a.channels || a.norm_channels % hd) return PKDA_ERR_SHAPE;
  if (a.dtype != PKDA_BF16 && a.dtype != PKDA_F32) return PKDA_ERR_DTYPE;
  p.batch = a.batch; p.seq_len = a.seq_len; p.channels = a.channels; p.slab = slab; p.taps = a.taps;
  p.head_lanes = hd / conv::kVec; p.norm_channels = a.norm_channels; p.eps = a.eps;
  p.spans_per_row = 0;
  p.x = a.x; p.w = a.weight; p.q = a.q; p.k = a.k; p.v = a.v;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv; p.dx = a.dx; p.part = nullptr;
  return PKDA_OK;
}

// Token spans (CTA rows of the grid) for a span of `tokens` tokens per CTA.
static dim3 conv_grid(ConvParams& p, int tokens) {
  p.spans_per_row = (p.seq_len + tokens - 1) / tokens;
  return dim3((p.channels + conv::kTileCh - 1) / conv::kTileCh, (unsigned)(p.batch * p.spans_per_row));
}

static bool aligned16(const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; }

template <typename K> static bool allow_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
}

template <typename T, int kHeadLanes>
static int launch_conv_fwd(const ConvParams& p, dim3 grid, cudaStream_t st) {
  if (!allow_smem(pkda_qkv_conv_fwd_kernel<T, kHeadLanes>, conv::fwd_smem<T>())) return PKDA_ERR_LAUNCH;
  begin_stage(kStageConvFwd, st);
  pkda_qkv_conv_fwd_kernel<T, kHeadLanes><<<grid, conv::kThreads, conv::fwd_smem<T>(), st>>>(p);
  end_stage(st);
  return PKDA_OK;
}

template <typename T, int kHeadLanes>
static int launch_conv_bwd(const ConvParams& p, dim3 grid, cudaStream_t st) {
  if (!allow_smem(pkda_qkv_conv_bwd_kernel<T, kHeadLanes>, conv::bwd_smem<T>())) return PKDA_ERR_LAUNCH;
  begin_stage(kStageConvBwd, st);
  pkda_qkv_conv_bwd_kernel<T, kHeadLanes><<<grid, conv::kThreads, conv::bwd_smem<T>(), st>>>(p);
  end_stage(st);
  return PKDA_OK;
}

// Picks the instantiation for the activation type and the lanes per head.
#define PKDA_CONV_DISPATCH(FN, T)                                   \
  switch (p.head_lanes) {                                           \
    case 2: rc = FN<T, 2>(p, grid, st); break;                      \
    case 4: rc = FN<T, 4>(p, grid, st); break;                      \
    case 8: rc = FN<T, 8>(p, grid, st); break;                      \
    case 16: rc = FN<T, 16>(p, grid, st); break;                    \
    default: rc = FN<T, 32>(p, grid, st); break;                    \
  }

int qkv_conv_fwd(const pkda_qkv_conv_args* a, cudaStream_t st) {
  ConvParams p;
  if (int rc = conv_check(*a, p)) return rc;
  if (a->batch == 0 || a->seq_len == 0) return PKDA_OK;
  if (!a->x || !a->weight || !a->q || !a->k || !a->v) return PKDA_ERR_NULL;
  if (!aligned16(a->x) || !aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v)) return PKDA_ERR_ALIGN;
  const dim3 grid = conv_grid(p, conv::kFwdTokens);
  int rc = PKDA_OK;
  if (a->dtype == PKDA_BF16) { PKDA_CONV_DISPATCH(launch_conv_fwd, bf16) } else { PKDA_CONV_DISPATCH(launch_conv_fwd, float) }
  if (rc != PKDA_OK) return rc;
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

size_t qkv_conv_bwd_workspace(const pkda_qkv_conv_args& a) {
  ConvParams p;
  if (conv_check(a, p) != PKDA_OK) return 0;
  const dim3 grid = conv_grid(p, conv::kBwdTokens * conv::kBwdTiles);
  return align_up((size_t)grid.y * a.channels * a.taps * sizeof(float));
}

int qkv_conv_bwd(const pkda_qkv_conv_args* a, cudaStream_t st) {
  ConvParams p;
  if (int rc = conv_check(*a, p)) return rc;
  if (!a->dweight) return PKDA_ERR_NULL;
  const int n = a->channels * a->taps;
  if (a->batch == 0 || a->seq_len == 0) {
    return cudaMemsetAsync(a->dweight, 0, (size_t)n * sizeof(float), st) == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
  }
  if (!a->x || !a->weight || !a->dq || !a->dk || !a->dv || !a->dx) return PKDA_ERR_NULL;
  if (!aligned16(a->x) || !aligned16(a->dq) || !aligned16(a->dk) || !aligned16(a->dv) || !aligned16(a->dx))
    return PKDA_ERR_ALIGN;
  if (!a->workspace || a->workspace_bytes < qkv_conv_bwd_workspace(*a)) return PKDA_ERR_WORKSPACE;
  p.part = static_cast<float*>(a->workspace);
  const dim3 grid = conv_grid(p, conv::kBwdTokens * conv::kBwdTiles);
  int rc = PKDA_OK;
  if (a->dtype == PKDA_BF16) { PKDA_CONV_DISPATCH(launch_conv_bwd, bf16) } else { PKDA_CONV_DISPATCH(launch_conv_bwd, float) }
  if (rc != PKDA_OK) return rc;
  begin_stage(kStageConvDw, st);
  pkda_qkv_conv_dw_kernel<<<(n + 255) / 256, 256, 0, st>>>(p.part, a->dweight, n, (int)grid.y);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
