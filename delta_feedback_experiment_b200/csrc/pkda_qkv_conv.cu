// Fused Q|K|V short convolution of the PKDA layer, forward and backward:
//   y[t][c] = sum_j w[c][j] * x[t - (taps-1) + j][c]      (causal, depthwise, <= 4 taps)
//   s = silu(y)
//   out = s * rsqrt(sum over the head of s^2 + eps)        for c < norm_channels (Q and K)
//   out = s                                                otherwise (V)
// written as three slabs q, k, v.  Pure streaming work.  A CTA owns 256 channels
// and a span of token tiles; each tile (plus the halo rows the filter reaches into)
// is staged in shared memory with 16-byte cp.async copies, double buffered, so the
// next tile lands while the current one is computed.  A thread walks a few tokens of
// 4 adjacent channels with the filter window in registers; the arithmetic is
// written on pairs of channels with the packed fp32x2 instructions of sm_100
// (fma.rn.f32x2 and friends: one issue slot for two lanes of work), because these
// kernels are bound by instruction issue, not by DRAM.  The per-head sums are
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
constexpr int kFwdTokens = 64;   // tokens per forward tile (16 per group)
constexpr int kFwdTiles = 4;     // tiles one forward CTA walks
constexpr int kBwdTokens = 32;   // tokens per backward tile (8 per group)
constexpr int kBwdTiles = 8;     // tiles one backward CTA walks (one weight-gradient partial per CTA)
constexpr int kBwdDyRows = kBwdTokens + kHalo;             // 35
constexpr int kBwdDyPerGroup = (kBwdDyRows + kGroups - 1) / kGroups;  // 9
template <typename T> __host__ __device__ constexpr int fwd_stage() { return (kFwdTokens + kHalo) * kTileCh * (int)sizeof(T); }
template <typename T> __host__ __device__ constexpr int fwd_smem() { return 2 * fwd_stage<T>(); }
template <typename T> __host__ __device__ constexpr int bwd_stage() {
  return ((kBwdTokens + 2 * kHalo) + kBwdDyRows) * kTileCh * (int)sizeof(T);
}
template <typename T> __host__ __device__ constexpr int bwd_smem() { return 2 * bwd_stage<T>() + kBwdDyRows * kTileCh * 4; }
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

// Packed fp32x2 arithmetic (two channels per instruction).
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// Four adjacent channels as two pairs.
template <typename T> struct Vec4;
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float2 (&f)[2]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    f[0] = unpack_bf16(u.x);
    f[1] = unpack_bf16(u.y);
  }
  static __device__ __forceinline__ void store(bf16* p, const float2 (&f)[2]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(f[0].x, f[0].y), pack_bf16(f[1].x, f[1].y));
  }
  // 0.5 * (1 + tanh(y / 2)) with the single-instruction tanh: relative error 2^-11,
  // below the bf16 rounding of the result.
  static __device__ __forceinline__ float2 sigmoid(float2 y) {
    const float2 h = mul2(y, f2(0.5f, 0.5f));
    float2 t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(h.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(h.y));
    return fma2(t, f2(0.5f, 0.5f), f2(0.5f, 0.5f));
  }
};
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float2 (&f)[2]) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = f2(u.x, u.y);
    f[1] = f2(u.z, u.w);
  }
  static __device__ __forceinline__ void store(float* p, const float2 (&f)[2]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0].x, f[0].y, f[1].x, f[1].y);
  }
  static __device__ __forceinline__ float2 sigmoid(float2 y) {
    return f2(1.f / (1.f + expf(-y.x)), 1.f / (1.f + expf(-y.y)));
  }
};

// Sum over the kHeadLanes adjacent lanes of one head (a power of two <= 32; a
// template parameter so that the token loops around it unroll without control flow).
template <int kHeadLanes>
__device__ __forceinline__ float head_sum(float v) {
#pragma unroll
  for (int o = kHeadLanes >> 1; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Two sums at once: the two halves of the head first trade one value each, so the
// butterfly runs on a single register (log2(L) + 1 shuffles instead of 2 log2(L)).
template <int kHeadLanes>
__device__ __forceinline__ void head_sum2(float& a, float& b, int lane) {
  if (kHeadLanes == 1) return;
  constexpr int kHalf = kHeadLanes / 2;
  const bool upper = lane & kHalf;
  float keep = upper ? b : a;
  const float send = upper ? a : b;
  keep += __shfl_xor_sync(0xffffffffu, send, kHalf);
#pragma unroll
  for (int o = kHalf >> 1; o >= 1; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
  const float other = __shfl_xor_sync(0xffffffffu, keep, kHalf);
  a = upper ? other : keep;
  b = upper ? keep : other;
}

// Stages rows [t_first, t_first + rows) x 256 channels of a [seq_len][row_channels]
// matrix into shared memory; rows outside [0, seq_len) and channels past the end
// read as zero.
template <typename T>
__device__ __forceinline__ void stage_col(T* scol, const T* gcol, bool col_ok, int t_first, int rows, int seq_len,
                                          size_t row_stride) {
  constexpr int kPiece = 16 / (int)sizeof(T), kPerRow = conv::kTileCh / kPiece;
  constexpr int kRowStep = conv::kThreads / kPerRow;  // a thread keeps its column piece, rows advance
  const int r0 = threadIdx.x / kPerRow;
  if (col_ok && t_first >= 0 && t_first + rows <= seq_len) {  // whole tile inside the row: no per-copy tests
    const T* g = gcol + (size_t)(t_first + r0) * row_stride;
    T* d = scol + r0 * conv::kTileCh;
    for (int r = r0; r < rows; r += kRowStep) {
      cp_async16(d, g, true);
      g += kRowStep * row_stride;
      d += kRowStep * conv::kTileCh;
    }
  } else {
    for (int r = r0; r < rows; r += kRowStep) {
      const int t = t_first + r;
      const bool ok = col_ok && t >= 0 && t < seq_len;
      cp_async16(scol + r * conv::kTileCh, gcol + (ok ? (size_t)t * row_stride : 0), ok);
    }
  }
}

template <typename T>
__device__ __forceinline__ void stage_rows(T* s, const T* g, int t_first, int rows, int seq_len, int c_first,
                                           int row_channels) {
  constexpr int kPiece = 16 / (int)sizeof(T), kPerRow = conv::kTileCh / kPiece;
  const int pc = (threadIdx.x % kPerRow) * kPiece, c = c_first + pc;
  const bool col_ok = c < row_channels;
  stage_col(s + pc, g + (col_ok ? c : 0), col_ok, t_first, rows, seq_len, (size_t)row_channels);
}

// The same for the output gradients, which live in three slabs [seq_len][slab]:
// channel c of the concatenated axis is channel c % slab of slab c / slab (a
// 16-byte piece never straddles slabs because the slab width is a multiple of 8).
template <typename T>
__device__ __forceinline__ void stage_grad_rows(T* s, const T* g0, const T* g1, const T* g2, int t_first, int rows,
                                                int seq_len, int c_first, int channels, int slab) {
  constexpr int kPiece = 16 / (int)sizeof(T), kPerRow = conv::kTileCh / kPiece;
  const int pc = (threadIdx.x % kPerRow) * kPiece, c = c_first + pc;
  const bool col_ok = c < channels;
  const int id = col_ok ? c / slab : 0;
  const T* gcol = (id == 0 ? g0 : id == 1 ? g1 : g2) + (col_ok ? c - id * slab : 0);
  stage_col(s + pc, gcol, col_ok, t_first, rows, seq_len, (size_t)slab);
}

// Filter taps of the thread's four channels as pairs: w[pair][tap], padded to four taps.
__device__ __forceinline__ void load_taps(const ConvParams& p, int c, bool active, float2 (&w)[2][4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int jj = j - (conv::kMaxTaps - p.taps);  // tap j of the filter padded to four taps
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (active && jj >= 0) ? p.w[(size_t)(c + i) * p.taps + jj] : 0.f;
    w[0][j] = f2(v[0], v[1]);
    w[1][j] = f2(v[2], v[3]);
  }
}

// Pre-activation of one token for the thread's two channel pairs.
__device__ __forceinline__ void conv4(float2 (&y)[2], const float2 (&w)[2][4], const float2 (&w0)[2],
                                      const float2 (&w1)[2], const float2 (&w2)[2], const float2 (&x)[2]) {
#pragma unroll
  for (int pr = 0; pr < 2; ++pr) {
    float2 a = mul2(w[pr][0], w0[pr]);
    a = fma2(w[pr][1], w1[pr], a);
    a = fma2(w[pr][2], w2[pr], a);
    y[pr] = fma2(w[pr][3], x[pr], a);
  }
}

// Forward for one group of 16 consecutive tokens of the thread's four channels:
// two halves of 8 tokens whose 11 input rows sit in registers, addressed statically.
// kGuard: the group reaches past the end of the row (stores are tested).
template <typename T, int kHeadLanes, bool kGuard>
__device__ __forceinline__ void conv_fwd_tokens(const T* col, T* orow, size_t ostride, const float2 (&w)[2][4],
                                                bool active, bool normed, float eps, int nvalid) {
  using namespace conv;
  constexpr int kHalf = kFwdTokens / kGroups / 2;
#pragma unroll
  for (int hseg = 0; hseg < 2; ++hseg) {
    float2 xr[kHalf + kHalo][2];
#pragma unroll
    for (int j = 0; j < kHalf + kHalo; ++j) Vec4<T>::load(col + (kHalf * hseg + j) * kTileCh, xr[j]);
#pragma unroll
    for (int u = 0; u < kHalf; ++u) {
      float2 y[2], s[2];
      conv4(y, w, xr[u], xr[u + 1], xr[u + 2], xr[u + 3]);
      s[0] = mul2(y[0], Vec4<T>::sigmoid(y[0]));
      s[1] = mul2(y[1], Vec4<T>::sigmoid(y[1]));
      const float2 sq = fma2(s[1], s[1], mul2(s[0], s[0]));
      const float ss = head_sum<kHeadLanes>(sq.x + sq.y);
      const float r = normed ? rsqrtf(ss + eps) : 1.f;
      s[0] = mul2(s[0], f2(r, r));
      s[1] = mul2(s[1], f2(r, r));
      const int tok = kHalf * hseg + u;
      if (active && (!kGuard || tok < nvalid)) Vec4<T>::store(orow + (size_t)tok * ostride, s);
    }
  }
}

// Backward phase A for one group: the gradient of the pre-activation of kTokens
// consecutive tokens (fp32, to shared memory) and the weight gradient of the first
// kOwn of them (the rest are look-ahead rows owned by the next tile).
template <typename T, int kHeadLanes, int kTokens, int kOwn>
__device__ __forceinline__ void conv_bwd_phase_a(const T* xc, const T* dc, float* yc, const float2 (&w)[2][4],
                                                 float2 (&dwacc)[2][4], bool normed, float eps, int lane32) {
  using namespace conv;
  float2 xr[kTokens + kHalo][2];
#pragma unroll
  for (int j = 0; j < kTokens + kHalo; ++j) Vec4<T>::load(xc + j * kTileCh, xr[j]);
#pragma unroll
  for (int u = 0; u < kTokens; ++u) {
    float2 da[2], y[2], sg[2], s[2];
    Vec4<T>::load(dc + u * kTileCh, da);
    conv4(y, w, xr[u], xr[u + 1], xr[u + 2], xr[u + 3]);
    sg[0] = Vec4<T>::sigmoid(y[0]);
    sg[1] = Vec4<T>::sigmoid(y[1]);
    s[0] = mul2(y[0], sg[0]);
    s[1] = mul2(y[1], sg[1]);
    const float2 sq = fma2(s[1], s[1], mul2(s[0], s[0]));
    const float2 sdv = fma2(s[1], da[1], mul2(s[0], da[0]));
    float ss = sq.x + sq.y, sdot = sdv.x + sdv.y;
    head_sum2<kHeadLanes>(ss, sdot, lane32);
    const float r = normed ? rsqrtf(ss + eps) : 1.f;
    const float back = normed ? -r * r * r * sdot : 0.f;
    float2 dy[2];
#pragma unroll
    for (int pr = 0; pr < 2; ++pr) {
      const float2 ds = fma2(s[pr], f2(back, back), mul2(da[pr], f2(r, r)));  // r d - s r^3 <s, d>
      const float2 om = fma2(sg[pr], f2(-1.f, -1.f), f2(1.f, 1.f));          // 1 - sig
      dy[pr] = mul2(ds, fma2(s[pr], om, sg[pr]));                             // silu' = sig + y sig (1 - sig)
    }
    *reinterpret_cast<float4*>(yc + u * kTileCh) = make_float4(dy[0].x, dy[0].y, dy[1].x, dy[1].y);
    if (u < kOwn) {
#pragma unroll
      for (int pr = 0; pr < 2; ++pr)
#pragma unroll
        for (int j = 0; j < 4; ++j) dwacc[pr][j] = fma2(dy[pr], xr[u + j][pr], dwacc[pr][j]);
    }
  }
}

// Backward phase B for one group of 8 own tokens: dx[t] = sum_j w[j] dy[t + 3 - j].
template <typename T, bool kGuard>
__device__ __forceinline__ void conv_bwd_phase_b(const float* dc, T* drow, size_t dstride, const float2 (&w)[2][4],
                                                 bool active, int nvalid) {
  using namespace conv;
  constexpr int kPer = kBwdTokens / kGroups;
  float2 dr[kPer + kHalo][2];
#pragma unroll
  for (int j = 0; j < kPer + kHalo; ++j) {
    const float4 d4 = *reinterpret_cast<const float4*>(dc + j * kTileCh);
    dr[j][0] = f2(d4.x, d4.y);
    dr[j][1] = f2(d4.z, d4.w);
  }
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    float2 dxv[2];
#pragma unroll
    for (int pr = 0; pr < 2; ++pr) {
      float2 a = mul2(w[pr][3], dr[u][pr]);
      a = fma2(w[pr][2], dr[u + 1][pr], a);
      a = fma2(w[pr][1], dr[u + 2][pr], a);
      dxv[pr] = fma2(w[pr][0], dr[u + 3][pr], a);
    }
    if (active && (!kGuard || u < nvalid)) Vec4<T>::store(drow + (size_t)u * dstride, dxv);
  }
}

template <typename T, int kHeadLanes>
__global__ void __launch_bounds__(conv::kThreads, 3)
pkda_qkv_conv_fwd_kernel(const ConvParams p) {
  using namespace conv;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* stage[2] = {reinterpret_cast<T*>(smem_raw), reinterpret_cast<T*>(smem_raw + fwd_stage<T>())};
  const int b = blockIdx.y / p.spans_per_row;
  const int span0 = (blockIdx.y - b * p.spans_per_row) * (kFwdTokens * kFwdTiles);
  const int cb = blockIdx.x * kTileCh;
  const int lane = threadIdx.x % kLanes, grp = threadIdx.x / kLanes;
  const int c = cb + kVec * lane;
  const bool active = c < p.channels;
  const T* xrow = static_cast<const T*>(p.x) + (size_t)b * p.seq_len * p.channels;
  const int ntiles = min(kFwdTiles, (p.seq_len - span0 + kFwdTokens - 1) / kFwdTokens);
  stage_rows(stage[0], xrow, span0 - kHalo, kFwdTokens + kHalo, p.seq_len, cb, p.channels);
  cp_async_commit();
  float2 w[2][4];
  load_taps(p, c, active, w);
  const int cc = active ? c : 0;
  const int slab_id = cc / p.slab, cs = cc - slab_id * p.slab;
  const bool normed = active && c < p.norm_channels;
  T* out = static_cast<T*>(slab_id == 0 ? p.q : slab_id == 1 ? p.k : p.v) + (size_t)b * p.seq_len * p.slab + cs;
  constexpr int kPer = kFwdTokens / kGroups;  // 16 tokens per thread and tile
  for (int tile = 0; tile < ntiles; ++tile) {
    const int t0 = span0 + tile * kFwdTokens;
    if (tile + 1 < ntiles) {
      stage_rows(stage[(tile + 1) & 1], xrow, t0 + kFwdTokens - kHalo, kFwdTokens + kHalo, p.seq_len, cb, p.channels);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const T* col = stage[tile & 1] + kVec * lane + (kPer * grp) * kTileCh;
    T* orow = out + (size_t)(t0 + kPer * grp) * p.slab;
    const int nvalid = p.seq_len - (t0 + kPer * grp);  // tokens of this group inside the row
    // (one code path with tested stores: a second, untested copy costs a CTA per SM in registers)
    conv_fwd_tokens<T, kHeadLanes, true>(col, orow, (size_t)p.slab, w, active, normed, p.eps, nvalid);
    __syncthreads();  // the buffer is staged again two tiles later
  }
}

template <typename T, int kHeadLanes>
__global__ void __launch_bounds__(conv::kThreads, 2)
pkda_qkv_conv_bwd_kernel(const ConvParams p) {
  using namespace conv;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // two stages of {x rows t0-3 .. t0+34, gradient rows t0 .. t0+34}, then the fp32 dy tile
  float* sdy = reinterpret_cast<float*>(smem_raw + 2 * bwd_stage<T>());
  const int b = blockIdx.y / p.spans_per_row;
  const int span0 = (blockIdx.y - b * p.spans_per_row) * (kBwdTokens * kBwdTiles);
  const int cb = blockIdx.x * kTileCh;
  const int lane = threadIdx.x % kLanes, grp = threadIdx.x / kLanes;
  const int c = cb + kVec * lane;
  const bool active = c < p.channels;
  const int cc = active ? c : 0;
  const bool normed = active && c < p.norm_channels;
  const T* xrow = static_cast<const T*>(p.x) + (size_t)b * p.seq_len * p.channels;
  const size_t doff = (size_t)b * p.seq_len * p.slab;
  const T *dq = static_cast<const T*>(p.dq) + doff, *dk = static_cast<const T*>(p.dk) + doff,
          *dv = static_cast<const T*>(p.dv) + doff;
  T* dxrow = static_cast<T*>(p.dx) + (size_t)b * p.seq_len * p.channels + cc;
  const int ntiles = min(kBwdTiles, (p.seq_len - span0 + kBwdTokens - 1) / kBwdTokens);
  auto stage_tile = [&](int tile) {
    T* sx = reinterpret_cast<T*>(smem_raw + (tile & 1) * bwd_stage<T>());
    T* sd = sx + (kBwdTokens + 2 * kHalo) * kTileCh;
    const int t0 = span0 + tile * kBwdTokens;
    stage_rows(sx, xrow, t0 - kHalo, kBwdTokens + 2 * kHalo, p.seq_len, cb, p.channels);
    stage_grad_rows(sd, dq, dk, dv, t0, kBwdDyRows, p.seq_len, cb, p.channels, p.slab);
    cp_async_commit();
  };
  stage_tile(0);
  float2 w[2][4], dwacc[2][4];
  load_taps(p, c, active, w);
#pragma unroll
  for (int pr = 0; pr < 2; ++pr)
#pragma unroll
    for (int j = 0; j < 4; ++j) dwacc[pr][j] = f2(0.f, 0.f);
  for (int tile = 0; tile < ntiles; ++tile) {
    const int t0 = span0 + tile * kBwdTokens;
    if (tile + 1 < ntiles) {
      stage_tile(tile + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const T* sx = reinterpret_cast<const T*>(smem_raw + (tile & 1) * bwd_stage<T>());
    const T* sd = sx + (kBwdTokens + 2 * kHalo) * kTileCh;
    // ---- phase A: gradient of the pre-activation for tokens t0 .. t0+34 and the weight gradient of
    // the tile's own 32 tokens.  Groups 0-2 take 9 own tokens each, group 3 five own tokens and the
    // three look-ahead rows.
    {
      const int i0 = kBwdDyPerGroup * grp;
      const T* xc = sx + kVec * lane + i0 * kTileCh;
      const T* dc = sd + kVec * lane + i0 * kTileCh;
      float* yc = sdy + kVec * lane + i0 * kTileCh;
      if (grp < kGroups - 1)
        conv_bwd_phase_a<T, kHeadLanes, kBwdDyPerGroup, kBwdDyPerGroup>(xc, dc, yc, w, dwacc, normed, p.eps,
                                                                         threadIdx.x & 31);
      else
        conv_bwd_phase_a<T, kHeadLanes, kBwdDyRows - (kGroups - 1) * kBwdDyPerGroup,
                         kBwdTokens - (kGroups - 1) * kBwdDyPerGroup>(xc, dc, yc, w, dwacc, normed, p.eps,
                                                                       threadIdx.x & 31);
    }
    __syncthreads();
    // ---- phase B: dx for the tile's own 32 tokens
    {
      constexpr int kPer = kBwdTokens / kGroups;  // 8
      const int j0 = kPer * grp;
      const float* dc = sdy + kVec * lane + j0 * kTileCh;
      T* drow = dxrow + (size_t)(t0 + j0) * p.channels;
      const int nvalid = p.seq_len - (t0 + j0);
      if (nvalid >= kPer) conv_bwd_phase_b<T, false>(dc, drow, (size_t)p.channels, w, active, nvalid);
      else conv_bwd_phase_b<T, true>(dc, drow, (size_t)p.channels, w, active, nvalid);
    }
    __syncthreads();
  }
  // ---- weight gradient: the four token groups in a fixed order, one partial per CTA
  float* sPart = sdy;  // [kGroups][kLanes][16]; entry 4 * channel + padded tap
#pragma unroll
  for (int pr = 0; pr < 2; ++pr)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sPart[(grp * kLanes + lane) * 16 + 4 * (2 * pr) + j] = dwacc[pr][j].x;
      sPart[(grp * kLanes + lane) * 16 + 4 * (2 * pr + 1) + j] = dwacc[pr][j].y;
    }
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
  return ensure_dynamic_smem(kernel, bytes);
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
  const dim3 grid = conv_grid(p, conv::kFwdTokens * conv::kFwdTiles);
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
