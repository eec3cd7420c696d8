// Fused Q|K|V short convolution of the PKDA layer, forward and backward:
//   y[t][c] = sum_j w[c][j] * x[t - (taps-1) + j][c]      (causal, depthwise, <= 4 taps)
//   s = silu(y)
//   out = s * rsqrt(sum over the head of s^2 + eps)        for c < norm_channels (Q and K)
//   out = s                                                otherwise (V)
// written as three slabs q, k, v.  The kernels are pure streaming work: one
// thread owns 4 adjacent channels and walks a strip of 64 tokens with the last
// three inputs in registers, so every input element is read once (plus a
// three-token halo per strip) and every output written once; the per-head sums
// are shuffle reductions inside a warp (a head is at most 32 lanes).  The backward
// recomputes the pre-activation instead of saving it, extends each strip by three
// tokens so that dx needs no atomics, and reduces the weight gradient in a fixed
// order (registers -> shared memory across the CTA's strips -> one partial per
// CTA row -> a small second kernel).
#include "pkda_common.cuh"
#include "pkda_launch.h"

namespace pkda {

namespace conv {
constexpr int kVec = 4;       // channels per thread
constexpr int kLanes = 64;    // threads along the channel axis (256 channels per CTA)
constexpr int kStrips = 4;    // token strips per CTA
constexpr int kStripTokens = 64;
constexpr int kMaxTaps = 4;
constexpr int kUnroll = 4;    // tokens whose loads are issued together
}  // namespace conv

struct ConvParams {
  int batch, seq_len, channels, slab, taps, head_lanes, norm_channels, strips_per_row;
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

// Sum over the lanes of one head (head_lanes is a power of two <= 32).
__device__ __forceinline__ float head_sum(float v, int head_lanes) {
  for (int o = head_lanes >> 1; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct ConvThread {
  int b, t0, c, slab_id, cs;
  bool active, normed;
};

__device__ __forceinline__ bool conv_thread(const ConvParams& p, ConvThread& th) {
  const int strip = blockIdx.y * conv::kStrips + threadIdx.y;
  th.b = strip / p.strips_per_row;
  if (th.b >= p.batch) return false;  // uniform per warp
  th.t0 = (strip - th.b * p.strips_per_row) * conv::kStripTokens;
  th.c = (blockIdx.x * conv::kLanes + threadIdx.x) * conv::kVec;
  th.active = th.c < p.channels;
  const int cc = th.active ? th.c : 0;
  th.slab_id = cc / p.slab;
  th.cs = cc - th.slab_id * p.slab;
  th.normed = th.active && th.c < p.norm_channels;
  return true;
}

__device__ __forceinline__ void load_taps(const ConvParams& p, const ConvThread& th, float (&w)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int jj = j - (conv::kMaxTaps - p.taps);  // tap j of the padded filter
      w[i][j] = (th.active && jj >= 0) ? p.w[(size_t)(th.c + i) * p.taps + jj] : 0.f;
    }
}

template <typename T>
__global__ void __launch_bounds__(conv::kLanes * conv::kStrips)
pkda_qkv_conv_fwd_kernel(const ConvParams p) {
  using namespace conv;
  ConvThread th;
  if (!conv_thread(p, th)) return;
  float w[4][4];
  load_taps(p, th, w);
  const T* xrow = static_cast<const T*>(p.x) + (size_t)th.b * p.seq_len * p.channels + (th.active ? th.c : 0);
  T* out = static_cast<T*>(th.slab_id == 0 ? p.q : th.slab_id == 1 ? p.k : p.v) +
           (size_t)th.b * p.seq_len * p.slab + th.cs;
  float win[3][4];  // x[t-3], x[t-2], x[t-1]
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int t = th.t0 - 3 + j;
#pragma unroll
    for (int i = 0; i < 4; ++i) win[j][i] = 0.f;
    if (th.active && t >= 0) Vec4<T>::load(xrow + (size_t)t * p.channels, win[j]);
  }
  const int tend = min(th.t0 + kStripTokens, p.seq_len);
  for (int tb = th.t0; tb < tend; tb += kUnroll) {
    float xa[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
      for (int i = 0; i < 4; ++i) xa[u][i] = 0.f;
      if (th.active && tb + u < tend) Vec4<T>::load(xrow + (size_t)(tb + u) * p.channels, xa[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int t = tb + u;
      float s[4], ss = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float y = w[i][0] * win[0][i] + w[i][1] * win[1][i] + w[i][2] * win[2][i] + w[i][3] * xa[u][i];
        s[i] = y * Vec4<T>::sigmoid(y);
        ss += s[i] * s[i];
        win[0][i] = win[1][i]; win[1][i] = win[2][i]; win[2][i] = xa[u][i];
      }
      ss = head_sum(ss, p.head_lanes);
      const float r = th.normed ? rsqrtf(ss + p.eps) : 1.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] *= r;
      if (th.active && t < tend) Vec4<T>::store(out + (size_t)t * p.slab, s);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(conv::kLanes * conv::kStrips)
pkda_qkv_conv_bwd_kernel(const ConvParams p) {
  using namespace conv;
  __shared__ float sPart[kStrips][kLanes][16];
  ConvThread th;
  const bool live = conv_thread(p, th);
  float dwacc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dwacc[i][j] = 0.f;
  if (live) {
    float w[4][4];
    load_taps(p, th, w);
    const T* xrow = static_cast<const T*>(p.x) + (size_t)th.b * p.seq_len * p.channels + (th.active ? th.c : 0);
    const T* drow = static_cast<const T*>(th.slab_id == 0 ? p.dq : th.slab_id == 1 ? p.dk : p.dv) +
                    (size_t)th.b * p.seq_len * p.slab + th.cs;
    T* dxrow = static_cast<T*>(p.dx) + (size_t)th.b * p.seq_len * p.channels + (th.active ? th.c : 0);
    float win[3][4], dxa[3][4];  // dxa: partial dx of tokens t-3, t-2, t-1
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int t = th.t0 - 3 + j;
#pragma unroll
      for (int i = 0; i < 4; ++i) win[j][i] = dxa[j][i] = 0.f;
      if (th.active && t >= 0) Vec4<T>::load(xrow + (size_t)t * p.channels, win[j]);
    }
    const int own_end = min(th.t0 + kStripTokens, p.seq_len);
    // three more tokens than the strip owns: their dy completes the strip's last dx rows
    for (int tb = th.t0; tb < th.t0 + kStripTokens + 3; tb += kUnroll) {
      if (tb - 3 >= own_end) break;
      float xa[kUnroll][4], da[kUnroll][4];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
        for (int i = 0; i < 4; ++i) xa[u][i] = da[u][i] = 0.f;
        if (th.active && tb + u < p.seq_len) {
          Vec4<T>::load(xrow + (size_t)(tb + u) * p.channels, xa[u]);
          Vec4<T>::load(drow + (size_t)(tb + u) * p.slab, da[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int t = tb + u;
        float y[4], sg[4], s[4], ss = 0.f, sd = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          y[i] = w[i][0] * win[0][i] + w[i][1] * win[1][i] + w[i][2] * win[2][i] + w[i][3] * xa[u][i];
          sg[i] = Vec4<T>::sigmoid(y[i]);
          s[i] = y[i] * sg[i];
          ss += s[i] * s[i];
          sd += s[i] * da[u][i];
        }
        ss = head_sum(ss, p.head_lanes);
        sd = head_sum(sd, p.head_lanes);
        const float r = th.normed ? rsqrtf(ss + p.eps) : 1.f;
        const float back = th.normed ? r * r * r * sd : 0.f;
        const bool owned = t < own_end;
        float dxnew[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float ds = r * da[u][i] - s[i] * back;
          const float dy = ds * (sg[i] + s[i] * (1.f - sg[i]));  // silu'(y) = sig + y sig (1 - sig)
          if (owned) {
            dwacc[i][0] += dy * win[0][i];
            dwacc[i][1] += dy * win[1][i];
            dwacc[i][2] += dy * win[2][i];
            dwacc[i][3] += dy * xa[u][i];
          }
          const float done = dxa[0][i] + w[i][0] * dy;  // dx of token t-3 is complete
          dxa[0][i] = dxa[1][i] + w[i][1] * dy;
          dxa[1][i] = dxa[2][i] + w[i][2] * dy;
          dxa[2][i] = w[i][3] * dy;
          dxnew[i] = done;
          win[0][i] = win[1][i]; win[1][i] = win[2][i]; win[2][i] = xa[u][i];
        }
        const int td = t - 3;
        if (th.active && td >= th.t0 && td < own_end) Vec4<T>::store(dxrow + (size_t)td * p.channels, dxnew);
      }
    }
  }
  // weight gradient: strips of this CTA in a fixed order, then one partial per CTA row
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) sPart[threadIdx.y][threadIdx.x][4 * i + j] = dwacc[i][j];
  __syncthreads();
  const int c = (blockIdx.x * kLanes + threadIdx.x) * kVec;
  if (threadIdx.y == 0 && c < p.channels) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      for (int j = 0; j < p.taps; ++j) {
        const int e = 4 * i + j + (kMaxTaps - p.taps);
        float a = 0.f;
#pragma unroll
        for (int sidx = 0; sidx < kStrips; ++sidx) a += sPart[sidx][threadIdx.x][e];
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
static int conv_check(const pkda_qkv_conv_args& a, ConvParams& p, dim3& grid) {
  if (a.batch < 0 || a.seq_len < 0 || a.channels <= 0 || a.channels % 3) return PKDA_ERR_SHAPE;
  if (a.taps < 1 || a.taps > conv::kMaxTaps) return PKDA_ERR_SHAPE;
  const int slab = a.channels / 3, hd = a.head_dim;
  if (hd < 4 || hd > 128 || (hd & (hd - 1)) || slab % hd) return PKDA_ERR_SHAPE;
  if (a.norm_channels < 0 || a.norm_channels > a.channels || a.norm_channels % hd) return PKDA_ERR_SHAPE;
  if (a.dtype != PKDA_BF16 && a.dtype != PKDA_F32) return PKDA_ERR_DTYPE;
  p.batch = a.batch; p.seq_len = a.seq_len; p.channels = a.channels; p.slab = slab; p.taps = a.taps;
  p.head_lanes = hd / conv::kVec; p.norm_channels = a.norm_channels; p.eps = a.eps;
  p.strips_per_row = (a.seq_len + conv::kStripTokens - 1) / conv::kStripTokens;
  p.x = a.x; p.w = a.weight; p.q = a.q; p.k = a.k; p.v = a.v;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv; p.dx = a.dx; p.part = nullptr;
  const long long strips = (long long)a.batch * p.strips_per_row;
  grid = dim3((a.channels / conv::kVec + conv::kLanes - 1) / conv::kLanes,
              (unsigned)((strips + conv::kStrips - 1) / conv::kStrips));
  return PKDA_OK;
}

static bool aligned16(const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; }

int qkv_conv_fwd(const pkda_qkv_conv_args* a, cudaStream_t st) {
  ConvParams p;
  dim3 grid;
  if (int rc = conv_check(*a, p, grid)) return rc;
  if (a->batch == 0 || a->seq_len == 0) return PKDA_OK;
  if (!a->x || !a->weight || !a->q || !a->k || !a->v) return PKDA_ERR_NULL;
  if (!aligned16(a->x) || !aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v)) return PKDA_ERR_ALIGN;
  const dim3 block(conv::kLanes, conv::kStrips);
  begin_stage(kStageConvFwd, st);
  if (a->dtype == PKDA_BF16) pkda_qkv_conv_fwd_kernel<bf16><<<grid, block, 0, st>>>(p);
  else pkda_qkv_conv_fwd_kernel<float><<<grid, block, 0, st>>>(p);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

size_t qkv_conv_bwd_workspace(const pkda_qkv_conv_args& a) {
  ConvParams p;
  dim3 grid;
  if (conv_check(a, p, grid) != PKDA_OK) return 0;
  return align_up((size_t)grid.y * a.channels * a.taps * sizeof(float));
}

int qkv_conv_bwd(const pkda_qkv_conv_args* a, cudaStream_t st) {
  ConvParams p;
  dim3 grid;
  if (int rc = conv_check(*a, p, grid)) return rc;
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
  const dim3 block(conv::kLanes, conv::kStrips);
  begin_stage(kStageConvBwd, st);
  if (a->dtype == PKDA_BF16) pkda_qkv_conv_bwd_kernel<bf16><<<grid, block, 0, st>>>(p);
  else pkda_qkv_conv_bwd_kernel<float><<<grid, block, 0, st>>>(p);
  end_stage(st);
  begin_stage(kStageConvDw, st);
  pkda_qkv_conv_dw_kernel<<<(n + 255) / 256, 256, 0, st>>>(p.part, a->dweight, n, (int)grid.y);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
