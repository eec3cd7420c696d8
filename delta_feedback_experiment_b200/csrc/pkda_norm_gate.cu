// Per-head RMS normalisation with a learned weight and a sigmoid output gate,
// the stage after the recurrence in the PKDA layer:
//   rstd = rsqrt(mean_c(x^2) + eps),   y = x * rstd * w * sigmoid(gate)
// and its backward
//   dyh = dy * w * sig,  xh = x * rstd,
//   dx = rstd * (dyh - xh * mean_c(dyh * xh)),  dgate = dy * xh * w * sig * (1 - sig),
//   dw = sum over rows of dy * xh * sig.
// Streaming kernels: a row of `dim` channels is held by dim/8 adjacent lanes
// (128-bit loads and stores for bf16), the row statistics are shuffle reductions,
// each thread keeps several rows in flight, and the weight gradient is reduced in
// a fixed order (registers -> shared memory -> one partial per CTA -> second kernel).
#include "pkda_common.cuh"
#include "pkda_launch.h"

namespace pkda {

namespace ng {
constexpr int kThreads = 256;
constexpr int kVec = 8;
constexpr int kRowsInFlight = 4;  // rows per thread whose loads are issued together
}  // namespace ng

struct NormGateParams {
  long long rows;
  int dim, lanes;  // lanes = dim / 8
  float eps, inv_dim;
  const void *x, *gate, *dy;
  const float* w;
  void *y, *dx, *dgate;
  float* rstd;
  float* part;  // [gridDim.x][dim]
};

template <typename T> struct Vec8;
template <> struct Vec8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16(w[j]);
      f[2 * j] = a.x;
      f[2 * j + 1] = a.y;
    }
  }
  static __device__ __forceinline__ void store(bf16* p, const float (&f)[8]) {
    *reinterpret_cast<uint4*>(p) =
        make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
  }
  static __device__ __forceinline__ float sigmoid(float g) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * g));
    return fmaf(0.5f, t, 0.5f);
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  static __device__ __forceinline__ float sigmoid(float g) { return 1.f / (1.f + expf(-g)); }
};

__device__ __forceinline__ float lane_group_sum(float v, int lanes) {
  for (int o = lanes >> 1; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Rows are dealt to (CTA, row slot) in a grid-stride loop; a CTA iteration covers
// kRowsInFlight * (kThreads / lanes) rows.
template <typename T>
__global__ void __launch_bounds__(ng::kThreads)
pkda_norm_gate_fwd_kernel(const NormGateParams p) {
  using namespace ng;
  const int lane_in_row = threadIdx.x % p.lanes, slot = threadIdx.x / p.lanes;
  const int slots = kThreads / p.lanes;
  const int c0 = lane_in_row * kVec;
  float w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = p.w[c0 + j];
  const long long per_iter = (long long)slots * kRowsInFlight;
  for (long long base = (long long)blockIdx.x * per_iter; base < p.rows; base += (long long)gridDim.x * per_iter) {
    float x[kRowsInFlight][8], g[kRowsInFlight][8];
#pragma unroll
    for (int u = 0; u < kRowsInFlight; ++u) {
      const long long r = base + (long long)u * slots + slot;
#pragma unroll
      for (int j = 0; j < 8; ++j) x[u][j] = g[u][j] = 0.f;
      if (r < p.rows) {
        Vec8<T>::load(static_cast<const T*>(p.x) + r * p.dim + c0, x[u]);
        Vec8<T>::load(static_cast<const T*>(p.gate) + r * p.dim + c0, g[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kRowsInFlight; ++u) {
      const long long r = base + (long long)u * slots + slot;
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[u][j] * x[u][j];
      ss = lane_group_sum(ss, p.lanes);
      const float rstd = rsqrtf(ss * p.inv_dim + p.eps);
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = x[u][j] * rstd * w[j] * Vec8<T>::sigmoid(g[u][j]);
      if (r < p.rows) {
        Vec8<T>::store(static_cast<T*>(p.y) + r * p.dim + c0, y);
        if (lane_in_row == 0) p.rstd[r] = rstd;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(ng::kThreads)
pkda_norm_gate_bwd_kernel(const NormGateParams p) {
  using namespace ng;
  __shared__ float sPart[kThreads][kVec + 1];
  const int lane_in_row = threadIdx.x % p.lanes, slot = threadIdx.x / p.lanes;
  const int slots = kThreads / p.lanes;
  const int c0 = lane_in_row * kVec;
  float w[8], dwacc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    w[j] = p.w[c0 + j];
    dwacc[j] = 0.f;
  }
  constexpr int kInFlight = 2;
  const long long per_iter = (long long)slots * kInFlight;
  for (long long base = (long long)blockIdx.x * per_iter; base < p.rows; base += (long long)gridDim.x * per_iter) {
    float x[kInFlight][8], g[kInFlight][8], dy[kInFlight][8], rs[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const long long r = base + (long long)u * slots + slot;
#pragma unroll
      for (int j = 0; j < 8; ++j) x[u][j] = g[u][j] = dy[u][j] = 0.f;
      rs[u] = 0.f;
      if (r < p.rows) {
        Vec8<T>::load(static_cast<const T*>(p.x) + r * p.dim + c0, x[u]);
        Vec8<T>::load(static_cast<const T*>(p.gate) + r * p.dim + c0, g[u]);
        Vec8<T>::load(static_cast<const T*>(p.dy) + r * p.dim + c0, dy[u]);
        rs[u] = p.rstd[r];
      }
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const long long r = base + (long long)u * slots + slot;
      float xh[8], dyh[8], sg[8], dot = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        sg[j] = Vec8<T>::sigmoid(g[u][j]);
        xh[j] = x[u][j] * rs[u];
        dyh[j] = dy[u][j] * w[j] * sg[j];
        dot += dyh[j] * xh[j];
        dwacc[j] += dy[u][j] * xh[j] * sg[j];
      }
      dot = lane_group_sum(dot, p.lanes) * p.inv_dim;
      float dx[8], dg[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dx[j] = rs[u] * (dyh[j] - xh[j] * dot);
        dg[j] = dy[u][j] * xh[j] * w[j] * sg[j] * (1.f - sg[j]);
      }
      if (r < p.rows) {
        Vec8<T>::store(static_cast<T*>(p.dx) + r * p.dim + c0, dx);
        Vec8<T>::store(static_cast<T*>(p.dgate) + r * p.dim + c0, dg);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sPart[threadIdx.x][j] = dwacc[j];
  __syncthreads();
  if (threadIdx.x < p.dim) {
    const int c = threadIdx.x, lr = c / kVec, j = c % kVec;
    float a = 0.f;
    for (int s = 0; s < slots; ++s) a += sPart[s * p.lanes + lr][j];
    p.part[(size_t)blockIdx.x * p.dim + c] = a;
  }
}

__global__ void pkda_norm_gate_dw_kernel(const float* part, float* dw, int dim, int groups) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float a = 0.f;
  for (int g = 0; g < groups; ++g) a += part[(size_t)g * dim + c];
  dw[c] = a;
}

// ------------------------------------------------------------------ host side
static int ng_grid(const pkda_norm_gate_args& a, int in_flight) {
  const int lanes = a.dim / ng::kVec;
  const long long per_iter = (long long)(ng::kThreads / lanes) * in_flight;
  const long long want = (a.rows + per_iter - 1) / per_iter;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long cap = (long long)sms * 8;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

static int ng_check(const pkda_norm_gate_args& a, NormGateParams& p) {
  if (a.rows < 0 || a.dim < 8 || a.dim > 256 || (a.dim & (a.dim - 1))) return PKDA_ERR_SHAPE;
  if (a.dtype != PKDA_BF16 && a.dtype != PKDA_F32) return PKDA_ERR_DTYPE;
  p.rows = a.rows; p.dim = a.dim; p.lanes = a.dim / ng::kVec; p.eps = a.eps; p.inv_dim = 1.f / (float)a.dim;
  p.x = a.x; p.gate = a.gate; p.dy = a.dy; p.w = a.weight; p.y = a.y; p.dx = a.dx; p.dgate = a.dgate;
  p.rstd = a.rstd; p.part = nullptr;
  return PKDA_OK;
}

static bool ng_aligned(const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; }

int norm_gate_fwd(const pkda_norm_gate_args* a, cudaStream_t st) {
  NormGateParams p;
  if (int rc = ng_check(*a, p)) return rc;
  if (a->rows == 0) return PKDA_OK;
  if (!a->x || !a->gate || !a->weight || !a->y || !a->rstd) return PKDA_ERR_NULL;
  if (!ng_aligned(a->x) || !ng_aligned(a->gate) || !ng_aligned(a->y)) return PKDA_ERR_ALIGN;
  const int grid = ng_grid(*a, ng::kRowsInFlight);
  begin_stage(kStageNormGateFwd, st);
  if (a->dtype == PKDA_BF16) pkda_norm_gate_fwd_kernel<bf16><<<grid, ng::kThreads, 0, st>>>(p);
  else pkda_norm_gate_fwd_kernel<float><<<grid, ng::kThreads, 0, st>>>(p);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

size_t norm_gate_bwd_workspace(const pkda_norm_gate_args& a) {
  NormGateParams p;
  if (ng_check(a, p) != PKDA_OK) return 0;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return align_up((size_t)sms * 8 * a.dim * sizeof(float));  // the grid never exceeds 8 CTAs per SM
}

int norm_gate_bwd(const pkda_norm_gate_args* a, cudaStream_t st) {
  NormGateParams p;
  if (int rc = ng_check(*a, p)) return rc;
  if (!a->dweight) return PKDA_ERR_NULL;
  if (a->rows == 0)
    return cudaMemsetAsync(a->dweight, 0, (size_t)a->dim * sizeof(float), st) == cudaSuccess ? PKDA_OK
                                                                                             : PKDA_ERR_LAUNCH;
  if (!a->x || !a->gate || !a->weight || !a->rstd || !a->dy || !a->dx || !a->dgate) return PKDA_ERR_NULL;
  if (!ng_aligned(a->x) || !ng_aligned(a->gate) || !ng_aligned(a->dy) || !ng_aligned(a->dx) || !ng_aligned(a->dgate))
    return PKDA_ERR_ALIGN;
  if (!a->workspace || a->workspace_bytes < norm_gate_bwd_workspace(*a)) return PKDA_ERR_WORKSPACE;
  p.part = static_cast<float*>(a->workspace);
  const int grid = ng_grid(*a, 2);
  begin_stage(kStageNormGateBwd, st);
  if (a->dtype == PKDA_BF16) pkda_norm_gate_bwd_kernel<bf16><<<grid, ng::kThreads, 0, st>>>(p);
  else pkda_norm_gate_bwd_kernel<float><<<grid, ng::kThreads, 0, st>>>(p);
  end_stage(st);
  begin_stage(kStageNormGateDw, st);
  pkda_norm_gate_dw_kernel<<<(a->dim + 127) / 128, 128, 0, st>>>(p.part, a->dweight, a->dim, grid);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
