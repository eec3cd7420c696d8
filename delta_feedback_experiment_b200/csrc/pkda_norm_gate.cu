// Per-head RMS normalisation with a learned weight and a sigmoid output gate,
// the stage after the recurrence in the PKDA layer:
//   rstd = rsqrt(mean_c(x^2) + eps),   y = x * rstd * w * sigmoid(gate)
// and its backward
//   dyh = dy * w * sig,  xh = x * rstd,
//   dx = rstd * (dyh - xh * mean_c(dyh * xh)),  dgate = dy * xh * w * sig * (1 - sig),
//   dw = sum over rows of dy * xh * sig.
// Streaming kernels.  A row of `dim` channels is held by dim/8 adjacent lanes; a
// thread's 8 channels of a row are one "unit".  Every thread streams its own units
// through a private ring of cp.async stages in shared memory (it only ever reads
// back what it copied itself, so the ring needs no barrier), which keeps several
// hundred bytes per thread in flight without holding them in registers.  Row
// statistics are shuffle reductions; the weight gradient is reduced in a fixed order
// (registers -> shared memory -> one partial per CTA -> second kernel).
#include "pkda_common.cuh"
#include "pkda_launch.h"

namespace pkda {

namespace ng {
constexpr int kThreads = 256;
constexpr int kVec = 8;
constexpr int kStages = 4;
constexpr int kUnits = 2;  // units (rows) per thread and stage
template <typename T> __host__ __device__ constexpr int unit_bytes() { return kVec * (int)sizeof(T); }
// ring: [stage][tensor][unit][thread] unit_bytes
template <typename T> __host__ __device__ constexpr int fwd_smem() { return kStages * 2 * kUnits * kThreads * unit_bytes<T>(); }
template <typename T> __host__ __device__ constexpr int bwd_smem() {
  return kStages * 3 * kUnits * kThreads * unit_bytes<T>();
}
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
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1)
    if (lanes > o) v += __shfl_xor_sync(0xffffffffu, v, o);  // uniform predicate, no loop control
  return v;
}

// One unit (8 channels of T) global -> this thread's slot of the ring.
template <typename T>
__device__ __forceinline__ void copy_unit(T* slot, const T* g, bool ok) {
  cp_async16(slot, ok ? g : g, ok);
  if (sizeof(T) == 4) cp_async16(slot + 4, ok ? g + 4 : g, ok);
}

// Iteration `it` of a CTA covers rows  (it * gridDim.x + blockIdx.x) * slots * kUnits + u * slots + slot.
template <typename T>
__global__ void __launch_bounds__(ng::kThreads)
pkda_norm_gate_fwd_kernel(const NormGateParams p) {
  using namespace ng;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* ring = reinterpret_cast<T*>(smem_raw);
  const int tid = threadIdx.x;
  const int lane_in_row = tid % p.lanes, slot = tid / p.lanes, slots = kThreads / p.lanes;
  const int c0 = lane_in_row * kVec;
  const long long per_iter = (long long)slots * kUnits;
  const long long n_iter_all = (p.rows + per_iter - 1) / per_iter;
  const int n_iter = (int)((n_iter_all - blockIdx.x + gridDim.x - 1) / gridDim.x);  // iterations of this CTA
  float w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = p.w[c0 + j];
  auto row_of = [&](int it, int u) { return ((long long)it * gridDim.x + blockIdx.x) * per_iter + (long long)u * slots + slot; };
  auto slot_ptr = [&](int stage, int tensor, int u) {
    return ring + ((size_t)((stage * 2 + tensor) * kUnits + u) * kThreads + tid) * kVec;
  };
  auto issue = [&](int it) {
    if (it < n_iter) {
      const int stage = it % kStages;
#pragma unroll
      for (int u = 0; u < kUnits; ++u) {
        const long long r = row_of(it, u);
        const bool ok = r < p.rows;
        const size_t off = ok ? (size_t)r * p.dim + c0 : 0;
        copy_unit(slot_ptr(stage, 0, u), static_cast<const T*>(p.x) + off, ok);
        copy_unit(slot_ptr(stage, 1, u), static_cast<const T*>(p.gate) + off, ok);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s);
  for (int it = 0; it < n_iter; ++it) {
    issue(it + kStages - 1);
    cp_async_wait<kStages - 1>();
    const int stage = it % kStages;
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
      const long long r = row_of(it, u);
      float x[8], g[8], y[8], ss = 0.f;
      Vec8<T>::load(slot_ptr(stage, 0, u), x);
      Vec8<T>::load(slot_ptr(stage, 1, u), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
      ss = lane_group_sum(ss, p.lanes);
      const float rstd = rsqrtf(ss * p.inv_dim + p.eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = x[j] * rstd * w[j] * Vec8<T>::sigmoid(g[j]);
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
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* ring = reinterpret_cast<T*>(smem_raw);
  const int tid = threadIdx.x;
  const int lane_in_row = tid % p.lanes, slot = tid / p.lanes, slots = kThreads / p.lanes;
  const int c0 = lane_in_row * kVec;
  const long long per_iter = (long long)slots * kUnits;
  const long long n_iter_all = (p.rows + per_iter - 1) / per_iter;
  const int n_iter = (int)((n_iter_all - blockIdx.x + gridDim.x - 1) / gridDim.x);
  float w[8], dwacc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    w[j] = p.w[c0 + j];
    dwacc[j] = 0.f;
  }
  auto row_of = [&](int it, int u) { return ((long long)it * gridDim.x + blockIdx.x) * per_iter + (long long)u * slots + slot; };
  auto slot_ptr = [&](int stage, int tensor, int u) {
    return ring + ((size_t)((stage * 3 + tensor) * kUnits + u) * kThreads + tid) * kVec;
  };
  auto issue = [&](int it) {
    if (it < n_iter) {
      const int stage = it % kStages;
#pragma unroll
      for (int u = 0; u < kUnits; ++u) {
        const long long r = row_of(it, u);
        const bool ok = r < p.rows;
        const size_t off = ok ? (size_t)r * p.dim + c0 : 0;
        copy_unit(slot_ptr(stage, 0, u), static_cast<const T*>(p.x) + off, ok);
        copy_unit(slot_ptr(stage, 1, u), static_cast<const T*>(p.gate) + off, ok);
        copy_unit(slot_ptr(stage, 2, u), static_cast<const T*>(p.dy) + off, ok);
      }
    }
    cp_async_commit();
  };
  // The rows' reciprocal deviations come by plain loads one iteration ahead (the lanes of a row read the
  // same word: one broadcast transaction), not through the ring: a 4-byte asynchronous copy per thread
  // costs as much of the shared-memory pipe as a 16-byte one.
  float rs_next[kUnits];
  auto load_rstd = [&](int it) {
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
      const long long r = row_of(it, u);
      rs_next[u] = (it < n_iter && r < p.rows) ? p.rstd[r] : 0.f;
    }
  };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s);
  load_rstd(0);
  for (int it = 0; it < n_iter; ++it) {
    issue(it + kStages - 1);
    float rs_cur[kUnits];
#pragma unroll
    for (int u = 0; u < kUnits; ++u) rs_cur[u] = rs_next[u];
    load_rstd(it + 1);
    cp_async_wait<kStages - 1>();
    const int stage = it % kStages;
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
      const long long r = row_of(it, u);
      float x[8], g[8], dy[8], dx[8], dg[8], dot = 0.f;
      Vec8<T>::load(slot_ptr(stage, 0, u), x);
      Vec8<T>::load(slot_ptr(stage, 1, u), g);
      Vec8<T>::load(slot_ptr(stage, 2, u), dy);
      const float rs = rs_cur[u];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = Vec8<T>::sigmoid(g[j]);
        const float xh = x[j] * rs;
        const float t = dy[j] * xh * sg;   // dy * xh * sig
        dwacc[j] += t;
        dot += t * w[j];                   // dyh * xh
        dg[j] = t * w[j] * (1.f - sg);
        dx[j] = dy[j] * w[j] * sg;         // dyh
        x[j] = xh;
      }
      dot = lane_group_sum(dot, p.lanes) * p.inv_dim;
#pragma unroll
      for (int j = 0; j < 8; ++j) dx[j] = rs * (dx[j] - x[j] * dot);
      if (r < p.rows) {
        Vec8<T>::store(static_cast<T*>(p.dx) + r * p.dim + c0, dx);
        Vec8<T>::store(static_cast<T*>(p.dgate) + r * p.dim + c0, dg);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  float* sPart = reinterpret_cast<float*>(smem_raw);  // [kThreads][kVec + 1]
#pragma unroll
  for (int j = 0; j < 8; ++j) sPart[tid * (kVec + 1) + j] = dwacc[j];
  __syncthreads();
  if (tid < p.dim) {
    const int lr = tid / kVec, j = tid % kVec;
    float a = 0.f;
    for (int s = 0; s < slots; ++s) a += sPart[(s * p.lanes + lr) * (kVec + 1) + j];
    p.part[(size_t)blockIdx.x * p.dim + tid] = a;
  }
}

// Sums the per-CTA partials: thread (sub, c) adds every kSub-th partial of channel c,
// then the kSub sub-sums are added in order.
__global__ void __launch_bounds__(1024) pkda_norm_gate_dw_kernel(const float* part, float* dw, int dim, int groups) {
  __shared__ float sSub[1024];
  const int c = threadIdx.x % dim, sub = threadIdx.x / dim, nsub = 1024 / dim;
  float a = 0.f;
  for (int g = sub; g < groups; g += nsub) a += part[(size_t)g * dim + c];
  sSub[threadIdx.x] = a;
  __syncthreads();
  if (sub == 0) {
    float t = 0.f;
    for (int s2 = 0; s2 < nsub; ++s2) t += sSub[s2 * dim + c];
    dw[c] = t;
  }
}

// ------------------------------------------------------------------ host side
static int sm_count() {
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

// Persistent grid: as many CTAs as are resident at once (never more than 8 per SM,
// the bound the backward's partial buffer is sized for), fewer for small inputs.
template <typename K> static int ng_grid(const pkda_norm_gate_args& a, K kernel, int smem) {
  const int lanes = a.dim / ng::kVec;
  const long long per_iter = (long long)(ng::kThreads / lanes) * ng::kUnits;
  const long long want = (a.rows + per_iter - 1) / per_iter;
  int per_sm = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, ng::kThreads, smem) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  if (per_sm > 8) per_sm = 8;
  const long long cap = (long long)sm_count() * per_sm;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

template <typename K> static bool ng_allow_smem(K kernel, int bytes) {
  return ensure_dynamic_smem(kernel, bytes);
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
  if (a->dtype == PKDA_BF16) {
    constexpr int smem = ng::fwd_smem<bf16>();
    if (!ng_allow_smem(pkda_norm_gate_fwd_kernel<bf16>, smem)) return PKDA_ERR_LAUNCH;
    const int grid = ng_grid(*a, pkda_norm_gate_fwd_kernel<bf16>, smem);
    begin_stage(kStageNormGateFwd, st);
    pkda_norm_gate_fwd_kernel<bf16><<<grid, ng::kThreads, smem, st>>>(p);
  } else {
    constexpr int smem = ng::fwd_smem<float>();
    if (!ng_allow_smem(pkda_norm_gate_fwd_kernel<float>, smem)) return PKDA_ERR_LAUNCH;
    const int grid = ng_grid(*a, pkda_norm_gate_fwd_kernel<float>, smem);
    begin_stage(kStageNormGateFwd, st);
    pkda_norm_gate_fwd_kernel<float><<<grid, ng::kThreads, smem, st>>>(p);
  }
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

size_t norm_gate_bwd_workspace(const pkda_norm_gate_args& a) {
  NormGateParams p;
  if (ng_check(a, p) != PKDA_OK) return 0;
  return align_up((size_t)sm_count() * 8 * a.dim * sizeof(float));  // the grid never exceeds 8 CTAs per SM
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
  int grid = 1;
  if (a->dtype == PKDA_BF16) {
    constexpr int smem = ng::bwd_smem<bf16>();
    if (!ng_allow_smem(pkda_norm_gate_bwd_kernel<bf16>, smem)) return PKDA_ERR_LAUNCH;
    grid = ng_grid(*a, pkda_norm_gate_bwd_kernel<bf16>, smem);
    begin_stage(kStageNormGateBwd, st);
    pkda_norm_gate_bwd_kernel<bf16><<<grid, ng::kThreads, smem, st>>>(p);
  } else {
    constexpr int smem = ng::bwd_smem<float>();
    if (!ng_allow_smem(pkda_norm_gate_bwd_kernel<float>, smem)) return PKDA_ERR_LAUNCH;
    grid = ng_grid(*a, pkda_norm_gate_bwd_kernel<float>, smem);
    begin_stage(kStageNormGateBwd, st);
    pkda_norm_gate_bwd_kernel<float><<<grid, ng::kThreads, smem, st>>>(p);
  }
  end_stage(st);
  begin_stage(kStageNormGateDw, st);
  pkda_norm_gate_dw_kernel<<<1, 1024, 0, st>>>(p.part, a->dweight, a->dim, grid);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
