// Control epilogue of the PKDA layer.  The layer projects its input once to a packed
// row  [decay hidden (D) | beta logits (H) | precond decay logits (H) | precond beta
// logits (H) | output-gate hidden (D)]  (delta_feedback_experiment/pkda.py:318-353);
// the two hidden slices go on to further projections unchanged and the three
// per-head slices become
//   beta     = sigmoid(logits)
//   g_atk    = -exp(A_log_precond) * softplus(logits + dt_bias_precond)      (fp32)
//   beta_atk = sigmoid(logits).
// Forward: one pass over the 3H logits of every row.  Backward: ONE pass that applies
// the three activations' derivatives and writes the packed gradient row directly,
// hidden slices included -- what the reference does with separate pointwise kernels
// plus pack_control_gradients (delta_feedback_experiment/cuda_kernels.py:1081-1172) --
// and reduces the two per-head parameter gradients in a fixed order.
// pkda_pack_control_gradients is that packer alone (five slices -> one row).
#include "pkda_common.cuh"
#include "pkda_launch.h"

namespace pkda {

struct CtrlParams {
  long long rows;
  int heads, hidden, total;
  const void* packed;
  const float *A_log, *dt_bias;
  void *beta, *beta_atk;
  float* g_atk;
  const void *d_hidden0, *d_beta, *d_beta_atk, *d_hidden1;
  const float* d_g_atk;
  void* d_packed;
  float* part;  // [gridDim.x][2][heads]
};

constexpr int kCtrlThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kCtrlThreads)
pkda_controls_fwd_kernel(const CtrlParams p) {
  const long long n = p.rows * p.heads;
  const T* packed = static_cast<const T*>(p.packed);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / p.heads;
    const int h = (int)(i - r * p.heads);
    const T* row = packed + r * p.total + p.hidden;
    const float lb = to_f(row[h]), ld = to_f(row[p.heads + h]), lp = to_f(row[2 * p.heads + h]);
    static_cast<T*>(p.beta)[i] = from_f<T>(1.f / (1.f + expf(-lb)));
    p.g_atk[i] = -expf(p.A_log[h]) * softplus_acc(ld + p.dt_bias[h]);
    static_cast<T*>(p.beta_atk)[i] = from_f<T>(1.f / (1.f + expf(-lp)));
  }
}

// One thread per (row, column of the packed gradient).  Columns of the three logit
// slices recompute their activation from the saved packed row.
template <typename T>
__global__ void __launch_bounds__(kCtrlThreads)
pkda_controls_bwd_kernel(const CtrlParams p) {
  extern __shared__ float sAcc[];  // [2][heads] per-CTA partial sums, then the block reduction scratch
  const int H = p.heads, D = p.hidden, total = p.total;
  for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) sAcc[i] = 0.f;
  __syncthreads();
  const T* packed = static_cast<const T*>(p.packed);
  T* out = static_cast<T*>(p.d_packed);
  // a CTA owns a contiguous range of rows, so that its per-head sums are added in a fixed order
  const long long rows_per = (p.rows + gridDim.x - 1) / gridDim.x;
  const long long r_begin = (long long)blockIdx.x * rows_per;
  const long long r_end = r_begin + rows_per < p.rows ? r_begin + rows_per : p.rows;
  for (long long r = r_begin; r < r_end; ++r) {
    for (int c = threadIdx.x; c < total; c += blockDim.x) {
      float v;
      if (c < D) {
        v = p.d_hidden0 ? to_f(static_cast<const T*>(p.d_hidden0)[r * D + c]) : 0.f;
      } else if (c >= D + 3 * H) {
        v = p.d_hidden1 ? to_f(static_cast<const T*>(p.d_hidden1)[r * D + (c - D - 3 * H)]) : 0.f;
      } else {
        const int s = (c - D) / H, h = (c - D) - s * H;
        const float logit = to_f(packed[r * total + c]);
        if (s == 1) {
          const float dg = p.d_g_atk ? p.d_g_atk[r * H + h] : 0.f;
          const float z = logit + p.dt_bias[h], ea = expf(p.A_log[h]);
          v = dg * (-ea) / (1.f + expf(-z));            // d softplus = sigmoid
          // fixed order: thread c alone accumulates head h of this CTA, rows ascending
          sAcc[h] += dg * (-ea) * softplus_acc(z);       // d/dA_log = g_atk
          sAcc[H + h] += v;                              // d/ddt_bias
        } else {
          const T* dsrc = static_cast<const T*>(s == 0 ? p.d_beta : p.d_beta_atk);
          const float dv = dsrc ? to_f(dsrc[r * H + h]) : 0.f;
          const float sg = 1.f / (1.f + expf(-logit));
          v = dv * sg * (1.f - sg);
        }
      }
      out[r * total + c] = from_f<T>(v);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) p.part[(size_t)blockIdx.x * 2 * H + i] = sAcc[i];
}

__global__ void pkda_controls_reduce_kernel(const float* part, float* dA_log, float* ddt_bias, int heads, int groups) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * heads) return;
  float a = 0.f;
  for (int g = 0; g < groups; ++g) a += part[(size_t)g * 2 * heads + i];
  if (i < heads) dA_log[i] = a; else ddt_bias[i - heads] = a;
}

// out[r][:] = concat of five slices
template <typename T>
__global__ void __launch_bounds__(kCtrlThreads)
pkda_pack_control_kernel(const T* g0, const T* g1, const T* g2, const T* g3, const T* g4, T* out, long long rows,
                         int s0, int s1, int s2, int s3, int s4) {
  const int total = s0 + s1 + s2 + s3 + s4;
  const long long n = rows * total;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / total;
    int c = (int)(i - r * total);
    T v;
    if (c < s0) v = g0[r * s0 + c];
    else if ((c -= s0) < s1) v = g1[r * s1 + c];
    else if ((c -= s1) < s2) v = g2[r * s2 + c];
    else if ((c -= s2) < s3) v = g3[r * s3 + c];
    else v = g4[r * s4 + (c - s3)];
    out[i] = v;
  }
}

// ------------------------------------------------------------------ host side
static int ctrl_check(const pkda_controls_args& a, CtrlParams& p) {
  if (a.rows < 0 || a.heads <= 0 || a.hidden <= 0) return PKDA_ERR_SHAPE;
  if (a.dtype != PKDA_BF16 && a.dtype != PKDA_F32) return PKDA_ERR_DTYPE;
  p.rows = a.rows; p.heads = a.heads; p.hidden = a.hidden; p.total = 2 * a.hidden + 3 * a.heads;
  p.packed = a.packed; p.A_log = a.A_log_precond; p.dt_bias = a.dt_bias_precond;
  p.beta = a.beta; p.beta_atk = a.beta_atk; p.g_atk = a.g_atk;
  p.d_hidden0 = a.d_decay_hidden; p.d_beta = a.d_beta; p.d_beta_atk = a.d_beta_atk; p.d_hidden1 = a.d_gate_hidden;
  p.d_g_atk = a.d_g_atk; p.d_packed = a.d_packed; p.part = nullptr;
  return PKDA_OK;
}

static int ctrl_bwd_grid(const pkda_controls_args& a) {
  const long long want = (a.rows + 31) / 32;  // at least 32 rows per CTA
  return (int)(want < 1 ? 1 : (want < 1184 ? want : 1184));
}

int controls_fwd(const pkda_controls_args* a, cudaStream_t st) {
  CtrlParams p;
  if (int rc = ctrl_check(*a, p)) return rc;
  if (a->rows == 0) return PKDA_OK;
  if (!a->packed || !a->A_log_precond || !a->dt_bias_precond || !a->beta || !a->g_atk || !a->beta_atk)
    return PKDA_ERR_NULL;
  const long long n = a->rows * a->heads;
  const int grid = (int)((n + kCtrlThreads - 1) / kCtrlThreads < 2368 ? (n + kCtrlThreads - 1) / kCtrlThreads : 2368);
  begin_stage(kStageControlsFwd, st);
  if (a->dtype == PKDA_BF16) pkda_controls_fwd_kernel<bf16><<<grid, kCtrlThreads, 0, st>>>(p);
  else pkda_controls_fwd_kernel<float><<<grid, kCtrlThreads, 0, st>>>(p);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

size_t controls_bwd_workspace(const pkda_controls_args& a) {
  if (a.rows < 0 || a.heads <= 0) return 0;
  return align_up((size_t)ctrl_bwd_grid(a) * 2 * a.heads * sizeof(float));
}

int controls_bwd(const pkda_controls_args* a, cudaStream_t st) {
  CtrlParams p;
  if (int rc = ctrl_check(*a, p)) return rc;
  if (!a->dA_log_precond || !a->ddt_bias_precond) return PKDA_ERR_NULL;
  if (a->rows == 0) {
    const size_t nb = (size_t)a->heads * sizeof(float);
    return (cudaMemsetAsync(a->dA_log_precond, 0, nb, st) == cudaSuccess &&
            cudaMemsetAsync(a->ddt_bias_precond, 0, nb, st) == cudaSuccess) ? PKDA_OK : PKDA_ERR_LAUNCH;
  }
  if (!a->packed || !a->A_log_precond || !a->dt_bias_precond || !a->d_packed) return PKDA_ERR_NULL;
  if (!a->workspace || a->workspace_bytes < controls_bwd_workspace(*a)) return PKDA_ERR_WORKSPACE;
  p.part = static_cast<float*>(a->workspace);
  const int grid = ctrl_bwd_grid(*a);
  const size_t smem = (size_t)2 * a->heads * sizeof(float);
  begin_stage(kStageControlsBwd, st);
  if (a->dtype == PKDA_BF16) pkda_controls_bwd_kernel<bf16><<<grid, kCtrlThreads, smem, st>>>(p);
  else pkda_controls_bwd_kernel<float><<<grid, kCtrlThreads, smem, st>>>(p);
  end_stage(st);
  begin_stage(kStageControlsBwd, st);
  pkda_controls_reduce_kernel<<<(2 * a->heads + 127) / 128, 128, 0, st>>>(p.part, a->dA_log_precond, a->ddt_bias_precond,
                                                                         a->heads, grid);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

int pack_control_gradients(const pkda_pack_control_args* a, cudaStream_t st) {
  if (a->rows < 0) return PKDA_ERR_SHAPE;
  for (int i = 0; i < 5; ++i)
    if (a->sizes[i] < 0) return PKDA_ERR_SHAPE;
  if (a->dtype != PKDA_BF16 && a->dtype != PKDA_F32) return PKDA_ERR_DTYPE;
  const int total = a->sizes[0] + a->sizes[1] + a->sizes[2] + a->sizes[3] + a->sizes[4];
  const long long n = a->rows * total;
  if (n == 0) return PKDA_OK;
  if (!a->out) return PKDA_ERR_NULL;
  for (int i = 0; i < 5; ++i)
    if (a->sizes[i] > 0 && !a->grads[i]) return PKDA_ERR_NULL;
  const long long blocks = (n + kCtrlThreads - 1) / kCtrlThreads;
  const int grid = (int)(blocks < 4736 ? blocks : 4736);
  begin_stage(kStagePackControl, st);
  if (a->dtype == PKDA_BF16)
    pkda_pack_control_kernel<bf16><<<grid, kCtrlThreads, 0, st>>>(
        static_cast<const bf16*>(a->grads[0]), static_cast<const bf16*>(a->grads[1]), static_cast<const bf16*>(a->grads[2]),
        static_cast<const bf16*>(a->grads[3]), static_cast<const bf16*>(a->grads[4]), static_cast<bf16*>(a->out), a->rows,
        a->sizes[0], a->sizes[1], a->sizes[2], a->sizes[3], a->sizes[4]);
  else
    pkda_pack_control_kernel<float><<<grid, kCtrlThreads, 0, st>>>(
        static_cast<const float*>(a->grads[0]), static_cast<const float*>(a->grads[1]),
        static_cast<const float*>(a->grads[2]), static_cast<const float*>(a->grads[3]),
        static_cast<const float*>(a->grads[4]), static_cast<float*>(a->out), a->rows, a->sizes[0], a->sizes[1],
        a->sizes[2], a->sizes[3], a->sizes[4]);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
