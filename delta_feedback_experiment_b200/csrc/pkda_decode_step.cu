// One cached decoding step of the PKDA layer's token mixer in ONE launch:
//   Q|K|V short convolution over the cached projection history (+ SiLU, per-head
//   L2 norm of Q and K)  ->  one step of the recurrence on the cached state  ->
//   per-head RMS norm x sigmoid output gate,
// with the convolution histories, the matrix state S and the preconditioner
// state A updated in place.  It replaces, for T = 1, the reference's sequence of
// pkda_qkv_conv on the history-prefixed rows (delta_feedback_experiment/pkda.py:239-288),
// fused_recurrent_precond_kda (pkda.py:473-474) and pkda_norm_gate (pkda.py:539-541),
// and the cache bookkeeping around them (model.py:775-787): no torch.cat of the
// history, no clone of the new history, no q/k/v/o round trips through HBM.
//
// One CTA owns one (row, head) and keeps the D x D fp32 state in registers, so the
// step still moves the state through HBM exactly once in each direction; everything
// else the step touches is about 3 % of that.
#include "pkda_common.cuh"
#include "pkda_launch.h"
#include "pkda_recurrent.cuh"

namespace pkda {

struct DecodeParams {
  int batch, heads, taps;
  float scale, ln_x, eps, qk_eps, norm_eps;
  const void* qkv;
  void* conv[3];
  const float* conv_w;
  const void* g;
  const float* g_atk;
  const void *beta_atk, *beta;
  const float *A_log, *dt_bias, *log_atk_scale;
  float *S, *A;          // states read here ...
  float *S_out, *A_out;  // ... and written here (the same arrays when the cache is updated in place)
  const void *q, *k, *v; // direct mode (qkv == nullptr): q, k, v [batch][heads][D] given, no convolution
  const void* gate;
  const float* norm_w;
  void* out;
};

template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f(from_f<T>(x)); }

template <int D, typename T>
__global__ void __launch_bounds__(RecCfg<D>::kThreads, D == 128 ? 2 : 1)
pkda_decode_step_kernel(const DecodeParams p) {
  using Cfg = RecCfg<D>;
  constexpr int VQ = Cfg::kVQ, KW = Cfg::kKW, R = Cfg::kR, kThreads = Cfg::kThreads;
  constexpr int kWarps = kThreads / 32;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.heads;
  const int n = blockIdx.x / H, h = blockIdx.x - n * H;
  const int W = H * D;

  __shared__ float s_qkv[3][D];  // silu(conv) of q, k, v; then q, k normalised and rounded
  __shared__ float s_k[D], s_wk[D], s_q[D], s_al[D];
  __shared__ __align__(16) float s_v[D];
  __shared__ __align__(16) float s_red[2][KW][D];
  __shared__ float s_stat[kWarps + 2];

  const bool active = tid < Cfg::kActive;
  const int kq = tid / VQ, vq = tid - kq * VQ;
  const int krow0 = kq * R;

  // ---- the state first: its loads are the step's memory time
  float4 S[R];
  const size_t sbase = ((size_t)n * H + h) * D * D;
  if (active) {
#pragma unroll
    for (int r = 0; r < R; ++r)
      S[r] = *reinterpret_cast<const float4*>(p.S + sbase + (size_t)(krow0 + r) * D + 4 * vq);
  }

  // ---- every other global read of the step is issued now as well, so that the step pays one
  // memory round trip, not one per stage
  const T* qkv = static_cast<const T*>(p.qkv) + (size_t)n * 3 * W;
  const int hist = p.taps - 1;
  const bool with_conv = p.qkv != nullptr;
  constexpr int kItems = (3 * D + kThreads - 1) / kThreads;  // (slab, channel) items per thread
  T xn[kItems], hv[kItems][3];
  float wv[kItems][4];
#pragma unroll
  for (int it = 0; it < kItems; ++it) {
    const int item = tid + it * kThreads;
    if (with_conv && item < 3 * D) {
      const int slab = item / D, d = item - slab * D, cs = h * D + d;
      const float* w = p.conv_w + (size_t)(slab * W + cs) * p.taps;
      const T* hs = static_cast<const T*>(p.conv[slab]) + ((size_t)n * W + cs) * hist;
      xn[it] = qkv[slab * W + cs];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        if (j < hist) { hv[it][j] = hs[j]; wv[it][j] = w[j]; }
      }
      wv[it][3] = w[hist];
    }
  }
  const size_t sidx = (size_t)n * H + h;
  const float ea = expf(p.A_log[h]);
  const float centre = p.log_atk_scale[h];
  float A = 0.f, r_pd = 0.f, r_ba = 0.f, r_b = 0.f, r_g = 0.f, r_bias = 0.f, r_gate = 0.f, r_nw = 0.f;
  float d_q = 0.f, d_k = 0.f, d_v = 0.f;
  const bool direct = p.qkv == nullptr;
  if (tid < D) {
    if (direct) {
      d_q = to_f(static_cast<const T*>(p.q)[sidx * D + tid]);
      d_k = to_f(static_cast<const T*>(p.k)[sidx * D + tid]);
      d_v = to_f(static_cast<const T*>(p.v)[sidx * D + tid]);
    }
    A = p.A ? p.A[sidx * D + tid] : 0.f;
    r_pd = p.g_atk[sidx];
    r_ba = to_f(static_cast<const T*>(p.beta_atk)[sidx]);
    r_b = to_f(static_cast<const T*>(p.beta)[sidx]);
    r_g = to_f(static_cast<const T*>(p.g)[sidx * D + tid]);
    r_bias = p.dt_bias[h * D + tid];
    if (p.gate) {
      r_gate = to_f(static_cast<const T*>(p.gate)[sidx * D + tid]);
      r_nw = p.norm_w[tid];
    }
  }

  // ---- convolution over the cached history, SiLU; the history moves up by one token
  if (with_conv) {
#pragma unroll
  for (int it = 0; it < kItems; ++it) {
    const int item = tid + it * kThreads;
    if (item < 3 * D) {
      const int slab = item / D, d = item - slab * D, cs = h * D + d;
      T* hs = static_cast<T*>(p.conv[slab]) + ((size_t)n * W + cs) * hist;
      float y = wv[it][3] * to_f(xn[it]);
#pragma unroll
      for (int j = 0; j < 3; ++j)
        if (j < hist) y += wv[it][j] * to_f(hv[it][j]);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (j + 1 < hist) hs[j] = hv[it][j + 1];
      if (hist > 0) hs[hist - 1] = xn[it];
      s_qkv[slab][d] = y / (1.f + expf(-y));
    }
  }
  __syncthreads();
  // ---- per-head L2 norm of q (warp 0) and k (warp 1); q, k, v rounded to the activation type,
  // as the separate operators hand them over
  if (warp < 2) {
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss += s_qkv[warp][d] * s_qkv[warp][d];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_stat[kWarps + warp] = rsqrtf(ss + p.qk_eps);
  }
  __syncthreads();
  }  // with_conv

  if (tid < D) {
    const float qn = direct ? d_q : round_to<T>(s_qkv[0][tid] * s_stat[kWarps + 0]);
    const float kc = direct ? d_k : round_to<T>(s_qkv[1][tid] * s_stat[kWarps + 1]);
    const float vv = direct ? d_v : round_to<T>(s_qkv[2][tid]);
    A = expf(r_pd) * A + r_ba * kc * kc;
    const float kw = kc * precond_factor(A, p.eps, centre, p.ln_x);
    s_k[tid] = kc;
    s_wk[tid] = r_b * kw;
    s_q[tid] = qn * p.scale;
    s_al[tid] = expf(-ea * softplus_acc(r_g + r_bias));
    s_v[tid] = vv;
  }
  __syncthreads();
  // ---- S <- diag(exp g) S ;  e = v - S^T k ;  S <- S + (beta kw) e^T ;  o = S^T (scale q)
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (active) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float al = s_al[krow0 + r], kk = s_k[krow0 + r];
      S[r].x *= al; S[r].y *= al; S[r].z *= al; S[r].w *= al;
      acc.x += S[r].x * kk; acc.y += S[r].y * kk; acc.z += S[r].z * kk; acc.w += S[r].w * kk;
    }
    *reinterpret_cast<float4*>(&s_red[0][kq][4 * vq]) = acc;
  }
  __syncthreads();
  if (active) {
    float4 e = *reinterpret_cast<const float4*>(&s_v[4 * vq]);
#pragma unroll
    for (int w = 0; w < KW; ++w) {
      const float4 pr = *reinterpret_cast<const float4*>(&s_red[0][w][4 * vq]);
      e.x -= pr.x; e.y -= pr.y; e.z -= pr.z; e.w -= pr.w;
    }
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float wk = s_wk[krow0 + r], qq = s_q[krow0 + r];
      S[r].x += wk * e.x; S[r].y += wk * e.y; S[r].z += wk * e.z; S[r].w += wk * e.w;
      acc.x += S[r].x * qq; acc.y += S[r].y * qq; acc.z += S[r].z * qq; acc.w += S[r].w * qq;
      *reinterpret_cast<float4*>(p.S_out + sbase + (size_t)(krow0 + r) * D + 4 * vq) = S[r];
    }
    *reinterpret_cast<float4*>(&s_red[1][kq][4 * vq]) = acc;
  }
  __syncthreads();
  // ---- o, then RMS norm x weight x sigmoid(gate)
  float o = 0.f;
  if (tid < D) {
#pragma unroll
    for (int w = 0; w < KW; ++w) o += s_red[1][w][tid];
    o = round_to<T>(o);
    if (p.A_out) p.A_out[sidx * D + tid] = A;
  }
  T* out = static_cast<T*>(p.out) + sidx * D;
  if (!p.gate) {
    if (tid < D) out[tid] = from_f<T>(o);
    return;
  }
  float sq = (tid < D) ? o * o : 0.f;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
  if (lane == 0) s_stat[warp] = sq;
  __syncthreads();
  if (tid < D) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) tot += s_stat[w];
    const float rstd = rsqrtf(tot / (float)D + p.norm_eps);
    out[tid] = from_f<T>(o * rstd * r_nw / (1.f + expf(-r_gate)));
  }
}

template <int D, typename T>
static int launch_decode(const DecodeParams& dp, int stage, cudaStream_t st) {
  begin_stage(stage, st);
  pkda_decode_step_kernel<D, T><<<dp.batch * dp.heads, RecCfg<D>::kThreads, 0, st>>>(dp);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

template <typename T>
static int dispatch_decode(int D, const DecodeParams& dp, int stage, cudaStream_t st) {
  switch (D) {
    case 8: return launch_decode<8, T>(dp, stage, st);
    case 16: return launch_decode<16, T>(dp, stage, st);
    case 32: return launch_decode<32, T>(dp, stage, st);
    case 64: return launch_decode<64, T>(dp, stage, st);
    case 128: return launch_decode<128, T>(dp, stage, st);
    default: return PKDA_ERR_SHAPE;
  }
}

int decode_step(const pkda_decode_step_args* a, cudaStream_t st) {
  if (a->batch < 0 || a->heads <= 0 || a->taps < 1 || a->taps > 4) return PKDA_ERR_SHAPE;
  if (a->dtype != PKDA_BF16 && a->dtype != PKDA_F32) return PKDA_ERR_DTYPE;
  if (a->batch == 0) return PKDA_OK;
  if (!a->qkv || !a->conv_weight || !a->g || !a->g_atk || !a->beta_atk || !a->beta || !a->A_log || !a->dt_bias ||
      !a->log_atk_scale || !a->state || !a->a_state || !a->out)
    return PKDA_ERR_NULL;
  if (a->taps > 1 && (!a->conv_q || !a->conv_k || !a->conv_v)) return PKDA_ERR_NULL;
  if (a->gate && !a->norm_weight) return PKDA_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(a->state) & 15) return PKDA_ERR_ALIGN;
  DecodeParams dp;
  dp.batch = a->batch; dp.heads = a->heads; dp.taps = a->taps;
  dp.scale = a->scale; dp.ln_x = logf(a->squash_x); dp.eps = a->squash_eps; dp.qk_eps = a->qk_eps;
  dp.norm_eps = a->norm_eps;
  dp.qkv = a->qkv; dp.conv[0] = a->conv_q; dp.conv[1] = a->conv_k; dp.conv[2] = a->conv_v;
  dp.conv_w = a->conv_weight; dp.g = a->g; dp.g_atk = a->g_atk; dp.beta_atk = a->beta_atk; dp.beta = a->beta;
  dp.A_log = a->A_log; dp.dt_bias = a->dt_bias; dp.log_atk_scale = a->log_atk_scale;
  dp.S = a->state; dp.A = a->a_state; dp.S_out = a->state; dp.A_out = a->a_state;
  dp.q = dp.k = dp.v = nullptr; dp.gate = a->gate; dp.norm_w = a->norm_weight; dp.out = a->out;
  if (a->dtype == PKDA_BF16) return dispatch_decode<bf16>(a->head_dim, dp, kStageDecodeStep, st);
  return dispatch_decode<float>(a->head_dim, dp, kStageDecodeStep, st);
}

// The plain single-token step of pkda_recurrent_fwd (q, k, v given, cached state in, new state
// out) through the same kernel: no convolution, no norm gate.
int decode_direct(const pkda_problem& p, void* o, float* final_state, float* final_A_state, cudaStream_t st) {
  DecodeParams dp;
  dp.batch = p.n_seqs; dp.heads = p.heads; dp.taps = 1;
  dp.scale = p.scale; dp.ln_x = logf(p.squash_x); dp.eps = p.squash_eps; dp.qk_eps = 0.f; dp.norm_eps = 0.f;
  dp.qkv = nullptr; dp.conv[0] = dp.conv[1] = dp.conv[2] = nullptr; dp.conv_w = nullptr;
  dp.g = p.g; dp.g_atk = p.g_atk; dp.beta_atk = p.beta_atk; dp.beta = p.beta;
  dp.A_log = p.A_log; dp.dt_bias = p.dt_bias; dp.log_atk_scale = p.log_atk_scale;
  dp.S = const_cast<float*>(p.initial_state); dp.A = const_cast<float*>(p.initial_A_state);
  dp.S_out = final_state; dp.A_out = final_A_state;
  dp.q = p.q; dp.k = p.k; dp.v = p.v; dp.gate = nullptr; dp.norm_w = nullptr; dp.out = o;
  if (p.dtype == PKDA_BF16) return dispatch_decode<bf16>(p.head_dim, dp, kStageRecurrent, st);
  return dispatch_decode<float>(p.head_dim, dp, kStageRecurrent, st);
}

}  // namespace pkda
