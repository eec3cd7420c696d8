// Token-by-token PKDA recurrence: the decode step, short cached prefill, and
// the exact fp32 forward.  One CTA owns one (sequence, head) and keeps the
// whole D x D fp32 state in registers for all of its tokens, so a decode step
// moves the state through HBM exactly once in each direction (128-bit loads
// and stores, one full state row per warp request).
//
// Follows delta_feedback_experiment/pkda.py:390-410 literally:
//   A  <- exp(gP) A + bP k^2 ;  kw = k * precond_factor(A)
//   S  <- diag(exp(g)) S ;  e = v - S^T k ;  S <- S + (beta kw) e^T ;  o = S^T (scale q)
#include "pkda_common.cuh"
#include "pkda_launch.h"
#include "pkda_recurrent.cuh"

namespace pkda {

struct RecParams {
  Geo geo;
  const void *q, *k, *v, *g;
  const float* g_atk;
  const void *beta_atk, *beta;
  const float *A_log, *dt_bias, *log_atk_scale;
  const float *S0, *A0;
  void* o;
  float *ST, *AT;
  float *Sb, *Ab;  // optional checkpoints at every 64-token boundary: [chunks][H][D][D], [chunks][H][D]
  float scale, ln_x, eps;
};

// kCkpt: also store the states entering every 64-token chunk (first pass of the exact
// backward); a separate instantiation so that the decode kernel keeps its register budget
// (two CTAs per SM at D = 128).
template <int D, typename T, bool kCkpt>
__global__ void __launch_bounds__(RecCfg<D>::kThreads, D == 128 ? 2 : 1)
pkda_recurrent_kernel(const RecParams p) {
  using Cfg = RecCfg<D>;
  constexpr int VQ = Cfg::kVQ, KW = Cfg::kKW, R = Cfg::kR;
  const int tid = threadIdx.x;
  const int n = blockIdx.x / p.geo.heads;
  const int h = blockIdx.x - n * p.geo.heads;
  const SeqInfo sq = seq_info(p.geo, n);
  const int H = p.geo.heads;

  __shared__ float s_k[D], s_wk[D], s_q[D], s_al[D];
  __shared__ __align__(16) float s_v[D];
  __shared__ __align__(16) float s_red[2][KW][D];

  const bool active = tid < Cfg::kActive;
  const int kq = tid / VQ, vq = tid - kq * VQ;
  const int krow0 = kq * R;

  float4 S[R];
  const size_t sbase = ((size_t)n * H + h) * D * D;
  if (active) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (p.S0) S[r] = *reinterpret_cast<const float4*>(p.S0 + sbase + (size_t)(krow0 + r) * D + 4 * vq);
      else S[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // per-channel persistent values (threads tid < D)
  float A = 0.f, bias = 0.f;
  const float ea = expf(p.A_log[h]);
  const float centre = p.log_atk_scale[h];
  if (tid < D) {
    A = p.A0 ? p.A0[((size_t)n * H + h) * D + tid] : 0.f;
    bias = p.dt_bias[h * D + tid];
  }
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const T* g = static_cast<const T*>(p.g);
  const T* bA = static_cast<const T*>(p.beta_atk);
  const T* bW = static_cast<const T*>(p.beta);
  T* o = static_cast<T*>(p.o);

  for (int t = 0; t < sq.len; ++t) {
    if (kCkpt && (t & (kChunk - 1)) == 0) {  // checkpoint the state entering this chunk
      const size_t chh = (size_t)(sq.chunk0 + t / kChunk) * H + h;
      if (active) {
#pragma unroll
        for (int r = 0; r < R; ++r)
          *reinterpret_cast<float4*>(p.Sb + chh * D * D + (size_t)(krow0 + r) * D + 4 * vq) = S[r];
      }
      if (tid < D) p.Ab[chh * D + tid] = A;
    }
    const size_t tok = (size_t)(sq.bos + t);
    const size_t sidx = tok * H + h;
    if (tid < D) {
      const size_t idx = sidx * D + tid;
      const float kc = to_f(k[idx]);
      const float pd = expf(p.g_atk[sidx]);
      A = pd * A + to_f(bA[sidx]) * kc * kc;
      const float kw = kc * precond_factor(A, p.eps, centre, p.ln_x);
      s_k[tid] = kc;
      s_wk[tid] = to_f(bW[sidx]) * kw;
      s_q[tid] = to_f(q[idx]) * p.scale;
      s_al[tid] = expf(-ea * softplus_acc(to_f(g[idx]) + bias));
      s_v[tid] = to_f(v[idx]);
    }
    __syncthreads();
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
      const bool last = p.ST && t == sq.len - 1;  // final state rows leave as soon as they are final
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float wk = s_wk[krow0 + r], qq = s_q[krow0 + r];
        S[r].x += wk * e.x; S[r].y += wk * e.y; S[r].z += wk * e.z; S[r].w += wk * e.w;
        acc.x += S[r].x * qq; acc.y += S[r].y * qq; acc.z += S[r].z * qq; acc.w += S[r].w * qq;
        if (last) *reinterpret_cast<float4*>(p.ST + sbase + (size_t)(krow0 + r) * D + 4 * vq) = S[r];
      }
      *reinterpret_cast<float4*>(&s_red[1][kq][4 * vq]) = acc;
    }
    __syncthreads();
    if (tid < D) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < KW; ++w) sum += s_red[1][w][tid];
      o[sidx * D + tid] = from_f<T>(sum);
    }
  }
  if (p.ST && active && sq.len == 0) {  // no token: the state passes through
#pragma unroll
    for (int r = 0; r < R; ++r)
      *reinterpret_cast<float4*>(p.ST + sbase + (size_t)(krow0 + r) * D + 4 * vq) = S[r];
  }
  if (p.AT && tid < D) p.AT[((size_t)n * H + h) * D + tid] = A;
}

template <int D, typename T>
static int launch_rec(const RecParams& rp, cudaStream_t st) {
  const bool ckpt = rp.Sb != nullptr;
  dim3 grid(rp.geo.n_seqs * rp.geo.heads), block(RecCfg<D>::kThreads);
  begin_stage(kStageRecurrent, st);
  if (ckpt) pkda_recurrent_kernel<D, T, true><<<grid, block, 0, st>>>(rp);
  else pkda_recurrent_kernel<D, T, false><<<grid, block, 0, st>>>(rp);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

template <typename T>
static int dispatch_rec(int D, const RecParams& rp, cudaStream_t st) {
  switch (D) {
    case 8: return launch_rec<8, T>(rp, st);
    case 16: return launch_rec<16, T>(rp, st);
    case 32: return launch_rec<32, T>(rp, st);
    case 64: return launch_rec<64, T>(rp, st);
    case 128: return launch_rec<128, T>(rp, st);
    default: return PKDA_ERR_SHAPE;
  }
}

int recurrent_fwd(const pkda_recurrent_args* a, cudaStream_t st) {
  const pkda_problem& p = a->p;
  int rc = check_problem(p);
  if (rc != PKDA_OK) return rc;
  if (p.n_seqs == 0 || p.total_tokens == 0) return PKDA_OK;
  if (!a->o) return PKDA_ERR_NULL;
  // One token per sequence on a cached state: the decode-step kernel (all loads of the step issued
  // up front), without its convolution and gate stages.
  if (!p.cu_seqlens && p.seq_len == 1 && p.initial_state && a->final_state &&
      (p.dtype == PKDA_BF16 || p.dtype == PKDA_F32))
    return decode_direct(p, a->o, a->final_state, a->final_A_state, st);
  RecParams rp;
  rp.geo = make_geo(p, nullptr);
  rp.q = p.q; rp.k = p.k; rp.v = p.v; rp.g = p.g; rp.g_atk = p.g_atk;
  rp.beta_atk = p.beta_atk; rp.beta = p.beta;
  rp.A_log = p.A_log; rp.dt_bias = p.dt_bias; rp.log_atk_scale = p.log_atk_scale;
  rp.S0 = p.initial_state; rp.A0 = p.initial_A_state;
  rp.o = a->o; rp.ST = a->final_state; rp.AT = a->final_A_state; rp.Sb = nullptr; rp.Ab = nullptr;
  rp.scale = p.scale; rp.ln_x = logf(p.squash_x); rp.eps = p.squash_eps;
  if (p.dtype == PKDA_BF16) return dispatch_rec<bf16>(p.head_dim, rp, st);
  if (p.dtype == PKDA_F32) return dispatch_rec<float>(p.head_dim, rp, st);
  return PKDA_ERR_DTYPE;
}

// Forward pass that also leaves the states at every chunk boundary (first pass of
// the exact backward).
int recurrent_fwd_checkpointed(const pkda_problem& p, const int* chunk_offsets, void* o_scratch, float* Sb,
                               float* Ab, cudaStream_t st) {
  RecParams rp;
  rp.geo = make_geo(p, chunk_offsets);
  rp.q = p.q; rp.k = p.k; rp.v = p.v; rp.g = p.g; rp.g_atk = p.g_atk;
  rp.beta_atk = p.beta_atk; rp.beta = p.beta;
  rp.A_log = p.A_log; rp.dt_bias = p.dt_bias; rp.log_atk_scale = p.log_atk_scale;
  rp.S0 = p.initial_state; rp.A0 = p.initial_A_state;
  rp.o = o_scratch; rp.ST = nullptr; rp.AT = nullptr; rp.Sb = Sb; rp.Ab = Ab;
  rp.scale = p.scale; rp.ln_x = logf(p.squash_x); rp.eps = p.squash_eps;
  if (p.dtype == PKDA_BF16) return dispatch_rec<bf16>(p.head_dim, rp, st);
  if (p.dtype == PKDA_F32) return dispatch_rec<float>(p.head_dim, rp, st);
  return PKDA_ERR_DTYPE;
}

}  // namespace pkda
