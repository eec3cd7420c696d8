// Exact (fp32) backward of the token-by-token recurrence, for fp32 activations
// and for head widths the chunked kernels do not cover.  One CTA owns one
// (sequence, head).  A first pass (the forward kernel) leaves the states S, A at
// every 64-token boundary; this kernel walks the chunks last to first, replays
// each chunk forward from its checkpoint while parking the 64 per-token states in
// global scratch, then walks its tokens backwards with the state cotangent dS in
// registers:
//   o = S^T qs            ->  dqs = S do,            dS += qs do^T
//   S = S' + w e^T        ->  dw = dS e,  de = dS^T w
//   e = v - S'^T k        ->  dv = de,   dS' = dS - k de^T,  dk_read = -S' de
//   S' = diag(exp g) S_-  ->  dg = rowsum(dS' * S'),  dS_- = exp(g) dS'
// (S' = S - w e^T is rebuilt from S, so no division by the decay is needed),
// followed per token by the write-key / preconditioner / gate chain rule.
#include "pkda_common.cuh"
#include "pkda_launch.h"
#include "pkda_recurrent.cuh"

namespace pkda {

struct RecBwdParams {
  Geo geo;
  const void *q, *k, *v, *g;
  const float* g_atk;
  const void *beta_atk, *beta;
  const float *A_log, *dt_bias, *log_atk_scale;
  const float *Sb, *Ab;        // checkpoints [chunks][H][D][D], [chunks][H][D]
  const void* d_o;
  const float* dST;
  float* St;                   // scratch [N*H][64][D][D]
  void *dq, *dk, *dv, *dg, *dbeta_atk, *dbeta;
  float* dg_atk;
  float *partA, *partB, *partC;  // per (sequence, head): [N*H], [N*H][D], [N*H]
  float *dS0, *dA0;
  float scale, ln_x, eps;
};

template <int D>
__host__ __device__ constexpr int rec_bwd_smem_floats() {
  return 2 * kChunk * D + D + 10 * D + 2 * RecCfg<D>::kKW * D + kChunk * 2;
}

// Sum over the kVQ lanes that share a state row (consecutive lanes of one warp).
template <int VQ>
__device__ __forceinline__ float row_sum(float x) {
#pragma unroll
  for (int o = VQ / 2; o >= 1; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <int D, typename T>
__global__ void __launch_bounds__(RecCfg<D>::kThreads)
pkda_recurrent_bwd_kernel(const RecBwdParams p) {
  using Cfg = RecCfg<D>;
  constexpr int VQ = Cfg::kVQ, KW = Cfg::kKW, R = Cfg::kR;
  extern __shared__ __align__(16) float sm[];
  float* s_e = sm;                        // [64][D] residuals e_t
  float* s_A = s_e + kChunk * D;          // [65][D] preconditioner state before token t (row 64: after the chunk)
  float* s_k = s_A + (kChunk + 1) * D;    // per-token vectors
  float* s_w = s_k + D;
  float* s_q = s_w + D;
  float* s_al = s_q + D;
  float* s_v = s_al + D;                  // v (forward) / do (backward)
  float* s_dqs = s_v + D;
  float* s_dw = s_dqs + D;
  float* s_dkr = s_dw + D;
  float* s_dgl = s_dkr + D;
  float* s_de = s_dgl + D;
  float* s_red = s_de + D;                // [2][KW][D]
  float* s_tok = s_red + 2 * KW * D;      // [64][2] per-token scalar gradients (d beta, d beta_atk / d g_atk)

  const int tid = threadIdx.x;
  const int n = blockIdx.x / p.geo.heads, h = blockIdx.x - n * p.geo.heads, H = p.geo.heads;
  const SeqInfo sq = seq_info(p.geo, n);
  const bool active = tid < Cfg::kActive;
  // Threads beyond kActive (D = 8 only) shadow a valid position so that every lane takes part
  // in the row-sum shuffles; all their stores are suppressed.
  const int kq = (tid / VQ) % KW, vq = tid % VQ, krow0 = kq * R;
  const size_t nh = (size_t)n * H + h;
  float4* St = reinterpret_cast<float4*>(p.St + nh * kChunk * D * D);

  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const T* g = static_cast<const T*>(p.g);
  const T* bA = static_cast<const T*>(p.beta_atk);
  const T* bW = static_cast<const T*>(p.beta);
  const T* d_o = static_cast<const T*>(p.d_o);
  const float ea = expf(p.A_log[h]);
  const float centre = p.log_atk_scale[h];
  const float bias = tid < D ? p.dt_bias[h * D + tid] : 0.f;

  float4 dS[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    dS[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active && p.dST) dS[r] = *reinterpret_cast<const float4*>(p.dST + nh * D * D + (size_t)(krow0 + r) * D + 4 * vq);
  }
  float lam = 0.f;                  // dL/dA carried backwards (threads tid < D)
  float accA = 0.f, accB = 0.f, accC = 0.f;  // per-thread partials of dA_log, ddt_bias[tid], dlog_atk_scale

  for (int c = sq.nchunks - 1; c >= 0; --c) {
    const int t0 = c * kChunk, nt = min(kChunk, sq.len - t0);
    const size_t chh = (size_t)(sq.chunk0 + c) * H + h;
    // ---------------- replay the chunk forward from its checkpoint
    float4 S[R];
    if (active) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        S[r] = *reinterpret_cast<const float4*>(p.Sb + chh * D * D + (size_t)(krow0 + r) * D + 4 * vq);
    }
    float A = tid < D ? p.Ab[chh * D + tid] : 0.f;
    for (int t = 0; t < nt; ++t) {
      const size_t sidx = (size_t)(sq.bos + t0 + t) * H + h;
      if (tid < D) {
        const size_t idx = sidx * D + tid;
        const float kc = to_f(k[idx]);
        s_A[t * D + tid] = A;
        A = expf(p.g_atk[sidx]) * A + to_f(bA[sidx]) * kc * kc;
        s_k[tid] = kc;
        s_w[tid] = to_f(bW[sidx]) * kc * precond_factor(A, p.eps, centre, p.ln_x);
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
        *reinterpret_cast<float4*>(&s_red[kq * D + 4 * vq]) = acc;
      }
      __syncthreads();
      if (active) {
        float4 e = *reinterpret_cast<const float4*>(&s_v[4 * vq]);
#pragma unroll
        for (int w = 0; w < KW; ++w) {
          const float4 pr = *reinterpret_cast<const float4*>(&s_red[w * D + 4 * vq]);
          e.x -= pr.x; e.y -= pr.y; e.z -= pr.z; e.w -= pr.w;
        }
        if (kq == 0) *reinterpret_cast<float4*>(&s_e[t * D + 4 * vq]) = e;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float wk = s_w[krow0 + r];
          S[r].x += wk * e.x; S[r].y += wk * e.y; S[r].z += wk * e.z; S[r].w += wk * e.w;
          St[((size_t)t * D + krow0 + r) * (D / 4) + vq] = S[r];
        }
      }
      __syncthreads();
    }
    if (tid < D) s_A[nt * D + tid] = A;
    __syncthreads();
    // ---------------- walk the chunk backwards
    for (int t = nt - 1; t >= 0; --t) {
      const size_t sidx = (size_t)(sq.bos + t0 + t) * H + h;
      float kc = 0.f, rawz = 0.f, Bf = 0.f, An = 0.f, Ap = 0.f, dec = 0.f, bp = 0.f, bw = 0.f, dev = 0.f;
      if (tid < D) {
        const size_t idx = sidx * D + tid;
        kc = to_f(k[idx]);
        Ap = s_A[t * D + tid];
        An = s_A[(t + 1) * D + tid];
        dec = expf(p.g_atk[sidx]);
        bp = to_f(bA[sidx]);
        bw = to_f(bW[sidx]);
        dev = logf(An + p.eps) - centre;
        Bf = expf(-p.ln_x * dev / (1.f + fabsf(dev)));
        rawz = to_f(g[idx]) + bias;
        s_k[tid] = kc;
        s_w[tid] = bw * kc * Bf;
        s_q[tid] = to_f(q[idx]) * p.scale;
        s_al[tid] = expf(-ea * softplus_acc(rawz));
        s_v[tid] = to_f(d_o[idx]);
      }
      __syncthreads();
      float4 de = make_float4(0.f, 0.f, 0.f, 0.f);
      {
        const float4 dov = *reinterpret_cast<const float4*>(&s_v[4 * vq]);
        const float4 ev = *reinterpret_cast<const float4*>(&s_e[t * D + 4 * vq]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float4 S4 = St[((size_t)t * D + krow0 + r) * (D / 4) + vq];
          const float qq = s_q[krow0 + r], wk = s_w[krow0 + r];
          // dqs[k] = sum_v S[k][v] do[v]
          const float dqs = row_sum<VQ>(S4.x * dov.x + S4.y * dov.y + S4.z * dov.z + S4.w * dov.w);
          dS[r].x += qq * dov.x; dS[r].y += qq * dov.y; dS[r].z += qq * dov.z; dS[r].w += qq * dov.w;
          const float dw = row_sum<VQ>(dS[r].x * ev.x + dS[r].y * ev.y + dS[r].z * ev.z + dS[r].w * ev.w);
          de.x += dS[r].x * wk; de.y += dS[r].y * wk; de.z += dS[r].z * wk; de.w += dS[r].w * wk;
          if (vq == 0 && active) { s_dqs[krow0 + r] = dqs; s_dw[krow0 + r] = dw; }
        }
        if (active) *reinterpret_cast<float4*>(&s_red[kq * D + 4 * vq]) = de;
      }
      __syncthreads();
      {
        de = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < KW; ++w) {
          const float4 pr = *reinterpret_cast<const float4*>(&s_red[w * D + 4 * vq]);
          de.x += pr.x; de.y += pr.y; de.z += pr.z; de.w += pr.w;
        }
        if (kq == 0 && active) *reinterpret_cast<float4*>(&s_de[4 * vq]) = de;
        const float4 ev = *reinterpret_cast<const float4*>(&s_e[t * D + 4 * vq]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float4 S4 = St[((size_t)t * D + krow0 + r) * (D / 4) + vq];
          const float wk = s_w[krow0 + r], kk = s_k[krow0 + r], al = s_al[krow0 + r];
          float4 Sp;  // S' = S - w e^T
          Sp.x = S4.x - wk * ev.x; Sp.y = S4.y - wk * ev.y; Sp.z = S4.z - wk * ev.z; Sp.w = S4.w - wk * ev.w;
          const float dkr = -row_sum<VQ>(Sp.x * de.x + Sp.y * de.y + Sp.z * de.z + Sp.w * de.w);
          dS[r].x -= kk * de.x; dS[r].y -= kk * de.y; dS[r].z -= kk * de.z; dS[r].w -= kk * de.w;
          const float dgl = row_sum<VQ>(dS[r].x * Sp.x + dS[r].y * Sp.y + dS[r].z * Sp.z + dS[r].w * Sp.w);
          dS[r].x *= al; dS[r].y *= al; dS[r].z *= al; dS[r].w *= al;
          if (vq == 0 && active) { s_dkr[krow0 + r] = dkr; s_dgl[krow0 + r] = dgl; }
        }
      }
      __syncthreads();
      // ---- per-channel chain rule (one thread per channel)
      float x_db = 0.f, x_dbp = 0.f, x_dgp = 0.f;
      if (tid < D) {
        const size_t idx = sidx * D + tid;
        const float kt = kc * Bf;
        const float dw = s_dw[tid];
        x_db = dw * kt;                       // d beta = <dw, kt>
        const float dkt = bw * dw;
        const float den = 1.f + fabsf(dev);
        const float ddev = -p.ln_x * dkt * kc * Bf / (den * den);
        accC -= ddev;
        lam += ddev / (An + p.eps);
        x_dbp = lam * kc * kc;
        x_dgp = lam * dec * Ap;
        const float dkv = s_dkr[tid] + dkt * Bf + 2.f * lam * bp * kc;
        lam *= dec;
        const float dgl = s_dgl[tid];
        const float gn = -ea * softplus_acc(rawz);
        const float dr = dgl * (-ea) / (1.f + expf(-rawz));
        accA += dgl * gn;
        accB += dr;
        static_cast<T*>(p.dq)[idx] = from_f<T>(s_dqs[tid] * p.scale);
        static_cast<T*>(p.dk)[idx] = from_f<T>(dkv);
        static_cast<T*>(p.dv)[idx] = from_f<T>(s_de[tid]);
        static_cast<T*>(p.dg)[idx] = from_f<T>(dr);
      }
      // three sums over the D channels (threads >= D contribute zero), fixed order
      s_red[tid] = x_db;
      s_red[Cfg::kThreads + tid] = x_dbp;
      s_red[2 * Cfg::kThreads + tid] = x_dgp;
      __syncthreads();
      if (tid < 3) {
        float s = 0.f;
        for (int j = 0; j < D; ++j) s += s_red[tid * Cfg::kThreads + j];
        if (tid == 0) static_cast<T*>(p.dbeta)[sidx] = from_f<T>(s);
        else if (tid == 1) static_cast<T*>(p.dbeta_atk)[sidx] = from_f<T>(s);
        else p.dg_atk[sidx] = s;
      }
      __syncthreads();
    }
  }
  if (p.dS0 && active) {
#pragma unroll
    for (int r = 0; r < R; ++r)
      *reinterpret_cast<float4*>(p.dS0 + nh * D * D + (size_t)(krow0 + r) * D + 4 * vq) = dS[r];
  }
  if (tid < D) {
    if (p.dA0) p.dA0[nh * D + tid] = lam;
    p.partB[nh * D + tid] = accB;
  }
  s_red[tid] = accA;
  s_red[Cfg::kThreads + tid] = accC;
  __syncthreads();
  if (tid < 2) {
    float s = 0.f;
    for (int j = 0; j < D; ++j) s += s_red[tid * Cfg::kThreads + j];
    (tid == 0 ? p.partA : p.partC)[nh] = s;
  }
}

// Sums the per-(sequence, head) partials over sequences: grid (H), D threads.
__global__ void pkda_recurrent_bwd_reduce_kernel(int n_seqs, int H, int D, const float* partA, const float* partB,
                                                 const float* partC, float* dA_log, float* ddt_bias, float* dcentre) {
  const int h = blockIdx.x, c = threadIdx.x;
  float b = 0.f;
  for (int n = 0; n < n_seqs; ++n) b += partB[((size_t)n * H + h) * D + c];
  ddt_bias[h * D + c] = b;
  if (c == 0) {
    float a = 0.f, cc = 0.f;
    for (int n = 0; n < n_seqs; ++n) { a += partA[(size_t)n * H + h]; cc += partC[(size_t)n * H + h]; }
    dA_log[h] = a;
    dcentre[h] = cc;
  }
}

struct RecBwdWorkspace {
  int* chunk_offsets;
  float *Sb, *Ab, *St, *partA, *partB, *partC;
  void* o_scratch;
  size_t bytes;
};

static RecBwdWorkspace carve_rec_bwd(const pkda_problem& p, void* base) {
  RecBwdWorkspace w;
  const size_t chunks = (size_t)chunk_bound(p), H = p.heads, D = p.head_dim, NH = (size_t)p.n_seqs * H;
  size_t off = 0;
  unsigned char* b = static_cast<unsigned char*>(base);
  auto take = [&](size_t bytes) { void* ptr = b + off; off += align_up(bytes); return ptr; };
  w.chunk_offsets = static_cast<int*>(take((size_t)(p.n_seqs + 1) * sizeof(int)));
  w.Sb = static_cast<float*>(take(chunks * H * D * D * 4));
  w.Ab = static_cast<float*>(take(chunks * H * D * 4));
  w.St = static_cast<float*>(take(NH * kChunk * D * D * 4));
  w.partA = static_cast<float*>(take(NH * 4));
  w.partB = static_cast<float*>(take(NH * D * 4));
  w.partC = static_cast<float*>(take(NH * 4));
  w.o_scratch = take((size_t)p.total_tokens * H * D * 4);
  w.bytes = off;
  return w;
}

size_t recurrent_bwd_workspace(const pkda_problem& p) { return carve_rec_bwd(p, nullptr).bytes; }

template <int D, typename T>
static int launch_rec_bwd(const RecBwdParams& bp, cudaStream_t st) {
  const int smem = rec_bwd_smem_floats<D>() * 4 + 3 * RecCfg<D>::kThreads * 4;
  if (!ensure_dynamic_smem(pkda_recurrent_bwd_kernel<D, T>, smem))
    return PKDA_ERR_LAUNCH;
  begin_stage(kStageRecurrent, st);
  pkda_recurrent_bwd_kernel<D, T><<<bp.geo.n_seqs * bp.geo.heads, RecCfg<D>::kThreads, smem, st>>>(bp);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

template <typename T>
static int dispatch_rec_bwd(int D, const RecBwdParams& bp, cudaStream_t st) {
  switch (D) {
    case 8: return launch_rec_bwd<8, T>(bp, st);
    case 16: return launch_rec_bwd<16, T>(bp, st);
    case 32: return launch_rec_bwd<32, T>(bp, st);
    case 64: return launch_rec_bwd<64, T>(bp, st);
    case 128: return launch_rec_bwd<128, T>(bp, st);
    default: return PKDA_ERR_SHAPE;
  }
}

__global__ void pkda_rec_chunk_offsets_kernel(const int* cu, int n_seqs, int* offs) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int acc = 0;
    offs[0] = 0;
    for (int n = 0; n < n_seqs; ++n) { acc += (cu[n + 1] - cu[n] + kChunk - 1) / kChunk; offs[n + 1] = acc; }
  }
}

int recurrent_bwd(const pkda_recurrent_bwd_args* a, cudaStream_t st) {
  const pkda_problem& p = a->p;
  int rc = check_problem(p);
  if (rc != PKDA_OK) return rc;
  if (p.n_seqs == 0 || p.total_tokens == 0) return PKDA_OK;
  if (!a->d_o || !a->dq || !a->dk || !a->dv || !a->dg || !a->dg_atk || !a->dbeta_atk || !a->dbeta || !a->dA_log ||
      !a->ddt_bias || !a->dlog_atk_scale)
    return PKDA_ERR_NULL;
  if (!a->workspace || a->workspace_bytes < recurrent_bwd_workspace(p)) return PKDA_ERR_WORKSPACE;
  RecBwdWorkspace ws = carve_rec_bwd(p, a->workspace);
  if (p.cu_seqlens) {
    begin_stage(kStageOffsets, st);
    pkda_rec_chunk_offsets_kernel<<<1, 32, 0, st>>>(p.cu_seqlens, p.n_seqs, ws.chunk_offsets);
    end_stage(st);
  }
  // pass 1: forward with checkpoints at every chunk boundary
  rc = recurrent_fwd_checkpointed(p, ws.chunk_offsets, ws.o_scratch, ws.Sb, ws.Ab, st);
  if (rc != PKDA_OK) return rc;
  RecBwdParams bp;
  bp.geo = make_geo(p, ws.chunk_offsets);
  bp.q = p.q; bp.k = p.k; bp.v = p.v; bp.g = p.g; bp.g_atk = p.g_atk; bp.beta_atk = p.beta_atk; bp.beta = p.beta;
  bp.A_log = p.A_log; bp.dt_bias = p.dt_bias; bp.log_atk_scale = p.log_atk_scale;
  bp.Sb = ws.Sb; bp.Ab = ws.Ab; bp.d_o = a->d_o; bp.dST = a->d_final_state; bp.St = ws.St;
  bp.dq = a->dq; bp.dk = a->dk; bp.dv = a->dv; bp.dg = a->dg; bp.dbeta_atk = a->dbeta_atk; bp.dbeta = a->dbeta;
  bp.dg_atk = a->dg_atk; bp.partA = ws.partA; bp.partB = ws.partB; bp.partC = ws.partC;
  bp.dS0 = a->d_initial_state; bp.dA0 = a->d_initial_A_state;
  bp.scale = p.scale; bp.ln_x = logf(p.squash_x); bp.eps = p.squash_eps;
  rc = p.dtype == PKDA_BF16 ? dispatch_rec_bwd<bf16>(p.head_dim, bp, st) : dispatch_rec_bwd<float>(p.head_dim, bp, st);
  if (rc != PKDA_OK) return rc;
  begin_stage(kStageParamReduce, st);
  pkda_recurrent_bwd_reduce_kernel<<<p.heads, p.head_dim, 0, st>>>(p.n_seqs, p.heads, p.head_dim, ws.partA, ws.partB,
                                                                  ws.partC, a->dA_log, a->ddt_bias, a->dlog_atk_scale);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

}  // namespace pkda
