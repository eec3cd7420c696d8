/*
 * pkda_b200 -- C ABI of the B200 (sm_100a) PKDA delta-rule attention kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * stream it is given, never synchronises, never allocates and returns an int
 * status (0 = ok).  Scratch memory is supplied by the caller, sized by the
 * *_workspace_bytes functions (the one exception is pkda_chunk_fwd_static, whose
 * scratch is an array inside the library).  The Python host code in
 * delta_feedback_experiment_b200/ binds these through ctypes; any other host
 * language binds them the same way.  Kernels run on the device that is current
 * when an entry point is called: the caller makes the tensors' device current.
 *
 * Device-side failures.  The tensor-core kernels wait on hardware barriers with
 * a bounded number of polls.  If such a wait ever gives up, the kernel records 1
 * in a 32-bit status word at the end of the call's workspace
 * (pkda_chunk_fwd_status_offset / pkda_chunk_bwd_status_offset bytes from its
 * start; pkda_static_status_ptr for the static-scratch entry point), and the
 * last kernel of the call overwrites part of the call's outputs (o; dq, dk,
 * dv) with NaN, so that a failed call cannot pass for a result: it reaches the
 * caller's non-finite check.  The return value of the entry point itself only
 * reports host-side errors (the call does not synchronise).
 *
 * Tensor conventions (identical to the reference operator boundary,
 * delta_feedback_experiment/fla_ops.py:255-349 and pkda.py:450-475):
 *   q,k,v,g        [tokens][H][D]   activations (bf16 or fp32), contiguous
 *   g_atk          [tokens][H]      fp32, preconditioner log-decay (<= 0)
 *   beta_atk,beta  [tokens][H]      activation dtype
 *   A_log [H], dt_bias [H*D], log_atk_scale [H]   fp32
 *   states         S [N][H][D][D] (key-major), A [N][H][D]   fp32
 * "tokens" is the flat axis B*T (dense) or the packed total; N is B (dense) or
 * the number of packed sequences.
 */
#ifndef PKDA_B200_H_
#define PKDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PKDA_ABI_VERSION 1
#define PKDA_CHUNK 64

enum pkda_status {
  PKDA_OK = 0,
  PKDA_ERR_NULL = 1,          /* a required pointer is NULL */
  PKDA_ERR_SHAPE = 2,         /* unsupported geometry (head_dim, sizes) */
  PKDA_ERR_DTYPE = 3,         /* unsupported activation dtype for this entry */
  PKDA_ERR_WORKSPACE = 4,     /* workspace missing or too small */
  PKDA_ERR_LAUNCH = 5,        /* a kernel launch failed (see cudaGetLastError) */
  PKDA_ERR_ALIGN = 6,         /* a pointer is not 16-byte aligned */
  PKDA_ERR_STATIC_LIMIT = 7   /* problem needs more scratch than the built-in static array holds */
};

enum pkda_dtype { PKDA_BF16 = 0, PKDA_F32 = 1 };

/* Geometry + inputs shared by all entry points. */
typedef struct pkda_problem {
  int32_t n_seqs;        /* N: batch rows, or packed sequences */
  int32_t seq_len;       /* T per row (dense); ignored when cu_seqlens != NULL */
  int32_t total_tokens;  /* N*T (dense) or packed total */
  int32_t heads;         /* H */
  int32_t head_dim;      /* D = K = V */
  int32_t dtype;         /* pkda_dtype of q,k,v,g,beta,beta_atk and of o / activation grads */
  float scale;           /* query scale (reference default D^-0.5, pkda.py:372) */
  float squash_x;        /* preconditioner base x (1.5, pkda.py:94) */
  float squash_eps;      /* preconditioner eps (1e-6, pkda.py:95) */
  int32_t reserved0;
  const int32_t* cu_seqlens; /* device int32 [N+1] cumulative offsets, or NULL (dense) */
  const void* q;
  const void* k;
  const void* v;
  const void* g;
  const float* g_atk;
  const void* beta_atk;
  const void* beta;
  const float* A_log;
  const float* dt_bias;
  const float* log_atk_scale;
  const float* initial_state;   /* [N][H][D][D] or NULL (zeros) */
  const float* initial_A_state; /* [N][H][D]    or NULL (zeros) */
} pkda_problem;

/*
 * Recurrent (token by token) forward: the decode step and short cached
 * prefill, exact in fp32.  Replaces fused_recurrent_precond_kda
 * (call site delta_feedback_experiment/pkda.py:473-474) and follows the
 * recurrence of pkda.py:390-410 literally.  Any T >= 1, D in {8,16,32,64,128},
 * bf16 or fp32 activations.  final_state may alias initial_state (in-place
 * decode); final_A_state may alias initial_A_state.
 */
typedef struct pkda_recurrent_args {
  pkda_problem p;
  void* o;               /* [tokens][H][D] activation dtype */
  float* final_state;    /* [N][H][D][D] or NULL */
  float* final_A_state;  /* [N][H][D] or NULL */
} pkda_recurrent_args;

int pkda_recurrent_fwd(const pkda_recurrent_args* args, void* cuda_stream);

/*
 * Exact backward of the recurrence (fp32 arithmetic throughout): the gradient
 * path for fp32 activations and for head widths other than 128, and an
 * independent check of the chunked backward.  Same gradients as
 * pkda_chunk_bwd (replaces the same reference code,
 * delta_feedback_experiment/fla_ops.py:423-499, and the autograd of
 * pkda.py:355-410); needs no saved intermediates: a checkpointed forward pass
 * runs first inside the call.  D in {8,16,32,64,128}, bf16 or fp32.
 */
typedef struct pkda_recurrent_bwd_args {
  pkda_problem p;
  const void* d_o;              /* [tokens][H][D] activation dtype */
  const float* d_final_state;   /* [N][H][D][D] or NULL */
  void* dq; void* dk; void* dv; void* dg;     /* activation dtype */
  float* dg_atk; void* dbeta_atk; void* dbeta;
  float* dA_log; float* ddt_bias; float* dlog_atk_scale;
  float* d_initial_state;    /* or NULL */
  float* d_initial_A_state;  /* or NULL */
  void* workspace; size_t workspace_bytes;
} pkda_recurrent_bwd_args;

size_t pkda_recurrent_bwd_workspace_bytes(const pkda_problem* p);
int pkda_recurrent_bwd(const pkda_recurrent_bwd_args* args, void* cuda_stream);

/*
 * Chunked forward (training / prefill), bf16 activations, D = 128, chunk 64.
 * Replaces kda_gate_chunk_cumsum + chunk_precond_kda_fwd
 * (delta_feedback_experiment/fla_ops.py:290-339) and chunk_precond_kda
 * (pkda.py:475).  Intermediates follow the shapes of
 * fla_ops.py:73-97 with "chunks" = the flat chunk axis (N*ceil(T/64) dense;
 * for packed input at most total_tokens/64 + N):
 *   Aqk, Akk        [tokens][H][64]      bf16
 *   k_precond       [tokens][H][D]       bf16
 *   ac_atk, a_atk   [chunks][H][D]       fp32
 *   sa_atk          [chunks][H]          fp32
 *   w, kg, v_new, qg [tokens][H][D]      bf16
 *   h               [chunks][H][D][D]    bf16
 * All of them must be supplied (the lean variant of the reference simply does
 * not keep the last five after the call).
 */
typedef struct pkda_chunk_fwd_args {
  pkda_problem p;
  void* o;
  float* final_state;   /* or NULL */
  float* final_A_state; /* or NULL */
  void* Aqk; void* Akk; void* k_precond;
  float* ac_atk; float* a_atk; float* sa_atk;
  void* w; void* kg; void* v_new; void* h; void* qg;
  void* workspace; size_t workspace_bytes;
} pkda_chunk_fwd_args;

size_t pkda_chunk_fwd_workspace_bytes(const pkda_problem* p);
int pkda_chunk_fwd(const pkda_chunk_fwd_args* args, void* cuda_stream);
/* Byte offset of the 32-bit device status word inside the forward workspace. */
size_t pkda_chunk_fwd_status_offset(const pkda_problem* p);

/*
 * pkda_chunk_fwd for hosts that cannot hand over scratch memory.  (No
 * counterpart in the reference, whose kernels always allocate through torch.)
 * Some embedders own every byte of device memory themselves and forbid the
 * code they call from allocating: a serving engine that sized its pools at
 * start-up, a plugin running inside another framework's execution callback
 * where cudaMalloc would stall the whole device, a hard real-time loop.  For
 * them this entry point runs exactly the same kernels as pkda_chunk_fwd but
 * takes its scratch from a fixed array of PKDA_STATIC_SCRATCH_BYTES that is part
 * of the library image (so every GPU that loads the library carries those
 * bytes until the process exits).  args->workspace / workspace_bytes are
 * ignored; inputs, outputs and the eleven intermediates are still the
 * caller's.  It calls no cudaMalloc/cudaFree and no allocating library routine.
 *
 *  - Limit: pkda_chunk_fwd_workspace_bytes(&args->p) must not exceed
 *    pkda_static_scratch_bytes() (16 MiB: about 60,000 (token, head) units,
 *    e.g. B*T = 3,840 tokens at H = 16); larger problems return
 *    PKDA_ERR_STATIC_LIMIT and launch nothing.
 *  - The first call on each device looks up the array's device address (with
 *    that device current).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps whatever the last
 *    call left; the kernels overwrite every byte they later read, so nothing
 *    needs clearing.  Two calls whose kernels overlap on the GPU (different
 *    streams, no ordering between them) race on it: serialise them.
 */
#define PKDA_STATIC_SCRATCH_BYTES (16u << 20)
size_t pkda_static_scratch_bytes(void);
int pkda_chunk_fwd_static(const pkda_chunk_fwd_args* args, void* cuda_stream);
/*
 * Device address (on the current device) of the status word the last
 * pkda_chunk_fwd_static call for problem p used.  Allocates nothing; like the
 * entry point itself, the first call on a device belongs outside stream capture.
 */
int pkda_static_status_ptr(const pkda_problem* p, const int32_t** device_ptr);

/*
 * Chunked backward.  Replaces kda_gate_chunk_cumsum + chunk_precond_kda_bwd +
 * kda_gate_bwd (delta_feedback_experiment/fla_ops.py:423-499).  Takes the
 * forward's intermediates (recompute = 1 rebuilds w, kg, v_new, h, qg into the
 * given buffers first, the reference's "lean" mode) and the cotangents d_o
 * (and optionally d_final_state); writes the ten input gradients
 * (dq,dk,dv,dg,dbeta,dbeta_atk in the activation dtype; dg_atk, dA_log,
 * ddt_bias, dlog_atk_scale fp32, as scripts/pkda_bench.py:197-201 requires)
 * and, when requested, the gradients of the two initial states.
 */
typedef struct pkda_chunk_bwd_args {
  pkda_problem p;
  const void* d_o;              /* [tokens][H][D] */
  const float* d_final_state;   /* [N][H][D][D] or NULL */
  int32_t recompute;            /* 1: rebuild w,kg,v_new,h,qg first */
  int32_t reserved1;
  const void* Aqk; const void* Akk; const void* k_precond;
  const float* ac_atk; const float* a_atk; const float* sa_atk;
  void* w; void* kg; void* v_new; void* h; void* qg;
  void* dq; void* dk; void* dv; void* dg;
  float* dg_atk; void* dbeta_atk; void* dbeta;
  float* dA_log; float* ddt_bias; float* dlog_atk_scale;
  float* d_initial_state;    /* [N][H][D][D] or NULL */
  float* d_initial_A_state;  /* [N][H][D] or NULL */
  void* workspace; size_t workspace_bytes;
} pkda_chunk_bwd_args;

size_t pkda_chunk_bwd_workspace_bytes(const pkda_problem* p);
int pkda_chunk_bwd(const pkda_chunk_bwd_args* args, void* cuda_stream);
/* Byte offset of the 32-bit device status word inside the backward workspace. */
size_t pkda_chunk_bwd_status_offset(const pkda_problem* p);

/* Introspection used by the bindings' self-checks. */
int pkda_abi_version(void);
const char* pkda_status_string(int status);
size_t pkda_sizeof_problem(void);
size_t pkda_sizeof_recurrent_args(void);
size_t pkda_sizeof_chunk_fwd_args(void);
size_t pkda_sizeof_chunk_bwd_args(void);
/* Number of kernels the last entry-point call enqueued (for launch accounting). */
int pkda_last_launch_count(void);

/*
 * Testing aid.  The chunked kernels pair tokens inside blocks of b rows through a
 * single reference row whenever the decay across the block is small enough, and
 * through a binary hierarchy of reference rows otherwise; b is chosen per
 * (chunk, head) from the data.  This caps b (a power of two in 1..64; 64 = no cap,
 * 1 = hierarchy only) so that tests can exercise every variant on the same input.
 */
int pkda_set_direct_block_cap(int cap);

/*
 * Testing aid.  Several stages exist in two implementations: the tcgen05 /
 * tensor-memory kernel that runs by default and an older mma.sync kernel that is
 * kept as a cross-check (and for shapes the default does not cover).
 * pkda_set_variant(stage name as pkda_stage_name reports it, 1) pins the older
 * kernel for that stage, (.., 0) restores the default.  Stages with two
 * implementations: "intra_fwd", "scan_fwd", "out_fwd", "scan_bwd", "intra_bwd".
 * "out_fwd" has three: by default the tcgen05 state scan produces the output
 * itself (no output launch), 2 runs the stand-alone tcgen05 output kernel, 1 the
 * mma.sync one.
 * Returns PKDA_ERR_SHAPE for any other name.  Process-wide; not thread-safe.
 */
int pkda_set_variant(const char* stage, int variant);

/*
 * Optional per-kernel timing for benchmarks.  pkda_stage_timing(1) makes every
 * later launch record a CUDA event pair on its stream (events come from a pool
 * that grows with cudaEventCreate; not for use under stream capture);
 * pkda_stage_timing_read waits for the recorded events, adds elapsed
 * milliseconds and launch counts per stage into ms[0..n) / counts[0..n) and
 * clears the records.  Stages are numbered 0 .. pkda_stage_count()-1.
 */
int pkda_stage_count(void);
const char* pkda_stage_name(int stage);
int pkda_stage_timing(int enable);
int pkda_stage_timing_read(float* ms, int* counts, int n_stages);

/* ------------------------------------------------------------------------
 * Neighbours of the recurrence inside the PKDA layer.
 *
 * pkda_qkv_conv_*  replace the custom ops delta_feedback::pkda_qkv_conv and
 * delta_feedback::pkda_qkv_conv_backward (delta_feedback_experiment/fla_ops.py:134-249;
 * portable definition delta_feedback_experiment/pkda.py:197-220 and :41-44): a
 * causal depthwise convolution of `taps` (1..4) taps over the concatenated Q|K|V
 * projection, SiLU, and a per-head L2 normalisation of the first `norm_channels`
 * channels, y = s * rsqrt(sum_head(s^2) + eps); outputs are three separate slabs.
 *   x       [batch][seq_len][channels]          channels = 3 * slab width
 *   weight  [channels][taps] fp32; tap j multiplies x[t - (taps-1) + j]
 *   q,k,v   [batch][seq_len][channels / 3]      activation dtype
 * Tokens before the start of a row read as zero (callers that continue a cached
 * row prepend the taps-1 previous projections as the reference does,
 * pkda.py:239-260).  head_dim must be a power of two in 8..128 and divide the slab
 * width; norm_channels must be a multiple of head_dim.
 */
typedef struct pkda_qkv_conv_args {
  int batch, seq_len, channels, taps, head_dim, norm_channels;
  int dtype;                 /* PKDA_BF16 or PKDA_F32: x, q, k, v and their gradients */
  float eps;
  const void* x;
  const float* weight;
  void *q, *k, *v;           /* forward outputs (unused by the backward) */
  const void *dq, *dk, *dv;  /* backward inputs */
  void* dx;                  /* backward output, layout of x */
  float* dweight;            /* backward output [channels][taps] fp32 */
  void* workspace;           /* backward only: pkda_qkv_conv_bwd_workspace_bytes() bytes */
  size_t workspace_bytes;
} pkda_qkv_conv_args;

int pkda_qkv_conv_fwd(const pkda_qkv_conv_args* args, void* cuda_stream);
size_t pkda_qkv_conv_bwd_workspace_bytes(const pkda_qkv_conv_args* args);
int pkda_qkv_conv_bwd(const pkda_qkv_conv_args* args, void* cuda_stream);

/*
 * pkda_norm_gate_*  replace delta_feedback::pkda_norm_gate and
 * delta_feedback::pkda_norm_gate_backward (fla_ops.py:572-657; portable
 * definition pkda.py:543-547): per-row RMS normalisation with a learned weight and
 * a sigmoid output gate,
 *   rstd = rsqrt(mean(x^2) + eps),  y = x * rstd * weight * sigmoid(gate).
 *   x, gate, y [rows][dim] activation dtype; weight [dim] fp32; rstd [rows] fp32.
 * dim must be a power of two in 8..256.  The backward returns dx, dgate and the
 * fp32 weight gradient [dim] (summed over rows in a fixed order).
 */
typedef struct pkda_norm_gate_args {
  long long rows;
  int dim;
  int dtype;
  float eps;
  const void *x, *gate;
  const float* weight;
  void* y;                /* forward output */
  float* rstd;            /* forward output, backward input */
  const void* dy;         /* backward input */
  void *dx, *dgate;       /* backward outputs */
  float* dweight;         /* backward output [dim] */
  void* workspace;        /* backward only: pkda_norm_gate_bwd_workspace_bytes() bytes */
  size_t workspace_bytes;
} pkda_norm_gate_args;

int pkda_norm_gate_fwd(const pkda_norm_gate_args* args, void* cuda_stream);
size_t pkda_norm_gate_bwd_workspace_bytes(const pkda_norm_gate_args* args);
int pkda_norm_gate_bwd(const pkda_norm_gate_args* args, void* cuda_stream);

/*
 * pkda_decode_step: one cached decoding step (one new token per row) of the
 * layer's token mixer in a single launch -- the reference's sequence
 * pkda_qkv_conv on the history-prefixed rows (delta_feedback_experiment/pkda.py:239-288),
 * fused_recurrent_precond_kda (pkda.py:473-474), pkda_norm_gate (pkda.py:539-541)
 * and the cache update around them (model.py:428-468, 775-787).  The three
 * convolution histories, the matrix state and the preconditioner state are
 * updated IN PLACE (they are the decode cache).
 *   qkv          [batch][3 * W]            new Q|K|V projection row, W = heads * head_dim
 *   conv_q/k/v   [batch][W][taps - 1]      previous projections, oldest first (the
 *                                          reference's conv_state layout, pkda.py:253-260)
 *   conv_weight  [3 * W][taps] fp32
 *   g            [batch][heads][head_dim]  raw decay;  g_atk fp32, beta_atk, beta [batch][heads]
 *   state        [batch][heads][D][D] fp32, a_state [batch][heads][D] fp32
 *   gate         [batch][heads][D] output-gate logits, or NULL: `out` is then the
 *                recurrence output o without the RMS-norm gate
 *   norm_weight  [D] fp32;  out [batch][heads][D]
 * head_dim in {8, 16, 32, 64, 128}; taps 1..4.
 */
typedef struct pkda_decode_step_args {
  int batch, heads, head_dim, taps;
  int dtype;
  float scale, squash_x, squash_eps, qk_eps, norm_eps;
  const void* qkv;
  void *conv_q, *conv_k, *conv_v;
  const float* conv_weight;
  const void* g;
  const float* g_atk;
  const void *beta_atk, *beta;
  const float *A_log, *dt_bias, *log_atk_scale;
  float *state, *a_state;
  const void* gate;
  const float* norm_weight;
  void* out;
} pkda_decode_step_args;

int pkda_decode_step(const pkda_decode_step_args* args, void* cuda_stream);
size_t pkda_sizeof_decode_step_args(void);

/*
 * Control epilogue of the layer (delta_feedback_experiment/pkda.py:318-353 and the
 * gradient packer delta_feedback_experiment/cuda_kernels.py:1081-1172).  A packed
 * control row is  [decay hidden (hidden) | beta logits (heads) | precond decay logits
 * (heads) | precond beta logits (heads) | output-gate hidden (hidden)].
 *   pkda_controls_fwd:  beta = sigmoid, beta_atk = sigmoid (activation dtype),
 *                       g_atk = -exp(A_log_precond) * softplus(logit + dt_bias_precond) (fp32),
 *                       each [rows][heads]; the two hidden slices are used in place by the caller.
 *   pkda_controls_bwd:  from the gradients of the five pieces (any may be NULL = zero)
 *                       writes the packed gradient row [rows][2*hidden + 3*heads] in one
 *                       pass and the fp32 gradients of the two per-head parameters.
 *   pkda_pack_control_gradients: the packer alone, out[r] = concat(grads[0][r] .. grads[4][r]).
 */
typedef struct pkda_controls_args {
  long long rows;
  int heads, hidden;
  int dtype;
  const void* packed;
  const float *A_log_precond, *dt_bias_precond;
  void* beta;
  float* g_atk;
  void* beta_atk;
  const void *d_decay_hidden, *d_beta;
  const float* d_g_atk;
  const void *d_beta_atk, *d_gate_hidden;
  void* d_packed;
  float *dA_log_precond, *ddt_bias_precond;
  void* workspace;
  size_t workspace_bytes;
} pkda_controls_args;

int pkda_controls_fwd(const pkda_controls_args* args, void* cuda_stream);
size_t pkda_controls_bwd_workspace_bytes(const pkda_controls_args* args);
int pkda_controls_bwd(const pkda_controls_args* args, void* cuda_stream);

typedef struct pkda_pack_control_args {
  long long rows;
  int sizes[5];
  int dtype;
  const void* grads[5];
  void* out;
} pkda_pack_control_args;

int pkda_pack_control_gradients(const pkda_pack_control_args* args, void* cuda_stream);
size_t pkda_sizeof_controls_args(void);
size_t pkda_sizeof_pack_control_args(void);

size_t pkda_sizeof_qkv_conv_args(void);
size_t pkda_sizeof_norm_gate_args(void);

#ifdef __cplusplus
}
#endif
#endif /* PKDA_B200_H_ */
