// Host-side glue shared by the translation units behind the C ABI.
#pragma once

#include <cuda_runtime.h>

#include "../../include/pkda_b200.h"
#include "pkda_common.cuh"

namespace pkda {

// Kernel stages, for launch accounting and the optional per-stage timing.
enum Stage {
  kStageOffsets = 0, kStagePackBeta, kStageAtkLocal, kStageAtkCarry, kStageIntraFwd, kStageScanFwd,
  kStageOutFwd, kStageScanBwd, kStageIntraBwd, kStageAtkBwdLocal, kStageAtkBwdCarry, kStageAtkBwdFinal,
  kStageParamReduce, kStageRecurrent, kStageConvFwd, kStageConvBwd, kStageConvDw, kStageNormGateFwd,
  kStageNormGateBwd, kStageNormGateDw, kStageDecodeStep, kStageControlsFwd, kStageControlsBwd,
  kStagePackControl, kStageStatusGuard, kStageBwdClassify, kStageIntraBwdRest, kStageIntraFwdRest, kStageCount
};

// begin_stage / end_stage bracket every kernel launch: they count launches and,
// when stage timing is switched on, record a CUDA event pair on the stream.
void begin_stage(int stage, cudaStream_t st);
void end_stage(cudaStream_t st);
void reset_launch_count();

// Testing aid behind pkda_set_variant: nonzero pins the older mma.sync kernel of a stage.
int stage_variant(int stage);

// Last launch of a chunked call: if the call's device status word is set (a bounded
// wait inside a kernel gave up), the first `n` elements of each given bf16 output are
// overwritten with NaN so that the failure reaches the caller's non-finite check.
int launch_status_guard(const int* status, void* out0, void* out1, void* out2, size_t n, cudaStream_t st);

// Raises a kernel's dynamic shared-memory limit, once per kernel and device (the attribute
// sticks to the function; asking again on every launch costs host time in eager mode).
// carveout >= 0 also sets the preferred shared-memory carve-out (percent).
bool dynamic_smem_once(const void* kernel, int bytes, int carveout);
template <typename K>
inline bool ensure_dynamic_smem(K kernel, int bytes, int carveout = -1) {
  return dynamic_smem_once(reinterpret_cast<const void*>(kernel), bytes, carveout);
}

// Upper limit for the kernels' direct block size (64 unless lowered through
// pkda_set_direct_block_cap, a testing aid).
int direct_block_cap();

// Validates the fields every entry point relies on.
int check_problem(const pkda_problem& p);

// chunk_offsets: device array for packed input (NULL for dense input).
Geo make_geo(const pkda_problem& p, const int* chunk_offsets);

// Upper bound on the number of 64-token chunks.
inline int chunk_bound(const pkda_problem& p) {
  if (p.cu_seqlens) return p.total_tokens / kChunk + p.n_seqs;
  return p.n_seqs * ((p.seq_len + kChunk - 1) / kChunk);
}

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

int recurrent_fwd(const pkda_recurrent_args* a, cudaStream_t st);
int chunk_fwd(const pkda_chunk_fwd_args* a, cudaStream_t st);
int chunk_bwd(const pkda_chunk_bwd_args* a, cudaStream_t st);
int recurrent_bwd(const pkda_recurrent_bwd_args* a, cudaStream_t st);
size_t recurrent_bwd_workspace(const pkda_problem& p);
int recurrent_fwd_checkpointed(const pkda_problem& p, const int* chunk_offsets, void* o_scratch, float* Sb,
                               float* Ab, cudaStream_t st);
size_t chunk_fwd_workspace(const pkda_problem& p);
size_t chunk_bwd_workspace(const pkda_problem& p);
size_t chunk_fwd_status_offset(const pkda_problem& p);
size_t chunk_bwd_status_offset(const pkda_problem& p);
int check_chunk_problem(const pkda_problem& p);
int qkv_conv_fwd(const pkda_qkv_conv_args* a, cudaStream_t st);
int qkv_conv_bwd(const pkda_qkv_conv_args* a, cudaStream_t st);
size_t qkv_conv_bwd_workspace(const pkda_qkv_conv_args& a);
int norm_gate_fwd(const pkda_norm_gate_args* a, cudaStream_t st);
int norm_gate_bwd(const pkda_norm_gate_args* a, cudaStream_t st);
size_t norm_gate_bwd_workspace(const pkda_norm_gate_args& a);
int decode_step(const pkda_decode_step_args* a, cudaStream_t st);
int decode_direct(const pkda_problem& p, void* o, float* final_state, float* final_A_state, cudaStream_t st);
int controls_fwd(const pkda_controls_args* a, cudaStream_t st);
int controls_bwd(const pkda_controls_args* a, cudaStream_t st);
size_t controls_bwd_workspace(const pkda_controls_args& a);
int pack_control_gradients(const pkda_pack_control_args* a, cudaStream_t st);

}  // namespace pkda
