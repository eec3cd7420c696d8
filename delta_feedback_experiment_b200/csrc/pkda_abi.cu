// extern "C" surface of libpkda_b200.so (declared in include/pkda_b200.h).
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "pkda_launch.h"

namespace pkda {

static thread_local int g_launches = 0;
void reset_launch_count() { g_launches = 0; }

static int g_direct_cap = 64;
int direct_block_cap() { return g_direct_cap; }

static int g_variant[kStageCount] = {};

bool dynamic_smem_once(const void* kernel, int bytes, int carveout) {
  static std::mutex mu;
  static std::unordered_map<const void*, unsigned long long> seen;  // kernel -> one bit per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  const unsigned long long bit = dev < 64 ? 1ull << dev : 0ull;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = seen.find(kernel);
    if (it != seen.end() && (it->second & bit)) return true;
  }
  if (carveout >= 0) cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, carveout);
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(mu);
  seen[kernel] |= bit;
  return true;
}
int stage_variant(int stage) { return (stage >= 0 && stage < kStageCount) ? g_variant[stage] : 0; }

__global__ void pkda_status_guard_kernel(const int* status, bf16* out0, bf16* out1, bf16* out2, size_t n) {
  if (*status == 0) return;
  const bf16 nan = __float2bfloat16(__int_as_float(0x7fc00000));
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    if (out0) out0[i] = nan;
    if (out1) out1[i] = nan;
    if (out2) out2[i] = nan;
  }
}

int launch_status_guard(const int* status, void* out0, void* out1, void* out2, size_t n, cudaStream_t st) {
  begin_stage(kStageStatusGuard, st);
  pkda_status_guard_kernel<<<4, 256, 0, st>>>(status, static_cast<bf16*>(out0), static_cast<bf16*>(out1),
                                              static_cast<bf16*>(out2), n);
  end_stage(st);
  return cudaGetLastError() == cudaSuccess ? PKDA_OK : PKDA_ERR_LAUNCH;
}

// Optional per-stage timing (used by the benchmark): one event pair per launch,
// taken from a pool that grows only while timing is enabled.
struct StageTimer {
  bool on = false;
  std::vector<cudaEvent_t> events;  // 2 per record
  std::vector<int> stage;
  size_t used = 0;
  bool open = false;
};
static StageTimer g_timer;

void begin_stage(int stage, cudaStream_t st) {
  if (!g_timer.on) return;
  if (g_timer.events.size() < 2 * (g_timer.used + 1)) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) { g_timer.on = false; return; }
    g_timer.events.push_back(a);
    g_timer.events.push_back(b);
  }
  if (g_timer.stage.size() <= g_timer.used) g_timer.stage.push_back(stage);
  else g_timer.stage[g_timer.used] = stage;
  cudaEventRecord(g_timer.events[2 * g_timer.used], st);
  g_timer.open = true;
}

void end_stage(cudaStream_t st) {
  ++g_launches;
  if (g_timer.on && g_timer.open) {
    cudaEventRecord(g_timer.events[2 * g_timer.used + 1], st);
    ++g_timer.used;
    g_timer.open = false;
  }
}

int check_problem(const pkda_problem& p) {
  if (p.n_seqs < 0 || p.total_tokens < 0 || p.heads <= 0 || p.head_dim <= 0) return PKDA_ERR_SHAPE;
  if (!p.cu_seqlens && (p.seq_len < 0 || (long long)p.n_seqs * p.seq_len != p.total_tokens))
    return PKDA_ERR_SHAPE;
  if (p.n_seqs == 0 || p.total_tokens == 0) return PKDA_OK;
  if (!p.q || !p.k || !p.v || !p.g || !p.g_atk || !p.beta_atk || !p.beta || !p.A_log || !p.dt_bias ||
      !p.log_atk_scale)
    return PKDA_ERR_NULL;
  const void* ptrs[] = {p.q, p.k, p.v, p.g, p.initial_state};
  for (const void* x : ptrs)
    if (x && (reinterpret_cast<uintptr_t>(x) & 15)) return PKDA_ERR_ALIGN;
  if (p.dtype != PKDA_BF16 && p.dtype != PKDA_F32) return PKDA_ERR_DTYPE;
  return PKDA_OK;
}

Geo make_geo(const pkda_problem& p, const int* chunk_offsets) {
  Geo g;
  g.n_seqs = p.n_seqs;
  g.seq_len = p.cu_seqlens ? 0 : p.seq_len;
  g.total_tokens = p.total_tokens;
  g.heads = p.heads;
  g.chunks_per_seq = p.cu_seqlens ? 0 : (p.seq_len + kChunk - 1) / kChunk;
  g.total_chunks = chunk_bound(p);
  g.cu_seqlens = p.cu_seqlens;
  g.chunk_offsets = p.cu_seqlens ? chunk_offsets : nullptr;
  return g;
}

}  // namespace pkda

extern "C" {

int pkda_recurrent_fwd(const pkda_recurrent_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::recurrent_fwd(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t pkda_recurrent_bwd_workspace_bytes(const pkda_problem* p) {
  return p ? pkda::recurrent_bwd_workspace(*p) : 0;
}

int pkda_recurrent_bwd(const pkda_recurrent_bwd_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::recurrent_bwd(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t pkda_chunk_fwd_workspace_bytes(const pkda_problem* p) {
  return p ? pkda::chunk_fwd_workspace(*p) : 0;
}

int pkda_chunk_fwd(const pkda_chunk_fwd_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::chunk_fwd(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t pkda_chunk_bwd_workspace_bytes(const pkda_problem* p) {
  return p ? pkda::chunk_bwd_workspace(*p) : 0;
}

size_t pkda_chunk_fwd_status_offset(const pkda_problem* p) { return p ? pkda::chunk_fwd_status_offset(*p) : 0; }
size_t pkda_chunk_bwd_status_offset(const pkda_problem* p) { return p ? pkda::chunk_bwd_status_offset(*p) : 0; }

int pkda_chunk_bwd(const pkda_chunk_bwd_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::chunk_bwd(args, static_cast<cudaStream_t>(cuda_stream));
}

int pkda_qkv_conv_fwd(const pkda_qkv_conv_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::qkv_conv_fwd(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t pkda_qkv_conv_bwd_workspace_bytes(const pkda_qkv_conv_args* args) {
  return args ? pkda::qkv_conv_bwd_workspace(*args) : 0;
}

int pkda_qkv_conv_bwd(const pkda_qkv_conv_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::qkv_conv_bwd(args, static_cast<cudaStream_t>(cuda_stream));
}

int pkda_norm_gate_fwd(const pkda_norm_gate_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::norm_gate_fwd(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t pkda_norm_gate_bwd_workspace_bytes(const pkda_norm_gate_args* args) {
  return args ? pkda::norm_gate_bwd_workspace(*args) : 0;
}

int pkda_norm_gate_bwd(const pkda_norm_gate_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::norm_gate_bwd(args, static_cast<cudaStream_t>(cuda_stream));
}

int pkda_decode_step(const pkda_decode_step_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::decode_step(args, static_cast<cudaStream_t>(cuda_stream));
}

int pkda_controls_fwd(const pkda_controls_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::controls_fwd(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t pkda_controls_bwd_workspace_bytes(const pkda_controls_args* args) {
  return args ? pkda::controls_bwd_workspace(*args) : 0;
}

int pkda_controls_bwd(const pkda_controls_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::controls_bwd(args, static_cast<cudaStream_t>(cuda_stream));
}

int pkda_pack_control_gradients(const pkda_pack_control_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  return pkda::pack_control_gradients(args, static_cast<cudaStream_t>(cuda_stream));
}

int pkda_abi_version(void) { return PKDA_ABI_VERSION; }

const char* pkda_status_string(int status) {
  switch (status) {
    case PKDA_OK: return "ok";
    case PKDA_ERR_NULL: return "a required pointer is NULL";
    case PKDA_ERR_SHAPE: return "unsupported geometry";
    case PKDA_ERR_DTYPE: return "unsupported activation dtype";
    case PKDA_ERR_WORKSPACE: return "workspace missing or too small";
    case PKDA_ERR_LAUNCH: return "kernel launch failed";
    case PKDA_ERR_ALIGN: return "pointer not 16-byte aligned";
    case PKDA_ERR_STATIC_LIMIT: return "problem exceeds the built-in static scratch (use pkda_chunk_fwd with a workspace)";
    default: return "unknown status";
  }
}

size_t pkda_sizeof_problem(void) { return sizeof(pkda_problem); }
size_t pkda_sizeof_recurrent_args(void) { return sizeof(pkda_recurrent_args); }
size_t pkda_sizeof_chunk_fwd_args(void) { return sizeof(pkda_chunk_fwd_args); }
size_t pkda_sizeof_chunk_bwd_args(void) { return sizeof(pkda_chunk_bwd_args); }
size_t pkda_sizeof_qkv_conv_args(void) { return sizeof(pkda_qkv_conv_args); }
size_t pkda_sizeof_norm_gate_args(void) { return sizeof(pkda_norm_gate_args); }
size_t pkda_sizeof_decode_step_args(void) { return sizeof(pkda_decode_step_args); }
size_t pkda_sizeof_controls_args(void) { return sizeof(pkda_controls_args); }
size_t pkda_sizeof_pack_control_args(void) { return sizeof(pkda_pack_control_args); }
int pkda_last_launch_count(void) { return pkda::g_launches; }

int pkda_set_direct_block_cap(int cap) {
  if (cap < 1 || cap > 64 || (cap & (cap - 1))) return PKDA_ERR_SHAPE;
  pkda::g_direct_cap = cap;
  return PKDA_OK;
}

int pkda_stage_count(void) { return pkda::kStageCount; }

int pkda_set_variant(const char* stage, int variant) {
  if (!stage) return PKDA_ERR_NULL;
  const int two_impl[] = {pkda::kStageIntraFwd, pkda::kStageScanFwd, pkda::kStageOutFwd, pkda::kStageScanBwd,
                          pkda::kStageIntraBwd};
  for (int s : two_impl)
    if (std::strcmp(stage, pkda_stage_name(s)) == 0) {
      pkda::g_variant[s] = (s == pkda::kStageOutFwd && variant == 2) ? 2 : (variant ? 1 : 0);
      return PKDA_OK;
    }
  return PKDA_ERR_SHAPE;
}

const char* pkda_stage_name(int stage) {
  static const char* names[] = {"chunk_offsets", "pack_beta", "atk_local", "atk_carry", "intra_fwd", "scan_fwd",
                                "out_fwd", "scan_bwd", "intra_bwd", "atk_bwd_local", "atk_bwd_carry",
                                "atk_bwd_final", "param_reduce", "recurrent", "qkv_conv_fwd", "qkv_conv_bwd",
                                "qkv_conv_dw", "norm_gate_fwd", "norm_gate_bwd", "norm_gate_dw", "decode_step", "controls_fwd", "controls_bwd", "pack_control",
                                "status_guard", "bwd_classify", "intra_bwd_rest", "intra_fwd_rest"};
  return (stage >= 0 && stage < pkda::kStageCount) ? names[stage] : "?";
}

int pkda_stage_timing(int enable) {
  pkda::g_timer.on = enable != 0;
  pkda::g_timer.used = 0;
  pkda::g_timer.open = false;
  return PKDA_OK;
}

int pkda_stage_timing_read(float* ms, int* counts, int n_stages) {
  if (!ms || !counts) return PKDA_ERR_NULL;
  for (int i = 0; i < n_stages; ++i) { ms[i] = 0.f; counts[i] = 0; }
  pkda::StageTimer& t = pkda::g_timer;
  for (size_t r = 0; r < t.used; ++r) {
    if (cudaEventSynchronize(t.events[2 * r + 1]) != cudaSuccess) return PKDA_ERR_LAUNCH;
    float e = 0.f;
    if (cudaEventElapsedTime(&e, t.events[2 * r], t.events[2 * r + 1]) != cudaSuccess) return PKDA_ERR_LAUNCH;
    const int s = t.stage[r];
    if (s >= 0 && s < n_stages) { ms[s] += e; counts[s] += 1; }
  }
  t.used = 0;
  return PKDA_OK;
}

}  // extern "C"
