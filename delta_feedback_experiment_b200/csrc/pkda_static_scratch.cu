// pkda_chunk_fwd_static: the chunked forward for callers that may not allocate
// device memory.  Its scratch is a fixed array that lives in the library image.
#include <mutex>

#include "pkda_launch.h"

namespace pkda {

constexpr size_t kStaticScratchBytes = size_t(PKDA_STATIC_SCRATCH_BYTES);

// File-scope device array.  In host code this name is only a handle for the
// runtime: it is NOT a device address and must never be handed to a kernel.
// The device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the CURRENT device (looked up on the
// first call per device, with that device current).
static int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return PKDA_ERR_LAUNCH;
  if (dev >= kMaxDevices) {  // beyond the cache: look the address up on every call
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return PKDA_ERR_LAUNCH;
    *out = ptr;
    return PKDA_OK;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return PKDA_ERR_LAUNCH;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return PKDA_OK;
}

}  // namespace pkda

extern "C" {

size_t pkda_static_scratch_bytes(void) { return pkda::kStaticScratchBytes; }

int pkda_chunk_fwd_static(const pkda_chunk_fwd_args* args, void* cuda_stream) {
  if (!args) return PKDA_ERR_NULL;
  pkda::reset_launch_count();
  int rc0 = pkda::check_chunk_problem(args->p);  // geometry errors are reported as such, not as a size problem
  if (rc0 != PKDA_OK) return rc0;
  const size_t need = pkda::chunk_fwd_workspace(args->p);
  if (need > pkda::kStaticScratchBytes) return PKDA_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  int rc = pkda::static_scratch_address(&scratch);
  if (rc != PKDA_OK) return rc;
  pkda_chunk_fwd_args local = *args;  // caller's inputs and outputs, our scratch
  local.workspace = scratch;
  local.workspace_bytes = pkda::kStaticScratchBytes;
  return pkda::chunk_fwd(&local, static_cast<cudaStream_t>(cuda_stream));
}

int pkda_static_status_ptr(const pkda_problem* p, const int32_t** device_ptr) {
  if (!p || !device_ptr) return PKDA_ERR_NULL;
  int rc = pkda::check_chunk_problem(*p);
  if (rc != PKDA_OK) return rc;
  if (pkda::chunk_fwd_workspace(*p) > pkda::kStaticScratchBytes) return PKDA_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  rc = pkda::static_scratch_address(&scratch);
  if (rc != PKDA_OK) return rc;
  *device_ptr = reinterpret_cast<const int32_t*>(static_cast<unsigned char*>(scratch) +
                                                 pkda::chunk_fwd_status_offset(*p));
  return PKDA_OK;
}

}  // extern "C"
