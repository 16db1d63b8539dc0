// Backward pass for callers that cannot allocate device memory.
//
// Some hosts of this library hand it a stream and operand buffers but have no
// way to obtain scratch memory for it: a runtime plug-in whose framework owns
// every allocation and offers no scratch allocator, a callback running while
// the memory pool is frozen, or an embedding that forbids cudaMalloc after
// start-up.  nb200_sdpa_bwd needs scratch (the per-row delta = rowsum(out*dout)
// and, for a broadcast bias, an fp32 gradient accumulator), so those callers
// could not run a backward pass at all.  This entry point runs the very same
// backward with that scratch placed in a fixed array that lives inside the
// library image on every GPU that loads it.
#include <mutex>

#include "sdpa_common.cuh"

namespace {

// The scratch itself.  Held by each device from library load until exit.
static __device__ __align__(256) unsigned char g_static_scratch[NB200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the array on the CURRENT device.  In host code the array's
// name is only a handle, so the address is looked up once per device through
// the runtime and cached.
int scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    nb200::set_error("static scratch: cannot identify the current device (%s)", cudaGetErrorString(e));
    return NB200_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      nb200::set_error("static scratch: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return NB200_ERR_LAUNCH;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return NB200_OK;
}

}  // namespace

extern "C" NB200_API int nb200_sdpa_bwd_static_scratch(const nb200_sdpa_params* p, void* cuda_stream) {
  if (!p) { nb200::set_error("params is NULL"); return NB200_ERR_INVALID; }
  size_t need = 0;
  if (int rc = nb200_sdpa_workspace_bytes(p, NB200_PASS_BWD, &need)) return rc;
  if (need > size_t(NB200_STATIC_SCRATCH_BYTES)) {
    nb200::set_error("nb200_sdpa_bwd_static_scratch: this problem needs %zu bytes of scratch but the built-in scratch "
                     "holds %zu; use nb200_sdpa_bwd with a caller-provided workspace", need,
                     size_t(NB200_STATIC_SCRATCH_BYTES));
    return NB200_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  if (int rc = scratch_address(&scratch)) return rc;
  nb200_sdpa_params local = *p;  // the caller's workspace fields are ignored
  local.workspace = scratch;
  local.workspace_bytes = size_t(NB200_STATIC_SCRATCH_BYTES);
  nb200::forbid_side_stream(true);   // this entry point creates nothing, streams and events included
  const int rc = nb200_sdpa_bwd(&local, cuda_stream);
  nb200::forbid_side_stream(false);
  return rc;
}
