// Peer mapping for the fused output all-gather (nb200_ipc_export / nb200_ipc_open / nb200_ipc_close).
//
// One process per GPU.  The forward kernel can store its output rows into other GPUs' buffers with plain global
// stores (sdpa_tc_fwd.cu, epilogue); for that the peers' buffers must be mapped into this process.  These helpers
// wrap the CUDA IPC calls so that a host layer only moves 128 opaque bytes between processes: the exporter names the
// cudaMalloc'ed block a pointer lies in plus the pointer's offset inside it, the importer maps the block (which also
// enables peer access between the two devices) and gets the equivalent pointer.  A block is mapped once per process
// however many pointers into it are opened; it is unmapped when the last of them is closed.
#include <string.h>

#include <map>
#include <mutex>
#include <string>

#include <cuda.h>

#include "sdpa_common.cuh"

namespace {

struct Wire {                       // layout of nb200_ipc_handle::bytes
  cudaIpcMemHandle_t mem;           // 64 bytes
  uint64_t offset;                  // of the exported pointer inside its allocation
  uint32_t magic;
};
static_assert(sizeof(Wire) <= sizeof(nb200_ipc_handle), "wire format must fit the opaque handle");
constexpr uint32_t kMagic = 0x4e423249u;  // "NB2I"

struct Mapping { void* base; int refs; };
std::mutex g_mutex;
std::map<std::string, Mapping> g_open;          // key: the 64 handle bytes
std::multimap<void*, std::string> g_by_ptr;     // pointer handed out -> key (one entry per open)

using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);

RangeFn range_fn() {
  static RangeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<RangeFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

}  // namespace

extern "C" {

NB200_API int nb200_ipc_export(const void* device_ptr, nb200_ipc_handle* handle) {
  using namespace nb200;
  if (!device_ptr || !handle) { set_error("nb200_ipc_export: NULL argument"); return NB200_ERR_INVALID; }
  RangeFn range = range_fn();
  if (!range) { set_error("nb200_ipc_export: cuMemGetAddressRange is unavailable"); return NB200_ERR_LAUNCH; }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range(&base, &size, reinterpret_cast<CUdeviceptr>(device_ptr)) != CUDA_SUCCESS) {
    set_error("nb200_ipc_export: the pointer is not inside a device allocation of this process");
    return NB200_ERR_INVALID;
  }
  Wire w;
  memset(&w, 0, sizeof(w));
  cudaError_t e = cudaIpcGetMemHandle(&w.mem, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error("nb200_ipc_export: cudaIpcGetMemHandle: %s (the block must come from cudaMalloc)", cudaGetErrorString(e));
    return NB200_ERR_LAUNCH;
  }
  w.offset = uint64_t(reinterpret_cast<CUdeviceptr>(device_ptr) - base);
  w.magic = kMagic;
  memset(handle->bytes, 0, sizeof(handle->bytes));
  memcpy(handle->bytes, &w, sizeof(w));
  return NB200_OK;
}

NB200_API int nb200_ipc_open(const nb200_ipc_handle* handle, void** device_ptr) {
  using namespace nb200;
  if (!handle || !device_ptr) { set_error("nb200_ipc_open: NULL argument"); return NB200_ERR_INVALID; }
  Wire w;
  memcpy(&w, handle->bytes, sizeof(w));
  if (w.magic != kMagic) { set_error("nb200_ipc_open: not a handle made by nb200_ipc_export"); return NB200_ERR_INVALID; }
  const std::string key(reinterpret_cast<const char*>(&w.mem), sizeof(w.mem));
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_open.find(key);
  if (it == g_open.end()) {
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, w.mem, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_error("nb200_ipc_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
      return NB200_ERR_LAUNCH;
    }
    it = g_open.emplace(key, Mapping{base, 0}).first;
  }
  it->second.refs += 1;
  void* p = static_cast<char*>(it->second.base) + w.offset;
  g_by_ptr.emplace(p, key);
  *device_ptr = p;
  return NB200_OK;
}

NB200_API int nb200_ipc_close(void* device_ptr) {
  using namespace nb200;
  std::lock_guard<std::mutex> lock(g_mutex);
  auto pit = g_by_ptr.find(device_ptr);
  if (pit == g_by_ptr.end()) { set_error("nb200_ipc_close: pointer was not returned by nb200_ipc_open"); return NB200_ERR_INVALID; }
  auto it = g_open.find(pit->second);
  g_by_ptr.erase(pit);
  if (it == g_open.end()) return NB200_OK;
  if (--it->second.refs > 0) return NB200_OK;
  cudaError_t e = cudaIpcCloseMemHandle(it->second.base);
  g_open.erase(it);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error("nb200_ipc_close: cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    return NB200_ERR_LAUNCH;
  }
  return NB200_OK;
}

}  // extern "C"
