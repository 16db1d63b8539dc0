// Tensor-core backward kernels (dq / dk / dv / dbias).
#include "sdpa_tc_bwd.cuh"

namespace nb200 {
namespace tc {

bool bwd_supported(const Problem&, int, int, const char** why) {
  *why = "the tensor-core backward is not available yet";
  return false;
}
size_t bwd_workspace_bytes(const Problem&, int, int) { return 0; }
int launch_bwd(const Problem&, int, int, void*, size_t, cudaStream_t) {
  set_error("the tensor-core backward is not available yet");
  return NB200_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace nb200
