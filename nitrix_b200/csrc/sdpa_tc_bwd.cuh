// Interface of the tensor-core backward kernels (sdpa_tc_bwd.cu).
#pragma once

#include "sdpa_tc_common.cuh"

namespace nb200 {
namespace tc {

bool bwd_supported(const Problem& pr, int dtype, int bias_dtype, const char** why);
size_t bwd_workspace_bytes(const Problem& pr, int dtype, int bias_dtype);
int launch_bwd(const Problem& pr, int dtype, int bias_dtype, void* ws, size_t ws_bytes, cudaStream_t stream);

}  // namespace tc
}  // namespace nb200
