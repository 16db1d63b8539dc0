// Argument block of the tensor-core forward kernel (sdpa_tc_fwd.cu).
#pragma once

#include "sdpa_tc_common.cuh"

namespace nb200 {
namespace tc {

struct FwdArgs {
  int H, S, T;
  int bh_begin;
  int causal;
  float scale;
  int bias_mode;
  int bias_b_mul, bias_h_mul;   // 0 when the bias is broadcast over batch / heads (tile mode)
  const void* bias;             // key mode: base pointer
  int64_t bias_bs, bias_hs;     // key mode: element strides over batch / heads
  MaskBits mask;
  void* out;
  int64_t os[3];                // element strides of out (b, h, row)
  float* lse;
  int* status;
};

int launch_fwd(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
               const CUtensorMap& tb, const FwdArgs& a, int n_qblocks, int bh_count, cudaStream_t st);

}  // namespace tc
}  // namespace nb200
