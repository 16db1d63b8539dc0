// Argument block of the tensor-core forward kernel (sdpa_tc_fwd.cu).
#pragma once

#include "sdpa_tc_common.cuh"

namespace nb200 {
namespace tc {

struct FwdArgs {
  int B, H, S, T;
  int bh_begin, bh_count;       // flattened (batch, head) range this launch covers
  int n_qblocks;                // 256-row query blocks per (batch, head): work items = n_qblocks * bh_count
  // Item order (both need the full (batch, head) range; a partial range is pair-major):
  //   1: head, query block, batch fastest -- neighbours share a head's K / V and bias in L2;
  //   2: query block (heaviest first), head, batch, dealt in rows of alternating direction -- evens out causal
  //      work when a CTA gets only a few items, at the price of K / V locality.
  //   3: batch element (longest kept length first, key-padding masks), head, query block, dealt the same way.
  int head_major;
  int causal;
  float scale;
  int bias_mode;
  int bias_b_mul, bias_h_mul;   // 0 when the bias is broadcast over batch / heads (tile mode)
  // Head dim 64, tile-mode bias, positive scale: the tensor core adds the bias tile to the scores,
  // S += bias (hi I + lo I) with hi + lo = 1 / scale in the operand dtype, and the softmax warps never read it.
  int bias_mma;
  float inv_scale_hi, inv_scale_lo;
  // Per-key terms (a bias with no query axis, a mask with no query axis) and a positive scale: the tensor core adds
  // them to every row of the score tile by one K = 16 step, S += W C^T, with C[key] = bias[key] / scale split into
  // three 16-bit terms (-inf for a dropped key); the softmax warps then neither read the bias nor apply the mask.
  int key_mma;
  const void* bias;             // key mode: base pointer
  int64_t bias_bs, bias_hs;     // key mode: element strides over batch / heads
  MaskBits mask;
  void* out;
  int64_t os[3];                // element strides of out (b, h, row)
  float* lse;
  // Fused output all-gather: every output row is also stored to these buffers (same strides as out; peers' copies of
  // a replicated result mapped into this process).  Rows are 32-byte aligned there (checked on the host).
  int n_out_peers;
  void* out_peers[NB200_MAX_OUT_PEERS];
  int* status;
  int smem_bytes;               // dynamic shared memory the launch requested (filled in by launch_fwd)
};

int launch_fwd(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
               const CUtensorMap& tb, const FwdArgs& a, cudaStream_t st);

}  // namespace tc
}  // namespace nb200
