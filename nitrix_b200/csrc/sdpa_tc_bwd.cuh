// Interface of the tensor-core backward kernels (sdpa_tc_bwd.cu).
#pragma once

#include "sdpa_tc_common.cuh"

namespace nb200 {
namespace tc {

// Argument block of the backward kernels (sdpa_tc_bwd.cu, sdpa_tc_bwd_d128.cu).
struct BwdArgs {
  int H, S, T;
  int bh_begin;
  int causal;
  float scale;
  int bias_mode;
  // Key-major kernel, tile-mode bias: added by the tensor core, scores^T += bias^T (hi I + lo I) with
  // hi + lo = 1 / scale split into two 16-bit values (lo = 0 when 1 / scale is exact in 16 bits).  Then
  // scores * scale holds scale * q.k + bias and the element-wise warps never read the bias column-wise.
  int bias_mma;
  float inv_scale_hi, inv_scale_lo;
  // Query-major kernel, per-key terms (a bias or a mask with no query axis) and a positive scale: added to the scores
  // by one K = 16 MMA step, scores += W C^T with C[key] = bias[key] / scale in three 16-bit terms, -inf for a dropped
  // key; the element-wise warps then neither read the bias nor apply that mask.
  int key_aug;
  int bias_b_mul, bias_h_mul;
  const void* bias;             // key mode base
  int64_t bias_bs, bias_hs;
  MaskBits mask;
  int mask_key_only;            // key-major: the mask has no query axis (use mask.rows per key)
  const float* lse;
  const float* delta;
  // Rows per (batch, head) of the lse / delta arrays handed to the kernels: S, or -- when S is not a multiple of 4, so
  // that 16-byte copies of 64-row blocks would start off their alignment -- S rounded up to 64 (padded copies in the
  // workspace, made by launch_bwd).
  int ld_rows;
  void* out1; int64_t o1s[3];   // key-major: dv
  void* out2; int64_t o2s[3];   // dq | dk
  void* dbias; int64_t dbs[4];  // query-major only; null when not requested
  // Gradient of a bias that is broadcast over some axis: fp32 sums over the broadcast axes, in an accumulator of the
  // bias' own extent (zero on entry; acc_s = its element strides over (b, h, row), 0 on broadcast axes, unit key
  // stride).  A bias with a query axis is summed by the query-major kernel (ds tiles added with 16-byte
  // reductions), a per-key bias by the key-major kernel (each thread sums its key's ds over the queries it
  // streams and adds once).
  float* dbias_acc; int64_t acc_s[3];
  float* dq_acc;                // one-kernel backwards: fp32 sums of ds K, zero on entry (layout: see the kernels)
  int acc_rows;                 // head dim 128: rows of the dq accumulator per (batch, head) (S rounded up to 64)
  int* status;
};

// One-kernel backward at head dim 128 (sdpa_tc_bwd_d128.cu): dq, dk, dv and the dbias tiles of a full-extent bias.
// maps: K and V (128-row boxes), Q and dO (64-row boxes), bias (64-row boxes), dbias (64 x 64 store boxes).
struct D128Maps { CUtensorMap k, v, q, dout, bias, dbias; };
bool d128_merged_supported(const Problem& pr, int bias_mode, bool bias_mma);
size_t d128_acc_bytes(const Problem& pr);
int launch_bwd_d128(const D128Maps& maps, const BwdArgs& a, bool bf16, bool tile_bias, int n_tiles, int bh_count,
                    cudaStream_t st);
int launch_dq_finish_d128(const Problem& pr, const float* acc, int acc_rows, bool bf16, cudaStream_t st);

bool bwd_supported(const Problem& pr, int dtype, int bias_dtype, const char** why);
size_t bwd_workspace_bytes(const Problem& pr, int dtype, int bias_dtype);
// ld_rows: rows per (batch, head) of pr.lse / pr.delta as passed (S, or the padded count of staged copies)
int launch_bwd(const Problem& pr, int dtype, int bias_dtype, void* ws, size_t ws_bytes, int ld_rows, cudaStream_t stream);

}  // namespace tc
}  // namespace nb200
