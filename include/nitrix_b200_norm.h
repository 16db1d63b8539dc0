/*
 * nitrix_b200_norm.h -- C ABI of the fused LayerNorm of the B200 (sm_100a) library: the sibling op of the
 * attention path (nitrix_b200_attention.h), behind the same shared library, status codes and dtype codes.
 *
 * The entry points stand where the reference keeps its fused-norm kernel module, which its dispatcher calls as
 * `layer_norm_pallas(x, weight, bias, eps=..., out_scale=...)` (reference src/nitrix/nn/norm/__init__.py:57-95,
 * :110-176; the module itself, src/nitrix/_kernels/cuda/norm.py:51-, only raises "not tileable" there: the reference
 * decided against building it, bench/PERF_LAYER_NORM.md:58-72).  The arithmetic follows the reference recipe
 * (src/nitrix/nn/norm/_reference.py:88-110): mean and BIASED variance over the trailing axis, rsqrt(var + eps),
 * optional per-channel weight and bias, then the constant out_scale; fp32 reductions and affine transform whatever
 * the storage dtype.
 *
 *   nb200_layer_norm_fwd   y = out_scale ((x - mean) rstd w + b); writes mean, rstd (fp32 per row) when given
 *   nb200_layer_norm_bwd   dx, and -- when asked -- dweight, dbias, from x, dy, weight, mean, rstd
 *                          (the gradient autodiff derives from the reference recipe)
 *
 * Layout.  x, y, dy, dx are dense [rows][channels] (every leading axis folded into rows), weight / bias / dweight /
 * dbias are [channels] of the same dtype as x.  Rows of a multiple of 16 bytes, at most 8192 channels and 16-byte
 * aligned pointers take the vector kernels (a row is read once and held in registers; dweight / dbias are summed in a
 * fixed order); anything else runs scalar kernels of the same library (dweight / dbias then through fp32 atomics).
 * Every pointer is a device pointer; all work is enqueued on the caller's stream; nothing is allocated: the
 * backward's column sums go through `workspace` (nb200_layer_norm_workspace_bytes; needed only when dweight or dbias
 * is wanted; the scalar path clears it on the stream).
 */
#ifndef NITRIX_B200_NORM_H_
#define NITRIX_B200_NORM_H_

#include "nitrix_b200_attention.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nb200_layer_norm_params {
  size_t struct_size;      /* sizeof(nb200_layer_norm_params) */
  const void* x;
  const void* weight;      /* NULL: no scaling */
  const void* bias;        /* NULL: no shift (forward only) */
  void* y;                 /* forward output */
  float* mean;             /* [rows] fp32: written by the forward when non-NULL, read by the backward */
  float* rstd;             /* [rows] fp32: likewise */
  const void* dy;          /* backward: dL/dy */
  void* dx;                /* backward: dL/dx */
  void* dweight;           /* backward: dL/dweight or NULL */
  void* dbias;             /* backward: dL/dbias or NULL */
  void* workspace;         /* backward, with dweight or dbias */
  size_t workspace_bytes;
  int64_t rows;
  int32_t channels;
  int32_t dtype;           /* nb200_dtype of x, y, dy, dx, weight, bias, dweight, dbias */
  float eps;
  float out_scale;
} nb200_layer_norm_params;

NB200_API int nb200_layer_norm_fwd(const nb200_layer_norm_params* p, void* cuda_stream);
NB200_API int nb200_layer_norm_bwd(const nb200_layer_norm_params* p, void* cuda_stream);
NB200_API int nb200_layer_norm_workspace_bytes(const nb200_layer_norm_params* p, size_t* bytes);

#ifdef __cplusplus
}
#endif
#endif /* NITRIX_B200_NORM_H_ */
