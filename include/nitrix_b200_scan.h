/*
 * nitrix_b200_scan.h -- C ABI of the Mamba / S6 selective scan of the B200 (sm_100a) library: the second sibling op
 * of the attention path (nitrix_b200_attention.h), behind the same shared library, status codes and dtype codes.
 *
 * The entry points stand where the reference's dispatcher calls its fused scan module (reference
 * src/nitrix/nn/ssm/__init__.py:80-125 `_selective_scan_pallas`, :127- `selective_scan`; the module:
 * src/nitrix/_kernels/cuda/selective_scan.py:4-36).  The arithmetic follows the reference recipe
 * (src/nitrix/nn/ssm/_reference.py:60-98, :262-279):
 *
 *   a_t = exp(delta_t A),  b_t = (delta_t B_t) x_t,  h_t = a_t h_{t-1} + b_t  (h_{-1} = 0),
 *   y_t = sum_n C_{t,n} h_{t,n}  (+ D x_t when D is given)
 *
 * per batch element, channel and state, in fp32 whatever the storage dtype.
 *
 *   nb200_selective_scan_fwd   y; when `checkpoints` is given, the state after every eighth step for the backward
 *   nb200_selective_scan_bwd   dx, ddelta, dA, dB, dC (and dD when D is given) from x, delta, A, B, C, D, dy and the
 *                              forward's checkpoints (the gradient autodiff derives from the recipe)
 *
 * Layout.  x, delta, y, dy, dx, ddelta are dense (batch, length, channels); A, dA (channels, states); B, C, dB, dC
 * (batch, length, states); D, dD (channels); one dtype for all.  states <= 64.  Every pointer is a device pointer;
 * all work is enqueued on the caller's stream; nothing is allocated: the checkpoints
 * (nb200_selective_scan_checkpoint_bytes, fp32) belong to the caller and travel from the forward to the backward,
 * the backward's fp32 accumulators go through `workspace` (nb200_selective_scan_workspace_bytes; cleared on the
 * stream).  dB, dC (sums over channels) and dA, dD (sums over batch and length) are accumulated with fp32 atomics:
 * the order of those sums is not fixed.
 */
#ifndef NITRIX_B200_SCAN_H_
#define NITRIX_B200_SCAN_H_

#include "nitrix_b200_attention.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nb200_selective_scan_params {
  size_t struct_size;      /* sizeof(nb200_selective_scan_params) */
  const void* x;
  const void* delta;
  const void* A;
  const void* B;
  const void* C;
  const void* D;           /* NULL: no skip term */
  void* y;                 /* forward output */
  float* checkpoints;      /* forward: written when non-NULL; backward: read (required when length > 8) */
  const void* dy;          /* backward: dL/dy */
  void* dx;
  void* ddelta;
  void* dA;
  void* dB;
  void* dC;
  void* dD;                /* required when D is given */
  void* workspace;         /* backward */
  size_t workspace_bytes;
  int32_t batch, length, channels, states;
  int32_t dtype;           /* nb200_dtype of every operand and gradient */
  int32_t reserved;
} nb200_selective_scan_params;

NB200_API int nb200_selective_scan_fwd(const nb200_selective_scan_params* p, void* cuda_stream);
NB200_API int nb200_selective_scan_bwd(const nb200_selective_scan_params* p, void* cuda_stream);
NB200_API int nb200_selective_scan_workspace_bytes(const nb200_selective_scan_params* p, size_t* bytes);
NB200_API int nb200_selective_scan_checkpoint_bytes(const nb200_selective_scan_params* p, size_t* bytes);

#ifdef __cplusplus
}
#endif
#endif /* NITRIX_B200_SCAN_H_ */
