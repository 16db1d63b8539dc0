/*
 * nitrix_b200_attention.h -- C ABI of the B200 (sm_100a) flash-attention path.
 *
 * This is the boundary a foreign-function layer binds (an XLA FFI handler under
 * JAX, ctypes under PyTorch).  Plain pointers, sizes and strides only; every
 * pointer is a DEVICE pointer owned by the caller and borrowed for the duration
 * of the enqueued work.  All work is enqueued on the caller's stream; no entry
 * point synchronises the device, allocates device memory or frees it.
 *
 * The entry points replace, for nitrix.nn's attention, the reference's private
 * fused-kernel module (reference src/nitrix/_kernels/cuda/attention.py):
 *
 *   nb200_sdpa_fwd   <->  _fused_forward_with_lse + _mha_forward   (:547-584, :159-264)
 *   nb200_sdpa_bwd   <->  _fused_backward + _mha_backward          (:600-653, :390-499)
 *   nb200_sdpa_plan  <->  _check_tileable (the shape gate)         (:708-765)
 *
 * Layout.  q is (B, H, S, D), k is (B, H, T, D), v is (B, H, T, Dv), out and
 * dout are (B, H, S, Dv); "B" is the product of all leading batch dimensions.
 * Each tensor is described by four ELEMENT strides (b, h, row, col); the col
 * stride of q, k, v, out, dout, dq, dk, dv must be 1.  bias and mask are
 * logically (B, H, S, T) and are described by strides as well: a broadcast axis
 * has stride 0, so no broadcast copy is ever materialised (the reference
 * materialises them, :560-569).  mask holds one byte per element, non-zero =
 * keep (reference _reference.py:165-172).  lse and delta are dense fp32
 * (B, H, S); lse is the base-2 log-sum-exp of the masked logits, m + log2(l)
 * (reference attention.py:156).
 */
#ifndef NITRIX_B200_ATTENTION_H_
#define NITRIX_B200_ATTENTION_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB200_ABI_VERSION 2

#if defined(__GNUC__)
#define NB200_API __attribute__((visibility("default")))
#else
#define NB200_API
#endif

/* element types */
enum nb200_dtype { NB200_F32 = 0, NB200_BF16 = 1, NB200_F16 = 2 };

/* status codes (0 = ok; negatives are errors; nothing aborts or traps) */
enum nb200_status {
  NB200_OK = 0,
  NB200_ERR_INVALID = -1,     /* null pointer, bad dtype, bad struct size ...      */
  NB200_ERR_UNSUPPORTED = -2, /* well-formed but no kernel covers it (e.g. D > 256) */
  NB200_ERR_ALIGNMENT = -3,   /* pointer / stride alignment a kernel needs is unmet */
  NB200_ERR_WORKSPACE = -4,   /* workspace missing or smaller than required         */
  NB200_ERR_LAUNCH = -5,      /* CUDA reported an error when enqueueing             */
  NB200_ERR_TIMEOUT = -6      /* a bounded device-side wait ran out (status word)   */
};

/* kernel families; `kernel` in the params selects, nb200_sdpa_plan reports */
enum nb200_kernel {
  NB200_KERNEL_AUTO = 0,
  NB200_KERNEL_SIMT = 1,   /* fp32-arithmetic CUDA-core kernels: any shape / dtype  */
  NB200_KERNEL_TCGEN05 = 2, /* TMA + tcgen05 (TMEM accumulators): bf16 / fp16 tiles */
  /* Reported by nb200_sdpa_plan only (not a value for `kernel`): the problem runs in the NB200_KERNEL_SIMT family
   * on its fp32-operand kernels that split every operand into two TF32 terms and use the warp-level tensor-core
   * path (3 x TF32, fp32 accuracy) -- the counterpart of what the reference's fused path accepts, fp32 only
   * (reference attention.py:736-744). */
  NB200_KERNEL_MMA_TF32X3 = 3
};

enum nb200_pass { NB200_PASS_FWD = 0, NB200_PASS_BWD = 1 };

typedef struct nb200_sdpa_params {
  uint32_t struct_size; /* = sizeof(nb200_sdpa_params); checked                      */
  int32_t dtype;        /* nb200_dtype of q, k, v, out, dout, dq, dk, dv             */
  int32_t bias_dtype;   /* nb200_dtype of bias and dbias (ignored when bias == NULL) */
  int32_t B, H, S, T, D, Dv;

  /* forward operands */
  const void* q;
  const void* k;
  const void* v;
  void* out;            /* written by fwd, read by bwd                               */
  float* lse;           /* (B,H,S) fp32, written by fwd, read by bwd                 */
  const void* bias;     /* may be NULL                                               */
  const uint8_t* mask;  /* may be NULL; one byte per element, non-zero keeps         */

  /* backward operands (ignored by fwd) */
  const void* dout;
  void* dq;
  void* dk;
  void* dv;
  void* dbias;          /* may be NULL: no bias gradient is produced                 */

  /* scratch: nb200_sdpa_workspace_bytes() says how much each pass needs */
  void* workspace;
  size_t workspace_bytes;

  /* element strides (b, h, row, col) */
  int64_t q_stride[4], k_stride[4], v_stride[4], out_stride[4];
  int64_t dout_stride[4], dq_stride[4], dk_stride[4], dv_stride[4];
  int64_t bias_stride[4], mask_stride[4], dbias_stride[4];

  float scale;          /* softmax temperature (reference default 1/sqrt(D))         */
  int32_t causal;       /* keep key j for query i iff j <= i (aligned at 0)          */
  int32_t kernel;       /* nb200_kernel: AUTO, or force one family                   */

  /* multi-GPU partition: this call processes flattened (b*H + h) indices in
   * [bh_begin, bh_end).  Pointers and strides always describe the whole
   * tensors; bh_begin = 0, bh_end = B*H processes everything. */
  int32_t bh_begin, bh_end;

  /* Backward produces the bias gradient iff dbias != NULL or want_dbias != 0.  The flag lets nb200_sdpa_plan and
   * nb200_sdpa_workspace_bytes answer for a backward with a bias gradient before the dbias buffer exists;
   * nb200_sdpa_bwd itself needs the pointer (want_dbias with dbias == NULL is NB200_ERR_INVALID there). */
  int32_t want_dbias;

  /* 0: `mask` is the byte mask described above.  1 or 2: `mask` points to a buffer filled by nb200_mask_pack for
   * this same problem (same B, H, S, T and mask_stride, which still tell which axes the mask broadcasts over):
   * 1 = packed without the transposed copy (enough for the forward, and for the backward of a mask with no
   * query axis), 2 = packed with it (forward and backward).  A packed mask is packed once and reused by the
   * forward, the backward and any number of later calls; only the tensor-core family consumes it
   * (NB200_ERR_UNSUPPORTED when the problem runs on the CUDA-core family). */
  int32_t mask_is_bitpacked;

  /* Fused output all-gather (forward only; the reference has no collective).  The forward kernel stores every
   * output row it produces into out AND into n_out_peers more buffers with the same shape and strides --
   * typically the peers' copies of a replicated (B, H, S, Dv) result, mapped into this process with
   * nb200_ipc_open.  Plain stores over NVLink from the epilogue; the caller synchronises the ranks afterwards
   * (each rank's rows are complete when its stream has passed the forward and all ranks have met).  Needs the
   * tensor-core family and 32-byte aligned rows; 0 <= n_out_peers <= NB200_MAX_OUT_PEERS. */
  int32_t n_out_peers;
  int32_t reserved0;
  void* out_peers[7];
} nb200_sdpa_params;

#define NB200_MAX_OUT_PEERS 7

/* ABI version of the loaded library (== NB200_ABI_VERSION it was built with). */
NB200_API int nb200_version(void);

/* Message for the last non-OK status returned on the calling thread. */
NB200_API const char* nb200_last_error(void);

/* Which kernel family would run this problem for `pass`; writes one of
 * NB200_KERNEL_SIMT / NB200_KERNEL_TCGEN05 / NB200_KERNEL_MMA_TF32X3 to *kernel.  When the params force a
 * family that does not cover the problem the status says why (the Python layer
 * turns that into the reference's decline -> warn-once contract,
 * reference nn/attention/__init__.py:207-220).  Never launches. */
NB200_API int nb200_sdpa_plan(const nb200_sdpa_params* p, int pass, int* kernel);

/* Scratch bytes `pass` needs for this problem: packed mask bits (forward and backward), and for the backward
 * the delta rows (B*H*S floats), an fp32 copy of a broadcast bias' gradient, and -- bf16/fp16 at head dim 64
 * without a bias gradient, where one kernel produces dq, dk and dv -- an fp32 copy of dq (B*H*S*64 floats).
 * plus padded copies of bias / dbias / lse / delta when their rows are not 16-byte addressable (lengths that are not
 * multiples of 8, strided keys).  The tensor-core kernels take bf16/fp16 with D == Dv in {64, 128}; everything else runs
 * on the fp32 CUDA-core family (nb200_sdpa_plan tells which). */
NB200_API int nb200_sdpa_workspace_bytes(const nb200_sdpa_params* p, int pass, size_t* bytes);

/* Forward: out = softmax(scale * q k^T + bias, masked) v and lse.
 * Replaces reference attention.py:547-584 (glue) and :159-264 (kernel launch). */
NB200_API int nb200_sdpa_fwd(const nb200_sdpa_params* p, void* cuda_stream);

/* Backward: dq, dk, dv and, when dbias != NULL, dbias (reduced over the
 * broadcast axes of bias, in bias dtype) from (q, k, v, bias, mask, out, lse,
 * dout).  Replaces reference attention.py:600-653 and :390-499.
 * All work is ordered on cuda_stream as seen by the caller.  For a small problem on the CUDA-core kernels two
 * independent kernels may run side by side: the second on a stream the library owns (one per host thread and
 * device, created at the first such call outside a graph capture), forked from and joined back into cuda_stream by
 * events, so the call can be captured into a CUDA graph like any other. */
NB200_API int nb200_sdpa_bwd(const nb200_sdpa_params* p, void* cuda_stream);

/* Backward pass for callers that cannot allocate device memory (no counterpart
 * in the reference, whose runtime allocates scratch for its kernels itself).
 * Same operands, results and status codes as nb200_sdpa_bwd, but the scratch the
 * backward needs (row-wise delta; fp32 accumulator of a broadcast bias gradient;
 * for the tensor-core kernels also the packed mask words -- row-major, key-major
 * and per-sequence key counts --, the fp32 dq sums of the one-kernel backwards and
 * any padded copies of bias / dbias / lse / delta) lives in a fixed
 * NB200_STATIC_SCRATCH_BYTES array inside the library image on every GPU that
 * loads it; p->workspace and p->workspace_bytes are ignored.
 *  - Allocates nothing: no cudaMalloc / cudaFree, no allocating library call.
 *  - A problem whose scratch (nb200_sdpa_workspace_bytes, backward pass) exceeds
 *    NB200_STATIC_SCRATCH_BYTES is rejected with NB200_ERR_WORKSPACE.
 *  - The first call on each device looks up the array's device address (with
 *    that device current); make that first call before any stream capture.
 *  - All calls on a device share the one array and it keeps the previous
 *    call's contents; what must start at zero is cleared on the stream by each
 *    call.  Calls whose GPU work may overlap (different streams) race on it:
 *    serialise them. */
#define NB200_STATIC_SCRATCH_BYTES (8u << 20)
NB200_API int nb200_sdpa_bwd_static_scratch(const nb200_sdpa_params* p, void* cuda_stream);

/* Number of kernels this library has enqueued since load (all threads). */
NB200_API uint64_t nb200_launch_count(void);

/* Per-kernel timing for measurements.  nb200_profile(1) clears earlier records and makes the library record a
 * CUDA event on the launching stream after each kernel it enqueues; nb200_profile(0) stops and clears.
 * nb200_profile_read synchronises those events and writes one line per kernel name,
 * "name<TAB>launches<TAB>total_ms", into buf (NUL-terminated, truncated to `bytes`); it returns the size the
 * full text needs.  The events cost a few microseconds per kernel: leave this off in production. */
NB200_API int nb200_profile(int enable);
NB200_API size_t nb200_profile_read(char* buf, size_t bytes);

/* Reads (and clears) the device-side status word kernels set when a bounded
 * wait expires; call after synchronising the stream.  NB200_OK or
 * NB200_ERR_TIMEOUT.  `device` is the CUDA device ordinal. */
NB200_API int nb200_device_status(int device);

/* Bit-packing of a boolean mask, done once and reused (no counterpart in the reference, which re-reads the byte
 * mask in every kernel, attention.py:118-126, :306-311, :366-371).  nb200_mask_pack_bytes: size of the packed
 * buffer for the mask described by p (dims, mask, mask_stride); with_transpose != 0 adds the key-major copy the
 * backward of a mask with a query axis needs (ignored for masks without a query axis).  nb200_mask_pack enqueues
 * the packing kernel on the stream; `packed` must be 256-byte aligned.  Pass the buffer as p->mask with
 * p->mask_is_bitpacked = 1 (packed without transpose) or 2 (with). */
NB200_API int nb200_mask_pack_bytes(const nb200_sdpa_params* p, int with_transpose, size_t* bytes);
NB200_API int nb200_mask_pack(const nb200_sdpa_params* p, int with_transpose, void* packed, size_t packed_bytes,
                              void* cuda_stream);

/* Peer mapping for the fused output all-gather (no counterpart in the reference).  One process per GPU:
 * nb200_ipc_export describes a device allocation of this process (any pointer inside a cudaMalloc'ed block) in
 * 128 opaque bytes that are sent to the peer processes by any host channel; nb200_ipc_open maps it into the
 * calling process (enabling peer access between the two GPUs) and returns the device pointer to use in
 * out_peers; nb200_ipc_close unmaps it.  Nothing is copied and no memory is allocated. */
typedef struct nb200_ipc_handle { unsigned char bytes[128]; } nb200_ipc_handle;
NB200_API int nb200_ipc_export(const void* device_ptr, nb200_ipc_handle* handle);
NB200_API int nb200_ipc_open(const nb200_ipc_handle* handle, void** device_ptr);
NB200_API int nb200_ipc_close(void* device_ptr);

/* RMS normalisation of q and k over the head dim -- the `qk_norm=True` pre-op -- and its gradient, each as one launch
 * for both tensors.  Replaces the element-wise ops the reference runs outside its fused kernels
 * (src/nitrix/nn/attention/__init__.py:184-197 `qk_rms_norm(q)`, `qk_rms_norm(k)`; the op:
 * src/nitrix/nn/attention/_reference.py:52-77): y = x * rsqrt(mean(x^2 over the head dim) + 1e-6), fp32 arithmetic,
 * no learnable scale.  It stays a pre-op, as in the reference: the attention entry points then take y.
 * A tensor is [B][H][N][head_dim] with element strides xs over (b, h, n) and a contiguous head dim; y (and, for the
 * gradient, g = dL/dy in, y = dL/dx out) are dense [B*H*N][head_dim].  Pointers and row starts 16-byte aligned; head_dim
 * a multiple of 16 bytes and at most 256; B * H * N may be 0.
 *   nb200_qk_rms_norm        y  = x r,                  r = rsqrt(mean(x^2) + eps)
 *   nb200_qk_rms_norm_grad   dx = r (g - (x r) mean(g x r))   (x is the un-normalised input again) */
typedef struct nb200_qk_norm_tensor {
  const void* x;
  const void* g;      /* gradient pass only */
  void* y;
  int64_t xs[3];
  int32_t B, H, N;
  int32_t reserved;
} nb200_qk_norm_tensor;
NB200_API int nb200_qk_rms_norm(const nb200_qk_norm_tensor* q, const nb200_qk_norm_tensor* k, int head_dim, int dtype,
                                void* cuda_stream);
NB200_API int nb200_qk_rms_norm_grad(const nb200_qk_norm_tensor* q, const nb200_qk_norm_tensor* k, int head_dim,
                                     int dtype, void* cuda_stream);

/* Diagnostic: runs the give-up branch of the bounded mbarrier wait all tensor-core kernels use (no counterpart in
 * the reference).  One warp waits, with a budget of a few thousand cycles, on a barrier nothing completes; the wait
 * expires within a few milliseconds, the kernel exits normally and the device status word holds a time-out code.
 * result_device points to two ints on the device: [0] = 1 if the wait (wrongly) reported completion, else 0;
 * [1] = the CTA abort flag the wait raised.  After synchronising, nb200_device_status() returns NB200_ERR_TIMEOUT
 * once and NB200_OK afterwards. */
NB200_API int nb200_selftest_bounded_wait(int* result_device, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* NITRIX_B200_ATTENTION_H_ */
