// XLA FFI handlers over the C ABI of the B200 attention library (include/nitrix_b200_attention.h).
//
// This is the layer a JAX program binds: two custom-call handlers, `nb200_sdpa_fwd_ffi` and `nb200_sdpa_bwd_ffi`,
// registered from Python with jax.ffi.register_ffi_target(..., platform="CUDA") and invoked through jax.ffi.ffi_call
// (nitrix_b200/jax_ffi.py).  They replace, for the reference's fused attention path, the Pallas kernel launches
// behind `_sdpa_p_fwd` / `_sdpa_p_bwd` (reference src/nitrix/_kernels/cuda/attention.py:661-700).
//
// Contract with XLA: every buffer is borrowed (XLA owns all memory, nothing is retained or freed here); the stream
// comes from the FFI context; nothing is allocated and the host never waits for the device -- the scratch the
// kernels need is an extra RESULT buffer whose size the Python side obtains from nb200_sdpa_workspace_bytes at trace
// time (shapes are static under jit).
//
// Operand convention (fixed by nitrix_b200/jax_ffi.py):
//   q (..., H, S, D), k (..., H, T, D), v (..., H, T, Dv): dense row-major, same leading dims (flattened to B here);
//   bias / mask: 4-D (Bb, Hb, Sb, Tb) with every extent either 1 (broadcast) or the full one; a missing bias / mask
//   is passed as a 1-element placeholder together with has_bias / has_mask = false; mask is one byte per element
//   (XLA's PRED), non-zero keeps;  lse (..., H, S) float32.
//
// Build (where jaxlib provides the headers; they are not present in this repository's build image, so this file is
// compiled by no test here):
//   g++ -O2 -std=c++17 -shared -fPIC -I$(python -c "import jax.ffi; print(jax.ffi.include_dir())") -Iinclude \
//       -I/usr/local/cuda/include ffi/nb200_ffi.cc -o libnitrix_b200_ffi.so \
//       -Lnitrix_b200/_lib -lnitrix_b200_attention -Wl,-rpath,'$ORIGIN'
#include <cstdint>
#include <cstring>

#include <cuda_runtime_api.h>

#include "nitrix_b200_attention.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

bool dtype_of(ffi::DataType t, int32_t* out) {
  switch (t) {
    case ffi::DataType::F32: *out = NB200_F32; return true;
    case ffi::DataType::BF16: *out = NB200_BF16; return true;
    case ffi::DataType::F16: *out = NB200_F16; return true;
    default: return false;
  }
}

// Dense row-major strides of a (B, H, rows, cols) view of a buffer whose last three dims are (H, rows, cols).
void dense_strides(int64_t H, int64_t rows, int64_t cols, int64_t stride[4]) {
  stride[3] = 1;
  stride[2] = cols;
  stride[1] = rows * cols;
  stride[0] = H * rows * cols;
}

// Strides of a 4-D bias / mask whose extents are 1 or full: dense over its own extents, 0 on broadcast axes.
ffi::Error own_extent_strides(ffi::AnyBuffer buf, const int64_t full[4], const char* what, int64_t stride[4]) {
  auto dims = buf.dimensions();
  if (dims.size() != 4) return ffi::Error::InvalidArgument(std::string(what) + " must be 4-D (Bb, Hb, Sb, Tb)");
  int64_t dense = 1;
  for (int a = 3; a >= 0; --a) {
    if (dims[a] != 1 && dims[a] != full[a])
      return ffi::Error::InvalidArgument(std::string(what) + " extents must be 1 or the full (B, H, S, T) extent");
    stride[a] = (dims[a] == 1 && full[a] != 1) ? 0 : dense;
    dense *= dims[a];
  }
  return ffi::Error::Success();
}

// Fills the part of the params that forward and backward share.
ffi::Error fill_common(nb200_sdpa_params* p, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer bias,
                       ffi::AnyBuffer mask, bool has_bias, bool has_mask, float scale, bool causal) {
  std::memset(p, 0, sizeof(*p));
  p->struct_size = sizeof(*p);
  if (!dtype_of(q.element_type(), &p->dtype) || q.element_type() != k.element_type() ||
      q.element_type() != v.element_type())
    return ffi::Error::InvalidArgument("q, k, v must share one of the dtypes float32, bfloat16, float16");
  auto qd = q.dimensions(), kd = k.dimensions(), vd = v.dimensions();
  const size_t r = qd.size();
  if (r < 3 || kd.size() != r || vd.size() != r) return ffi::Error::InvalidArgument("q, k, v must be (..., h, s, d)");
  int64_t B = 1;
  for (size_t i = 0; i + 3 < r; ++i) {
    if (kd[i] != qd[i] || vd[i] != qd[i]) return ffi::Error::InvalidArgument("leading dims of q, k, v differ");
    B *= qd[i];
  }
  const int64_t H = qd[r - 3], S = qd[r - 2], D = qd[r - 1], T = kd[r - 2], Dv = vd[r - 1];
  if (kd[r - 3] != H || vd[r - 3] != H || kd[r - 1] != D || vd[r - 2] != T)
    return ffi::Error::InvalidArgument("q, k, v head counts, head dims or key lengths do not agree");
  p->B = int32_t(B); p->H = int32_t(H); p->S = int32_t(S); p->T = int32_t(T); p->D = int32_t(D); p->Dv = int32_t(Dv);
  p->q = q.untyped_data(); p->k = k.untyped_data(); p->v = v.untyped_data();
  dense_strides(H, S, D, p->q_stride);
  dense_strides(H, T, D, p->k_stride);
  dense_strides(H, T, Dv, p->v_stride);
  dense_strides(H, S, Dv, p->out_stride);
  const int64_t full[4] = {B, H, S, T};
  if (has_bias) {
    if (!dtype_of(bias.element_type(), &p->bias_dtype)) return ffi::Error::InvalidArgument("bias dtype is not supported");
    if (auto e = own_extent_strides(bias, full, "bias", p->bias_stride); e.failure()) return e;
    p->bias = bias.untyped_data();
  }
  if (has_mask) {
    if (mask.element_type() != ffi::DataType::PRED && mask.element_type() != ffi::DataType::U8)
      return ffi::Error::InvalidArgument("mask must be bool or uint8");
    if (auto e = own_extent_strides(mask, full, "mask", p->mask_stride); e.failure()) return e;
    p->mask = static_cast<const uint8_t*>(mask.untyped_data());
  }
  p->scale = scale;
  p->causal = causal ? 1 : 0;
  p->kernel = NB200_KERNEL_AUTO;
  p->bh_begin = 0;
  p->bh_end = int32_t(B * H);
  return ffi::Error::Success();
}

ffi::Error status_to_error(int rc) {
  if (rc == NB200_OK) return ffi::Error::Success();
  if (rc == NB200_ERR_INVALID || rc == NB200_ERR_UNSUPPORTED || rc == NB200_ERR_ALIGNMENT)
    return ffi::Error::InvalidArgument(nb200_last_error());
  return ffi::Error::Internal(nb200_last_error());
}

ffi::Error SdpaFwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer bias,
                   ffi::AnyBuffer mask, float scale, bool causal, bool has_bias, bool has_mask,
                   ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> lse,
                   ffi::Result<ffi::AnyBuffer> scratch) {
  nb200_sdpa_params p;
  if (auto e = fill_common(&p, q, k, v, bias, mask, has_bias, has_mask, scale, causal); e.failure()) return e;
  if (lse->element_type() != ffi::DataType::F32) return ffi::Error::InvalidArgument("lse must be float32");
  p.out = out->untyped_data();
  p.lse = static_cast<float*>(lse->untyped_data());
  p.workspace = scratch->untyped_data();
  p.workspace_bytes = scratch->size_bytes();
  return status_to_error(nb200_sdpa_fwd(&p, stream));
}

ffi::Error SdpaBwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer bias,
                   ffi::AnyBuffer mask, ffi::AnyBuffer out, ffi::AnyBuffer lse, ffi::AnyBuffer dout, float scale,
                   bool causal, bool has_bias, bool has_mask, bool want_dbias, ffi::Result<ffi::AnyBuffer> dq,
                   ffi::Result<ffi::AnyBuffer> dk, ffi::Result<ffi::AnyBuffer> dv, ffi::Result<ffi::AnyBuffer> dbias,
                   ffi::Result<ffi::AnyBuffer> scratch) {
  nb200_sdpa_params p;
  if (auto e = fill_common(&p, q, k, v, bias, mask, has_bias, has_mask, scale, causal); e.failure()) return e;
  if (lse.element_type() != ffi::DataType::F32) return ffi::Error::InvalidArgument("lse must be float32");
  if (want_dbias && !has_bias) return ffi::Error::InvalidArgument("want_dbias without a bias");
  p.out = const_cast<void*>(out.untyped_data());                     // read only by the backward
  p.lse = static_cast<float*>(const_cast<void*>(lse.untyped_data()));
  p.dout = dout.untyped_data();
  p.dq = dq->untyped_data();
  p.dk = dk->untyped_data();
  p.dv = dv->untyped_data();
  std::memcpy(p.dout_stride, p.out_stride, sizeof(p.out_stride));
  std::memcpy(p.dq_stride, p.q_stride, sizeof(p.q_stride));
  std::memcpy(p.dk_stride, p.k_stride, sizeof(p.k_stride));
  std::memcpy(p.dv_stride, p.v_stride, sizeof(p.v_stride));
  if (want_dbias) {
    // dbias has the bias' own 4-D shape (broadcast axes already summed) and dtype: dense strides over that shape
    auto bd = bias.dimensions();
    p.dbias = dbias->untyped_data();
    p.want_dbias = 1;
    int64_t dense = 1;
    for (int a = 3; a >= 0; --a) { p.dbias_stride[a] = dense; dense *= bd[a]; }
  }
  p.workspace = scratch->untyped_data();
  p.workspace_bytes = scratch->size_bytes();
  return status_to_error(nb200_sdpa_bwd(&p, stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(nb200_sdpa_fwd_ffi, SdpaFwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // bias (placeholder when has_bias is false)
                                  .Arg<ffi::AnyBuffer>()   // mask (placeholder when has_mask is false)
                                  .Attr<float>("scale")
                                  .Attr<bool>("causal")
                                  .Attr<bool>("has_bias")
                                  .Attr<bool>("has_mask")
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Ret<ffi::AnyBuffer>()   // lse
                                  .Ret<ffi::AnyBuffer>()); // scratch

XLA_FFI_DEFINE_HANDLER_SYMBOL(nb200_sdpa_bwd_ffi, SdpaBwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // bias
                                  .Arg<ffi::AnyBuffer>()   // mask
                                  .Arg<ffi::AnyBuffer>()   // out
                                  .Arg<ffi::AnyBuffer>()   // lse
                                  .Arg<ffi::AnyBuffer>()   // dout
                                  .Attr<float>("scale")
                                  .Attr<bool>("causal")
                                  .Attr<bool>("has_bias")
                                  .Attr<bool>("has_mask")
                                  .Attr<bool>("want_dbias")
                                  .Ret<ffi::AnyBuffer>()   // dq
                                  .Ret<ffi::AnyBuffer>()   // dk
                                  .Ret<ffi::AnyBuffer>()   // dv
                                  .Ret<ffi::AnyBuffer>()   // dbias (1 element when want_dbias is false)
                                  .Ret<ffi::AnyBuffer>()); // scratch
