// XLA FFI handlers over the C ABI of the fused LayerNorm (include/nitrix_b200_norm.h).
//
// Two custom-call handlers, `nb200_layer_norm_fwd_ffi` and `nb200_layer_norm_bwd_ffi`, registered from Python with
// jax.ffi.register_ffi_target(..., platform="CUDA") and invoked through jax.ffi.ffi_call
// (nitrix_b200/jax_norm_ffi.py).  They stand where the reference's dispatcher calls its fused-norm module,
// `layer_norm_pallas(x, weight, bias, eps=..., out_scale=...)` (reference src/nitrix/nn/norm/__init__.py:57-95;
// src/nitrix/_kernels/cuda/norm.py:51-, which there declines every shape).
//
// Contract with XLA: every buffer is borrowed, the stream comes from the FFI context, nothing is allocated and the
// host never waits for the device; the backward's column-sum scratch is an extra RESULT buffer whose size the
// Python side obtains from nb200_layer_norm_workspace_bytes at trace time (shapes are static under jit).
//
// Operand convention (fixed by nitrix_b200/jax_norm_ffi.py): x, y, dy, dx are dense row-major (..., c), every
// leading axis folded into rows here; weight / bias / dweight / dbias are (c,) of x's dtype, a missing one is passed
// as a 1-element placeholder together with has_weight / has_bias = false; mean and rstd are (rows,) float32.
//
// Build (where jaxlib provides the headers; they are not present in this repository's build image, so this file is
// compiled by no test here):
//   g++ -O2 -std=c++17 -shared -fPIC -I$(python -c "import jax.ffi; print(jax.ffi.include_dir())") -Iinclude \
//       -I/usr/local/cuda/include ffi/nb200_norm_ffi.cc -o libnitrix_b200_norm_ffi.so \
//       -Lnitrix_b200/_lib -lnitrix_b200_attention -Wl,-rpath,'$ORIGIN'
#include <cstdint>
#include <string>

#include <cuda_runtime_api.h>

#include "nitrix_b200_norm.h"
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

ffi::Error status_to_error(int rc) {
  if (rc == NB200_OK) return ffi::Error::Success();
  if (rc == NB200_ERR_INVALID || rc == NB200_ERR_UNSUPPORTED || rc == NB200_ERR_ALIGNMENT)
    return ffi::Error::InvalidArgument(nb200_last_error());
  return ffi::Error::Internal(nb200_last_error());
}

// rows x channels of a dense (..., c) buffer, and the dtype code
ffi::Error fill_common(nb200_layer_norm_params* p, ffi::AnyBuffer x, float eps, float out_scale) {
  *p = nb200_layer_norm_params{};
  p->struct_size = sizeof(nb200_layer_norm_params);
  auto dims = x.dimensions();
  if (dims.size() < 1) return ffi::Error::InvalidArgument("x must have a trailing channel axis");
  if (!dtype_of(x.element_type(), &p->dtype)) return ffi::Error::InvalidArgument("x must be float32, bfloat16 or float16");
  int64_t rows = 1;
  for (size_t a = 0; a + 1 < dims.size(); ++a) rows *= dims[a];
  p->rows = rows;
  p->channels = static_cast<int32_t>(dims.back());
  p->x = x.untyped_data();
  p->eps = eps;
  p->out_scale = out_scale;
  return ffi::Error::Success();
}

ffi::Error check_vector(ffi::AnyBuffer v, const nb200_layer_norm_params& p, const char* what) {
  auto dims = v.dimensions();
  int32_t dt = -1;
  if (dims.size() != 1 || dims[0] != p.channels || !dtype_of(v.element_type(), &dt) || dt != p.dtype)
    return ffi::Error::InvalidArgument(std::string(what) + " must have shape (c,) and x's dtype");
  return ffi::Error::Success();
}

ffi::Error LayerNormFwd(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer weight, ffi::AnyBuffer bias, float eps,
                        float out_scale, bool has_weight, bool has_bias, ffi::Result<ffi::AnyBuffer> y,
                        ffi::Result<ffi::AnyBuffer> mean, ffi::Result<ffi::AnyBuffer> rstd) {
  nb200_layer_norm_params p;
  if (auto e = fill_common(&p, x, eps, out_scale); e.failure()) return e;
  if (has_weight) {
    if (auto e = check_vector(weight, p, "weight"); e.failure()) return e;
    p.weight = weight.untyped_data();
  }
  if (has_bias) {
    if (auto e = check_vector(bias, p, "bias"); e.failure()) return e;
    p.bias = bias.untyped_data();
  }
  if (mean->element_type() != ffi::DataType::F32 || rstd->element_type() != ffi::DataType::F32)
    return ffi::Error::InvalidArgument("mean and rstd must be float32");
  p.y = y->untyped_data();
  p.mean = static_cast<float*>(mean->untyped_data());
  p.rstd = static_cast<float*>(rstd->untyped_data());
  return status_to_error(nb200_layer_norm_fwd(&p, stream));
}

ffi::Error LayerNormBwd(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer weight, ffi::AnyBuffer mean,
                        ffi::AnyBuffer rstd, ffi::AnyBuffer dy, float eps, float out_scale, bool has_weight,
                        bool want_dweight, bool want_dbias, ffi::Result<ffi::AnyBuffer> dx,
                        ffi::Result<ffi::AnyBuffer> dweight, ffi::Result<ffi::AnyBuffer> dbias,
                        ffi::Result<ffi::AnyBuffer> scratch) {
  nb200_layer_norm_params p;
  if (auto e = fill_common(&p, x, eps, out_scale); e.failure()) return e;
  if (has_weight) {
    if (auto e = check_vector(weight, p, "weight"); e.failure()) return e;
    p.weight = weight.untyped_data();
  }
  if (mean.element_type() != ffi::DataType::F32 || rstd.element_type() != ffi::DataType::F32)
    return ffi::Error::InvalidArgument("mean and rstd must be float32");
  p.mean = static_cast<float*>(mean.untyped_data());
  p.rstd = static_cast<float*>(rstd.untyped_data());
  p.dy = dy.untyped_data();
  p.dx = dx->untyped_data();
  if (want_dweight) p.dweight = dweight->untyped_data();   // (1-element placeholders otherwise)
  if (want_dbias) p.dbias = dbias->untyped_data();
  p.workspace = scratch->untyped_data();
  p.workspace_bytes = scratch->size_bytes();
  return status_to_error(nb200_layer_norm_bwd(&p, stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(nb200_layer_norm_fwd_ffi, LayerNormFwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // x
                                  .Arg<ffi::AnyBuffer>()   // weight (placeholder when has_weight is false)
                                  .Arg<ffi::AnyBuffer>()   // bias (placeholder when has_bias is false)
                                  .Attr<float>("eps")
                                  .Attr<float>("out_scale")
                                  .Attr<bool>("has_weight")
                                  .Attr<bool>("has_bias")
                                  .Ret<ffi::AnyBuffer>()   // y
                                  .Ret<ffi::AnyBuffer>()   // mean
                                  .Ret<ffi::AnyBuffer>()); // rstd

XLA_FFI_DEFINE_HANDLER_SYMBOL(nb200_layer_norm_bwd_ffi, LayerNormBwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // x
                                  .Arg<ffi::AnyBuffer>()   // weight
                                  .Arg<ffi::AnyBuffer>()   // mean
                                  .Arg<ffi::AnyBuffer>()   // rstd
                                  .Arg<ffi::AnyBuffer>()   // dy
                                  .Attr<float>("eps")
                                  .Attr<float>("out_scale")
                                  .Attr<bool>("has_weight")
                                  .Attr<bool>("want_dweight")
                                  .Attr<bool>("want_dbias")
                                  .Ret<ffi::AnyBuffer>()   // dx
                                  .Ret<ffi::AnyBuffer>()   // dweight (1 element when want_dweight is false)
                                  .Ret<ffi::AnyBuffer>()   // dbias (1 element when want_dbias is false)
                                  .Ret<ffi::AnyBuffer>()); // scratch
