// XLA FFI handlers over the C ABI of the selective scan (include/nitrix_b200_scan.h).
//
// Two custom-call handlers, `nb200_selective_scan_fwd_ffi` and `nb200_selective_scan_bwd_ffi`, registered from Python
// with jax.ffi.register_ffi_target(..., platform="CUDA") and invoked through jax.ffi.ffi_call
// (nitrix_b200/jax_scan_ffi.py).  They stand where the reference's dispatcher calls its fused scan module,
// `_selective_scan_pallas(x, delta, A, B, C, D)` (reference src/nitrix/nn/ssm/__init__.py:80-125;
// src/nitrix/_kernels/cuda/selective_scan.py:4-36).
//
// Contract with XLA: every buffer is borrowed, the stream comes from the FFI context, nothing is allocated and the
// host never waits for the device; the forward's checkpoints and the backward's accumulators are extra RESULT
// buffers whose sizes the Python side obtains from nb200_selective_scan_checkpoint_bytes / _workspace_bytes at trace
// time (shapes are static under jit).
//
// Operand convention (fixed by nitrix_b200/jax_scan_ffi.py): x, delta, y, dy, dx, ddelta dense (batch, l, d) with every
// leading axis folded into batch; A, dA (d, n); B, C, dB, dC (batch, l, n); D, dD (d,), a missing D is passed as a
// 1-element placeholder together with has_d = false; one dtype for all; checkpoints float32.
//
// Build (where jaxlib provides the headers; they are not present in this repository's build image, so this file is
// compiled by no test here):
//   g++ -O2 -std=c++17 -shared -fPIC -I$(python -c "import jax.ffi; print(jax.ffi.include_dir())") -Iinclude \
//       -I/usr/local/cuda/include ffi/nb200_scan_ffi.cc -o libnitrix_b200_scan_ffi.so \
//       -Lnitrix_b200/_lib -lnitrix_b200_attention -Wl,-rpath,'$ORIGIN'
#include <cstdint>
#include <string>

#include <cuda_runtime_api.h>

#include "nitrix_b200_scan.h"
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

ffi::Error fill_common(nb200_selective_scan_params* p, ffi::AnyBuffer x, ffi::AnyBuffer delta, ffi::AnyBuffer A,
                       ffi::AnyBuffer B, ffi::AnyBuffer C, ffi::AnyBuffer D, bool has_d) {
  *p = nb200_selective_scan_params{};
  p->struct_size = sizeof(nb200_selective_scan_params);
  auto xd = x.dimensions();
  auto ad = A.dimensions();
  auto bd = B.dimensions();
  if (xd.size() != 3 || ad.size() != 2 || bd.size() != 3)
    return ffi::Error::InvalidArgument("x must be (batch, l, d), A (d, n), B and C (batch, l, n)");
  if (!dtype_of(x.element_type(), &p->dtype)) return ffi::Error::InvalidArgument("x must be float32, bfloat16 or float16");
  for (ffi::AnyBuffer* o : {&delta, &A, &B, &C})
    if (o->element_type() != x.element_type()) return ffi::Error::InvalidArgument("every operand must have x's dtype");
  if (ad[0] != xd[2] || bd[0] != xd[0] || bd[1] != xd[1] || bd[2] != ad[1] || delta.dimensions() != xd ||
      C.dimensions() != bd)
    return ffi::Error::InvalidArgument("operand shapes do not match (batch, l, d) / (d, n) / (batch, l, n)");
  p->batch = static_cast<int32_t>(xd[0]);
  p->length = static_cast<int32_t>(xd[1]);
  p->channels = static_cast<int32_t>(xd[2]);
  p->states = static_cast<int32_t>(ad[1]);
  p->x = x.untyped_data();
  p->delta = delta.untyped_data();
  p->A = A.untyped_data();
  p->B = B.untyped_data();
  p->C = C.untyped_data();
  if (has_d) {
    if (D.dimensions().size() != 1 || D.dimensions()[0] != xd[2] || D.element_type() != x.element_type())
      return ffi::Error::InvalidArgument("D must have shape (d,) and x's dtype");
    p->D = D.untyped_data();
  }
  return ffi::Error::Success();
}

ffi::Error ScanFwd(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer delta, ffi::AnyBuffer A, ffi::AnyBuffer B,
                   ffi::AnyBuffer C, ffi::AnyBuffer D, bool has_d, ffi::Result<ffi::AnyBuffer> y,
                   ffi::Result<ffi::AnyBuffer> checkpoints) {
  nb200_selective_scan_params p;
  if (auto e = fill_common(&p, x, delta, A, B, C, D, has_d); e.failure()) return e;
  if (checkpoints->element_type() != ffi::DataType::F32) return ffi::Error::InvalidArgument("checkpoints must be float32");
  p.y = y->untyped_data();
  p.checkpoints = static_cast<float*>(checkpoints->untyped_data());
  return status_to_error(nb200_selective_scan_fwd(&p, stream));
}

ffi::Error ScanBwd(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer delta, ffi::AnyBuffer A, ffi::AnyBuffer B,
                   ffi::AnyBuffer C, ffi::AnyBuffer D, ffi::AnyBuffer checkpoints, ffi::AnyBuffer dy, bool has_d,
                   ffi::Result<ffi::AnyBuffer> dx, ffi::Result<ffi::AnyBuffer> ddelta, ffi::Result<ffi::AnyBuffer> dA,
                   ffi::Result<ffi::AnyBuffer> dB, ffi::Result<ffi::AnyBuffer> dC, ffi::Result<ffi::AnyBuffer> dD,
                   ffi::Result<ffi::AnyBuffer> scratch) {
  nb200_selective_scan_params p;
  if (auto e = fill_common(&p, x, delta, A, B, C, D, has_d); e.failure()) return e;
  if (checkpoints.element_type() != ffi::DataType::F32) return ffi::Error::InvalidArgument("checkpoints must be float32");
  p.checkpoints = static_cast<float*>(checkpoints.untyped_data());
  p.dy = dy.untyped_data();
  p.dx = dx->untyped_data();
  p.ddelta = ddelta->untyped_data();
  p.dA = dA->untyped_data();
  p.dB = dB->untyped_data();
  p.dC = dC->untyped_data();
  if (has_d) p.dD = dD->untyped_data();   // (a 1-element placeholder otherwise)
  p.workspace = scratch->untyped_data();
  p.workspace_bytes = scratch->size_bytes();
  return status_to_error(nb200_selective_scan_bwd(&p, stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(nb200_selective_scan_fwd_ffi, ScanFwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // x
                                  .Arg<ffi::AnyBuffer>()   // delta
                                  .Arg<ffi::AnyBuffer>()   // A
                                  .Arg<ffi::AnyBuffer>()   // B
                                  .Arg<ffi::AnyBuffer>()   // C
                                  .Arg<ffi::AnyBuffer>()   // D (placeholder when has_d is false)
                                  .Attr<bool>("has_d")
                                  .Ret<ffi::AnyBuffer>()   // y
                                  .Ret<ffi::AnyBuffer>()); // checkpoints

XLA_FFI_DEFINE_HANDLER_SYMBOL(nb200_selective_scan_bwd_ffi, ScanBwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // x
                                  .Arg<ffi::AnyBuffer>()   // delta
                                  .Arg<ffi::AnyBuffer>()   // A
                                  .Arg<ffi::AnyBuffer>()   // B
                                  .Arg<ffi::AnyBuffer>()   // C
                                  .Arg<ffi::AnyBuffer>()   // D
                                  .Arg<ffi::AnyBuffer>()   // checkpoints
                                  .Arg<ffi::AnyBuffer>()   // dy
                                  .Attr<bool>("has_d")
                                  .Ret<ffi::AnyBuffer>()   // dx
                                  .Ret<ffi::AnyBuffer>()   // ddelta
                                  .Ret<ffi::AnyBuffer>()   // dA
                                  .Ret<ffi::AnyBuffer>()   // dB
                                  .Ret<ffi::AnyBuffer>()   // dC
                                  .Ret<ffi::AnyBuffer>()   // dD (1 element when has_d is false)
                                  .Ret<ffi::AnyBuffer>()); // scratch
