// RMS normalisation of q and k over the head dim (the `qk_norm=True` pre-op of attention) and its gradient, each as
// ONE launch for both tensors.
//
// The reference applies this outside its fused kernels, as separate element-wise XLA ops whose VJP autodiff chains
// onto the kernels' (reference src/nitrix/nn/attention/__init__.py:184-197; the op itself:
// src/nitrix/nn/attention/_reference.py:52-77, y = x * rsqrt(mean(x^2) + 1e-6), no learnable scale, fp32
// accumulation).  Here the pre-op keeps that place in the call sequence -- so the attention kernels and their
// gradients are untouched -- but costs one read and one write per tensor instead of a chain of element-wise passes:
// one warp per row, 16-byte loads, the row held in registers between the reduction and the scaling.
//
//   forward   y = x r,                       r = rsqrt(mean(x^2) + eps)
//   gradient  dx = r (g - y mean(g y))       (exact, eps included: dr/dx_i = -r^3 x_i / D)
#include <math.h>

#include "sdpa_common.cuh"

namespace nb200 {
namespace {

constexpr float kEps = 1e-6f;

struct NormTensor {
  const void* x;      // [b][h][n][D], last dim contiguous
  const void* g;      // gradient pass: dL/dy, dense [rows][D]
  void* y;            // forward: y; gradient pass: dx -- dense [rows][D]
  int64_t xs[3];      // element strides of x over (b, h, n)
  int H, N;
  int64_t rows;       // B * H * N
};

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row; a lane holds kPer consecutive-by-32 chunks of kVec elements (16 bytes each).  D <= 32 * kVec * kPer.
template <typename T, bool kGrad>
__global__ void __launch_bounds__(256) qk_rms_norm_kernel(NormTensor a, NormTensor b, int D) {
  constexpr int kVec = 16 / int(sizeof(T));
  constexpr int kPer = sizeof(T) == 4 ? 2 : 1;     // head dims up to 256
  const int lane = threadIdx.x & 31;
  const int64_t row_all = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const bool second = row_all >= a.rows;
  const NormTensor& t = second ? b : a;
  const int64_t row = second ? row_all - a.rows : row_all;
  if (row >= t.rows) return;
  const int64_t n = row % t.N, bh = row / t.N;
  const int64_t h = bh % t.H, bb = bh / t.H;
  const T* x = reinterpret_cast<const T*>(t.x) + bb * t.xs[0] + h * t.xs[1] + n * t.xs[2];
  float xv[kPer][kVec], gv[kPer][kVec];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < kPer; ++p) {
    const int c0 = (p * 32 + lane) * kVec;
    if (c0 < D) {
      const uint4 w = *reinterpret_cast<const uint4*>(x + c0);
      const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        xv[p][i] = to_f<T>(e[i]);
        ss = fmaf(xv[p][i], xv[p][i], ss);
      }
      if constexpr (kGrad) {
        const uint4 wg = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(t.g) + row * D + c0);
        const T* eg = reinterpret_cast<const T*>(&wg);
#pragma unroll
        for (int i = 0; i < kVec; ++i) gv[p][i] = to_f<T>(eg[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kVec; ++i) xv[p][i] = gv[p][i] = 0.f;
    }
  }
  const float r = rsqrtf(warp_sum(ss) / float(D) + kEps);
  float m = 0.f;
  if constexpr (kGrad) {
    float gy = 0.f;
#pragma unroll
    for (int p = 0; p < kPer; ++p)
#pragma unroll
      for (int i = 0; i < kVec; ++i) gy = fmaf(gv[p][i], xv[p][i] * r, gy);
    m = warp_sum(gy) / float(D);
  }
  T* y = reinterpret_cast<T*>(t.y) + row * D;
#pragma unroll
  for (int p = 0; p < kPer; ++p) {
    const int c0 = (p * 32 + lane) * kVec;
    if (c0 < D) {
      uint4 w;
      T* e = reinterpret_cast<T*>(&w);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const float yi = xv[p][i] * r;
        e[i] = from_f<T>(kGrad ? r * (gv[p][i] - yi * m) : yi);
      }
      *reinterpret_cast<uint4*>(y + c0) = w;
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check(const nb200_qk_norm_tensor& t, int D, int dtype, bool grad, const char* name, NormTensor* out) {
  const int esz = dtype == NB200_F32 ? 4 : 2;
  const int vec = 16 / esz;
  if (t.B < 0 || t.H <= 0 || t.N < 0) { set_error("qk_rms_norm: bad extents of %s", name); return NB200_ERR_INVALID; }
  out->rows = int64_t(t.B) * t.H * t.N;
  if (out->rows == 0) return NB200_OK;
  if (!t.x || !t.y || (grad && !t.g)) { set_error("qk_rms_norm: NULL pointer in %s", name); return NB200_ERR_INVALID; }
  if (!aligned16(t.x) || !aligned16(t.y) || (grad && !aligned16(t.g)) || t.xs[0] % vec || t.xs[1] % vec || t.xs[2] % vec) {
    set_error("qk_rms_norm: %s needs 16-byte aligned rows (pointer and strides)", name);
    return NB200_ERR_ALIGNMENT;
  }
  out->x = t.x; out->g = t.g; out->y = t.y;
  for (int i = 0; i < 3; ++i) out->xs[i] = t.xs[i];
  out->H = t.H; out->N = t.N;
  return NB200_OK;
}

template <bool kGrad>
int launch(const nb200_qk_norm_tensor* q, const nb200_qk_norm_tensor* k, int D, int dtype, void* cuda_stream) {
  if (!q || !k) { set_error("qk_rms_norm: NULL tensor description"); return NB200_ERR_INVALID; }
  if (dtype != NB200_F32 && dtype != NB200_BF16 && dtype != NB200_F16) { set_error("qk_rms_norm: bad dtype"); return NB200_ERR_INVALID; }
  const int vec = dtype == NB200_F32 ? 4 : 8;
  if (D <= 0 || D > 256 || D % vec) {
    set_error("qk_rms_norm: head dim %d must be a multiple of %d and at most 256", D, vec);
    return NB200_ERR_UNSUPPORTED;
  }
  NormTensor a{}, b{};
  if (int rc = check(*q, D, dtype, kGrad, "q", &a)) return rc;
  if (int rc = check(*k, D, dtype, kGrad, "k", &b)) return rc;
  const int64_t rows = a.rows + b.rows;
  if (rows == 0) return NB200_OK;
  const int64_t blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffff) { set_error("qk_rms_norm: too many rows"); return NB200_ERR_UNSUPPORTED; }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  prof_call_begin(st);
  if (dtype == NB200_F32) qk_rms_norm_kernel<float, kGrad><<<unsigned(blocks), 256, 0, st>>>(a, b, D);
  else if (dtype == NB200_BF16) qk_rms_norm_kernel<__nv_bfloat16, kGrad><<<unsigned(blocks), 256, 0, st>>>(a, b, D);
  else qk_rms_norm_kernel<__half, kGrad><<<unsigned(blocks), 256, 0, st>>>(a, b, D);
  count_launch();
  return check_launch(kGrad ? "qk_rms_norm_grad_kernel" : "qk_rms_norm_kernel");
}

}  // namespace
}  // namespace nb200

extern "C" NB200_API int nb200_qk_rms_norm(const nb200_qk_norm_tensor* q, const nb200_qk_norm_tensor* k, int head_dim,
                                           int dtype, void* cuda_stream) {
  return nb200::launch<false>(q, k, head_dim, dtype, cuda_stream);
}

extern "C" NB200_API int nb200_qk_rms_norm_grad(const nb200_qk_norm_tensor* q, const nb200_qk_norm_tensor* k, int head_dim,
                                                int dtype, void* cuda_stream) {
  return nb200::launch<true>(q, k, head_dim, dtype, cuda_stream);
}
