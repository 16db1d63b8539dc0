// LayerNorm over the trailing axis, forward and backward -- the sibling op of the attention path behind the same
// library (reference src/nitrix/nn/norm/__init__.py:110-176 is the dispatcher, src/nitrix/nn/norm/_reference.py:44-110
// the recipe: biased variance, rsqrt(var + eps), optional per-channel affine, then the constant `out_scale`; a 16-bit
// input is upcast to fp32 for the reductions and the affine transform and the result cast back).
//
//   forward   xhat = (x - mean) rstd,  y = out_scale (xhat w + b);  mean and rstd (fp32 per row) are kept for the
//             backward when the caller passes buffers for them
//   backward  gy = out_scale dy,  dxhat = gy w,  dx = rstd (dxhat - mean(dxhat) - xhat mean(dxhat xhat)),
//             dw = sum_rows gy xhat,  db = sum_rows gy
//
// Rows that are a multiple of 16 bytes (<= 8192 channels, aligned pointers) take the vector kernels below; the rest
// the scalar ones at the end.  The op is bound by HBM traffic (x once in, y once out; the backward x and dy in, dx
// out), so a row is read ONCE with 16-byte loads and held in registers between the reductions and the write: by one
// warp (rows of up to 32 x 16 B x 8) or by one 256-thread CTA (longer rows).  The variance is taken about the mean
// (two passes over the registers, as the reference's `var` does), not as E[x^2] - mean^2.  dw / db: every CTA walks
// rows in a grid-stride loop, keeps its column sums in shared memory, leaves one partial row per CTA in a
// workspace, and a second kernel adds the partials in a fixed order -- deterministic, no atomics.
#include <math.h>

#include "nitrix_b200_norm.h"
#include "sdpa_common.cuh"

namespace nb200 {
namespace {

constexpr int kThreads = 256;

struct LnArgs {
  const void* x;
  const void* w;
  const void* b;
  void* y;
  float* mean;
  float* rstd;
  const void* dy;
  void* dx;
  float* part;   // [2][grid][C] partial dw, db
  int64_t rows;
  int C;
  float eps, out_scale;
};

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the threads that share a row: the warp, or the whole CTA through shared memory.  `red` holds eight
// floats per use; consecutive uses alternate between buffers (the callers pass red + 8 k), so that ONE barrier per
// reduction is enough: a buffer is rewritten only after a later barrier has shown that every thread has read it.
template <bool kCta>
__device__ __forceinline__ float row_sum(float v, float* red) {
  v = warp_sum_f(v);
  if constexpr (kCta) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    v = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) v += red[i];
  }
  return v;
}
// two sums at once (red: 16 floats per use)
template <bool kCta>
__device__ __forceinline__ float2 row_sum2(float a, float b, float* red) {
  a = warp_sum_f(a);
  b = warp_sum_f(b);
  if constexpr (kCta) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
      red[warp] = a;
      red[8 + warp] = b;
    }
    __syncthreads();
    a = b = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) {
      a += red[i];
      b += red[8 + i];
    }
  }
  return make_float2(a, b);
}

template <typename T, int kVec>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[kVec]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
  for (int i = 0; i < kVec; ++i) out[i] = to_f32<T>(e[i]);
}
// The same as pairs: the arithmetic below runs on the packed fp32x2 pipe (one instruction per two elements; each
// lane rounds as the scalar instruction would, so results do not change).  At 16-bit widths the kernels are bound
// by instruction issue as much as by memory.
template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack_pair<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float2 v);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float2 v) {
  const __nv_bfloat162 r = __floats2bfloat162_rn(v.x, v.y);
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float2 v) {
  const __half2 r = __floats2half2_rn(v.x, v.y);
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <typename T, int kVec>
__device__ __forceinline__ void load_pairs(const T* p, float2 (&out)[kVec / 2]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  if constexpr (sizeof(T) == 4) {
    out[0] = make_float2(__uint_as_float(w.x), __uint_as_float(w.y));
    out[1] = make_float2(__uint_as_float(w.z), __uint_as_float(w.w));
  } else {
    out[0] = unpack_pair<T>(w.x);
    out[1] = unpack_pair<T>(w.y);
    out[2] = unpack_pair<T>(w.z);
    out[3] = unpack_pair<T>(w.w);
  }
}
template <typename T, int kVec>
__device__ __forceinline__ void store_pairs(T* p, const float2 (&v)[kVec / 2]) {
  uint4 w;
  if constexpr (sizeof(T) == 4) {
    w = make_uint4(__float_as_uint(v[0].x), __float_as_uint(v[0].y), __float_as_uint(v[1].x), __float_as_uint(v[1].y));
  } else {
    w = make_uint4(pack_pair<T>(v[0]), pack_pair<T>(v[1]), pack_pair<T>(v[2]), pack_pair<T>(v[3]));
  }
  *reinterpret_cast<uint4*>(p) = w;
}
template <typename T, int kVec>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[kVec]) {
  uint4 w;
  T* e = reinterpret_cast<T*>(&w);
#pragma unroll
  for (int i = 0; i < kVec; ++i) e[i] = from_f32<T>(v[i]);
  *reinterpret_cast<uint4*>(p) = w;
}

// A row is split over kCta ? 256 : 32 threads; a thread holds kPer chunks of kVec = 16 / sizeof(T) elements, chunk p
// at column (p * threads + thread) * kVec.
template <typename T, int kPer, bool kCta>
__global__ void __launch_bounds__(kThreads, kPer <= 4 ? 4 : 2) ln_fwd_kernel(LnArgs a) {
  constexpr int kVec = 16 / int(sizeof(T));
  constexpr int kTpr = kCta ? kThreads : 32;
  __shared__ float red[2 * (kThreads / 32)];
  const int tin = kCta ? threadIdx.x : (threadIdx.x & 31);
  const int64_t row = kCta ? int64_t(blockIdx.x) : int64_t(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
  if (row >= a.rows) return;   // (a whole CTA, or a whole warp of a warp-per-row CTA, which never meets a barrier)
  const T* x = reinterpret_cast<const T*>(a.x) + row * a.C;
  constexpr int kPairs = kVec / 2;
  float2 xv[kPer][kPairs];
  float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int p = 0; p < kPer; ++p) {
    const int c0 = (p * kTpr + tin) * kVec;
    if (c0 < a.C) {
      load_pairs<T, kVec>(x + c0, xv[p]);
#pragma unroll
      for (int i = 0; i < kPairs; ++i) s2 = __fadd2_rn(s2, xv[p][i]);
    }
  }
  const float mean = row_sum<kCta>(s2.x + s2.y, red) / float(a.C);
  const float2 nmean = make_float2(-mean, -mean);
  float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int p = 0; p < kPer; ++p)
    if ((p * kTpr + tin) * kVec < a.C) {
#pragma unroll
      for (int i = 0; i < kPairs; ++i) {
        xv[p][i] = __fadd2_rn(xv[p][i], nmean);      // x - mean, kept
        q2 = __ffma2_rn(xv[p][i], xv[p][i], q2);
      }
    }
  const float rstd = rsqrtf(row_sum<kCta>(q2.x + q2.y, red + 8) / float(a.C) + a.eps);
  if (tin == 0) {
    if (a.mean) a.mean[row] = mean;
    if (a.rstd) a.rstd[row] = rstd;
  }
  T* y = reinterpret_cast<T*>(a.y) + row * a.C;
  const T* w = reinterpret_cast<const T*>(a.w);
  const T* b = reinterpret_cast<const T*>(a.b);
  const float2 rstd2 = make_float2(rstd, rstd), os2 = make_float2(a.out_scale, a.out_scale);
#pragma unroll
  for (int p = 0; p < kPer; ++p) {
    const int c0 = (p * kTpr + tin) * kVec;
    if (c0 < a.C) {
      float2 wv[kPairs], bv[kPairs], out[kPairs];
      if (w) load_pairs<T, kVec>(w + c0, wv);
      if (b) load_pairs<T, kVec>(b + c0, bv);
#pragma unroll
      for (int i = 0; i < kPairs; ++i) {
        float2 v = __fmul2_rn(xv[p][i], rstd2);
        if (w) v = __fmul2_rn(v, wv[i]);
        if (b) v = __fadd2_rn(v, bv[i]);
        out[i] = __fmul2_rn(os2, v);
      }
      store_pairs<T, kVec>(y + c0, out);
    }
  }
}

// Backward.  Grid-stride over rows (a warp's or a CTA's).  The column sums of dw, db live in shared memory, every
// thread adding only to its own columns (in registers they cost 2 x kPer x kVec registers and left one CTA per SM).
template <typename T, int kPer, bool kCta>
__global__ void __launch_bounds__(kThreads) ln_bwd_kernel(LnArgs a) {
  constexpr int kVec = 16 / int(sizeof(T));
  constexpr int kTpr = kCta ? kThreads : 32;
  constexpr int kRowsPerCta = kCta ? 1 : kThreads / 32;
  // [2][kRowsPerCta][kPad]: dw sums, then db sums, per row owner.  Column c of an owner sits at slot(c): the two
  // 16-byte halves of a 16-bit thread's chunk go to separate planes, so that the threads of a quarter-warp touch
  // consecutive 16-byte words (bank-conflict free) when they update their sums.
  extern __shared__ __align__(16) float wsum[];
  constexpr int kPad = kPer * kTpr * kVec;
  auto slot4 = [](int p, int i4, int tin_) { return ((p * (kVec / 4) + i4) * kTpr + tin_) * 4; };
  __shared__ float red[4 * (kThreads / 32)];   // two uses of 16 floats, alternating by row
  const int tin = kCta ? threadIdx.x : (threadIdx.x & 31);
  const int sub = kCta ? 0 : (threadIdx.x >> 5);
  int flip = 0;
  const T* w = reinterpret_cast<const T*>(a.w);
  float* sw = wsum + sub * kPad;
  float* sb = wsum + (kRowsPerCta + sub) * kPad;
  const bool sums = a.part != nullptr;
  if (sums) {
#pragma unroll
    for (int p = 0; p < kPer; ++p) {
      const int c0 = (p * kTpr + tin) * kVec;
      if (c0 < a.C) {
#pragma unroll
        for (int i = 0; i < kVec; i += 4) {
          *reinterpret_cast<float4*>(sw + slot4(p, i / 4, tin)) = make_float4(0.f, 0.f, 0.f, 0.f);
          *reinterpret_cast<float4*>(sb + slot4(p, i / 4, tin)) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
  }
  // (in a CTA-per-row kernel every thread of the CTA runs the same number of iterations: the barriers in row_sum match)
  for (int64_t row = int64_t(blockIdx.x) * kRowsPerCta + sub; row < a.rows; row += int64_t(gridDim.x) * kRowsPerCta) {
    const T* x = reinterpret_cast<const T*>(a.x) + row * a.C;
    const T* g = reinterpret_cast<const T*>(a.dy) + row * a.C;
    const float mean = a.mean[row], rstd = a.rstd[row];
    float xh[kPer][kVec], dxh[kPer][kVec];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int p = 0; p < kPer; ++p) {
      const int c0 = (p * kTpr + tin) * kVec;
      if (c0 < a.C) {
        load_vec<T, kVec>(x + c0, xh[p]);
        load_vec<T, kVec>(g + c0, dxh[p]);
      }
    }
#pragma unroll
    for (int p = 0; p < kPer; ++p) {
      const int c0 = (p * kTpr + tin) * kVec;
      if (c0 < a.C) {
        float wv[kVec];
        if (w) load_vec<T, kVec>(w + c0, wv);   // (a few KB that stay in L1)
#pragma unroll
        for (int i = 0; i < kVec; i += 4) {
          float4 aw, ab;
          if (sums) {
            aw = *reinterpret_cast<const float4*>(sw + slot4(p, i / 4, tin));
            ab = *reinterpret_cast<const float4*>(sb + slot4(p, i / 4, tin));
          }
          float* pw = reinterpret_cast<float*>(&aw);
          float* pb = reinterpret_cast<float*>(&ab);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float xhv = (xh[p][i + u] - mean) * rstd;
            const float gy = a.out_scale * dxh[p][i + u];
            pw[u] = fmaf(gy, xhv, pw[u]);
            pb[u] += gy;
            const float d = w ? gy * wv[i + u] : gy;
            xh[p][i + u] = xhv;
            dxh[p][i + u] = d;
            s1 += d;
            s2 = fmaf(d, xhv, s2);
          }
          if (sums) {
            *reinterpret_cast<float4*>(sw + slot4(p, i / 4, tin)) = aw;
            *reinterpret_cast<float4*>(sb + slot4(p, i / 4, tin)) = ab;
          }
        }
      }
    }
    const float2 cs = row_sum2<kCta>(s1, s2, red + 16 * flip);
    flip ^= 1;
    const float c1 = cs.x / float(a.C), c2 = cs.y / float(a.C);
    T* dx = reinterpret_cast<T*>(a.dx) + row * a.C;
#pragma unroll
    for (int p = 0; p < kPer; ++p) {
      const int c0 = (p * kTpr + tin) * kVec;
      if (c0 < a.C) {
        float out[kVec];
#pragma unroll
        for (int i = 0; i < kVec; ++i) out[i] = rstd * (dxh[p][i] - c1 - xh[p][i] * c2);
        store_vec<T, kVec>(dx + c0, out);
      }
    }
  }
  if (!sums) return;
  // this CTA's partial row: the row owners' sums added in owner order
  float* pw = a.part + int64_t(blockIdx.x) * a.C;
  float* pb = a.part + (int64_t(gridDim.x) + blockIdx.x) * a.C;
  __syncthreads();
  for (int c = threadIdx.x; c < a.C; c += kThreads) {
    const int chunk = c / kVec, i = c % kVec;
    const int at = slot4(chunk / kTpr, i / 4, chunk % kTpr) + (i & 3);
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < kRowsPerCta; ++k) {
      tw += wsum[k * kPad + at];
      tb += wsum[(kRowsPerCta + k) * kPad + at];
    }
    pw[c] = tw;
    pb[c] = tb;
  }
}

// dw[c] = sum over the CTAs' partial rows.  A CTA takes 32 columns (lane = column: 128-byte reads); its eight warps
// take the partial rows in turn, four loads in flight each, and their eight sums are added in warp order -- the
// order of the whole sum is fixed by (grid, column) alone.
template <typename T>
__global__ void __launch_bounds__(kThreads) ln_bwd_finish_kernel(const float* part, int grid, int C, T* dw, T* db) {
  __shared__ float sw[kThreads / 32][32], sb[kThreads / 32][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 32 + lane;
  float tw[4] = {0.f, 0.f, 0.f, 0.f}, tb[4] = {0.f, 0.f, 0.f, 0.f};
  if (c < C) {
    const float* pw = part + c;
    const float* pb = part + int64_t(grid) * C + c;
    int k = warp;
    for (; k + 3 * (kThreads / 32) < grid; k += 4 * (kThreads / 32)) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        tw[u] += pw[int64_t(k + u * (kThreads / 32)) * C];
        tb[u] += pb[int64_t(k + u * (kThreads / 32)) * C];
      }
    }
    for (; k < grid; k += kThreads / 32) {
      tw[0] += pw[int64_t(k) * C];
      tb[0] += pb[int64_t(k) * C];
    }
  }
  sw[warp][lane] = (tw[0] + tw[1]) + (tw[2] + tw[3]);
  sb[warp][lane] = (tb[0] + tb[1]) + (tb[2] + tb[3]);
  __syncthreads();
  if (warp == 0 && c < C) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) {
      a += sw[i][lane];
      b += sb[i][lane];
    }
    if (dw) dw[c] = from_f32<T>(a);
    if (db) db[c] = from_f32<T>(b);
  }
}

// Any other row (channels not a multiple of 16 bytes, longer than 8192, unaligned pointers): one CTA per row in
// scalar strided passes; the row is re-read from L1 / L2.  dw / db are added to a zeroed [2][C] fp32 workspace with
// atomics (the one place where the order of a sum is not fixed).
template <typename T>
__global__ void __launch_bounds__(kThreads) ln_fwd_generic_kernel(LnArgs a) {
  __shared__ float red[2 * (kThreads / 32)];
  const int64_t row = blockIdx.x;
  const T* x = reinterpret_cast<const T*>(a.x) + row * a.C;
  float s = 0.f;
  for (int c = threadIdx.x; c < a.C; c += kThreads) s += to_f32<T>(x[c]);
  const float mean = row_sum<true>(s, red) / float(a.C);
  float q = 0.f;
  for (int c = threadIdx.x; c < a.C; c += kThreads) {
    const float d = to_f32<T>(x[c]) - mean;
    q = fmaf(d, d, q);
  }
  const float rstd = rsqrtf(row_sum<true>(q, red + 8) / float(a.C) + a.eps);
  if (threadIdx.x == 0) {
    if (a.mean) a.mean[row] = mean;
    if (a.rstd) a.rstd[row] = rstd;
  }
  T* y = reinterpret_cast<T*>(a.y) + row * a.C;
  const T* w = reinterpret_cast<const T*>(a.w);
  const T* b = reinterpret_cast<const T*>(a.b);
  for (int c = threadIdx.x; c < a.C; c += kThreads) {
    float v = (to_f32<T>(x[c]) - mean) * rstd;
    if (w) v *= to_f32<T>(w[c]);
    if (b) v += to_f32<T>(b[c]);
    y[c] = from_f32<T>(a.out_scale * v);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) ln_bwd_generic_kernel(LnArgs a) {
  __shared__ float red[4 * (kThreads / 32)];
  const T* w = reinterpret_cast<const T*>(a.w);
  int flip = 0;
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const T* x = reinterpret_cast<const T*>(a.x) + row * a.C;
    const T* g = reinterpret_cast<const T*>(a.dy) + row * a.C;
    const float mean = a.mean[row], rstd = a.rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x; c < a.C; c += kThreads) {
      const float xh = (to_f32<T>(x[c]) - mean) * rstd;
      const float dxh = a.out_scale * to_f32<T>(g[c]) * (w ? to_f32<T>(w[c]) : 1.f);
      s1 += dxh;
      s2 = fmaf(dxh, xh, s2);
    }
    const float2 cs = row_sum2<true>(s1, s2, red + 16 * flip);
    flip ^= 1;
    const float c1 = cs.x / float(a.C), c2 = cs.y / float(a.C);
    T* dx = reinterpret_cast<T*>(a.dx) + row * a.C;
    for (int c = threadIdx.x; c < a.C; c += kThreads) {
      const float xh = (to_f32<T>(x[c]) - mean) * rstd;
      const float gy = a.out_scale * to_f32<T>(g[c]);
      const float dxh = gy * (w ? to_f32<T>(w[c]) : 1.f);
      dx[c] = from_f32<T>(rstd * (dxh - c1 - xh * c2));
      if (a.part) {
        atomicAdd(a.part + c, gy * xh);
        atomicAdd(a.part + a.C + c, gy);
      }
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

struct Shape {
  int vec, per;
  bool cta;
};

// the smallest per-thread chunk count that covers a row; the backward keeps twice the registers per chunk
bool pick(int C, int dtype, bool backward, Shape* s) {
  s->vec = dtype == NB200_F32 ? 4 : 8;
  if (C <= 0 || C % s->vec) return false;
  const int max_per = backward ? (dtype == NB200_F32 ? 8 : 4) : 8;
  const int warp_max = backward ? 4 : 8;
  for (int per = 1; per <= warp_max; per *= 2)
    if (C <= 32 * s->vec * per) { s->per = per; s->cta = false; return true; }
  for (int per = 1; per <= max_per; per *= 2)
    if (C <= kThreads * s->vec * per) { s->per = per; s->cta = true; return true; }
  return false;
}

// The backward's grid: as many CTAs as are resident at once (`per_sm` from the occupancy calculator; more CTAs only
// add partial rows to sum), at most one per row unit.  per_sm = 8 bounds it for sizing the workspace.
int bwd_grid(int64_t rows, const Shape& s, int per_sm) {
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int64_t units = s.cta ? rows : (rows + kThreads / 32 - 1) / (kThreads / 32);
  const int64_t cap = int64_t(sms) * per_sm;
  return int(units < cap ? (units > 0 ? units : 1) : cap);
}

int check_common(const nb200_layer_norm_params* p, const char* what) {
  if (!p) { set_error("%s: NULL parameter block", what); return NB200_ERR_INVALID; }
  if (p->struct_size != sizeof(nb200_layer_norm_params)) {
    set_error("%s: ABI mismatch: struct_size %zu, library expects %zu", what, size_t(p->struct_size),
              sizeof(nb200_layer_norm_params));
    return NB200_ERR_INVALID;
  }
  if (p->dtype != NB200_F32 && p->dtype != NB200_BF16 && p->dtype != NB200_F16) { set_error("%s: bad dtype", what); return NB200_ERR_INVALID; }
  if (p->rows < 0 || p->channels <= 0) { set_error("%s: bad extents", what); return NB200_ERR_INVALID; }
  return NB200_OK;
}

template <typename T, bool kBwd, typename F>
int dispatch(const Shape& s, F&& go) {
  // go(kernel) launches; one instantiation per (chunks, warp / CTA)
  if (!s.cta) {
    switch (s.per) {
      case 1: return go(kBwd ? ln_bwd_kernel<T, 1, false> : ln_fwd_kernel<T, 1, false>);
      case 2: return go(kBwd ? ln_bwd_kernel<T, 2, false> : ln_fwd_kernel<T, 2, false>);
      case 4: return go(kBwd ? ln_bwd_kernel<T, 4, false> : ln_fwd_kernel<T, 4, false>);
      default: return go(kBwd ? ln_bwd_kernel<T, 4, false> : ln_fwd_kernel<T, 8, false>);
    }
  }
  switch (s.per) {
    case 1: return go(kBwd ? ln_bwd_kernel<T, 1, true> : ln_fwd_kernel<T, 1, true>);
    case 2: return go(kBwd ? ln_bwd_kernel<T, 2, true> : ln_fwd_kernel<T, 2, true>);
    case 4: return go(kBwd ? ln_bwd_kernel<T, 4, true> : ln_fwd_kernel<T, 4, true>);
    default: return go(kBwd ? ln_bwd_kernel<T, sizeof(T) == 4 ? 8 : 4, true> : ln_fwd_kernel<T, 8, true>);
  }
}

template <typename T>
int fwd_t(const nb200_layer_norm_params* p, const Shape& s, cudaStream_t st) {
  LnArgs a{};
  a.x = p->x; a.w = p->weight; a.b = p->bias; a.y = p->y; a.mean = p->mean; a.rstd = p->rstd;
  a.rows = p->rows; a.C = p->channels; a.eps = p->eps; a.out_scale = p->out_scale;
  const int64_t blocks = s.cta ? p->rows : (p->rows + kThreads / 32 - 1) / (kThreads / 32);
  if (blocks > 0x7fffffff) { set_error("layer_norm: too many rows"); return NB200_ERR_UNSUPPORTED; }
  return dispatch<T, false>(s, [&](auto kernel) {
    kernel<<<unsigned(blocks), kThreads, 0, st>>>(a);
    count_launch();
    return check_launch("layer_norm_fwd_kernel");
  });
}

template <typename T>
int bwd_t(const nb200_layer_norm_params* p, const Shape& s, cudaStream_t st) {
  LnArgs a{};
  a.x = p->x; a.w = p->weight; a.dy = p->dy; a.dx = p->dx; a.mean = p->mean; a.rstd = p->rstd;
  a.rows = p->rows; a.C = p->channels; a.eps = p->eps; a.out_scale = p->out_scale;
  const bool want_params = p->dweight || p->dbias;
  int grid = bwd_grid(p->rows, s, 8);
  if (want_params) {
    const size_t need = sizeof(float) * 2 * size_t(grid) * size_t(p->channels);
    if (!p->workspace || p->workspace_bytes < need) {
      set_error("layer_norm_bwd: workspace of %zu bytes needed (nb200_layer_norm_workspace_bytes), %zu given", need,
                size_t(p->workspace_bytes));
      return NB200_ERR_INVALID;
    }
    a.part = static_cast<float*>(p->workspace);
  }
  // (rows padded to the kernel's per * threads * vec columns)
  const size_t smem = want_params ? sizeof(float) * 2 * (s.cta ? 1 : kThreads / 32) * size_t(s.per) *
                                        (s.cta ? kThreads : 32) * s.vec
                                  : 0;
  int rc = dispatch<T, true>(s, [&](auto kernel) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
      set_error("layer_norm_bwd: cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(cudaGetLastError()));
      return int(NB200_ERR_LAUNCH);
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem) != cudaSuccess || per_sm < 1) {
      cudaGetLastError();
      per_sm = 1;
    }
    grid = bwd_grid(p->rows, s, per_sm < 8 ? per_sm : 8);
    kernel<<<unsigned(grid), kThreads, smem, st>>>(a);
    count_launch();
    return check_launch("layer_norm_bwd_kernel");
  });
  if (rc || !want_params) return rc;
  ln_bwd_finish_kernel<T><<<(p->channels + 31) / 32, kThreads, 0, st>>>(
      a.part, grid, p->channels, static_cast<T*>(p->dweight), static_cast<T*>(p->dbias));
  count_launch();
  return check_launch("layer_norm_bwd_finish_kernel");
}

template <typename T>
int fwd_generic_t(const nb200_layer_norm_params* p, cudaStream_t st) {
  LnArgs a{};
  a.x = p->x; a.w = p->weight; a.b = p->bias; a.y = p->y; a.mean = p->mean; a.rstd = p->rstd;
  a.rows = p->rows; a.C = p->channels; a.eps = p->eps; a.out_scale = p->out_scale;
  if (p->rows > 0x7fffffff) { set_error("layer_norm: too many rows"); return NB200_ERR_UNSUPPORTED; }
  ln_fwd_generic_kernel<T><<<unsigned(p->rows), kThreads, 0, st>>>(a);
  count_launch();
  return check_launch("layer_norm_fwd_generic_kernel");
}

template <typename T>
int bwd_generic_t(const nb200_layer_norm_params* p, cudaStream_t st) {
  LnArgs a{};
  a.x = p->x; a.w = p->weight; a.dy = p->dy; a.dx = p->dx; a.mean = p->mean; a.rstd = p->rstd;
  a.rows = p->rows; a.C = p->channels; a.eps = p->eps; a.out_scale = p->out_scale;
  const bool want_params = p->dweight || p->dbias;
  if (want_params) {
    const size_t need = sizeof(float) * 2 * size_t(p->channels);
    if (!p->workspace || p->workspace_bytes < need) {
      set_error("layer_norm_bwd: workspace of %zu bytes needed (nb200_layer_norm_workspace_bytes), %zu given", need,
                size_t(p->workspace_bytes));
      return NB200_ERR_INVALID;
    }
    a.part = static_cast<float*>(p->workspace);
    if (cudaMemsetAsync(a.part, 0, need, st) != cudaSuccess) return check_launch("layer_norm_bwd: clearing the workspace");
  }
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t cap = int64_t(sms > 0 ? sms : 148) * 8;
  const int grid = int(p->rows < cap ? (p->rows > 0 ? p->rows : 1) : cap);
  ln_bwd_generic_kernel<T><<<unsigned(grid), kThreads, 0, st>>>(a);
  count_launch();
  if (int rc = check_launch("layer_norm_bwd_generic_kernel")) return rc;
  if (!want_params) return NB200_OK;
  ln_bwd_finish_kernel<T><<<(p->channels + 31) / 32, kThreads, 0, st>>>(
      a.part, 1, p->channels, static_cast<T*>(p->dweight), static_cast<T*>(p->dbias));
  count_launch();
  return check_launch("layer_norm_bwd_finish_kernel");
}

// the vector kernels need 16-byte rows: channels a multiple of 16 bytes (<= 8192) and aligned pointers
bool vector_path(const nb200_layer_norm_params* p, bool backward, Shape* s) {
  Shape b;
  if (!pick(p->channels, p->dtype, true, &b)) return false;       // (one limit for both directions)
  if (!pick(p->channels, p->dtype, backward, s)) return false;
  if (!aligned16(p->x) || (p->weight && !aligned16(p->weight))) return false;
  if (backward) return aligned16(p->dy) && aligned16(p->dx);
  return aligned16(p->y) && (!p->bias || aligned16(p->bias));
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" NB200_API int nb200_layer_norm_workspace_bytes(const nb200_layer_norm_params* p, size_t* bytes) {
  if (!bytes) { set_error("bytes out-pointer is NULL"); return NB200_ERR_INVALID; }
  if (int rc = check_common(p, "layer_norm_workspace_bytes")) return rc;
  // (sized for the vector kernels' per-CTA partial rows, which is never less than the scalar kernels' [2][C])
  Shape s;
  const int grid = pick(p->channels, p->dtype, true, &s) ? bwd_grid(p->rows, s, 8) : 1;
  *bytes = sizeof(float) * 2 * size_t(grid) * size_t(p->channels);
  return NB200_OK;
}

extern "C" NB200_API int nb200_layer_norm_fwd(const nb200_layer_norm_params* p, void* cuda_stream) {
  if (int rc = check_common(p, "layer_norm_fwd")) return rc;
  if (p->rows == 0) return NB200_OK;
  if (!p->x || !p->y) { set_error("layer_norm_fwd: NULL x or y"); return NB200_ERR_INVALID; }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  prof_call_begin(st);
  Shape s;
  const bool vec = vector_path(p, false, &s);
  switch (p->dtype) {
    case NB200_F32: return vec ? fwd_t<float>(p, s, st) : fwd_generic_t<float>(p, st);
    case NB200_BF16: return vec ? fwd_t<__nv_bfloat16>(p, s, st) : fwd_generic_t<__nv_bfloat16>(p, st);
    default: return vec ? fwd_t<__half>(p, s, st) : fwd_generic_t<__half>(p, st);
  }
}

extern "C" NB200_API int nb200_layer_norm_bwd(const nb200_layer_norm_params* p, void* cuda_stream) {
  if (int rc = check_common(p, "layer_norm_bwd")) return rc;
  if (p->rows == 0 && !p->dweight && !p->dbias) return NB200_OK;
  if ((p->rows > 0 && (!p->x || !p->dy || !p->dx || !p->mean || !p->rstd))) {
    set_error("layer_norm_bwd: x, dy, dx, mean and rstd are required");
    return NB200_ERR_INVALID;
  }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  prof_call_begin(st);
  Shape s;
  const bool vec = vector_path(p, true, &s);
  switch (p->dtype) {
    case NB200_F32: return vec ? bwd_t<float>(p, s, st) : bwd_generic_t<float>(p, st);
    case NB200_BF16: return vec ? bwd_t<__nv_bfloat16>(p, s, st) : bwd_generic_t<__nv_bfloat16>(p, st);
    default: return vec ? bwd_t<__half>(p, s, st) : bwd_generic_t<__half>(p, st);
  }
}
