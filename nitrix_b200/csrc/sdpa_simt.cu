// CUDA-core (SIMT) attention kernels: fp32 arithmetic on any dtype, any shape.
//
// These cover what the tensor-core kernels decline (fp32 inputs, head dims
// other than 64/128, ragged S/T, d_v != d, arbitrary bias/mask strides), so the
// library never needs a host fallback.  They follow the same flash recurrence
// as the reference's fused kernels (reference src/nitrix/_kernels/cuda/
// attention.py:85-156 forward, :272-387 backward) but in true fp32 FMA
// arithmetic: base-2 online softmax carry (m, l), lse = m + log2(l), recompute
// of p = exp2(s - lse) in the backward, one kernel for dq(+dbias) and one for
// dk, dv.  A fully masked query row yields NaN like the reference's jnp path
// (reference src/nitrix/nn/attention/_reference.py:133-135).
//
// Work decomposition: one warp owns one query row (forward, dq) or one key row
// (dk/dv); the 32 lanes of a warp take 32 consecutive rows of the opposite
// operand, which a CTA stages in shared memory as fp32 and shares among its
// warps.  Row sums use warp shuffles; nothing is atomically accumulated except
// the optional broadcast-bias gradient.
#include <math.h>

#include "sdpa_common.cuh"

namespace nb200 {
namespace {

constexpr int kWarps = 8;           // warps (rows) per CTA
constexpr int kTile = 32;           // opposite-operand rows per step (one per lane)
constexpr int kMaxChunks = 8;       // supports head dims up to 32 * 8 = 256

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Stage `rows` x `dim` elements of a (row, col)-strided matrix as fp32 in shared
// memory with leading dimension `ld`; rows at or past `limit` become zero.
template <typename T>
__device__ __forceinline__ void stage_tile(float* dst, int ld, const T* src, int64_t row_stride,
                                           int row0, int limit, int dim) {
  // one warp per row, lanes over the columns: coalesced, and no division per element
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (int r = warp; r < kTile; r += n_warps) {
    const int row = row0 + r;
    const T* srow = src + row * row_stride;
    float* drow = dst + r * ld;
    if (row < limit) {
      for (int c = lane; c < dim; c += 32) drow[c] = to_f32<T>(srow[c]);
    } else {
      for (int c = lane; c < dim; c += 32) drow[c] = 0.f;
    }
  }
}

// Dot product of two fp32 rows in shared memory: four independent chains (the order of the sum is fixed, so
// results stay run-to-run identical).
__device__ __forceinline__ float dot_rows(const float* a, const float* b, int n) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int d = 0;
  for (; d + 4 <= n; d += 4) {
    s0 = fmaf(a[d], b[d], s0);
    s1 = fmaf(a[d + 1], b[d + 1], s1);
    s2 = fmaf(a[d + 2], b[d + 2], s2);
    s3 = fmaf(a[d + 3], b[d + 3], s3);
  }
  for (; d < n; ++d) s0 = fmaf(a[d], b[d], s0);
  return (s0 + s1) + (s2 + s3);
}

__device__ __forceinline__ bool keep_entry(const Problem& pr, int b, int h, int i, int j) {
  if (j >= pr.T || i >= pr.S) return false;
  if (pr.causal && j > i) return false;
  if (pr.mask) {
    return pr.mask[b * pr.ms[0] + h * pr.ms[1] + i * pr.ms[2] + j * pr.ms[3]] != 0;
  }
  return true;
}

__device__ __forceinline__ float bias2(const Problem& pr, int bias_dtype, int b, int h, int i, int j) {
  if (!pr.bias) return 0.f;
  return kLog2e * load_as_f32(pr.bias, b * pr.bs[0] + h * pr.bs[1] + i * pr.bs[2] + j * pr.bs[3], bias_dtype);
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_fwd_kernel(Problem pr, int bias_dtype) {
  extern __shared__ float smem[];
  const int D = pr.D, Dv = pr.Dv, DP = D + 1;
  float* Ks = smem;               // [32][D+1]
  float* Vs = Ks + kTile * DP;    // [32][Dv]
  float* Qs = Vs + kTile * Dv;    // [kWarps][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int row0 = blockIdx.x * kWarps;
  const int i = row0 + warp;
  const bool row_ok = i < pr.S;
  const T* qp = reinterpret_cast<const T*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const T* kp = reinterpret_cast<const T*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const T* vp = reinterpret_cast<const T*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];

  for (int d = lane; d < D; d += 32) Qs[warp * D + d] = row_ok ? to_f32<T>(qp[i * pr.qs[2] + d]) : 0.f;

  float acc[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) acc[c] = 0.f;
  float m = -INFINITY, l = 0.f;
  const float s2scale = pr.scale * kLog2e;
  // causal: no row of this CTA sees keys past its last row
  const int t_end = pr.causal ? min(pr.T, min(row0 + kWarps, pr.S)) : pr.T;

  for (int kt = 0; kt < t_end; kt += kTile) {
    __syncthreads();
    stage_tile<T>(Ks, DP, kp, pr.ks[2], kt, pr.T, D);
    stage_tile<T>(Vs, Dv, vp, pr.vs[2], kt, pr.T, Dv);
    __syncthreads();
    if (!row_ok) continue;
    const int j = kt + lane;
    const float* qrow = Qs + warp * D;
    const float* krow = Ks + lane * DP;
    const float dot = dot_rows(qrow, krow, D);
    const bool keep = keep_entry(pr, b, h, i, j);
    float s2 = keep ? fmaf(dot, s2scale, bias2(pr, bias_dtype, b, h, i, j)) : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s2));
    if (m_new == -INFINITY) continue;  // nothing kept so far (warp-uniform)
    const float alpha = exp2f(m - m_new);
    const float p = keep ? exp2f(s2 - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) acc[c] *= alpha;
    for (int jj = 0; jj < kTile; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* vrow = Vs + jj * Dv;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        if (32 * c >= Dv) break;   // warp-uniform: chunks past the head dim cost nothing
        const int col = lane + 32 * c;
        if (col < Dv) acc[c] = fmaf(pj, vrow[col], acc[c]);
      }
    }
  }
  if (!row_ok) return;
  // l == 0 (fully masked row): 0 * inf = NaN, as the reference's softmax gives
  const float inv = 1.f / l;
  T* op = reinterpret_cast<T*>(pr.out) + b * pr.os[0] + h * pr.os[1] + i * pr.os[2];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int col = lane + 32 * c;
    if (col < Dv) op[col] = from_f32<T>(l == 0.f ? NAN : acc[c] * inv);
  }
  if (lane == 0) pr.lse[(int64_t(b) * pr.H + h) * pr.S + i] = m + log2f(l);
}

// ---------------------------------------------------------------------------
// delta = rowsum(out * dout)   (reference attention.py:621-622, an XLA op there)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) delta_kernel(Problem pr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int i = blockIdx.x * kWarps + warp;
  if (i >= pr.S) return;
  const T* op = reinterpret_cast<const T*>(pr.out) + b * pr.os[0] + h * pr.os[1] + i * pr.os[2];
  const T* gp = reinterpret_cast<const T*>(pr.dout) + b * pr.dos[0] + h * pr.dos[1] + i * pr.dos[2];
  float s = 0.f;
  for (int d = lane; d < pr.Dv; d += 32) s = fmaf(to_f32<T>(op[d]), to_f32<T>(gp[d]), s);
  s = warp_sum(s);
  if (lane == 0) pr.delta[(int64_t(b) * pr.H + h) * pr.S + i] = s;
}

// 16-bit rows with 16-byte alignment: one 16-byte load of out and of dout per
// thread, kLanes = Dv / 8 threads per row, shuffle reduction inside the group.
template <typename T, int kLanes>
__global__ void __launch_bounds__(256) delta_vec_kernel(Problem pr) {
  constexpr int kRows = 256 / kLanes;
  const int sub = threadIdx.x % kLanes;
  const int i = blockIdx.x * kRows + threadIdx.x / kLanes;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  float s = 0.f;
  if (i < pr.S) {
    const T* op = reinterpret_cast<const T*>(pr.out) + b * pr.os[0] + h * pr.os[1] + i * pr.os[2] + sub * 8;
    const T* gp = reinterpret_cast<const T*>(pr.dout) + b * pr.dos[0] + h * pr.dos[1] + i * pr.dos[2] + sub * 8;
    const uint4 ov = __ldg(reinterpret_cast<const uint4*>(op));
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gp));
    const T* o8 = reinterpret_cast<const T*>(&ov);
    const T* g8 = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) s = fmaf(to_f32<T>(o8[e]), to_f32<T>(g8[e]), s);
  }
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (sub == 0 && i < pr.S) pr.delta[(int64_t(b) * pr.H + h) * pr.S + i] = s;
}

// ---------------------------------------------------------------------------
// backward, query side: dq (+ dbias).  One warp per query row, lanes over keys.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_bwd_dq_kernel(Problem pr, int bias_dtype) {
  extern __shared__ float smem[];
  const int D = pr.D, Dv = pr.Dv, DP = D + 1, DVP = Dv + 1;
  float* Ks = smem;                 // [32][D+1]
  float* Vs = Ks + kTile * DP;      // [32][Dv+1]
  float* Qs = Vs + kTile * DVP;     // [kWarps][D]
  float* Gs = Qs + kWarps * D;      // [kWarps][Dv]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int row0 = blockIdx.x * kWarps;
  const int i = row0 + warp;
  const bool row_ok = i < pr.S;
  const T* qp = reinterpret_cast<const T*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const T* kp = reinterpret_cast<const T*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const T* vp = reinterpret_cast<const T*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  const T* gp = reinterpret_cast<const T*>(pr.dout) + b * pr.dos[0] + h * pr.dos[1];
  for (int d = lane; d < D; d += 32) Qs[warp * D + d] = row_ok ? to_f32<T>(qp[i * pr.qs[2] + d]) : 0.f;
  for (int d = lane; d < Dv; d += 32) Gs[warp * Dv + d] = row_ok ? to_f32<T>(gp[i * pr.dos[2] + d]) : 0.f;
  const int64_t ridx = (int64_t(b) * pr.H + h) * pr.S + (row_ok ? i : 0);
  const float lse = pr.lse[ridx], delta = pr.delta[ridx];
  const float s2scale = pr.scale * kLog2e;
  float acc[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) acc[c] = 0.f;
  const int t_end = pr.causal ? min(pr.T, min(row0 + kWarps, pr.S)) : pr.T;
  const bool want_db = pr.dbias != nullptr || pr.dbias_accum != nullptr;

  for (int kt = 0; kt < t_end; kt += kTile) {
    __syncthreads();
    stage_tile<T>(Ks, DP, kp, pr.ks[2], kt, pr.T, D);
    stage_tile<T>(Vs, DVP, vp, pr.vs[2], kt, pr.T, Dv);
    __syncthreads();
    if (!row_ok) continue;
    const int j = kt + lane;
    const float* qrow = Qs + warp * D;
    const float* krow = Ks + lane * DP;
    const float dot = dot_rows(qrow, krow, D);
    const float* grow = Gs + warp * Dv;
    const float* vrow = Vs + lane * DVP;
    const float dp = dot_rows(grow, vrow, Dv);
    const bool keep = keep_entry(pr, b, h, i, j);
    const float p = keep ? exp2f(fmaf(dot, s2scale, bias2(pr, bias_dtype, b, h, i, j)) - lse) : 0.f;
    const float ds = p * (dp - delta);
    if (want_db && j < pr.T) {
      const int64_t off = b * pr.dbs[0] + h * pr.dbs[1] + i * pr.dbs[2] + j * pr.dbs[3];
      if (pr.dbias_accum) {
        if (ds != 0.f) atomicAdd(pr.dbias_accum + off, ds);
      } else {
        store_from_f32(pr.dbias, off, bias_dtype, ds);
      }
    }
    for (int jj = 0; jj < kTile; ++jj) {
      const float dsj = __shfl_sync(0xffffffffu, ds, jj);
      const float* kr = Ks + jj * DP;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        if (32 * c >= D) break;    // warp-uniform
        const int col = lane + 32 * c;
        if (col < D) acc[c] = fmaf(dsj, kr[col], acc[c]);
      }
    }
  }
  if (!row_ok) return;
  // causal rows never visit keys past the diagonal, yet a dense dbias must be
  // written everywhere: those entries are exact zeros
  if (want_db && !pr.dbias_accum && t_end < pr.T) {
    for (int j = ((t_end + kTile - 1) / kTile) * kTile + lane; j < pr.T; j += 32)
      store_from_f32(pr.dbias, b * pr.dbs[0] + h * pr.dbs[1] + i * pr.dbs[2] + j * pr.dbs[3], bias_dtype, 0.f);
  }
  T* dqp = reinterpret_cast<T*>(pr.dq) + b * pr.dqs[0] + h * pr.dqs[1] + i * pr.dqs[2];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int col = lane + 32 * c;
    if (col < D) dqp[col] = from_f32<T>(acc[c] * pr.scale);
  }
}

// ---------------------------------------------------------------------------
// backward, key side: dk, dv.  One warp per key row, lanes over queries.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_bwd_dkv_kernel(Problem pr, int bias_dtype) {
  extern __shared__ float smem[];
  const int D = pr.D, Dv = pr.Dv, DP = D + 1, DVP = Dv + 1;
  float* Qt = smem;                 // [32][D+1]   query tile
  float* Gt = Qt + kTile * DP;      // [32][Dv+1]  dout tile
  float* Kr = Gt + kTile * DVP;     // [kWarps][D]
  float* Vr = Kr + kWarps * D;      // [kWarps][Dv]
  float* Ls = Vr + kWarps * Dv;     // [32] lse
  float* Ds = Ls + kTile;           // [32] delta
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int key0 = blockIdx.x * kWarps;
  const int j = key0 + warp;
  const bool key_ok = j < pr.T;
  const T* qp = reinterpret_cast<const T*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const T* kp = reinterpret_cast<const T*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const T* vp = reinterpret_cast<const T*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  const T* gp = reinterpret_cast<const T*>(pr.dout) + b * pr.dos[0] + h * pr.dos[1];
  for (int d = lane; d < D; d += 32) Kr[warp * D + d] = key_ok ? to_f32<T>(kp[j * pr.ks[2] + d]) : 0.f;
  for (int d = lane; d < Dv; d += 32) Vr[warp * Dv + d] = key_ok ? to_f32<T>(vp[j * pr.vs[2] + d]) : 0.f;
  const float s2scale = pr.scale * kLog2e;
  float dk[kMaxChunks], dv[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) dk[c] = dv[c] = 0.f;
  // causal: queries before this CTA's first key see none of its keys
  const int s_begin = pr.causal ? (key0 / kTile) * kTile : 0;
  const int64_t rbase = (int64_t(b) * pr.H + h) * pr.S;

  for (int qt = s_begin; qt < pr.S; qt += kTile) {
    __syncthreads();
    stage_tile<T>(Qt, DP, qp, pr.qs[2], qt, pr.S, D);
    stage_tile<T>(Gt, DVP, gp, pr.dos[2], qt, pr.S, Dv);
    if (threadIdx.x < kTile) {
      const int r = qt + threadIdx.x;
      Ls[threadIdx.x] = r < pr.S ? pr.lse[rbase + r] : 0.f;
      Ds[threadIdx.x] = r < pr.S ? pr.delta[rbase + r] : 0.f;
    }
    __syncthreads();
    if (!key_ok) continue;
    const int i = qt + lane;
    const float* qrow = Qt + lane * DP;
    const float* krow = Kr + warp * D;
    const float dot = dot_rows(qrow, krow, D);
    const float* grow = Gt + lane * DVP;
    const float* vrow = Vr + warp * Dv;
    const float dp = dot_rows(grow, vrow, Dv);
    const bool keep = keep_entry(pr, b, h, i, j);
    const float p = keep ? exp2f(fmaf(dot, s2scale, bias2(pr, bias_dtype, b, h, i, j)) - Ls[lane]) : 0.f;
    const float ds = p * (dp - Ds[lane]);
    for (int ii = 0; ii < kTile; ++ii) {
      const float pi = __shfl_sync(0xffffffffu, p, ii);
      const float dsi = __shfl_sync(0xffffffffu, ds, ii);
      const float* gr = Gt + ii * DVP;
      const float* qr = Qt + ii * DP;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        if (32 * c >= D && 32 * c >= Dv) break;   // warp-uniform
        const int col = lane + 32 * c;
        if (col < Dv) dv[c] = fmaf(pi, gr[col], dv[c]);
        if (col < D) dk[c] = fmaf(dsi, qr[col], dk[c]);
      }
    }
  }
  if (!key_ok) return;
  T* dkp = reinterpret_cast<T*>(pr.dk) + b * pr.dks[0] + h * pr.dks[1] + j * pr.dks[2];
  T* dvp = reinterpret_cast<T*>(pr.dv) + b * pr.dvs[0] + h * pr.dvs[1] + j * pr.dvs[2];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int col = lane + 32 * c;
    if (col < D) dkp[col] = from_f32<T>(dk[c] * pr.scale);
    if (col < Dv) dvp[col] = from_f32<T>(dv[c]);
  }
}

// dbias_accum (fp32, dense over bias' own extent) -> dbias in bias dtype
__global__ void dbias_finish_kernel(const float* accum, void* dbias, int bias_dtype, int64_t n,
                                    int64_t e1, int64_t e2, int64_t e3, int64_t s0, int64_t s1,
                                    int64_t s2, int64_t s3) {
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < n;
       idx += int64_t(gridDim.x) * blockDim.x) {
    int64_t r = idx;
    const int64_t i3 = r % e3; r /= e3;
    const int64_t i2 = r % e2; r /= e2;
    const int64_t i1 = r % e1; r /= e1;
    store_from_f32(dbias, r * s0 + i1 * s1 + i2 * s2 + i3 * s3, bias_dtype, accum[idx]);
  }
}

size_t fwd_smem(const Problem& pr) {
  return sizeof(float) * (size_t(kTile) * (pr.D + 1) + size_t(kTile) * pr.Dv + size_t(kWarps) * pr.D);
}
size_t bwd_smem(const Problem& pr) {
  return sizeof(float) * (size_t(kTile) * (pr.D + 1) + size_t(kTile) * (pr.Dv + 1) +
                          size_t(kWarps) * (pr.D + pr.Dv) + 2 * kTile);
}

template <typename K>
int prepare(K kernel, size_t smem) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(%zu bytes): %s", smem, cudaGetErrorString(e));
      return NB200_ERR_LAUNCH;
    }
  }
  return NB200_OK;
}

template <typename T>
int fwd_t(const Problem& pr, int bias_dtype, cudaStream_t st) {
  const size_t smem = fwd_smem(pr);
  if (int rc = prepare(simt_fwd_kernel<T>, smem)) return rc;
  dim3 grid((pr.S + kWarps - 1) / kWarps, pr.bh_count);
  simt_fwd_kernel<T><<<grid, kWarps * 32, smem, st>>>(pr, bias_dtype);
  count_launch();
  return check_launch("simt_fwd_kernel");
}

template <typename T>
int bwd_t(const Problem& pr, int bias_dtype, cudaStream_t st) {
  const size_t smem = bwd_smem(pr);
  if (int rc = prepare(simt_bwd_dq_kernel<T>, smem)) return rc;
  if (int rc = prepare(simt_bwd_dkv_kernel<T>, smem)) return rc;
  if (pr.S > 0) {
    dim3 gq((pr.S + kWarps - 1) / kWarps, pr.bh_count);
    simt_bwd_dq_kernel<T><<<gq, kWarps * 32, smem, st>>>(pr, bias_dtype);
    count_launch();
    if (int rc = check_launch("simt_bwd_dq_kernel")) return rc;
  }
  if (pr.T > 0) {
    dim3 gk((pr.T + kWarps - 1) / kWarps, pr.bh_count);
    simt_bwd_dkv_kernel<T><<<gk, kWarps * 32, smem, st>>>(pr, bias_dtype);
    count_launch();
    return check_launch("simt_bwd_dkv_kernel");
  }
  return NB200_OK;
}

}  // namespace

int simt_forward(const Problem& pr, int dtype, int bias_dtype, cudaStream_t st) {
  if (pr.bh_count <= 0 || pr.S <= 0) return NB200_OK;
  switch (dtype) {
    case NB200_F32: return fwd_t<float>(pr, bias_dtype, st);
    case NB200_BF16: return fwd_t<__nv_bfloat16>(pr, bias_dtype, st);
    default: return fwd_t<__half>(pr, bias_dtype, st);
  }
}

int simt_backward(const Problem& pr, int dtype, int bias_dtype, cudaStream_t st) {
  if (pr.bh_count <= 0) return NB200_OK;
  switch (dtype) {
    case NB200_F32: return bwd_t<float>(pr, bias_dtype, st);
    case NB200_BF16: return bwd_t<__nv_bfloat16>(pr, bias_dtype, st);
    default: return bwd_t<__half>(pr, bias_dtype, st);
  }
}

int launch_delta(const Problem& pr, int dtype, cudaStream_t st) {
  if (pr.bh_count <= 0 || pr.S <= 0) return NB200_OK;
  const bool aligned = reinterpret_cast<uintptr_t>(pr.out) % 16 == 0 && reinterpret_cast<uintptr_t>(pr.dout) % 16 == 0 &&
                       pr.os[0] % 8 == 0 && pr.os[1] % 8 == 0 && pr.os[2] % 8 == 0 && pr.dos[0] % 8 == 0 &&
                       pr.dos[1] % 8 == 0 && pr.dos[2] % 8 == 0;
  if (dtype != NB200_F32 && aligned && (pr.Dv == 64 || pr.Dv == 128)) {
    const int lanes = pr.Dv / 8, rows = 256 / lanes;
    dim3 vgrid((pr.S + rows - 1) / rows, pr.bh_count);
    if (dtype == NB200_BF16) {
      if (lanes == 8) delta_vec_kernel<__nv_bfloat16, 8><<<vgrid, 256, 0, st>>>(pr);
      else delta_vec_kernel<__nv_bfloat16, 16><<<vgrid, 256, 0, st>>>(pr);
    } else {
      if (lanes == 8) delta_vec_kernel<__half, 8><<<vgrid, 256, 0, st>>>(pr);
      else delta_vec_kernel<__half, 16><<<vgrid, 256, 0, st>>>(pr);
    }
    count_launch();
    return check_launch("delta_vec_kernel");
  }
  dim3 grid((pr.S + kWarps - 1) / kWarps, pr.bh_count);
  switch (dtype) {
    case NB200_F32: delta_kernel<float><<<grid, kWarps * 32, 0, st>>>(pr); break;
    case NB200_BF16: delta_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, st>>>(pr); break;
    default: delta_kernel<__half><<<grid, kWarps * 32, 0, st>>>(pr); break;
  }
  count_launch();
  return check_launch("delta_kernel");
}

int launch_dbias_finish(const float* accum, void* dbias, int bias_dtype, const int64_t e[4],
                        const int64_t stride[4], cudaStream_t st) {
  const int64_t n = e[0] * e[1] * e[2] * e[3];
  if (n <= 0) return NB200_OK;
  const int threads = 256;
  const int64_t want = (n + threads - 1) / threads;
  const int blocks = int(want < 148 * 8 ? want : 148 * 8);
  dbias_finish_kernel<<<blocks, threads, 0, st>>>(accum, dbias, bias_dtype, n, e[1], e[2], e[3], stride[0],
                                                  stride[1], stride[2], stride[3]);
  count_launch();
  return check_launch("dbias_finish_kernel");
}

}  // namespace nb200
