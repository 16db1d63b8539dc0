// Attention kernels outside the tcgen05 family: fp32 arithmetic on any dtype, any shape.
//
// These cover what the tcgen05 kernels decline (fp32 inputs, head dims other than 64/128, lengths that are not
// multiples of 8, d_v != d, arbitrary bias/mask strides), so the library never needs a host fallback.  They follow the
// same flash recurrence as the reference's fused kernels (reference src/nitrix/_kernels/cuda/attention.py:85-156
// forward, :272-387 backward): base-2 online softmax carry (m, l), lse = m + log2(l), recompute of
// p = exp2(s - lse) in the backward, one kernel for dq(+dbias) and one for dk, dv.  A fully masked query row yields
// NaN like the reference's jnp path (reference src/nitrix/nn/attention/_reference.py:133-135).
//
// Forward, by operand type and head dims:
//   fwd_tf32x3_kernel      fp32 operands, head dims multiples of 8 (<= 128): 3 x TF32 on mma.sync.m16n8k8
//   simt_fwd_tiled_kernel  head dims multiples of 4 / 32 (<= 128): register-tiled FMA, float4 shared-memory operands
//   simt_fwd_kernel        everything else: one warp per query row, 32 lanes over 32 keys
// Backward, fp32 operands on grids of >= 96 CTAs: bwd_dq_tf32x3_kernel and bwd_dkv_tf32x3_kernel
// (D == Dv in {32, 64, 128}), the same 3 x TF32 tiling; smaller problems at head dims 32 / 64 split each CTA's
// tiles of the opposite operand over groups of warps (forward, dq) or over the CTAs of a cluster (dk / dv; the
// smallest problems: forward and dq as well).  Otherwise:
// one warp owns one query row (dq) or one key row (dk/dv); the 32 lanes take 32 consecutive rows of the
// opposite operand, staged in shared memory as fp32.  Row sums use warp shuffles; nothing is atomically accumulated
// except the optional broadcast-bias gradient, and every sum runs in a fixed order.
#include <cooperative_groups.h>
#include <math.h>

#include "sdpa_common.cuh"

namespace nb200 {
namespace {

namespace cg = cooperative_groups;

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
// forward, register-tiled: the fp32 workhorse (head dims that are multiples of 4 / 32, up to 128)
// ---------------------------------------------------------------------------
// A CTA of 128 threads owns 64 query rows and streams 64-key tiles.  Thread (ty, tx) = (tid / 8, tid % 8) holds a
// 4 x 8 micro-tile of the scores (rows ty + 16 i, keys tx + 8 j) and 4 rows x Dv / 8 columns of the output; both
// products read their operands from shared memory as float4 (12 loads per 128 FMAs), the probabilities pass through
// a shared tile.  Row maxima / sums need the 8 threads of a row: three xor-shuffles.  Same recurrence, same masking
// and NaN semantics as simt_fwd_kernel; the summation order is fixed, so results are run-to-run identical.
constexpr int kBN = 64, kTiledThreads = 128;

template <typename T>
__device__ __forceinline__ void stage_rows(float* dst, int ld, const T* src, int64_t row_stride, int row0, int n_rows,
                                           int limit, int dim) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (int r = warp; r < n_rows; r += n_warps) {
    const int row = row0 + r;
    float* drow = dst + r * ld;
    if (row < limit) {
      const T* srow = src + row * row_stride;
      for (int c = lane; c < dim; c += 32) drow[c] = to_f32<T>(srow[c]);
    } else {
      for (int c = lane; c < dim; c += 32) drow[c] = 0.f;
    }
  }
}

// fp32 rows whose start and stride are 16-byte aligned: asynchronous 16-byte copies straight into shared memory, all
// in flight at once (a load-then-store loop pays the global latency once per iteration); rows past `limit` are
// zero-filled by a copy of source size 0.  The caller's __syncthreads() follows the wait below.
__device__ __forceinline__ void stage_rows_f4(float* dst, int ld, const float* src, int64_t row_stride, int row0,
                                              int n_rows, int limit, int dim, int tid = threadIdx.x,
                                              int n_threads = blockDim.x) {
  const int per_row = dim >> 2;
  for (int idx = tid; idx < n_rows * per_row; idx += n_threads) {
    const int r = idx / per_row, c4 = idx - r * per_row;
    const int row = row0 + r;
    const bool in = row < limit;
    const float* g = src + (in ? row : 0) * row_stride + 4 * c4;
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(dst + r * ld + 4 * c4));
    const int bytes = in ? 16 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(g), "r"(bytes) : "memory");
  }
}
__device__ __forceinline__ void stage_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// `wait = false` leaves the asynchronous copies in flight (stage_wait() completes them); the synchronous fall-back
// path has always finished on return.
template <typename T>
__device__ __forceinline__ void stage_rows_any(float* dst, int ld, const T* src, int64_t row_stride, int row0, int n_rows,
                                               int limit, int dim, bool wait = true) {
  if constexpr (sizeof(T) == 4) {
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (row_stride & 3) == 0 && (dim & 3) == 0) {
      stage_rows_f4(dst, ld, reinterpret_cast<const float*>(src), row_stride, row0, n_rows, limit, dim);
      if (wait) stage_wait();
      return;
    }
  }
  stage_rows<T>(dst, ld, src, row_stride, row0, n_rows, limit, dim);
}

template <typename T, int kVChunks, int kR>   // kVChunks = Dv / 32; kR rows per thread: the CTA owns 16 kR query rows
__global__ void __launch_bounds__(kTiledThreads) simt_fwd_tiled_kernel(Problem pr, int bias_dtype) {
  extern __shared__ __align__(16) float smem[];
  constexpr int kBM = 16 * kR;
  const int D = pr.D, Dv = pr.Dv;
  const int LDQ = D + 4, LDV = Dv + 4, LDP = kBN + 4;
  float* Qs = smem;                  // [kBM][LDQ]
  float* Ks = Qs + kBM * LDQ;        // [kBN][LDQ]
  float* Vs = Ks + kBN * LDQ;        // [kBN][LDV]
  float* Ps = Vs + kBN * LDV;        // [kBM][LDP]
  const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int row0 = blockIdx.x * kBM;
  const T* qp = reinterpret_cast<const T*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const T* kp = reinterpret_cast<const T*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const T* vp = reinterpret_cast<const T*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  stage_rows_any<T>(Qs, LDQ, qp, pr.qs[2], row0, kBM, pr.S, D);
  // element offsets of this thread's four rows into bias and mask (the key term is added per element)
  int64_t boff[kR], moff[kR];
#pragma unroll
  for (int i = 0; i < kR; ++i) {
    const int rr = min(row0 + ty + 16 * i, pr.S - 1);
    boff[i] = pr.bias ? b * pr.bs[0] + h * pr.bs[1] + rr * pr.bs[2] : 0;
    moff[i] = pr.mask ? b * pr.ms[0] + h * pr.ms[1] + rr * pr.ms[2] : 0;
  }

  float o[kR][kVChunks][4];
  float m[kR], l[kR];
#pragma unroll
  for (int i = 0; i < kR; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < kVChunks; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[i][c][e] = 0.f;
  }
  const float s2scale = pr.scale * kLog2e;
  // causal: no row of this CTA sees keys past its last row
  const int t_end = pr.causal ? min(pr.T, min(row0 + kBM, pr.S)) : pr.T;

  for (int kt = 0; kt < t_end; kt += kBN) {
    __syncthreads();   // the previous tile's K, V and P are no longer read
    stage_rows_any<T>(Ks, LDQ, kp, pr.ks[2], kt, kBN, pr.T, D);
    stage_rows_any<T>(Vs, LDV, vp, pr.vs[2], kt, kBN, pr.T, Dv);
    __syncthreads();
    // ---- scores: s[i][j] = q[ty + 16 i] . k[tx + 8 j] ----
    float sc[kR][8];
#pragma unroll
    for (int i = 0; i < kR; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) sc[i][j] = 0.f;
    for (int d = 0; d < D; d += 4) {
      float4 qv[kR], kv[8];
#pragma unroll
      for (int i = 0; i < kR; ++i) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty + 16 * i) * LDQ + d);
#pragma unroll
      for (int j = 0; j < 8; ++j) kv[j] = *reinterpret_cast<const float4*>(Ks + (tx + 8 * j) * LDQ + d);
      // one head-dim element at a time over the whole micro-tile: 32 independent FMAs back to back
#pragma unroll
      for (int i = 0; i < kR; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) sc[i][j] = fmaf(qv[i].x, kv[j].x, sc[i][j]);
#pragma unroll
      for (int i = 0; i < kR; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) sc[i][j] = fmaf(qv[i].y, kv[j].y, sc[i][j]);
#pragma unroll
      for (int i = 0; i < kR; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) sc[i][j] = fmaf(qv[i].z, kv[j].z, sc[i][j]);
#pragma unroll
      for (int i = 0; i < kR; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) sc[i][j] = fmaf(qv[i].w, kv[j].w, sc[i][j]);
    }
    // ---- logits in base 2, masks, online softmax per row ----
#pragma unroll
    for (int i = 0; i < kR; ++i) {
      const int row = row0 + ty + 16 * i;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int key = kt + tx + 8 * j;
        bool keep = key < pr.T && row < pr.S && !(pr.causal && key > row);
        if (keep && pr.mask) keep = pr.mask[moff[i] + key * pr.ms[3]] != 0;
        const float bias = (keep && pr.bias) ? kLog2e * load_as_f32(pr.bias, boff[i] + key * pr.bs[3], bias_dtype) : 0.f;
        sc[i][j] = keep ? fmaf(sc[i][j], s2scale, bias) : -INFINITY;
        mx = fmaxf(mx, sc[i][j]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float m_new = fmaxf(m[i], mx);
      const float m_ref = m_new == -INFINITY ? 0.f : m_new;   // nothing kept so far: every p is 0
      const float alpha = exp2f(m[i] - m_ref);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p = exp2f(sc[i][j] - m_ref);
        sum += p;
        Ps[(ty + 16 * i) * LDP + tx + 8 * j] = p;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      l[i] = l[i] * alpha + sum;
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < kVChunks; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][c][e] *= alpha;
    }
    __syncthreads();   // P is complete
    // ---- out[ty + 16 i][4 tx + 32 c + e] += sum_j p[.][j] v[j][.] ----
    for (int j4 = 0; j4 < kBN; j4 += 4) {
      float4 pv[kR];
#pragma unroll
      for (int i = 0; i < kR; ++i) pv[i] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * i) * LDP + j4);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        float4 vv[kVChunks];
#pragma unroll
        for (int c = 0; c < kVChunks; ++c) vv[c] = *reinterpret_cast<const float4*>(Vs + (j4 + jj) * LDV + 4 * tx + 32 * c);
#pragma unroll
        for (int i = 0; i < kR; ++i) {
          const float p = jj == 0 ? pv[i].x : (jj == 1 ? pv[i].y : (jj == 2 ? pv[i].z : pv[i].w));
#pragma unroll
          for (int c = 0; c < kVChunks; ++c) {
            o[i][c][0] = fmaf(p, vv[c].x, o[i][c][0]);
            o[i][c][1] = fmaf(p, vv[c].y, o[i][c][1]);
            o[i][c][2] = fmaf(p, vv[c].z, o[i][c][2]);
            o[i][c][3] = fmaf(p, vv[c].w, o[i][c][3]);
          }
        }
      }
    }
  }
  // ---- out = o / l (NaN for a row with no kept key, as the reference's softmax gives), lse ----
#pragma unroll
  for (int i = 0; i < kR; ++i) {
    const int row = row0 + ty + 16 * i;
    if (row >= pr.S) continue;
    const float inv = 1.f / l[i];
    T* op = reinterpret_cast<T*>(pr.out) + b * pr.os[0] + h * pr.os[1] + row * pr.os[2];
#pragma unroll
    for (int c = 0; c < kVChunks; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) op[4 * tx + 32 * c + e] = from_f32<T>(l[i] == 0.f ? NAN : o[i][c][e] * inv);
    if (tx == 0) pr.lse[(int64_t(b) * pr.H + h) * pr.S + row] = m[i] + log2f(l[i]);
  }
}

// ---------------------------------------------------------------------------
// forward for fp32 operands on the warp-level tensor-core path: 3 x TF32
// ---------------------------------------------------------------------------
// Every fp32 operand x is split as hi = tf32(x), lo = x - hi; a product a b is taken as
// a_hi b_hi + a_hi b_lo + a_lo b_hi (three mma.sync.m16n8k8 TF32 instructions, fp32 accumulate), which keeps about
// 20 bits -- inside the 1e-4 relative budget of the fp32 path.  A CTA of 4 warps owns 64 query rows, a warp 16 of
// them against the whole 64-key tile: scores and output live in accumulator fragments (row g = lane / 4 and g + 8,
// columns 2 t, 2 t + 1 with t = lane % 4), so row maxima / sums need the 4 lanes of a quad.  The probabilities go
// from the score fragment straight into the A operand of P V: within an 8-key block operand column t stands for
// key 2 t and column t + 4 for key 2 t + 1, and the V rows are fetched in that order.
//
// The split itself is two instructions: hi keeps the top 19 bits of x (sign, exponent, 10 mantissa bits -- a TF32
// number), lo = x - hi is exact in fp32, and the tensor core reads only the TF32 bits of lo's register.  (Rounding
// both terms with cvt.rna.tf32 costs several integer instructions per conversion, and the splits -- 320 per warp
// and tile -- were then a third of all instructions issued.)  What is dropped is a_lo b_lo and the truncated tails
// of the lo terms, each below 2^-20 of |a| |b|.  Measured against fp64 (max error over max |reference|, out and
// gradients, S 344..2048): 2.3e-6..4.7e-6, against 1.4e-6..3.1e-6 with both terms rounded and 1.3e-6..3.5e-6 with
// hi rounded (one more instruction); the kernels run 1.25x (forward) to 1.7x (dk / dv at head dim 128) faster.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// c += a b with both operands split: the three leading terms
__device__ __forceinline__ void mma_3xtf32(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                           const uint32_t (&bh)[2], const uint32_t (&bl)[2]) {
  mma_tf32(c, al, bh);
  mma_tf32(c, ah, bl);
  mma_tf32(c, ah, bh);
}

// 2^x for x <= 0 (and -inf -> 0): one MUFU instruction, relative error 2^-22
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One 64-key tile of the 3 x TF32 forward for this warp's 16 query rows: scores, logits and masks, online softmax,
// out += P V.  Ks / Vs: the tile in shared memory (rows past T zero-filled); kt: its first key.  boff / moff: element
// offsets of the bias / mask rows of this thread's two query rows.
template <int kDvBlocks>
__device__ __forceinline__ void fwd_tf32x3_tile(const Problem& pr, int bias_dtype, const float* Qs, const float* Ks,
                                                const float* Vs, int LDQ, int LDV, int D, int kt, int row0,
                                                const int (&lr)[2], const int64_t (&boff)[2], const int64_t (&moff)[2],
                                                float s2scale, int g, int t, float (&o)[kDvBlocks][4], float (&m)[2],
                                                float (&l)[2]) {
  // ---- scores: 8 blocks of 8 keys ----
  float sc[8][4];
#pragma unroll
  for (int nb = 0; nb < 8; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) sc[nb][e] = 0.f;
#pragma unroll 2
  for (int kk = 0; kk < D; kk += 8) {
    uint32_t ah[4], al[4];
    split_tf32(Qs[lr[0] * LDQ + kk + t], ah[0], al[0]);
    split_tf32(Qs[lr[1] * LDQ + kk + t], ah[1], al[1]);
    split_tf32(Qs[lr[0] * LDQ + kk + t + 4], ah[2], al[2]);
    split_tf32(Qs[lr[1] * LDQ + kk + t + 4], ah[3], al[3]);
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      uint32_t bh2[2], bl2[2];
      split_tf32(Ks[(8 * nb + g) * LDQ + kk + t], bh2[0], bl2[0]);
      split_tf32(Ks[(8 * nb + g) * LDQ + kk + t + 4], bh2[1], bl2[1]);
      mma_3xtf32(sc[nb], ah, al, bh2, bl2);
    }
  }
  // ---- logits in base 2, masks, online softmax (rows g and g + 8 of the warp's 16) ----
  // ---- logits in base 2, masks, online softmax (rows g and g + 8 of the warp's 16) ----
  // The last key each row keeps in this tile (as an index into the tile) covers T, S and the causal diagonal.
  // Bias and mask are read in the fragment layout -- this thread's keys are kt + 2 t + (8 nb + c) -- through
  // pointers set up once per tile, with the dtype decided once per tile: a 64-bit index product, bounds tests and
  // a dtype switch per element were two thirds of a tile's instructions.
  float mx[2] = {-INFINITY, -INFINITY};
  int last[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + lr[i];
    last[i] = row < pr.S ? (pr.causal ? min(pr.T - 1, row) : pr.T - 1) - kt : -1;
  }
  if (!pr.bias && !pr.mask) {
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        sc[nb][e] = 8 * nb + 2 * t + (e & 1) <= last[e >> 1] ? sc[nb][e] * s2scale : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], sc[nb][e]);
      }
  } else {
    const int k0 = kt + 2 * t;
    auto logits = [&](auto tag) {
      using BT = decltype(tag);
      const BT* bp[2];
      const uint8_t* mp[2];
      const int64_t bs3 = pr.bs[3], ms3 = pr.ms[3];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        bp[i] = pr.bias ? reinterpret_cast<const BT*>(pr.bias) + boff[i] + k0 * bs3 : nullptr;
        mp[i] = pr.mask ? pr.mask + moff[i] + k0 * ms3 : nullptr;
      }
#pragma unroll
      for (int nb = 0; nb < 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1, col = 8 * nb + (e & 1);      // key = k0 + col
          bool keep = col + 2 * t <= last[i];
          if (keep && mp[i]) keep = mp[i][col * ms3] != 0;
          const float bias = (keep && bp[i]) ? kLog2e * to_f32<BT>(bp[i][col * bs3]) : 0.f;
          sc[nb][e] = keep ? fmaf(sc[nb][e], s2scale, bias) : -INFINITY;
          mx[i] = fmaxf(mx[i], sc[nb][e]);
        }
    };
    if (bias_dtype == NB200_F32) logits(float{});
    else if (bias_dtype == NB200_BF16) logits(__nv_bfloat16{});
    else logits(__half{});
  }
  float alpha[2], m_ref[2], sum[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    const float m_new = fmaxf(m[i], mx[i]);
    m_ref[i] = m_new == -INFINITY ? 0.f : m_new;   // nothing kept so far: every p is 0
    alpha[i] = exp2f(m[i] - m_ref[i]);
    m[i] = m_new;
  }
#pragma unroll
  for (int nb = 0; nb < 8; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = ex2_fast(sc[nb][e] - m_ref[e >> 1]);
      sc[nb][e] = p;
      sum[e >> 1] += p;
    }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
    sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
    l[i] = l[i] * alpha[i] + sum[i];
  }
#pragma unroll
  for (int nb = 0; nb < kDvBlocks; ++nb) {
    o[nb][0] *= alpha[0];
    o[nb][1] *= alpha[0];
    o[nb][2] *= alpha[1];
    o[nb][3] *= alpha[1];
  }
  // ---- out += P V: key block kb supplies operand columns (t -> key 2 t, t + 4 -> key 2 t + 1) ----
#pragma unroll
  for (int kb = 0; kb < 8; ++kb) {
    uint32_t ah[4], al[4];
    split_tf32(sc[kb][0], ah[0], al[0]);   // row g,     key 2 t
    split_tf32(sc[kb][2], ah[1], al[1]);   // row g + 8, key 2 t
    split_tf32(sc[kb][1], ah[2], al[2]);   // row g,     key 2 t + 1
    split_tf32(sc[kb][3], ah[3], al[3]);   // row g + 8, key 2 t + 1
    const float* v0 = Vs + (8 * kb + 2 * t) * LDV + g;
    const float* v1 = v0 + LDV;
#pragma unroll
    for (int nb = 0; nb < kDvBlocks; ++nb) {
      uint32_t bh2[2], bl2[2];
      split_tf32(v0[8 * nb], bh2[0], bl2[0]);
      split_tf32(v1[8 * nb], bh2[1], bl2[1]);
      mma_3xtf32(o[nb], ah, al, bh2, bl2);
    }
  }
}

// kSquare (D == Dv): both row pitches are compile-time constants, so every fragment offset is an immediate.
// kC > 1 (the SMALLEST problems, launched as clusters of kC CTAs along x): the CTAs of a cluster own the same 64 query
// rows and take the key tiles in turn, each with a full register file; ranks 1.. leave their partial (out, m, l) in
// their own shared memory and rank 0 merges them over distributed shared memory in rank order.
template <int kDvBlocks, bool kSquare, int kC = 1>   // Dv / 8
__global__ void __launch_bounds__(kTiledThreads) fwd_tf32x3_kernel(Problem pr, int bias_dtype) {
  extern __shared__ __align__(16) float smem[];
  constexpr int kBM = 64;
  constexpr int Dv = 8 * kDvBlocks;
  const int D = kSquare ? Dv : pr.D;
  const int LDQ = D + 4, LDV = Dv + 4;   // + 4: rows 16 bytes apart modulo 128, fragment loads hit distinct banks
  float* Qs = smem;                  // [kBM][LDQ]
  float* Kbuf = Qs + kBM * LDQ;      // 2 x [kBN][LDQ]
  float* Vbuf = Kbuf + 2 * kBN * LDQ;  // 2 x [kBN][LDV]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int crank = kC > 1 ? int(blockIdx.x) % kC : 0;   // rank in the cluster (cluster dims (kC, 1, 1))
  const int row0 = (int(blockIdx.x) / kC) * kBM;
  const float* qp = reinterpret_cast<const float*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const float* kp = reinterpret_cast<const float*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const float* vp = reinterpret_cast<const float*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  stage_rows_any<float>(Qs, LDQ, qp, pr.qs[2], row0, kBM, pr.S, D, false);

  // this thread's two rows: r[0] = 16 warp + g, r[1] = r[0] + 8
  const int lr[2] = {16 * warp + g, 16 * warp + g + 8};
  int64_t boff[2], moff[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = min(row0 + lr[i], pr.S - 1);
    boff[i] = pr.bias ? b * pr.bs[0] + h * pr.bs[1] + rr * pr.bs[2] : 0;
    moff[i] = pr.mask ? b * pr.ms[0] + h * pr.ms[1] + rr * pr.ms[2] : 0;
  }
  float o[kDvBlocks][4];
#pragma unroll
  for (int nb = 0; nb < kDvBlocks; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nb][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float s2scale = pr.scale * kLog2e;
  const int t_end = pr.causal ? min(pr.T, min(row0 + kBM, pr.S)) : pr.T;

  // K / V tiles are double-buffered: tile i + 1 is copied while tile i is computed, one barrier per tile
  const int k_first = crank * kBN;
  if (k_first < t_end) {
    stage_rows_any<float>(Kbuf, LDQ, kp, pr.ks[2], k_first, kBN, pr.T, D, false);
    stage_rows_any<float>(Vbuf, LDV, vp, pr.vs[2], k_first, kBN, pr.T, Dv, false);
  }
  int it = 0;
  for (int kt = k_first; kt < t_end; kt += kC * kBN, ++it) {
    stage_wait();
    __syncthreads();   // tile `it` (and, the first time, Q) has landed; nobody reads the other buffer any more
    const float* Ks = Kbuf + (it & 1) * kBN * LDQ;
    const float* Vs = Vbuf + (it & 1) * kBN * LDV;
    if (kt + kC * kBN < t_end) {
      stage_rows_any<float>(Kbuf + ((it + 1) & 1) * kBN * LDQ, LDQ, kp, pr.ks[2], kt + kC * kBN, kBN, pr.T, D, false);
      stage_rows_any<float>(Vbuf + ((it + 1) & 1) * kBN * LDV, LDV, vp, pr.vs[2], kt + kC * kBN, kBN, pr.T, Dv, false);
    }
    fwd_tf32x3_tile<kDvBlocks>(pr, bias_dtype, Qs, Ks, Vs, LDQ, LDV, D, kt, row0, lr, boff, moff, s2scale, g, t, o, m, l);
  }
  if constexpr (kC > 1) {
    // partial [kBM][Dv + 2] = (out, m, l) in this CTA's K stages; rank 0 merges ranks 1.. in order
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int LDP = Dv + 2;
    float* part = Kbuf;
    stage_wait();      // (a rank without a key tile still has its Q copy in flight)
    __syncthreads();   // the last tile's operands are no longer read
    if (crank > 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float* prow = part + lr[i] * LDP;
#pragma unroll
        for (int nb = 0; nb < kDvBlocks; ++nb)
          *reinterpret_cast<float2*>(prow + 8 * nb + 2 * t) = make_float2(o[nb][2 * i], o[nb][2 * i + 1]);
        if (t == 0) *reinterpret_cast<float2*>(prow + Dv) = make_float2(m[i], l[i]);
      }
    }
    cluster.sync();
    if (crank == 0) {
      for (int r = 1; r < kC; ++r) {
        const float* rp = cluster.map_shared_rank(part, r);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float* prow = rp + lr[i] * LDP;
          const float2 ml = *reinterpret_cast<const float2*>(prow + Dv);
          const float m_new = fmaxf(m[i], ml.x);
          const float m_ref = m_new == -INFINITY ? 0.f : m_new;   // nothing kept on either side: both weights are 0
          const float wa = exp2f(m[i] - m_ref), wb = exp2f(ml.x - m_ref);
          l[i] = l[i] * wa + ml.y * wb;
          m[i] = m_new;
#pragma unroll
          for (int nb = 0; nb < kDvBlocks; ++nb) {
            const float2 a = *reinterpret_cast<const float2*>(prow + 8 * nb + 2 * t);
            o[nb][2 * i] = o[nb][2 * i] * wa + a.x * wb;
            o[nb][2 * i + 1] = o[nb][2 * i + 1] * wa + a.y * wb;
          }
        }
      }
    }
    cluster.sync();    // nobody leaves while rank 0 still reads its shared memory
    if (crank > 0) return;
  }
  // ---- out = o / l (NaN for a row with no kept key, as the reference's softmax gives), lse ----
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + lr[i];
    if (row >= pr.S) continue;
    const float inv = 1.f / l[i];
    float* op = reinterpret_cast<float*>(pr.out) + b * pr.os[0] + h * pr.os[1] + row * pr.os[2];
#pragma unroll
    for (int nb = 0; nb < kDvBlocks; ++nb) {
      op[8 * nb + 2 * t] = l[i] == 0.f ? NAN : o[nb][2 * i] * inv;
      op[8 * nb + 2 * t + 1] = l[i] == 0.f ? NAN : o[nb][2 * i + 1] * inv;
    }
    if (t == 0) pr.lse[(int64_t(b) * pr.H + h) * pr.S + row] = m[i] + log2f(l[i]);
  }
}

// The same forward for SMALL problems: kG groups of four warps share a CTA's 64 query rows and take the key tiles in
// turn (group j tiles j, j + kG, ...), each with a K / V stage of its own and its own named barrier; at the end the
// groups' partial (m, l, out) are merged through shared memory by group 0.  The 3 x TF32 loop is bound by the
// latency of its mma.sync chain, not by the tensor pipe (one warp per scheduler keeps it about a tenth busy), and a
// problem of a hundred-odd CTAs cannot put more than four warps on an SM otherwise.
template <int kDvBlocks, int kG, bool kSquare>
__global__ void __launch_bounds__(kTiledThreads * kG) fwd_tf32x3_split_kernel(Problem pr, int bias_dtype) {
  extern __shared__ __align__(16) float smem[];
  constexpr int kBM = 64;
  constexpr int Dv = 8 * kDvBlocks;
  const int D = kSquare ? Dv : pr.D;
  const int LDQ = D + 4, LDV = Dv + 4;
  float* Qs = smem;                          // [kBM][LDQ]
  float* KV = Qs + kBM * LDQ;                // kG x ([kBN][LDQ] + [kBN][LDV]); afterwards the partial results
  const int kg = threadIdx.x >> 7, tg = threadIdx.x & 127;
  const int warp = tg >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  float* Ks = KV + kg * (kBN * LDQ + kBN * LDV);
  float* Vs = Ks + kBN * LDQ;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int row0 = blockIdx.x * kBM;
  const float* qp = reinterpret_cast<const float*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const float* kp = reinterpret_cast<const float*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const float* vp = reinterpret_cast<const float*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  stage_rows_f4(Qs, LDQ, qp, pr.qs[2], row0, kBM, pr.S, D);   // (the launcher checked the 16-byte alignment)
  stage_wait();
  __syncthreads();

  const int lr[2] = {16 * warp + g, 16 * warp + g + 8};
  int64_t boff[2], moff[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = min(row0 + lr[i], pr.S - 1);
    boff[i] = pr.bias ? b * pr.bs[0] + h * pr.bs[1] + rr * pr.bs[2] : 0;
    moff[i] = pr.mask ? b * pr.ms[0] + h * pr.ms[1] + rr * pr.ms[2] : 0;
  }
  float o[kDvBlocks][4];
#pragma unroll
  for (int nb = 0; nb < kDvBlocks; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nb][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float s2scale = pr.scale * kLog2e;
  const int t_end = pr.causal ? min(pr.T, min(row0 + kBM, pr.S)) : pr.T;
  auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + kg) : "memory"); };

  for (int kt = kg * kBN; kt < t_end; kt += kG * kBN) {
    group_sync();   // the group's previous tile is no longer read
    stage_rows_f4(Ks, LDQ, kp, pr.ks[2], kt, kBN, pr.T, D, tg, kTiledThreads);
    stage_rows_f4(Vs, LDV, vp, pr.vs[2], kt, kBN, pr.T, Dv, tg, kTiledThreads);
    stage_wait();
    group_sync();
    fwd_tf32x3_tile<kDvBlocks>(pr, bias_dtype, Qs, Ks, Vs, LDQ, LDV, D, kt, row0, lr, boff, moff, s2scale, g, t, o, m, l);
  }

  // ---- merge the groups: partial [kG - 1][64 rows][Dv + 2] = (out, m, l), in the K / V stages ----
  __syncthreads();
  const int LDP = Dv + 2;
  if (kg > 0) {
    float* part = KV + (kg - 1) * kBM * LDP;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float* prow = part + lr[i] * LDP;
#pragma unroll
      for (int nb = 0; nb < kDvBlocks; ++nb) {
        prow[8 * nb + 2 * t] = o[nb][2 * i];
        prow[8 * nb + 2 * t + 1] = o[nb][2 * i + 1];
      }
      if (t == 0) {
        prow[Dv] = m[i];
        prow[Dv + 1] = l[i];
      }
    }
  }
  __syncthreads();
  if (kg > 0) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    for (int j = 0; j < kG - 1; ++j) {
      const float* prow = KV + j * kBM * LDP + lr[i] * LDP;
      const float m2 = prow[Dv], l2 = prow[Dv + 1];
      const float m_new = fmaxf(m[i], m2);
      const float m_ref = m_new == -INFINITY ? 0.f : m_new;   // nothing kept on either side: both weights are 0
      const float wa = exp2f(m[i] - m_ref), wb = exp2f(m2 - m_ref);
      l[i] = l[i] * wa + l2 * wb;
      m[i] = m_new;
#pragma unroll
      for (int nb = 0; nb < kDvBlocks; ++nb) {
        o[nb][2 * i] = o[nb][2 * i] * wa + prow[8 * nb + 2 * t] * wb;
        o[nb][2 * i + 1] = o[nb][2 * i + 1] * wa + prow[8 * nb + 2 * t + 1] * wb;
      }
    }
    const int row = row0 + lr[i];
    if (row >= pr.S) continue;
    const float inv = 1.f / l[i];
    float* op = reinterpret_cast<float*>(pr.out) + b * pr.os[0] + h * pr.os[1] + row * pr.os[2];
#pragma unroll
    for (int nb = 0; nb < kDvBlocks; ++nb) {
      op[8 * nb + 2 * t] = l[i] == 0.f ? NAN : o[nb][2 * i] * inv;
      op[8 * nb + 2 * t + 1] = l[i] == 0.f ? NAN : o[nb][2 * i + 1] * inv;
    }
    if (t == 0) pr.lse[(int64_t(b) * pr.H + h) * pr.S + row] = m[i] + log2f(l[i]);
  }
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
// backward, query side, fp32 operands: 3 x TF32 on mma.sync (same tiling as fwd_tf32x3_kernel)
// ---------------------------------------------------------------------------
// A warp owns 16 query rows against a 64-key tile: S = Q K^T and dP = dO V^T in accumulator fragments,
// p = exp2(s - lse), ds = p (dP - delta) in place, then dQ += ds K with the ds fragment as the A operand (key 2 t /
// 2 t + 1 of a block stand in operand columns t / t + 4; the K rows are fetched in that order).
// One 64-key tile of the 3 x TF32 dq backward for this warp's 16 query rows: S and dP, p and ds (dbias on the way),
// dQ += ds K.  Ks / Vs: the tile in shared memory; kt: its first key.
template <int kDBlocks>
__device__ __forceinline__ void bwd_dq_tf32x3_tile(const Problem& pr, int bias_dtype, const float* Qs, const float* Gs,
                                                   const float* Ks, const float* Vs, int LDQ, int LDV, int D, int Dv,
                                                   int kt, int row0, const int (&lr)[2], const int64_t (&boff)[2],
                                                   const int64_t (&moff)[2], const int64_t (&dboff)[2],
                                                   const float (&lse)[2], const float (&delta)[2], float s2scale,
                                                   bool want_db, int g, int t, float (&dq)[kDBlocks][4]) {
  float sc[8][4], dp[8][4];
#pragma unroll
  for (int nb = 0; nb < 8; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) sc[nb][e] = dp[nb][e] = 0.f;
#pragma unroll 2
  for (int kk = 0; kk < D; kk += 8) {
    uint32_t ah[4], al[4];
    split_tf32(Qs[lr[0] * LDQ + kk + t], ah[0], al[0]);
    split_tf32(Qs[lr[1] * LDQ + kk + t], ah[1], al[1]);
    split_tf32(Qs[lr[0] * LDQ + kk + t + 4], ah[2], al[2]);
    split_tf32(Qs[lr[1] * LDQ + kk + t + 4], ah[3], al[3]);
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      uint32_t bh2[2], bl2[2];
      split_tf32(Ks[(8 * nb + g) * LDQ + kk + t], bh2[0], bl2[0]);
      split_tf32(Ks[(8 * nb + g) * LDQ + kk + t + 4], bh2[1], bl2[1]);
      mma_3xtf32(sc[nb], ah, al, bh2, bl2);
    }
  }
#pragma unroll 2
  for (int kk = 0; kk < Dv; kk += 8) {
    uint32_t ah[4], al[4];
    split_tf32(Gs[lr[0] * LDV + kk + t], ah[0], al[0]);
    split_tf32(Gs[lr[1] * LDV + kk + t], ah[1], al[1]);
    split_tf32(Gs[lr[0] * LDV + kk + t + 4], ah[2], al[2]);
    split_tf32(Gs[lr[1] * LDV + kk + t + 4], ah[3], al[3]);
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      uint32_t bh2[2], bl2[2];
      split_tf32(Vs[(8 * nb + g) * LDV + kk + t], bh2[0], bl2[0]);
      split_tf32(Vs[(8 * nb + g) * LDV + kk + t + 4], bh2[1], bl2[1]);
      mma_3xtf32(dp[nb], ah, al, bh2, bl2);
    }
  }
  // ---- p = exp2(logit2 - lse), ds = p (dP - delta); ds replaces the score fragment ----
  if (!pr.bias && !pr.mask && !want_db) {
    // nothing to load: keeping a key is a comparison with the last key of the row in this tile
    int last[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + lr[i];
      last[i] = row < pr.S ? (pr.causal ? min(pr.T - 1, row) : pr.T - 1) - kt : -1;
    }
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const float p = 8 * nb + 2 * t + (e & 1) <= last[i] ? ex2_fast(fmaf(sc[nb][e], s2scale, -lse[i])) : 0.f;
        sc[nb][e] = p * (dp[nb][e] - delta[i]);
      }
  } else {
    // bias / mask / dbias in the fragment layout: this thread's elements are keys kt + 2 t + (8 nb + c) of rows
    // lr[0], lr[1].  Pointers to the first of them once per tile, the dtype decided once per tile (a 64-bit
    // index product and a dtype switch per element were most of a tile's instructions).
    int last[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + lr[i];
      last[i] = row < pr.S ? (pr.causal ? min(pr.T - 1, row) : pr.T - 1) - kt : -1;
    }
    const int k0 = kt + 2 * t;
    auto ew = [&](auto tag) {
      using BT = decltype(tag);
      const BT* bp[2];
      BT* dbp[2];
      const uint8_t* mp[2];
      float* ap[2];
      const int64_t bs3 = pr.bs[3], ms3 = pr.ms[3], dbs3 = pr.dbs[3];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        bp[i] = pr.bias ? reinterpret_cast<const BT*>(pr.bias) + boff[i] + k0 * bs3 : nullptr;
        mp[i] = pr.mask ? pr.mask + moff[i] + k0 * ms3 : nullptr;
        dbp[i] = pr.dbias ? reinterpret_cast<BT*>(pr.dbias) + dboff[i] + k0 * dbs3 : nullptr;
        ap[i] = pr.dbias_accum ? pr.dbias_accum + dboff[i] + k0 * dbs3 : nullptr;
      }
#pragma unroll
      for (int nb = 0; nb < 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1, col = 8 * nb + (e & 1);      // key = k0 + col
          bool keep = col + 2 * t <= last[i];
          if (keep && mp[i]) keep = mp[i][col * ms3] != 0;
          const float bias = (keep && bp[i]) ? kLog2e * to_f32<BT>(bp[i][col * bs3]) : 0.f;
          const float p = keep ? ex2_fast(fmaf(sc[nb][e], s2scale, bias) - lse[i]) : 0.f;
          const float ds = p * (dp[nb][e] - delta[i]);
          sc[nb][e] = ds;
          if (want_db && k0 + col < pr.T && row0 + lr[i] < pr.S) {
            if (ap[i]) {
              if (ds != 0.f) atomicAdd(ap[i] + col * dbs3, ds);
            } else {
              dbp[i][col * dbs3] = from_f32<BT>(ds);
            }
          }
        }
    };
    if (bias_dtype == NB200_F32) ew(float{});
    else if (bias_dtype == NB200_BF16) ew(__nv_bfloat16{});
    else ew(__half{});
  }
  // ---- dQ += ds K ----
#pragma unroll
  for (int kb = 0; kb < 8; ++kb) {
    uint32_t ah[4], al[4];
    split_tf32(sc[kb][0], ah[0], al[0]);   // row g,     key 2 t
    split_tf32(sc[kb][2], ah[1], al[1]);   // row g + 8, key 2 t
    split_tf32(sc[kb][1], ah[2], al[2]);   // row g,     key 2 t + 1
    split_tf32(sc[kb][3], ah[3], al[3]);   // row g + 8, key 2 t + 1
    const float* k0 = Ks + (8 * kb + 2 * t) * LDQ + g;
    const float* k1 = k0 + LDQ;
#pragma unroll
    for (int nb = 0; nb < kDBlocks; ++nb) {
      uint32_t bh2[2], bl2[2];
      split_tf32(k0[8 * nb], bh2[0], bl2[0]);
      split_tf32(k1[8 * nb], bh2[1], bl2[1]);
      mma_3xtf32(dq[nb], ah, al, bh2, bl2);
    }
  }
}

//
// kC > 1 (the SMALLEST problems, launched as clusters of kC CTAs along x): the CTAs of a cluster own the same 64
// query rows and take the key tiles in turn -- kC times as many warps for the same latency-bound chain, each with a
// full register file (the in-CTA split above is capped at 128 registers a thread from four groups on); ranks 1..
// leave their partial dq tile in their own shared memory and rank 0 adds them over distributed shared memory in
// rank order.  Every dbias element is still written, or added, by exactly one CTA.
template <int kDBlocks, bool kSquare, int kC = 1>   // D / 8; kSquare: D == Dv, both row pitches compile-time constants
__global__ void __launch_bounds__(kTiledThreads) bwd_dq_tf32x3_kernel(Problem pr, int bias_dtype) {
  extern __shared__ __align__(16) float smem[];
  constexpr int kBM = 64;
  constexpr int D = 8 * kDBlocks;
  const int Dv = kSquare ? D : pr.Dv;
  const int LDQ = D + 4, LDV = Dv + 4;
  float* Qs = smem;                    // [kBM][LDQ]
  float* Gs = Qs + kBM * LDQ;          // [kBM][LDV]   dout rows
  float* Kbuf = Gs + kBM * LDV;        // 2 x [kBN][LDQ]
  float* Vbuf = Kbuf + 2 * kBN * LDQ;  // 2 x [kBN][LDV]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int crank = kC > 1 ? int(blockIdx.x) % kC : 0;   // rank in the cluster (cluster dims (kC, 1, 1))
  const int row0 = (int(blockIdx.x) / kC) * kBM;
  const float* qp = reinterpret_cast<const float*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const float* kp = reinterpret_cast<const float*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const float* vp = reinterpret_cast<const float*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  const float* gp = reinterpret_cast<const float*>(pr.dout) + b * pr.dos[0] + h * pr.dos[1];
  stage_rows_any<float>(Qs, LDQ, qp, pr.qs[2], row0, kBM, pr.S, D, false);
  stage_rows_any<float>(Gs, LDV, gp, pr.dos[2], row0, kBM, pr.S, Dv, false);

  const int lr[2] = {16 * warp + g, 16 * warp + g + 8};
  int64_t boff[2], moff[2], dboff[2];
  float lse[2], delta[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = min(row0 + lr[i], pr.S - 1);
    boff[i] = pr.bias ? b * pr.bs[0] + h * pr.bs[1] + rr * pr.bs[2] : 0;
    moff[i] = pr.mask ? b * pr.ms[0] + h * pr.ms[1] + rr * pr.ms[2] : 0;
    dboff[i] = b * pr.dbs[0] + h * pr.dbs[1] + rr * pr.dbs[2];
    const int64_t ridx = (int64_t(b) * pr.H + h) * pr.S + rr;
    lse[i] = pr.lse[ridx];
    delta[i] = pr.delta[ridx];
  }
  float dq[kDBlocks][4];
#pragma unroll
  for (int nb = 0; nb < kDBlocks; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) dq[nb][e] = 0.f;
  const float s2scale = pr.scale * kLog2e;
  const int t_end = pr.causal ? min(pr.T, min(row0 + kBM, pr.S)) : pr.T;
  const bool want_db = pr.dbias != nullptr || pr.dbias_accum != nullptr;

  const int k_first = crank * kBN;
  if (k_first < t_end) {
    stage_rows_any<float>(Kbuf, LDQ, kp, pr.ks[2], k_first, kBN, pr.T, D, false);
    stage_rows_any<float>(Vbuf, LDV, vp, pr.vs[2], k_first, kBN, pr.T, Dv, false);
  }
  int it = 0;
  for (int kt = k_first; kt < t_end; kt += kC * kBN, ++it) {
    stage_wait();
    __syncthreads();
    const float* Ks = Kbuf + (it & 1) * kBN * LDQ;
    const float* Vs = Vbuf + (it & 1) * kBN * LDV;
    if (kt + kC * kBN < t_end) {
      stage_rows_any<float>(Kbuf + ((it + 1) & 1) * kBN * LDQ, LDQ, kp, pr.ks[2], kt + kC * kBN, kBN, pr.T, D, false);
      stage_rows_any<float>(Vbuf + ((it + 1) & 1) * kBN * LDV, LDV, vp, pr.vs[2], kt + kC * kBN, kBN, pr.T, Dv, false);
    }
    bwd_dq_tf32x3_tile<kDBlocks>(pr, bias_dtype, Qs, Gs, Ks, Vs, LDQ, LDV, D, Dv, kt, row0, lr, boff, moff, dboff, lse,
                                 delta, s2scale, want_db, g, t, dq);
  }
  if constexpr (kC > 1) {
    // partial tiles [kBM][D] in this CTA's K stages; rank 0 adds ranks 1.. in order
    cg::cluster_group cluster = cg::this_cluster();
    float* part = Kbuf;
    stage_wait();      // (a rank without a key tile still has its Q / dout copies in flight)
    __syncthreads();   // the last tile's operands are no longer read
    if (crank > 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int nb = 0; nb < kDBlocks; ++nb)
          *reinterpret_cast<float2*>(part + lr[i] * D + 8 * nb + 2 * t) = make_float2(dq[nb][2 * i], dq[nb][2 * i + 1]);
    }
    cluster.sync();
    if (crank == 0) {
      for (int r = 1; r < kC; ++r) {
        const float* rp = cluster.map_shared_rank(part, r);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int nb = 0; nb < kDBlocks; ++nb) {
            const float2 a = *reinterpret_cast<const float2*>(rp + lr[i] * D + 8 * nb + 2 * t);
            dq[nb][2 * i] += a.x;
            dq[nb][2 * i + 1] += a.y;
          }
      }
    }
    cluster.sync();    // nobody leaves while rank 0 still reads its shared memory
    if (crank > 0) return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + lr[i];
    if (row >= pr.S) continue;
    // causal rows never visit keys past the CTA's last row, yet a dense dbias is written everywhere: exact zeros
    if (want_db && !pr.dbias_accum && t_end < pr.T) {
      for (int key = ((t_end + kBN - 1) / kBN) * kBN + t; key < pr.T; key += 4)
        store_from_f32(pr.dbias, dboff[i] + key * pr.dbs[3], bias_dtype, 0.f);
    }
    float* dqp = reinterpret_cast<float*>(pr.dq) + b * pr.dqs[0] + h * pr.dqs[1] + row * pr.dqs[2];
#pragma unroll
    for (int nb = 0; nb < kDBlocks; ++nb) {
      dqp[8 * nb + 2 * t] = dq[nb][2 * i] * pr.scale;
      dqp[8 * nb + 2 * t + 1] = dq[nb][2 * i + 1] * pr.scale;
    }
  }
}

// The dq backward for SMALL problems, as the forward's fwd_tf32x3_split_kernel: kG groups of four warps share a CTA's
// 64 query rows and take the key tiles in turn; their partial dq tiles are summed through shared memory by group 0.
// (Every dbias element is still written, or added, by exactly one group.)
template <int kDBlocks, int kG, bool kSquare>
__global__ void __launch_bounds__(kTiledThreads * kG) bwd_dq_tf32x3_split_kernel(Problem pr, int bias_dtype) {
  extern __shared__ __align__(16) float smem[];
  constexpr int kBM = 64;
  constexpr int D = 8 * kDBlocks;
  const int Dv = kSquare ? D : pr.Dv;
  const int LDQ = D + 4, LDV = Dv + 4;
  float* Qs = smem;                    // [kBM][LDQ]
  float* Gs = Qs + kBM * LDQ;          // [kBM][LDV]   dout rows
  float* KV = Gs + kBM * LDV;          // kG x ([kBN][LDQ] + [kBN][LDV]); afterwards the partial dq tiles
  const int kg = threadIdx.x >> 7, tg = threadIdx.x & 127;
  const int warp = tg >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  float* Ks = KV + kg * (kBN * LDQ + kBN * LDV);
  float* Vs = Ks + kBN * LDQ;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int row0 = blockIdx.x * kBM;
  const float* qp = reinterpret_cast<const float*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const float* kp = reinterpret_cast<const float*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const float* vp = reinterpret_cast<const float*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  const float* gp = reinterpret_cast<const float*>(pr.dout) + b * pr.dos[0] + h * pr.dos[1];
  stage_rows_f4(Qs, LDQ, qp, pr.qs[2], row0, kBM, pr.S, D);     // (the launcher checked the 16-byte alignment)
  stage_rows_f4(Gs, LDV, gp, pr.dos[2], row0, kBM, pr.S, Dv);
  stage_wait();
  __syncthreads();

  const int lr[2] = {16 * warp + g, 16 * warp + g + 8};
  int64_t boff[2], moff[2], dboff[2];
  float lse[2], delta[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = min(row0 + lr[i], pr.S - 1);
    boff[i] = pr.bias ? b * pr.bs[0] + h * pr.bs[1] + rr * pr.bs[2] : 0;
    moff[i] = pr.mask ? b * pr.ms[0] + h * pr.ms[1] + rr * pr.ms[2] : 0;
    dboff[i] = b * pr.dbs[0] + h * pr.dbs[1] + rr * pr.dbs[2];
    const int64_t ridx = (int64_t(b) * pr.H + h) * pr.S + rr;
    lse[i] = pr.lse[ridx];
    delta[i] = pr.delta[ridx];
  }
  float dq[kDBlocks][4];
#pragma unroll
  for (int nb = 0; nb < kDBlocks; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) dq[nb][e] = 0.f;
  const float s2scale = pr.scale * kLog2e;
  const int t_end = pr.causal ? min(pr.T, min(row0 + kBM, pr.S)) : pr.T;
  const bool want_db = pr.dbias != nullptr || pr.dbias_accum != nullptr;
  auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + kg) : "memory"); };

  for (int kt = kg * kBN; kt < t_end; kt += kG * kBN) {
    group_sync();   // the group's previous tile is no longer read
    stage_rows_f4(Ks, LDQ, kp, pr.ks[2], kt, kBN, pr.T, D, tg, kTiledThreads);
    stage_rows_f4(Vs, LDV, vp, pr.vs[2], kt, kBN, pr.T, Dv, tg, kTiledThreads);
    stage_wait();
    group_sync();
    bwd_dq_tf32x3_tile<kDBlocks>(pr, bias_dtype, Qs, Gs, Ks, Vs, LDQ, LDV, D, Dv, kt, row0, lr, boff, moff, dboff, lse,
                                 delta, s2scale, want_db, g, t, dq);
  }

  // ---- sum the groups' dq tiles: partial [kG - 1][64 rows][D], in the K / V stages ----
  __syncthreads();
  if (kg > 0) {
    float* part = KV + (kg - 1) * kBM * D;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int nb = 0; nb < kDBlocks; ++nb) {
        part[lr[i] * D + 8 * nb + 2 * t] = dq[nb][2 * i];
        part[lr[i] * D + 8 * nb + 2 * t + 1] = dq[nb][2 * i + 1];
      }
  }
  __syncthreads();
  if (kg > 0) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + lr[i];
    if (row >= pr.S) continue;
    // causal rows never visit keys past the CTA's last row, yet a dense dbias is written everywhere: exact zeros
    if (want_db && !pr.dbias_accum && t_end < pr.T) {
      for (int key = ((t_end + kBN - 1) / kBN) * kBN + t; key < pr.T; key += 4)
        store_from_f32(pr.dbias, dboff[i] + key * pr.dbs[3], bias_dtype, 0.f);
    }
    float* dqp = reinterpret_cast<float*>(pr.dq) + b * pr.dqs[0] + h * pr.dqs[1] + row * pr.dqs[2];
#pragma unroll
    for (int nb = 0; nb < kDBlocks; ++nb) {
      float x0 = dq[nb][2 * i], x1 = dq[nb][2 * i + 1];
      for (int j = 0; j < kG - 1; ++j) {
        x0 += KV[j * kBM * D + lr[i] * D + 8 * nb + 2 * t];
        x1 += KV[j * kBM * D + lr[i] * D + 8 * nb + 2 * t + 1];
      }
      dqp[8 * nb + 2 * t] = x0 * pr.scale;
      dqp[8 * nb + 2 * t + 1] = x1 * pr.scale;
    }
  }
}

// ---------------------------------------------------------------------------
// backward, key side, fp32 operands: 3 x TF32 on mma.sync
// ---------------------------------------------------------------------------
// A warp owns 16 keys against a 64-query tile: S^T = K Q^T and dP^T = V dO^T in accumulator fragments (row = key,
// column = query), p and ds in place, then dV += p^T-fragment dO and dK += ds-fragment Q with the fragments as A
// operands (query 2 t / 2 t + 1 of a block stand in operand columns t / t + 4).  lse and delta of the tile's
// queries sit in shared memory.  Head dims D == Dv in {32, 64, 128} (at 128 the two accumulator sets fill the
// register file: 255 registers and a few spilled words).
//
// kC > 1 (SMALL problems, launched as clusters of kC CTAs along x): the kC CTAs of a cluster own the same 64 keys and
// take the query tiles in turn, which puts kC times as many warps on the machine for the same latency-bound chain;
// ranks 1.. leave their partial dk / dv tiles in their own shared memory and rank 0 sums them over distributed
// shared memory in a fixed order (deterministic) before it writes.
template <int kBlocks, int kC = 1>   // D / 8 == Dv / 8
__global__ void __launch_bounds__(kTiledThreads) bwd_dkv_tf32x3_kernel(Problem pr, int bias_dtype) {
  extern __shared__ __align__(16) float smem[];
  constexpr int kBK = 64;
  constexpr int D = 8 * kBlocks, LD = D + 4;   // compile-time row pitch: every fragment offset is an immediate
  float* Ks = smem;                    // [kBK][LD]  owner keys
  float* Vs = Ks + kBK * LD;           // [kBK][LD]
  float* Qbuf = Vs + kBK * LD;         // 2 x [kBN][LD]
  float* Gbuf = Qbuf + 2 * kBN * LD;   // 2 x [kBN][LD]  dout rows
  float* Lbuf = Gbuf + 2 * kBN * LD;   // 2 x [kBN]  lse
  float* Dbuf = Lbuf + 2 * kBN;        // 2 x [kBN]  delta
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int bh = pr.bh_begin + blockIdx.y;
  const int b = bh / pr.H, h = bh - b * pr.H;
  const int crank = kC > 1 ? int(blockIdx.x) % kC : 0;   // rank in the cluster (cluster dims (kC, 1, 1))
  const int key0 = (int(blockIdx.x) / kC) * kBK;
  const float* qp = reinterpret_cast<const float*>(pr.q) + b * pr.qs[0] + h * pr.qs[1];
  const float* kp = reinterpret_cast<const float*>(pr.k) + b * pr.ks[0] + h * pr.ks[1];
  const float* vp = reinterpret_cast<const float*>(pr.v) + b * pr.vs[0] + h * pr.vs[1];
  const float* gp = reinterpret_cast<const float*>(pr.dout) + b * pr.dos[0] + h * pr.dos[1];
  const int64_t rbase = (int64_t(b) * pr.H + h) * pr.S;
  stage_rows_any<float>(Ks, LD, kp, pr.ks[2], key0, kBK, pr.T, D, false);
  stage_rows_any<float>(Vs, LD, vp, pr.vs[2], key0, kBK, pr.T, D, false);

  const int lr[2] = {16 * warp + g, 16 * warp + g + 8};
  int64_t boff[2], moff[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int kk = min(key0 + lr[i], pr.T - 1);
    boff[i] = pr.bias ? b * pr.bs[0] + h * pr.bs[1] + kk * pr.bs[3] : 0;
    moff[i] = pr.mask ? b * pr.ms[0] + h * pr.ms[1] + kk * pr.ms[3] : 0;
  }
  float dk[kBlocks][4], dv[kBlocks][4];
#pragma unroll
  for (int nb = 0; nb < kBlocks; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk[nb][e] = dv[nb][e] = 0.f;
  const float s2scale = pr.scale * kLog2e;
  // causal: queries before this CTA's first key see none of its keys
  const int s_begin = pr.causal ? min(pr.S, key0) : 0;

  auto prefetch = [&](int qt, int buf) {
    stage_rows_any<float>(Qbuf + buf * kBN * LD, LD, qp, pr.qs[2], qt, kBN, pr.S, D, false);
    stage_rows_any<float>(Gbuf + buf * kBN * LD, LD, gp, pr.dos[2], qt, kBN, pr.S, D, false);
    if (threadIdx.x < kBN) {
      const int q = qt + threadIdx.x;
      Lbuf[buf * kBN + threadIdx.x] = q < pr.S ? pr.lse[rbase + q] : 0.f;
      Dbuf[buf * kBN + threadIdx.x] = q < pr.S ? pr.delta[rbase + q] : 0.f;
    }
  };
  const int q_first = s_begin + crank * kBN;
  if (q_first < pr.S) prefetch(q_first, 0);
  int it = 0;
  for (int qt = q_first; qt < pr.S; qt += kC * kBN, ++it) {
    stage_wait();
    __syncthreads();   // tile `it` (and, the first time, K and V) has landed; nobody reads the other buffers any more
    const float* Qt = Qbuf + (it & 1) * kBN * LD;
    const float* Gt = Gbuf + (it & 1) * kBN * LD;
    const float* Lt = Lbuf + (it & 1) * kBN;
    const float* Dt = Dbuf + (it & 1) * kBN;
    if (qt + kC * kBN < pr.S) prefetch(qt + kC * kBN, (it + 1) & 1);
    float sc[8][4], dp[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[nb][e] = dp[nb][e] = 0.f;
#pragma unroll 2
    for (int kk = 0; kk < D; kk += 8) {
      uint32_t ah[4], al[4], ch[4], cl[4];
      split_tf32(Ks[lr[0] * LD + kk + t], ah[0], al[0]);
      split_tf32(Ks[lr[1] * LD + kk + t], ah[1], al[1]);
      split_tf32(Ks[lr[0] * LD + kk + t + 4], ah[2], al[2]);
      split_tf32(Ks[lr[1] * LD + kk + t + 4], ah[3], al[3]);
      split_tf32(Vs[lr[0] * LD + kk + t], ch[0], cl[0]);
      split_tf32(Vs[lr[1] * LD + kk + t], ch[1], cl[1]);
      split_tf32(Vs[lr[0] * LD + kk + t + 4], ch[2], cl[2]);
      split_tf32(Vs[lr[1] * LD + kk + t + 4], ch[3], cl[3]);
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        uint32_t bh2[2], bl2[2];
        split_tf32(Qt[(8 * nb + g) * LD + kk + t], bh2[0], bl2[0]);
        split_tf32(Qt[(8 * nb + g) * LD + kk + t + 4], bh2[1], bl2[1]);
        mma_3xtf32(sc[nb], ah, al, bh2, bl2);
        split_tf32(Gt[(8 * nb + g) * LD + kk + t], bh2[0], bl2[0]);
        split_tf32(Gt[(8 * nb + g) * LD + kk + t + 4], bh2[1], bl2[1]);
        mma_3xtf32(dp[nb], ch, cl, bh2, bl2);
      }
    }
    // ---- p (kept in sc) and ds (kept in dp); row = key, column = query ----
    if (!pr.bias && !pr.mask) {
      // nothing to load: a query keeps the keys up to a last one (none past S)
#pragma unroll
      for (int nb = 0; nb < 8; ++nb)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int ql = 8 * nb + 2 * t + c, q = qt + ql;
          const int last = q < pr.S ? (pr.causal ? min(pr.T - 1, q) : pr.T - 1) - key0 : -1;
          const float lq = Lt[ql], dq_ = Dt[ql];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int e = 2 * i + c;
            const float p = lr[i] <= last ? ex2_fast(fmaf(sc[nb][e], s2scale, -lq)) : 0.f;
            sc[nb][e] = p;
            dp[nb][e] = p * (dp[nb][e] - dq_);
          }
        }
    } else
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1, ql = 8 * nb + 2 * t + (e & 1);
        const int key = key0 + lr[i], q = qt + ql;
        bool keep = key < pr.T && q < pr.S && !(pr.causal && key > q);
        if (keep && pr.mask) keep = pr.mask[moff[i] + q * pr.ms[2]] != 0;
        const float bias = (keep && pr.bias) ? kLog2e * load_as_f32(pr.bias, boff[i] + q * pr.bs[2], bias_dtype) : 0.f;
        const float p = keep ? ex2_fast(fmaf(sc[nb][e], s2scale, bias) - Lt[ql]) : 0.f;
        sc[nb][e] = p;
        dp[nb][e] = p * (dp[nb][e] - Dt[ql]);
      }
    // ---- dV += p dO, dK += ds Q (contraction over the tile's queries) ----
#pragma unroll
    for (int qb = 0; qb < 8; ++qb) {
      uint32_t ph[4], pl[4], sh[4], sl[4];
      split_tf32(sc[qb][0], ph[0], pl[0]);
      split_tf32(sc[qb][2], ph[1], pl[1]);
      split_tf32(sc[qb][1], ph[2], pl[2]);
      split_tf32(sc[qb][3], ph[3], pl[3]);
      split_tf32(dp[qb][0], sh[0], sl[0]);
      split_tf32(dp[qb][2], sh[1], sl[1]);
      split_tf32(dp[qb][1], sh[2], sl[2]);
      split_tf32(dp[qb][3], sh[3], sl[3]);
      const float* g0 = Gt + (8 * qb + 2 * t) * LD + g;
      const float* q0 = Qt + (8 * qb + 2 * t) * LD + g;
#pragma unroll
      for (int nb = 0; nb < kBlocks; ++nb) {
        uint32_t bh2[2], bl2[2];
        split_tf32(g0[8 * nb], bh2[0], bl2[0]);
        split_tf32(g0[LD + 8 * nb], bh2[1], bl2[1]);
        mma_3xtf32(dv[nb], ph, pl, bh2, bl2);
        split_tf32(q0[8 * nb], bh2[0], bl2[0]);
        split_tf32(q0[LD + 8 * nb], bh2[1], bl2[1]);
        mma_3xtf32(dk[nb], sh, sl, bh2, bl2);
      }
    }
  }
  if constexpr (kC > 1) {
    // partial tiles [2][kBK][D] (dk, dv) in this CTA's query stages; rank 0 adds ranks 1.. in order
    cg::cluster_group cluster = cg::this_cluster();
    float* part = Qbuf;
    stage_wait();      // (a rank without a query tile still has its K / V copies in flight)
    __syncthreads();   // the last tile's operands are no longer read
    if (crank > 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int nb = 0; nb < kBlocks; ++nb) {
          *reinterpret_cast<float2*>(part + lr[i] * D + 8 * nb + 2 * t) = make_float2(dk[nb][2 * i], dk[nb][2 * i + 1]);
          *reinterpret_cast<float2*>(part + (kBK + lr[i]) * D + 8 * nb + 2 * t) = make_float2(dv[nb][2 * i], dv[nb][2 * i + 1]);
        }
    }
    cluster.sync();
    if (crank == 0) {
      for (int r = 1; r < kC; ++r) {
        const float* rp = cluster.map_shared_rank(part, r);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int nb = 0; nb < kBlocks; ++nb) {
            const float2 a = *reinterpret_cast<const float2*>(rp + lr[i] * D + 8 * nb + 2 * t);
            const float2 c = *reinterpret_cast<const float2*>(rp + (kBK + lr[i]) * D + 8 * nb + 2 * t);
            dk[nb][2 * i] += a.x; dk[nb][2 * i + 1] += a.y;
            dv[nb][2 * i] += c.x; dv[nb][2 * i + 1] += c.y;
          }
      }
    }
    cluster.sync();    // nobody leaves while rank 0 still reads its shared memory
    if (crank > 0) return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int key = key0 + lr[i];
    if (key >= pr.T) continue;
    float* dkp = reinterpret_cast<float*>(pr.dk) + b * pr.dks[0] + h * pr.dks[1] + key * pr.dks[2];
    float* dvp = reinterpret_cast<float*>(pr.dv) + b * pr.dvs[0] + h * pr.dvs[1] + key * pr.dvs[2];
#pragma unroll
    for (int nb = 0; nb < kBlocks; ++nb) {
      dkp[8 * nb + 2 * t] = dk[nb][2 * i] * pr.scale;
      dkp[8 * nb + 2 * t + 1] = dk[nb][2 * i + 1] * pr.scale;
      dvp[8 * nb + 2 * t] = dv[nb][2 * i];
      dvp[8 * nb + 2 * t + 1] = dv[nb][2 * i + 1];
    }
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

template <typename T, int kVChunks, int kR>
int fwd_tiled_r(const Problem& pr, int bias_dtype, cudaStream_t st) {
  constexpr int kBM = 16 * kR;
  const size_t smem = sizeof(float) * (size_t(kBM + kBN) * (pr.D + 4) + size_t(kBN) * (pr.Dv + 4) + size_t(kBM) * (kBN + 4));
  if (int rc = prepare(simt_fwd_tiled_kernel<T, kVChunks, kR>, smem)) return rc;
  dim3 grid((pr.S + kBM - 1) / kBM, pr.bh_count);
  simt_fwd_tiled_kernel<T, kVChunks, kR><<<grid, kTiledThreads, smem, st>>>(pr, bias_dtype);
  count_launch();
  return check_launch("simt_fwd_tiled_kernel");
}

template <typename T, int kVChunks>
int fwd_tiled_t(const Problem& pr, int bias_dtype, cudaStream_t st) {
  // small problems: 32-row CTAs, so that every SM gets at least two of them
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t ctas64 = int64_t((pr.S + 63) / 64) * pr.bh_count;
  if (ctas64 < 3 * int64_t(sms > 0 ? sms : 148)) return fwd_tiled_r<T, kVChunks, 2>(pr, bias_dtype, st);
  return fwd_tiled_r<T, kVChunks, 4>(pr, bias_dtype, st);
}

template <int kDvBlocks, int kG, bool kSquare>
int fwd_tf32x3_split_t(const Problem& pr, int bias_dtype, cudaStream_t st) {
  const size_t smem = sizeof(float) * (size_t(64) * (pr.D + 4) + size_t(kG) * kBN * (pr.D + 4 + pr.Dv + 4));
  if (int rc = prepare(fwd_tf32x3_split_kernel<kDvBlocks, kG, kSquare>, smem)) return rc;
  dim3 grid((pr.S + 63) / 64, pr.bh_count);
  fwd_tf32x3_split_kernel<kDvBlocks, kG, kSquare><<<grid, kTiledThreads * kG, smem, st>>>(pr, bias_dtype);
  count_launch();
  return check_launch("fwd_tf32x3_kernel");
}

template <int kDvBlocks, bool kSquare>
int fwd_tf32x3_t(const Problem& pr, int bias_dtype, cudaStream_t st) {
  // A small problem (fewer 64-row CTAs than two per SM would hold) with several key tiles: groups of warps split the
  // keys inside each CTA (see fwd_tf32x3_split_kernel).  Needs 16-byte aligned fp32 rows for the asynchronous copies.
  {
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t ctas = int64_t((pr.S + 63) / 64) * pr.bh_count;
    const int tiles = (pr.T + kBN - 1) / kBN;
    auto rows16 = [](const void* p, const int64_t* st3) {
      return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && st3[0] % 4 == 0 && st3[1] % 4 == 0 && st3[2] % 4 == 0;
    };
    const bool aligned = rows16(pr.q, pr.qs) && rows16(pr.k, pr.ks) && rows16(pr.v, pr.vs);
    // the smallest problems: clusters of four CTAs per 64-row tile, while all of them are resident at once and the
    // in-CTA split below could not give every key tile a warp group with a full register file
    if constexpr (kDvBlocks <= 8)
    if (tiles >= 4 && pr.D <= 64 && 4 * ctas <= 2 * int64_t(sms > 0 ? sms : 148)) {
      const size_t smem = sizeof(float) * (size_t(64 + 2 * kBN) * (pr.D + 4) + size_t(2 * kBN) * (pr.Dv + 4));
      if (int rc = prepare(fwd_tf32x3_kernel<kDvBlocks, kSquare, 4>, smem)) return rc;
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(unsigned((pr.S + 63) / 64) * 4, pr.bh_count);
      cfg.blockDim = dim3(kTiledThreads);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = st;
      cudaLaunchAttribute attr{};
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 4;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      (void)cudaLaunchKernelEx(&cfg, fwd_tf32x3_kernel<kDvBlocks, kSquare, 4>, pr, bias_dtype);   // errors: check_launch
      count_launch();
      return check_launch("fwd_tf32x3_kernel");
    }
    if constexpr (kDvBlocks <= 8)
    if (aligned && ctas <= 2 * int64_t(sms > 0 ? sms : 148) && tiles >= 2 && pr.D <= 64 && pr.Dv <= 64) {
      if (tiles >= 4) return fwd_tf32x3_split_t<kDvBlocks, 4, kSquare>(pr, bias_dtype, st);
      if (tiles == 3) return fwd_tf32x3_split_t<kDvBlocks, 3, kSquare>(pr, bias_dtype, st);
      return fwd_tf32x3_split_t<kDvBlocks, 2, kSquare>(pr, bias_dtype, st);
    }
  }
  const size_t smem = sizeof(float) * (size_t(64 + 2 * kBN) * (pr.D + 4) + size_t(2 * kBN) * (pr.Dv + 4));
  if (int rc = prepare(fwd_tf32x3_kernel<kDvBlocks, kSquare>, smem)) return rc;
  dim3 grid((pr.S + 63) / 64, pr.bh_count);
  fwd_tf32x3_kernel<kDvBlocks, kSquare><<<grid, kTiledThreads, smem, st>>>(pr, bias_dtype);
  count_launch();
  return check_launch("fwd_tf32x3_kernel");
}

template <typename T>
int fwd_t(const Problem& pr, int bias_dtype, cudaStream_t st) {
  if constexpr (sizeof(T) == 4) {
    // fp32 operands with head dims in whole 8-column MMA blocks: 3 x TF32 on the warp-level tensor-core path
    if (pr.D % 8 == 0 && pr.D <= 128 && pr.Dv % 8 == 0 && pr.Dv <= 128) {
      switch (pr.Dv / 8) {
        case 4: return pr.D == 32 ? fwd_tf32x3_t<4, true>(pr, bias_dtype, st) : fwd_tf32x3_t<4, false>(pr, bias_dtype, st);
        case 8: return pr.D == 64 ? fwd_tf32x3_t<8, true>(pr, bias_dtype, st) : fwd_tf32x3_t<8, false>(pr, bias_dtype, st);
        case 16: return pr.D == 128 ? fwd_tf32x3_t<16, true>(pr, bias_dtype, st) : fwd_tf32x3_t<16, false>(pr, bias_dtype, st);
        default: break;
      }
    }
  }
  // the register-tiled kernel takes head dims it can read as float4 and split over 8 threads in float4 chunks
  if (pr.D % 4 == 0 && pr.D <= 128 && pr.Dv % 32 == 0 && pr.Dv <= 128) {
    switch (pr.Dv / 32) {
      case 1: return fwd_tiled_t<T, 1>(pr, bias_dtype, st);
      case 2: return fwd_tiled_t<T, 2>(pr, bias_dtype, st);
      case 3: return fwd_tiled_t<T, 3>(pr, bias_dtype, st);
      default: return fwd_tiled_t<T, 4>(pr, bias_dtype, st);
    }
  }
  const size_t smem = fwd_smem(pr);
  if (int rc = prepare(simt_fwd_kernel<T>, smem)) return rc;
  dim3 grid((pr.S + kWarps - 1) / kWarps, pr.bh_count);
  simt_fwd_kernel<T><<<grid, kWarps * 32, smem, st>>>(pr, bias_dtype);
  count_launch();
  return check_launch("simt_fwd_kernel");
}

int sm_count() {
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

bool fp32_rows16(const void* p, const int64_t* st3) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && st3[0] % 4 == 0 && st3[1] % 4 == 0 && st3[2] % 4 == 0;
}

// Small fp32 problems, dq: the number of warp groups that split the key tiles inside each 64-row CTA
// (bwd_dq_tf32x3_split_kernel), 0 when that kernel does not apply.
int bwd_dq_split_groups(const Problem& pr) {
  const int64_t ctas = int64_t((pr.S + 63) / 64) * pr.bh_count;
  const int tiles = (pr.T + kBN - 1) / kBN;
  if (!(pr.S > 0 && (pr.D == 32 || pr.D == 64) && (pr.Dv == 32 || pr.Dv == 64) && tiles >= 2 &&
        ctas <= 2 * int64_t(sm_count()) && fp32_rows16(pr.q, pr.qs) && fp32_rows16(pr.k, pr.ks) &&
        fp32_rows16(pr.v, pr.vs) && fp32_rows16(pr.dout, pr.dos)))
    return 0;
  return (tiles >= 5 || tiles == 3) ? 3 : 2;
}

// The smallest fp32 problems, dq: the number of CTAs per cluster that split the key tiles of each 64-row tile
// (bwd_dq_tf32x3_kernel<., ., kC>), 0 when that does not apply: every CTA of the launch must be resident at once
// (two per SM: ~236 registers a thread), and it has to beat the in-CTA split, which shares the Q / dout stage --
// so only where the in-CTA split cannot give every key tile a warp group of its own.
int bwd_dq_cluster_size(const Problem& pr) {
  const int64_t ctas = int64_t((pr.S + 63) / 64) * pr.bh_count;
  const int tiles = (pr.T + kBN - 1) / kBN;
  if (!(pr.S > 0 && (pr.D == 32 || pr.D == 64) && (pr.Dv == 32 || pr.Dv == 64) && tiles >= 4)) return 0;
  return 4 * ctas <= 2 * int64_t(sm_count()) ? 4 : 0;
}

// Small fp32 problems, dk / dv: the number of CTAs per cluster that split the query tiles of each 64-key tile
// (bwd_dkv_tf32x3_kernel<., kC>), 0 when a cluster launch does not apply -- it does as long as every CTA of the
// launch is resident at once (two per SM: ~200 registers a thread): the point is more warps per SM, not more waves.
// Measured, fp32 D 64, dk / dv kernel alone: B2 H8 S256 114 -> 39 us (four CTAs per cluster), B4 H6 S344
// 100 -> 72 us (two), B1 H8 S1024 244 -> 154 us (two).
int bwd_dkv_cluster_size(const Problem& pr) {
  const int64_t ctas = int64_t((pr.T + 63) / 64) * pr.bh_count;
  const int q_tiles = (pr.S + 63) / 64;
  const int64_t resident = 2 * int64_t(sm_count());
  if (!(pr.T > 0 && pr.D == pr.Dv && (pr.D == 32 || pr.D == 64) && q_tiles >= 2 && 2 * ctas <= resident)) return 0;
  return (q_tiles >= 3 && 4 * ctas <= resident) ? 4 : 2;
}

template <typename T>
int bwd_t(const Problem& pr, int bias_dtype, cudaStream_t st) {
  const size_t smem = bwd_smem(pr);
  if (int rc = prepare(simt_bwd_dq_kernel<T>, smem)) return rc;
  if (int rc = prepare(simt_bwd_dkv_kernel<T>, smem)) return rc;
  // The dq (+ dbias) kernel and the dk / dv kernel are independent.  On a small problem neither fills the GPU (each
  // is bound by the latency of one warp's chain of dependent steps over the opposite operand's tiles, not by
  // throughput), so the second one runs on a side stream between a fork and a join event and the pair takes about as
  // long as the slower one.
  cudaStream_t st_kv = st;
  const SideStream* side = nullptr;
  {
    const int64_t ctas_q = int64_t((pr.S + kWarps - 1) / kWarps) * pr.bh_count;
    const int64_t ctas_k = int64_t((pr.T + kWarps - 1) / kWarps) * pr.bh_count;
    // (C1, fp32 B2 H4 L256: 0.149 -> 0.106 ms per step.  Twice that many rows and the two kernels already cover
    // the machine between them: B2 H8 S256 73 -> 71 us per backward, B1 H8 S1024 272 -> 298 us.)
    if (pr.S > 0 && pr.T > 0 && ctas_q + ctas_k <= 4 * 148) side = side_stream(st);
    if (side) {
      if (cudaEventRecord(side->fork, st) == cudaSuccess && cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess) {
        st_kv = side->stream;
      } else {
        cudaGetLastError();
        side = nullptr;
      }
    }
  }
  auto join = [&](int rc) -> int {
    if (side && (cudaEventRecord(side->join, side->stream) != cudaSuccess ||
                 cudaStreamWaitEvent(st, side->join, 0) != cudaSuccess)) {
      set_error("joining the side stream: %s", cudaGetErrorString(cudaGetLastError()));
      return rc ? rc : NB200_ERR_LAUNCH;
    }
    return rc;
  };
  bool dq_done = false;
  if constexpr (sizeof(T) == 4) {
    // the smallest problems: clusters of CTAs split the key tiles of each 64-row tile
    if (const int kc = bwd_dq_cluster_size(pr)) {
      const size_t sm = sizeof(float) * (size_t(64 + 2 * kBN) * (pr.D + 4) + size_t(64 + 2 * kBN) * (pr.Dv + 4));
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(unsigned((pr.S + 63) / 64) * kc, pr.bh_count);
      cfg.blockDim = dim3(kTiledThreads);
      cfg.dynamicSmemBytes = sm;
      cfg.stream = st;
      cudaLaunchAttribute attr{};
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = kc;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int rc = NB200_OK;
      auto go = [&](auto kernel) {
        if ((rc = prepare(kernel, sm)) != NB200_OK) return;
        (void)cudaLaunchKernelEx(&cfg, kernel, pr, bias_dtype);   // a failure is read by check_launch below
      };
      const bool sq = pr.D == pr.Dv;
      if (pr.D == 32) { if (sq) go(bwd_dq_tf32x3_kernel<4, true, 4>); else go(bwd_dq_tf32x3_kernel<4, false, 4>); }
      else { if (sq) go(bwd_dq_tf32x3_kernel<8, true, 4>); else go(bwd_dq_tf32x3_kernel<8, false, 4>); }
      if (rc) return join(rc);
      count_launch();
      if (int rc2 = check_launch("bwd_dq_tf32x3_kernel")) return join(rc2);
      dq_done = true;
    }
    // small problems: groups of warps split the key tiles inside each 64-row CTA
    if (!dq_done)
    if (const int kg = bwd_dq_split_groups(pr)) {
      const size_t sm = sizeof(float) * size_t(64 + kg * kBN) * (pr.D + 4 + pr.Dv + 4);
      dim3 gq((pr.S + 63) / 64, pr.bh_count);
      int rc = NB200_OK;
      auto go = [&](auto kernel) {
        if ((rc = prepare(kernel, sm)) == NB200_OK) kernel<<<gq, kTiledThreads * kg, sm, st>>>(pr, bias_dtype);
      };
      const bool sq = pr.D == pr.Dv;
      if (pr.D == 32) {
        if (kg == 3) { if (sq) go(bwd_dq_tf32x3_split_kernel<4, 3, true>); else go(bwd_dq_tf32x3_split_kernel<4, 3, false>); }
        else { if (sq) go(bwd_dq_tf32x3_split_kernel<4, 2, true>); else go(bwd_dq_tf32x3_split_kernel<4, 2, false>); }
      } else {
        if (kg == 3) { if (sq) go(bwd_dq_tf32x3_split_kernel<8, 3, true>); else go(bwd_dq_tf32x3_split_kernel<8, 3, false>); }
        else { if (sq) go(bwd_dq_tf32x3_split_kernel<8, 2, true>); else go(bwd_dq_tf32x3_split_kernel<8, 2, false>); }
      }
      if (rc) return join(rc);
      count_launch();
      if (int rc2 = check_launch("bwd_dq_tf32x3_kernel")) return join(rc2);
      dq_done = true;
    }
  }
  if constexpr (sizeof(T) == 4) {
    if (!dq_done)
    // fp32 operands with head dims in whole 8-column MMA blocks: 3 x TF32 on the warp-level tensor-core path
    // (a grid of fewer than ~100 CTAs of 64 rows leaves most SMs idle: tiny problems keep the 8-row CUDA-core CTAs)
    if (pr.S > 0 && pr.Dv % 8 == 0 && pr.Dv <= 128 && (pr.D == 32 || pr.D == 64 || pr.D == 128) &&
        int64_t((pr.S + 63) / 64) * pr.bh_count >= 96) {
      const size_t sm = sizeof(float) * (size_t(64 + 2 * kBN) * (pr.D + 4) + size_t(64 + 2 * kBN) * (pr.Dv + 4));
      dim3 gq((pr.S + 63) / 64, pr.bh_count);
      int rc = NB200_OK;
      auto go = [&](auto kernel) {
        if ((rc = prepare(kernel, sm)) == NB200_OK) kernel<<<gq, kTiledThreads, sm, st>>>(pr, bias_dtype);
      };
      const bool sq = pr.D == pr.Dv;
      if (pr.D == 32) { if (sq) go(bwd_dq_tf32x3_kernel<4, true>); else go(bwd_dq_tf32x3_kernel<4, false>); }
      else if (pr.D == 64) { if (sq) go(bwd_dq_tf32x3_kernel<8, true>); else go(bwd_dq_tf32x3_kernel<8, false>); }
      else { if (sq) go(bwd_dq_tf32x3_kernel<16, true>); else go(bwd_dq_tf32x3_kernel<16, false>); }
      if (rc) return join(rc);
      count_launch();
      if (int rc2 = check_launch("bwd_dq_tf32x3_kernel")) return join(rc2);
      dq_done = true;
    }
  }
  if (pr.S > 0 && !dq_done) {
    dim3 gq((pr.S + kWarps - 1) / kWarps, pr.bh_count);
    simt_bwd_dq_kernel<T><<<gq, kWarps * 32, smem, st>>>(pr, bias_dtype);
    count_launch();
    if (int rc = check_launch("simt_bwd_dq_kernel")) return join(rc);
  }
  if constexpr (sizeof(T) == 4) {
    // small problems: clusters of CTAs split the query tiles of each 64-key tile
    if (const int kc = bwd_dkv_cluster_size(pr)) {
      const size_t sm = sizeof(float) * (size_t(6 * 64) * (pr.D + 4) + 4 * kBN);
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(unsigned((pr.T + 63) / 64) * kc, pr.bh_count);
      cfg.blockDim = dim3(kTiledThreads);
      cfg.dynamicSmemBytes = sm;
      cfg.stream = st_kv;
      cudaLaunchAttribute attr{};
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = kc;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int rc = NB200_OK;
      auto go = [&](auto kernel) {
        if ((rc = prepare(kernel, sm)) != NB200_OK) return;
        (void)cudaLaunchKernelEx(&cfg, kernel, pr, bias_dtype);   // a failure is read by check_launch below
      };
      if (pr.D == 32) {
        if (kc == 4) go(bwd_dkv_tf32x3_kernel<4, 4>); else go(bwd_dkv_tf32x3_kernel<4, 2>);
      } else {
        if (kc == 4) go(bwd_dkv_tf32x3_kernel<8, 4>); else go(bwd_dkv_tf32x3_kernel<8, 2>);
      }
      if (rc) return join(rc);
      count_launch();
      return join(check_launch("bwd_dkv_tf32x3_kernel"));
    }
    if (pr.T > 0 && pr.D == pr.Dv && (pr.D == 32 || pr.D == 64 || pr.D == 128) &&
        int64_t((pr.T + 63) / 64) * pr.bh_count >= 96) {
      const size_t sm = sizeof(float) * (size_t(6 * 64) * (pr.D + 4) + 4 * kBN);
      dim3 gk((pr.T + 63) / 64, pr.bh_count);
      int rc = NB200_OK;
      if (pr.D == 32) {
        if ((rc = prepare(bwd_dkv_tf32x3_kernel<4>, sm)) == NB200_OK) bwd_dkv_tf32x3_kernel<4><<<gk, kTiledThreads, sm, st_kv>>>(pr, bias_dtype);
      } else if (pr.D == 64) {
        if ((rc = prepare(bwd_dkv_tf32x3_kernel<8>, sm)) == NB200_OK) bwd_dkv_tf32x3_kernel<8><<<gk, kTiledThreads, sm, st_kv>>>(pr, bias_dtype);
      } else {
        if ((rc = prepare(bwd_dkv_tf32x3_kernel<16>, sm)) == NB200_OK) bwd_dkv_tf32x3_kernel<16><<<gk, kTiledThreads, sm, st_kv>>>(pr, bias_dtype);
      }
      if (rc) return join(rc);
      count_launch();
      return join(check_launch("bwd_dkv_tf32x3_kernel"));
    }
  }
  if (pr.T > 0) {
    dim3 gk((pr.T + kWarps - 1) / kWarps, pr.bh_count);
    simt_bwd_dkv_kernel<T><<<gk, kWarps * 32, smem, st_kv>>>(pr, bias_dtype);
    count_launch();
    return join(check_launch("simt_bwd_dkv_kernel"));
  }
  return join(NB200_OK);
}

}  // namespace

bool simt_family_uses_tensor_path(const Problem& pr, int dtype, int pass) {
  // mirrors the selection in fwd_t / bwd_t above
  if (dtype != NB200_F32) return false;
  const bool dv_ok = pr.Dv == 32 || pr.Dv == 64 || pr.Dv == 128;
  if (pass == NB200_PASS_FWD) return pr.D % 8 == 0 && pr.D <= 128 && dv_ok;
  const bool d_ok = pr.D == 32 || pr.D == 64 || pr.D == 128;
  const bool dq = bwd_dq_cluster_size(pr) != 0 || bwd_dq_split_groups(pr) != 0 ||
                  (pr.S > 0 && pr.Dv % 8 == 0 && pr.Dv <= 128 && d_ok && int64_t((pr.S + 63) / 64) * pr.bh_count >= 96);
  const bool dkv = bwd_dkv_cluster_size(pr) != 0 ||
                   (pr.T > 0 && pr.D == pr.Dv && d_ok && int64_t((pr.T + 63) / 64) * pr.bh_count >= 96);
  return dq && dkv;
}

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
