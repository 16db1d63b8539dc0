// Mamba / S6 selective scan, forward and backward -- the second sibling op behind the same library (reference
// src/nitrix/nn/ssm/__init__.py:127- is the dispatcher, src/nitrix/nn/ssm/_reference.py:60-98 the recipe):
//
//   a_t = exp(delta_t A),  b_t = (delta_t B_t) x_t,  h_t = a_t h_{t-1} + b_t  (h_{-1} = 0),
//   y_t = sum_n C_{t,n} h_{t,n} (+ D x_t)
//
// per batch element, channel d and state n; x, delta (batch, l, d), A (d, n), B, C (batch, l, n), D (d); fp32
// recurrence and readout whatever the storage dtype (reference _reference.py:262-279).
//
// Four lanes own one channel of one batch element, a quarter of its n states each, and walk the sequence with them in
// registers (the recurrence is sequential in t; the parallelism is batch x channels x 4); a CTA is 64 channels, and
// the B_t / C_t rows its threads share are staged through shared memory eight steps at a time, double-buffered, with
// the next chunk's operands already in flight.  Nothing of size (l, d, n) is ever
// materialised: the forward leaves the state after every eighth step in a checkpoint array (batch, l / 8, n, d), and
// the backward walks the chunks in reverse, recomputes a chunk's eight states from its checkpoint into shared
// memory and runs the adjoint recurrence g_{t-1} = a_t g_t, g_t += C_t dy_t through them.  dB_t and dC_t are sums
// over channels: the threads' terms of a chunk go into a shared-memory tile whose columns the CTA adds once per chunk
// (up to 32 states; at 64 the warps reduce by shuffles), then one atomic per sum into fp32 accumulators; dA and dD
// are sums over batch and time: kept per thread and added once at the end.  A second kernel converts the
// accumulators to the storage dtype.
#include <math.h>

#include "nitrix_b200_scan.h"
#include "sdpa_common.cuh"

namespace nb200 {
namespace {

constexpr int kCh = 64;     // channels (threads) per CTA
constexpr int kStep = 8;    // steps per staged chunk = checkpoint interval

struct SsArgs {
  const void *x, *delta, *A, *B, *C, *D, *dy;
  void *y, *dx, *ddelta;
  float* ckpt;            // [batch][chunks][N][Dc]
  float *accB, *accC;     // [batch][L][N]
  float *accA, *accD;     // [Dc][N], [Dc]
  int batch, L, Dc, N, chunks;
};

// a_t = exp(delta_t A) as one multiply and one ex2.approx (relative error 2^-22): A is held pre-multiplied by log2(e)
__device__ __forceinline__ float ex2_ss(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kLog2eSs = 1.4426950408889634f;

// Forward.  Four adjacent lanes share a channel and hold a quarter of its states each (the readout is a sum over
// the four lanes: two shuffles per step): four times the warps of one-thread-per-channel for the same work, which is
// what the sequential recurrence lacks -- one warp per scheduler left the issue slots 20 % busy.  A CTA is 64 channels
// = 256 threads.
constexpr int kSplit = 4;
constexpr int kFwdThreads = kCh * kSplit;

template <typename T, int kN>
__global__ void __launch_bounds__(kFwdThreads) ss_fwd_kernel(SsArgs a) {
  constexpr int kQ = kN / kSplit;                            // states per thread
  constexpr int kRows = kStep * kN;                          // elements of a chunk's B (or C) block
  constexpr int kShare = (kRows + kFwdThreads - 1) / kFwdThreads;
  __shared__ float sB[2][kRows], sC[2][kRows];               // double-buffered: one barrier per chunk
  const int tid = threadIdx.x, part = tid & (kSplit - 1);
  const int d = blockIdx.x * kCh + (tid >> 2), b = blockIdx.y;
  const bool live = d < a.Dc;
  const T* xp = reinterpret_cast<const T*>(a.x) + int64_t(b) * a.L * a.Dc + d;
  const T* dp = reinterpret_cast<const T*>(a.delta) + int64_t(b) * a.L * a.Dc + d;
  T* yp = reinterpret_cast<T*>(a.y) + int64_t(b) * a.L * a.Dc + d;
  const T* Bp = reinterpret_cast<const T*>(a.B) + int64_t(b) * a.L * a.N;
  const T* Cp = reinterpret_cast<const T*>(a.C) + int64_t(b) * a.L * a.N;
  float Ar[kQ], h[kQ];
#pragma unroll
  for (int q = 0; q < kQ; ++q) {
    const int n = part * kQ + q;
    Ar[q] = (live && n < a.N) ? kLog2eSs * to_f32<T>(reinterpret_cast<const T*>(a.A)[int64_t(d) * a.N + n]) : 0.f;
    h[q] = 0.f;
  }
  const float Dd = (a.D && live) ? to_f32<T>(reinterpret_cast<const T*>(a.D)[d]) : 0.f;
  // the next chunk's operands: issued before the current chunk is computed
  float ndl[kStep], nxv[kStep], nbq[kShare], ncq[kShare];
  auto load = [&](int t0) {
#pragma unroll
    for (int s = 0; s < kStep; ++s) {
      const bool in = live && t0 + s < a.L;
      ndl[s] = in ? to_f32<T>(dp[int64_t(t0 + s) * a.Dc]) : 0.f;
      nxv[s] = in ? to_f32<T>(xp[int64_t(t0 + s) * a.Dc]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kShare; ++j) {
      const int i = tid + kFwdThreads * j, s = i / kN, n = i - s * kN;   // (compile-time divisor)
      const bool in = i < kRows && n < a.N && t0 + s < a.L;
      nbq[j] = in ? to_f32<T>(Bp[int64_t(t0 + s) * a.N + n]) : 0.f;
      ncq[j] = in ? to_f32<T>(Cp[int64_t(t0 + s) * a.N + n]) : 0.f;
    }
  };
  load(0);
  for (int c = 0; c < a.chunks; ++c) {
    const int t0 = c * kStep;
    float dls[kStep], xvs[kStep];
#pragma unroll
    for (int s = 0; s < kStep; ++s) {
      dls[s] = ndl[s];
      xvs[s] = nxv[s];
    }
    float* rb = sB[c & 1];
    float* rc = sC[c & 1];
#pragma unroll
    for (int j = 0; j < kShare; ++j) {
      const int i = tid + kFwdThreads * j;
      if (i < kRows) {
        rb[i] = nbq[j];
        rc[i] = ncq[j];
      }
    }
    __syncthreads();   // (the buffer written two chunks ago was last read before the previous barrier)
    if (c + 1 < a.chunks) load(t0 + kStep);
#pragma unroll
    for (int s = 0; s < kStep; ++s) {
      const int t = t0 + s;
      if (t < a.L) {   // (uniform over the CTA: the shuffles below are executed by whole warps)
        const float dl = dls[s], xv = xvs[s];
        float y = 0.f;
#pragma unroll
        for (int q = 0; q < kQ; ++q) {
          const int n = part * kQ + q;
          h[q] = fmaf(ex2_ss(dl * Ar[q]), h[q], (dl * rb[s * kN + n]) * xv);   // (rows past N are zero)
          y = fmaf(rc[s * kN + n], h[q], y);
        }
        y += __shfl_xor_sync(0xffffffffu, y, 1);
        y += __shfl_xor_sync(0xffffffffu, y, 2);
        if (a.D) y = fmaf(Dd, xv, y);
        if (live && part == 0) yp[int64_t(t) * a.Dc] = from_f32<T>(y);
      }
    }
    if (a.ckpt && live) {
      float* ck = a.ckpt + (int64_t(b) * a.chunks + c) * a.N * a.Dc + d;
#pragma unroll
      for (int q = 0; q < kQ; ++q) {
        const int n = part * kQ + q;
        if (n < a.N) ck[int64_t(n) * a.Dc] = h[q];
      }
    }
  }
}

// Backward: chunks in reverse, four lanes per channel as in the forward.  hs[0] = the state before the chunk
// (checkpoint c - 1, zero for the first chunk), hs[s + 1] = the state after step s of the chunk, recomputed; then the
// adjoint recurrence from the chunk's last step down.  A thread reads and writes only its own states in hs.
template <typename T, int kN>
__global__ void __launch_bounds__(kFwdThreads) ss_bwd_kernel(SsArgs a) {
  constexpr int kQ = kN / kSplit;                            // states per thread
  constexpr int kRows = kStep * kN;
  constexpr int kShare = (kRows + kFwdThreads - 1) / kFwdThreads;
  extern __shared__ float smem_ss[];
  float* hs = smem_ss;                                   // [kStep + 1][kN][kCh]
  float* sBb = hs + (kStep + 1) * kN * kCh;              // 2 x [kStep][kN]
  float* sCb = sBb + 2 * kRows;                          // 2 x [kStep][kN]
  // up to 32 states: the chunk's dB / dC terms as a tile [kStep][2][kN][kCh] (128 KB at 32 states); 64 states would
  // not fit beside the states and reduce over the warp's eight channels by shuffles instead
  constexpr bool kTile = kN <= 32;
  float* ct = sCb + 2 * kRows;
  const int tid = threadIdx.x, lane = tid & 31, part = tid & (kSplit - 1), ch = tid >> 2;
  const int d = blockIdx.x * kCh + ch, b = blockIdx.y;
  const bool live = d < a.Dc;
  const int64_t base = int64_t(b) * a.L * a.Dc + d;
  const T* xp = reinterpret_cast<const T*>(a.x) + base;
  const T* dp = reinterpret_cast<const T*>(a.delta) + base;
  const T* gp = reinterpret_cast<const T*>(a.dy) + base;
  T* dxp = reinterpret_cast<T*>(a.dx) + base;
  T* ddp = reinterpret_cast<T*>(a.ddelta) + base;
  const T* Bp = reinterpret_cast<const T*>(a.B) + int64_t(b) * a.L * a.N;
  const T* Cp = reinterpret_cast<const T*>(a.C) + int64_t(b) * a.L * a.N;
  float Ar[kQ], g[kQ], dA[kQ];
#pragma unroll
  for (int q = 0; q < kQ; ++q) {
    const int n = part * kQ + q;
    Ar[q] = (live && n < a.N) ? kLog2eSs * to_f32<T>(reinterpret_cast<const T*>(a.A)[int64_t(d) * a.N + n]) : 0.f;
    g[q] = dA[q] = 0.f;
  }
  const float Dd = (a.D && live) ? to_f32<T>(reinterpret_cast<const T*>(a.D)[d]) : 0.f;
  float dD = 0.f;
  // the next chunk's operands: issued before the current chunk is computed
  float ndl[kStep], nxv[kStep], ngy[kStep], nbq[kShare], ncq[kShare];
  auto load = [&](int t0) {
#pragma unroll
    for (int s = 0; s < kStep; ++s) {
      const bool in = live && t0 + s < a.L;
      ndl[s] = in ? to_f32<T>(dp[int64_t(t0 + s) * a.Dc]) : 0.f;
      nxv[s] = in ? to_f32<T>(xp[int64_t(t0 + s) * a.Dc]) : 0.f;
      ngy[s] = in ? to_f32<T>(gp[int64_t(t0 + s) * a.Dc]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kShare; ++j) {
      const int i = tid + kFwdThreads * j, s = i / kN, n = i - s * kN;   // (compile-time divisor)
      const bool in = i < kRows && n < a.N && t0 + s < a.L;
      nbq[j] = in ? to_f32<T>(Bp[int64_t(t0 + s) * a.N + n]) : 0.f;
      ncq[j] = in ? to_f32<T>(Cp[int64_t(t0 + s) * a.N + n]) : 0.f;
    }
  };
  if (a.chunks > 0) load((a.chunks - 1) * kStep);
  for (int c = a.chunks - 1; c >= 0; --c) {
    const int t0 = c * kStep;
    float dls[kStep], xvs[kStep], gys[kStep];
#pragma unroll
    for (int s = 0; s < kStep; ++s) {
      dls[s] = ndl[s];
      xvs[s] = nxv[s];
      gys[s] = ngy[s];
    }
    float* sB = sBb + (c & 1) * kRows;
    float* sC = sCb + (c & 1) * kRows;
#pragma unroll
    for (int j = 0; j < kShare; ++j) {
      const int i = tid + kFwdThreads * j;
      if (i < kRows) {
        sB[i] = nbq[j];
        sC[i] = ncq[j];
      }
    }
    __syncthreads();   // (the buffer written two chunks ago, and the tile, were last read before the previous barrier)
    if (c > 0) load(t0 - kStep);
    // ---- recompute the chunk's states ----
    {
      float h[kQ];
      const float* ck = c > 0 ? a.ckpt + (int64_t(b) * a.chunks + (c - 1)) * a.N * a.Dc + d : nullptr;
#pragma unroll
      for (int q = 0; q < kQ; ++q) {
        const int n = part * kQ + q;
        h[q] = (live && ck && n < a.N) ? ck[int64_t(n) * a.Dc] : 0.f;
        hs[(0 * kN + n) * kCh + ch] = h[q];
      }
#pragma unroll
      for (int s = 0; s < kStep; ++s) {
        const float dl = dls[s], xv = xvs[s];   // (zeros past the sequence's end: the state stays as it is)
#pragma unroll
        for (int q = 0; q < kQ; ++q) {
          const int n = part * kQ + q;
          h[q] = fmaf(ex2_ss(dl * Ar[q]), h[q], (dl * sB[s * kN + n]) * xv);
          hs[((s + 1) * kN + n) * kCh + ch] = h[q];
        }
      }
    }
    // ---- adjoint recurrence, last step of the chunk first ----
#pragma unroll
    for (int s = kStep - 1; s >= 0; --s) {
      const int t = t0 + s;
      if (t >= a.L) continue;   // (uniform over the CTA)
      const float dl = dls[s], xv = xvs[s], gy = gys[s];
      float ddl = 0.f, dxv = 0.f;
      if (part == 0) dD = fmaf(gy, xv, dD);
#pragma unroll
      for (int q = 0; q < kQ; ++q) {
        const int n = part * kQ + q;
        // a dead lane (past the last channel) and a state past N carry zeros throughout
        const float hprev = hs[(s * kN + n) * kCh + ch], hcur = hs[((s + 1) * kN + n) * kCh + ch];
        const float av = ex2_ss(dl * Ar[q]);
        const float bt = sB[s * kN + n];
        g[q] = fmaf(sC[s * kN + n], gy, g[q]);       // dL/dh_t
        const float da = g[q] * hprev * av;          // dL/d(delta_t A_n), natural units
        ddl = fmaf(da, Ar[q] * (1.f / kLog2eSs), ddl);
        dA[q] = fmaf(da, dl, dA[q]);
        ddl = fmaf(g[q] * bt, xv, ddl);
        dxv = fmaf(g[q] * dl, bt, dxv);
        // dB_t, dC_t: sums over the channels
        if constexpr (kTile) {
          // this thread's terms go into the chunk's tile; the CTA adds the columns once per chunk (below)
          ct[((s * 2 + 0) * kN + n) * kCh + ch] = g[q] * dl * xv;
          ct[((s * 2 + 1) * kN + n) * kCh + ch] = gy * hcur;
        } else {
          // the warp's eight channels by shuffles (lanes 4 apart hold the same states), then one atomic each
          float vb = g[q] * dl * xv, vc = gy * hcur;
#pragma unroll
          for (int o = 16; o >= kSplit; o >>= 1) {
            vb += __shfl_xor_sync(0xffffffffu, vb, o);
            vc += __shfl_xor_sync(0xffffffffu, vc, o);
          }
          if (lane < kSplit && n < a.N) {
            atomicAdd(a.accB + (int64_t(b) * a.L + t) * a.N + n, vb);
            atomicAdd(a.accC + (int64_t(b) * a.L + t) * a.N + n, vc);
          }
        }
        g[q] *= av;                                  // dL/dh_{t-1} so far
      }
      // dx_t, ddelta_t: sums over the channel's states, i.e. over the four lanes
      ddl += __shfl_xor_sync(0xffffffffu, ddl, 1);
      ddl += __shfl_xor_sync(0xffffffffu, ddl, 2);
      dxv += __shfl_xor_sync(0xffffffffu, dxv, 1);
      dxv += __shfl_xor_sync(0xffffffffu, dxv, 2);
      if (a.D) dxv = fmaf(Dd, gy, dxv);
      if (live && part == 0) {
        dxp[int64_t(t) * a.Dc] = from_f32<T>(dxv);
        ddp[int64_t(t) * a.Dc] = from_f32<T>(ddl);
      }
    }
    if constexpr (kTile) {
      // column sums of the chunk's tile: sum v = (step, B or C, n) over the 64 channels, read with a per-thread skew
      // so that the threads of a warp hit different banks; then one atomic per sum and CTA
      __syncthreads();
      for (int v = tid; v < kStep * 2 * kN; v += kFwdThreads) {
        const int sv = v / (2 * kN), rest = v - sv * 2 * kN, which = rest / kN, n = rest - which * kN;
        const int t = t0 + sv;
        if (n < a.N && t < a.L) {
          const float* col = ct + v * kCh;
          float acc = 0.f;
#pragma unroll 8
          for (int k = 0; k < kCh; ++k) acc += col[(k + tid) & (kCh - 1)];
          atomicAdd((which ? a.accC : a.accB) + (int64_t(b) * a.L + t) * a.N + n, acc);
        }
      }
      // (the tile is rewritten only after the next chunk's barrier)
    }
  }
  if (live) {
#pragma unroll
    for (int q = 0; q < kQ; ++q) {
      const int n = part * kQ + q;
      if (n < a.N) atomicAdd(a.accA + int64_t(d) * a.N + n, dA[q]);
    }
    if (a.accD && part == 0) atomicAdd(a.accD + d, dD);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ss_finish_kernel(const float* acc, T* out, int64_t n) {
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i < n) out[i] = from_f32<T>(acc[i]);
}

int pick_n(int N) { return N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : 0)); }

int check_common(const nb200_selective_scan_params* p, const char* what) {
  if (!p) { set_error("%s: NULL parameter block", what); return NB200_ERR_INVALID; }
  if (p->struct_size != sizeof(nb200_selective_scan_params)) {
    set_error("%s: ABI mismatch: struct_size %zu, library expects %zu", what, size_t(p->struct_size),
              sizeof(nb200_selective_scan_params));
    return NB200_ERR_INVALID;
  }
  if (p->dtype != NB200_F32 && p->dtype != NB200_BF16 && p->dtype != NB200_F16) { set_error("%s: bad dtype", what); return NB200_ERR_INVALID; }
  if (p->batch < 0 || p->length < 0 || p->channels <= 0 || p->states <= 0) { set_error("%s: bad extents", what); return NB200_ERR_INVALID; }
  if (!pick_n(p->states)) { set_error("%s: more than 64 states per channel (%d)", what, p->states); return NB200_ERR_UNSUPPORTED; }
  if (p->batch > 65535) { set_error("%s: more than 65535 batch elements", what); return NB200_ERR_UNSUPPORTED; }
  return NB200_OK;
}

SsArgs args_of(const nb200_selective_scan_params* p) {
  SsArgs a{};
  a.x = p->x; a.delta = p->delta; a.A = p->A; a.B = p->B; a.C = p->C; a.D = p->D; a.dy = p->dy;
  a.y = p->y; a.dx = p->dx; a.ddelta = p->ddelta; a.ckpt = p->checkpoints;
  a.batch = p->batch; a.L = p->length; a.Dc = p->channels; a.N = p->states;
  a.chunks = (p->length + kStep - 1) / kStep;
  return a;
}

template <typename T>
int fwd_t(const nb200_selective_scan_params* p, cudaStream_t st) {
  SsArgs a = args_of(p);
  dim3 grid((p->channels + kCh - 1) / kCh, p->batch);
  switch (pick_n(p->states)) {
    case 16: ss_fwd_kernel<T, 16><<<grid, kFwdThreads, 0, st>>>(a); break;
    case 32: ss_fwd_kernel<T, 32><<<grid, kFwdThreads, 0, st>>>(a); break;
    default: ss_fwd_kernel<T, 64><<<grid, kFwdThreads, 0, st>>>(a); break;
  }
  count_launch();
  return check_launch("selective_scan_fwd_kernel");
}

size_t acc_floats(const nb200_selective_scan_params* p) {
  return 2 * size_t(p->batch) * p->length * p->states + size_t(p->channels) * p->states + size_t(p->channels);
}

template <typename T, int kN>
int bwd_launch(const SsArgs& a, dim3 grid, cudaStream_t st) {
  const size_t smem = sizeof(float) * (size_t(kStep + 1) * kN * kCh + 4 * kStep * kN +
                                       (kN <= 32 ? size_t(kStep) * 2 * kN * kCh : 0));
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(ss_bwd_kernel<T, kN>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
    set_error("selective_scan_bwd: cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(cudaGetLastError()));
    return NB200_ERR_LAUNCH;
  }
  ss_bwd_kernel<T, kN><<<grid, kFwdThreads, smem, st>>>(a);
  count_launch();
  return check_launch("selective_scan_bwd_kernel");
}

template <typename T>
int bwd_t(const nb200_selective_scan_params* p, cudaStream_t st) {
  SsArgs a = args_of(p);
  const size_t need = sizeof(float) * acc_floats(p);
  if (!p->workspace || p->workspace_bytes < need) {
    set_error("selective_scan_bwd: workspace of %zu bytes needed (nb200_selective_scan_workspace_bytes), %zu given",
              need, size_t(p->workspace_bytes));
    return NB200_ERR_WORKSPACE;
  }
  float* acc = static_cast<float*>(p->workspace);
  if (cudaMemsetAsync(acc, 0, need, st) != cudaSuccess) return check_launch("selective_scan_bwd: clearing the workspace");
  const size_t bln = size_t(p->batch) * p->length * p->states, dn = size_t(p->channels) * p->states;
  a.accB = acc; a.accC = acc + bln; a.accA = acc + 2 * bln; a.accD = p->D ? acc + 2 * bln + dn : nullptr;
  if (p->batch > 0 && p->length > 0) {   // (nothing to walk otherwise: dA and dD are the zeros just written)
    dim3 grid((p->channels + kCh - 1) / kCh, p->batch);
    int rc;
    switch (pick_n(p->states)) {
      case 16: rc = bwd_launch<T, 16>(a, grid, st); break;
      case 32: rc = bwd_launch<T, 32>(a, grid, st); break;
      default: rc = bwd_launch<T, 64>(a, grid, st); break;
    }
    if (rc) return rc;
  }
  auto finish = [&](const float* src, void* dst, size_t n) {
    if (!dst || n == 0) return;
    ss_finish_kernel<T><<<unsigned((n + 255) / 256), 256, 0, st>>>(src, static_cast<T*>(dst), int64_t(n));
    count_launch();
  };
  finish(a.accB, p->dB, bln);
  finish(a.accC, p->dC, bln);
  finish(a.accA, p->dA, dn);
  if (p->D) finish(a.accD, p->dD, size_t(p->channels));
  return check_launch("selective_scan_finish_kernel");
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" NB200_API int nb200_selective_scan_workspace_bytes(const nb200_selective_scan_params* p, size_t* bytes) {
  if (!bytes) { set_error("bytes out-pointer is NULL"); return NB200_ERR_INVALID; }
  if (int rc = check_common(p, "selective_scan_workspace_bytes")) return rc;
  *bytes = sizeof(float) * acc_floats(p);
  return NB200_OK;
}

extern "C" NB200_API int nb200_selective_scan_checkpoint_bytes(const nb200_selective_scan_params* p, size_t* bytes) {
  if (!bytes) { set_error("bytes out-pointer is NULL"); return NB200_ERR_INVALID; }
  if (int rc = check_common(p, "selective_scan_checkpoint_bytes")) return rc;
  *bytes = sizeof(float) * size_t(p->batch) * ((p->length + kStep - 1) / kStep) * p->states * p->channels;
  return NB200_OK;
}

extern "C" NB200_API int nb200_selective_scan_fwd(const nb200_selective_scan_params* p, void* cuda_stream) {
  if (int rc = check_common(p, "selective_scan_fwd")) return rc;
  if (p->batch == 0 || p->length == 0) return NB200_OK;
  if (!p->x || !p->delta || !p->A || !p->B || !p->C || !p->y) { set_error("selective_scan_fwd: NULL operand"); return NB200_ERR_INVALID; }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  prof_call_begin(st);
  switch (p->dtype) {
    case NB200_F32: return fwd_t<float>(p, st);
    case NB200_BF16: return fwd_t<__nv_bfloat16>(p, st);
    default: return fwd_t<__half>(p, st);
  }
}

extern "C" NB200_API int nb200_selective_scan_bwd(const nb200_selective_scan_params* p, void* cuda_stream) {
  if (int rc = check_common(p, "selective_scan_bwd")) return rc;
  const bool empty = p->batch == 0 || p->length == 0;
  if (!p->dA || (p->D && !p->dD) ||
      (!empty && (!p->x || !p->delta || !p->A || !p->B || !p->C || !p->dy || !p->dx || !p->ddelta || !p->dB || !p->dC ||
                  (p->length > kStep && !p->checkpoints)))) {
    set_error("selective_scan_bwd: NULL operand (x, delta, A, B, C, dy, checkpoints and every gradient are required)");
    return NB200_ERR_INVALID;
  }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  prof_call_begin(st);
  switch (p->dtype) {
    case NB200_F32: return bwd_t<float>(p, st);
    case NB200_BF16: return bwd_t<__nv_bfloat16>(p, st);
    default: return bwd_t<__half>(p, st);
  }
}
