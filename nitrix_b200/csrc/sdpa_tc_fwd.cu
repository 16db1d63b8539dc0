// Forward flash attention for sm_100a: TMA -> shared memory -> tcgen05.mma with
// TMEM accumulators, fp32 online softmax in registers.
//
// Replaces the reference's forward kernel `_fwd_kernel` and its launch glue
// (reference src/nitrix/_kernels/cuda/attention.py:85-156, :159-264): same
// recurrence (running max m, running sum l, lse = m + log2 l in base 2, causal
// key tiles past the diagonal skipped) on 128 x 128 tiles instead of 32 x 32.
//
// One CTA owns TWO 128-row query tiles of one (batch, head) and streams the key
// tiles once for both.  Twelve warps:
//   warp 0      TMA producer for Q (once) and the K / V rings
//   warp 1      TMA producer for the bias ring (128 x 64 slots)
//   warp 2      issues every tcgen05.mma (one elected lane)
//   warp 3      owns the TMEM allocation
//   warps 4-7   softmax of query tile 0 (one row per thread)
//   warps 8-11  softmax of query tile 1
// TMEM columns: [0,128) S0 / P0, [128,256) S1 / P1, [256,256+D) O0, then O1.
// P (16-bit) overwrites the first 64 columns of its S tile and feeds the PV
// MMA as the TMEM A operand; V is consumed from shared memory as an MN-major B
// operand, so nothing is transposed or staged through shared memory.
//
// Per key tile j and query tile g the dependency chain is
//   QK_g(j) -> softmax_g(j) -> PV_g(j) -> QK_g(j+1),
// and the two query tiles interleave so one's MMAs run under the other's
// softmax.  All waits are bounded (sdpa_tc_common.cuh).
#include "sdpa_tc_common.cuh"
#include "sdpa_tc_fwd.cuh"

namespace nb200 {
namespace tc {

using namespace sm100;

namespace {

constexpr int kThreads = 384;
constexpr int kStages = 2;  // K and V ring depth
// register split after start-up (setmaxnreg): 128 * kProducerRegs + 256 * kSoftmaxRegs <= 65536
constexpr int kProducerRegs = 56;
constexpr int kSoftmaxRegs = 216;

template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;        // one Q / K / V tile
  static constexpr int kBiasSlots = D == 64 ? 8 : 2;      // 16 KB slots
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kBias = kV + kStages * kTileBytes;
  static constexpr int kBars = kBias + kBiasSlots * kBoxBytes;
  // barriers: q_full[2] k_full[S] k_empty[S] v_full[S] v_empty[S] s_full[2] p_ready[2] o_done[2]
  //           bias_full[2][slots] (one set per query tile) bias_empty[slots]
  static constexpr int kNumBars = 2 + 4 * kStages + 6 + 3 * kBiasSlots;
  static constexpr int kMisc = kBars + 8 * kNumBars;      // tmem base (4 B) + abort flag (4 B)
  static constexpr int kTotal = kMisc + 16;
};

// Bias-ring sequence number of (key tile j, query tile g): slots are produced
// and consumed in the order  for j: for g (active at j): half 0, half 1.
__device__ __forceinline__ int bias_seq(int j, int g, int nt0, int nt1) {
  return 2 * (min(j, nt0) + min(j, nt1) + ((g == 1 && j < nt0) ? 1 : 0));
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_bias,
                   const FwdArgs a) {
  using L = FwdSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the 1024 the swizzle needs
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);

  auto bar = [&](int i) { return smem_u32(bars + i); };
  constexpr int Q_FULL = 0, K_FULL = 2, K_EMPTY = K_FULL + kStages, V_FULL = K_EMPTY + kStages,
                V_EMPTY = V_FULL + kStages, S_FULL = V_EMPTY + kStages, P_READY = S_FULL + 2, O_DONE = P_READY + 2,
                B_FULL = O_DONE + 2, B_EMPTY = B_FULL + 2 * L::kBiasSlots;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = a.bh_begin + blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  // heavier (later) causal blocks first
  const int qblock = a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int q0 = qblock * 2 * kTile;
  const int n_kt = (a.T + kTile - 1) / kTile;
  int nt[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int q0g = q0 + g * kTile;
    nt[g] = q0g >= a.S ? 0 : (a.causal ? min(n_kt, q0g / kTile + 1) : n_kt);
  }
  const int nt_max = max(nt[0], nt[1]);

  if (threadIdx.x == 0) {
    for (int i = 0; i < L::kNumBars; ++i) {
      uint32_t count = 1;
      if (i >= P_READY && i < P_READY + 2) count = 128;                     // every softmax thread
      if (i >= B_EMPTY && i < B_EMPTY + L::kBiasSlots) count = 4;           // one lane per softmax warp
      mbar_init(bar(i), count);
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 3) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tm_S[2] = {tmem, tmem + 128};
  const uint32_t tm_O[2] = {tmem + 256, tmem + 256 + D};

  // the softmax warpgroups hold a whole score row in registers; the producer / MMA warpgroup needs few
  if (warp < 4) {
  reg_dealloc<kProducerRegs>();
  if (warp == 0) {
    // ---------------- Q / K / V producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (nt[g] == 0) continue;
        mbar_expect_tx(bar(Q_FULL + g), L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sbase + L::kQ + g * L::kTileBytes + x * kBoxBytes, &tm_q, bar(Q_FULL + g), x * 64,
                      q0 + g * kTile, h, b);
      }
      for (int j = 0; j < nt_max; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!wait_or_abort(bar(K_EMPTY + st), ph ^ 1, abort_flag, a.status, 101)) break;
        mbar_expect_tx(bar(K_FULL + st), L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sbase + L::kK + st * L::kTileBytes + x * kBoxBytes, &tm_k, bar(K_FULL + st), x * 64,
                      j * kTile, h, b);
        if (!wait_or_abort(bar(V_EMPTY + st), ph ^ 1, abort_flag, a.status, 102)) break;
        mbar_expect_tx(bar(V_FULL + st), L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sbase + L::kV + st * L::kTileBytes + x * kBoxBytes, &tm_v, bar(V_FULL + st), x * 64,
                      j * kTile, h, b);
      }
    }
  } else if (warp == 1) {
    // ---------------- bias producer ----------------
    if (a.bias_mode == kBiasTile && elect_one()) {
      tma_prefetch_desc(&tm_bias);
      int seq = 0;
      bool ok = true;
      for (int j = 0; j < nt_max && ok; ++j) {
        for (int g = 0; g < 2 && ok; ++g) {
          if (j >= nt[g]) continue;
          for (int half = 0; half < 2; ++half, ++seq) {
            const int slot = seq % L::kBiasSlots;
            const uint32_t ph = (seq / L::kBiasSlots) & 1;
            if (!wait_or_abort(bar(B_EMPTY + slot), ph ^ 1, abort_flag, a.status, 103)) { ok = false; break; }
            // the slots are shared by both query tiles, but each tile has its own "full" barriers:
            // a waiter must see consecutive phases of a barrier, and the tiles alternate on a slot
            const uint32_t full = bar(B_FULL + g * L::kBiasSlots + slot);
            mbar_expect_tx(full, kBoxBytes);
            tma_load_4d(sbase + L::kBias + slot * kBoxBytes, &tm_bias, full,
                        j * kTile + half * kSlotCols, q0 + g * kTile, h * a.bias_h_mul, b * a.bias_b_mul);
          }
        }
      }
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc_qk = make_idesc(kBf16, kTile, kTile, false, false);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, kTile, D, false, true);
      bool ok = true;
      for (int g = 0; g < 2 && ok; ++g)
        if (nt[g] > 0) ok = wait_or_abort(bar(Q_FULL + g), 0, abort_flag, a.status, 104);
      for (int j = 0; j <= nt_max && ok; ++j) {
        const int st = j % kStages;
        const int stp = (j + kStages - 1) % kStages;  // stage of tile j - 1
        if (j < nt_max) ok = wait_or_abort(bar(K_FULL + st), (j / kStages) & 1, abort_flag, a.status, 105);
        if (ok && j > 0) ok = wait_or_abort(bar(V_FULL + stp), ((j - 1) / kStages) & 1, abort_flag, a.status, 106);
        if (!ok) break;
        tc_fence_after_sync();
        for (int g = 0; g < 2 && ok; ++g) {
          if (j > 0 && j - 1 < nt[g]) {
            // O_g += P_g(j-1) V(j-1)
            ok = wait_or_abort(bar(P_READY + g), (j - 1) & 1, abort_flag, a.status, 107);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t vbase = sbase + L::kV + stp * L::kTileBytes;
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk) {
              const uint64_t bdesc = make_smem_desc(vbase + kk * 2048, kBoxBytes, 1024);
              mma_ts(tm_O[g], tm_S[g] + kk * 8, bdesc, idesc_pv, (j - 1 > 0 || kk > 0) ? 1u : 0u);
            }
            if (j == nt[g]) mma_commit(bar(O_DONE + g));
          }
          if (j < nt[g]) {
            // S_g = Q_g K(j)^T
            const uint32_t qbase = sbase + L::kQ + g * L::kTileBytes;
            const uint32_t kbase = sbase + L::kK + st * L::kTileBytes;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
              mma_ss(tm_S[g], make_smem_desc(qbase + off, 16, 1024), make_smem_desc(kbase + off, 16, 1024),
                     idesc_qk, kk > 0 ? 1u : 0u);
            }
            mma_commit(bar(S_FULL + g));
          }
        }
        if (!ok) break;
        if (j < nt_max) mma_commit(bar(K_EMPTY + st));
        if (j > 0) mma_commit(bar(V_EMPTY + stp));
      }
    }
  }
  } else {
    reg_alloc<kSoftmaxRegs>();
    // ---------------- softmax (one query row per thread) ----------------
    const int g = (warp - 4) >> 2;
    const int wq = warp & 3;                    // TMEM lane quarter this warp may access
    const int r = wq * 32 + lane;               // row within the tile
    const int row = q0 + g * kTile + r;
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    const uint32_t tS = tm_S[g] + lane_addr, tO = tm_O[g] + lane_addr;
    const int my_nt = nt[g];
    float m = -INFINITY, l = 0.f;  // m: reference max in logit units (see the lazy rescale below)
    bool ok = true;
    // no bias and a non-negative scale: the scale is folded into the exponent's multiplier and the max runs on raw scores
    const bool fold_scale = a.bias_mode == kBiasNone && a.scale >= 0.f;
    const float mul = fold_scale ? a.scale * kLog2e : kLog2e;   // exponent = (t - m) * mul, base 2
    const float thr = mul > 0.f ? 8.f / mul : INFINITY;         // reference max lags the true max by at most 2^8
    const float2 scale2 = make_float2(a.scale, a.scale), mul2 = make_float2(mul, mul);
    uint32_t bias_phase = 0;  // bit s = parity this tile's next wait on its "full" barrier of slot s uses

    const uint32_t* mrow = nullptr;
    if (a.mask.rows) {
      mrow = a.mask.rows + b * a.mask.b_stride + h * a.mask.h_stride + int64_t(min(row, a.S - 1)) * a.mask.row_stride;
    }
    const uint8_t* bias_key = nullptr;
    if (a.bias_mode == kBiasKey)
      bias_key = reinterpret_cast<const uint8_t*>(a.bias) + 2 * (b * a.bias_bs + h * a.bias_hs);

    for (int j = 0; j < my_nt && ok; ++j) {
      const int key0 = j * kTile;
      // keep-bits of this row for this key tile
      uint32_t keep[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      bool need_mask = false;
      if (mrow) {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(mrow + j * 4));
        keep[0] = w.x; keep[1] = w.y; keep[2] = w.z; keep[3] = w.w;
        need_mask = true;
      }
      int n_keep = a.T - key0;
      if (a.causal) n_keep = min(n_keep, row - key0 + 1);
      if (n_keep < kTile) {
        limit_bits(keep, n_keep);
        need_mask = true;
      }
      need_mask = __any_sync(0xffffffffu, need_mask);

      ok = wait_or_abort(bar(S_FULL + g), j & 1, abort_flag, a.status, 108);
      if (!ok) break;
      tc_fence_after_sync();

      // the whole score row: four TMEM loads in flight, one wait; handled as 64 fp32 pairs
      float2 t[kTile / 2];
      {
        uint32_t raw[kTile];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[c * 32]));
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < kTile / 2; ++i) t[i] = make_float2(__uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1]));
      }
      // logits: t = s * scale + bias (natural units); without a bias the scale is folded into the exponent
      if (a.bias_mode == kBiasTile) {
        const int seq0 = bias_seq(j, g, nt[0], nt[1]);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int seq = seq0 + half;
          const int slot = seq % L::kBiasSlots;
          ok = wait_or_abort(bar(B_FULL + g * L::kBiasSlots + slot), (bias_phase >> slot) & 1u, abort_flag, a.status,
                             109);
          if (!ok) break;
          bias_phase ^= 1u << slot;
          const uint8_t* srow = smem + L::kBias + slot * kBoxBytes + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 w = *reinterpret_cast<const uint4*>(srow + ((c ^ (r & 7)) << 4));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              t[half * 32 + c * 4 + e] = __ffma2_rn(t[half * 32 + c * 4 + e], scale2, unpack2<kBf16>(ww[e]));
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_EMPTY + slot));
        }
        if (!ok) break;
      } else if (a.bias_mode == kBiasKey) {
        const uint4* bk = reinterpret_cast<const uint4*>(bias_key + 2 * key0);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const uint4 w = __ldg(bk + c);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) t[c * 4 + e] = __ffma2_rn(t[c * 4 + e], scale2, unpack2<kBf16>(ww[e]));
        }
      } else if (!fold_scale) {
#pragma unroll
        for (int i = 0; i < kTile / 2; ++i) t[i] = __fmul2_rn(t[i], scale2);
      }
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < kTile / 2; ++i) {
          if (!((keep[i >> 4] >> ((2 * i) & 31)) & 1u)) t[i].x = -INFINITY;
          if (!((keep[i >> 4] >> ((2 * i + 1) & 31)) & 1u)) t[i].y = -INFINITY;
        }
      }
      // row max: four independent chains of three-input max
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kTile / 2; ++i) mx4[i & 3] = max3(mx4[i & 3], t[i].x, t[i].y);
      const float mx = max3(mx4[0], mx4[1], fmaxf(mx4[2], mx4[3]));
      // the exponentials use a reference max that is only moved when the true max has run more than
      // 2^8 ahead of it (so p <= 256 and the running output is rescaled rarely); l uses the same reference
      const bool bump = mx > m + thr;
      const float m_use = bump ? mx : m;
      const float alpha = bump ? ex2((m - m_use) * mul) : 1.f;
      const float neg = m_use == -INFINITY ? 0.f : -m_use * mul;
      const float2 neg2 = make_float2(neg, neg);
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t pk[kTile / 2];
#pragma unroll
      for (int i = 0; i < kTile / 2; ++i) {
        const float2 x = __ffma2_rn(t[i], mul2, neg2);
        const float2 p = make_float2(ex2(x.x), ex2(x.y));
        sum2[i & 1] = __fadd2_rn(sum2[i & 1], p);
        pk[i] = pack2<kBf16>(p.x, p.y);
      }
      l = l * alpha + ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y));
      // rescale the running output when some row of this warp moved its reference max
      if (j > 0 && __any_sync(0xffffffffu, bump)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tO + c * 32, o);
        }
      }
      m = m_use;
      // P (16-bit pairs) over the first 64 columns of the S tile
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t chunk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) chunk[i] = pk[c * 32 + i];
        tmem_st32(tS + c * 32, chunk);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(P_READY + g));
    }

    // ---------------- epilogue: out = O / l, lse = m log2e + log2 l ----------------
    if (ok && my_nt > 0) ok = wait_or_abort(bar(O_DONE + g), 0, abort_flag, a.status, 110);
    if (ok && my_nt > 0) {
      tc_fence_after_sync();
      const float inv = 1.f / l;  // l == 0 (no kept key): 0 * inf = NaN, as the reference's softmax gives
      uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + 2 * (b * a.os[0] + h * a.os[1] + int64_t(row) * a.os[2]);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_wait_ld();
        if (row < a.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2<kBf16>(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = pack2<kBf16>(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = pack2<kBf16>(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = pack2<kBf16>(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + (c * 32 + i) * 2) = w;
          }
        }
      }
      if (row < a.S) a.lse[(int64_t(b) * a.H + h) * a.S + row] = m * mul + log2f(l);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) drain_after_abort();
  if (warp == 3) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

template <int D, bool kBf16>
int launch_one(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tb,
               const FwdArgs& a, int n_qblocks, int bh_count, cudaStream_t st) {
  auto kernel = sdpa_fwd_tc_kernel<D, kBf16>;
  const int smem = FwdSmem<D>::kTotal + 1024;  // slack for the 1024-byte round-up
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(sdpa_fwd_tc_kernel, %d): %s", smem, cudaGetErrorString(e));
    return NB200_ERR_LAUNCH;
  }
  dim3 grid(n_qblocks, bh_count);
  kernel<<<grid, kThreads, smem, st>>>(tq, tk, tv, tb, a);
  count_launch();
  return check_launch("sdpa_fwd_tc_kernel");
}

}  // namespace

int launch_fwd(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
               const CUtensorMap& tb, const FwdArgs& a, int n_qblocks, int bh_count, cudaStream_t st) {
  if (D == 64) return bf16 ? launch_one<64, true>(tq, tk, tv, tb, a, n_qblocks, bh_count, st)
                           : launch_one<64, false>(tq, tk, tv, tb, a, n_qblocks, bh_count, st);
  return bf16 ? launch_one<128, true>(tq, tk, tv, tb, a, n_qblocks, bh_count, st)
              : launch_one<128, false>(tq, tk, tv, tb, a, n_qblocks, bh_count, st);
}

}  // namespace tc
}  // namespace nb200
