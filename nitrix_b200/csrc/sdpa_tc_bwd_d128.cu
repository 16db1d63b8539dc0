// Backward flash attention at head dim 128 in ONE kernel: dq, dk, dv and -- for a bias of full (B, H, S, T) extent --
// the dbias tiles, with S = Q K^T and dP = dO V^T computed once per tile pair.  (The two-kernel backward of
// sdpa_tc_bwd.cu computes both products twice at this head dim, because a dq tile does not fit beside the dk / dv
// accumulators in TMEM; the reference does the same in its `_bwd_kv_kernel` / `_bwd_q_kernel` pair, reference
// src/nitrix/_kernels/cuda/attention.py:272-387.)
//
// A CTA owns 128 keys of one (batch, head) and streams the queries in steps of 64 (key-major).  Per step:
//   P1 = K Q^T (+ bias^T / scale, - lse / (scale log2e)),  P2 = V dO^T (- delta)     SS MMAs, 128 x 64, fp32 in TMEM
//   p = exp2(P1 scale log2e), ds = p P2                                                 element-wise warps, one key each
//   p  -> TMEM (16-bit)                    dV += p^T dO                                 TS MMA
//   ds -> shared memory, TRANSPOSED: a [64 queries x 128 keys] tile with keys contiguous (128-byte swizzled rows,
//         two 64-key boxes).  That one tile is
//           the A operand (MN-major) of     dK   += ds^T Q          (128 x 128, K = 64)
//           the B operand (K-major) of      dQ^T  = K^T ds^T        (128 x 64,  K = 128; d on the TMEM lanes)
//           the source of a TMA store into dbias[b, h, queries, keys] (rows past S / keys past T are dropped).
//   dQ^T goes from TMEM to an fp32 accumulator in global memory by 16-byte reductions (`red.global.add.v4.f32`,
//   512 contiguous bytes per warp instruction); dq_finish_d128_kernel scales, casts and un-permutes it.
// TMEM (512 columns): dV 0-127, dK 128-255, P1 256-319, P2 320-383 (one stage: the products of step n + 1 are issued
// as soon as the warps of step n hold P in registers), p of stage s at 384 + 32 s, dQ^T at 448-511.
// Twelve warps: 0 TMA producer (K, V once; Q / dO / lse / delta ring), 1 bias tiles in and dbias tiles out (one
// polling thread), 2 MMA issuer, 3 per-query addends (-lse, -delta) as MMA operands + TMEM owner, 4-7 / 8-11 two
// element-wise groups taking alternate steps.  The group of step n also drains dQ^T of step n - 1.  All waits bounded.
#include <math.h>

#include "sdpa_tc_bwd.cuh"

namespace nb200 {
namespace tc {

using namespace sm100;

namespace {

constexpr int kThreads = 384;
constexpr int kStep = 64;                     // streamed queries per step
constexpr int kYBoxBytes = kStep * 128;       // one 64-row x 128-byte box
constexpr int kD = 128;
constexpr int kProducerRegs = 88;
constexpr int kWorkerRegs = 208;
constexpr int kLaunchRegs = 168;              // what __launch_bounds__(384, 1) gives
static_assert((kLaunchRegs - kProducerRegs) * 128 >= (kWorkerRegs - kLaunchRegs) * 256,
              "worker warps would wait forever for registers the producer warps never release");

#ifdef NB200_PROBE
// Development aid (not compiled into the library): cycles one element-wise warp spends in each phase of its steps.
__device__ long long g_probe[32];
#define PROBE_DECL long long pt_ = clock64(); const bool probe_ = blockIdx.x == 3 && blockIdx.y == 1 && warp == 4 && lane == 0
#define IPROBE_DECL long long ipt_ = clock64(); const bool iprobe_ = blockIdx.x == 3 && blockIdx.y == 1
#define IPROBE(i) do { const long long now_ = clock64(); if (iprobe_) g_probe[i] += now_ - ipt_; ipt_ = now_; } while (0)
#define PROBE(i) do { const long long now_ = clock64(); if (probe_) g_probe[i] += now_ - pt_; pt_ = now_; } while (0)
#else
#define PROBE_DECL
#define PROBE(i)
#define IPROBE_DECL
#define IPROBE(i)
#endif

template <bool kTileBias>
struct Smem {
  static constexpr int kXBytes = kTile * kD * 2;                // K or V tile
  static constexpr int kYBytes = kStep * kD * 2;                // Q or dO step
  // Q / dO ring: a stage is held from its products until its dV / dK, two steps later, and a refill takes about a
  // step to arrive; without bias tiles there is room for a fourth stage
  static constexpr int kYStages = kTileBias ? 3 : 4;
  static constexpr int kYStageBytes = 2 * kYBytes + 1024;       // Q, dO, then lse[64] + delta[64]
  static constexpr int kBiasSlots = kTileBias ? 2 : 0;          // [64 queries x 128 keys] = two 64 x 64 boxes, 16 KB
  // One ds^T tile: the writer of step n + 1 waits for the MMAs (and the dbias store) of step n, which are issued
  // half a step earlier.
  static constexpr int kDsBufs = 1;
  static constexpr int kX = 0;
  static constexpr int kY = kX + 2 * kXBytes;
  static constexpr int kBias = kY + kYStages * kYStageBytes;
  static constexpr int kDs = kBias + kBiasSlots * kBoxBytes;
  // hi * I16 and lo * I16: 16 x 16 K-major tiles without swizzle (512 bytes each), the B operand of the N = 16
  // MMAs that add a bias tile to the transposed scores 16 queries at a time
  static constexpr int kIdent = kDs + kDsBufs * kBoxBytes;
  static constexpr int kWeightBytes = (kTile / 8) * 256;
  static constexpr int kAugTileBytes = (kStep / 8) * 256;
  static constexpr int kAugSlotBytes = 2 * kAugTileBytes;      // lse tile, delta tile
  static constexpr int kWeights = kIdent + 1024;
  static constexpr int kAug = kWeights + kWeightBytes;          // two slots
  static constexpr int kBars = kAug + 2 * kAugSlotBytes;
  static constexpr int kNumBars = 1 + 2 * kYStages + 2 * 14 + 1;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static_assert(kY % 1024 == 0 && kBias % 1024 == 0 && kDs % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  static_assert(kTotal + 1024 <= 232448, "shared memory exceeds the per-CTA limit");
};

template <bool kBf16, bool kTileBias, bool kDbias>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_bwd_tc_d128_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                        const __grid_constant__ CUtensorMap tm_bias, const __grid_constant__ CUtensorMap tm_dbias,
                        const BwdArgs a) {
  using L = Smem<kTileBias>;
  constexpr int NY = L::kYStages, NDS = L::kDsBufs;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);
  auto bar = [&](int i) { return smem_u32(bars + i); };
  constexpr int X_FULL = 0, Y_FULL = 1, Y_EMPTY = Y_FULL + NY, PROD_FULL = Y_EMPTY + NY, P_FREE = PROD_FULL + 4,
                E_READY = P_FREE + 4, E_FREE = E_READY + 2, DS_FREE = E_FREE + 2, DQ_FULL = DS_FREE + 2,
                DQ_FREE = DQ_FULL + 2, B_FULL = DQ_FREE + 2, B_EMPTY = B_FULL + 2, AUG_FULL = B_EMPTY + 2,
                AUG_FREE = AUG_FULL + 2, ACC_DONE = AUG_FREE + 2, P_READY = ACC_DONE + 1;
  static_assert(P_READY + 2 == L::kNumBars, "barrier count");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = a.bh_begin + blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int o0 = blockIdx.x * kTile;              // first key of this CTA
  int s_begin = 0, s_end = (a.S + kStep - 1) / kStep;
  if (a.causal) s_begin = min(s_end, o0 / kStep);   // queries i >= first key
  // key-only mask (key padding): a tile whose keys are all past the last kept one contributes nothing
  const int kept = kept_key_length(a.mask, b, h, a.T);
  if (o0 >= kept) s_end = s_begin;
  const int n_steps = s_end - s_begin;
  // The CTAs of one (batch, head) run side by side and all add into the same dq accumulator; were they to walk the
  // queries in the same order they would hit the same lines with their reductions at the same moment.  Each key tile
  // therefore starts its walk at a different query step and wraps around.
  const int rot = n_steps > 0 ? int((blockIdx.x * 2u) % uint32_t(n_steps)) : 0;
  auto step_row = [&](int n) {   // first query row of the n-th step this CTA visits
    int j = n + rot;
    if (j >= n_steps) j -= n_steps;
    return (s_begin + j) * kStep;
  };
  constexpr bool store_dbias = kDbias;   // the ds tile doubles as the source of the dbias TMA stores

  if (threadIdx.x < L::kNumBars) {
    const int i = threadIdx.x;
    uint32_t count = 1;
    if (i >= P_FREE && i < P_FREE + 4) count = 4;      // one lane per warp of the group
    if (i >= E_READY && i < E_READY + 2) count = 4;
    if (i >= P_READY && i < P_READY + 2) count = 4;
    if (i >= DQ_FREE && i < DQ_FREE + 2) count = 4;
    if (i >= DS_FREE && i < DS_FREE + 2) count = store_dbias ? 2 : 1;   // the MMAs, and the dbias store
    mbar_init(bar(i), count);
    if (i == 0) *abort_flag = 0;
    mbar_init_fence();
  }
  __syncwarp();
  static_assert(L::kNumBars <= 64, "barrier initialisation assumes the first two warps cover all barriers");
  if (threadIdx.x < 64) asm volatile("bar.sync 1, 64;" ::: "memory");
  if (threadIdx.x == 0 && n_steps > 0) {
    // owner tiles, the first ring stages and the first bias slots: their latency runs under the rest of the start-up
    mbar_expect_tx(bar(X_FULL), 2 * L::kXBytes);
#pragma unroll
    for (int x = 0; x < kD / 64; ++x) {
      tma_load_4d(sbase + L::kX + x * kBoxBytes, &tm_k, bar(X_FULL), x * 64, o0, h, b);
      tma_load_4d(sbase + L::kX + L::kXBytes + x * kBoxBytes, &tm_v, bar(X_FULL), x * 64, o0, h, b);
    }
    const int n_first = n_steps < NY ? n_steps : NY;
    for (int n = 0; n < n_first; ++n) {
      const int r0 = step_row(n);
      const uint32_t ybase = sbase + L::kY + n * L::kYStageBytes;
      const uint32_t row_bytes = 4u * uint32_t(min(kStep, a.ld_rows - r0));
      mbar_expect_tx(bar(Y_FULL + n), 2 * L::kYBytes + 2 * row_bytes);
#pragma unroll
      for (int x = 0; x < kD / 64; ++x) {
        tma_load_4d(ybase + x * kYBoxBytes, &tm_q, bar(Y_FULL + n), x * 64, r0, h, b);
        tma_load_4d(ybase + L::kYBytes + x * kYBoxBytes, &tm_do, bar(Y_FULL + n), x * 64, r0, h, b);
      }
      const int64_t ro = (int64_t(b) * a.H + h) * a.ld_rows + r0;
      bulk_load(ybase + 2 * L::kYBytes, a.lse + ro, row_bytes, bar(Y_FULL + n));
      bulk_load(ybase + 2 * L::kYBytes + 256, a.delta + ro, row_bytes, bar(Y_FULL + n));
      if (kTileBias && n < 2) {
        mbar_expect_tx(bar(B_FULL + n), kBoxBytes);
        const uint32_t dst = sbase + L::kBias + n * kBoxBytes;
        tma_load_4d(dst, &tm_bias, bar(B_FULL + n), o0, r0, h * a.bias_h_mul, b * a.bias_b_mul);
        tma_load_4d(dst + kYBoxBytes, &tm_bias, bar(B_FULL + n), o0 + 64, r0, h * a.bias_h_mul, b * a.bias_b_mul);
      }
    }
  }
  {
    // weight rows (w0, w1, w2, 0, ...): a query's addend is sum_j w_j c_j with c_j 16-bit; bf16 has fp32's range, so
    // three unit weights give 24 bits; fp16 spreads the terms over 2^8, 1, 2^-8
    uint4* wt = reinterpret_cast<uint4*>(smem + L::kWeights);
    const uint32_t w01 = kBf16 ? 0x3F803F80u : 0x3C005C00u;
    const uint32_t w2 = kBf16 ? 0x00003F80u : 0x00001C00u;
    for (int idx = threadIdx.x; idx < L::kWeightBytes / 16; idx += kThreads)
      wt[idx] = (idx & 8) ? make_uint4(0, 0, 0, 0) : make_uint4(w01, w2, 0, 0);
    uint4* aug = reinterpret_cast<uint4*>(smem + L::kAug);
    for (int idx = threadIdx.x; idx < 2 * L::kAugSlotBytes / 16; idx += kThreads) aug[idx] = make_uint4(0, 0, 0, 0);
    if (kTileBias) {
      // two 16 x 16 tiles, hi * I and lo * I with hi + lo = 1 / scale: K-major without swizzle, 8-row groups of 256
      // bytes = [8 rows x 16 bytes (K 0-7)][8 rows x 16 bytes (K 8-15)]; one 16-byte chunk per thread
      if (threadIdx.x < 64) {
        const int tile = threadIdx.x >> 5, c = threadIdx.x & 31;   // chunk c: group g, K half kh, row r8
        const int g = c >> 4, kh = (c >> 3) & 1, r8 = c & 7;
        const int row = g * 8 + r8;                                  // n index; the chunk holds k = kh * 8 .. + 7
        const float val = tile == 0 ? a.inv_scale_hi : a.inv_scale_lo;
        const uint16_t one = kBf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        const int k = row - kh * 8;
        if (k >= 0 && k < 8) w[k >> 1] = uint32_t(one) << ((k & 1) * 16);
        reinterpret_cast<uint4*>(smem + L::kIdent + tile * 512)[c] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    fence_proxy_async_smem();   // written by threads, read by the tensor core
  }
  if (warp == 3) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tm_dv = tmem, tm_dk = tmem + 128, tm_p1 = tmem + 256, tm_p2 = tmem + 320, tm_e = tmem + 384,
                 tm_dq = tmem + 448;

  if (warp < 4) {
  reg_dealloc<kProducerRegs>();
  if (warp == 1) {
    // ---------------- every TMA duty of the step loop: ONE thread probes the three barriers ----------------
    // Q / dO ring refills, bias tiles in, dbias tiles out.  (Blocking loops in several lanes of a warp would depend on
    // how divergent lanes are scheduled; one thread that waits on each barrier in turn, suspended in hardware for at
    // most a short time hint, does not, and it serves whichever duty completes first.)
    if (lane == 0 && n_steps > 0) {
      int yn = min(n_steps, NY);                         // next ring stage to refill (the first NY went out at start-up)
      int bn = kTileBias ? min(n_steps, 2) : n_steps;    // next bias tile to fetch (the first two went out at start-up)
      int sn = store_dbias ? 0 : n_steps;                // next dbias tile to store
      const long long t0 = clock64();
      uint32_t idle = 0;
      while (yn < n_steps || bn < n_steps || sn < n_steps) {
        const int pending = (yn < n_steps) + (bn < n_steps) + (sn < n_steps);
        const uint32_t hint = pending > 1 ? 64u : 4096u;
        bool progressed = false;
        if (yn < n_steps && mbar_try_wait_hint(bar(Y_EMPTY + yn % NY), ((yn / NY) & 1) ^ 1, hint)) {
          const int st = yn % NY, r0 = step_row(yn);
          const uint32_t ybase = sbase + L::kY + st * L::kYStageBytes;
          // lse / delta rows of the step that exist (a multiple of 4 rows, so the copy stays a multiple of 16 bytes)
          const uint32_t row_bytes = 4u * uint32_t(min(kStep, a.ld_rows - r0));
          mbar_expect_tx(bar(Y_FULL + st), 2 * L::kYBytes + 2 * row_bytes);
#pragma unroll
          for (int x = 0; x < kD / 64; ++x) {
            tma_load_4d(ybase + x * kYBoxBytes, &tm_q, bar(Y_FULL + st), x * 64, r0, h, b);
            tma_load_4d(ybase + L::kYBytes + x * kYBoxBytes, &tm_do, bar(Y_FULL + st), x * 64, r0, h, b);
          }
          const int64_t ro = (int64_t(b) * a.H + h) * a.ld_rows + r0;
          bulk_load(ybase + 2 * L::kYBytes, a.lse + ro, row_bytes, bar(Y_FULL + st));
          bulk_load(ybase + 2 * L::kYBytes + 256, a.delta + ro, row_bytes, bar(Y_FULL + st));
          ++yn;
          progressed = true;
        }
        if (bn < n_steps && mbar_try_wait_hint(bar(B_EMPTY + (bn & 1)), ((bn >> 1) & 1) ^ 1, hint)) {
          const int slot = bn & 1, r0 = step_row(bn);
          mbar_expect_tx(bar(B_FULL + slot), kBoxBytes);
          const uint32_t dst = sbase + L::kBias + slot * kBoxBytes;
          tma_load_4d(dst, &tm_bias, bar(B_FULL + slot), o0, r0, h * a.bias_h_mul, b * a.bias_b_mul);
          tma_load_4d(dst + kYBoxBytes, &tm_bias, bar(B_FULL + slot), o0 + 64, r0, h * a.bias_h_mul, b * a.bias_b_mul);
          ++bn;
          progressed = true;
        }
        if (sn < n_steps && mbar_try_wait_hint(bar(E_READY + (sn & 1)), (sn >> 1) & 1, hint)) {
          // the group's writes were fenced towards the async proxy before it arrived on E_READY
          const uint32_t src = sbase + L::kDs + (sn % NDS) * kBoxBytes;
          const int r0 = step_row(sn);
          tma_store_4d(&tm_dbias, src, o0, r0, h, b);
          if (o0 + 64 < a.T) tma_store_4d(&tm_dbias, src + kYBoxBytes, o0 + 64, r0, h, b);
          bulk_commit_group();
          bulk_wait_group_read0();                 // the tile has been read: its buffer may be rewritten
          mbar_arrive(bar(DS_FREE + (sn & 1)));
          ++sn;
          progressed = true;
        }
        if (!progressed && (++idle & 0x3F) == 0) {
          if (*abort_flag) break;
          if (*reinterpret_cast<volatile int*>(a.status) != 0) { *abort_flag = 1; break; }
          if (clock64() - t0 > 20 * kWaitCycles) {   // the whole CTA's life is bounded as well
            *abort_flag = 1;
            atomicExch(a.status, 302);
            break;
          }
        }
      }
      if (store_dbias) bulk_wait_group0();         // every dbias tile has reached global memory
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer 1: the products of every step ----------------
    // Two threads issue MMAs, this one the products and warp 0 the accumulating ones.  A single issuing thread
    // needs ~2000 cycles of instruction issue per step for the 40-odd MMAs, as much as the element-wise warps need
    // for their step, and in one instruction stream the products of step n + 2 queue behind the accumulating MMAs of
    // step n, which wait for the element-wise warps -- the very warps that then wait for those products.
    if (elect_one() && n_steps > 0) {
      constexpr uint32_t idesc_prod = make_idesc(kBf16, kTile, kStep, false, false);
      constexpr uint32_t idesc_bias = make_idesc(kBf16, kTile, 16, true, false);    // bias^T (MN-major) x 16 x 16 identity
      bool ok = wait_or_abort(bar(X_FULL), 0, abort_flag, a.status, 303);
      const uint64_t kdesc = make_smem_desc(sbase + L::kX, 16, 1024);
      const uint64_t vdesc = make_smem_desc(sbase + L::kX + L::kXBytes, 16, 1024);
      const uint64_t wdesc = make_smem_desc_noswizzle(sbase + L::kWeights, 128, 256);
      IPROBE_DECL;
      for (int n = 0; n < n_steps && ok; ++n) {
        const int st = n % NY, s = n & 1;
        IPROBE(16);
        ok = wait_or_abort(bar(Y_FULL + st), (n / NY) & 1, abort_flag, a.status, 304);
        IPROBE(17);
        // One stage per product, each with its own pair of barriers (PROD_FULL / P_FREE + 0, 1: scores; + 2, 3: dP):
        // a product may be overwritten once the warps of step n - 1 hold it in registers, and the warps take the
        // scores of step n -- and start on their exponentials -- while the tensor core still computes its dP.
        if (ok && n >= 1) ok = wait_or_abort(bar(P_FREE + ((n - 1) & 1)), ((n - 1) >> 1) & 1, abort_flag, a.status, 309);
        IPROBE(18);
        if (ok) ok = wait_or_abort(bar(AUG_FULL + s), (n >> 1) & 1, abort_flag, a.status, 312);
        IPROBE(19);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t ybase = sbase + L::kY + st * L::kYStageBytes;
        const uint64_t qdesc = make_smem_desc(ybase, 16, 1024), gdesc = make_smem_desc(ybase + L::kYBytes, 16, 1024);
        const uint32_t aslot = sbase + L::kAug + s * L::kAugSlotBytes;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint64_t xo = uint64_t(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
          const uint64_t yo = uint64_t(((kk / 4) * kYBoxBytes + (kk % 4) * 32) >> 4);
          mma_ss(tm_p1, kdesc + xo, qdesc + yo, idesc_prod, kk > 0 ? 1u : 0u);
        }
        // P1 += W C1^T (C1: -lse / (scale log2e))
        mma_ss(tm_p1, wdesc, make_smem_desc_noswizzle(aslot, 128, 256), idesc_prod, 1u);
        if constexpr (kTileBias) {
          // P1[key, q] += bias^T[key, q'] (hi I + lo I)[q', q], 16 queries at a time: A = 16 rows of the slot read
          // MN-major (two 64-key boxes), B = the 16 x 16 scaled identity, D = 16 columns of P1
          IPROBE(16);
          ok = wait_or_abort(bar(B_FULL + s), (n >> 1) & 1, abort_flag, a.status, 311);
          IPROBE(20);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(sbase + L::kBias + s * kBoxBytes, kYBoxBytes, 1024);
          const int n_ident = a.inv_scale_lo != 0.f ? 2 : 1;
          for (int tile = 0; tile < n_ident; ++tile) {
            const uint64_t bdesc = make_smem_desc_noswizzle(sbase + L::kIdent + tile * 512, 128, 256);
#pragma unroll
            for (int kk = 0; kk < kStep / 16; ++kk)
              mma_ss(tm_p1 + kk * 16, adesc + uint64_t((kk * 2048) >> 4), bdesc, idesc_bias, 1u);
          }
          mma_commit(bar(B_EMPTY + s));
        }
        mma_commit(bar(PROD_FULL + s));
        IPROBE(16);
        if (n >= 1) ok = wait_or_abort(bar(P_FREE + 2 + ((n - 1) & 1)), ((n - 1) >> 1) & 1, abort_flag, a.status, 319);
        IPROBE(23);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint64_t xo = uint64_t(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
          const uint64_t yo = uint64_t(((kk / 4) * kYBoxBytes + (kk % 4) * 32) >> 4);
          mma_ss(tm_p2, vdesc + xo, gdesc + yo, idesc_prod, kk > 0 ? 1u : 0u);
        }
        // P2 += W C2^T (C2: -delta)
        mma_ss(tm_p2, wdesc, make_smem_desc_noswizzle(aslot + L::kAugTileBytes, 128, 256), idesc_prod, 1u);
        mma_commit(bar(AUG_FREE + s));
        mma_commit(bar(PROD_FULL + 2 + s));
      }
    }
  } else if (warp == 0) {
    // ---------------- MMA issuer 2: dV, dK and dQ^T of every step ----------------
    if (elect_one() && n_steps > 0) {
      constexpr uint32_t idesc_acc = make_idesc(kBf16, kTile, kD, false, true);     // dV: A from TMEM, B = dO MN-major
      constexpr uint32_t idesc_dk = make_idesc(kBf16, kTile, kD, kDbias, true);     // dK: A = ds (MN-major when [query x key]), B = Q MN-major
      constexpr uint32_t idesc_dq = make_idesc(kBf16, kTile, kStep, true, !kDbias); // dQ^T: A = K MN-major, B = ds (K-major when [query x key])
      bool ok = wait_or_abort(bar(X_FULL), 0, abort_flag, a.status, 303);
      const uint64_t kmn = make_smem_desc(sbase + L::kX, kBoxBytes, 1024);          // K as [d x key], d contiguous
      for (int m = 0; m < n_steps && ok; ++m) {
        const int st = m % NY, s = m & 1;
        const uint32_t ybase = sbase + L::kY + st * L::kYStageBytes;
        const uint64_t qmn = make_smem_desc(ybase, kYBoxBytes, 1024);                    // Q as [query x d], d contiguous
        const uint64_t gmn = make_smem_desc(ybase + L::kYBytes, kYBoxBytes, 1024);      // dO likewise
        const uint32_t dsbuf = sbase + L::kDs + (m % NDS) * kBoxBytes;
        // ds as the A operand of dK (M = key, K = query): [query x key] is MN-major, 16 queries = 16 rows of a box;
        // [key x query] is K-major, 16 queries = 32 bytes of a row
        const uint64_t ds_a = kDbias ? make_smem_desc(dsbuf, kYBoxBytes, 1024) : make_smem_desc(dsbuf, 16, 1024);
        constexpr int ds_a_step = kDbias ? 2048 : 32;
        const uint32_t e1 = tm_e + s * 32;
        // dV += p^T dO (p from TMEM) as soon as p is there: it runs while the warps still form ds
        ok = wait_or_abort(bar(P_READY + s), (m >> 1) & 1, abort_flag, a.status, 319);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kStep / 16; ++kk)
          mma_ts(tm_dv, e1 + kk * 8, gmn + uint64_t((kk * 2048) >> 4), idesc_acc, (m > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar(E_FREE + s));             // p of this stage may be rewritten
        // dK += ds^T Q once the ds tile is in shared memory
        ok = wait_or_abort(bar(E_READY + s), (m >> 1) & 1, abort_flag, a.status, 305);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kStep / 16; ++kk)
          mma_ss(tm_dk, ds_a + uint64_t((kk * ds_a_step) >> 4), qmn + uint64_t((kk * 2048) >> 4), idesc_dk,
                 (m > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar(Y_EMPTY + st));           // the last readers of this Q / dO stage
        // dQ^T[d, query] = sum_key K[key, d] ds[key, query]; the previous tile must have been drained
        if (m >= 1) {
          ok = wait_or_abort(bar(DQ_FREE + ((m - 1) & 1)), ((m - 1) >> 1) & 1, abort_flag, a.status, 315);
          if (!ok) break;
          tc_fence_after_sync();
        }
        // ds as the B operand of dQ^T (N = query, K = key): [query x key] is K-major, 16 keys = 32 bytes of a query
        // row (second box from key 64 on); [key x query] is MN-major, 16 keys = 16 rows
        const uint64_t ds_b = kDbias ? make_smem_desc(dsbuf, 16, 1024) : make_smem_desc(dsbuf, kBoxBytes, 1024);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          const uint64_t bo = kDbias ? uint64_t(((kk / 4) * kYBoxBytes + (kk % 4) * 32) >> 4) : uint64_t((kk * 2048) >> 4);
          mma_ss(tm_dq, kmn + uint64_t((kk * 2048) >> 4), ds_b + bo, idesc_dq, kk > 0 ? 1u : 0u);
        }
        mma_commit(bar(DQ_FULL + (m & 1)));
        mma_commit(bar(DS_FREE + (m & 1)));      // the ds^T tile has been read by dK and dQ^T
        if (m == n_steps - 1) mma_commit(bar(ACC_DONE));
      }
    }
  } else {
    // ---------------- warp 3: per-query addends as MMA operands ----------------
    const float inv_mul = 1.f / (a.scale * kLog2e);
    bool ok = true;
    for (int n = 0; n < n_steps && ok; ++n) {
      const int st = n % NY, s = n & 1;
      ok = wait_or_abort(bar(Y_FULL + st), (n / NY) & 1, abort_flag, a.status, 313);
      if (ok && n >= 2) ok = wait_or_abort(bar(AUG_FREE + s), ((n - 2) >> 1) & 1, abort_flag, a.status, 314);
      if (!ok) break;
      const float* ld = reinterpret_cast<const float*>(smem + L::kY + st * L::kYStageBytes + 2 * L::kYBytes);
      uint8_t* slot = smem + L::kAug + s * L::kAugSlotBytes;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int q = lane + 32 * e;
        const bool live = step_row(n) + q < a.S;   // rows past S were not copied; the addend must be finite
        const float c[2] = {live ? -ld[q] * inv_mul : 0.f, live ? -ld[kStep + q] : 0.f};
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
          float rem = c[tile];
          uint32_t hh[3];
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            const float w = kBf16 ? 1.f : (j == 0 ? 256.f : (j == 1 ? 1.f : 0.00390625f));
            const float v = rem * (1.f / w);
            float back;
            if constexpr (kBf16) {
              const __nv_bfloat16 hv = __float2bfloat16_rn(v);
              hh[j] = __bfloat16_as_ushort(hv);
              back = __bfloat162float(hv);
            } else {
              const __half hv = __float2half_rn(v);
              hh[j] = __half_as_ushort(hv);
              back = __half2float(hv);
            }
            rem = fmaf(-back, w, rem);
          }
          *reinterpret_cast<uint4*>(slot + tile * L::kAugTileBytes + (q >> 3) * 256 + (q & 7) * 16) =
              make_uint4(hh[0] | (hh[1] << 16), hh[2], 0u, 0u);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(AUG_FULL + s));
    }
  }
  } else {
    reg_alloc<kWorkerRegs>();
    // ---------------- element-wise groups (one key per thread) ----------------
    const int grp = (warp - 4) >> 2;
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int key = o0 + r;
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    bool ok = true;
    // a tiled bias was added (divided by the scale) by the tensor core: the scale folds into the exponent's multiplier
    const bool fold_scale = a.bias_mode != kBiasKey;
    const float mul = fold_scale ? a.scale * kLog2e : kLog2e;
    const float2 mul2 = make_float2(mul, mul), scale2 = make_float2(a.scale, a.scale);
    const uint32_t* mbits = nullptr;
    bool key_dropped = false;
    if (a.mask.rows) {
      if (a.mask_key_only) {
        const uint32_t* krow = a.mask.rows + b * a.mask.b_stride + h * a.mask.h_stride;
        key_dropped = key >= a.T || !((krow[key >> 5] >> (key & 31)) & 1u);
      } else {
        mbits = a.mask.cols + b * a.mask.tb_stride + h * a.mask.th_stride + int64_t(min(key, a.T - 1)) * a.mask.tkey_stride;
      }
    }
    float bias_own = 0.f;   // per-key bias: one value for this thread's key
    if (a.bias_mode == kBiasKey && key < a.T) {
      const uint16_t raw = reinterpret_cast<const uint16_t*>(a.bias)[b * a.bias_bs + h * a.bias_hs + key];
      bias_own = kBf16 ? __uint_as_float(uint32_t(raw) << 16) : __half2float(__ushort_as_half(raw));
    }
    // The ds tile (16 KB, 128-byte swizzle) feeds dK += ds^T Q and dQ^T = K^T ds^T; either orientation serves both
    // MMAs (operand majors are free), so the layout follows the third use:
    //  * with a dbias to store it is [64 queries x 128 keys] (two boxes of 64 keys), exactly a dbias tile, which leaves
    //    by TMA; a thread (one key) then writes 64 separate 16-bit elements: element (query c, key r) lives in box
    //    r / 64, row c, 16-byte chunk ((r % 64) / 8) ^ (c % 8)
    //  * without, it is [128 keys x 64 queries]: a thread writes its own 128-byte row as eight 16-byte chunks,
    //    chunk i at position i ^ (r % 8)
    // (the tile base is 1024-byte aligned and the other terms leave bits 4-6 clear, so the swizzle is one XOR)
    const uint32_t ds_thread = kDbias ? uint32_t(r >> 6) * kYBoxBytes + uint32_t(r & 7) * 2 + (uint32_t((r & 63) >> 3) << 4)
                                      : uint32_t(r) * 128 + (uint32_t(r & 7) << 4);
    // dq accumulator of this (batch, head): [query / 4][d][query % 4] floats, so that one warp-wide reduction of
    // four queries covers 512 contiguous bytes (lanes = 32 consecutive d)

    PROBE_DECL;
    auto drain = [&](int j) -> bool {
      PROBE(0);
      if (!wait_or_abort(bar(DQ_FULL + (j & 1)), (j >> 1) & 1, abort_flag, a.status, 316)) return false;
      PROBE(10);
      tc_fence_after_sync();
      uint32_t v[kStep];
      tmem_ld32(tm_dq + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld32(tm_dq + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_FREE + (j & 1)));
      PROBE(11);
      float* dst = a.dq_acc + int64_t(blockIdx.y) * a.acc_rows * kD + r * 4 + int64_t(step_row(j) / 4) * (kD * 4);
#pragma unroll
      for (int c = 0; c < kStep / 4; ++c) red_add_v4(dst + c * (kD * 4), v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      PROBE(12);
      return true;
    };

    uint2 mnext = make_uint2(0xffffffffu, 0xffffffffu);
    if (mbits && grp < n_steps) mnext = __ldg(reinterpret_cast<const uint2*>(mbits + (step_row(grp) >> 5)));
    for (int n = grp; n < n_steps && ok; n += 2) {
      const int s = n & 1;
      const int r0 = step_row(n);
      // keep bits over the step's 64 queries: query r0 + c needs c < S - r0 and (causal) r0 + c >= key
      // (the mask words of this step were fetched a step of this group ago; the next fetch runs under this step)
      uint32_t keep[2] = {mnext.x, mnext.y};
      if (mbits && n + 2 < n_steps) mnext = __ldg(reinterpret_cast<const uint2*>(mbits + (step_row(n + 2) >> 5)));
      {
        const int hi = a.S - r0;
        const int lo = a.causal ? key - r0 : 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int nh = hi - 32 * i, nl = lo - 32 * i;
          const uint32_t mh = nh >= 32 ? 0xffffffffu : (nh <= 0 ? 0u : ((1u << nh) - 1u));
          const uint32_t ml = nl <= 0 ? 0xffffffffu : (nl >= 32 ? 0u : ~((1u << nl) - 1u));
          keep[i] &= mh & ml;
        }
        if (key_dropped) keep[0] = keep[1] = 0u;
      }

      PROBE(1);
      ok = wait_or_abort(bar(PROD_FULL + s), (n >> 1) & 1, abort_flag, a.status, 306);
      if (!ok) break;
      PROBE(2);
      tc_fence_after_sync();
      // the scores first: p = exp2(t log2e) (they arrive with -lse already added) while dP is still being computed
      float2 t[kStep / 2];
      {
        uint32_t raw[kStep];
        tmem_ld32(tm_p1 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
        tmem_ld32(tm_p1 + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
        tmem_wait_ld();
        // the scores are in registers: the MMA issuer may compute the next step's
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_FREE + s));
        PROBE(3);
#pragma unroll
        for (int i = 0; i < kStep / 2; ++i) t[i] = make_float2(__uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1]));
      }
      if (!fold_scale) {
        const float2 own2 = make_float2(bias_own, bias_own);
#pragma unroll
        for (int c = 0; c < kStep / 2; ++c) t[c] = __ffma2_rn(t[c], scale2, own2);
      }
      uint32_t e1[kStep / 2], e2[kStep / 2];
      const bool need_mask = __any_sync(0xffffffffu, (keep[0] & keep[1]) != 0xffffffffu);
#pragma unroll
      for (int c = 0; c < kStep / 2; ++c) {
        float2 x = __fmul2_rn(t[c], mul2);
        if (need_mask) {
          if (!((keep[c >> 4] >> ((2 * c) & 31)) & 1u)) x.x = -INFINITY;
          if (!((keep[c >> 4] >> ((2 * c + 1) & 31)) & 1u)) x.y = -INFINITY;
        }
        t[c] = make_float2(ex2(x.x), ex2(x.y));
        e1[c] = pack2<kBf16>(t[c].x, t[c].y);
      }
      PROBE(4);
      // p of this stage is still being read by dV of step n - 2
      if (n >= 2) {
        ok = wait_or_abort(bar(E_FREE + s), ((n - 2) >> 1) & 1, abort_flag, a.status, 310);
        if (!ok) break;
        tc_fence_after_sync();
      }
      PROBE(5);
      tmem_st32(tm_e + s * 32 + lane_addr, e1);
      // ds = p dP (dP arrives with -delta already added)
      ok = wait_or_abort(bar(PROD_FULL + 2 + s), (n >> 1) & 1, abort_flag, a.status, 318);
      if (!ok) break;
      PROBE(9);
      // p is in TMEM by now (its store was issued before the wait): dV += p^T dO may start while ds is formed
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_READY + s));
      tc_fence_after_sync();
      {
        uint32_t raw[kStep];
        tmem_ld32(tm_p2 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
        tmem_ld32(tm_p2 + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_FREE + 2 + s));
#pragma unroll
        for (int c = 0; c < kStep / 2; ++c) {
          const float2 ds = __fmul2_rn(t[c], make_float2(__uint_as_float(raw[2 * c]), __uint_as_float(raw[2 * c + 1])));
          e2[c] = pack2<kBf16>(ds.x, ds.y);
        }
      }
      PROBE(13);
      // the ds^T buffer was last read by the MMAs (and the dbias store) of step n - NDS
      if (n >= NDS) {
        const int m = n - NDS;
        ok = wait_or_abort(bar(DS_FREE + (m & 1)), (m >> 1) & 1, abort_flag, a.status, 317);
        if (!ok) break;
      }
      PROBE(6);
      {
        const uint32_t tile = sbase + L::kDs + (n % NDS) * kBoxBytes + ds_thread;
        if constexpr (kDbias) {
  #pragma unroll
          for (int c = 0; c < kStep / 2; ++c) {
            const uint32_t lo16 = e2[c] & 0xffffu, hi16 = e2[c] >> 16;
            asm volatile("st.shared.u16 [%0], %1;" ::"r"((tile ^ (((2 * c) & 7) << 4)) + (2 * c) * 128), "h"(uint16_t(lo16)) : "memory");
            asm volatile("st.shared.u16 [%0], %1;" ::"r"((tile ^ (((2 * c + 1) & 7) << 4)) + (2 * c + 1) * 128), "h"(uint16_t(hi16)) : "memory");
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile ^ (uint32_t(i) << 4)), "r"(e2[4 * i]),
                         "r"(e2[4 * i + 1]), "r"(e2[4 * i + 2]), "r"(e2[4 * i + 3])
                         : "memory");
        }
        fence_proxy_async_smem();
      }
      PROBE(7);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(E_READY + s));
      PROBE(8);
      // dQ^T of the previous step (the other group's) is complete by now: add it to the accumulator
      if (n >= 1) ok = drain(n - 1);
    }
    // the last step's dQ^T is drained by the group that did not produce it
    if (ok && n_steps > 0 && grp == (n_steps & 1)) ok = drain(n_steps - 1);

    // ---------------- epilogue: group 0 writes dv, group 1 writes dk * scale ----------------
    if (ok && n_steps > 0) ok = wait_or_abort(bar(ACC_DONE), 0, abort_flag, a.status, 308);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t tacc = (grp == 0 ? tm_dv : tm_dk) + lane_addr;
      const float omul = grp == 0 ? 1.f : a.scale;
      void* outp = grp == 0 ? a.out1 : a.out2;
      const int64_t* os = grp == 0 ? a.o1s : a.o2s;
      uint8_t* orow_ptr = reinterpret_cast<uint8_t*>(outp) + 2 * (b * os[0] + h * os[1] + int64_t(key) * os[2]);
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t o[32];
        if (n_steps > 0) {
          tmem_ld32(tacc + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (key < a.T) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2<kBf16>(__uint_as_float(o[i]) * omul, __uint_as_float(o[i + 1]) * omul);
            w.y = pack2<kBf16>(__uint_as_float(o[i + 2]) * omul, __uint_as_float(o[i + 3]) * omul);
            w.z = pack2<kBf16>(__uint_as_float(o[i + 4]) * omul, __uint_as_float(o[i + 5]) * omul);
            w.w = pack2<kBf16>(__uint_as_float(o[i + 6]) * omul, __uint_as_float(o[i + 7]) * omul);
            *reinterpret_cast<uint4*>(orow_ptr + (c * 32 + i) * 2) = w;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) drain_after_abort();
  if (warp == 3) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// dq = scale * (fp32 sums) in the operand dtype.  The accumulator holds, per (batch, head), [query / 4][d][query % 4].
// One thread takes four queries x eight consecutive d: eight 16-byte loads (128 contiguous bytes), four 16-byte stores.
template <bool kBf16>
__global__ void dq_finish_d128_kernel(const float* __restrict__ acc, void* dq, int64_t s_b, int64_t s_h, int64_t s_row,
                                      int H, int S, int acc_rows, int bh_begin, int64_t n_items, float scale) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_items) return;
  const int dchunk = int(i & 15);                 // 16 chunks of 8 d
  const int64_t qg = i >> 4;                      // global 4-query group
  const int groups_per_bh = (S + 3) / 4;
  const int bh_local = int(qg / groups_per_bh);
  const int g = int(qg - int64_t(bh_local) * groups_per_bh);
  const int bh = bh_begin + bh_local;
  const int b = bh / H, h = bh - b * H;
  const float* src = acc + (int64_t(bh_local) * acc_rows / 4 + g) * (kD * 4) + dchunk * 32;
  float4 v[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) v[d] = __ldg(reinterpret_cast<const float4*>(src) + d);
  uint8_t* base = reinterpret_cast<uint8_t*>(dq) + 2 * (b * s_b + h * s_h + dchunk * 8);
#pragma unroll
  for (int qq = 0; qq < 4; ++qq) {
    const int q = g * 4 + qq;
    if (q >= S) break;
    float x[8];
#pragma unroll
    for (int d = 0; d < 8; ++d) x[d] = (qq == 0 ? v[d].x : qq == 1 ? v[d].y : qq == 2 ? v[d].z : v[d].w) * scale;
    uint4 w;
    w.x = pack2<kBf16>(x[0], x[1]);
    w.y = pack2<kBf16>(x[2], x[3]);
    w.z = pack2<kBf16>(x[4], x[5]);
    w.w = pack2<kBf16>(x[6], x[7]);
    *reinterpret_cast<uint4*>(base + 2 * int64_t(q) * s_row) = w;
  }
}

template <bool kBf16, bool kTileBias, bool kDbias>
int launch_one(const D128Maps& m, const BwdArgs& a, int n_tiles, int bh_count, cudaStream_t st) {
  auto kernel = sdpa_bwd_tc_d128_kernel<kBf16, kTileBias, kDbias>;
  const int smem = Smem<kTileBias>::kTotal + 1024;
  static bool ready[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev < 0 || !ready[dev]) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess || attr.numRegs != kLaunchRegs) {
      // the register hand-over inside the kernel is balanced for exactly kLaunchRegs per thread at launch
      set_error("sdpa_bwd_tc_d128_kernel was built with %d registers per thread, expected %d", attr.numRegs, kLaunchRegs);
      return NB200_ERR_LAUNCH;
    }
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(sdpa_bwd_tc_d128_kernel, %d): %s", smem, cudaGetErrorString(e));
      return NB200_ERR_LAUNCH;
    }
    if (dev >= 0) ready[dev] = true;
  }
  dim3 grid(n_tiles, bh_count);
  kernel<<<grid, kThreads, smem, st>>>(m.k, m.v, m.q, m.dout, m.bias, m.dbias, a);
  count_launch();
  return check_launch("sdpa_bwd_tc_kernel<one-pass d128>");
}

}  // namespace

bool d128_merged_supported(const Problem& pr, int bias_mode, bool bias_mma) {
  if (pr.D != 128 || pr.Dv != 128) return false;
  if (bias_mode == kBiasTile && !bias_mma) return false;   // the tile bias reaches the scores through the tensor core only
  if (pr.dbias_accum) return false;                        // a broadcast bias' gradient needs fp32 sums (two-kernel path)
  if (pr.want_dbias) {
    if (bias_mode != kBiasTile) return false;
    if ((pr.B > 1 && pr.bs[0] == 0) || (pr.H > 1 && pr.bs[1] == 0)) return false;   // shared over batch / heads: fp32 sums
    // dbias tiles leave through TMA: dense rows like any tile map; skipped regions are zeroed by one memset, which
    // needs the whole buffer to be one contiguous block
    if (!pr.dbias) return true;                            // planning: no buffer yet
    if (!tile_map_ok(pr.dbias, pr.dbs[2], pr.dbs[1], pr.dbs[0], pr.H, pr.B, false)) return false;
    const bool needs_zero_fill = pr.causal || mask_key_only(pr);
    const bool dense = pr.dbs[1] == int64_t(pr.S) * pr.dbs[2] && pr.dbs[0] == int64_t(pr.H) * pr.S * pr.dbs[2];
    if (needs_zero_fill && !dense) return false;
  }
  return true;
}

size_t d128_acc_bytes(const Problem& pr) {
  const int64_t rows = (int64_t(pr.S) + kStep - 1) / kStep * kStep;
  return sizeof(float) * size_t(pr.bh_count) * size_t(rows) * kD;
}

int launch_bwd_d128(const D128Maps& maps, const BwdArgs& a, bool bf16, bool tile_bias, int n_tiles, int bh_count,
                    cudaStream_t st) {
  if (tile_bias && a.dbias)
    return bf16 ? launch_one<true, true, true>(maps, a, n_tiles, bh_count, st)
                : launch_one<false, true, true>(maps, a, n_tiles, bh_count, st);
  if (tile_bias)
    return bf16 ? launch_one<true, true, false>(maps, a, n_tiles, bh_count, st)
                : launch_one<false, true, false>(maps, a, n_tiles, bh_count, st);
  return bf16 ? launch_one<true, false, false>(maps, a, n_tiles, bh_count, st)
              : launch_one<false, false, false>(maps, a, n_tiles, bh_count, st);
}

int launch_dq_finish_d128(const Problem& pr, const float* acc, int acc_rows, bool bf16, cudaStream_t st) {
  const int64_t n_items = int64_t(pr.bh_count) * ((pr.S + 3) / 4) * 16;
  const int blocks = int((n_items + 255) / 256);
  if (bf16)
    dq_finish_d128_kernel<true><<<blocks, 256, 0, st>>>(acc, pr.dq, pr.dqs[0], pr.dqs[1], pr.dqs[2], pr.H, pr.S, acc_rows,
                                                        pr.bh_begin, n_items, pr.scale);
  else
    dq_finish_d128_kernel<false><<<blocks, 256, 0, st>>>(acc, pr.dq, pr.dqs[0], pr.dqs[1], pr.dqs[2], pr.H, pr.S, acc_rows,
                                                         pr.bh_begin, n_items, pr.scale);
  count_launch();
  return check_launch("dq_finish_d128_kernel");
}

}  // namespace tc
}  // namespace nb200

#ifdef NB200_PROBE
extern "C" NB200_API int nb200_debug_probe(long long* out32, int reset) {
  long long zero[32] = {};
  if (out32) cudaMemcpyFromSymbol(out32, nb200::tc::g_probe, sizeof(zero));
  if (reset) cudaMemcpyToSymbol(nb200::tc::g_probe, zero, sizeof(zero));
  return 0;
}
#endif
