// Backward flash attention for sm_100a: TMA -> shared memory -> tcgen05.mma with
// TMEM accumulators; p and ds are recomputed per tile from (q, k, v, bias,
// mask, lse, delta) as in the reference's backward kernels
// (reference src/nitrix/_kernels/cuda/attention.py:272-332 `_bwd_kv_kernel`,
// :335-387 `_bwd_q_kernel`), on 128 x 64 tiles instead of 32 x 32.
//
// One kernel template serves both directions:
//   query-major (kKeyMajor = false): a CTA owns 128 query rows, streams 64-key
//     steps; S = Q K^T, dP = dO V^T, ds = p (dP - delta); dQ += ds K; writes
//     dq and, when asked, the dbias tile (ds in bias dtype).
//   key-major (kKeyMajor = true): a CTA owns 128 keys, streams 64-query steps;
//     S^T = K Q^T, dP^T = V dO^T; dV += p^T dO; dK += ds^T Q; writes dk, dv.
// Naming below: X1, X2 are the owner's two 128-row operands (Q, dO | K, V);
// Y1, Y2 the streamed 64-row operands (K, V | Q, dO).  Per step:
//   P1 = X1 Y1^T, P2 = X2 Y2^T            (SS tcgen05.mma, 128 x 64, fp32 in TMEM)
//   E1 = p, E2 = ds as 16-bit             (written over P1 / P2 in TMEM)
//   ACC1 += E1 Y2 (key-major: dV), ACC2 += E2 Y1 (dQ | dK)
//                                          (TS tcgen05.mma, Y consumed MN-major)
// TMEM columns (512): D = 128: products of stage s in {0,1} at 128 s (P1) and 128 s + 64 (P2), E tiles written over
// them, ACC1 at 256, ACC2 at 384.  D = 64: products as above, E tiles of their own at 256 + 64 s, ACC1 at 384,
// ACC2 at 448 (a stage's products are recomputed as soon as the element-wise warps hold them in registers).
// Merged variant (key-major, D = 64, no bias gradient): ds goes to shared memory instead of TMEM and also feeds
// dQ = ds K per pair of steps (a 128 x 64 tile at TMEM column 320), which the element-wise warps add to an fp32
// accumulator in global memory; the query-major kernel is then not needed.
// Twelve warps: 0 issues the accumulating MMAs, 1 the TMA copies of the step loop (ring refills and bias tiles, one
// thread serving both), 2 issues the products, 3 owns TMEM and builds the per-query (key-major) or per-key
// (query-major) addends as MMA operands, 4-7 / 8-11 are two element-wise groups that take alternate steps (one
// owner row per thread).  The owner tiles and the first ring stages are issued by thread 0 during start-up.  All
// waits are bounded.  At head dim 128 these kernels only serve what the one-kernel backward of
// sdpa_tc_bwd_d128.cu declines (a bias gradient that needs fp32 sums).
#include <math.h>
#include <stdlib.h>

#include "sdpa_tc_bwd.cuh"

namespace nb200 {
namespace tc {

using namespace sm100;

namespace {

constexpr int kThreads = 384;
constexpr int kStep = 64;                     // streamed rows per step
constexpr int kYBoxBytes = kStep * 128;       // one 64-row x 128-byte TMA box
// register split after start-up (setmaxnreg): 128 * kProducerRegs + 256 * kWorkerRegs <= 65536
constexpr int kProducerRegs = 88;
constexpr int kWorkerRegs = 208;
// setmaxnreg.inc blocks (without bound) until the CTA's OWN pool -- the registers it was launched with, here
// kLaunchRegs per thread -- holds enough released registers, so the hand-over must balance at compile time.
constexpr int kLaunchRegs = 168;  // what __launch_bounds__(384, 1) gives: 65536 / 384 rounded down to a multiple of 8
static_assert((kLaunchRegs - kProducerRegs) * 128 >= (kWorkerRegs - kLaunchRegs) * 256,
              "worker warps would wait forever for registers the producer warps never release");


template <int D, bool kMerged>
struct BwdSmem {
  static constexpr int kXBytes = kTile * D * 2;                 // one owner operand
  static constexpr int kYBytes = kStep * D * 2;                 // one streamed operand
  static constexpr int kYStages = D == 64 ? 4 : 3;
  static constexpr int kYStageBytes = 2 * kYBytes + 1024;       // Y1, Y2, then lse[64] + delta[64] (key-major)
  static constexpr int kBiasSlots = 2;                          // 16 KB each
  static constexpr int kX = 0;
  static constexpr int kY = kX + 2 * kXBytes;
  static constexpr int kBias = kY + kYStages * kYStageBytes;
  // hi * I and lo * I (64 x 64 each), the second operand of the MMAs that add a bias tile to the transposed scores
  static constexpr int kIdentBytes = 2 * kStep * 128;
  static constexpr int kIdent = kBias + kBiasSlots * kBoxBytes;
  // Key-major: -lse / (scale log2e) and -delta of a step's 64 queries are added to the two products by one more
  // K = 16 MMA step each, products += W * C^T with W (128 x 16) the same row of weights for every key and
  // C (64 x 16) the query's value split over the first columns.  Both are K-major without swizzle: 8-row groups of
  // 256 bytes = [8 rows x 16 bytes (K 0-7)][8 rows x 16 bytes (K 8-15, zero)].
  static constexpr int kWeightBytes = (kTile / 8) * 256;
  static constexpr int kAugTileBytes = (kStep / 8) * 256;
  static constexpr int kAugSlotBytes = 2 * kAugTileBytes;      // lse tile, delta tile
  static constexpr int kWeights = kIdent + kIdentBytes;
  static constexpr int kAug = kWeights + kWeightBytes;          // two slots
  // Merged kernel: ds tiles (128 keys x 64 queries, 16-bit, 128-byte-swizzled rows) of the last four steps.  The
  // tensor core reads a tile K-major for dK and a pair of tiles MN-major for dQ.  Must stay 1024-byte aligned.
  static constexpr int kDsSlots = 4;
  static constexpr int kDs = (kAug + 2 * kAugSlotBytes + 1023) / 1024 * 1024;
  static constexpr int kBars = kDs + (kMerged ? kDsSlots * kBoxBytes : 0);
  // x_full, y_full[n], y_empty[n], prod_full[2], e_ready[2], acc_done, bias_full[2], bias_empty[2], p_free[2], e_free[2],
  // aug_full[2], aug_free[2], dq_full, dq_free
  static constexpr int kNumBars = 1 + 2 * kYStages + 2 + 2 + 1 + 4 + 4 + 4 + 2;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
};

template <int D, bool kBf16, bool kKeyMajor, bool kMerged>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x1, const __grid_constant__ CUtensorMap tm_x2,
                   const __grid_constant__ CUtensorMap tm_y1, const __grid_constant__ CUtensorMap tm_y2,
                   const __grid_constant__ CUtensorMap tm_bias, const BwdArgs a) {
  static_assert(!kMerged || (kKeyMajor && D == 64), "the merged kernel is the key-major kernel at head dim 64");
  using L = BwdSmem<D, kMerged>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);
  auto bar = [&](int i) { return smem_u32(bars + i); };
  constexpr int NY = L::kYStages;
  constexpr int X_FULL = 0, Y_FULL = 1, Y_EMPTY = Y_FULL + NY, PROD_FULL = Y_EMPTY + NY, E_READY = PROD_FULL + 2,
                ACC_DONE = E_READY + 2, B_FULL = ACC_DONE + 1, B_EMPTY = B_FULL + 2, P_FREE = B_EMPTY + 2,
                E_FREE = P_FREE + 2, AUG_FULL = E_FREE + 2, AUG_FREE = AUG_FULL + 2, DQ_FULL = AUG_FREE + 2, DQ_FREE = DQ_FULL + 1;
  // D = 64 has TMEM room for E tiles of their own.  Then a stage's products can be recomputed as soon as the
  // element-wise group has read them out (P_FREE).  At D = 128 the E tiles lie over the products, which can be
  // recomputed only once the accumulating MMAs of two steps earlier have read them (E_FREE).
  constexpr bool kDeep = D == 64;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = a.bh_begin + blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int n_owner = kKeyMajor ? a.T : a.S;     // owner axis length
  const int n_stream = kKeyMajor ? a.S : a.T;    // streamed axis length
  // causal work per owner tile grows with the query index and shrinks with the key index: heaviest first
  const int otile = (a.causal && !kKeyMajor) ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int o0 = otile * kTile;
  int s_begin = 0, s_end = (n_stream + kStep - 1) / kStep;
  if (a.causal) {
    if (kKeyMajor) s_begin = min(s_end, o0 / kStep);                       // queries i >= first key
    else s_end = min(s_end, (min(o0 + kTile, n_owner) + kStep - 1) / kStep);  // keys j <= last query
  }
  // key-only mask (key padding): keys at or past the last kept one contribute nothing
  const int kept = kept_key_length(a.mask, b, h, a.T);
  if (kKeyMajor) {
    if (o0 >= kept) s_end = s_begin;                                  // every key of this tile is dropped: dk = dv = 0
  } else {
    s_end = max(s_begin, min(s_end, (kept + kStep - 1) / kStep));     // stream the kept keys only
  }
  const int n_steps = s_end - s_begin;

  // Start-up is a visible share of a short CTA's life (16 steps at L = 2048), so it is kept short: the barriers are
  // initialised by one thread each, and thread 0 then starts the first copies (owner tiles, first ring stages, first
  // bias slots) itself, so that their latency runs under the rest of the start-up (operand tiles below, TMEM
  // allocation, register hand-over) instead of after it.
  if (threadIdx.x < L::kNumBars) {
    const int i = threadIdx.x;
    uint32_t count = 1;
    if (i >= E_READY && i < E_READY + 2) count = 4;   // one lane per warp of the group
    if (i >= P_FREE && i < P_FREE + 2) count = 4;
    if (i >= B_EMPTY && i < B_EMPTY + 2) count = a.bias_mma ? 1 : 4;   // released by the MMA issuer or by the group's warps
    if (i == DQ_FREE) count = 8;                       // every element-wise warp has read its part of the dq tile
    mbar_init(bar(i), count);
    if (i == 0) *abort_flag = 0;
    mbar_init_fence();
  }
  __syncwarp();
  static_assert(L::kNumBars <= 64, "barrier initialisation assumes the first two warps cover all barriers");
  // named barrier over the first two warps: every barrier is initialised before thread 0 hands any of them to TMA
  if (threadIdx.x < 64) asm volatile("bar.sync 1, 64;" ::: "memory");
  if (threadIdx.x == 0 && n_steps > 0) {
    mbar_expect_tx(bar(X_FULL), 2 * L::kXBytes);
#pragma unroll
    for (int x = 0; x < D / 64; ++x) {
      tma_load_4d(sbase + L::kX + x * kBoxBytes, &tm_x1, bar(X_FULL), x * 64, o0, h, b);
      tma_load_4d(sbase + L::kX + L::kXBytes + x * kBoxBytes, &tm_x2, bar(X_FULL), x * 64, o0, h, b);
    }
    const int n_first = n_steps < NY ? n_steps : NY;
    for (int n = 0; n < n_first; ++n) {
      const int r0 = (s_begin + n) * kStep;
      const uint32_t ybase = sbase + L::kY + n * L::kYStageBytes;
      const uint32_t row_bytes = 4u * uint32_t(min(kStep, a.ld_rows - r0));
      mbar_expect_tx(bar(Y_FULL + n), 2 * L::kYBytes + (kKeyMajor ? 2 * row_bytes : 0));
#pragma unroll
      for (int x = 0; x < D / 64; ++x) {
        tma_load_4d(ybase + x * kYBoxBytes, &tm_y1, bar(Y_FULL + n), x * 64, r0, h, b);
        tma_load_4d(ybase + L::kYBytes + x * kYBoxBytes, &tm_y2, bar(Y_FULL + n), x * 64, r0, h, b);
      }
      if (kKeyMajor) {
        const int64_t ro = (int64_t(b) * a.H + h) * a.ld_rows + r0;
        bulk_load(ybase + 2 * L::kYBytes, a.lse + ro, row_bytes, bar(Y_FULL + n));
        bulk_load(ybase + 2 * L::kYBytes + 256, a.delta + ro, row_bytes, bar(Y_FULL + n));
      }
      if (a.bias_mode == kBiasTile && n < 2) {
        mbar_expect_tx(bar(B_FULL + n), kBoxBytes);
        const uint32_t dst = sbase + L::kBias + n * kBoxBytes;
        if (kKeyMajor) {
          tma_load_4d(dst, &tm_bias, bar(B_FULL + n), o0, r0, h * a.bias_h_mul, b * a.bias_b_mul);
          tma_load_4d(dst + kYBoxBytes, &tm_bias, bar(B_FULL + n), o0 + 64, r0, h * a.bias_h_mul, b * a.bias_b_mul);
        } else {
          tma_load_4d(dst, &tm_bias, bar(B_FULL + n), r0, o0, h * a.bias_h_mul, b * a.bias_b_mul);
        }
      }
    }
  }
  if (kKeyMajor || a.key_aug) {
    {
      // weight rows (w0, w1, w2, 0, ...): a query's addend is sum_j w_j c_j with c_j 16-bit; bf16 has fp32's range,
      // so three unit weights give 24 bits; fp16 spreads the terms over 2^8, 1, 2^-8 to cover magnitudes up to 1.6e7
      uint4* wt = reinterpret_cast<uint4*>(smem + L::kWeights);
      const uint32_t w01 = kBf16 ? 0x3F803F80u : 0x3C005C00u;   // (w0, w1): bf16 (1, 1); fp16 (256, 1)
      const uint32_t w2 = kBf16 ? 0x00003F80u : 0x00001C00u;    // (w2, 0):  bf16 1; fp16 2^-8
      for (int idx = threadIdx.x; idx < L::kWeightBytes / 16; idx += kThreads)
        wt[idx] = (idx & 8) ? make_uint4(0, 0, 0, 0) : make_uint4(w01, w2, 0, 0);
      uint4* aug = reinterpret_cast<uint4*>(smem + L::kAug);
      for (int idx = threadIdx.x; idx < 2 * L::kAugSlotBytes / 16; idx += kThreads) aug[idx] = make_uint4(0, 0, 0, 0);
      fence_proxy_async_smem();
    }
    if (kKeyMajor && a.bias_mma) {
      // Two 64 x 64 tiles, hi * I and lo * I with hi + lo = 1 / scale to 16 + 16 bits, as K-major 128-byte-swizzled
      // operands (rows of 64 elements = 128 bytes).  Tile 0 at kIdent, tile 1 at kIdent + 8 KB.
      uint4* ident = reinterpret_cast<uint4*>(smem + L::kIdent);
      for (int idx = threadIdx.x; idx < 2 * kStep * 8; idx += kThreads) {   // one 16-byte chunk each
        const int tile = idx / (kStep * 8), rem = idx - tile * kStep * 8;
        const int row = rem >> 3, chunk = (rem & 7) ^ (row & 7);             // logical chunk stored at this slot
        const int col0 = chunk * 8;                                          // first logical column of the chunk
        const float val = tile == 0 ? a.inv_scale_hi : a.inv_scale_lo;
        const uint16_t one = kBf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (row >= col0 && row < col0 + 8) w[(row - col0) >> 1] = uint32_t(one) << (((row - col0) & 1) * 16);
        ident[idx] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async_smem();   // written by threads, read by the tensor core
    }
  }
  if (warp == 3) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns.  Products: stage s at 128 s (P1) and 128 s + 64 (P2).
  //   D = 64 (kDeep): E tiles of stage s at 256 + 64 s (E1, 32 columns) and + 32 (E2); ACC1 at 384, ACC2 at 448.
  //   D = 128: no room for separate E tiles: E1 / E2 overwrite P1 / P2; ACC1 at 256, ACC2 at 384.
  //   merged: E1 of stage s at 256 + 32 s (ds goes to shared memory instead of E2), the dq tile (128 queries x 64) at 320.
  const uint32_t tm_e = kDeep ? tmem + 256 : tmem;
  constexpr int kEStage = kMerged ? 32 : (kDeep ? 64 : 128), kE2Off = kDeep ? 32 : 64;
  const uint32_t tm_dq = tmem + 320;
  const uint32_t tm_acc1 = tmem + (kDeep ? 384 : 256), tm_acc2 = tm_acc1 + D;

  if (warp < 4) {
  reg_dealloc<kProducerRegs>();
  if (warp == 1) {
    // ---------------- TMA duties of the step loop: ring refills and bias tiles, ONE thread ----------------
    // (the owner tiles, the first NY stages and the first two bias slots were issued during start-up).  The thread
    // waits on each duty's barrier in turn, suspended in hardware for at most a short time hint while both are
    // pending, so whichever completes first is served at once.
    if (lane == 0 && n_steps > 0) {
      int yn = min(n_steps, NY);
      int bn = a.bias_mode == kBiasTile ? min(n_steps, 2) : n_steps;
      const long long t0 = clock64();
      uint32_t idle = 0;
      while (yn < n_steps || bn < n_steps) {
        const uint32_t hint = (yn < n_steps && bn < n_steps) ? 64u : 4096u;
        bool progressed = false;
        if (yn < n_steps && mbar_try_wait_hint(bar(Y_EMPTY + yn % NY), ((yn / NY) & 1) ^ 1, hint)) {
          const int st = yn % NY;
          const int r0 = (s_begin + yn) * kStep;
          const uint32_t ybase = sbase + L::kY + st * L::kYStageBytes;
          // lse / delta rows of the step that exist (a multiple of 4 rows, so the copy stays a multiple of 16 bytes)
          const uint32_t row_bytes = 4u * uint32_t(min(kStep, a.ld_rows - r0));
          mbar_expect_tx(bar(Y_FULL + st), 2 * L::kYBytes + (kKeyMajor ? 2 * row_bytes : 0));
#pragma unroll
          for (int x = 0; x < D / 64; ++x) {
            tma_load_4d(ybase + x * kYBoxBytes, &tm_y1, bar(Y_FULL + st), x * 64, r0, h, b);
            tma_load_4d(ybase + L::kYBytes + x * kYBoxBytes, &tm_y2, bar(Y_FULL + st), x * 64, r0, h, b);
          }
          if (kKeyMajor) {
            // lse and delta of the step's 64 queries: two 256-byte bulk copies on the same barrier
            const int64_t ro = (int64_t(b) * a.H + h) * a.ld_rows + r0;
            bulk_load(ybase + 2 * L::kYBytes, a.lse + ro, row_bytes, bar(Y_FULL + st));
            bulk_load(ybase + 2 * L::kYBytes + 256, a.delta + ro, row_bytes, bar(Y_FULL + st));
          }
          ++yn;
          progressed = true;
        }
        if (bn < n_steps && mbar_try_wait_hint(bar(B_EMPTY + (bn & 1)), ((bn >> 1) & 1) ^ 1, hint)) {
          const int slot = bn & 1;
          const int r0 = (s_begin + bn) * kStep;
          mbar_expect_tx(bar(B_FULL + slot), kBoxBytes);
          const uint32_t dst = sbase + L::kBias + slot * kBoxBytes;
          if (kKeyMajor) {  // 64 query rows x 128 keys: two 64 x 64 boxes
            tma_load_4d(dst, &tm_bias, bar(B_FULL + slot), o0, r0, h * a.bias_h_mul, b * a.bias_b_mul);
            tma_load_4d(dst + kYBoxBytes, &tm_bias, bar(B_FULL + slot), o0 + 64, r0, h * a.bias_h_mul, b * a.bias_b_mul);
          } else {          // 128 query rows x 64 keys: one 64 x 128 box
            tma_load_4d(dst, &tm_bias, bar(B_FULL + slot), r0, o0, h * a.bias_h_mul, b * a.bias_b_mul);
          }
          ++bn;
          progressed = true;
        }
        if (!progressed && (++idle & 0x3F) == 0) {
          if (*abort_flag) break;
          if (*reinterpret_cast<volatile int*>(a.status) != 0) { *abort_flag = 1; break; }
          if (clock64() - t0 > 20 * kWaitCycles) {   // the whole CTA's life is bounded as well
            *abort_flag = 1;
            atomicExch(a.status, 201);
            break;
          }
        }
      }
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer 1: the two products of every step ----------------
    // Two threads issue MMAs: this one the products, warp 0 the accumulating ones.  One issuing thread needs about
    // as long for a step's 30 to 40 MMA instructions as the element-wise warps need for the step, and in a single
    // instruction stream the products of a later step queue behind accumulating MMAs that wait for those warps.
    if (elect_one() && n_steps > 0) {
      constexpr uint32_t idesc_prod = make_idesc(kBf16, kTile, kStep, false, false);
      bool ok = wait_or_abort(bar(X_FULL), 0, abort_flag, a.status, 203);
      // descriptors are built once; an offset only moves the 16-byte start-address field
      const uint64_t x1desc = make_smem_desc(sbase + L::kX, 16, 1024);
      const uint64_t x2desc = make_smem_desc(sbase + L::kX + L::kXBytes, 16, 1024);
      for (int n = 0; n < n_steps && ok; ++n) {
        const int st = n % NY, s = n & 1;
        ok = wait_or_abort(bar(Y_FULL + st), (n / NY) & 1, abort_flag, a.status, 204);
        if (ok && n >= 2) {
          // the stage is rewritten: with E tiles of their own (D = 64) once step n - 2 has read the products out,
          // otherwise (the E tiles lie over the products) once the accumulating MMAs of step n - 2 have read them
          ok = wait_or_abort(bar((kDeep ? P_FREE : E_FREE) + s), ((n - 2) >> 1) & 1, abort_flag, a.status, 209);
        }
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t ybase = sbase + L::kY + st * L::kYStageBytes;
        const uint64_t y1desc = make_smem_desc(ybase, 16, 1024), y2desc = make_smem_desc(ybase + L::kYBytes, 16, 1024);
        const uint32_t p1 = tmem + s * 128, p2 = p1 + 64;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t xo = uint64_t(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
          const uint64_t yo = uint64_t(((kk / 4) * kYBoxBytes + (kk % 4) * 32) >> 4);
          mma_ss(p1, x1desc + xo, y1desc + yo, idesc_prod, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t xo = uint64_t(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
          const uint64_t yo = uint64_t(((kk / 4) * kYBoxBytes + (kk % 4) * 32) >> 4);
          mma_ss(p2, x2desc + xo, y2desc + yo, idesc_prod, kk > 0 ? 1u : 0u);
        }
        if (a.bias_mma) {
          // scores += bias * (I / scale): the bias slot is consumed straight from shared memory by the tensor core
          const int slot = n & 1;
          ok = wait_or_abort(bar(B_FULL + slot), (n >> 1) & 1, abort_flag, a.status, 211);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t bslot = sbase + L::kBias + slot * kBoxBytes;
          // P1[key, q] += bias^T[key, q'] (hi I + lo I)[q', q]: A = the slot (64 q' rows, two 64-key boxes) read
          // MN-major, B = the identity tiles, K-major
          constexpr uint32_t idesc_bias = make_idesc(kBf16, kTile, kStep, true, false);
          const uint64_t adesc = make_smem_desc(bslot, kYBoxBytes, 1024);
          const int n_tiles = a.inv_scale_lo != 0.f ? 2 : 1;
          for (int tile = 0; tile < n_tiles; ++tile) {
            const uint64_t bdesc = make_smem_desc(sbase + L::kIdent + tile * kYBoxBytes, 16, 1024);
#pragma unroll
            for (int kk = 0; kk < kStep / 16; ++kk)
              mma_ss(p1, adesc + uint64_t((kk * 2048) >> 4), bdesc + uint64_t((kk * 32) >> 4), idesc_bias, 1u);
          }
        }
        if constexpr (kKeyMajor) {
          // P1 += W C1^T (C1: -lse / (scale log2e)), P2 += W C2^T (C2: -delta)
          ok = wait_or_abort(bar(AUG_FULL + s), (n >> 1) & 1, abort_flag, a.status, 212);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t wdesc = make_smem_desc_noswizzle(sbase + L::kWeights, 128, 256);
          const uint32_t aslot = sbase + L::kAug + s * L::kAugSlotBytes;
          mma_ss(p1, wdesc, make_smem_desc_noswizzle(aslot, 128, 256), idesc_prod, 1u);
          mma_ss(p2, wdesc, make_smem_desc_noswizzle(aslot + L::kAugTileBytes, 128, 256), idesc_prod, 1u);
        }
        if constexpr (!kKeyMajor) {
          if (a.key_aug) {
            // P1 += W C^T: the per-key addends land on every query row
            ok = wait_or_abort(bar(AUG_FULL + s), (n >> 1) & 1, abort_flag, a.status, 212);
            if (!ok) break;
            tc_fence_after_sync();
            const uint64_t wdesc = make_smem_desc_noswizzle(sbase + L::kWeights, 128, 256);
            mma_ss(p1, wdesc, make_smem_desc_noswizzle(sbase + L::kAug + s * L::kAugSlotBytes, 128, 256), idesc_prod, 1u);
          }
        }
        mma_commit(bar(PROD_FULL + s));
        if (kKeyMajor || a.key_aug) mma_commit(bar(AUG_FREE + s));
        if (a.bias_mma) mma_commit(bar(B_EMPTY + (n & 1)));   // the slot may be refilled once these MMAs are done
      }
    }
  } else if (warp == 0) {
    // ---------------- MMA issuer 2: the accumulating MMAs of every step ----------------
    // (every commit below covers all MMAs this thread issued before it: a stage's E_FREE therefore also tells that
    // the ds tiles of the steps before it have been read)
    if (elect_one() && n_steps > 0) {
      constexpr uint32_t idesc_acc = make_idesc(kBf16, kTile, D, false, true);
      bool ok = wait_or_abort(bar(X_FULL), 0, abort_flag, a.status, 203);
      for (int m = 0; m < n_steps && ok; ++m) {
        const int st = m % NY, s = m & 1;
        ok = wait_or_abort(bar(E_READY + s), (m >> 1) & 1, abort_flag, a.status, 205);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t ybase = sbase + L::kY + st * L::kYStageBytes;
        const uint64_t y1mn = make_smem_desc(ybase, kYBoxBytes, 1024);
        const uint64_t y2mn = make_smem_desc(ybase + L::kYBytes, kYBoxBytes, 1024);
        const uint32_t e1 = tm_e + s * kEStage, e2 = e1 + kE2Off;
        if constexpr (kMerged) {
          // dV += p^T dO (p from TMEM), dK += ds^T Q (ds from its shared-memory tile, K-major)
          const uint64_t dsk = make_smem_desc(sbase + L::kDs + (m % L::kDsSlots) * kBoxBytes, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < kStep / 16; ++kk) {
            const uint32_t acc = (m > 0 || kk > 0) ? 1u : 0u;
            mma_ts(tm_acc1, e1 + kk * 8, y2mn + uint64_t((kk * 2048) >> 4), idesc_acc, acc);
            mma_ss(tm_acc2, dsk + uint64_t((kk * 32) >> 4), y1mn + uint64_t((kk * 2048) >> 4), idesc_acc, acc);
          }
          mma_commit(bar(Y_EMPTY + st));          // the last readers of this ring stage
          if (m & 1) {
            // dq tile of the pair (m - 1, m): (128 queries x 128 keys) (128 keys x 64) = ds K; A = the two ds tiles
            // read MN-major (queries contiguous, tiles 16 KB apart), B = the K tile read MN-major
            const int j = m >> 1;
            if (j >= 1) {
              ok = wait_or_abort(bar(DQ_FREE), (j - 1) & 1, abort_flag, a.status, 215);
              if (!ok) break;
              tc_fence_after_sync();
            }
            constexpr uint32_t idesc_dq = make_idesc(kBf16, kTile, D, true, true);
            const uint64_t dsm = make_smem_desc(sbase + L::kDs + ((m - 1) % L::kDsSlots) * kBoxBytes, kBoxBytes, 1024);
            const uint64_t kmn = make_smem_desc(sbase + L::kX, kBoxBytes, 1024);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              mma_ss(tm_dq, dsm + uint64_t((kk * 2048) >> 4), kmn + uint64_t((kk * 2048) >> 4), idesc_dq, kk > 0 ? 1u : 0u);
            mma_commit(bar(DQ_FULL));
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < kStep / 16; ++kk) {
            const uint32_t acc = (m > 0 || kk > 0) ? 1u : 0u;
            if (kKeyMajor) mma_ts(tm_acc1, e1 + kk * 8, y2mn + uint64_t((kk * 2048) >> 4), idesc_acc, acc);
            mma_ts(tm_acc2, e2 + kk * 8, y1mn + uint64_t((kk * 2048) >> 4), idesc_acc, acc);
          }
          mma_commit(bar(Y_EMPTY + st));
        }
        // D = 64: the E tiles of this stage may be rewritten; D = 128 (E tiles over the products): the stage's
        // products may be recomputed
        mma_commit(bar(E_FREE + s));
        if (m == n_steps - 1) mma_commit(bar(ACC_DONE));
      }
    }
  } else if (!kKeyMajor) {
    // ---------------- warp 3 (query-major): per-key addends as an MMA operand ----------------
    if (a.key_aug) {
      const float inv_scale = 1.f / a.scale;
      const uint16_t* bk = a.bias_mode == kBiasKey
                               ? reinterpret_cast<const uint16_t*>(a.bias) + (b * a.bias_bs + h * a.bias_hs)
                               : nullptr;
      const uint32_t* mk = a.mask_key_only ? a.mask.rows + b * a.mask.b_stride + h * a.mask.h_stride : nullptr;
      bool ok = true;
      for (int n = 0; n < n_steps && ok; ++n) {
        const int s = n & 1;
        if (n >= 2) ok = wait_or_abort(bar(AUG_FREE + s), ((n - 2) >> 1) & 1, abort_flag, a.status, 214);
        if (!ok) break;
        uint8_t* slot = smem + L::kAug + s * L::kAugSlotBytes;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kl = lane + 32 * e, key = (s_begin + n) * kStep + kl;
          float c = 0.f;
          if (key >= a.T) {
            c = -INFINITY;   // past the last key (the tile is padded with zero rows)
          } else {
            if (bk) {
              const uint16_t raw = __ldg(bk + key);
              c = (kBf16 ? __uint_as_float(uint32_t(raw) << 16) : __half2float(__ushort_as_half(raw))) * inv_scale;
            }
            if (mk && !((__ldg(mk + (key >> 5)) >> (key & 31)) & 1u)) c = -INFINITY;
          }
          uint32_t hh[3] = {0u, 0u, 0u};
          float rem = c;
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
            if (!(fabsf(back) < INFINITY)) break;   // an infinite (or NaN) term carries the value alone
            rem = fmaf(-back, w, rem);
          }
          *reinterpret_cast<uint4*>(slot + (kl >> 3) * 256 + (kl & 7) * 16) = make_uint4(hh[0] | (hh[1] << 16), hh[2], 0u, 0u);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(AUG_FULL + s));
      }
    }
  } else {
    // ---------------- warp 3: per-query addends as MMA operands ----------------
    const float inv_mul = 1.f / (a.scale * kLog2e);
    bool ok = true;
    for (int n = 0; n < n_steps && ok; ++n) {
      const int st = n % NY, s = n & 1;
      ok = wait_or_abort(bar(Y_FULL + st), (n / NY) & 1, abort_flag, a.status, 213);
      if (ok && n >= 2) ok = wait_or_abort(bar(AUG_FREE + s), ((n - 2) >> 1) & 1, abort_flag, a.status, 214);
      if (!ok) break;
      const float* ld = reinterpret_cast<const float*>(smem + L::kY + st * L::kYStageBytes + 2 * L::kYBytes);
      uint8_t* slot = smem + L::kAug + s * L::kAugSlotBytes;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int q = lane + 32 * e;
        // queries past S were not copied (their columns are masked; the addend must still be finite)
        const bool live = (s_begin + n) * kStep + q < a.S;
        const float c[2] = {live ? -ld[q] * inv_mul : 0.f, live ? -ld[kStep + q] : 0.f};
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
          // c = w0 c0 + w1 c1 + w2 c2 with the remainder carried in fp32
          float rem = c[tile];
          uint32_t h[3];
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            const float w = kBf16 ? 1.f : (j == 0 ? 256.f : (j == 1 ? 1.f : 0.00390625f));
            const float v = rem * (1.f / w);
            float back;
            if constexpr (kBf16) {
              const __nv_bfloat16 hv = __float2bfloat16_rn(v);
              h[j] = __bfloat16_as_ushort(hv);
              back = __bfloat162float(hv);
            } else {
              const __half hv = __float2half_rn(v);
              h[j] = __half_as_ushort(hv);
              back = __half2float(hv);
            }
            rem = fmaf(-back, w, rem);
          }
          *reinterpret_cast<uint4*>(slot + tile * L::kAugTileBytes + (q >> 3) * 256 + (q & 7) * 16) =
              make_uint4(h[0] | (h[1] << 16), h[2], 0u, 0u);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(AUG_FULL + s));
    }
  }
  } else {
    reg_alloc<kWorkerRegs>();
    // ---------------- element-wise groups (one owner row per thread) ----------------
    const int grp = (warp - 4) >> 2;
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int orow = o0 + r;                       // query row (query-major) or key (key-major)
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    bool ok = true;
    // without a bias the scale is folded into the exponent's multiplier: p = exp2(s * (scale log2e) - lse)
    // (the same holds when the tensor core has already added bias / scale to the scores)
    const bool key_aug = !kKeyMajor && a.key_aug;
    const bool fold_scale = a.bias_mode == kBiasNone || a.bias_mma || key_aug;
    const float mul = fold_scale ? a.scale * kLog2e : kLog2e;
    const float2 mul2 = make_float2(mul, mul), scale2 = make_float2(a.scale, a.scale);
    float lse_row = 0.f, delta_row = 0.f;
    if (!kKeyMajor && orow < a.S) {
      const int64_t ro = (int64_t(b) * a.H + h) * a.ld_rows + orow;
      lse_row = a.lse[ro];
      delta_row = a.delta[ro];
    }
    // packed mask words of this owner row
    const uint32_t* mbits = nullptr;
    bool key_dropped = false;
    if (a.mask.rows) {
      if (!kKeyMajor) {
        if (!(key_aug && a.mask_key_only))   // a key-only mask was added to the scores as -inf
          mbits = a.mask.rows + b * a.mask.b_stride + h * a.mask.h_stride + int64_t(min(orow, a.S - 1)) * a.mask.row_stride;
      } else if (a.mask_key_only) {
        const uint32_t* krow = a.mask.rows + b * a.mask.b_stride + h * a.mask.h_stride;
        key_dropped = orow >= a.T || !((krow[orow >> 5] >> (orow & 31)) & 1u);
      } else {
        mbits = a.mask.cols + b * a.mask.tb_stride + h * a.mask.th_stride + int64_t(min(orow, a.T - 1)) * a.mask.tkey_stride;
      }
    }
    const uint8_t* bias_key = nullptr;
    float bias_own = 0.f;  // key-major per-key bias: one value for this thread's key
    if (a.bias_mode == kBiasKey) {
      bias_key = reinterpret_cast<const uint8_t*>(a.bias) + 2 * (b * a.bias_bs + h * a.bias_hs);
      if (kKeyMajor && orow < a.T) {
        const uint16_t raw = *reinterpret_cast<const uint16_t*>(bias_key + 2 * orow);
        bias_own = kBf16 ? __uint_as_float(uint32_t(raw) << 16) : __half2float(__ushort_as_half(raw));
      }
    }

    // key-major, per-key bias gradient: running sum of this thread's key (the identity tiles are not used then)
    float* key_ds_sum = reinterpret_cast<float*>(smem + L::kIdent) + (threadIdx.x - 128);
    if (kKeyMajor && !kMerged && a.dbias_acc) *key_ds_sum = 0.f;
    float* acc_row = nullptr;                    // query-major, broadcast tile bias: this query's accumulator row
    if (!kKeyMajor && a.dbias_acc && orow < a.S)
      acc_row = a.dbias_acc + b * a.acc_s[0] + h * a.acc_s[1] + int64_t(orow) * a.acc_s[2];
    const bool acc_vec = (a.T & 3) == 0;
    // merged: pair j of steps (2j, 2j + 1) leaves a 128-query x 64 dq tile in TMEM; this group adds its 32 columns
    // of it to the fp32 accumulator in global memory (thread = query row)
    int next_pair = 0;
    auto drain_pair = [&](int j) -> bool {
      if (!wait_or_abort(bar(DQ_FULL), j & 1, abort_flag, a.status, 216)) return false;
      tc_fence_after_sync();
      uint32_t v[32];
      tmem_ld32(tm_dq + lane_addr + grp * 32, v);
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_FREE));
      // The accumulator is laid out so that one warp-wide reduction covers 512 contiguous bytes: per 128-query tile
      // [column half g][warp w][4-column chunk c][lane][4] holds dq[128 tile + 32 w + lane][32 g + 4 c + 0..3].
      const int64_t tile = int64_t(blockIdx.y) * (a.S / kTile) + ((s_begin + 2 * j) >> 1);
      float* dst = a.dq_acc + tile * (kTile * D) + ((grp * 4 + wq) * 8) * 128 + lane * 4;
#pragma unroll
      for (int c = 0; c < 8; ++c) red_add_v4(dst + c * 128, v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      return true;
    };

    for (int n = grp; n < n_steps && ok; n += 2) {
      const int s = n & 1;
      const int st = n % NY;
      const int r0 = (s_begin + n) * kStep;          // first streamed row of the step
      if constexpr (kMerged) {
        // group 0 takes pair j before step 2j + 4, group 1 after step 2j + 3: both between the pair's MMAs
        // (issued after the products of step 2j + 3) and the next pair's (after the products of step 2j + 5)
        if (grp == 0 && n >= 4) {
          ok = drain_pair(next_pair++);
          if (!ok) break;
        }
      }
      // keep bits over the step's 64 streamed rows
      uint32_t keep[2] = {0xffffffffu, 0xffffffffu};
      if (mbits) {
        const uint2 w = __ldg(reinterpret_cast<const uint2*>(mbits + (r0 >> 5)));
        keep[0] = w.x; keep[1] = w.y;
      }
      if (kKeyMajor) {
        // queries r0 + c: need c < S - r0, and (causal) r0 + c >= key
        const int hi = a.S - r0;
        const int lo = a.causal ? orow - r0 : 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int nh = hi - 32 * i, nl = lo - 32 * i;
          const uint32_t mh = nh >= 32 ? 0xffffffffu : (nh <= 0 ? 0u : ((1u << nh) - 1u));
          const uint32_t ml = nl <= 0 ? 0xffffffffu : (nl >= 32 ? 0u : ~((1u << nl) - 1u));
          keep[i] &= mh & ml;
        }
        if (key_dropped) keep[0] = keep[1] = 0u;
      } else {
        int n_keep = a.T - r0;
        if (a.causal) n_keep = min(n_keep, orow - r0 + 1);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int nk = n_keep - 32 * i;
          keep[i] &= nk >= 32 ? 0xffffffffu : (nk <= 0 ? 0u : ((1u << nk) - 1u));
        }
      }

      ok = wait_or_abort(bar(PROD_FULL + s), (n >> 1) & 1, abort_flag, a.status, 206);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tP1 = tmem + s * 128 + lane_addr, tP2 = tP1 + 64;
      // both products of the step: four TMEM loads in flight, one wait; handled as fp32 pairs
      float2 t[kStep / 2], dp[kStep / 2];
      {
        uint32_t raw[2 * kStep];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tmem_ld32(tP1 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[c * 32]));
          tmem_ld32(tP2 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[kStep + c * 32]));
        }
        tmem_wait_ld();
        if constexpr (kDeep) {
          // both products are in registers: the MMA issuer may recompute this stage
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(P_FREE + s));
        }
#pragma unroll
        for (int i = 0; i < kStep / 2; ++i) {
          t[i] = make_float2(__uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1]));
          dp[i] = make_float2(__uint_as_float(raw[kStep + 2 * i]), __uint_as_float(raw[kStep + 2 * i + 1]));
        }
      }
      // logits t = s * scale + bias
      if (a.bias_mode == kBiasTile && !a.bias_mma) {
        const int slot = n & 1;
        ok = wait_or_abort(bar(B_FULL + slot), (n >> 1) & 1, abort_flag, a.status, 207);
        if (!ok) break;
        const uint8_t* sl = smem + L::kBias + slot * kBoxBytes;
        if (kKeyMajor) {
          // element (query c, key r): box r / 64, row c, 16-byte chunk ((r % 64) / 8) ^ (c % 8)
          const uint8_t* colbase = sl + (r >> 6) * kYBoxBytes + (r & 7) * 2;
          const int chunk = (r & 63) >> 3;
#pragma unroll
          for (int c = 0; c < kStep / 2; ++c) {
            const uint16_t r0w = *reinterpret_cast<const uint16_t*>(colbase + (2 * c) * 128 + ((chunk ^ ((2 * c) & 7)) << 4));
            const uint16_t r1w =
                *reinterpret_cast<const uint16_t*>(colbase + (2 * c + 1) * 128 + ((chunk ^ ((2 * c + 1) & 7)) << 4));
            const float2 bv = unpack2<kBf16>(uint32_t(r0w) | (uint32_t(r1w) << 16));
            t[c] = __ffma2_rn(t[c], scale2, bv);
          }
        } else {
          const uint8_t* srow = sl + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 w = *reinterpret_cast<const uint4*>(srow + ((c ^ (r & 7)) << 4));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) t[c * 4 + e] = __ffma2_rn(t[c * 4 + e], scale2, unpack2<kBf16>(ww[e]));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_EMPTY + slot));
      } else if (a.bias_mode == kBiasKey && !kKeyMajor && !key_aug) {
        const uint4* bk = reinterpret_cast<const uint4*>(bias_key + 2 * r0);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 w = r0 + 8 * c < a.T ? __ldg(bk + c) : make_uint4(0, 0, 0, 0);   // T is a multiple of 8
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) t[c * 4 + e] = __ffma2_rn(t[c * 4 + e], scale2, unpack2<kBf16>(ww[e]));
        }
      } else if (!fold_scale) {
        const float2 own2 = make_float2(bias_own, bias_own);
#pragma unroll
        for (int c = 0; c < kStep / 2; ++c) t[c] = __ffma2_rn(t[c], scale2, own2);
      }
      // p = exp2(t log2e - lse), ds = p (dp - delta); key-major products arrive with -lse and -delta already added
      uint32_t e1[kStep / 2], e2[kStep / 2];
      const bool need_mask = __any_sync(0xffffffffu, (keep[0] & keep[1]) != 0xffffffffu);
#pragma unroll
      for (int c4 = 0; c4 < kStep / 4; ++c4) {
        const float2 nls = make_float2(-lse_row, -lse_row), ndl = make_float2(-delta_row, -delta_row);  // query-major
        float2 ds4[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = c4 * 2 + e;  // pair index: streamed rows 2c, 2c + 1
          float2 x = kKeyMajor ? __fmul2_rn(t[c], mul2) : __ffma2_rn(t[c], mul2, nls);
          if (need_mask) {
            if (!((keep[c >> 4] >> ((2 * c) & 31)) & 1u)) x.x = -INFINITY;
            if (!((keep[c >> 4] >> ((2 * c + 1) & 31)) & 1u)) x.y = -INFINITY;
          }
          const float2 p = make_float2(ex2(x.x), ex2(x.y));
          const float2 ds = kKeyMajor ? __fmul2_rn(p, dp[c]) : __fmul2_rn(p, __fadd2_rn(dp[c], ndl));
          e1[c] = pack2<kBf16>(p.x, p.y);
          e2[c] = pack2<kBf16>(ds.x, ds.y);
          if constexpr (!kKeyMajor) ds4[e] = ds;
        }
        if constexpr (!kKeyMajor) {
          // broadcast bias: this row's ds of four consecutive keys joins the fp32 sums over the broadcast axes
          if (acc_row && r0 + 4 * c4 < a.T) {
            if (acc_vec) {
              red_add_v4(acc_row + r0 + 4 * c4, __float_as_uint(ds4[0].x), __float_as_uint(ds4[0].y),
                         __float_as_uint(ds4[1].x), __float_as_uint(ds4[1].y));
            } else {   // key count not a multiple of 4: rows of the accumulator are not 16-byte aligned
              const float d4[4] = {ds4[0].x, ds4[0].y, ds4[1].x, ds4[1].y};
#pragma unroll
              for (int e4 = 0; e4 < 4; ++e4)
                if (r0 + 4 * c4 + e4 < a.T) atomicAdd(acc_row + r0 + 4 * c4 + e4, d4[e4]);
            }
          }
        }
      }
      if constexpr (kKeyMajor && !kMerged) {
        // gradient of a per-key bias: this key's ds summed over the step's queries (from the 16-bit values the
        // tensor core will consume); the running sum waits in shared memory so that it holds no register
        if (a.dbias_acc) {
          float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int c = 0; c < kStep / 2; ++c) sum2 = __fadd2_rn(sum2, unpack2<kBf16>(e2[c]));
          *key_ds_sum += sum2.x + sum2.y;
        }
      }
      if constexpr (kDeep) {
        // the E tiles of this stage are still being read by the accumulating MMAs of step n - 2
        if (n >= 2) {
          ok = wait_or_abort(bar(E_FREE + s), ((n - 2) >> 1) & 1, abort_flag, a.status, 210);
          if (!ok) break;
          tc_fence_after_sync();
        }
      }
      const uint32_t tE1 = tm_e + s * kEStage + lane_addr, tE2 = tE1 + kE2Off;
      if (kKeyMajor) tmem_st32(tE1, e1);
      if constexpr (kMerged) {
        // ds row of this key: 64 queries = 128 bytes, chunks swizzled as TMA would have written them.  The slot was
        // last read by MMAs issued before this step's products, and those have completed (PROD_FULL came after).
        uint8_t* dsrow = smem + L::kDs + (n % L::kDsSlots) * kBoxBytes + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(dsrow + ((c ^ (r & 7)) << 4)) = make_uint4(e2[c * 4], e2[c * 4 + 1], e2[c * 4 + 2], e2[c * 4 + 3]);
        fence_proxy_async_smem();
      } else {
        tmem_st32(tE2, e2);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(E_READY + s));
      if constexpr (kMerged) {
        if (grp == 1 && n >= 3) ok = drain_pair(next_pair++);
      }
      if constexpr (!kKeyMajor) {
        if (a.dbias) {
          // dbias[row, r0 .. r0+63] = ds in bias dtype (the 16-bit pairs already packed in e2).  A thread holds one
          // row, so direct stores would touch 32 lines per instruction; the warp turns its 32 x 64 tile over in
          // shared memory (two halves of 32 keys; the space of the identity tiles is free in this kernel) and
          // stores 8 rows x 64 contiguous bytes per instruction.
          uint8_t* stage = smem + L::kIdent + (warp - 4) * 2048;
          uint8_t* dbase = reinterpret_cast<uint8_t*>(a.dbias) + 2 * (b * a.dbs[0] + h * a.dbs[1] + r0);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
              *reinterpret_cast<uint4*>(stage + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4)) =
                  make_uint4(e2[half * 16 + c * 4], e2[half * 16 + c * 4 + 1], e2[half * 16 + c * 4 + 2],
                             e2[half * 16 + c * 4 + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rl = 8 * i + (lane >> 2), ch = lane & 3;
              const uint4 v = *reinterpret_cast<const uint4*>(stage + rl * 64 + ((ch ^ ((rl >> 1) & 3)) << 4));
              const int row = o0 + wq * 32 + rl;
              if (row < a.S && r0 + half * 32 + ch * 8 < a.T)
                *reinterpret_cast<uint4*>(dbase + 2 * (int64_t(row) * a.dbs[2] + half * 32 + ch * 8)) = v;
            }
            __syncwarp();
          }
        }
      }
    }

    // ---------------- epilogue ----------------
    if (!kKeyMajor && a.dbias && orow < a.S) {
      // key steps past the diagonal (causal) or past the last kept key are never visited: their dbias is exactly zero
      if (grp == 0) {
        uint8_t* dst = reinterpret_cast<uint8_t*>(a.dbias) + 2 * (b * a.dbs[0] + h * a.dbs[1] + int64_t(orow) * a.dbs[2]);
        for (int k0 = s_end * kStep; k0 < a.T; k0 += 8)
          *reinterpret_cast<uint4*>(dst + 2 * k0) = make_uint4(0, 0, 0, 0);
      }
    }
    if constexpr (kKeyMajor && !kMerged) {
      // both groups hold a partial sum of the same key (they took alternate steps)
      if (a.dbias_acc && n_steps > 0 && orow < a.T)
        atomicAdd(a.dbias_acc + b * a.acc_s[0] + h * a.acc_s[1] + orow, *key_ds_sum);
    }
    if constexpr (kMerged) {
      while (ok && next_pair < n_steps / 2) ok = drain_pair(next_pair++);
    }
    if (ok && n_steps > 0) ok = wait_or_abort(bar(ACC_DONE), 0, abort_flag, a.status, 208);
    if (ok) {
      tc_fence_after_sync();
      // key-major: group 0 writes dv (ACC1), group 1 writes dk (ACC2 * scale).
      // query-major: both groups write dq (ACC2 * scale), half of the columns each.
      const uint32_t tacc = ((kKeyMajor && grp == 0) ? tm_acc1 : tm_acc2) + lane_addr;
      const float mul = (kKeyMajor && grp == 0) ? 1.f : a.scale;
      void* outp = (kKeyMajor && grp == 0) ? a.out1 : a.out2;
      const int64_t* os = (kKeyMajor && grp == 0) ? a.o1s : a.o2s;
      uint8_t* orow_ptr = reinterpret_cast<uint8_t*>(outp) + 2 * (b * os[0] + h * os[1] + int64_t(orow) * os[2]);
      const int c_begin = kKeyMajor ? 0 : grp * (D / 64);
      const int c_end = kKeyMajor ? D / 32 : (grp + 1) * (D / 64);
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t o[32];
        if (n_steps > 0) {
          tmem_ld32(tacc + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (orow < n_owner) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2<kBf16>(__uint_as_float(o[i]) * mul, __uint_as_float(o[i + 1]) * mul);
            w.y = pack2<kBf16>(__uint_as_float(o[i + 2]) * mul, __uint_as_float(o[i + 3]) * mul);
            w.z = pack2<kBf16>(__uint_as_float(o[i + 4]) * mul, __uint_as_float(o[i + 5]) * mul);
            w.w = pack2<kBf16>(__uint_as_float(o[i + 6]) * mul, __uint_as_float(o[i + 7]) * mul);
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

template <int D, bool kBf16, bool kKeyMajor, bool kMerged = false>
int launch_one(const CUtensorMap* maps, const BwdArgs& a, int n_tiles, int bh_count, cudaStream_t st) {
  auto kernel = sdpa_bwd_tc_kernel<D, kBf16, kKeyMajor, kMerged>;
  const int smem = BwdSmem<D, kMerged>::kTotal + 1024;
  // checked and configured once per device and kernel instance (setting it again would be harmless)
  static bool ready[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev < 0 || !ready[dev]) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess || attr.numRegs != kLaunchRegs) {
      // the register hand-over inside the kernel is balanced for exactly kLaunchRegs per thread at launch
      set_error("sdpa_bwd_tc_kernel was built with %d registers per thread, expected %d", attr.numRegs, kLaunchRegs);
      return NB200_ERR_LAUNCH;
    }
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(sdpa_bwd_tc_kernel, %d): %s", smem, cudaGetErrorString(e));
      return NB200_ERR_LAUNCH;
    }
    if (dev >= 0) ready[dev] = true;
  }
  dim3 grid(n_tiles, bh_count);
  kernel<<<grid, kThreads, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], a);
  count_launch();
  return check_launch(kMerged ? "sdpa_bwd_tc_kernel<merged>"
                              : (kKeyMajor ? "sdpa_bwd_tc_kernel<key-major>" : "sdpa_bwd_tc_kernel<query-major>"));
}

// dq = scale * (fp32 sums) in the operand dtype; one thread per 8 head-dim elements (16-byte store)
template <bool kBf16>
__global__ void dq_finish_kernel(const float* __restrict__ acc, void* dq, int64_t s_b, int64_t s_h, int64_t s_row, int H,
                                 int S, int bh_begin, int64_t n_chunks, float scale) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_chunks) return;
  // consecutive threads take consecutive queries of one 8-column chunk, so the reads are contiguous
  const int64_t blk = i >> 8;               // 32 queries x 8 chunks per block of 256 threads
  const int c = int(i >> 5) & 7;            // 8 chunks of 8 elements per 64-wide row
  const int64_t row = blk * 32 + (i & 31);  // (local pair, query)
  const int q = int(row % S);
  const int bh = bh_begin + int(row / S);
  const int b = bh / H, h = bh - b * H;
  // accumulator layout (see the merged kernel): per 128-query tile [column half][warp][4-column chunk][lane][4]
  const int64_t tile = row >> 7;
  const int wq = int(row >> 5) & 3, lane = int(row) & 31, g = c >> 2, c4 = (c & 3) * 2;
  const float* src = acc + tile * (128 * 64) + (((g * 4 + wq) * 8 + c4) * 32 + lane) * 4;
  const float4 lo = __ldg(reinterpret_cast<const float4*>(src));
  const float4 hi = __ldg(reinterpret_cast<const float4*>(src + 128));
  uint4 w;
  w.x = pack2<kBf16>(lo.x * scale, lo.y * scale);
  w.y = pack2<kBf16>(lo.z * scale, lo.w * scale);
  w.z = pack2<kBf16>(hi.x * scale, hi.y * scale);
  w.w = pack2<kBf16>(hi.z * scale, hi.w * scale);
  uint8_t* dst = reinterpret_cast<uint8_t*>(dq) + 2 * (b * s_b + h * s_h + int64_t(q) * s_row + c * 8);
  *reinterpret_cast<uint4*>(dst) = w;
}

template <bool kKeyMajor>
int launch_dir(int D, bool bf16, const CUtensorMap* maps, const BwdArgs& a, int n_tiles, int bh_count, cudaStream_t st) {
  if (D == 64) return bf16 ? launch_one<64, true, kKeyMajor>(maps, a, n_tiles, bh_count, st)
                           : launch_one<64, false, kKeyMajor>(maps, a, n_tiles, bh_count, st);
  return bf16 ? launch_one<128, true, kKeyMajor>(maps, a, n_tiles, bh_count, st)
              : launch_one<128, false, kKeyMajor>(maps, a, n_tiles, bh_count, st);
}

int bias_mode_of(const Problem& pr) {
  if (!pr.bias) return kBiasNone;
  return (pr.bs[2] == 0 || pr.S == 1) ? kBiasKey : kBiasTile;
}

}  // namespace

bool bwd_supported(const Problem& pr, int dtype, int bias_dtype, const char** why) {
  // forward coverage (dtype, head dims, lengths, q/k/v/bias layout) was checked by the caller
  if (pr.scale == 0.f || !isfinite(1.f / pr.scale) || !isfinite(pr.scale)) {
    *why = "scale is zero or not finite";   // the key-major kernel divides lse by scale
    return false;
  }
  if (pr.mask_packed == 1 && !mask_key_only(pr)) {
    *why = "the mask was packed without the transposed copy the backward needs (nb200_mask_pack with_transpose = 1)";
    return false;
  }
  if (pr.dout && (!tile_map_ok(pr.dout, pr.dos[2], pr.dos[1], pr.dos[0], pr.H, pr.B, false))) {
    *why = "dout strides / alignment do not fit a TMA descriptor";
    return false;
  }
  const void* outs[3] = {pr.dq, pr.dk, pr.dv};
  const int64_t* strides[3] = {pr.dqs, pr.dks, pr.dvs};
  for (int i = 0; i < 3; ++i) {
    if (outs[i] && (reinterpret_cast<uintptr_t>(outs[i]) % 16 || strides[i][0] % 8 || strides[i][1] % 8 ||
                    strides[i][2] % 8)) {
      *why = "dq/dk/dv are not 16-byte aligned";
      return false;
    }
  }
  if (pr.dbias) {
    // A bias of full extent gets its gradient as 16-byte row segments in bias dtype, straight from the kernel; a
    // broadcast bias is summed in fp32 (an accumulator of the bias' own extent in the workspace) and cast by
    // dbias_finish_kernel, which takes any dbias layout.
    const int64_t full[4] = {pr.B, pr.H, pr.S, pr.T};
    bool broadcast = false;
    for (int ax = 0; ax < 4; ++ax) broadcast = broadcast || (pr.bs[ax] == 0 && full[ax] > 1);
    if (!broadcast && (pr.dbs[3] != 1 || reinterpret_cast<uintptr_t>(pr.dbias) % 16 || pr.dbs[0] % 8 ||
                       pr.dbs[1] % 8 || pr.dbs[2] % 8)) {
      *why = "dbias layout is not 16-byte aligned with a unit key stride";
      return false;
    }
  }
  (void)dtype;
  (void)bias_dtype;
  return true;
}

namespace {
// One kernel for dq, dk and dv (head dim 64, no bias gradient): the key-major kernel also forms ds K per pair of
// steps and adds it to an fp32 copy of dq, which a last kernel scales and casts.
bool use_merged(const Problem& pr) { return pr.D == 64 && !pr.want_dbias && pr.S % kTile == 0; }
size_t round_up_256(size_t x) { return (x + 255) / 256 * 256; }

// Head dim 128: the one-kernel backward of sdpa_tc_bwd_d128.cu (NB200_BWD_D128_ONEPASS=0 in the environment keeps
// the query-major + key-major pair, for comparisons).
bool use_d128(const Problem& pr, int dtype) {
  static const bool enabled = [] {
    const char* e = getenv("NB200_BWD_D128_ONEPASS");
    return !(e && e[0] == '0');
  }();
  if (!enabled || pr.D != 128) return false;
  const int mode = bias_mode_of(pr);
  float hi = 0.f, lo = 0.f;
  const bool bias_mma = mode == kBiasTile && split_inv_scale(pr.scale, dtype == NB200_BF16, &hi, &lo);
  return d128_merged_supported(pr, mode, bias_mma);
}
}  // namespace

size_t bwd_workspace_bytes(const Problem& pr, int dtype, int) {
  size_t mask_ws = 0;
  mask_plan_for_pass(pr, true, &mask_ws);
  size_t bytes = round_up_256(mask_ws);
  if (use_merged(pr)) bytes += sizeof(float) * size_t(pr.bh_count) * pr.S * pr.D;
  else if (use_d128(pr, dtype)) bytes += d128_acc_bytes(pr);
  return bytes;
}

int launch_bwd(const Problem& pr, int dtype, int bias_dtype, void* ws, size_t ws_bytes, int ld_rows, cudaStream_t stream) {
  (void)bias_dtype;
  const char* why = "";
  const bool key_only = mask_key_only(pr);
  size_t mask_ws = 0;
  const MaskPackPlan mp = mask_plan_for_pass(pr, true, &mask_ws);
  mask_ws = round_up_256(mask_ws);
  const bool merged = use_merged(pr);
  const bool d128 = !merged && use_d128(pr, dtype);
  const size_t acc_bytes = merged ? sizeof(float) * size_t(pr.bh_count) * pr.S * pr.D : (d128 ? d128_acc_bytes(pr) : 0);
  if (mask_ws + acc_bytes > ws_bytes) {
    set_error("tensor-core backward needs %zu workspace bytes", mask_ws + acc_bytes);
    return NB200_ERR_WORKSPACE;
  }
  BwdArgs a{};
  if (int rc = launch_mask_pack(pr, mp, ws, &a.mask, stream)) return rc;
  a.mask_key_only = key_only ? 1 : 0;
  a.H = pr.H; a.S = pr.S; a.T = pr.T; a.bh_begin = pr.bh_begin;
  a.causal = pr.causal; a.scale = pr.scale;
  a.bias_mode = bias_mode_of(pr);
  a.bias_mma = 0;
  a.inv_scale_hi = a.inv_scale_lo = 0.f;
  if (a.bias_mode == kBiasTile && split_inv_scale(pr.scale, dtype == NB200_BF16, &a.inv_scale_hi, &a.inv_scale_lo))
    a.bias_mma = 1;
  a.bias_b_mul = (pr.B > 1 && pr.bs[0] != 0) ? 1 : 0;
  a.bias_h_mul = (pr.H > 1 && pr.bs[1] != 0) ? 1 : 0;
  a.bias = pr.bias; a.bias_bs = pr.bs[0]; a.bias_hs = pr.bs[1];
  a.lse = pr.lse; a.delta = pr.delta; a.ld_rows = ld_rows;
  a.status = device_status_word();
  if (!a.status) { set_error("device status word is unavailable"); return NB200_ERR_LAUNCH; }

  // tensor maps: 128-row boxes for owner operands, 64-row boxes for streamed ones
  CUtensorMap q128, k128, v128, g128, q64, k64, v64, g64, bias_q, bias_k;
  bool ok = make_tile_map(&q128, pr.q, pr.S, pr.D, pr.H, pr.B, pr.qs[2], pr.qs[1], pr.qs[0], kTile, &why) &&
            make_tile_map(&g128, pr.dout, pr.S, pr.D, pr.H, pr.B, pr.dos[2], pr.dos[1], pr.dos[0], kTile, &why) &&
            make_tile_map(&k128, pr.k, pr.T, pr.D, pr.H, pr.B, pr.ks[2], pr.ks[1], pr.ks[0], kTile, &why) &&
            make_tile_map(&v128, pr.v, pr.T, pr.D, pr.H, pr.B, pr.vs[2], pr.vs[1], pr.vs[0], kTile, &why) &&
            make_tile_map(&q64, pr.q, pr.S, pr.D, pr.H, pr.B, pr.qs[2], pr.qs[1], pr.qs[0], kStep, &why) &&
            make_tile_map(&g64, pr.dout, pr.S, pr.D, pr.H, pr.B, pr.dos[2], pr.dos[1], pr.dos[0], kStep, &why) &&
            make_tile_map(&k64, pr.k, pr.T, pr.D, pr.H, pr.B, pr.ks[2], pr.ks[1], pr.ks[0], kStep, &why) &&
            make_tile_map(&v64, pr.v, pr.T, pr.D, pr.H, pr.B, pr.vs[2], pr.vs[1], pr.vs[0], kStep, &why);
  bias_q = q128;
  bias_k = q128;
  if (ok && a.bias_mode == kBiasTile)
    ok = make_tile_map(&bias_q, pr.bias, pr.S, pr.T, pr.H, pr.B, pr.bs[2], pr.bs[1], pr.bs[0], kTile, &why) &&
         make_tile_map(&bias_k, pr.bias, pr.S, pr.T, pr.H, pr.B, pr.bs[2], pr.bs[1], pr.bs[0], kStep, &why);
  if (!ok) { set_error("tensor map: %s", why); return NB200_ERR_LAUNCH; }
  const bool bf16 = dtype == NB200_BF16;

  if (merged) {
    BwdArgs ak = a;
    ak.dq_acc = reinterpret_cast<float*>(static_cast<char*>(ws) + mask_ws);
    cudaError_t e = cudaMemsetAsync(ak.dq_acc, 0, acc_bytes, stream);
    if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return NB200_ERR_LAUNCH; }
    ak.out1 = pr.dv;
    ak.out2 = pr.dk;
    for (int i = 0; i < 3; ++i) { ak.o1s[i] = pr.dvs[i]; ak.o2s[i] = pr.dks[i]; }
    const CUtensorMap maps[5] = {k128, v128, q64, g64, bias_k};
    const int rc = bf16 ? launch_one<64, true, true, true>(maps, ak, (pr.T + kTile - 1) / kTile, pr.bh_count, stream)
                        : launch_one<64, false, true, true>(maps, ak, (pr.T + kTile - 1) / kTile, pr.bh_count, stream);
    if (rc) return rc;
    const int64_t n_chunks = int64_t(pr.bh_count) * pr.S * 8;
    const int blocks = int((n_chunks + 255) / 256);
    if (bf16)
      dq_finish_kernel<true><<<blocks, 256, 0, stream>>>(ak.dq_acc, pr.dq, pr.dqs[0], pr.dqs[1], pr.dqs[2], pr.H, pr.S,
                                                         pr.bh_begin, n_chunks, pr.scale);
    else
      dq_finish_kernel<false><<<blocks, 256, 0, stream>>>(ak.dq_acc, pr.dq, pr.dqs[0], pr.dqs[1], pr.dqs[2], pr.H, pr.S,
                                                          pr.bh_begin, n_chunks, pr.scale);
    count_launch();
    return check_launch("dq_finish_kernel");
  }
  if (d128) {
    // one kernel for dq, dk, dv (and the dbias tiles): fp32 dq sums in the workspace, zero on entry
    BwdArgs ak = a;
    ak.dq_acc = reinterpret_cast<float*>(static_cast<char*>(ws) + mask_ws);
    ak.acc_rows = (pr.S + kStep - 1) / kStep * kStep;
    cudaError_t e = cudaMemsetAsync(ak.dq_acc, 0, acc_bytes, stream);
    if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return NB200_ERR_LAUNCH; }
    ak.out1 = pr.dv;
    ak.out2 = pr.dk;
    for (int i = 0; i < 3; ++i) { ak.o1s[i] = pr.dvs[i]; ak.o2s[i] = pr.dks[i]; }
    D128Maps maps{k128, v128, q64, g64, bias_k, q64};
    if (pr.dbias) {
      ak.dbias = pr.dbias;
      for (int i = 0; i < 4; ++i) ak.dbs[i] = pr.dbs[i];
      if (!make_tile_map(&maps.dbias, pr.dbias, pr.S, pr.T, pr.H, pr.B, pr.dbs[2], pr.dbs[1], pr.dbs[0], kStep, &why)) {
        set_error("dbias tensor map: %s", why);
        return NB200_ERR_LAUNCH;
      }
      if (pr.causal || key_only) {
        // query / key ranges the kernel never visits (above the diagonal, past the last kept key) get exact zeros
        e = cudaMemsetAsync(pr.dbias, 0, size_t(pr.B) * pr.H * pr.S * size_t(pr.dbs[2]) * 2, stream);
        if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return NB200_ERR_LAUNCH; }
      }
    }
    if (int rc = launch_bwd_d128(maps, ak, bf16, a.bias_mode == kBiasTile, (pr.T + kTile - 1) / kTile, pr.bh_count, stream))
      return rc;
    return launch_dq_finish_d128(pr, ak.dq_acc, ak.acc_rows, bf16, stream);
  }
  // query-major: dq (+ dbias)
  {
    BwdArgs aq = a;
    // query-major reads the bias row-wise with 16-byte loads, which is cheap; the tensor-core add only pays in
    // the key-major kernel, where the bias would be read column-wise, two bytes at a time
    aq.bias_mma = 0;
    aq.key_aug = (a.bias_mode != kBiasTile && (a.bias_mode == kBiasKey || key_only) && pr.scale > 0.f) ? 1 : 0;
    aq.out2 = pr.dq;
    for (int i = 0; i < 3; ++i) aq.o2s[i] = pr.dqs[i];
    if (pr.dbias_accum) {
      // broadcast bias: fp32 sums; the per-key case is summed by the key-major kernel below
      if (a.bias_mode == kBiasTile) {
        aq.dbias_acc = pr.dbias_accum;
        for (int i = 0; i < 3; ++i) aq.acc_s[i] = pr.dbs[i];
      }
    } else {
      aq.dbias = pr.dbias;
      for (int i = 0; i < 4; ++i) aq.dbs[i] = pr.dbs[i];
    }
    const CUtensorMap maps[5] = {q128, g128, k64, v64, bias_q};
    if (int rc = launch_dir<false>(pr.D, bf16, maps, aq, (pr.S + kTile - 1) / kTile, pr.bh_count, stream)) return rc;
  }
  // key-major: dk, dv
  {
    BwdArgs ak = a;
    ak.out1 = pr.dv;
    ak.out2 = pr.dk;
    for (int i = 0; i < 3; ++i) { ak.o1s[i] = pr.dvs[i]; ak.o2s[i] = pr.dks[i]; }
    if (pr.dbias_accum && a.bias_mode == kBiasKey) {
      ak.dbias_acc = pr.dbias_accum;
      for (int i = 0; i < 3; ++i) ak.acc_s[i] = pr.dbs[i];
    }
    const CUtensorMap maps[5] = {k128, v128, q64, g64, bias_k};
    if (int rc = launch_dir<true>(pr.D, bf16, maps, ak, (pr.T + kTile - 1) / kTile, pr.bh_count, stream)) return rc;
  }
  return NB200_OK;
}

}  // namespace tc
}  // namespace nb200
