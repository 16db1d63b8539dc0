// Forward flash attention for sm_100a: TMA -> shared memory -> tcgen05.mma with
// TMEM accumulators, fp32 online softmax in registers.
//
// Replaces the reference's forward kernel `_fwd_kernel` and its launch glue
// (reference src/nitrix/_kernels/cuda/attention.py:85-156, :159-264): same
// recurrence (running max m, running sum l, lse = m + log2 l in base 2, causal
// key tiles past the diagonal skipped) on 128 x 128 tiles instead of 32 x 32.
//
// PERSISTENT kernel: one CTA per SM walks a static list of work items; an item
// is TWO 128-row query tiles of one (batch, head), for which the key tiles are
// streamed once.  Barriers, TMEM and tensor-map prefetch are set up once per
// CTA, and the next item's loads and first MMAs run under the current item's
// epilogue.  Items are ordered heaviest first (causal) and, when the bias is
// shared over the batch, batch-fastest so concurrent CTAs hit the same bias
// tiles in L2.  Twelve warps:
//   warp 0      TMA producer for Q (per item) and the K / V rings
//   warp 1      TMA producer for the bias ring (128 x 64 slots)
//   warp 2      issues tcgen05.mma for query tile 0 (one elected lane)
//   warp 3      issues tcgen05.mma for query tile 1; owns the TMEM allocation
//   warps 4-7   softmax of query tile 0 (one row per thread)
//   warps 8-11  softmax of query tile 1
// TMEM (512 columns).  D = 128: [0,128) S0, [128,256) S1, then O0, O1.  There is no
// room for separate P tiles, so a key tile is taken as two halves of 64 keys: each
// half has its own 64-column S buffer and its P (16-bit, 32 columns) overwrites
// that buffer.  QK(half u+1) is issued right after PV(half u-1) and runs while the
// softmax warps work on half u; only a rescale of O waits for the previous PV.
// Both query tiles' soft-maxes then run at the same time and share the special-
// function unit, so a quarter of the exponentials are computed on the FMA pipe.
// D = 64 leaves room for separate P tiles ([256,384)), so QK(j+1) is issued as
// soon as softmax(j) has read S out and runs underneath it.
// P feeds the PV MMA as the TMEM A operand; V is consumed from shared memory as
// an MN-major B operand, so nothing is transposed or staged through shared memory.
// All waits are bounded (sdpa_tc_common.cuh).
#include "sdpa_tc_common.cuh"
#include "sdpa_tc_fwd.cuh"

namespace nb200 {
namespace tc {

using namespace sm100;

namespace {

constexpr int kThreads = 384;
// register split after start-up (setmaxnreg): the softmax warps hold a whole score row
constexpr int kProducerRegs = 56;
constexpr int kSoftmaxRegs = 216;
#ifndef NB200_POLY_PERIOD
#define NB200_POLY_PERIOD 4
#endif
// D = 128: one pair in this many computes 2^x without the special-function unit (0: none).  There the two query
// tiles' soft-maxes run at the same time and share the unit; at D = 64 the extra arithmetic costs more than it saves.
constexpr int kPolyPeriod = NB200_POLY_PERIOD;
// setmaxnreg.inc blocks (without bound) until the CTA's OWN pool -- the registers it was launched with, here
// kLaunchRegs per thread -- holds enough released registers, so the hand-over must balance at compile time.
constexpr int kLaunchRegs = 168;  // what __launch_bounds__(384, 1) gives: 65536 / 384 rounded down to a multiple of 8
static_assert((kLaunchRegs - kProducerRegs) * 128 >= (kSoftmaxRegs - kLaunchRegs) * 256,
              "softmax warps would wait forever for registers the producer warps never release");

#ifdef NB200_PROBE
// Development aid (not compiled into the library): cycles one softmax warp spends in each phase of its tiles.
__device__ unsigned long long g_fprobe[16];
#define FPROBE_DECL long long fpt_ = clock64(); const bool fprobe_ = blockIdx.x == 5 && warp == 4 && lane == 0; unsigned fp_[12] = {}
#define FPROBE(i) do { const long long now_ = clock64(); fp_[i] += unsigned(now_ - fpt_); fpt_ = now_; } while (0)
#define FPROBE_FLUSH do { if (fprobe_) for (int i_ = 0; i_ < 12; ++i_) g_fprobe[i_] += fp_[i_]; } while (0)
#define FPROBE_TILES(n) do { fp_[11] += unsigned(n); } while (0)
#else
#define FPROBE_DECL
#define FPROBE(i)
#define FPROBE_FLUSH
#define FPROBE_TILES(n)
#endif

template <int D, bool kTileBias>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;        // one Q / K / V tile
  // K and V ring depth.  A TMA tile takes 1-2 us from L2 / HBM while a key tile is consumed in well under
  // 1 us, so two stages leave the MMAs waiting for loads; D = 64 tiles are small enough for four.
  // With bias tiles D = 64 keeps three stages and five bias slots (a round consumes four); without them five stages.
  static constexpr int kStages = D == 64 ? (kTileBias ? 3 : 5) : 2;
  static constexpr int kBiasSlots = kTileBias ? (D == 64 ? 5 : 2) : 1;      // 16 KB slots
  // D = 64: hi * I and lo * I (64 x 64 each), second operand of the MMAs that add a bias tile to the scores
  static constexpr int kIdentBytes = (D == 64 && kTileBias) ? 2 * 64 * 128 : 0;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kBias = kV + kStages * kTileBytes;
  static constexpr int kIdent = kBias + kBiasSlots * kBoxBytes;
  static constexpr int kBars = kIdent + kIdentBytes;
  // q_full[2] q_empty[2] k_full[S] k_empty[S] v_full[S] v_empty[S] s_full[2] p_ready[2] o_done[2] o_free[2]
  // s_free[2] pv_done[2] bias_full[2][slots] bias_empty[slots]
  // Without bias tiles the (single) bias slot holds the operands of the per-key add: the weight tile (128 rows x 16,
  // no swizzle, 4 KB) and a ring of three 128-key x 16 tiles (4 KB each).
  static constexpr int kAugSlots = 3;
  static constexpr int kAugTileBytes = (kTile / 8) * 256;
  static constexpr int kNumBars = 4 + 4 * kStages + 16 + 3 * kBiasSlots + 2 * kAugSlots;
  static constexpr int kMisc = kBars + 8 * kNumBars;      // tmem base (4 B) + abort flag (4 B)
  static constexpr int kOrder = kMisc + 16;               // batch indices by kept length (item order 3), 16-bit each
  static constexpr int kTotal = kOrder + 2 * kThreads;
};

// One work item: two query tiles of one (batch, head).
struct Item {
  int b, h, q0;
  int nt[2], nt_max;
};

__device__ __forceinline__ Item decode_item(const FwdArgs& a, int item, const uint16_t* order) {
  Item it;
  // CTAs that run side by side take consecutive items, so the order decides what they share in L2 and how evenly
  // the work is spread.
  int rank;
  if (a.head_major == 1) {
    const int per_head = a.n_qblocks * a.B;
    it.h = item / per_head;
    const int rem = item - it.h * per_head;
    rank = rem / a.B;
    it.b = rem - rank * a.B;
  } else if (a.head_major == 2) {
    // Items sorted by weight (query block, heaviest causal block first), then head, batch fastest, and dealt to the
    // CTAs in rows of gridDim.x that alternate direction ("snake"): CTA c takes sorted positions c, 2G - 1 - c,
    // 2G + c, ...  With causal weights 16, 14, ..., 2 rounds a plain round-robin over a head-major order left the
    // busiest CTA 22 % above the mean (C2); this order leaves 3 %.  Neighbouring CTAs still share a head's bias
    // tiles (same head and query block, other batches).
    const int G = int(gridDim.x), n_items = a.n_qblocks * a.bh_count;
    const int row = item / G, col = item - row * G;
    const bool full_row = (row + 1) * G <= n_items;
    const int pos = row * G + ((row & 1) && full_row ? G - 1 - col : col);
    const int per_rank = a.bh_count;          // = B * H here
    rank = pos / per_rank;
    const int rem = pos - rank * per_rank;
    it.h = rem / a.B;
    it.b = rem - it.h * a.B;
  } else if (a.head_major == 3) {
    // Key-padding masks: an item's work is proportional to its batch element's kept length.  Items sorted by that
    // length (longest first; `order` = batch indices by descending length), then head, then query block, and dealt
    // in rows of alternating direction as above.  Neighbours share one (batch, head) pair's K / V.
    const int G = int(gridDim.x), n_items = a.n_qblocks * a.bh_count;
    const int row = item / G, col = item - row * G;
    const bool full_row = (row + 1) * G <= n_items;
    const int pos = row * G + ((row & 1) && full_row ? G - 1 - col : col);
    const int per_batch = a.H * a.n_qblocks;
    const int rb = pos / per_batch;
    const int rem = pos - rb * per_batch;
    it.b = order[rb];
    it.h = rem / a.n_qblocks;
    rank = rem - it.h * a.n_qblocks;
  } else {  // a partial (batch, head) range: keep each pair's query blocks together
    const int bh = a.bh_begin + item / a.n_qblocks;
    rank = item % a.n_qblocks;
    it.b = bh / a.H;
    it.h = bh - it.b * a.H;
  }
  const int qblock = a.causal ? (a.n_qblocks - 1 - rank) : rank;
  it.q0 = qblock * 2 * kTile;
  // key-only mask (key padding): tiles past the last kept key are skipped; one tile is always visited
  // so that a batch with no kept key still produces its (NaN) rows
  const int kept = kept_key_length(a.mask, it.b, it.h, a.T);
  const int n_kt = max(1, (kept + kTile - 1) / kTile);
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int q0g = it.q0 + g * kTile;
    it.nt[g] = q0g >= a.S ? 0 : (a.causal ? min(n_kt, q0g / kTile + 1) : n_kt);
  }
  it.nt_max = max(it.nt[0], it.nt[1]);
  return it;
}

template <int D, bool kBf16, bool kTileBias>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_bias,
                   const FwdArgs a) {
  using L = FwdSmem<D, kTileBias>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the swizzled tiles need a 1024-byte aligned base; the launch reserves the slack for rounding up
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (smem + L::kTotal > smem_raw + a.smem_bytes) {  // never expected; refuse rather than overrun
    if (threadIdx.x == 0) atomicExch(a.status, 199);
    return;
  }
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);

  auto bar = [&](int i) { return smem_u32(bars + i); };
  constexpr int Q_FULL = 0, Q_EMPTY = 2, K_FULL = 4, K_EMPTY = K_FULL + kStages, V_FULL = K_EMPTY + kStages,
                V_EMPTY = V_FULL + kStages, S_FULL = V_EMPTY + kStages, P_READY = S_FULL + 4, O_DONE = P_READY + 4,
                O_FREE = O_DONE + 2, S_FREE = O_FREE + 2, PV_DONE = S_FREE + 2, B_FULL = PV_DONE + 2,
                B_EMPTY = B_FULL + 2 * L::kBiasSlots, AUG_FULL = B_EMPTY + L::kBiasSlots, AUG_FREE = AUG_FULL + L::kAugSlots;
  // D = 128 fills TMEM (2 x 128 S + 2 x 128 O), so P must overwrite S: a key tile is taken as two halves of 64
  //   keys, each with its own 64-column S buffer and P written over that buffer, and the scores of the next half
  //   are computed while the softmax warps work on the current one.
  // D = 64 leaves room for separate P tiles, so the next score MMA can run under the current softmax.
  constexpr bool kAlias = D == 128;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = a.n_qblocks * a.bh_count;

  if (threadIdx.x == 0) {
    for (int i = 0; i < L::kNumBars; ++i) {
      uint32_t count = 1;
      if (i >= P_READY && i < P_READY + 4) count = 4;                       // one lane per softmax warp of the tile
      if (i >= K_EMPTY && i < K_EMPTY + kStages) count = 2;    // one arrival per MMA issuer
      if (i >= V_EMPTY && i < V_EMPTY + kStages) count = 2;
      if (i >= O_FREE && i < O_FREE + 2) count = 4;                         // one lane per softmax warp of the tile
      if (i >= S_FREE && i < S_FREE + 2) count = 4;
      if (i >= B_EMPTY && i < B_EMPTY + L::kBiasSlots) count = a.bias_mma ? 1 : 4;   // MMA issuer or the tile's warps
      if (i >= AUG_FREE && i < AUG_FREE + L::kAugSlots) count = 2;        // one arrival per MMA issuer
      mbar_init(bar(i), count);
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if constexpr (D == 64 && kTileBias) {
    if (a.bias_mma) {
      // two 64 x 64 K-major, 128-byte-swizzled tiles: tile 0 = hi * I, tile 1 = lo * I
      uint4* ident = reinterpret_cast<uint4*>(smem + L::kIdent);
      for (int idx = threadIdx.x; idx < 2 * 64 * 8; idx += kThreads) {   // one 16-byte chunk each
        const int tile = idx / (64 * 8), rem = idx - tile * 64 * 8;
        const int row = rem >> 3, chunk = (rem & 7) ^ (row & 7);           // logical chunk stored at this slot
        const int col0 = chunk * 8;
        const float val = tile == 0 ? a.inv_scale_hi : a.inv_scale_lo;
        const uint16_t one = kBf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (row >= col0 && row < col0 + 8) w[(row - col0) >> 1] = uint32_t(one) << (((row - col0) & 1) * 16);
        ident[idx] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async_smem();   // written by threads, read by the tensor core
    }
  }
  if constexpr (!kTileBias) {
    if (a.key_mma) {
      // weight rows (w0, w1, w2, 0, ...): bf16 (1, 1, 1); fp16 (256, 1, 2^-8) to cover magnitudes up to 1.6e7
      uint4* wt = reinterpret_cast<uint4*>(smem + L::kBias);
      const uint32_t w01 = kBf16 ? 0x3F803F80u : 0x3C005C00u;
      const uint32_t w2 = kBf16 ? 0x00003F80u : 0x00001C00u;
      for (int idx = threadIdx.x; idx < L::kAugTileBytes / 16; idx += kThreads)
        wt[idx] = (idx & 8) ? make_uint4(0, 0, 0, 0) : make_uint4(w01, w2, 0, 0);
      uint4* aug = reinterpret_cast<uint4*>(smem + L::kBias + L::kAugTileBytes);
      for (int idx = threadIdx.x; idx < L::kAugSlots * L::kAugTileBytes / 16; idx += kThreads) aug[idx] = make_uint4(0, 0, 0, 0);
      fence_proxy_async_smem();
    }
  }
  const uint16_t* const order = reinterpret_cast<const uint16_t*>(smem + L::kOrder);
  if (a.head_major == 3 && int(threadIdx.x) < a.B) {
    // rank of this batch element among the kept lengths (ties by index): B <= kThreads loads per thread, once per CTA
    const int mine = a.mask.kv_len[threadIdx.x * a.mask.len_b_stride];
    int r = 0;
    for (int j = 0; j < a.B; ++j) {
      const int other = __ldg(a.mask.kv_len + j * a.mask.len_b_stride);
      r += (other > mine || (other == mine && j < int(threadIdx.x))) ? 1 : 0;
    }
    reinterpret_cast<uint16_t*>(smem + L::kOrder)[r] = uint16_t(threadIdx.x);
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
  const uint32_t tm_P[2] = {kAlias ? tmem : tmem + 256, kAlias ? tmem + 128 : tmem + 320};
  const uint32_t tm_O[2] = {kAlias ? tmem + 256 : tmem + 384, kAlias ? tmem + 256 + D : tmem + 384 + D};

  // Phase bookkeeping across items (every role derives the same numbers from the same item list):
  //   kv   key tiles streamed so far            -> ring stage kv % kStages, phase (kv / kStages) & 1
  //   tc_g tiles query tile g has processed     -> phase of s_full / p_ready / s_free / pv_done
  //   oc_g items in which query tile g was live -> phase of q_full / q_empty / o_done / o_free
  if (warp < 4) {
  reg_dealloc<kProducerRegs>();
  if (warp == 0) {
    // ---------------- Q / K / V producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      int kv = 0, oc[2] = {0, 0};
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const Item it = decode_item(a, item, order);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          if (it.nt[g] == 0) continue;
          // the previous item's last score MMA must have finished reading Q_g
          if (oc[g] > 0) ok = ok && wait_or_abort(bar(Q_EMPTY + g), (oc[g] - 1) & 1, abort_flag, a.status, 100);
          if (!ok) break;
          mbar_expect_tx(bar(Q_FULL + g), L::kTileBytes);
#pragma unroll
          for (int x = 0; x < D / 64; ++x)
            tma_load_4d(sbase + L::kQ + g * L::kTileBytes + x * kBoxBytes, &tm_q, bar(Q_FULL + g), x * 64,
                        it.q0 + g * kTile, it.h, it.b);
          ++oc[g];
        }
        for (int j = 0; j < it.nt_max && ok; ++j, ++kv) {
          const int st = kv % kStages;
          const uint32_t ph = (kv / kStages) & 1;
          if (!wait_or_abort(bar(K_EMPTY + st), ph ^ 1, abort_flag, a.status, 101)) { ok = false; break; }
          mbar_expect_tx(bar(K_FULL + st), L::kTileBytes);
#pragma unroll
          for (int x = 0; x < D / 64; ++x)
            tma_load_4d(sbase + L::kK + st * L::kTileBytes + x * kBoxBytes, &tm_k, bar(K_FULL + st), x * 64,
                        j * kTile, it.h, it.b);
          if (!wait_or_abort(bar(V_EMPTY + st), ph ^ 1, abort_flag, a.status, 102)) { ok = false; break; }
          mbar_expect_tx(bar(V_FULL + st), L::kTileBytes);
#pragma unroll
          for (int x = 0; x < D / 64; ++x)
            tma_load_4d(sbase + L::kV + st * L::kTileBytes + x * kBoxBytes, &tm_v, bar(V_FULL + st), x * 64,
                        j * kTile, it.h, it.b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- bias producer ----------------
    if constexpr (!kTileBias) {
      if (a.key_mma) {
        // per-key addends of each streamed key tile as an MMA operand: lane -> keys lane, lane + 32, ...
        const float inv_scale = 1.f / a.scale;
        int kv = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
          const Item it = decode_item(a, item, order);
          const uint16_t* bk = a.bias_mode == kBiasKey
                                   ? reinterpret_cast<const uint16_t*>(a.bias) + (it.b * a.bias_bs + it.h * a.bias_hs)
                                   : nullptr;
          const uint32_t* mk = a.mask.kv_len ? a.mask.rows + it.b * a.mask.b_stride + it.h * a.mask.h_stride : nullptr;
          for (int j = 0; j < it.nt_max && ok; ++j, ++kv) {
            const int slot = kv % L::kAugSlots;
            if (kv >= L::kAugSlots)
              ok = wait_or_abort(bar(AUG_FREE + slot), ((kv / L::kAugSlots) - 1) & 1, abort_flag, a.status, 117);
            if (!ok) break;
            uint8_t* ctile = smem + L::kBias + L::kAugTileBytes * (1 + slot);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int kl = lane + 32 * e, key = j * kTile + kl;
              float c = 0.f;
              if (key >= a.T) {
                c = -INFINITY;   // past the last key (the tile is padded with zero rows)
              } else if (bk) {
                const uint16_t raw = __ldg(bk + key);
                c = (kBf16 ? __uint_as_float(uint32_t(raw) << 16) : __half2float(__ushort_as_half(raw))) * inv_scale;
              }
              if (mk && key < a.T && !((__ldg(mk + (key >> 5)) >> (key & 31)) & 1u)) c = -INFINITY;
              uint32_t h[3] = {0u, 0u, 0u};
              float rem = c;
#pragma unroll
              for (int t3 = 0; t3 < 3; ++t3) {
                const float w = kBf16 ? 1.f : (t3 == 0 ? 256.f : (t3 == 1 ? 1.f : 0.00390625f));
                const float v = rem * (1.f / w);
                float back;
                if constexpr (kBf16) {
                  const __nv_bfloat16 hv = __float2bfloat16_rn(v);
                  h[t3] = __bfloat16_as_ushort(hv);
                  back = __bfloat162float(hv);
                } else {
                  const __half hv = __float2half_rn(v);
                  h[t3] = __half_as_ushort(hv);
                  back = __half2float(hv);
                }
                if (!(fabsf(back) < INFINITY)) break;   // an infinite (or NaN) term carries the value alone
                rem = fmaf(-back, w, rem);
              }
              *reinterpret_cast<uint4*>(ctile + (kl >> 3) * 256 + (kl & 7) * 16) = make_uint4(h[0] | (h[1] << 16), h[2], 0u, 0u);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(AUG_FULL + slot));
          }
        }
      }
    }
    if (a.bias_mode == kBiasTile && elect_one()) {
      tma_prefetch_desc(&tm_bias);
      int seq = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const Item it = decode_item(a, item, order);
        // slots are filled in the order: for each key tile, for each live query tile, column half 0 then 1
        for (int j = 0; j < it.nt_max && ok; ++j) {
          for (int g = 0; g < 2 && ok; ++g) {
            if (j >= it.nt[g]) continue;
            for (int half = 0; half < 2; ++half, ++seq) {
              const int slot = seq % L::kBiasSlots;
              const uint32_t ph = (seq / L::kBiasSlots) & 1;
              if (!wait_or_abort(bar(B_EMPTY + slot), ph ^ 1, abort_flag, a.status, 103)) { ok = false; break; }
              // the slots are shared by both query tiles, but each tile has its own "full" barriers:
              // a waiter must see consecutive phases of a barrier, and the tiles alternate on a slot
              const uint32_t full = bar(B_FULL + g * L::kBiasSlots + slot);
              mbar_expect_tx(full, kBoxBytes);
              tma_load_4d(sbase + L::kBias + slot * kBoxBytes, &tm_bias, full, j * kTile + half * kSlotCols,
                          it.q0 + g * kTile, it.h * a.bias_h_mul, it.b * a.bias_b_mul);
            }
          }
        }
      }
    }
  } else {
    // ---------------- MMA issuers ----------------
    // Warp 2 issues the chain of query tile 0, warp 3 that of query tile 1; a tile's next score MMA runs under
    // its own softmax, so the two chains are independent (one thread issuing both was measured slower at both
    // head sizes: it needs some 50 cycles per instruction and a wait for one tile holds up the other).
    // An issuer observes every key tile of the rings, also those its query tile skips, and commits once per
    // tile to the "empty" barriers (with nothing outstanding the arrival is immediate): one arrival per
    // issuer per phase.
    const int g_begin = warp - 2, g_end = warp - 1;
    if (elect_one()) {
      constexpr uint32_t idesc_qk = make_idesc(kBf16, kTile, kTile, false, false);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, kTile, D, false, true);
      // descriptors are built once; a tile offset only moves the 16-byte start-address field
      uint64_t qdesc[2], kdesc[kStages], vdesc[kStages];
#pragma unroll
      for (int g = 0; g < 2; ++g) qdesc[g] = make_smem_desc(sbase + L::kQ + g * L::kTileBytes, 16, 1024);
#pragma unroll
      for (int s = 0; s < kStages; ++s) {
        kdesc[s] = make_smem_desc(sbase + L::kK + s * L::kTileBytes, 16, 1024);
        vdesc[s] = make_smem_desc(sbase + L::kV + s * L::kTileBytes, kBoxBytes, 1024);
      }
      bool ok = true;
      int kv = 0, tc[2] = {0, 0}, oc[2] = {0, 0};
      int seq_base = 0;            // bias slots filled before this item
      uint32_t bias_phase = 0;     // bit s = parity of this issuer's next wait on its tile's "full" barrier of slot s
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const Item it = decode_item(a, item, order);
        if constexpr (kAlias) {
          // D = 128: key tiles are taken in two halves of 64 keys.  A query tile's S region holds two 64-column
          // buffers, one per half, and P (16-bit, 32 columns) is written over its own buffer, so the scores of the
          // next half are computed while the softmax warps work on the current one.  Round u (half u = 2 j + hf):
          // the score MMAs of half u of this issuer's query tile, then the output MMAs of half u - 1.  Everything that
          // touches a query tile's buffers is issued by this one thread and the tensor core runs it in order: the
          // scores of half u follow the output MMA of half u - 2, which read P out of the same buffer.
          constexpr uint32_t idesc_qk64 = make_idesc(kBf16, kTile, kTile / 2, false, false);
          const int n_sub = 2 * it.nt_max;
          for (int u = 0; u <= n_sub && ok; ++u) {
            const int j = u >> 1, hf = u & 1;                 // scores: tile j, half hf
            const int jp = (u - 1) >> 1, hp = (u - 1) & 1;    // outputs: tile jp, half hp
            const int st = (kv + j) % kStages, stp = (kv + jp) % kStages;
            const int aslot = (kv + j) % L::kAugSlots;
            if (u < n_sub && hf == 0) {
              ok = wait_or_abort(bar(K_FULL + st), ((kv + j) / kStages) & 1, abort_flag, a.status, 105);
              if (!kTileBias && a.key_mma && ok)
                ok = wait_or_abort(bar(AUG_FULL + aslot), ((kv + j) / L::kAugSlots) & 1, abort_flag, a.status, 118);
              if (!ok) break;
              tc_fence_after_sync();
            }
            if (u < n_sub) {
              for (int g = g_begin; g < g_end && ok; ++g) {
                if (j >= it.nt[g]) continue;
                if (u == 0) {
                  ok = wait_or_abort(bar(Q_FULL + g), oc[g] & 1, abort_flag, a.status, 104);
                  if (!ok) break;
                  tc_fence_after_sync();
                }
                const uint32_t tS = tm_S[g] + hf * 64;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                  const uint64_t off = uint64_t(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
                  mma_ss(tS, qdesc[g] + off, kdesc[st] + off + uint64_t((hf * 64 * 128) >> 4), idesc_qk64, kk > 0 ? 1u : 0u);
                }
                if constexpr (!kTileBias) {
                  if (a.key_mma) {
                    // S += W C^T for the 64 keys of this half (8 groups of 8 keys, 256 bytes each, into the tile)
                    const uint64_t wdesc = make_smem_desc_noswizzle(sbase + L::kBias, 128, 256);
                    const uint64_t cdesc = make_smem_desc_noswizzle(sbase + L::kBias + L::kAugTileBytes * (1 + aslot) + hf * 2048, 128, 256);
                    mma_ss(tS, wdesc, cdesc, idesc_qk64, 1u);
                  }
                }
                mma_commit(bar(S_FULL + 2 * g + hf));
                if (u == 2 * it.nt[g] - 1) mma_commit(bar(Q_EMPTY + g));   // Q_g may be reloaded once these are done
              }
              if (!ok) break;
              if (hf == 1) {
                mma_commit(bar(K_EMPTY + st));
                if (!kTileBias && a.key_mma) mma_commit(bar(AUG_FREE + aslot));
              }
            }
            if (u >= 1) {
              if (hp == 0) {
                ok = wait_or_abort(bar(V_FULL + stp), ((kv + jp) / kStages) & 1, abort_flag, a.status, 106);
                if (!ok) break;
              }
              for (int g = g_begin; g < g_end && ok; ++g) {
                if (jp >= it.nt[g]) continue;
                ok = wait_or_abort(bar(P_READY + 2 * g + hp), (tc[g] + jp) & 1, abort_flag, a.status, 107);
                // the previous item's epilogue must have read O_g out before the first half overwrites it
                if (ok && u == 1 && oc[g] > 0)
                  ok = wait_or_abort(bar(O_FREE + g), (oc[g] - 1) & 1, abort_flag, a.status, 115);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tP = tm_S[g] + hp * 64;
#pragma unroll
                for (int kk = 0; kk < kTile / 32; ++kk)
                  mma_ts(tm_O[g], tP + kk * 8, vdesc[stp] + uint64_t(((hp * 4 + kk) * 2048) >> 4), idesc_pv,
                         (u > 1 || kk > 0) ? 1u : 0u);
                mma_commit(bar(PV_DONE + g));
                if (u == 2 * it.nt[g]) mma_commit(bar(O_DONE + g));
              }
              if (!ok) break;
              if (hp == 1) mma_commit(bar(V_EMPTY + stp));
            }
          }
        } else {
        // round j: score MMA of key tile j and output MMA of key tile j - 1
        for (int j = 0; j <= it.nt_max && ok; ++j) {
          const int st = (kv + j) % kStages, stp = (kv + j + kStages - 1) % kStages;
          if (j < it.nt_max) ok = wait_or_abort(bar(K_FULL + st), ((kv + j) / kStages) & 1, abort_flag, a.status, 105);
          if (ok && j > 0) ok = wait_or_abort(bar(V_FULL + stp), ((kv + j - 1) / kStages) & 1, abort_flag, a.status, 106);
          const int aslot = (kv + j) % L::kAugSlots;
          if (!kTileBias && a.key_mma && ok && j < it.nt_max)
            ok = wait_or_abort(bar(AUG_FULL + aslot), ((kv + j) / L::kAugSlots) & 1, abort_flag, a.status, 118);
          if (!ok) break;
          tc_fence_after_sync();
          for (int g = g_begin; g < g_end && ok; ++g) {
            const int nt = it.nt[g];
            auto round_pv = [&]() {
              const int jj = j - 1;
              if (j == 0 || jj >= nt) return;
              ok = wait_or_abort(bar(P_READY + g), (tc[g] + jj) & 1, abort_flag, a.status, 107);
              // the previous item's epilogue must have read O_g out before the first tile overwrites it
              if (ok && jj == 0 && oc[g] > 0)
                ok = wait_or_abort(bar(O_FREE + g), (oc[g] - 1) & 1, abort_flag, a.status, 115);
              if (!ok) return;
              tc_fence_after_sync();
#pragma unroll
              for (int kk = 0; kk < kTile / 16; ++kk)
                mma_ts(tm_O[g], tm_P[g] + kk * 8, vdesc[stp] + uint64_t((kk * 2048) >> 4), idesc_pv,
                       (jj > 0 || kk > 0) ? 1u : 0u);
              mma_commit(bar(PV_DONE + g));
              if (jj == nt - 1) mma_commit(bar(O_DONE + g));
            };
            auto round_qk = [&]() {
              if (j >= nt) return;
              const int gt = tc[g] + j;
              if (j == 0) ok = wait_or_abort(bar(Q_FULL + g), oc[g] & 1, abort_flag, a.status, 104);
              if (ok && gt > 0) ok = wait_or_abort(bar(S_FREE + g), (gt - 1) & 1, abort_flag, a.status, 111);
              if (!ok) return;
              tc_fence_after_sync();
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk) {
                const uint64_t off = uint64_t(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
                mma_ss(tm_S[g], qdesc[g] + off, kdesc[st] + off, idesc_qk, kk > 0 ? 1u : 0u);
              }
              if constexpr (!kTileBias) {
                if (a.key_mma) {
                  // S_g += W C^T: the per-key addends land on every query row
                  const uint64_t wdesc = make_smem_desc_noswizzle(sbase + L::kBias, 128, 256);
                  const uint64_t cdesc = make_smem_desc_noswizzle(sbase + L::kBias + L::kAugTileBytes * (1 + aslot), 128, 256);
                  mma_ss(tm_S[g], wdesc, cdesc, idesc_qk, 1u);
                }
              }
              if constexpr (D == 64 && kTileBias) {
                if (a.bias_mma) {
                  // S_g += bias tile (hi I + lo I): each 64-key half of the tile is one slot, read K-major as it
                  // was written by TMA.  Slot order as the bias producer fills them.
                  constexpr uint32_t idesc_bias = make_idesc(kBf16, kTile, 64, false, false);
                  const int seq0 = seq_base + 2 * (min(j, it.nt[0]) + min(j, it.nt[1]) + ((g == 1 && j < it.nt[0]) ? 1 : 0));
                  const int n_ident = a.inv_scale_lo != 0.f ? 2 : 1;
                  for (int half = 0; half < 2 && ok; ++half) {
                    const int slot = (seq0 + half) % L::kBiasSlots;
                    ok = wait_or_abort(bar(B_FULL + g * L::kBiasSlots + slot), (bias_phase >> slot) & 1u, abort_flag,
                                       a.status, 116);
                    if (!ok) return;
                    bias_phase ^= 1u << slot;
                    tc_fence_after_sync();
                    const uint64_t adesc = make_smem_desc(sbase + L::kBias + slot * kBoxBytes, 16, 1024);
                    for (int tile = 0; tile < n_ident; ++tile) {
                      const uint64_t bdesc = make_smem_desc(sbase + L::kIdent + tile * 8192, 16, 1024);
#pragma unroll
                      for (int kk = 0; kk < 4; ++kk)
                        mma_ss(tm_S[g] + half * 64, adesc + uint64_t((kk * 32) >> 4), bdesc + uint64_t((kk * 32) >> 4),
                               idesc_bias, 1u);
                    }
                    mma_commit(bar(B_EMPTY + slot));   // the slot may be refilled once these MMAs are done
                  }
                }
              }
              mma_commit(bar(S_FULL + g));
              if (j == nt - 1) mma_commit(bar(Q_EMPTY + g));   // Q_g may be reloaded once these are done
            };
            round_qk();   // S_g was read out early in softmax(j-1): the next scores run underneath it
            if (ok) round_pv();
          }
          if (!ok) break;
          if (j < it.nt_max) mma_commit(bar(K_EMPTY + st));
          if (!kTileBias && a.key_mma && j < it.nt_max) mma_commit(bar(AUG_FREE + aslot));
          if (j > 0) mma_commit(bar(V_EMPTY + stp));
        }
        }
        kv += it.nt_max;
        seq_base += 2 * (it.nt[0] + it.nt[1]);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          tc[g] += it.nt[g];
          oc[g] += it.nt[g] > 0 ? 1 : 0;
        }
      }
    }
  }
  } else {
    reg_alloc<kSoftmaxRegs>();
    // ---------------- softmax (one query row per thread) ----------------
    const int g = (warp - 4) >> 2;
    const int wq = warp & 3;                    // TMEM lane quarter this warp may access
    const int r = wq * 32 + lane;               // row within the tile
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    const uint32_t tS = tm_S[g] + lane_addr, tP = tm_P[g] + lane_addr, tO = tm_O[g] + lane_addr;
    bool ok = true;
    // no bias and a non-negative scale: the scale is folded into the exponent's multiplier and the max runs on raw scores
    // (the same holds when the tensor core has already added bias / scale to the scores)
    const bool key_mma = !kTileBias && a.key_mma;
    const bool fold_scale = (a.bias_mode == kBiasNone || a.bias_mma || key_mma) && a.scale >= 0.f;
    const float mul = fold_scale ? a.scale * kLog2e : kLog2e;   // exponent = (t - m) * mul, base 2
    const float thr = mul > 0.f ? 8.f / mul : INFINITY;         // reference max lags the true max by at most 2^8
    const float2 scale2 = make_float2(a.scale, a.scale), mul2 = make_float2(mul, mul);
    uint32_t bias_phase = 0;  // bit s = parity of this tile's next wait on its "full" barrier of slot s
    int tc = 0, oc = 0, seq_base = 0;
    FPROBE_DECL;

    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const Item it = decode_item(a, item, order);
      const int my_nt = it.nt[g];
      const int row = it.q0 + g * kTile + r;
      const int b = it.b, h = it.h;
      float m = -INFINITY, l = 0.f;  // m: reference max in logit units (see the lazy rescale below)

      const uint32_t* mrow = nullptr;
      if (a.mask.rows && !(key_mma && a.mask.kv_len)) {   // a key-only mask was added to the scores as -inf
        mrow = a.mask.rows + b * a.mask.b_stride + h * a.mask.h_stride + int64_t(min(row, a.S - 1)) * a.mask.row_stride;
      }
      const uint8_t* bias_key = nullptr;
      if (a.bias_mode == kBiasKey && !key_mma)
        bias_key = reinterpret_cast<const uint8_t*>(a.bias) + 2 * (b * a.bias_bs + h * a.bias_hs);

      // D = 128 takes a key tile as two halves of 64 keys (one S buffer each, P written over its own buffer);
      // D = 64 takes it whole
      constexpr int kSub = kAlias ? kTile / 2 : kTile;   // keys per pass
      constexpr int kSubs = kTile / kSub;
      uint32_t mnext[kSub / 32];   // keep-bits of this row for the coming pass
      auto load_mask_words = [](const uint32_t* src, uint32_t (&dst)[kSub / 32]) {
        if constexpr (kSub == 64) {
          const uint2 w = __ldg(reinterpret_cast<const uint2*>(src));
          dst[0] = w.x; dst[1] = w.y;
        } else {
          const uint4 w = __ldg(reinterpret_cast<const uint4*>(src));
          dst[0] = w.x; dst[1] = w.y; dst[2] = w.z; dst[3] = w.w;
        }
      };
#pragma unroll
      for (int i = 0; i < kSub / 32; ++i) mnext[i] = 0xffffffffu;
      if (mrow && my_nt > 0) load_mask_words(mrow, mnext);
      for (int j = 0; j < my_nt && ok; ++j) {
        const int gt = tc + j;   // this tile's running index for this query tile
#pragma unroll 1
        for (int hf = 0; hf < kSubs && ok; ++hf) {
        const int key0 = j * kTile + hf * kSub;
        const bool first = j == 0 && hf == 0;
        const int sbar = kAlias ? 2 * g + hf : g;
        const uint32_t tSh = tS + hf * kSub;
        // keep-bits of this row for these keys
        uint32_t keep[kSub / 32];
#pragma unroll
        for (int i = 0; i < kSub / 32; ++i) keep[i] = 0xffffffffu;
        bool need_mask = false;
        if (mrow) {
          // this pass's words were fetched a pass ago; the next pass's fetch runs under this pass's arithmetic
          uint32_t all = 0xffffffffu;
#pragma unroll
          for (int i = 0; i < kSub / 32; ++i) {
            keep[i] = mnext[i];
            all &= mnext[i];
          }
          need_mask = all != 0xffffffffu;   // keys the mask keeps whole need no selects
          const int nj = hf + 1 < kSubs ? j : j + 1, nh = hf + 1 < kSubs ? hf + 1 : 0;
          if (nj < my_nt) load_mask_words(mrow + nj * 4 + nh * (kSub / 32), mnext);
        }
        int n_keep = a.T - key0;
        if (a.causal) n_keep = min(n_keep, row - key0 + 1);
        if (n_keep < kSub) {
#pragma unroll
          for (int i = 0; i < kSub / 32; ++i) {
            const int n = n_keep - 32 * i;
            keep[i] &= n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u));
          }
          need_mask = true;
        }
        need_mask = __any_sync(0xffffffffu, need_mask);

        FPROBE(0);
        ok = wait_or_abort(bar(S_FULL + sbar), gt & 1, abort_flag, a.status, 108);
        FPROBE(1);
        if (!ok) break;
        tc_fence_after_sync();

        // the whole score row of this pass: all TMEM loads in flight, one wait; handled as fp32 pairs
        float2 t[kSub / 2];
        {
          uint32_t raw[kSub];
#pragma unroll
          for (int c = 0; c < kSub / 32; ++c) tmem_ld32(tSh + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[c * 32]));
          tmem_wait_ld();
          if constexpr (!kAlias) {
            // the scores are in registers: S_g may be overwritten by the next tile's MMA right away
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(S_FREE + g));
          }
#pragma unroll
          for (int i = 0; i < kSub / 2; ++i)
            t[i] = make_float2(__uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1]));
        }
        // logits: t = s * scale + bias (natural units); without a bias the scale is folded into the exponent
        FPROBE(2);
        if (a.bias_mode == kBiasTile && !a.bias_mma) {
          // slots filled before this (tile, query tile): every live query tile of the earlier key tiles, and
          // query tile 0 of this one when this is query tile 1.  One slot per 64 keys.
          const int seq0 = seq_base + 2 * (min(j, it.nt[0]) + min(j, it.nt[1]) + ((g == 1 && j < it.nt[0]) ? 1 : 0));
#pragma unroll
          for (int hh = 0; hh < kSub / 64; ++hh) {
            const int slot = (seq0 + (kAlias ? hf : hh)) % L::kBiasSlots;
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
                t[hh * 32 + c * 4 + e] = __ffma2_rn(t[hh * 32 + c * 4 + e], scale2, unpack2<kBf16>(ww[e]));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_EMPTY + slot));
          }
          if (!ok) break;
        } else if (a.bias_mode == kBiasKey && !key_mma) {
          const uint4* bk = reinterpret_cast<const uint4*>(bias_key + 2 * key0);
#pragma unroll
          for (int c = 0; c < kSub / 8; ++c) {
            const uint4 w = key0 + 8 * c < a.T ? __ldg(bk + c) : make_uint4(0, 0, 0, 0);   // T is a multiple of 8
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) t[c * 4 + e] = __ffma2_rn(t[c * 4 + e], scale2, unpack2<kBf16>(ww[e]));
          }
        } else if (!fold_scale) {
#pragma unroll
          for (int i = 0; i < kSub / 2; ++i) t[i] = __fmul2_rn(t[i], scale2);
        }
        FPROBE(3);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < kSub / 2; ++i) {
            if (!((keep[i >> 4] >> ((2 * i) & 31)) & 1u)) t[i].x = -INFINITY;
            if (!((keep[i >> 4] >> ((2 * i + 1) & 31)) & 1u)) t[i].y = -INFINITY;
          }
        }
        FPROBE(4);
        // row max: four independent chains of three-input max
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < kSub / 2; ++i) mx4[i & 3] = max3(mx4[i & 3], t[i].x, t[i].y);
        const float mx = max3(mx4[0], mx4[1], fmaxf(mx4[2], mx4[3]));
        // the exponentials use a reference max that is only moved when the true max has run more than
        // 2^8 ahead of it (so p <= 256 and the running output is rescaled rarely); l uses the same reference
        const bool bump = mx > m + thr;
        const float m_use = bump ? mx : m;
        const float alpha = bump ? ex2((m - m_use) * mul) : 1.f;
        const float neg = m_use == -INFINITY ? 0.f : -m_use * mul;
        const float2 neg2 = make_float2(neg, neg);
        float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        uint32_t pk[kSub / 2];
#pragma unroll
        for (int i = 0; i < kSub / 2; ++i) {
          const float2 x = __ffma2_rn(t[i], mul2, neg2);
          // every kPolyPeriod-th pair takes its exponentials on the FMA pipe (see ex2_poly2)
          const float2 p = (kAlias && kPolyPeriod > 0 && i % (kPolyPeriod > 0 ? kPolyPeriod : 1) == 0) ? ex2_poly2(x)
                                                                                             : make_float2(ex2(x.x), ex2(x.y));
          sum2[i & 1] = __fadd2_rn(sum2[i & 1], p);
          pk[i] = pack2<kBf16>(p.x, p.y);
        }
        l = l * alpha + ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y));
        const bool rescale = !first && __any_sync(0xffffffffu, bump);
        if constexpr (!kAlias) {
          // O_g and P_g are still in use by the previous tile's output MMA until it has completed
          // (the first tile of an item follows the previous item's epilogue, which waited for that)
          if (j > 0) {
            ok = wait_or_abort(bar(PV_DONE + g), (gt - 1) & 1, abort_flag, a.status, 112);
            if (!ok) break;
            tc_fence_after_sync();
          }
        } else if (rescale) {
          // O_g is being accumulated into by the previous half's output MMA until that has completed (its P buffer
          // is the other one, and this buffer's earlier reader ran before these scores).  Output MMA number
          // 2 gt + hf - 1 of this query tile: at most one phase of the barrier is outstanding, so parity names it.
          ok = wait_or_abort(bar(PV_DONE + g), (2 * gt + hf - 1) & 1, abort_flag, a.status, 112);
          if (!ok) break;
          tc_fence_after_sync();
        }
        FPROBE(6);
        // rescale the running output when some row of this warp moved its reference max
        if (rescale) {
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
        FPROBE(7);
        // P as 16-bit pairs: half as many columns as keys (over its own S buffer when aliased)
        const uint32_t tPh = kAlias ? tSh : tP;
#pragma unroll
        for (int c = 0; c < kSub / 64; ++c) tmem_st32(tPh + c * 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[c * 32]));
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_READY + sbar));
        FPROBE(8);
        }
      }

      FPROBE(9);
      // ---------------- epilogue: out = O / l, lse = m * mul + log2 l ----------------
      if (ok && my_nt > 0) ok = wait_or_abort(bar(O_DONE + g), oc & 1, abort_flag, a.status, 110);
      if (ok && my_nt > 0) {
        tc_fence_after_sync();
        const float inv = 1.f / l;  // l == 0 (no kept key): 0 * inf = NaN, as the reference's softmax gives
        const int64_t out_off = 2 * (b * a.os[0] + h * a.os[1] + int64_t(row) * a.os[2]);
        uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + out_off;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
          if (c == D / 32 - 1) {
            // O_g is in registers: the next item's first output MMA may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(O_FREE + g));
          }
          if (row < a.S) {
            uint4 w[4];
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4& x = w[i >> 3];
              x.x = pack2<kBf16>(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              x.y = pack2<kBf16>(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              x.z = pack2<kBf16>(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              x.w = pack2<kBf16>(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + (c * 32 + i) * 2) = x;
            }
            // fused all-gather: the same 64 bytes go to every peer's copy, two whole 32-byte sectors per thread
            for (int pi = 0; pi < a.n_out_peers; ++pi) {
              uint8_t* prow = reinterpret_cast<uint8_t*>(a.out_peers[pi]) + out_off + c * 64;
              st_global_v8(prow, w[0], w[1]);
              st_global_v8(prow + 32, w[2], w[3]);
            }
          }
        }
        if (row < a.S) a.lse[(int64_t(b) * a.H + h) * a.S + row] = m * mul + log2f(l);
      }
      tc += my_nt;
      oc += my_nt > 0 ? 1 : 0;
      seq_base += 2 * (it.nt[0] + it.nt[1]);
      FPROBE(10);
      FPROBE_TILES(my_nt);
    }
    FPROBE_FLUSH;
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

template <int D, bool kBf16, bool kTileBias>
int launch_one(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tb,
               FwdArgs a, cudaStream_t st) {
  auto kernel = sdpa_fwd_tc_kernel<D, kBf16, kTileBias>;
  using L = FwdSmem<D, kTileBias>;
  constexpr int kLimit = 232448;  // 227 KB per CTA
  const int smem = L::kTotal + 1024 <= kLimit ? L::kTotal + 1024 : kLimit;
  static_assert(L::kTotal <= kLimit, "forward shared memory exceeds the per-CTA limit");
  a.smem_bytes = smem;
  // checked and configured once per device and kernel instance (setting it again would be harmless)
  static bool ready[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev < 0 || !ready[dev]) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess || attr.numRegs != kLaunchRegs) {
      // the register hand-over inside the kernel is balanced for exactly kLaunchRegs per thread at launch
      set_error("sdpa_fwd_tc_kernel was built with %d registers per thread, expected %d", attr.numRegs, kLaunchRegs);
      return NB200_ERR_LAUNCH;
    }
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(sdpa_fwd_tc_kernel, %d): %s", smem, cudaGetErrorString(e));
      return NB200_ERR_LAUNCH;
    }
    if (dev >= 0) ready[dev] = true;
  }
  const int n_items = a.n_qblocks * a.bh_count;
  const int sms = sm_count();
  dim3 grid(n_items < sms ? n_items : sms);
  kernel<<<grid, kThreads, smem, st>>>(tq, tk, tv, tb, a);
  count_launch();
  return check_launch("sdpa_fwd_tc_kernel");
}

}  // namespace


int launch_fwd(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
               const CUtensorMap& tb, const FwdArgs& a, cudaStream_t st) {
  const bool tiles = a.bias_mode == kBiasTile;
  if (D == 64) {
    if (tiles) return bf16 ? launch_one<64, true, true>(tq, tk, tv, tb, a, st) : launch_one<64, false, true>(tq, tk, tv, tb, a, st);
    return bf16 ? launch_one<64, true, false>(tq, tk, tv, tb, a, st) : launch_one<64, false, false>(tq, tk, tv, tb, a, st);
  }
  if (tiles) return bf16 ? launch_one<128, true, true>(tq, tk, tv, tb, a, st) : launch_one<128, false, true>(tq, tk, tv, tb, a, st);
  return bf16 ? launch_one<128, true, false>(tq, tk, tv, tb, a, st) : launch_one<128, false, false>(tq, tk, tv, tb, a, st);
}

}  // namespace tc
}  // namespace nb200

#ifdef NB200_PROBE
extern "C" NB200_API int nb200_debug_fprobe(unsigned long long* out16, int reset) {
  unsigned long long zero[16] = {};
  if (out16) cudaMemcpyFromSymbol(out16, nb200::tc::g_fprobe, sizeof(zero));
  if (reset) cudaMemcpyToSymbol(nb200::tc::g_fprobe, zero, sizeof(zero));
  return 0;
}
#endif
