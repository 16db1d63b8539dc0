// Host/device pieces shared by the tensor-core (TMA + tcgen05) attention
// kernels: tensor-map creation, the bit-packed mask, bounded waits with a
// CTA-wide abort flag, and the softmax-tile helpers.
#pragma once

#include <cuda.h>

#include "sdpa_common.cuh"
#include "sm100_primitives.cuh"

namespace nb200 {
namespace tc {

constexpr int kTile = 128;         // query rows / key columns per tcgen05 tile
constexpr int kSlotCols = 64;      // 16-bit elements per 128-byte swizzled row
constexpr int kBoxBytes = kTile * 128;  // one TMA box: 128 rows x 128 bytes

enum BiasMode : int {
  kBiasNone = 0,
  kBiasTile = 1,  // (rows, keys) tiles fetched by TMA into a ring of 16 KB slots
  kBiasKey = 2    // one value per key, shared by every query row (row stride 0)
};

// ---- tensor maps (host) -----------------------------------------------------
// 4-D map over a (B, H, rows, cols) tensor of 16-bit elements with unit column
// stride; box = 64 columns x `box_rows` rows, 128-byte swizzle, out-of-bounds -> zero.
// An axis that is broadcast (stride 0) is encoded with extent 1; kernels pass
// coordinate 0 for it.  Returns false when the driver entry point is missing or
// the encode call rejects the layout.
bool make_tile_map(CUtensorMap* map, const void* base, int rows, int cols, int H, int B, int64_t row_stride,
                   int64_t h_stride, int64_t b_stride, int box_rows, const char** why);

// 1 / scale as hi + lo, both exactly representable in the 16-bit operand type (lo = 0 for a power-of-two scale).
// False when the scale is zero / not finite or 1 / scale overflows the type.
bool split_inv_scale(float scale, bool bf16, float* hi, float* lo);

// Number of SMs of the current device (cached per device).
int sm_count();

// True when a tensor with these element strides can be described by make_tile_map.  `allow_broadcast`: a stride-0
// head / batch axis is acceptable (the bias, whose loads scale their coordinates; not q, k, v, dout).
bool tile_map_ok(const void* base, int64_t row_stride, int64_t h_stride, int64_t b_stride, int H, int B,
                 bool allow_broadcast);

// ---- bit-packed mask ----------------------------------------------------------
// The byte mask (own extent Bm, Hm, Sm, Tm with strides, broadcast axes = 1) is
// packed once per call into 32-key words: bits[bm][hm][sm][w], w < words_per_row,
// bit i of word w = keep(row, 32 w + i).  words_per_row is padded to a multiple
// of 4 so a row's 128-key group is one aligned 16-byte load; padding bits and
// keys >= T are 0 (dropped).  With `transposed` a second array indexed
// [bm][hm][key][w] holds bit i = keep(32 w + i, key) for the key-major kernels.
struct MaskBits {
  const uint32_t* rows;     // null when there is no mask
  const uint32_t* cols;     // transposed copy (backward only) or null
  int64_t b_stride, h_stride, row_stride;       // in words; 0 on broadcast axes
  int64_t tb_stride, th_stride, tkey_stride;    // transposed array
  // Key-only masks (no query axis, e.g. key padding): 1 + index of the last kept key per (bm, hm), so that
  // kernels skip the key tiles past it altogether.  Null for masks with a query axis.
  const int* kv_len;
  int64_t len_b_stride, len_h_stride;
};

struct MaskPackPlan {
  int64_t extent[4];          // Bm, Hm, Sm(1 or S), 1
  int words_per_row;          // over T
  int words_per_col;          // over S (transposed)
  size_t rows_bytes, cols_bytes, len_bytes;
  size_t total() const { return rows_bytes + cols_bytes + len_bytes; }
};

#ifdef __CUDACC__
// Number of leading keys of (b, h) that can matter: T without a key-only mask, else 1 + last kept key.
__device__ __forceinline__ int kept_key_length(const MaskBits& m, int b, int h, int T) {
  if (!m.kv_len) return T;
  return min(T, m.kv_len[b * m.len_b_stride + h * m.len_h_stride]);
}
#endif
MaskPackPlan plan_mask_pack(const Problem& pr, bool transposed);
// True when the mask has no query axis (key padding and the like).
bool mask_key_only(const Problem& pr);
// Layout of the mask bits a forward / backward call works with, and the workspace bytes it needs for them (none when
// the caller passes a mask that nb200_mask_pack packed earlier; launch_mask_pack then only forms the views).
MaskPackPlan mask_plan_for_pass(const Problem& pr, bool backward, size_t* ws_bytes);
int launch_mask_pack(const Problem& pr, const MaskPackPlan& plan, void* ws, MaskBits* out, cudaStream_t stream);

// ---- staging of operands whose layout the kernels cannot address directly --------
// TMA needs 16-byte aligned bases and row strides, and the backward copies 64-row blocks of lse / delta with 16-byte
// granularity.  A bias (or dbias) whose key count is not a multiple of 8, whose rows are strided oddly or whose key
// axis is not contiguous, and lse / delta with a query count that is not a multiple of 4, therefore go through
// padded copies in the workspace: bias is copied in before the kernels, dbias is written padded and copied out after
// them, lse / delta are copied into rows padded to 64.  Lengths that are multiples of 8 with dense operands need
// none of this.
struct Staging {
  bool bias, dbias, rows;        // which operands are staged
  int Tp, Sp;                    // padded key count (multiple of 8) and query count (multiple of 64)
  int64_t extent[4];             // bias' own extent (1 on broadcast axes)
  size_t bias_bytes, dbias_bytes, rows_bytes;   // each a multiple of 256; rows_bytes is for ONE of lse / delta
  size_t total() const { return bias_bytes + dbias_bytes + 2 * rows_bytes; }
};
Staging plan_staging(const Problem& pr, int pass);
// The problem as the kernels see it: staged operands replaced by their padded copies at `base` (bias, then dbias,
// then lse, then delta).  With base == nullptr (planning) the staged pointers are aligned placeholders.
Problem staged_view(const Problem& pr, const Staging& sg, void* base);
// Copies before the kernels (bias in; lse / delta into padded rows -- delta must have been computed already) and
// after them (dbias out).
int stage_in(const Problem& pr, const Problem& staged, const Staging& sg, int pass, cudaStream_t stream);
int stage_out(const Problem& pr, const Problem& staged, const Staging& sg, cudaStream_t stream);

// ---- device helpers -----------------------------------------------------------
#ifdef __CUDACC__

constexpr uint32_t kWaitHintNs = 16384;         // a waiting thread may sleep this long per try_wait before it re-checks
constexpr long long kWaitCycles = 400000000LL;  // ~0.2 s of SM clock: far beyond any real wait (microseconds)

// Wait on an mbarrier phase unless the CTA has aborted.  On timeout: raise the
// CTA abort flag, record `code` in the device status word, return false.  A
// status word already set by another CTA aborts this one as well, so one
// protocol failure ends the whole grid quickly instead of once per CTA.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                              int code, long long budget_cycles = kWaitCycles) {
  if (sm100::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (true) {
    if (sm100::mbar_try_wait_hint(bar, parity, kWaitHintNs)) return true;
    if ((++polls & 0xFF) == 0) {
      if (*abort_flag) return false;
      if (*reinterpret_cast<volatile int*>(status) != 0) {
        *abort_flag = 1;
        return false;
      }
      if (clock64() - t0 > budget_cycles) {
        *abort_flag = 1;
        atomicExch(status, code);
        return false;
      }
    }
  }
}

// After an abort: give copies already in flight time to land before the CTA's
// shared memory is released (bounded; a healthy copy takes microseconds).
__device__ __forceinline__ void drain_after_abort() {
  for (int i = 0; i < 64; ++i) __nanosleep(2000);
}

// single-instruction helpers
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for a pair on the FMA and integer pipes instead of the special-function unit (which serves 16 lanes a
// clock per SM and bounds the soft-max when every exponential goes through it).  x = n + f with n the nearest
// integer (the magic-constant add leaves n in the low mantissa bits) and f in [-0.5, 0.5]; 2^f by a cubic
// (relative error 7.5e-5, far below the rounding of the 16-bit P it feeds), then n goes into the exponent
// field.  Inputs below -127 (masked keys: -inf) are clamped; there the exponent field wraps negative and the
// signed max returns exactly +0, as ex2 does.  Valid for x <= 100.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  x.x = fmaxf(x.x, -127.f);
  x.y = fmaxf(x.y, -127.f);
  const float2 magic = make_float2(12582912.f, 12582912.f), neg_magic = make_float2(-12582912.f, -12582912.f);
  const float2 t = __fadd2_rn(x, magic);
  const float2 n = __fadd2_rn(t, neg_magic);
  const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
  float2 p = __ffma2_rn(make_float2(0.0551716648f, 0.0551716648f), f, make_float2(0.2426111251f, 0.2426111251f));
  p = __ffma2_rn(p, f, make_float2(0.6932609677f, 0.6932609677f));
  p = __ffma2_rn(p, f, make_float2(0.9999280572f, 0.9999280572f));
  const int bx = max(__float_as_int(p.x) + (__float_as_int(t.x) << 23), 0);
  const int by = max(__float_as_int(p.y) + (__float_as_int(t.y) << 23), 0);
  return make_float2(__int_as_float(bx), __int_as_float(by));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (kBf16) {
    return make_float2(bf16_lo(w), bf16_hi(w));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// 128-bit keep mask of one row against one 128-key tile, combining the packed
// user mask, the causal bound and the key-length bound.  `n_keep` = number of
// leading keys of the tile the row may see from causal / length limits
// (<= 0 none, >= 128 all).
__device__ __forceinline__ void limit_bits(uint32_t (&w)[4], int n_keep) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = n_keep - 32 * i;
    const uint32_t lim = n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u));
    w[i] &= lim;
  }
}

#endif  // __CUDACC__

}  // namespace tc
}  // namespace nb200
