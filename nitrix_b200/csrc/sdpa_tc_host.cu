// Host side of the tensor-core kernels: coverage gate, workspace plan, tensor
// maps, the mask bit-packing kernel and the launches.
#include <mutex>
#include <stdlib.h>

#include "sdpa_tc_bwd.cuh"
#include "sdpa_tc_common.cuh"
#include "sdpa_tc_fwd.cuh"

namespace nb200 {
namespace tc {

// ---- tensor maps ------------------------------------------------------------
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

}  // namespace

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool tile_map_ok(const void* base, int64_t row_stride, int64_t h_stride, int64_t b_stride, int H, int B,
                 bool allow_broadcast) {
  if (reinterpret_cast<uintptr_t>(base) % 16) return false;
  if (row_stride <= 0 || row_stride % 8) return false;
  // A broadcast (stride 0) head or batch axis is encoded with extent 1, and only the bias loads scale their
  // head / batch coordinate accordingly; q, k, v and dout are addressed by the absolute (b, h), so an expanded
  // view of them is declined here and runs on the CUDA-core family, which indexes by stride.
  if (H > 1 && (h_stride % 8 || h_stride < 0 || (h_stride == 0 && !allow_broadcast))) return false;
  if (B > 1 && (b_stride % 8 || b_stride < 0 || (b_stride == 0 && !allow_broadcast))) return false;
  return true;
}

bool make_tile_map(CUtensorMap* map, const void* base, int rows, int cols, int H, int B, int64_t row_stride,
                   int64_t h_stride, int64_t b_stride, int box_rows, const char** why) {
  EncodeFn fn = encode_fn();
  if (!fn) { if (why) *why = "cuTensorMapEncodeTiled is unavailable"; return false; }
  // broadcast or singleton axes: extent 1 with a harmless natural stride
  const bool h_bc = H <= 1 || h_stride == 0, b_bc = B <= 1 || b_stride == 0;
  const int64_t hs = h_bc ? int64_t(rows) * row_stride : h_stride;
  const int64_t bs = b_bc ? hs * (h_bc ? 1 : H) : b_stride;
  cuuint64_t dims[4] = {cuuint64_t(cols), cuuint64_t(rows), cuuint64_t(h_bc ? 1 : H), cuuint64_t(b_bc ? 1 : B)};
  cuuint64_t strides[3] = {cuuint64_t(row_stride) * 2, cuuint64_t(hs) * 2, cuuint64_t(bs) * 2};
  cuuint32_t box[4] = {cuuint32_t(kSlotCols), cuuint32_t(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { if (why) *why = "cuTensorMapEncodeTiled rejected the layout"; return false; }
  return true;
}

// ---- mask packing -------------------------------------------------------------
namespace {

// One CTA packs a 32-row x 32-key tile: row-major words by warp ballot over the
// keys of a row, transposed words by ballot over the rows of a key.
__global__ void __launch_bounds__(256) mask_pack_kernel(const uint8_t* mask, int64_t sb, int64_t sh, int64_t ss,
                                                        int64_t st, int Hm, int Sm, int S, int T,
                                                        uint32_t* rows_out, int words_per_row,
                                                        uint32_t* cols_out, int words_per_col, int* kv_len) {
  __shared__ uint8_t tile[32][33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bm = blockIdx.z / Hm, hm = blockIdx.z - bm * Hm;
  const int key0 = blockIdx.x * 32, row0 = blockIdx.y * 32;
  const uint8_t* base = mask + bm * sb + hm * sh;
  const int n_rows = cols_out ? S : Sm;  // the transposed copy always spans every query row
  for (int rl = warp; rl < 32; rl += 8) {
    const int row = row0 + rl, key = key0 + lane;
    const bool in = row < n_rows && key < T;
    const uint8_t v = in ? (base[int64_t(Sm == 1 ? 0 : row) * ss + int64_t(key) * st] != 0) : 0;
    tile[rl][lane] = v;
    const uint32_t word = __ballot_sync(0xffffffffu, v != 0);
    if (lane == 0 && row < Sm) {
      rows_out[(int64_t(blockIdx.z) * Sm + row) * words_per_row + blockIdx.x] = word;
      // key-only mask: remember the last kept key (1 + index) so that fully dropped tail tiles are skipped
      if (kv_len && word != 0u) atomicMax(kv_len + blockIdx.z, key0 + 32 - __clz(word));
    }
  }
  if (!cols_out) return;
  __syncthreads();
  for (int kl = warp; kl < 32; kl += 8) {
    const int key = key0 + kl;
    const uint32_t word = __ballot_sync(0xffffffffu, tile[lane][kl] != 0);
    if (lane == 0 && key < T) cols_out[(int64_t(blockIdx.z) * T + key) * words_per_col + blockIdx.y] = word;
  }
}

// Fast path for a mask with a query axis, unit key stride and 16-byte aligned rows: one CTA packs a 256-row x
// 256-key tile.  Rows are read as 16-byte vectors (16 keys per lane, a warp covers two 256-byte row segments per
// load); the row-major words go out as they are formed and are kept in shared memory, from which each warp then
// builds the transposed words of 32 keys by ballot over 32 rows, 8 row-words (32 bytes) per key.
__global__ void __launch_bounds__(256) mask_pack_tile_kernel(const uint8_t* mask, int64_t sb, int64_t sh, int64_t ss, int Hm,
                                                             int S, int T, uint32_t* rows_out, int words_per_row,
                                                             uint32_t* cols_out, int words_per_col) {
  __shared__ uint32_t sw[256][9];   // [row][key word], padded against bank conflicts
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bm = blockIdx.z / Hm, hm = blockIdx.z - bm * Hm;
  const int key0 = blockIdx.x * 256, row0 = blockIdx.y * 256;
  const uint8_t* base = mask + bm * sb + hm * sh + int64_t(row0) * ss + key0;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int rl = warp * 32 + 2 * i + (lane >> 4);     // row within the tile
    const int chunk = lane & 15;                        // 16 keys
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(base + int64_t(rl) * ss + chunk * 16));
    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
    uint32_t bits = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t nz = __vcmpne4(in[e], 0u) & 0x01010101u;          // one bit per non-zero byte
      bits |= ((nz * 0x01020408u) >> 24 & 0xFu) << (4 * e);            // byte k of the word -> bit k
    }
    const uint32_t hi = __shfl_down_sync(0xffffffffu, bits, 1);
    if (!(lane & 1)) {
      const uint32_t word = bits | (hi << 16);
      sw[rl][chunk >> 1] = word;
      rows_out[(int64_t(blockIdx.z) * S + row0 + rl) * words_per_row + (key0 >> 5) + (chunk >> 1)] = word;
    }
  }
  if (!cols_out) return;
  __syncthreads();
  // warp w transposes key word w: lane = key, 8 row-words each
  uint32_t out[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t w = sw[32 * j + lane][warp];          // lane = row within the group of 32
    uint32_t mine = 0;
#pragma unroll
    for (int b = 0; b < 32; ++b) {
      const uint32_t t = __ballot_sync(0xffffffffu, (w >> b) & 1u);
      if (lane == b) mine = t;
    }
    out[j] = mine;
  }
  uint32_t* dst = cols_out + (int64_t(blockIdx.z) * T + key0 + warp * 32 + lane) * words_per_col + (row0 >> 5);
  *reinterpret_cast<uint4*>(dst) = make_uint4(out[0], out[1], out[2], out[3]);
  *reinterpret_cast<uint4*>(dst + 4) = make_uint4(out[4], out[5], out[6], out[7]);
}

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

}  // namespace

// ---- staging ---------------------------------------------------------------------
namespace {

// dst[i0][i1][i2][i3] = src[...] for 16-bit elements, both sides described by element strides
__global__ void copy16_4d_kernel(const uint16_t* __restrict__ src, int64_t s0, int64_t s1, int64_t s2, int64_t s3,
                                 uint16_t* __restrict__ dst, int64_t d0, int64_t d1, int64_t d2, int64_t d3, int64_t e1,
                                 int64_t e2, int64_t e3, int64_t n) {
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t i3 = i % e3, r = i / e3;
    const int64_t i2 = r % e2, r2 = r / e2;
    const int64_t i1 = r2 % e1, i0 = r2 / e1;
    dst[i0 * d0 + i1 * d1 + i2 * d2 + i3 * d3] = src[i0 * s0 + i1 * s1 + i2 * s2 + i3 * s3];
  }
}

// (BH, S) fp32 rows -> (BH, Sp) rows, zero beyond S
__global__ void pad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int S, int Sp, int64_t n) {
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t bh = i / Sp;
    const int r = int(i - bh * Sp);
    dst[i] = r < S ? src[bh * S + r] : 0.f;
  }
}

inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }
inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int launch_copy16(const void* src, const int64_t ss[4], void* dst, const int64_t ds[4], const int64_t e[4], cudaStream_t st,
                  const char* what) {
  const int64_t n = e[0] * e[1] * e[2] * e[3];
  if (n <= 0) return NB200_OK;
  const int64_t want = (n + 255) / 256;
  const int blocks = int(want < 148 * 16 ? want : 148 * 16);
  copy16_4d_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(src), ss[0], ss[1], ss[2], ss[3],
                                           static_cast<uint16_t*>(dst), ds[0], ds[1], ds[2], ds[3], e[1], e[2], e[3], n);
  count_launch();
  return check_launch(what);
}

}  // namespace

Staging plan_staging(const Problem& pr, int pass) {
  Staging sg{};
  sg.Tp = (pr.T + 7) / 8 * 8;
  sg.Sp = (pr.S + kTile / 2 - 1) / (kTile / 2) * (kTile / 2);
  const int64_t full[4] = {pr.B, pr.H, pr.S, pr.T};
  for (int a = 0; a < 4; ++a) sg.extent[a] = (!pr.bias || pr.bs[a] == 0 || full[a] == 1) ? 1 : full[a];
  const bool tile_bias = pr.bias && !(pr.bs[2] == 0 || pr.S == 1);
  if (tile_bias) {
    const bool direct = (pr.T == 1 || pr.bs[3] == 1) && tile_map_ok(pr.bias, pr.bs[2], pr.bs[1], pr.bs[0], pr.H, pr.B, true);
    if (!direct) {
      sg.bias = true;
      sg.bias_bytes = up256(size_t(sg.extent[0] * sg.extent[1] * pr.S) * sg.Tp * 2);
    }
  }
  // a gradient of full extent (no axis of the bias is broadcast) is written by the kernels in 16-byte row segments
  // or by TMA: same layout rules as the bias tiles
  const bool broadcast = (pr.B > 1 && pr.bs[0] == 0) || (pr.H > 1 && pr.bs[1] == 0) || (pr.S > 1 && pr.bs[2] == 0);
  if (pr.bias && pass == NB200_PASS_BWD && pr.want_dbias && !broadcast) {
    const bool direct = pr.T % 8 == 0 && (!pr.dbias || (pr.dbs[3] == 1 && aligned16(pr.dbias) && pr.dbs[0] % 8 == 0 &&
                                                        pr.dbs[1] % 8 == 0 && pr.dbs[2] % 8 == 0));
    if (!direct) {
      sg.dbias = true;
      sg.dbias_bytes = up256(size_t(pr.B) * pr.H * pr.S * sg.Tp * 2);
    }
  }
  if (pass == NB200_PASS_BWD && (pr.S % 4 != 0 || (pr.lse && !aligned16(pr.lse)))) {
    sg.rows = true;
    sg.rows_bytes = up256(sizeof(float) * size_t(pr.B) * pr.H * sg.Sp);
  }
  return sg;
}

Problem staged_view(const Problem& pr, const Staging& sg, void* base) {
  Problem v = pr;
  char* p = base ? static_cast<char*>(base) : reinterpret_cast<char*>(uintptr_t(1) << 20);
  if (sg.bias) {
    v.bias = p;
    // dense over the bias' own extent with rows of Tp keys; broadcast axes keep stride 0
    v.bs[3] = 1;
    v.bs[2] = sg.Tp;
    v.bs[1] = sg.extent[1] == 1 ? 0 : int64_t(pr.S) * sg.Tp;
    v.bs[0] = sg.extent[0] == 1 ? 0 : sg.extent[1] * int64_t(pr.S) * sg.Tp;
    p += sg.bias_bytes;
  }
  if (sg.dbias) {
    v.dbias = p;
    v.dbs[3] = 1;
    v.dbs[2] = sg.Tp;
    v.dbs[1] = int64_t(pr.S) * sg.Tp;
    v.dbs[0] = int64_t(pr.H) * pr.S * sg.Tp;
    p += sg.dbias_bytes;
  }
  if (sg.rows) {
    v.lse = reinterpret_cast<float*>(p);
    v.delta = reinterpret_cast<float*>(p + sg.rows_bytes);
  }
  return v;
}

int stage_in(const Problem& pr, const Problem& v, const Staging& sg, int pass, cudaStream_t stream) {
  if (sg.bias) {
    const int64_t e[4] = {sg.extent[0], sg.extent[1], pr.S, pr.T};
    if (int rc = launch_copy16(pr.bias, pr.bs, const_cast<void*>(v.bias), v.bs, e, stream, "bias_pad_kernel")) return rc;
  }
  if (sg.rows && pass == NB200_PASS_BWD) {
    const int64_t n = int64_t(pr.B) * pr.H * sg.Sp;
    const int blocks = int(((n + 255) / 256) < 148 * 16 ? ((n + 255) / 256) : 148 * 16);
    pad_rows_kernel<<<blocks, 256, 0, stream>>>(pr.lse, v.lse, pr.S, sg.Sp, n);
    pad_rows_kernel<<<blocks, 256, 0, stream>>>(pr.delta, v.delta, pr.S, sg.Sp, n);
    count_launch(2);
    if (int rc = check_launch("pad_rows_kernel")) return rc;
  }
  return NB200_OK;
}

int stage_out(const Problem& pr, const Problem& v, const Staging& sg, cudaStream_t stream) {
  if (!sg.dbias || !pr.dbias) return NB200_OK;
  const int64_t e[4] = {pr.B, pr.H, pr.S, pr.T};
  return launch_copy16(v.dbias, v.dbs, pr.dbias, pr.dbs, e, stream, "dbias_unpad_kernel");
}

bool split_inv_scale(float scale, bool bf16, float* hi, float* lo) {
  *hi = *lo = 0.f;
  if (scale == 0.f || !isfinite(scale) || !isfinite(1.f / scale)) return false;
  const float inv = 1.f / scale;
  const float h = bf16 ? __bfloat162float(__float2bfloat16_rn(inv)) : __half2float(__float2half_rn(inv));
  if (!isfinite(h) || h == 0.f) return false;
  const float rest = inv - h;
  *hi = h;
  *lo = bf16 ? __bfloat162float(__float2bfloat16_rn(rest)) : __half2float(__float2half_rn(rest));
  return true;
}

MaskPackPlan plan_mask_pack(const Problem& pr, bool transposed) {
  MaskPackPlan p{};
  if (!pr.mask) return p;
  const int64_t full[4] = {pr.B, pr.H, pr.S, pr.T};
  for (int a = 0; a < 3; ++a) p.extent[a] = (pr.ms[a] == 0 || full[a] == 1) ? 1 : full[a];
  p.extent[3] = 1;
  p.words_per_row = round_up((pr.T + 31) / 32, 4);
  p.words_per_col = round_up((pr.S + 31) / 32, 4);
  p.rows_bytes = size_t(p.extent[0] * p.extent[1] * p.extent[2]) * p.words_per_row * 4;
  p.rows_bytes = (p.rows_bytes + 255) / 256 * 256;
  p.cols_bytes = transposed ? size_t(p.extent[0] * p.extent[1]) * pr.T * p.words_per_col * 4 : 0;
  p.cols_bytes = (p.cols_bytes + 255) / 256 * 256;
  p.len_bytes = p.extent[2] == 1 ? (size_t(p.extent[0] * p.extent[1]) * 4 + 255) / 256 * 256 : 0;
  return p;
}

bool mask_key_only(const Problem& pr) { return pr.mask && (pr.ms[2] == 0 || pr.S == 1); }

MaskPackPlan mask_plan_for_pass(const Problem& pr, bool backward, size_t* ws_bytes) {
  // a mask without a query axis never needs the transposed copy; a caller-packed mask has the layout it was packed with
  const bool transposed = !mask_key_only(pr) && (pr.mask_packed ? pr.mask_packed == 2 : backward);
  const MaskPackPlan mp = plan_mask_pack(pr, pr.mask && transposed);
  if (ws_bytes) *ws_bytes = pr.mask_packed ? 0 : mp.total();
  return mp;
}

namespace {
// Views into a packed-mask buffer laid out as `plan` says: rows, transposed copy, key lengths.
void mask_views(const Problem& pr, const MaskPackPlan& plan, void* buf, MaskBits* out) {
  uint32_t* rows = static_cast<uint32_t*>(buf);
  uint32_t* cols = plan.cols_bytes ? reinterpret_cast<uint32_t*>(static_cast<char*>(buf) + plan.rows_bytes) : nullptr;
  int* kv_len = plan.len_bytes ? reinterpret_cast<int*>(static_cast<char*>(buf) + plan.rows_bytes + plan.cols_bytes) : nullptr;
  const int Hm = int(plan.extent[1]), Bm = int(plan.extent[0]), Sm = int(plan.extent[2]);
  out->rows = rows;
  out->row_stride = Sm == 1 ? 0 : plan.words_per_row;
  out->h_stride = Hm == 1 ? 0 : int64_t(Sm) * plan.words_per_row;
  out->b_stride = Bm == 1 ? 0 : int64_t(Hm) * Sm * plan.words_per_row;
  out->cols = cols;
  out->tkey_stride = plan.words_per_col;
  out->th_stride = Hm == 1 ? 0 : int64_t(pr.T) * plan.words_per_col;
  out->tb_stride = Bm == 1 ? 0 : int64_t(Hm) * pr.T * plan.words_per_col;
  out->kv_len = kv_len;
  out->len_h_stride = Hm == 1 ? 0 : 1;
  out->len_b_stride = Bm == 1 ? 0 : Hm;
}
}  // namespace

int launch_mask_pack(const Problem& pr, const MaskPackPlan& plan, void* ws, MaskBits* out, cudaStream_t stream) {
  *out = MaskBits{};
  if (!pr.mask) return NB200_OK;
  if (pr.mask_packed) {
    // packed earlier by nb200_mask_pack: nothing to launch
    mask_views(pr, plan, const_cast<uint8_t*>(pr.mask), out);
    return NB200_OK;
  }
  uint32_t* rows = static_cast<uint32_t*>(ws);
  uint32_t* cols = plan.cols_bytes ? reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + plan.rows_bytes) : nullptr;
  const int Bm = int(plan.extent[0]), Hm = int(plan.extent[1]), Sm = int(plan.extent[2]);
  const int n_rows = cols ? pr.S : Sm;
  // padding words beyond ceil(T/32) (and ceil(S/32)) must read as "dropped"
  int* kv_len = plan.len_bytes ? reinterpret_cast<int*>(static_cast<char*>(ws) + plan.rows_bytes + plan.cols_bytes) : nullptr;
  cudaError_t e = cudaMemsetAsync(ws, 0, plan.total(), stream);
  if (e != cudaSuccess) { set_error("cudaMemsetAsync(mask bits): %s", cudaGetErrorString(e)); return NB200_ERR_LAUNCH; }
  const bool tiled = Sm == pr.S && pr.S % 256 == 0 && pr.T % 256 == 0 && pr.ms[3] == 1 && pr.ms[2] % 16 == 0 &&
                     (Bm == 1 || pr.ms[0] % 16 == 0) && (Hm == 1 || pr.ms[1] % 16 == 0) &&
                     reinterpret_cast<uintptr_t>(pr.mask) % 16 == 0;
  if (tiled) {
    dim3 grid(pr.T / 256, pr.S / 256, Bm * Hm);
    mask_pack_tile_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(pr.mask), pr.ms[0], pr.ms[1], pr.ms[2], Hm,
                                                    pr.S, pr.T, rows, plan.words_per_row, cols, plan.words_per_col);
  } else {
    dim3 grid((pr.T + 31) / 32, (n_rows + 31) / 32, Bm * Hm);
    mask_pack_kernel<<<grid, 256, 0, stream>>>(pr.mask, pr.ms[0], pr.ms[1], pr.ms[2], pr.ms[3], Hm, Sm, pr.S, pr.T, rows,
                                               plan.words_per_row, cols, plan.words_per_col, kv_len);
  }
  count_launch();
  if (int rc = check_launch(tiled ? "mask_pack_tile_kernel" : "mask_pack_kernel")) return rc;
  mask_views(pr, plan, ws, out);
  return NB200_OK;
}

}  // namespace tc

// ---- coverage gate -----------------------------------------------------------
namespace {

struct BiasPlan { int mode; };

bool bias_plan(const Problem& pr, int dtype, int bias_dtype, BiasPlan* bp, const char** why) {
  bp->mode = tc::kBiasNone;
  if (!pr.bias) return true;
  if (bias_dtype != dtype) { *why = "bias dtype differs from q/k/v dtype"; return false; }
  const bool row_bc = pr.bs[2] == 0 || pr.S == 1;
  if (pr.T > 1 && pr.bs[3] != 1) { *why = "bias needs a unit stride over keys"; return false; }
  if (row_bc) {
    // with a positive scale the per-key bias is read element by element (and added by the tensor core); only the
    // path for other scales reads it in 16-byte vectors
    const bool scalar_reads = pr.scale > 0.f && isfinite(1.f / pr.scale);
    if (!scalar_reads && (reinterpret_cast<uintptr_t>(pr.bias) % 16 || pr.bs[0] % 8 || pr.bs[1] % 8 || pr.T % 8)) {
      *why = "per-key bias is not 16-byte aligned";
      return false;
    }
    bp->mode = tc::kBiasKey;
    return true;
  }
  if (!tc::tile_map_ok(pr.bias, pr.bs[2], pr.bs[1], pr.bs[0], pr.H, pr.B, true)) {
    *why = "bias strides / alignment do not fit a TMA descriptor";
    return false;
  }
  bp->mode = tc::kBiasTile;
  return true;
}

}  // namespace

bool tc_supported(const Problem& original, int dtype, int bias_dtype, int pass, const char** why) {
  const char* dummy;
  if (!why) why = &dummy;
  // judged on the problem as the kernels will see it (operands with awkward layouts go through padded copies)
  const tc::Staging sg = tc::plan_staging(original, pass);
  const Problem pr = tc::staged_view(original, sg, nullptr);
  if (dtype != NB200_BF16 && dtype != NB200_F16) { *why = "dtype is not bf16/fp16"; return false; }
  if (pr.D != pr.Dv || (pr.D != 64 && pr.D != 128)) { *why = "head dims must be equal and 64 or 128"; return false; }
  // Lengths need not fill whole 128-row tiles, nor be multiples of anything: TMA zero-fills rows past the end, the
  // kernels mask keys past T and store only rows below S, and the operands with 16-byte row segments (bias, dbias,
  // lse, delta) are staged through padded copies when the lengths leave those segments ragged.
  if (pr.bh_count > 65535 || int64_t(pr.B) * pr.H > 65535) {
    *why = "more than 65535 (batch, head) pairs (grid limit of the backward and mask-packing launches)";
    return false;
  }
  if (pr.S <= 0 || pr.T <= 0) {
    *why = "query and key lengths must be positive";
    return false;
  }
  if (!tc::tile_map_ok(pr.q, pr.qs[2], pr.qs[1], pr.qs[0], pr.H, pr.B, false) ||
      !tc::tile_map_ok(pr.k, pr.ks[2], pr.ks[1], pr.ks[0], pr.H, pr.B, false) ||
      !tc::tile_map_ok(pr.v, pr.vs[2], pr.vs[1], pr.vs[0], pr.H, pr.B, false)) {
    *why = "q/k/v strides or alignment do not fit a TMA descriptor (expanded views over batch / heads included)";
    return false;
  }
  if (reinterpret_cast<uintptr_t>(pr.out) % 16 || pr.os[0] % 8 || pr.os[1] % 8 || pr.os[2] % 8) {
    *why = "out is not 16-byte aligned";
    return false;
  }
  BiasPlan bp;
  if (!bias_plan(pr, dtype, bias_dtype, &bp, why)) return false;
  if (pass == NB200_PASS_BWD) return tc::bwd_supported(pr, dtype, bias_dtype, why);
  return true;
}

size_t tc_workspace_bytes(const Problem& pr, int dtype, int bias_dtype, int pass) {
  const tc::Staging sg = tc::plan_staging(pr, pass);
  if (pass == NB200_PASS_BWD)
    return (tc::bwd_workspace_bytes(tc::staged_view(pr, sg, nullptr), dtype, bias_dtype) + 255) / 256 * 256 + sg.total();
  size_t bytes = 0;
  tc::mask_plan_for_pass(pr, false, &bytes);
  return (bytes + 255) / 256 * 256 + sg.total();
}

int tc_forward(const Problem& original, int dtype, int bias_dtype, void* ws, size_t ws_bytes, cudaStream_t stream) {
  const char* why = "";
  size_t mask_ws = 0;
  const tc::MaskPackPlan mp = tc::mask_plan_for_pass(original, false, &mask_ws);
  const tc::Staging sg = tc::plan_staging(original, NB200_PASS_FWD);
  const size_t staging_off = (mask_ws + 255) / 256 * 256;
  if (staging_off + sg.total() > ws_bytes || ((mask_ws || sg.total()) && !ws)) {
    set_error("forward needs %zu workspace bytes (mask bits, padded bias)", staging_off + sg.total());
    return NB200_ERR_WORKSPACE;
  }
  const Problem pr = tc::staged_view(original, sg, static_cast<char*>(ws) + staging_off);
  if (int rc = tc::stage_in(original, pr, sg, NB200_PASS_FWD, stream)) return rc;
  BiasPlan bp;
  if (!bias_plan(pr, dtype, bias_dtype, &bp, &why)) { set_error("%s", why); return NB200_ERR_UNSUPPORTED; }
  tc::FwdArgs a{};
  if (int rc = tc::launch_mask_pack(pr, mp, ws, &a.mask, stream)) return rc;
  CUtensorMap tq, tk, tv, tb;
  if (!tc::make_tile_map(&tq, pr.q, pr.S, pr.D, pr.H, pr.B, pr.qs[2], pr.qs[1], pr.qs[0], tc::kTile, &why) ||
      !tc::make_tile_map(&tk, pr.k, pr.T, pr.D, pr.H, pr.B, pr.ks[2], pr.ks[1], pr.ks[0], tc::kTile, &why) ||
      !tc::make_tile_map(&tv, pr.v, pr.T, pr.Dv, pr.H, pr.B, pr.vs[2], pr.vs[1], pr.vs[0], tc::kTile, &why)) {
    set_error("tensor map: %s", why);
    return NB200_ERR_LAUNCH;
  }
  tb = tq;  // placeholder when the bias is not tiled (never dereferenced)
  if (bp.mode == tc::kBiasTile &&
      !tc::make_tile_map(&tb, pr.bias, pr.S, pr.T, pr.H, pr.B, pr.bs[2], pr.bs[1], pr.bs[0], tc::kTile, &why)) {
    set_error("bias tensor map: %s", why);
    return NB200_ERR_LAUNCH;
  }
  a.H = pr.H; a.S = pr.S; a.T = pr.T; a.bh_begin = pr.bh_begin;
  a.causal = pr.causal; a.scale = pr.scale;
  a.bias_mode = bp.mode;
  a.bias_b_mul = (pr.B > 1 && pr.bs[0] != 0) ? 1 : 0;
  a.bias_h_mul = (pr.H > 1 && pr.bs[1] != 0) ? 1 : 0;
  a.bias = pr.bias; a.bias_bs = pr.bs[0]; a.bias_hs = pr.bs[1];
  a.bias_mma = 0;
  if (pr.D == 64 && bp.mode == tc::kBiasTile && pr.scale > 0.f &&
      tc::split_inv_scale(pr.scale, dtype == NB200_BF16, &a.inv_scale_hi, &a.inv_scale_lo))
    a.bias_mma = 1;
  a.key_mma = 0;
  if (bp.mode != tc::kBiasTile && pr.scale > 0.f && isfinite(1.f / pr.scale) &&
      (bp.mode == tc::kBiasKey || a.mask.kv_len != nullptr))
    a.key_mma = 1;
  a.out = pr.out;
  for (int i = 0; i < 3; ++i) a.os[i] = pr.os[i];
  a.lse = pr.lse;
  a.n_out_peers = pr.n_out_peers;
  for (int i = 0; i < pr.n_out_peers; ++i) {
    a.out_peers[i] = pr.out_peers[i];
    if (reinterpret_cast<uintptr_t>(pr.out_peers[i]) % 32 || pr.os[0] % 16 || pr.os[1] % 16 || pr.os[2] % 16) {
      set_error("fused output all-gather: peer rows must be 32-byte aligned");
      return NB200_ERR_ALIGNMENT;
    }
  }
  a.status = device_status_word();
  if (!a.status) { set_error("device status word is unavailable"); return NB200_ERR_LAUNCH; }
  a.B = pr.B;
  a.bh_count = pr.bh_count;
  a.n_qblocks = (pr.S + 2 * tc::kTile - 1) / (2 * tc::kTile);
  // the whole (batch, head) range: order the items head-major / query block / batch (see decode_item)
  a.head_major = (pr.bh_begin == 0 && pr.bh_count == pr.B * pr.H) ? 1 : 0;
  // causal items differ in length by up to the number of key tiles; with few items per CTA that imbalance costs
  // more than the K / V locality of the head-major order
  if (a.head_major && pr.causal && int64_t(a.n_qblocks) * pr.bh_count <= 16 * int64_t(tc::sm_count())) a.head_major = 2;
  // key padding: items by kept length, longest first (the kernel ranks the batch elements itself)
  if (a.head_major && !pr.causal && a.mask.kv_len && a.mask.len_h_stride == 0 && a.mask.len_b_stride != 0 && pr.B > 1 && pr.B <= 384)
    a.head_major = 3;
  return tc::launch_fwd(pr.D, dtype == NB200_BF16, tq, tk, tv, tb, a, stream);
}

size_t tc_mask_pack_bytes(const Problem& pr, bool with_transpose) {
  if (!pr.mask) return 0;
  return tc::plan_mask_pack(pr, with_transpose && !tc::mask_key_only(pr)).total();
}

int tc_mask_pack(const Problem& pr, bool with_transpose, void* packed, size_t packed_bytes, cudaStream_t stream) {
  if (!pr.mask) return NB200_OK;
  if (pr.mask_packed) { set_error("the mask is already packed"); return NB200_ERR_INVALID; }
  const tc::MaskPackPlan mp = tc::plan_mask_pack(pr, with_transpose && !tc::mask_key_only(pr));
  if (!packed || packed_bytes < mp.total()) {
    set_error("the packed mask needs %zu bytes, got %zu", mp.total(), packed ? packed_bytes : size_t(0));
    return NB200_ERR_WORKSPACE;
  }
  if (reinterpret_cast<uintptr_t>(packed) % 256) { set_error("the packed-mask buffer must be 256-byte aligned"); return NB200_ERR_ALIGNMENT; }
  tc::MaskBits unused;
  return tc::launch_mask_pack(pr, mp, packed, &unused, stream);
}

int tc_backward(const Problem& original, int dtype, int bias_dtype, void* ws, size_t ws_bytes, cudaStream_t stream) {
  // padded copies (bias in; lse / delta rows; dbias out) sit behind the kernels' own scratch
  const tc::Staging sg = tc::plan_staging(original, NB200_PASS_BWD);
  const size_t inner = (tc::bwd_workspace_bytes(tc::staged_view(original, sg, nullptr), dtype, bias_dtype) + 255) / 256 * 256;
  if (inner + sg.total() > ws_bytes) {
    set_error("tensor-core backward needs %zu workspace bytes", inner + sg.total());
    return NB200_ERR_WORKSPACE;
  }
  const Problem pr = tc::staged_view(original, sg, static_cast<char*>(ws) + inner);
  if (int rc = tc::stage_in(original, pr, sg, NB200_PASS_BWD, stream)) return rc;
  if (int rc = tc::launch_bwd(pr, dtype, bias_dtype, ws, inner, sg.rows ? sg.Sp : original.S, stream)) return rc;
  return tc::stage_out(original, pr, sg, stream);
}

}  // namespace nb200
