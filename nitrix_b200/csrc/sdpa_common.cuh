// Shared host/device helpers of the attention kernels: the internal problem
// descriptor the C-ABI params are lowered to, dtype conversion, and the launch
// bookkeeping (error text, launch counter, device status word).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nitrix_b200_attention.h"

namespace nb200 {

constexpr float kLog2e = 1.4426950408889634f;

// Problem descriptor passed by value to every kernel.  Strides are in
// elements; a broadcast axis has stride 0.
struct Problem {
  int B, H, S, T, D, Dv;
  int bh_begin, bh_count;
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  const void* bias;
  const uint8_t* mask;
  const void* dout;
  void* dq;
  void* dk;
  void* dv;
  void* dbias;
  float* delta;        // (B,H,S) fp32 scratch: rowsum(out * dout)
  float* dbias_accum;  // fp32 scratch of bias' own (un-broadcast) extent, or null
  int64_t qs[3], ks[3], vs[3], os[3], dos[3], dqs[3], dks[3], dvs[3];  // b, h, row
  int64_t bs[4], ms[4], dbs[4];                                          // b, h, row, col
  float scale;
  int causal;
  int want_dbias;      // the backward produces a bias gradient (dbias may still be null while planning)
  int mask_packed;     // 0: byte mask; 1 / 2: `mask` is a buffer made by nb200_mask_pack (2: with the transposed copy)
  int n_out_peers;     // forward: further destinations of every output row (same strides as out)
  void* out_peers[NB200_MAX_OUT_PEERS];
};

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float load_as_f32(const void* base, int64_t idx, int dtype) {
  if (dtype == NB200_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == NB200_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

__device__ __forceinline__ void store_from_f32(void* base, int64_t idx, int dtype, float x) {
  if (dtype == NB200_F32) reinterpret_cast<float*>(base)[idx] = x;
  else if (dtype == NB200_BF16) reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(x);
  else reinterpret_cast<__half*>(base)[idx] = __float2half_rn(x);
}

__host__ __device__ __forceinline__ int dtype_size(int dtype) { return dtype == NB200_F32 ? 4 : 2; }

// ---- host-side bookkeeping (sdpa_api.cu) -----------------------------------
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
int check_launch(const char* what);
// Call once at the start of an entry point that launches kernels on `st` (per-kernel timing: nb200_profile).
void prof_call_begin(cudaStream_t st);
// Address (on the current device) of the status word bounded waits report to.
int* device_status_word();
// A second stream of the calling thread on the current device, with the two events of a fork / join: small problems
// run their two independent backward kernels side by side on it.  Created at first use; null when per-kernel timing
// is on (its events bracket kernels on ONE in-order stream), inside nb200_sdpa_bwd_static_scratch (which creates
// nothing), when `main` is being captured into a graph before the stream exists (nothing is created during a
// capture), or when creation fails -- callers then launch on their own stream.
struct SideStream { cudaStream_t stream; cudaEvent_t fork, join; };
const SideStream* side_stream(cudaStream_t main);
void forbid_side_stream(bool on);

// ---- SIMT kernels (sdpa_simt.cu) -------------------------------------------
int simt_forward(const Problem& pr, int dtype, int bias_dtype, cudaStream_t stream);
int simt_backward(const Problem& pr, int dtype, int bias_dtype, cudaStream_t stream);
// True when this family runs the problem's `pass` on its 3 x TF32 mma.sync kernels (fp32 operands) rather than on
// plain FMA units.
bool simt_family_uses_tensor_path(const Problem& pr, int dtype, int pass);
// delta = rowsum(out*dout) and, when dbias_accum is used, its zero-fill / final cast
int launch_delta(const Problem& pr, int dtype, cudaStream_t stream);
int launch_dbias_finish(const float* accum, void* dbias, int bias_dtype, const int64_t extent[4],
                        const int64_t stride[4], cudaStream_t stream);


// ---- tensor-core kernels (sdpa_tc_*.cu) -------------------------------------
// Returns true when the TMA + tcgen05 kernels cover the problem for `pass`;
// otherwise `why` (when non-null) receives a short reason.
bool tc_supported(const Problem& pr, int dtype, int bias_dtype, int pass, const char** why);
size_t tc_workspace_bytes(const Problem& pr, int dtype, int bias_dtype, int pass);
int tc_forward(const Problem& pr, int dtype, int bias_dtype, void* ws, size_t ws_bytes, cudaStream_t stream);
int tc_backward(const Problem& pr, int dtype, int bias_dtype, void* ws, size_t ws_bytes, cudaStream_t stream);
// Packing of the byte mask into the tensor-core kernels' bit layout, as a call of its own (nb200_mask_pack).
size_t tc_mask_pack_bytes(const Problem& pr, bool with_transpose);
int tc_mask_pack(const Problem& pr, bool with_transpose, void* packed, size_t packed_bytes, cudaStream_t stream);

}  // namespace nb200
