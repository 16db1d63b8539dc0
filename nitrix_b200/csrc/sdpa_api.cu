// C-ABI entry points (include/nitrix_b200_attention.h): validation, kernel
// selection, workspace carving and dispatch.  Nothing here allocates device
// memory or synchronises; every launch goes to the caller's stream.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "sdpa_common.cuh"

namespace nb200 {

static thread_local char g_error[512] = "";
static std::atomic<uint64_t> g_launches{0};

// Set by kernels whose bounded waits run out; read by nb200_device_status().
__device__ int g_device_status = 0;

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(uint64_t(n), std::memory_order_relaxed); }

// ---- optional per-kernel timing (nb200_profile / nb200_profile_read) ----------
// When enabled, an event is recorded on the launching stream after every kernel
// this library enqueues (and one at the start of each forward / backward call);
// consecutive events on the in-order stream bracket one kernel each.
namespace {
struct ProfMark { const char* name; cudaEvent_t ev; };
std::atomic<bool> g_prof_on{false};
std::mutex g_prof_mutex;
std::vector<ProfMark> g_prof_marks;
thread_local cudaStream_t g_prof_stream = nullptr;

void prof_mark(const char* name) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  cudaEvent_t ev;
  if (cudaEventCreate(&ev) != cudaSuccess) { cudaGetLastError(); return; }
  cudaEventRecord(ev, g_prof_stream);
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_prof_marks.push_back({name, ev});
}
}  // namespace

// Start of one entry point's kernels on `st`: the per-kernel timing brackets every kernel between this marker (or the
// previous kernel's) and its own.
void prof_call_begin(cudaStream_t st) {
  g_prof_stream = st;
  prof_mark(nullptr);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return NB200_ERR_LAUNCH;
  }
  prof_mark(what);
  return NB200_OK;
}

namespace {
thread_local bool g_no_side_stream = false;
}
void forbid_side_stream(bool on) { g_no_side_stream = on; }

const SideStream* side_stream(cudaStream_t main) {
  if (g_no_side_stream || g_prof_on.load(std::memory_order_relaxed)) return nullptr;
  static thread_local SideStream cache[64] = {};
  static thread_local bool made[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!made[dev]) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(main, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      return nullptr;
    }
    SideStream ss{};
    if (cudaStreamCreateWithFlags(&ss.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&ss.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ss.join, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cache[dev] = ss;
    made[dev] = true;
  }
  return &cache[dev];
}

int* device_status_word() {
  // the symbol's address is fixed per device: looked up once and remembered (host threads may race here)
  static std::atomic<int*> known[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev >= 0) {
    if (int* hit = known[dev].load(std::memory_order_acquire)) return hit;
  }
  int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_device_status) != cudaSuccess) return nullptr;
  if (dev >= 0) known[dev].store(p, std::memory_order_release);
  return p;
}

namespace {

constexpr size_t kAlign = 256;
inline size_t align_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

struct Lowered {
  Problem pr;
  int dtype, bias_dtype;
  bool bias_broadcast;        // some bias axis is broadcast over an extent > 1
  int64_t bias_extent[4];     // bias' own (un-broadcast) extents
  int64_t dbias_stride[4];    // caller's dbias strides
};

bool valid_dtype(int d) { return d == NB200_F32 || d == NB200_BF16 || d == NB200_F16; }

int lower(const nb200_sdpa_params* p, int pass, Lowered* out) {
  if (!p) { set_error("params is NULL"); return NB200_ERR_INVALID; }
  if (p->struct_size != sizeof(nb200_sdpa_params)) {
    set_error("params.struct_size=%u, library expects %zu (ABI mismatch)", p->struct_size,
              sizeof(nb200_sdpa_params));
    return NB200_ERR_INVALID;
  }
  if (!valid_dtype(p->dtype)) { set_error("unknown dtype %d", p->dtype); return NB200_ERR_INVALID; }
  if (p->bias && !valid_dtype(p->bias_dtype)) {
    set_error("unknown bias_dtype %d", p->bias_dtype);
    return NB200_ERR_INVALID;
  }
  if (p->B < 0 || p->H < 0 || p->S < 0 || p->T < 0 || p->D <= 0 || p->Dv <= 0) {
    set_error("negative extent or empty head dim (B=%d H=%d S=%d T=%d D=%d Dv=%d)", p->B, p->H, p->S, p->T,
              p->D, p->Dv);
    return NB200_ERR_INVALID;
  }
  const int64_t BH = int64_t(p->B) * p->H;
  if (p->bh_begin < 0 || p->bh_end < p->bh_begin || p->bh_end > BH) {
    set_error("bh range [%d, %d) outside [0, %lld)", p->bh_begin, p->bh_end, (long long)BH);
    return NB200_ERR_INVALID;
  }
  const bool empty = BH == 0 || p->S == 0 || p->bh_end == p->bh_begin;
  if (!empty) {
    if (!p->q || !p->k || !p->v || !p->out || !p->lse) {
      set_error("q, k, v, out and lse must be non-NULL");
      return NB200_ERR_INVALID;
    }
    if (pass == NB200_PASS_BWD && (!p->dout || !p->dq || !p->dk || !p->dv)) {
      set_error("dout, dq, dk and dv must be non-NULL for the backward pass");
      return NB200_ERR_INVALID;
    }
  }
  if (p->q_stride[3] != 1 || p->k_stride[3] != 1 || p->v_stride[3] != 1 || p->out_stride[3] != 1) {
    set_error("q, k, v and out need a unit stride on the head dimension");
    return NB200_ERR_INVALID;
  }
  if (pass == NB200_PASS_BWD &&
      (p->dout_stride[3] != 1 || p->dq_stride[3] != 1 || p->dk_stride[3] != 1 || p->dv_stride[3] != 1)) {
    set_error("dout, dq, dk and dv need a unit stride on the head dimension");
    return NB200_ERR_INVALID;
  }
  if (pass == NB200_PASS_BWD && (p->dbias || p->want_dbias) && !p->bias) {
    set_error("dbias requested without bias");
    return NB200_ERR_INVALID;
  }
  if (p->mask && (p->mask_is_bitpacked < 0 || p->mask_is_bitpacked > 2)) {
    set_error("mask_is_bitpacked must be 0, 1 or 2 (got %d)", p->mask_is_bitpacked);
    return NB200_ERR_INVALID;
  }
  if (p->n_out_peers < 0 || p->n_out_peers > NB200_MAX_OUT_PEERS) {
    set_error("n_out_peers must be in [0, %d] (got %d)", NB200_MAX_OUT_PEERS, p->n_out_peers);
    return NB200_ERR_INVALID;
  }
  Problem& pr = out->pr;
  memset(&pr, 0, sizeof(pr));
  pr.B = p->B; pr.H = p->H; pr.S = p->S; pr.T = p->T; pr.D = p->D; pr.Dv = p->Dv;
  pr.bh_begin = p->bh_begin; pr.bh_count = p->bh_end - p->bh_begin;
  pr.q = p->q; pr.k = p->k; pr.v = p->v; pr.out = p->out; pr.lse = p->lse;
  pr.bias = p->bias; pr.mask = p->mask;
  pr.scale = p->scale; pr.causal = p->causal != 0;
  pr.mask_packed = p->mask ? p->mask_is_bitpacked : 0;
  pr.want_dbias = (pass == NB200_PASS_BWD && (p->dbias || p->want_dbias)) ? 1 : 0;
  if (pass == NB200_PASS_FWD) {
    pr.n_out_peers = p->n_out_peers;
    for (int i = 0; i < p->n_out_peers; ++i) {
      if (!p->out_peers[i]) { set_error("out_peers[%d] is NULL", i); return NB200_ERR_INVALID; }
      pr.out_peers[i] = p->out_peers[i];
    }
  }
  for (int a = 0; a < 3; ++a) {
    pr.qs[a] = p->q_stride[a]; pr.ks[a] = p->k_stride[a]; pr.vs[a] = p->v_stride[a];
    pr.os[a] = p->out_stride[a];
  }
  for (int a = 0; a < 4; ++a) { pr.bs[a] = p->bias ? p->bias_stride[a] : 0; pr.ms[a] = p->mask ? p->mask_stride[a] : 0; }
  out->dtype = p->dtype;
  out->bias_dtype = p->bias ? p->bias_dtype : p->dtype;
  out->bias_broadcast = false;
  const int64_t full[4] = {p->B, p->H, p->S, p->T};
  for (int a = 0; a < 4; ++a) {
    const bool bc = !p->bias || p->bias_stride[a] == 0 || full[a] == 1;
    out->bias_extent[a] = bc ? 1 : full[a];
    if (p->bias && p->bias_stride[a] == 0 && full[a] > 1) out->bias_broadcast = true;
    out->dbias_stride[a] = p->dbias_stride[a];
  }
  if (pass == NB200_PASS_BWD) {
    pr.dout = p->dout; pr.dq = p->dq; pr.dk = p->dk; pr.dv = p->dv; pr.dbias = p->dbias;
    for (int a = 0; a < 3; ++a) {
      pr.dos[a] = p->dout_stride[a]; pr.dqs[a] = p->dq_stride[a]; pr.dks[a] = p->dk_stride[a];
      pr.dvs[a] = p->dv_stride[a];
    }
    for (int a = 0; a < 4; ++a) pr.dbs[a] = out->bias_extent[a] == 1 ? 0 : p->dbias_stride[a];
  }
  return NB200_OK;
}

int choose(const nb200_sdpa_params* p, const Lowered& lw, int pass, int* kernel) {
  const char* why = "";
  const bool tc = tc_supported(lw.pr, lw.dtype, lw.bias_dtype, pass, &why);
  if (p->kernel == NB200_KERNEL_TCGEN05) {
    if (!tc) { set_error("tcgen05 kernels do not cover this problem: %s", why); return NB200_ERR_UNSUPPORTED; }
    *kernel = NB200_KERNEL_TCGEN05;
    return NB200_OK;
  }
  if (p->kernel != NB200_KERNEL_AUTO && p->kernel != NB200_KERNEL_SIMT) {
    set_error("unknown kernel family %d", p->kernel);
    return NB200_ERR_INVALID;
  }
  if (p->kernel == NB200_KERNEL_AUTO && tc) { *kernel = NB200_KERNEL_TCGEN05; return NB200_OK; }
  if (lw.pr.bh_count > 65535) {
    // the CUDA-core launches put the (batch, head) index on grid.y
    set_error("more than 65535 (batch, head) pairs in one call (%d): split the range with bh_begin / bh_end",
              lw.pr.bh_count);
    return NB200_ERR_UNSUPPORTED;
  }
  if (lw.pr.D > 256 || lw.pr.Dv > 256) {
    set_error("head dims above 256 are not supported (D=%d Dv=%d)", lw.pr.D, lw.pr.Dv);
    return NB200_ERR_UNSUPPORTED;
  }
  if (lw.pr.mask_packed) {
    set_error("a bit-packed mask is consumed by the tensor-core kernels only, and they do not cover this problem (%s): "
              "pass the byte mask", why);
    return NB200_ERR_UNSUPPORTED;
  }
  if (lw.pr.n_out_peers > 0) {
    set_error("the fused output all-gather needs the tensor-core kernels, and they do not cover this problem (%s)", why);
    return NB200_ERR_UNSUPPORTED;
  }
  *kernel = NB200_KERNEL_SIMT;
  return NB200_OK;
}

// backward scratch shared by both families: delta, then the optional fp32
// accumulator for a broadcast bias gradient; family-specific scratch follows.
struct BwdScratch { size_t delta_off, accum_off, family_off, total; int64_t accum_elems; };

BwdScratch bwd_scratch(const nb200_sdpa_params* p, const Lowered& lw, size_t family_bytes) {
  BwdScratch s{};
  size_t off = 0;
  s.delta_off = off;
  off += align_up(sizeof(float) * size_t(p->B) * p->H * p->S);
  s.accum_off = off;
  s.accum_elems = 0;
  if ((p->dbias || p->want_dbias) && lw.bias_broadcast) {
    s.accum_elems = lw.bias_extent[0] * lw.bias_extent[1] * lw.bias_extent[2] * lw.bias_extent[3];
    off += align_up(sizeof(float) * size_t(s.accum_elems));
  }
  s.family_off = off;
  off += align_up(family_bytes);
  s.total = off;
  return s;
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" {

NB200_API int nb200_version(void) { return NB200_ABI_VERSION; }

NB200_API const char* nb200_last_error(void) { return g_error; }

NB200_API uint64_t nb200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

NB200_API int nb200_device_status(int device) {
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    set_error("cudaSetDevice(%d) failed", device);
    return NB200_ERR_INVALID;
  }
  int word = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&word, g_device_status, sizeof(int));
  if (e == cudaSuccess && word != 0) e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  if (prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) {
    set_error("reading the device status word: %s", cudaGetErrorString(e));
    return NB200_ERR_LAUNCH;
  }
  if (word != 0) {
    set_error("a device-side bounded wait expired (code %d)", word);
    return NB200_ERR_TIMEOUT;
  }
  return NB200_OK;
}

NB200_API int nb200_profile(int enable) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  for (auto& m : g_prof_marks) cudaEventDestroy(m.ev);
  g_prof_marks.clear();
  g_prof_on.store(enable != 0, std::memory_order_relaxed);
  return NB200_OK;
}

NB200_API size_t nb200_profile_read(char* buf, size_t bytes) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  std::map<std::string, std::pair<long, double>> agg;   // name -> (launches, total ms)
  for (size_t i = 1; i < g_prof_marks.size(); ++i) {
    if (!g_prof_marks[i].name) continue;                // a call's start marker brackets nothing
    if (cudaEventSynchronize(g_prof_marks[i].ev) != cudaSuccess) { cudaGetLastError(); continue; }
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, g_prof_marks[i - 1].ev, g_prof_marks[i].ev) != cudaSuccess) { cudaGetLastError(); continue; }
    auto& a = agg[g_prof_marks[i].name];
    a.first += 1;
    a.second += ms;
  }
  std::string out;
  char line[256];
  for (auto& kv : agg) {
    snprintf(line, sizeof(line), "%s\t%ld\t%.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
    out += line;
  }
  if (buf && bytes) {
    const size_t n = out.size() < bytes - 1 ? out.size() : bytes - 1;
    memcpy(buf, out.data(), n);
    buf[n] = 0;
  }
  return out.size() + 1;
}

NB200_API int nb200_sdpa_plan(const nb200_sdpa_params* p, int pass, int* kernel) {
  if (!kernel) { set_error("kernel out-pointer is NULL"); return NB200_ERR_INVALID; }
  Lowered lw;
  if (int rc = lower(p, pass, &lw)) return rc;
  if (int rc = choose(p, lw, pass, kernel)) return rc;
  if (*kernel == NB200_KERNEL_SIMT && simt_family_uses_tensor_path(lw.pr, lw.dtype, pass)) *kernel = NB200_KERNEL_MMA_TF32X3;
  return NB200_OK;
}

NB200_API int nb200_sdpa_workspace_bytes(const nb200_sdpa_params* p, int pass, size_t* bytes) {
  if (!bytes) { set_error("bytes out-pointer is NULL"); return NB200_ERR_INVALID; }
  Lowered lw;
  if (int rc = lower(p, pass, &lw)) return rc;
  int kernel = 0;
  if (int rc = choose(p, lw, pass, &kernel)) return rc;
  const size_t fam = kernel == NB200_KERNEL_TCGEN05 ? tc_workspace_bytes(lw.pr, lw.dtype, lw.bias_dtype, pass) : 0;
  *bytes = pass == NB200_PASS_FWD ? align_up(fam) : bwd_scratch(p, lw, fam).total;
  return NB200_OK;
}

NB200_API int nb200_mask_pack_bytes(const nb200_sdpa_params* p, int with_transpose, size_t* bytes) {
  if (!bytes) { set_error("bytes out-pointer is NULL"); return NB200_ERR_INVALID; }
  Lowered lw;
  if (int rc = lower(p, NB200_PASS_FWD, &lw)) return rc;
  if (lw.pr.mask_packed) { set_error("the mask is already packed"); return NB200_ERR_INVALID; }
  *bytes = align_up(tc_mask_pack_bytes(lw.pr, with_transpose != 0));
  return NB200_OK;
}

NB200_API int nb200_mask_pack(const nb200_sdpa_params* p, int with_transpose, void* packed, size_t packed_bytes,
                              void* cuda_stream) {
  Lowered lw;
  if (int rc = lower(p, NB200_PASS_FWD, &lw)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  g_prof_stream = st;
  prof_mark(nullptr);
  if (!lw.pr.mask || lw.pr.bh_count == 0 || lw.pr.S == 0 || lw.pr.T == 0) return NB200_OK;
  return tc_mask_pack(lw.pr, with_transpose != 0, packed, packed_bytes, st);
}

NB200_API int nb200_sdpa_fwd(const nb200_sdpa_params* p, void* cuda_stream) {
  Lowered lw;
  if (int rc = lower(p, NB200_PASS_FWD, &lw)) return rc;
  int kernel = 0;
  if (int rc = choose(p, lw, NB200_PASS_FWD, &kernel)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  g_prof_stream = st;
  prof_mark(nullptr);   // start of this call's kernels
  if (lw.pr.bh_count == 0 || lw.pr.S == 0) return NB200_OK;
  if (kernel == NB200_KERNEL_TCGEN05) {
    const size_t need = tc_workspace_bytes(lw.pr, lw.dtype, lw.bias_dtype, NB200_PASS_FWD);
    if (need && (!p->workspace || p->workspace_bytes < need)) {
      set_error("forward needs %zu workspace bytes, got %zu", need, p->workspace ? p->workspace_bytes : size_t(0));
      return NB200_ERR_WORKSPACE;
    }
    return tc_forward(lw.pr, lw.dtype, lw.bias_dtype, p->workspace, p->workspace_bytes, st);
  }
  return simt_forward(lw.pr, lw.dtype, lw.bias_dtype, st);
}

NB200_API int nb200_sdpa_bwd(const nb200_sdpa_params* p, void* cuda_stream) {
  Lowered lw;
  if (int rc = lower(p, NB200_PASS_BWD, &lw)) return rc;
  int kernel = 0;
  if (int rc = choose(p, lw, NB200_PASS_BWD, &kernel)) return rc;
  if (p->want_dbias && !p->dbias) {
    set_error("want_dbias is set but dbias is NULL");
    return NB200_ERR_INVALID;
  }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  g_prof_stream = st;
  prof_mark(nullptr);   // start of this call's kernels
  if (lw.pr.bh_count == 0) return NB200_OK;
  const size_t fam = kernel == NB200_KERNEL_TCGEN05 ? tc_workspace_bytes(lw.pr, lw.dtype, lw.bias_dtype, NB200_PASS_BWD) : 0;
  const BwdScratch sc = bwd_scratch(p, lw, fam);
  if (!p->workspace || p->workspace_bytes < sc.total) {
    set_error("backward needs %zu workspace bytes, got %zu", sc.total, p->workspace ? p->workspace_bytes : size_t(0));
    return NB200_ERR_WORKSPACE;
  }
  if (reinterpret_cast<uintptr_t>(p->workspace) % kAlign) {
    set_error("workspace must be %zu-byte aligned", kAlign);
    return NB200_ERR_ALIGNMENT;
  }
  char* ws = static_cast<char*>(p->workspace);
  Problem& pr = lw.pr;
  pr.delta = reinterpret_cast<float*>(ws + sc.delta_off);
  if (sc.accum_elems) {
    pr.dbias_accum = reinterpret_cast<float*>(ws + sc.accum_off);
    // dense strides over bias' own extent; broadcast axes collapse to stride 0
    int64_t st_dense = 1;
    for (int a = 3; a >= 0; --a) {
      pr.dbs[a] = lw.bias_extent[a] == 1 ? 0 : st_dense;
      st_dense *= lw.bias_extent[a];
    }
    cudaError_t e = cudaMemsetAsync(pr.dbias_accum, 0, sizeof(float) * size_t(sc.accum_elems), st);
    if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return NB200_ERR_LAUNCH; }
  }
  if (pr.S > 0) {
    if (int rc = launch_delta(pr, lw.dtype, st)) return rc;
  }
  int rc;
  if (kernel == NB200_KERNEL_TCGEN05)
    rc = tc_backward(pr, lw.dtype, lw.bias_dtype, ws + sc.family_off, fam, st);
  else
    rc = simt_backward(pr, lw.dtype, lw.bias_dtype, st);
  if (rc) return rc;
  if (sc.accum_elems)
    return launch_dbias_finish(pr.dbias_accum, pr.dbias, lw.bias_dtype, lw.bias_extent, lw.dbias_stride, st);
  return NB200_OK;
}

}  // extern "C"
