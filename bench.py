#!/usr/bin/env python
"""Benchmark of the attention hot path: forward + backward TFLOP/s on B200.

``python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c1|c2|c4|c5] [--impl ours|reference]``

A *step* is one forward + backward pass of ``scaled_dot_product_attention`` over one synthetic batch of the named
workload (the five benchmark configurations).  The default, and the headline ``value``, is ``c3`` -- bf16, B=4, H=32,
L=4096, D=128, per-batch bias with gradient, (B,1,L,L) boolean mask -- the largest configuration that one GPU holds
and the only one with a bias gradient and a full mask.  Throughput counts ALGORITHMIC flops only:
``14 * B * H * S * T_eff * D`` per step (4 forward + 10 backward; causal halves the pairs, key padding counts kept
keys only); softmax work is not counted.

Timing.  One step is captured into a CUDA graph (same kernels, same buffers as eager launches).  The timed region is
R blocks of K replays (K = ``--steps``), each block bracketed by a barrier + synchronize and two CUDA events; R is
chosen so that the region lasts about a second, which lets the GPU reach the clock it sustains under load and gives
the clock sampler time to see it.  ``ms_per_step`` is the median block (max over ranks); the spread of the blocks is
reported beside it.

Rank 0 prints ONE JSON line:

* ``value``: whole-job TFLOP/s of the headline workload with operands resident in HBM (multi-GPU: every rank runs
  the full workload on its own batch -> weak scaling, no collective);
* ``e2e``: the same metric through the public entry point with HOST (pinned) operands: H2D of q, k, v, bias, mask,
  dout and D2H of out, dq, dk, dv (dbias) inside the timed region;
* ``roofline``: achieved vs measured peak for the kernel that dominates the step;
* ``workloads`` (1 GPU): the same measurement for each of the five configurations;
* ``partition`` (N > 1): the split the configurations name -- c5 with 16 / N heads per GPU, c4 with 32 / N sequences
  per GPU (strong scaling through ``bh_begin / bh_end``-style slices), with the optional output all-gather timed
  both as an NCCL collective after the kernels and fused into the forward kernel's epilogue;
* ``cpu_baseline``: the CPU oracle (torch, all host threads) on a fixed, bounded sample;
* ``layer_norm`` (1 GPU): the sibling op on the shapes the reference's own norm benchmark uses -- time per forward
  and per backward call, and the algorithmic bytes each moves per second against the measured copy bandwidth;
* ``selective_scan`` (1 GPU): the second sibling op on a Mamba-block shape, time per forward and backward call.

``--impl reference`` times only that CPU implementation (the reference's own ``jnp`` path cannot run: jax is not
installed; the op-for-op torch restatement stands in, ``cpu_baseline.kind = "port"``).
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time

# the CPU arm uses every host core; torchrun pins OMP_NUM_THREADS=1 for its children, so lift that before torch loads
if "reference" in sys.argv or "--impl=reference" in sys.argv:
    os.environ["OMP_NUM_THREADS"] = os.environ["MKL_NUM_THREADS"] = str(os.cpu_count() or 1)

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

# Share of a step's ALGORITHMIC flops (14 S T_eff D per (batch, head): QK^T, PV forward; QK^T, dO V^T, P^T dO,
# dS^T Q, dS K backward) attributed to each kernel.  The query-major backward recomputes QK^T and dO V^T, which
# the key-major kernel is already credited with; only its dS K product counts.
KERNEL_FLOP_SHARE = {
    "sdpa_fwd_tc_kernel": 4 / 14,
    "sdpa_bwd_tc_kernel<key-major>": 8 / 14,
    "sdpa_bwd_tc_kernel<query-major>": 2 / 14,
    "sdpa_bwd_tc_kernel<merged>": 10 / 14,      # one kernel for dq, dk, dv
    "sdpa_bwd_tc_kernel<one-pass d128>": 10 / 14,
    "fwd_tf32x3_kernel": 4 / 14,
    "bwd_dkv_tf32x3_kernel": 8 / 14,
    "bwd_dq_tf32x3_kernel": 2 / 14,
    "simt_fwd_kernel": 4 / 14,
    "simt_fwd_tiled_kernel": 4 / 14,
    "simt_bwd_dkv_kernel": 8 / 14,
    "simt_bwd_dq_kernel": 2 / 14,
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures summarised
# under profiles/ (each entry names its summary).  Filled in only for kernels whose capture was taken from the build
# that is being timed; a workload without an entry reports traffic = null.
NCU_TRAFFIC_BYTES = {
    # profiles/c3_b1_attention_kernels_ncu_full.md: captured at batch 1 (the recipe's size rule), x 4 for the bench's
    # batch 4 -- every (batch, head) pair has its own bias / dbias, so traffic grows in proportion
    "c3": {"sdpa_bwd_tc_kernel<one-pass d128>": 4 * (1.355364e9 + 1.181375e9), "sdpa_fwd_tc_kernel": 4 * (1.191293e9 + 0.039252e9)},
    # profiles/c2_attention_kernels_ncu_full.md, profiles/c4_attention_kernels_ncu_full.md: captured at full size
    "c2": {"sdpa_bwd_tc_kernel<merged>": 671.002368e6 + 123.455744e6, "sdpa_fwd_tc_kernel": 250.225664e6 + 25.214464e6},
    "c4": {"sdpa_bwd_tc_kernel<merged>": 176.488704e6 + 84.309760e6, "sdpa_fwd_tc_kernel": 74.746368e6 + 6.363136e6},
}

METRIC = "fwd+bwd attention TFLOP/s"
UNIT = "TFLOP/s"
HEADLINE = "c3"

WORKLOADS = {
    "c1": dict(B=2, H=4, L=256, D=64, dtype="f32", desc="fp32 B2 H4 L256 D64 bias(B,H,L,L)+dBias key-mask"),
    "c2": dict(B=8, H=16, L=2048, D=64, dtype="bf16", desc="bf16 B8 H16 L2048 D64 causal ALiBi bias(1,H,L,L)"),
    "c3": dict(B=4, H=32, L=4096, D=128, dtype="bf16", desc="bf16 B4 H32 L4096 D128 bias(B,H,L,L)+dBias mask(B,1,L,L)"),
    "c4": dict(B=32, H=8, L=1024, D=64, dtype="f16", desc="fp16 B32 H8 L1024 D64 key-padding mask"),
    "c5": dict(B=1, H=16, L=65536, D=128, dtype="bf16", desc="bf16 B1 H16 L65536 D128 causal key-bias(1,H,1,L)"),
}
# fixed CPU-oracle samples (batch, head pairs; c5 additionally a block of query rows): the same sample every run
CPU_SAMPLE_PAIRS = {"c1": 8, "c2": 8, "c3": 4, "c4": 8, "c5": 2}
L2_BYTES = 126e6


def workload_bytes(name, B=None, H=None):
    """Algorithmic bytes of one step: every operand once per pass at its stored dtype and un-broadcast size."""
    w = WORKLOADS[name]
    B, H, L, D = B or w["B"], H or w["H"], w["L"], w["D"]
    esz = 4 if w["dtype"] == "f32" else 2
    qkv = B * H * L * D * esz
    by = 4 * qkv + B * H * L * 4                    # fwd: q k v out lse
    by += 8 * qkv + 2 * B * H * L * 4               # bwd: q k v out dout dq dk dv lse delta
    bias = {"c1": B * H * L * L, "c2": H * L * L, "c3": B * H * L * L, "c4": 0, "c5": H * L}[name] * esz
    by += 2 * bias + (bias if name in ("c1", "c3") else 0)
    mask = {"c1": B * L, "c2": 0, "c3": B * L * L, "c4": B * L, "c5": 0}[name]
    return float(by + 2 * mask)


def make_config(name, world, batch=None):
    """The `config` object of the JSON line; identical for the GPU arm and the CPU reference arm."""
    w = WORKLOADS[name]
    b = batch or w["B"]
    ws = workload_bytes(name, B=b)
    cfg = {"workload": f"{name}: {w['desc']}" + (f" [batch overridden to {batch}]" if batch else ""),
           "per_gpu_batch": b, "global_batch": b * world,
           "sharding": f"dp{world} over batch x heads, no collective",
           "launch": "CUDA graph replay of one fwd+bwd step",
           "l2": ("L2 flushed between steps" if ws < 2 * L2_BYTES else f"operands ({ws / 1e6:.0f} MB) exceed the 126 MB L2")}
    return cfg


def build_workload(name, device, seed=0, B=None, H=None, L=None):
    """Synthetic operands of the workload on `device` (seeded), plus flop / byte accounting."""
    import _cases

    w = WORKLOADS[name]
    B = B or w["B"]
    H = H or w["H"]
    L = L or w["L"]
    D = w["D"]
    want_dbias = name in ("c1", "c3")
    if name == "c1":
        q, k, v, kw = _cases.config1()
        q, k, v = q.to(device), k.to(device), v.to(device)
        kw = {k_: (v_.to(device) if torch.is_tensor(v_) else v_) for k_, v_ in kw.items()}
    else:
        builder = getattr(_cases, "config" + name[1])
        q, k, v, kw = builder(B=B, H=H, L=L, D=D, device=device, seed=seed)
    mask = kw.get("mask")
    causal = bool(kw.get("causal", False))
    pairs = float(B * H) * L * L
    if causal:
        pairs *= 0.5 * (1.0 + 1.0 / L)
    if name == "c4":
        pairs = float(H) * L * float(mask.reshape(B, L).sum().item())
    flops = 14.0 * pairs * D
    return dict(q=q, k=k, v=v, kw=kw, want_dbias=want_dbias, flops=flops, bytes=workload_bytes(name, B=B, H=H),
                B=B, H=H, L=L, D=D)


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs (NVML in a thread; read-only queries)."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index, period_s=0.02):
        self.index, self.period, self.samples, self.stop = index, period_s, [], threading.Event()
        self.thread, self.handle, self.nvml, self.max_mhz = None, None, None, None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - no NVML: fall back to nvidia-smi below
            self.nvml = None

    @staticmethod
    def _physical_index(index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if index < len(ids) and ids[index].isdigit():
                return int(ids[index])
        return index

    def _poll_nvml(self):
        n = self.nvml
        while not self.stop.is_set():
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                reasons = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)) if hasattr(
                    n, "nvmlDeviceGetCurrentClocksEventReasons") else int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                util = int(n.nvmlDeviceGetUtilizationRates(self.handle).gpu)
                self.samples.append((mhz, reasons, util))
            except Exception:  # noqa: BLE001
                pass
            self.stop.wait(self.period)

    def _poll_smi(self):
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={fields}",
                                     "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                    stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.proc = proc
        for line in proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz, self.max_mhz = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            bits = 0
            for (name, bit), val in zip(self.REASONS, parts[2:6]):
                if val.lower().startswith("active"):
                    bits |= bit
            self.samples.append((mhz, bits, 100))
            if self.stop.is_set():
                break

    def __enter__(self):
        self.thread = threading.Thread(target=self._poll_nvml if self.nvml else self._poll_smi, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop.set()
        proc = getattr(self, "proc", None)
        if proc is not None:
            proc.terminate()   # the exact child started above
            try:
                proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        loaded = [s for s in self.samples if s[2] >= 50] or self.samples
        if not loaded:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        bits = 0
        for s in loaded:
            bits |= s[1]
        reasons = sorted(name for name, bit in self.REASONS if bits & bit)
        return {"sm_mhz": statistics.median(s[0] for s in loaded), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(loaded)}


def bind_near_gpu(index):
    """Pins this process to the host cores of the NUMA node its GPU hangs off (read from sysfs), so that the pinned
    staging buffers it allocates afterwards are placed in that node's memory and the ranks of a multi-GPU run do not
    all stream through one node.  Returns the node number, or None when the topology is not exposed."""
    try:
        prop = torch.cuda.get_device_properties(index)
        bus = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:  # noqa: BLE001 - no sysfs topology, or not permitted: keep the inherited affinity
        return None


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], burst=p["bf16_tflops"], sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, source="fallback")


def cpu_reference_step(wl_name, repeats=5, warmup=1):
    """Times the CPU oracle (fwd + autograd bwd, fp32, all host threads) on a FIXED bounded sample of the workload:
    the first n (batch, head) pairs (each pair is independent), for c5 additionally the last block of query rows.
    One warm-up run, then `repeats` runs; the median is reported.  Returns (TFLOP/s, cores, sample, seconds, spread)."""
    from oracle import sdpa_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    w = WORKLOADS[wl_name]
    L, rows = w["L"], w["L"]
    n_pairs = min(CPU_SAMPLE_PAIRS[wl_name], w["B"] * w["H"])
    if wl_name == "c5":
        rows = 512   # the last (fullest causal) block of 512 query rows against all keys

    if wl_name == "c5":
        g = torch.Generator().manual_seed(0)
        D = w["D"]
        q = torch.randn(1, n_pairs, rows, D, generator=g).bfloat16()
        k = torch.randn(1, n_pairs, L, D, generator=g).bfloat16()
        v = torch.randn(1, n_pairs, L, D, generator=g).bfloat16()
        bias = torch.randn(1, n_pairs, 1, L, generator=g).bfloat16()
        mask = (torch.arange(L)[None, :] <= (L - rows + torch.arange(rows))[:, None])
        dout = torch.randn(1, n_pairs, rows, D, generator=g).bfloat16()
        flops = 14.0 * float(n_pairs) * float(mask.sum().item()) * D
        args, kw, want = (q, k, v, dout), dict(bias=bias, mask=mask), False
    elif wl_name == "c1":
        sub = build_workload("c1", "cpu")
        dout = torch.randn(sub["q"].shape, generator=torch.Generator().manual_seed(5)).to(sub["q"].dtype)
        flops, args, kw, want = sub["flops"], (sub["q"], sub["k"], sub["v"], dout), dict(sub["kw"]), True
    else:
        sub = build_workload(wl_name, "cpu", B=1, H=n_pairs)
        dout = torch.randn(sub["q"].shape, generator=torch.Generator().manual_seed(5)).to(sub["q"].dtype)
        flops, args, kw, want = sub["flops"], (sub["q"], sub["k"], sub["v"], dout), dict(sub["kw"]), sub["want_dbias"]

    def run():
        t0 = time.perf_counter()
        O.reference_grads_torch(*args, want_dbias=want, **kw)
        return time.perf_counter() - t0

    for _ in range(max(1, warmup)):
        run()
    times = [run() for _ in range(max(3, repeats))]
    sec = statistics.median(times)
    total = w["B"] * w["H"]
    sample = (f"first {n_pairs} of {total} (batch, head) pairs"
              + (f", last {rows} query rows of L={L}" if wl_name == "c5" else f" at full L={L}")
              + f"; median of {len(times)} runs after {max(1, warmup)} warm-up")
    return flops / sec / 1e12, cores, sample, sec, [min(times), max(times)]


# ---------------------------------------------------------------------------------------------------------------
# GPU measurement of one workload (whole, or this rank's shard of it)
# ---------------------------------------------------------------------------------------------------------------
class Runner:
    """Operands of one workload on this rank's GPU and the step (fwd + bwd through the public entry point)."""

    def __init__(self, name, dev, backend, seed=0, B=None, H=None):
        from nitrix_b200.nn import attention as att

        self.att, self.name, self.dev, self.backend = att, name, dev, backend
        wl = build_workload(name, dev, seed=seed, B=B, H=H)
        self.wl = wl
        self.q, self.k, self.v, kw = wl["q"], wl["k"], wl["v"], wl["kw"]
        self.bias, self.mask = kw.get("bias"), kw.get("mask")
        self.causal, self.scale = bool(kw.get("causal", False)), kw.get("scale")
        self.dout = torch.randn(self.q.shape, generator=torch.Generator(device=dev).manual_seed(5 + seed), device=dev,
                                dtype=torch.float32).to(self.q.dtype)
        for t in (self.q, self.k, self.v):
            t.requires_grad_(True)
        self.wrt = [self.q, self.k, self.v]
        if self.bias is not None and wl["want_dbias"]:
            self.bias.requires_grad_(True)
            self.wrt.append(self.bias)
        self.need_flush = wl["bytes"] < 2 * L2_BYTES
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if self.need_flush else None
        self.graph = None

    def step(self):
        out = self.att.scaled_dot_product_attention(self.q, self.k, self.v, bias=self.bias, mask=self.mask,
                                                    causal=self.causal, scale=self.scale, backend=self.backend)
        grads = torch.autograd.grad(out, self.wrt, grad_outputs=self.dout)
        return out, grads

    def capture(self):
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.step()
            for _ in range(2):
                g.replay()
            torch.cuda.synchronize()
            self.graph = g
            return None
        except Exception as exc:  # noqa: BLE001 - any capture problem falls back to eager launches
            torch.cuda.synchronize()
            self.graph = None
            return str(exc)[:200]

    def run_once(self, i=0):
        if self.need_flush:
            self.flush.fill_(i & 0xFF)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step()


def measure(runner, steps, warmup, region_s, barrier, local_rank, agree=float, max_blocks=2000):
    """Timed region of R blocks x `steps` replays; returns per-step median ms, spread, clocks, launches per step.

    `barrier` brackets every block (all ranks + device synchronize); `agree` turns this rank's calibration time into
    the number every rank uses (max over ranks), so that all ranks run the same number of blocks.  A workload whose
    operands fit in L2 has the L2 flushed before every step; the flush is kept out of the step's time by timing
    each step with its own pair of events inside the block."""
    from nitrix_b200 import _cabi

    lib = _cabi.lib()
    import warnings
    warnings.simplefilter("ignore")
    for _ in range(max(warmup, 3)):
        runner.step()
    torch.cuda.synchronize()
    launches0 = lib.nb200_launch_count()
    runner.step()
    torch.cuda.synchronize()
    launches_per_step = int(lib.nb200_launch_count() - launches0)
    graph_error = runner.capture()

    def block():
        """K steps between a barrier + synchronize on both sides; returns the milliseconds the steps took."""
        if runner.need_flush:
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            barrier()
            for i, (a, b) in enumerate(evs):
                runner.flush.fill_(i & 0xFF)
                a.record()
                if runner.graph is not None:
                    runner.graph.replay()
                else:
                    runner.step()
                b.record()
            barrier()
            return sum(a.elapsed_time(b) for a, b in evs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for i in range(steps):
            runner.run_once(i)
        b.record()
        barrier()
        return a.elapsed_time(b)

    block_ms = agree(max(block(), 1e-3))   # calibration block: sizes the region
    blocks = int(min(max_blocks, max(3, round(region_s * 1e3 / block_ms))))
    times = []
    with ClockSampler(local_rank) as clocks:
        for _ in range(blocks):
            times.append(block() / steps)
    assert lib.nb200_device_status(local_rank) == 0, _cabi.last_error()
    return dict(ms=statistics.median(times), spread=[min(times), max(times)], blocks=blocks, clocks=clocks.summary(),
                launches_per_step=launches_per_step, graph_error=graph_error, region_ms=sum(times) * steps)


def kernel_times(runner, steps):
    """Average launch duration of every kernel of a step: the library records a CUDA event on the launching stream
    after each kernel it enqueues (eager launches; a few microseconds per kernel, kept out of the headline region)."""
    from nitrix_b200 import _cabi

    lib = _cabi.lib()
    lib.nb200_profile(1)
    for i in range(steps):
        if runner.need_flush:
            runner.flush.fill_(i & 0xFF)
        runner.step()
    torch.cuda.synchronize()
    ms = _cabi.kernel_times()
    lib.nb200_profile(0)
    return {n: v[1] / v[0] for n, v in ms.items()}, {n: v[0] for n, v in ms.items()}


def roofline_record(name, wl, step_ms, kernels, peaks, with_traffic=True):
    """Roofline of the dominant kernel plus the whole step against both tensor peaks and the HBM bound."""
    if not kernels:
        return None
    dom = max(kernels, key=lambda n: kernels[n])
    share = KERNEL_FLOP_SHARE.get(dom)
    dom_flops = wl["flops"] * share if share is not None else None
    achieved = dom_flops / (kernels[dom] * 1e-3) / 1e12 if dom_flops else None
    t_burst = max(wl["flops"] / (peaks["burst"] * 1e12), wl["bytes"] / (peaks["hbm"] * 1e9))
    t_sust = max(wl["flops"] / (peaks["sustained"] * 1e12), wl["bytes"] / (peaks["hbm"] * 1e9))
    return {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["burst"], "unit": "TFLOP/s",
            "frac": achieved / peaks["burst"] if achieved else None,
            "frac_of_sustained": achieved / peaks["sustained"] if achieved else None,
            "traffic": NCU_TRAFFIC_BYTES.get(name, {}).get(dom) if with_traffic else None,
            "avg_launch_ms": kernels[dom], "algorithmic_flops_per_launch": dom_flops,
            "peak_source": (f"bf16 dense, of {peaks['source']}: frac uses the burst figure ({peaks['burst']:.0f}; the kernel's "
                            f"launch time comes from a pass in which it is timed by itself), frac_of_sustained the "
                            f"seconds-long figure ({peaks['sustained']:.0f})"),
            "kernels_ms": {n: round(v, 5) for n, v in sorted(kernels.items())},
            "step_vs_roofline": {"burst": t_burst / (step_ms * 1e-3), "sustained": t_sust / (step_ms * 1e-3),
                                 "tensor_bound_ms": wl["flops"] / (peaks["burst"] * 1e12) * 1e3,
                                 "hbm_bound_ms": wl["bytes"] / (peaks["hbm"] * 1e9) * 1e3}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--backend", default="auto")
    ap.add_argument("--batch", type=int, default=None, help="override the workload's batch size (profiling captures)")
    ap.add_argument("--region-seconds", type=float, default=1.0, help="length of the headline timed region")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the per-workload table and the partition record")
    ap.add_argument("--layer-norm-only", action="store_true",
                    help="print only the sibling ops' records (small: for profiling captures)")
    args = ap.parse_args()

    if args.layer_norm_only:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        print(json.dumps({"layer_norm": layer_norm_record(dev, load_peaks()),
                          "selective_scan": selective_scan_record(dev, load_peaks())}))
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl_name = args.workload
    w = WORKLOADS[wl_name]
    config = make_config(wl_name, world, args.batch)

    if args.impl == "reference":
        if rank != 0:
            return
        val, cores, sample, sec, spread = cpu_reference_step(wl_name)
        line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "config": config,
                "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                 "spread_s": spread},
                "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch.distributed as dist
    from nitrix_b200 import _cabi
    from nitrix_b200.parallel import max_over_ranks

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    lib = _cabi.lib()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- headline: the whole workload on every rank ----
    runner = Runner(wl_name, dev, args.backend, seed=rank, B=args.batch)
    wl = runner.wl
    m = measure(runner, args.steps, args.warmup, args.region_seconds, barrier, local_rank,
                agree=lambda x: max_over_ranks(x, dev))
    if m["graph_error"]:
        config["launch"], config["graph_error"] = "eager launches", m["graph_error"]
    step_ms = max_over_ranks(m["ms"], dev)
    value = world * wl["flops"] / (step_ms * 1e-3) / 1e12
    kernels, kernel_launches = ({}, {})
    if rank == 0:
        kernels, kernel_launches = kernel_times(runner, min(args.steps, 10))

    # ---- end to end: host operands, copies inside the timed region ----
    e2e = None
    if not args.no_e2e:
        try:
            numa = bind_near_gpu(local_rank) if world > 1 else None
            host_in = {n: t.detach().cpu().pin_memory() for n, t in (("q", runner.q), ("k", runner.k), ("v", runner.v),
                                                                    ("dout", runner.dout))}
            if runner.bias is not None:
                host_in["bias"] = runner.bias.detach().cpu().pin_memory()
            if runner.mask is not None:
                host_in["mask"] = runner.mask.cpu().pin_memory()
            # batch chunks move up, run and come down on three streams at once (nitrix_b200.nn.host_pipeline)
            from nitrix_b200.nn.host_pipeline import HostPipeline
            pipe = HostPipeline(host_in, device=dev, causal=runner.causal, scale=runner.scale, want_dbias=wl["want_dbias"],
                                chunks=8, backend=args.backend)
            h2d = pipe.h2d_bytes()
            pipe.run()
            d2h = pipe.d2h_bytes()
            pipe.run()
            torch.cuda.synchronize()
            n_e2e = 5 if wl["bytes"] > 1e9 else max(5, min(args.steps, 20))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            for _ in range(n_e2e):
                pipe.run()
            e1.record()
            barrier()
            my_ms = e0.elapsed_time(e1) / n_e2e
            e2e_ms = max_over_ranks(my_ms, dev)
            e2e = {"value": world * wl["flops"] / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                   "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                   "h2d_gbs_per_rank": h2d / (my_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (my_ms * 1e-3) / 1e9,
                   "kernel_ms_per_step": step_ms, "numa_node_of_staging": numa,
                   "limiter": "host<->device copies (PCIe): copy-in, kernels and copy-out of batch chunks overlap on "
                              "three streams, so a step lasts as long as its larger copy direction",
                   "how": f"{len(pipe.slices)} batch chunks pipelined over copy-in / kernel / copy-out streams"}
            del pipe, host_in
        except Exception as exc:  # noqa: BLE001 - e.g. pinned host memory refused: report, keep the device numbers
            e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                   "error": str(exc)[:200]}
            torch.cuda.synchronize()

    peaks = load_peaks()
    roofline = roofline_record(wl_name, wl, step_ms, kernels, peaks, with_traffic=not args.batch) if rank == 0 else None
    headline_clocks = m["clocks"]
    headline_launches = m["launches_per_step"]
    del runner
    torch.cuda.empty_cache()

    # ---- every configuration on one GPU ----
    workloads = None
    if world == 1 and not args.no_extra and not args.batch:
        workloads = []
        for name in sorted(WORKLOADS):
            try:
                if name == wl_name:
                    mm, kk, ww = m, kernels, wl
                else:
                    r = Runner(name, dev, args.backend, seed=0)
                    mm = measure(r, args.steps, args.warmup, 0.4, barrier, local_rank)
                    kk, _ = kernel_times(r, min(args.steps, 10))
                    ww = r.wl
                    del r
                    torch.cuda.empty_cache()
                rec = roofline_record(name, ww, mm["ms"], kk, peaks)
                mhz = mm["clocks"]["sm_mhz"]
                workloads.append({"workload": f"{name}: {WORKLOADS[name]['desc']}", "ms_per_step": mm["ms"],
                                  "ms_spread": mm["spread"], "blocks": mm["blocks"],
                                  "tflops": ww["flops"] / (mm["ms"] * 1e-3) / 1e12,
                                  "ms_x_sm_mhz": mm["ms"] * mhz if mhz else None,
                                  "step_vs_roofline": rec["step_vs_roofline"] if rec else None,
                                  "dominant_kernel": rec["kernel"] if rec else None, "frac": rec["frac"] if rec else None,
                                  "kernels_ms": rec["kernels_ms"] if rec else None, "clocks": mm["clocks"],
                                  "launches_per_step": mm["launches_per_step"],
                                  "launch": "eager" if mm["graph_error"] else "graph"})
            except Exception as exc:  # noqa: BLE001
                workloads.append({"workload": name, "error": str(exc)[:200]})
                torch.cuda.synchronize()

    # ---- the sibling op: fused LayerNorm on the reference's norm-benchmark shapes (HBM-bound) ----
    layer_norm = None
    if world == 1 and not args.no_extra and not args.batch:
        try:
            layer_norm = layer_norm_record(dev, peaks)
        except Exception as exc:  # noqa: BLE001
            layer_norm = {"error": str(exc)[:200]}
            torch.cuda.synchronize()

    selective_scan = None
    if world == 1 and not args.no_extra and not args.batch:
        try:
            selective_scan = selective_scan_record(dev, peaks)
        except Exception as exc:  # noqa: BLE001
            selective_scan = {"error": str(exc)[:200]}
            torch.cuda.synchronize()

    # ---- the split the configurations name: c5 heads / c4 sequences over the GPUs of the box ----
    partition = None
    if world > 1 and not args.no_extra:
        partition = partition_record(world, rank, local_rank, dev, args, barrier, peaks)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        val, cores, sample, _, spread = cpu_reference_step(wl_name)
        cpu = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample, "spread_s": spread}
    mhz = headline_clocks["sm_mhz"]
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "ms_spread": m["spread"], "blocks": m["blocks"],
            "timed_region_ms": m["region_ms"], "ms_x_sm_mhz": step_ms * mhz if mhz else None,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": config, "clocks": headline_clocks, "e2e": e2e,
            "gpu_launches": int(headline_launches) * args.steps * m["blocks"], "launches_per_step": headline_launches,
            "roofline": roofline, "cpu_baseline": cpu, "workloads": workloads, "partition": partition,
            "layer_norm": layer_norm, "selective_scan": selective_scan}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# (batch, tokens, channels) of the reference's norm benchmark (its bench/PERF_LAYER_NORM.md:17-32); each moves more
# than the 126 MB L2 per pass except the smallest, so the L2 is flushed between calls
LAYER_NORM_SHAPES = [("bf16", (8, 1024, 2048)), ("bf16", (8, 1024, 8192)), ("bf16", (32, 512, 1024)),
                     ("f32", (8, 1024, 1024)), ("f32", (8, 1024, 4096))]


def layer_norm_record(dev, peaks):
    """Forward and backward of the fused LayerNorm on device-resident operands.  K independent sets of operands,
    together several times the L2, run back to back as one replayed CUDA graph (so every call finds its inputs in
    HBM, and launch gaps are the graph's, not Python's); time per call = median replay / K.  Algorithmic bytes --
    forward x in and y out, backward x and dy in and dx out; the [c] vectors, the fp32 row statistics and the
    partial column sums are noise -- over that time, against the measured copy bandwidth."""
    from nitrix_b200.nn import norm

    out = []
    for dt_name, shape in LAYER_NORM_SHAPES:
        dt = torch.bfloat16 if dt_name == "bf16" else torch.float32
        rows, c = shape[0] * shape[1], shape[2]
        nbytes = rows * c * (2 if dt_name == "bf16" else 4)
        k_sets = int(min(32, max(4, -(-3 * L2_BYTES // (2 * nbytes)))))
        g = torch.Generator(device=dev).manual_seed(0)
        xs = [torch.randn(rows, c, device=dev, generator=g).to(dt) for _ in range(k_sets)]
        dys = [torch.randn(rows, c, device=dev, generator=g).to(dt) for _ in range(k_sets)]
        w = torch.ones(c, device=dev, dtype=dt)
        b = torch.zeros(c, device=dev, dtype=dt)
        stats = [norm.layer_norm_forward(x, w, b, 1e-5, 1.0)[1:] for x in xs]

        def graph_ms(fn):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    fn()
            ts = []
            for _ in range(8):
                a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                graph.replay()
                e.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(e))
            return statistics.median(ts[3:]) / k_sets

        def fwd_all():
            for x in xs:
                norm.layer_norm_forward(x, w, b, 1e-5, 1.0)

        def bwd_all():
            for x, dy, (mean, rstd) in zip(xs, dys, stats):
                norm.layer_norm_backward(x, w, dy, mean, rstd, 1e-5, 1.0, True, True)

        t_f, t_b = graph_ms(fwd_all), graph_ms(bwd_all)
        rec = {"shape": list(shape), "dtype": dt_name, "operand_sets": k_sets, "fwd_ms": t_f, "bwd_ms": t_b,
               "fwd_gbs": 2 * nbytes / (t_f * 1e-3) / 1e9, "bwd_gbs": 3 * nbytes / (t_b * 1e-3) / 1e9}
        if peaks:
            rec["fwd_frac_of_hbm"] = rec["fwd_gbs"] / peaks["hbm"]
            rec["bwd_frac_of_hbm"] = rec["bwd_gbs"] / peaks["hbm"]
        out.append(rec)
        del xs, dys, stats
        torch.cuda.empty_cache()
    return {"unit": "GB/s of algorithmic bytes per call; peak = measured copy bandwidth",
            "peak_gbs": peaks["hbm"] if peaks else None, "shapes": out}


# (batch, length, channels, states): a Mamba block's scan at model width 1024 (d_inner 2048, 16 states)
SELECTIVE_SCAN_SHAPES = [("f32", (8, 1024, 2048, 16)), ("bf16", (8, 2048, 2048, 16))]


def selective_scan_record(dev, peaks):
    """Forward and backward of the selective scan on device-resident operands: four operand sets replayed back to
    back as one CUDA graph; time per call = median replay / 4.  Reported with the state updates per second
    (batch x length x channels x states per pass) and the algorithmic bytes per second -- forward x, delta in and y
    out; backward x, delta, dy in and dx, ddelta out, plus the checkpoints either way -- against the measured copy
    bandwidth.  The recurrence is sequential in time: the parallelism is batch x channels threads."""
    from nitrix_b200.nn import ssm

    out = []
    for dt_name, (bsz, length, d, n) in SELECTIVE_SCAN_SHAPES:
        dt = torch.bfloat16 if dt_name == "bf16" else torch.float32
        esz = 2 if dt_name == "bf16" else 4
        g = torch.Generator(device=dev).manual_seed(0)
        sets = []
        for _ in range(4):
            x = torch.randn(bsz, length, d, device=dev, generator=g).to(dt)
            delta = (torch.rand(bsz, length, d, device=dev, generator=g) * 0.5 + 0.01).to(dt)
            a_mat = (-(torch.rand(d, n, device=dev, generator=g) * 1.5 + 0.2)).to(dt)
            b_mat = torch.randn(bsz, length, n, device=dev, generator=g).to(dt)
            c_mat = torch.randn(bsz, length, n, device=dev, generator=g).to(dt)
            skip = torch.randn(d, device=dev, generator=g).to(dt)
            dy = torch.randn(bsz, length, d, device=dev, generator=g).to(dt)
            ck = ssm.selective_scan_forward(x, delta, a_mat, b_mat, c_mat, skip, True)[1]
            sets.append((x, delta, a_mat, b_mat, c_mat, skip, ck, dy))

        def graph_ms(fn):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    fn()
            ts = []
            for _ in range(6):
                a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                graph.replay()
                e.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(e))
            return statistics.median(ts[2:]) / len(sets)

        def fwd_all():
            for x, delta, a_mat, b_mat, c_mat, skip, _, _ in sets:
                ssm.selective_scan_forward(x, delta, a_mat, b_mat, c_mat, skip, True)

        def bwd_all():
            for x, delta, a_mat, b_mat, c_mat, skip, ck, dy in sets:
                ssm.selective_scan_backward(x, delta, a_mat, b_mat, c_mat, skip, ck, dy)

        t_f, t_b = graph_ms(fwd_all), graph_ms(bwd_all)
        updates = bsz * length * d * n
        ck_bytes = bsz * ((length + 7) // 8) * d * n * 4
        f_bytes = 3 * bsz * length * d * esz + ck_bytes
        b_bytes = 5 * bsz * length * d * esz + ck_bytes
        rec = {"shape": [bsz, length, d, n], "dtype": dt_name, "fwd_ms": t_f, "bwd_ms": t_b,
               "fwd_gupdates_per_s": updates / (t_f * 1e-3) / 1e9, "bwd_gupdates_per_s": updates / (t_b * 1e-3) / 1e9,
               "fwd_gbs": f_bytes / (t_f * 1e-3) / 1e9, "bwd_gbs": b_bytes / (t_b * 1e-3) / 1e9}
        if peaks:
            rec["fwd_frac_of_hbm"] = rec["fwd_gbs"] / peaks["hbm"]
            rec["bwd_frac_of_hbm"] = rec["bwd_gbs"] / peaks["hbm"]
        out.append(rec)
        del sets
        torch.cuda.empty_cache()
    return {"unit": "state updates per second; GB/s of algorithmic bytes against the measured copy bandwidth",
            "peak_gbs": peaks["hbm"] if peaks else None, "shapes": out}


def partition_record(world, rank, local_rank, dev, args, barrier, peaks):
    """c5 with 16 / N heads per GPU and c4 with 32 / N sequences per GPU (strong scaling): every rank builds and
    runs only its shard; no collective in the timed loop.  For c5 the optional replicated output is timed twice:
    NCCL all-gather after the forward, and the forward kernel storing straight into the peers' buffers."""
    import torch.distributed as dist
    from nitrix_b200 import parallel as P
    from nitrix_b200.parallel import max_over_ranks

    rec = {}
    for name, axis in (("c5", "heads"), ("c4", "batch")):
        w = WORKLOADS[name]
        item = {"axis": axis}
        ms = float("nan")
        flops = 0.0
        runner = None
        try:
            n = w["H"] if axis == "heads" else w["B"]
            lo, hi = P.bh_partition(n, world, rank)
            kw = dict(H=hi - lo) if axis == "heads" else dict(B=hi - lo)
            runner = Runner(name, dev, args.backend, seed=100 + rank, **kw)
            flops = runner.wl["flops"]
            item["per_gpu"] = f"{hi - lo} {axis if axis == 'heads' else 'sequences'}"
        except Exception as exc:  # noqa: BLE001 - every rank still takes part in the collectives below
            item["error"] = str(exc)[:200]
        local = None
        if runner is not None:
            try:
                local = measure(runner, args.steps, args.warmup, 0.5, lambda: torch.cuda.synchronize(), local_rank)
                ms = local["ms"]
            except Exception as exc:  # noqa: BLE001
                item["error"] = str(exc)[:200]
                torch.cuda.synchronize()
        barrier()
        ms_max = max_over_ranks(ms, dev)
        total = torch.tensor([flops], dtype=torch.float64, device=dev)
        dist.all_reduce(total)
        item.update({"ms_per_step": ms_max, "tflops": float(total.item()) / (ms_max * 1e-3) / 1e12 if ms_max == ms_max else None,
                     "clocks": local["clocks"] if local else None})
        if name == "c5" and runner is not None:
            item.update(gather_timing(runner, world, rank, dev, barrier))
        rec[name] = item
        del runner
        torch.cuda.empty_cache()
    return rec


def gather_timing(runner, world, rank, dev, barrier, reps=5):
    """Forward of this rank's heads followed by an NCCL all-gather of the output, against the forward whose epilogue
    stores the output rows into every rank's buffer itself.  Times are per forward, max over ranks."""
    import torch.distributed as dist
    from nitrix_b200 import parallel as P
    from nitrix_b200.nn import attention as att
    from nitrix_b200.parallel import max_over_ranks

    out = {}
    q, k, v, bias = (t.detach() for t in (runner.q, runner.k, runner.v, runner.bias))
    scale = q.shape[-1] ** -0.5
    B, Hl, S, D = q.shape

    def timed(fn):
        for _ in range(2):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        barrier()
        return max_over_ranks(a.elapsed_time(b) / reps, dev)

    try:
        out["fwd_ms"] = timed(lambda: att.sdpa_forward(q, k, v, bias, None, scale=scale, causal=True))
        out["fwd_plus_nccl_all_gather_ms"] = timed(
            lambda: P.all_gather_output(att.sdpa_forward(q, k, v, bias, None, scale=scale, causal=True)[0], "heads"))
        out["all_gather_bytes_per_rank"] = int(q.numel() * q.element_size())
    except Exception as exc:  # noqa: BLE001
        out["gather_error"] = str(exc)[:200]
        torch.cuda.synchronize()
    ok = torch.ones(1, dtype=torch.int32, device=dev)
    rep = None
    try:
        rep = P.ReplicatedOutput((B, Hl * world, S, D), q.dtype, dev)
    except Exception as exc:  # noqa: BLE001
        out["fused_gather_error"] = str(exc)[:200]
        ok.zero_()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 1:
        view = rep.local.narrow(1, rank * Hl, Hl)
        peers = rep.peers_of(view)

        def fused():
            att.sdpa_forward(q, k, v, bias, None, scale=scale, causal=True, out=view, out_peers=peers)
            rep.wait()

        out["fwd_fused_all_gather_ms"] = timed(fused)
        rep.close()
    return out


if __name__ == "__main__":
    main()
