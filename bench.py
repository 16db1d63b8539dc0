#!/usr/bin/env python
"""Benchmark of the attention hot path: forward + backward TFLOP/s on B200.

``python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5|c1] [--impl ours|reference]``

A *step* is one forward + backward pass of ``scaled_dot_product_attention``
over one synthetic batch of the named workload (the five benchmark configurations;
default ``c2``: bf16, B=8, H=16, L=2048, D=64, causal, ALiBi bias (1,H,L,L),
gradients for q, k, v).  Throughput counts ALGORITHMIC flops only:
``14 * B * H * S * T_eff * D`` per step (4 forward + 10 backward, causal halves
the pairs, key padding counts kept keys only); softmax work is not counted.

One JSON line is printed by rank 0 with

* ``value``: whole-job TFLOP/s with operands resident in HBM: K replays of a
  CUDA graph of one step between two CUDA events, max over ranks (multi-GPU: every rank runs the full workload on its
  own shard of a batch N times larger -> weak scaling, no collective);
* ``e2e``: the same metric through the public entry point with HOST (pinned)
  operands: H2D of q, k, v, bias, mask, dout and D2H of out, dq, dk, dv (dbias)
  inside the timed region;
* ``roofline``: achieved vs measured peak for the pass that dominates the step;
* ``cpu_baseline``: the CPU oracle (torch, all host threads) on a bounded sample.

``--impl reference`` times only that CPU implementation (the reference's own
``jnp`` path cannot run: jax is not installed; the op-for-op torch restatement
stands in, ``cpu_baseline.kind = "port"``).
"""
from __future__ import annotations

import argparse
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
    "sdpa_bwd_tc_kernel<merged>": 10 / 14,      # head dim 64 without a bias gradient: dq, dk, dv from one kernel
    "simt_fwd_kernel": 4 / 14,
    "simt_bwd_dkv_kernel": 8 / 14,
    "simt_bwd_dq_kernel": 2 / 14,
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu captures (profiles/), full-size
# workload, same command line as the default bench run.
NCU_TRAFFIC_BYTES = {
    "c2": {"sdpa_fwd_tc_kernel": 203.8e6, "sdpa_bwd_tc_kernel<merged>": 796.9e6},
}

METRIC = "fwd+bwd attention TFLOP/s"
UNIT = "TFLOP/s"

WORKLOADS = {
    # name: (builder, kwargs, dtype string, want_dbias, description)
    "c1": dict(B=2, H=4, L=256, D=64, dtype="f32", desc="fp32 B2 H4 L256 D64 bias(B,H,L,L)+dBias key-mask"),
    "c2": dict(B=8, H=16, L=2048, D=64, dtype="bf16", desc="bf16 B8 H16 L2048 D64 causal ALiBi bias(1,H,L,L)"),
    "c3": dict(B=4, H=32, L=4096, D=128, dtype="bf16", desc="bf16 B4 H32 L4096 D128 bias(B,H,L,L)+dBias mask(B,1,L,L)"),
    "c4": dict(B=32, H=8, L=1024, D=64, dtype="f16", desc="fp16 B32 H8 L1024 D64 key-padding mask"),
    "c5": dict(B=1, H=16, L=65536, D=128, dtype="bf16", desc="bf16 B1 H16 L65536 D128 causal key-bias(1,H,1,L)"),
}


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
    esz = q.element_size()
    bias = kw.get("bias")
    by = 3 * q.numel() * esz + q.numel() * esz + B * H * L * 4  # fwd: q k v out lse
    by += 8 * q.numel() * esz + 2 * B * H * L * 4               # bwd: q k v out dout dq dk dv lse delta
    if bias is not None:
        by += 2 * bias.numel() * bias.element_size() + (bias.numel() * bias.element_size() if want_dbias else 0)
    if mask is not None:
        by += 2 * mask.numel()
    return dict(q=q, k=k, v=v, kw=kw, want_dbias=want_dbias, flops=flops, fwd_flops=flops * 4 / 14,
                bwd_flops=flops * 10 / 14, bytes=float(by), B=B, H=H, L=L, D=D)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()  # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], burst=p["bf16_tflops"], sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, source="fallback")


def cpu_reference_step(wl_name, seconds_target=10.0, steps=1, warmup=0):
    """Times the CPU oracle (fwd + autograd bwd, fp32, all host threads) on a bounded sample of the workload:
    a subset of (batch, head) pairs (each pair is independent), for c5 additionally a block of query rows.
    Returns (TFLOP/s, cores, sample description, seconds per step)."""
    from oracle import sdpa_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    w = WORKLOADS[wl_name]
    L = w["L"]
    rows = L
    if wl_name == "c5":
        L, rows = 65536, 512  # one block of 512 query rows (the last, fullest causal block) against all keys

    def run(n_pairs):
        if wl_name == "c5":
            g = torch.Generator().manual_seed(0)
            D = w["D"]
            q = torch.randn(1, n_pairs, rows, D, generator=g).bfloat16()
            k = torch.randn(1, n_pairs, L, D, generator=g).bfloat16()
            v = torch.randn(1, n_pairs, L, D, generator=g).bfloat16()
            bias = torch.randn(1, n_pairs, 1, L, generator=g).bfloat16()
            # rows are the LAST block of the sequence: every key is visible except the strict upper triangle
            mask = (torch.arange(L)[None, :] <= (L - rows + torch.arange(rows))[:, None])
            dout = torch.randn(1, n_pairs, rows, D, generator=g).bfloat16()
            t0 = time.perf_counter()
            O.reference_grads_torch(q, k, v, dout, bias=bias, mask=mask, want_dbias=False)
            dt = time.perf_counter() - t0
            pairs = float(n_pairs) * mask.sum().item()
            return dt, 14.0 * pairs * D
        sub = build_workload(wl_name, "cpu", B=1, H=n_pairs)
        dout = torch.randn(sub["q"].shape, generator=torch.Generator().manual_seed(5)).to(sub["q"].dtype)
        kw = dict(sub["kw"])
        t0 = time.perf_counter()
        O.reference_grads_torch(sub["q"], sub["k"], sub["v"], dout, want_dbias=sub["want_dbias"], **kw)
        return time.perf_counter() - t0, sub["flops"]

    t1, _ = run(1)  # calibration (also the warm-up)
    total_pairs = w["B"] * w["H"]
    n = max(1, min(total_pairs, int(seconds_target / max(t1, 1e-3))))
    n = min(n, 16)
    for _ in range(warmup):
        run(n)
    times, flops = [], 0.0
    for _ in range(max(1, steps)):
        dt, flops = run(n)
        times.append(dt)
    sec = statistics.median(times)
    sample = f"{n} of {total_pairs} (batch, head) pairs" + (f", last {rows} query rows of L={L}" if wl_name == "c5" else f" at full L={w['L']}")
    return flops / sec / 1e12, cores, sample, sec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--backend", default="auto")
    ap.add_argument("--batch", type=int, default=None, help="override the workload's batch size (profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl_name = args.workload
    w = WORKLOADS[wl_name]
    config = {"workload": f"{wl_name}: {w['desc']}", "per_gpu_batch": w["B"], "global_batch": w["B"] * world,
              "sharding": f"dp{world} over batch x heads, no collective"}

    if args.impl == "reference":
        if rank != 0:
            return
        val, cores, sample, sec = cpu_reference_step(wl_name, seconds_target=5.0, steps=args.steps if args.steps < 5 else 3,
                                                     warmup=min(args.warmup, 1))
        line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "config": config,
                "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
                "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch.distributed as dist
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import attention as att
    from nitrix_b200.parallel import max_over_ranks

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.lib()

    wl = build_workload(wl_name, dev, seed=rank, B=args.batch)
    if args.batch:
        config["per_gpu_batch"], config["global_batch"] = args.batch, args.batch * world
        config["workload"] += f" [batch overridden to {args.batch}]"
    q, k, v, kw = wl["q"], wl["k"], wl["v"], wl["kw"]
    bias = kw.get("bias")
    mask = kw.get("mask")
    causal = bool(kw.get("causal", False))
    scale = kw.get("scale")
    dout = torch.randn(q.shape, generator=torch.Generator(device=dev).manual_seed(5 + rank), device=dev,
                       dtype=torch.float32).to(q.dtype)
    q.requires_grad_(True)
    k.requires_grad_(True)
    v.requires_grad_(True)
    if bias is not None and wl["want_dbias"]:
        bias.requires_grad_(True)
    wrt = [q, k, v] + ([bias] if (bias is not None and wl["want_dbias"]) else [])

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    working_set = wl["bytes"]
    need_flush = working_set < 2 * 126e6

    def step(ev=None):
        if ev:
            ev[0].record()
        out = att.scaled_dot_product_attention(q, k, v, bias=bias, mask=mask, causal=causal, scale=scale,
                                               backend=args.backend)
        if ev:
            ev[1].record()
        grads = torch.autograd.grad(out, wrt, grad_outputs=dout)
        if ev:
            ev[2].record()
        return out, grads

    import warnings
    warnings.simplefilter("ignore")
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches0 = lib.nb200_launch_count()
    barrier()
    with ClockSampler(local_rank) as clocks:
        for i in range(args.steps):
            if need_flush:
                flush.fill_(i & 0xFF)
            step(events[i])
        barrier()
    launches = lib.nb200_launch_count() - launches0
    assert lib.nb200_device_status(local_rank) == 0, _cabi.last_error()
    # second pass over the same steps with the library's per-kernel events on (a few microseconds per kernel,
    # so it is kept out of the headline region): average launch duration of every kernel
    kernel_ms = {}
    if rank == 0:
        lib.nb200_profile(1)
        for i in range(args.steps):
            if need_flush:
                flush.fill_(i & 0xFF)
            step()
        torch.cuda.synchronize()
        kernel_ms = _cabi.kernel_times()
        lib.nb200_profile(0)
    fwd_ms = [e[0].elapsed_time(e[1]) for e in events]
    bwd_ms = [e[1].elapsed_time(e[2]) for e in events]
    eager_ms = statistics.fmean(f + b for f, b in zip(fwd_ms, bwd_ms))
    # The step is a handful of sub-millisecond kernels, so host launch latency shows up as soon as several ranks
    # share the host's cores.  The headline region therefore replays a CUDA graph of one step (same kernels, same
    # buffers): K replays between two events, a barrier and a synchronize on both sides.  If the capture fails the
    # eagerly launched steps above are the measurement.
    step_ms, graphed = eager_ms, False
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for _ in range(3):
            graph.replay()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with ClockSampler(local_rank) as clocks_g:
            g0.record()
            for i in range(args.steps):
                if need_flush:
                    flush.fill_(i & 0xFF)
                graph.replay()
            g1.record()
            barrier()
        assert lib.nb200_device_status(local_rank) == 0, _cabi.last_error()
        step_ms, graphed, clocks = g0.elapsed_time(g1) / args.steps, True, clocks_g
    except Exception as exc:  # noqa: BLE001 - any capture problem falls back to the eager measurement
        config["graph_error"] = str(exc)[:200]
        torch.cuda.synchronize()
    config["launch"] = "CUDA graph replay of one fwd+bwd step" if graphed else "eager launches"
    step_ms = max_over_ranks(step_ms, dev)
    value = world * wl["flops"] / (step_ms * 1e-3) / 1e12

    # ---- end to end: host operands, copies inside the timed region ----
    e2e = None
    if not args.no_e2e:
        host_in = {n: t.detach().cpu().pin_memory() for n, t in (("q", q), ("k", k), ("v", v), ("dout", dout))}
        if bias is not None:
            host_in["bias"] = bias.detach().cpu().pin_memory()
        if mask is not None:
            host_in["mask"] = mask.cpu().pin_memory()
        # batch chunks move up, run and come down on three streams at once (nitrix_b200.nn.host_pipeline)
        from nitrix_b200.nn.host_pipeline import HostPipeline
        pipe = HostPipeline(host_in, device=dev, causal=causal, scale=scale, want_dbias=wl["want_dbias"],
                            chunks=8, backend=args.backend)
        h2d = pipe.h2d_bytes()

        def e2e_step():
            pipe.run()
            return pipe.d2h_bytes()

        d2h = e2e_step()
        e2e_step()
        n_e2e = max(3, min(args.steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1) / n_e2e, dev)
        e2e = {"value": world * wl["flops"] / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
               "how": f"{len(pipe.slices)} batch chunks pipelined over copy-in / kernel / copy-out streams"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    f_ms, b_ms = statistics.fmean(fwd_ms), statistics.fmean(bwd_ms)
    peak = peaks["burst"]
    # dominant kernel: per-kernel CUDA-event times recorded by the library on its launching stream
    dom = max(kernel_ms, key=lambda n: kernel_ms[n][1]) if kernel_ms else None
    roofline = None
    if dom is not None:
        dom_launches, total_ms = kernel_ms[dom]
        avg_ms = total_ms / dom_launches
        share = KERNEL_FLOP_SHARE.get(dom)
        dom_flops = wl["flops"] * share if share is not None else None
        achieved = dom_flops / (avg_ms * 1e-3) / 1e12 if dom_flops else None
        traffic = NCU_TRAFFIC_BYTES.get(wl_name, {}).get(dom) if not args.batch else None
        roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak if achieved else None, "traffic": traffic,
                    "avg_launch_ms": avg_ms, "launches": dom_launches,
                    "algorithmic_flops_per_launch": dom_flops,
                    "peak_source": f"bf16 dense burst (kernels timed alone), of {peaks['source']}",
                    "kernels_ms": {n: round(v[1] / v[0], 5) for n, v in sorted(kernel_ms.items())},
                    "fwd": {"ms": f_ms, "tflops": wl["fwd_flops"] / (f_ms * 1e-3) / 1e12},
                    "bwd": {"ms": b_ms, "tflops": wl["bwd_flops"] / (b_ms * 1e-3) / 1e12},
                    "eager_ms_per_step": eager_ms,
                    "step_vs_roofline": max(wl["flops"] / (peak * 1e12), wl["bytes"] / (peaks["hbm"] * 1e9)) / (step_ms * 1e-3)}
    cpu = None
    if not args.no_cpu_baseline and world == 1:
        val, cores, sample, _ = cpu_reference_step(wl_name, seconds_target=10.0)
        cpu = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic",
            "config": dict(config, l2="L2 flushed between steps" if need_flush else
                           f"operands ({working_set / 1e6:.0f} MB) exceed the 126 MB L2"),
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
            "cpu_baseline": cpu}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
