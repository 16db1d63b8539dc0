"""Attention forward + backward on operands that live in (pinned) host memory.

The kernels work on device memory; a caller whose arrays sit on the host pays
for the PCIe copies as well.  This helper hides most of that cost: the batch is
cut into chunks, and three CUDA streams move chunk ``c + 1`` up, run the
kernels of chunk ``c`` and bring the results of chunk ``c - 1`` down at the
same time (PCIe is full duplex).  Operands that are shared by the whole batch
(a bias or mask whose batch extent is 1) go up once, first.

It calls the public entry point (`scaled_dot_product_attention` and its
autograd backward) once per chunk; every (batch, head) pair is independent, so
chunking changes no result.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .attention import scaled_dot_product_attention


class HostPipeline:
    """Reusable state (streams, device staging buffers, events) for one problem shape.

    ``host_in``: pinned tensors ``q, k, v, dout`` (``(B, H, L, D)``) and optionally ``bias`` / ``mask``
    broadcastable to ``(B, H, S, T)``.  ``run()`` returns pinned host tensors ``out, dq, dk, dv`` (and
    ``dbias`` when ``want_dbias`` and the bias has the batch's extent).
    """

    def __init__(self, host_in: Dict[str, torch.Tensor], *, device: torch.device, causal: bool, scale: float,
                 want_dbias: bool = False, chunks: int = 4, backend: str = "auto"):
        self.host_in = host_in
        self.device = device
        self.causal, self.scale, self.backend = causal, scale, backend
        B = host_in["q"].shape[0]
        bias = host_in.get("bias")
        self.want_dbias = bool(want_dbias and bias is not None)
        bias_batched = bias is not None and bias.dim() == 4 and bias.shape[0] == B and B > 1
        if self.want_dbias and not bias_batched:
            chunks = 1   # the gradient of a bias shared by the batch (any rank) sums over all chunks: keep one chunk
        chunks = max(1, min(chunks, B))
        bounds = [round(i * B / chunks) for i in range(chunks + 1)]
        self.slices = [slice(bounds[i], bounds[i + 1]) for i in range(chunks) if bounds[i + 1] > bounds[i]]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device) for _ in range(3))
        # full-size device staging buffers, filled and consumed chunk by chunk
        self.dev = {n: torch.empty(t.shape, dtype=t.dtype, device=device) for n, t in host_in.items()}
        self.batched = {n: (t.dim() == 4 and t.shape[0] == B and B > 1) or n in ("q", "k", "v", "dout")
                        for n, t in host_in.items()}
        self.host_out: Optional[Dict[str, torch.Tensor]] = None
        self.ev_run_done = [None] * len(self.slices)   # last step's kernels of a chunk (its inputs may be rewritten)

    def h2d_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.host_in.values())

    def d2h_bytes(self) -> int:
        assert self.host_out is not None
        return sum(t.numel() * t.element_size() for t in self.host_out.values())

    def run(self) -> Dict[str, torch.Tensor]:
        # The operands are host memory, so nothing on the caller's stream has to finish first; the three streams
        # order themselves by events, and a step's copy-in may start while the previous step's copy-out still runs.
        cur = torch.cuda.current_stream(self.device)
        shared = [n for n, b in self.batched.items() if not b]
        ev_shared = None
        if shared:
            with torch.cuda.stream(self.s_in):
                # a shared operand is read by every chunk of the previous step
                for ev in self.ev_run_done:
                    if ev is not None:
                        self.s_in.wait_event(ev)
                for n in shared:
                    self.dev[n].copy_(self.host_in[n], non_blocking=True)
                ev_shared = torch.cuda.Event()
                ev_shared.record(self.s_in)
        for c, sl in enumerate(self.slices):
            with torch.cuda.stream(self.s_in):
                if self.ev_run_done[c] is not None:
                    self.s_in.wait_event(self.ev_run_done[c])
                for n, b in self.batched.items():
                    if b:
                        self.dev[n][sl].copy_(self.host_in[n][sl], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ev_in)
                if ev_shared is not None:
                    self.s_run.wait_event(ev_shared)
                q, k, v = (self.dev[n][sl].requires_grad_(True) for n in ("q", "k", "v"))
                wrt = [q, k, v]
                bias = self.dev.get("bias")
                if bias is not None and self.batched["bias"]:
                    bias = bias[sl]
                if bias is not None and self.want_dbias:
                    # a fresh leaf over the staging buffer (the buffer itself is overwritten by the next step's copy)
                    bias = bias.detach().requires_grad_(True)
                    wrt.append(bias)
                mask = self.dev.get("mask")
                if mask is not None and self.batched["mask"]:
                    mask = mask[sl]
                out = scaled_dot_product_attention(q, k, v, bias=bias, mask=mask, causal=self.causal, scale=self.scale,
                                                   backend=self.backend)
                grads = torch.autograd.grad(out, wrt, grad_outputs=self.dev["dout"][sl])
                ev_run = torch.cuda.Event()
                ev_run.record(self.s_run)
                self.ev_run_done[c] = ev_run
            res = [out.detach(), *grads]
            if self.host_out is None:
                names = ["out", "dq", "dk", "dv"] + (["dbias"] if self.want_dbias else [])
                B = self.host_in["q"].shape[0]
                self._names = names
                self.host_out = {}
                for n, t in zip(names, res):
                    full = (B,) + tuple(t.shape[1:]) if (n != "dbias" or self.batched["bias"]) else tuple(t.shape)
                    self.host_out[n] = torch.empty(full, dtype=t.dtype).pin_memory()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_run)
                for n, t in zip(self._names, res):
                    dst = self.host_out[n]
                    if n != "dbias" or self.batched["bias"]:
                        dst = dst[sl]          # this chunk's batch rows
                    dst.copy_(t, non_blocking=True)
                    t.record_stream(self.s_out)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_run)
        return self.host_out
