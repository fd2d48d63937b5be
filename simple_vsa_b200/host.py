"""Host-resident training step: VSA forward+backward for tensors that live in (pinned) host memory.

The ``(batch, head)`` slices of the operator are independent, so a step whose inputs and results
live on the host can be cut into chunks of slices and pipelined: while chunk ``i`` computes, chunk
``i+1`` is copied in and the results of chunk ``i-1`` are copied out, on three CUDA streams.  The
numbers are identical to one big call; only the PCIe transfers overlap the kernels.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch
from torch import Tensor

from . import b200_vsa


def _chunk_spans(total: int, per_chunk: int):
    """Chunks of ``per_chunk`` slices with a short ramp at both ends (1, 2, ... slices): the first copy-in and
    the last copy-out cannot overlap with any compute, so they should be small."""
    per_chunk = max(1, min(per_chunk, total))
    head, size = [], 1
    while size < per_chunk and sum(head) + size <= total // 4:
        head.append(size)
        size *= 2
    tail = list(reversed(head))
    middle = total - sum(head) - sum(tail)
    sizes = head + [per_chunk] * (middle // per_chunk) + ([middle % per_chunk] if middle % per_chunk else []) + tail
    spans, lo = [], 0
    for n in sizes:
        spans.append((lo, lo + n))
        lo += n
    assert lo == total
    return spans


def vsa_step_from_host(q: Tensor, k: Tensor, v: Tensor, dout: Tensor, variable_block_sizes: Tensor,
                       q_variable_block_sizes: Tensor, topk: int, block_size, gate: Optional[Tensor] = None, *,
                       out: Dict[str, Tensor], device=None, slices_per_chunk: int = 8) -> None:
    """Forward+backward of ``b200_vsa`` for host tensors ``[B,H,L,D]``; results land in ``out``.

    ``out`` maps ``"out", "dq", "dk", "dv"`` (and ``"dgate"`` when a gate is given) to host tensors of
    q's shape (pinned memory makes the copies asynchronous).  Returns after everything has arrived.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, L, D = q.shape
    BH = B * H
    names = ["q", "k", "v", "dout"] + (["gate"] if gate is not None else [])
    host_in = {"q": q, "k": k, "v": v, "dout": dout}
    if gate is not None:
        host_in["gate"] = gate
    host_in = {n: t.reshape(1, BH, t.shape[2], D) for n, t in host_in.items()}
    host_out = {n: t.reshape(1, BH, L, D) for n, t in out.items()}
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    compute = torch.cuda.current_stream(device)
    spans = _chunk_spans(BH, slices_per_chunk)
    width = max(hi - lo for lo, hi in spans)
    # two fixed sets of device input buffers (no allocator traffic between streams); results are the
    # operator's own fresh tensors and are kept referenced until their copy-out has finished
    ring = [{n: torch.empty((1, width, host_in[n].shape[2], D), device=device, dtype=q.dtype) for n in names}
            for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_in.wait_stream(compute)

    def stage(i):
        lo, hi = spans[i]
        b = i & 1
        with torch.cuda.stream(copy_in):
            if i >= 2:
                copy_in.wait_event(consumed[b])          # chunk i-2 no longer reads this buffer set
            for n in names:
                ring[b][n][:, :hi - lo].copy_(host_in[n][:, lo:hi], non_blocking=True)
            in_ready[b].record(copy_in)

    in_flight = []
    stage(0)
    for i, (lo, hi) in enumerate(spans):
        b = i & 1
        if i + 1 < len(spans):
            stage(i + 1)
        compute.wait_event(in_ready[b])
        dev = {n: ring[b][n][:, :hi - lo] for n in names}
        ql, kl, vl = (dev[n].detach().requires_grad_() for n in ("q", "k", "v"))
        gl = dev["gate"].detach().requires_grad_() if gate is not None else None
        o = b200_vsa(ql, kl, vl, variable_block_sizes, q_variable_block_sizes, topk, block_size, gl)
        o.backward(dev["dout"])
        consumed[b].record(compute)
        results = {"out": o.detach(), "dq": ql.grad, "dk": kl.grad, "dv": vl.grad}
        if gl is not None:
            results["dgate"] = gl.grad
        copied = torch.cuda.Event()
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(consumed[b])
            for n, t in results.items():
                host_out[n][:, lo:hi].copy_(t, non_blocking=True)
            copied.record(copy_out)
        in_flight.append((results, copied))
        del o, ql, kl, vl, gl, results
        if len(in_flight) > 2:                           # free a chunk's results only after they have left the GPU
            in_flight.pop(0)[1].synchronize()
    for _, ev in in_flight:
        ev.synchronize()
    compute.wait_stream(copy_out)
