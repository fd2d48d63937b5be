"""Host-resident training step: VSA forward+backward for tensors that live in (pinned) host memory.

The ``(batch, head)`` slices of the operator are independent, so a step whose inputs and results
live on the host can be cut into chunks of slices and pipelined: while chunk ``i`` computes, chunk
``i+1`` is copied in and the results of chunk ``i-1`` are copied out, on three CUDA streams.  The
numbers are identical to one big call; only the PCIe transfers overlap the kernels.

``copy_schedule_only=True`` runs the very same copies on the same streams with the operator left out
(the results copied back are the device input buffers): the time of that run is the floor the transfers
alone set for a host-resident step on this machine.

``bind_to_gpu_numa_node`` pins the calling process to the CPUs of the NUMA node its GPU hangs off; pinned
host buffers allocated afterwards land in that node's memory, which keeps the DMA traffic of several ranks
off the inter-socket link.
"""

from __future__ import annotations

import os
from typing import Dict, Optional

import torch
from torch import Tensor

from . import _lib, b200_vsa


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


def _parse_cpulist(text: str):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(device_index: int, sysfs_root: str = "/sys") -> Optional[int]:
    """Restrict this process to the CPUs of the NUMA node of GPU ``device_index`` (a process setting, undone by
    nothing else than another ``sched_setaffinity``).  Call it BEFORE allocating pinned host memory.  Returns
    the node, or None when the topology cannot be read (no such sysfs entry, a single node, an empty CPU set)
    -- in which case nothing is changed."""
    try:
        p = torch.cuda.get_device_properties(device_index)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open(os.path.join(sysfs_root, "bus/pci/devices", bdf.lower(), "numa_node")) as fh:
            node = int(fh.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs_root, "devices/system/node", f"node{node}", "cpulist")) as fh:
            cpus = _parse_cpulist(fh.read())
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


def vsa_step_from_host(q: Tensor, k: Tensor, v: Tensor, dout: Tensor, variable_block_sizes: Tensor,
                       q_variable_block_sizes: Tensor, topk: int, block_size, gate: Optional[Tensor] = None, *,
                       out: Dict[str, Tensor], device=None, slices_per_chunk: int = 8,
                       copy_schedule_only: bool = False) -> None:
    """Forward+backward of ``b200_vsa`` for host tensors ``[B,H,L,D]``; results land in ``out``.

    ``out`` maps ``"out", "dq", "dk", "dv"`` (and ``"dgate"`` exactly when a gate is given) to host tensors of
    q's shape (pinned memory makes the copies asynchronous).  Returns after everything has arrived, and raises
    ``VsaError`` if a bounded device-side wait ran out on the way (the results are not valid then).
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, L, D = q.shape
    BH = B * H
    names = ["q", "k", "v", "dout"] + (["gate"] if gate is not None else [])
    out_names = ["out", "dq", "dk", "dv"] + (["dgate"] if gate is not None else [])
    # everything that can be refused is refused before the first copy is queued
    if sorted(out) != sorted(out_names):
        raise ValueError(f"out must hold exactly {out_names} (dgate only with a gate), got {sorted(out)}")
    for n in out_names:
        if tuple(out[n].shape) != (B, H, L, D) or out[n].dtype != q.dtype:
            raise ValueError(f"out[{n!r}] must have q's shape {tuple(q.shape)} and dtype")
    host_in = {"q": q, "k": k, "v": v, "dout": dout}
    if gate is not None:
        host_in["gate"] = gate
    host_in = {n: t.reshape(1, BH, t.shape[2], D) for n, t in host_in.items()}
    host_out = {n: t.reshape(1, BH, L, D) for n, t in out.items()}
    # the two size vectors go to the device once, not once per chunk on the compute stream
    kv_sizes = variable_block_sizes.to(device=device, dtype=torch.int32)
    q_sizes = q_variable_block_sizes.to(device=device, dtype=torch.int32)
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    compute = torch.cuda.current_stream(device)
    spans = _chunk_spans(BH, slices_per_chunk)
    width = max(hi - lo for lo, hi in spans)
    # three fixed sets of device input buffers (no allocator traffic between streams): two copies-in may be in
    # flight while a third chunk computes; results are the operator's own fresh tensors and are kept referenced
    # until their copy-out has finished
    depth = 3
    ring = [{n: torch.empty((1, width, host_in[n].shape[2], D), device=device, dtype=q.dtype) for n in names}
            for _ in range(depth)]
    in_ready = [torch.cuda.Event() for _ in range(depth)]
    consumed = [torch.cuda.Event() for _ in range(depth)]
    copy_in.wait_stream(compute)

    def stage(i):
        lo, hi = spans[i]
        b = i % depth
        with torch.cuda.stream(copy_in):
            if i >= depth:
                copy_in.wait_event(consumed[b])          # chunk i-depth no longer reads this buffer set
            for n in names:
                ring[b][n][:, :hi - lo].copy_(host_in[n][:, lo:hi], non_blocking=True)
            in_ready[b].record(copy_in)

    in_flight = []
    for i in range(min(depth - 1, len(spans))):
        stage(i)
    for i, (lo, hi) in enumerate(spans):
        b = i % depth
        if i + depth - 1 < len(spans):
            stage(i + depth - 1)
        compute.wait_event(in_ready[b])
        dev = {n: ring[b][n][:, :hi - lo] for n in names}
        if copy_schedule_only:
            results = {"out": dev["q"], "dq": dev["k"], "dk": dev["v"], "dv": dev["dout"]}
            if gate is not None:
                results["dgate"] = dev["gate"]
        else:
            ql, kl, vl = (dev[n].detach().requires_grad_() for n in ("q", "k", "v"))
            gl = dev["gate"].detach().requires_grad_() if gate is not None else None
            o = b200_vsa(ql, kl, vl, kv_sizes, q_sizes, topk, block_size, gl)
            o.backward(dev["dout"])
            results = {"out": o.detach(), "dq": ql.grad, "dk": kl.grad, "dv": vl.grad}
            if gl is not None:
                results["dgate"] = gl.grad
            del o, ql, kl, vl, gl
        done = torch.cuda.Event()
        done.record(compute)
        copied = torch.cuda.Event()
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            for n, t in results.items():
                host_out[n][:, lo:hi].copy_(t, non_blocking=True)
            copied.record(copy_out)
        # the input buffers are free again once the kernels have read them -- and, in the copy-only schedule,
        # once the copy-out that reads them directly has finished
        if copy_schedule_only:
            compute.wait_event(copied)
        consumed[b].record(compute)
        in_flight.append((results, copied))
        del results
        if len(in_flight) > 2:                           # free a chunk's results only after they have left the GPU
            in_flight.pop(0)[1].synchronize()
    for _, ev in in_flight:
        ev.synchronize()
    compute.wait_stream(copy_out)
    compute.synchronize()
    if not copy_schedule_only:
        with torch.cuda.device(device):
            _lib.raise_on_device_timeout("vsa_step_from_host")
