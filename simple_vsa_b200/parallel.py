"""Multi-GPU layer of the VSA operator (one process per GPU, ``torch.distributed``).

Two modes, neither of which exists in the reference project (its kernels index every
``(batch, head)`` slice independently, ``vsa/triton_impl.py:83-86``, and it has no collective):

* **head sharding** -- the ``batch*heads`` slices are cut into contiguous ranges, one per rank, and
  each rank runs the ordinary operator on its range.  No data-path collective.
* **sequence parallelism** (long sequences) -- each rank owns ``L/W`` query tokens and the matching
  K/V shard.  K and V are all-gathered into local HBM (NCCL over NVLink) and stay in the rank-major
  layout ``[W, B, H, L/W, D]`` the collective leaves: the fine kernels address that layout in place
  (no re-layout copy after the gather), and write their partial dK/dV the same way, so that the
  backward's reduce-scatter takes them as they are.  The pooled keys/values are not recomputed from
  the gathered tokens: every rank pools its own shard and the small ``[B, H, Kb/W, D]`` results are
  all-gathered.  The rank then runs pooled scores ``[Qb/W, Kb]``, Top-K and the fine kernels with its
  local queries on global key-block ids (``Lq != Lkv``).  Remote data is always copied into the GPU's
  own memory first; no kernel reads a peer's memory.  Tensors the shard-major kernels do not cover
  (anything but bf16 / head dim 128 / block volume 64, 128 or 256, and CPU ranks with a stand-in operator)
  take the generic form: gather, re-lay-out to ``[B, H, L, D]``, ordinary operator.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def shard_slices(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous range ``(first, count)`` of ``total`` slices owned by ``rank`` (remainder to the low ranks)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    per, extra = divmod(total, world)
    return rank * per + min(rank, extra), per + (1 if rank < extra else 0)


def shard_heads(x: Tensor, world: int, rank: int) -> Tensor:
    """``[B,H,L,D] -> [1, count, L, D]``: this rank's contiguous share of the ``B*H`` slices."""
    B, H, L, D = x.shape
    first, count = shard_slices(B * H, world, rank)
    return x.reshape(1, B * H, L, D)[:, first:first + count]


class _GatherSequence(torch.autograd.Function):
    """all-gather along the sequence axis; the backward reduce-scatters the gradient."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:
        world = dist.get_world_size(group)
        ctx.group, ctx.world = group, world
        x = x.contiguous()
        B, H, l, D = x.shape
        gathered = torch.empty((world * B, H, l, D), device=x.device, dtype=x.dtype)   # rank-major concatenation
        dist.all_gather_into_tensor(gathered, x, group=group)
        return gathered.view(world, B, H, l, D).permute(1, 2, 0, 3, 4).reshape(B, H, world * l, D)

    @staticmethod
    def backward(ctx, grad: Tensor):
        world, group = ctx.world, ctx.group
        B, H, L, D = grad.shape
        l = L // world
        parts = grad.reshape(B, H, world, l, D).permute(2, 0, 1, 3, 4).contiguous()
        if dist.get_backend(group) == "nccl":
            out = torch.empty((B, H, l, D), device=grad.device, dtype=grad.dtype)
            dist.reduce_scatter_tensor(out, parts.view(world * B, H, l, D), op=dist.ReduceOp.SUM, group=group)
        else:   # backends without reduce-scatter (gloo on CPU): all-reduce, keep the own part
            dist.all_reduce(parts, op=dist.ReduceOp.SUM, group=group)
            out = parts[dist.get_rank(group)].contiguous()
        return out, None


class _GatherShards(torch.autograd.Function):
    """all-gather that keeps the collective's own layout: ``[B,H,l,D]`` shards -> ``[W,B,H,l,D]`` (rank-major).
    The backward reduce-scatters a gradient of that shape, which is already contiguous per owner rank."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:
        world = dist.get_world_size(group)
        ctx.group, ctx.world = group, world
        x = x.contiguous()
        gathered = torch.empty((world,) + tuple(x.shape), device=x.device, dtype=x.dtype)
        dist.all_gather_into_tensor(gathered.view((world * x.shape[0],) + tuple(x.shape[1:])), x, group=group)
        return gathered

    @staticmethod
    def backward(ctx, grad: Tensor):
        world, group = ctx.world, ctx.group
        grad = grad.contiguous()
        out = torch.empty(tuple(grad.shape[1:]), device=grad.device, dtype=grad.dtype)
        dist.reduce_scatter_tensor(out, grad.view((world * grad.shape[1],) + tuple(grad.shape[2:])),
                                   op=dist.ReduceOp.SUM, group=group)
        return out, None


def gather_shards(x: Tensor, group=None) -> Tensor:
    """Differentiable all-gather of ``[B,H,L/W,D]`` shards into the rank-major ``[W,B,H,L/W,D]``."""
    return _GatherShards.apply(x, group)


def gather_pooled(x_local: Tensor, sizes_local: Tensor, block_elements: int, group=None) -> Tensor:
    """Block means of this rank's shard, all-gathered into ``[B,H,Kb,D]`` in global block order (no gradient:
    the pooled-branch gradients reach K and V through the dK/dV kernel of the shard-major operator)."""
    from .ops import block_mean
    world = dist.get_world_size(group)
    with torch.no_grad():
        mean = block_mean(x_local.detach(), sizes_local, block_elements)            # [B,H,Kb/W,D]
        B, H, nbl, D = mean.shape
        out = torch.empty((world * B, H, nbl, D), device=mean.device, dtype=mean.dtype)
        dist.all_gather_into_tensor(out, mean.contiguous(), group=group)
        return out.view(world, B, H, nbl, D).permute(1, 2, 0, 3, 4).reshape(B, H, world * nbl, D)


def gather_sequence(x: Tensor, group=None) -> Tensor:
    """Differentiable all-gather of ``[B,H,L/W,D]`` shards into ``[B,H,L,D]`` (rank order = sequence order)."""
    return _GatherSequence.apply(x, group)


def _head_chunks(heads: int, chunks: int):
    chunks = max(1, min(chunks, heads))
    per, extra = divmod(heads, chunks)
    spans, lo = [], 0
    for i in range(chunks):
        n = per + (1 if i < extra else 0)
        spans.append((lo, lo + n))
        lo += n
    return spans


def sequence_parallel_vsa(q_local: Tensor, k_local: Tensor, v_local: Tensor, variable_block_sizes: Tensor,
                          q_variable_block_sizes_local: Tensor, topk: int, block_size=64,
                          compress_attn_weight_local: Optional[Tensor] = None, *, group=None,
                          local_op: Optional[Callable] = None, head_chunks: int = 4) -> Tensor:
    """VSA with the sequence split over the ranks of ``group``.

    ``q_local/k_local/v_local`` are this rank's ``[B,H,L/W,D]`` shards (rank r holds tokens
    ``[r*L/W, (r+1)*L/W)``; ``L/W`` must be a multiple of the block volume),
    ``variable_block_sizes`` lists ALL key blocks, ``q_variable_block_sizes_local`` this rank's query
    blocks.  Returns the local ``[B,H,L/W,D]`` output; gradients reach the local q/k/v (dK/dV are
    summed over ranks by the reduce-scatter) and the local gate.  ``local_op`` defaults to the CUDA
    operator and exists so that the glue can be exercised on CPU ranks with a stand-in.  The heads are
    processed in ``head_chunks`` groups so that the collectives of one group overlap the kernels of another.
    """
    sharded = False
    if local_op is None:
        from . import b200_vsa as local_op
        from .ops import as_block_elements, sharded_supported
        sharded = sharded_supported(q_local, as_block_elements(block_size), topk) and \
            dist.get_backend(group) == "nccl"
    H = q_local.shape[1]
    spans = _head_chunks(H, head_chunks)
    on_gpu = q_local.is_cuda
    if sharded:
        return _sequence_parallel_sharded(q_local, k_local, v_local, variable_block_sizes,
                                          q_variable_block_sizes_local, topk, block_size,
                                          compress_attn_weight_local, group, spans)
    if len(spans) == 1 or not on_gpu:
        outs = []
        for h0, h1 in spans:     # same arithmetic as the overlapped form below, on one stream
            gate = compress_attn_weight_local[:, h0:h1] if compress_attn_weight_local is not None else None
            outs.append(local_op(q_local[:, h0:h1], gather_sequence(k_local[:, h0:h1], group),
                                 gather_sequence(v_local[:, h0:h1], group), variable_block_sizes,
                                 q_variable_block_sizes_local, topk, block_size, gate))
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)

    # Heads are independent, so the exchange of one group of heads can run while another group computes.  The
    # gathers are issued on a side stream one group ahead of the compute; autograd runs each node's backward on
    # the stream of its forward, so the reduce-scatter of a group's dK/dV likewise overlaps the backward
    # compute of the group before it.  Exposed communication: the first gather and the last reduce-scatter.
    main = torch.cuda.current_stream(q_local.device)
    comm = _comm_stream(q_local.device)

    def start_gather(h0, h1):
        comm.wait_stream(main)                  # the shards (and whatever produced them) are ready
        with torch.cuda.stream(comm):
            kf = gather_sequence(k_local[:, h0:h1], group)
            vf = gather_sequence(v_local[:, h0:h1], group)
            done = torch.cuda.Event()
            done.record(comm)
        return kf, vf, done

    pending = [start_gather(*spans[0])]
    outs = []
    for i, (h0, h1) in enumerate(spans):
        if i + 1 < len(spans):
            pending.append(start_gather(*spans[i + 1]))
        kf, vf, done = pending[i]
        main.wait_event(done)
        kf.record_stream(main)
        vf.record_stream(main)
        gate = compress_attn_weight_local[:, h0:h1] if compress_attn_weight_local is not None else None
        outs.append(local_op(q_local[:, h0:h1], kf, vf, variable_block_sizes, q_variable_block_sizes_local, topk,
                             block_size, gate))
    return torch.cat(outs, dim=1)


def _sequence_parallel_sharded(q_local, k_local, v_local, variable_block_sizes, q_sizes_local, topk, block_size,
                               gate_local, group, spans):
    """The GPU form: per head group, K/V shards and pooled blocks are gathered on a side stream one group ahead of
    the compute and consumed in the layout the collective leaves."""
    from .ops import as_block_elements, vsa_on_gathered_shards
    be = as_block_elements(block_size)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    nbl = k_local.shape[2] // be
    sizes_local = variable_block_sizes[rank * nbl:(rank + 1) * nbl]
    main = torch.cuda.current_stream(q_local.device)
    comm = _comm_stream(q_local.device)

    def start_gather(h0, h1):
        comm.wait_stream(main)
        with torch.cuda.stream(comm):
            k_sh = gather_shards(k_local[:, h0:h1], group)
            v_sh = gather_shards(v_local[:, h0:h1], group)
            kc = gather_pooled(k_local[:, h0:h1], sizes_local, be, group)
            vc = gather_pooled(v_local[:, h0:h1], sizes_local, be, group)
            done = torch.cuda.Event()
            done.record(comm)
        return k_sh, v_sh, kc, vc, done

    pending = [start_gather(*spans[0])]
    outs = []
    for i, (h0, h1) in enumerate(spans):
        if i + 1 < len(spans):
            pending.append(start_gather(*spans[i + 1]))
        k_sh, v_sh, kc, vc, done = pending[i]
        main.wait_event(done)
        for t in (k_sh, v_sh, kc, vc):
            t.record_stream(main)
        gate = gate_local[:, h0:h1] if gate_local is not None else None
        outs.append(vsa_on_gathered_shards(q_local[:, h0:h1], k_sh, v_sh, kc, vc, variable_block_sizes, q_sizes_local,
                                           topk, block_size, gate))
    return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)


_COMM_STREAMS = {}


def _comm_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = torch.cuda.Stream(device)
    return _COMM_STREAMS[key]
