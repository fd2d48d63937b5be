"""Host side of the VSA operator: argument checks, buffers, autograd wiring.

Mirrors the reference project's operator layer (``vsa/triton_impl.py:1530-1765``:
``_TritonSparseAttention``, ``_triton_sparse_attention``,
``_vsa_with_sparse_executor``) with one difference in structure: the whole
operator is a single ``autograd.Function`` so that the pooled-branch backward
runs before the fine backward and the block-mean gradients are accumulated
straight into dq/dk/dv instead of through three extra full-size tensors.

All compute goes through the C ABI of ``libvsa_b200.so``; torch is used for
device memory, the current stream and autograd only.
"""

from __future__ import annotations

import math
import os
import warnings
from typing import Optional, Sequence, Tuple, Union

import torch
from torch import Tensor

from . import _lib
from ._lib import call

BlockSize = Union[int, Sequence[int]]


def as_block_elements(block_size: BlockSize) -> int:
    """An int is a cube edge, a tuple is multiplied out (``vsa/common.py:39-42``)."""
    if isinstance(block_size, int):
        return block_size * block_size * block_size
    return int(math.prod(block_size))


def validate_vsa_inputs(q, k, v, variable_block_sizes, q_variable_block_sizes, topk: int, be: int) -> None:
    """Shape contract of the operator; messages keep the reference's wording (``vsa/common.py:97-134``)."""
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, and v must have shape [batch, heads, seq_len, dim]")
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    if k.shape[0] != B or v.shape[0] != B or k.shape[1] != H or v.shape[1] != H:
        raise ValueError("q, k, and v must share batch and head dimensions")
    if v.shape[2] != Lkv:
        raise ValueError("k and v must have the same sequence length")
    if k.shape[-1] != D or v.shape[-1] != D:
        raise ValueError("q, k, and v must have the same head dimension")
    if Lq % be or Lkv % be:
        raise ValueError(f"q/kv sequence lengths must be divisible by block_elements={be}")
    if variable_block_sizes.numel() != Lkv // be:
        raise ValueError(
            f"variable_block_sizes must have length {Lkv // be}, got {variable_block_sizes.numel()}")
    if q_variable_block_sizes.numel() != Lq // be:
        raise ValueError(
            f"q_variable_block_sizes must have length {Lq // be}, got {q_variable_block_sizes.numel()}")
    if not 1 <= topk <= Lkv // be:
        raise ValueError(f"topk must be in [1, {Lkv // be}]")


def _check_device_dtype(q: Tensor, k: Tensor, v: Tensor) -> int:
    """Same refusals as the reference launcher (``vsa/triton_impl.py:371-384``)."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("the B200 implementation requires CUDA tensors")
    if not (q.device == k.device == v.device):
        raise ValueError("q, k, and v must be on the same CUDA device")
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k, and v must have the same dtype")
    if q.dtype == torch.bfloat16:
        return _lib.VSA_BF16
    if q.dtype == torch.float32:
        return _lib.VSA_F32
    if q.dtype == torch.float16:
        return _lib.VSA_F16
    raise ValueError("the B200 path supports bfloat16, float16 and float32")


_warned_slow_path = False


def _warn_if_far_off_the_tensor_path(dt: int, B: int, H: int, Lq: int, D: int, be: int, topk: int) -> None:
    """One warning per process when a large problem lands on the CUDA-core kernels.  They exist as the validation
    mode (fp32) and for shapes the reference accepts but its benchmarks never use; per FLOP they are two to three
    orders of magnitude slower than the tcgen05 kernels, which a caller should learn from more than a slow step."""
    global _warned_slow_path
    if _warned_slow_path or 14.0 * B * H * Lq * topk * be * D < 1e11:
        return
    if _lib.lib.vsa_sparse_kernel_family(D, be, topk, dt) > 0:      # tcgen05 or warp-level tensor-core kernels
        return
    _warned_slow_path = True
    warnings.warn("simple_vsa_b200: this shape runs on the CUDA-core validation kernels (the tensor-core paths need "
                  "bf16 or fp16, head dim 64 or 128, block volume 64, 128 or 256, and VSA_B200_KERNELS unset or =mma); expect a step hundreds of times slower per FLOP", RuntimeWarning, stacklevel=3)


def _dense(x: Tensor) -> Tensor:
    """Contiguous and 16-byte aligned (the kernels use 16-byte vector accesses)."""
    x = x.contiguous()
    if x.data_ptr() % 16:
        x = x.clone()
    return x


def _sizes(sizes: Tensor, device) -> Tensor:
    return sizes.to(device=device, dtype=torch.int32).contiguous()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[Tensor]):
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------------------------
# thin launch wrappers (no autograd); every tensor is dense and on one device
# --------------------------------------------------------------------------------------------
def sparse_forward(q, k, v, selected, kv_sizes, be: int, scale: float, want_lse: bool, combine_with=None):
    """Fine branch.  ``combine_with = (out_c, gate_or_None)`` also returns ``out = out_s + out_c[block] * gate``,
    written by the same kernel on its way out (third element of the result)."""
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    dt = _check_device_dtype(q, k, v)
    out = torch.empty_like(q)
    # the statistic buffer is always handed over: the tcgen05 forward needs it as scratch (4 bytes per row)
    lse = torch.empty((B, H, Lq), device=q.device, dtype=torch.float32)
    if combine_with is not None:
        out_c, gate = combine_with
        total = torch.empty_like(q)
        call("vsa_sparse_fwd_combine", q.data_ptr(), k.data_ptr(), v.data_ptr(), selected.data_ptr(),
             kv_sizes.data_ptr(), out.data_ptr(), _ptr(lse), out_c.data_ptr(), _ptr(gate), total.data_ptr(), B * H, Lq,
             Lkv, D, be, selected.shape[-1], scale, dt, _stream(q.device))
        return out, (lse if want_lse else None), total
    call("vsa_sparse_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), selected.data_ptr(), kv_sizes.data_ptr(),
         out.data_ptr(), _ptr(lse), B * H, Lq, Lkv, D, be, selected.shape[-1], scale, dt, _stream(q.device))
    return out, (lse if want_lse else None)


def invert_routes(selected: Tensor, key_blocks: int):
    """CSR of key block -> query blocks: (inverse [B,H,Qb*tk], offsets [B,H,Kb], counts [B,H,Kb]), int32.

    Same triple, in the same order, as the reference's ``_invert_indices`` (``vsa/triton_impl.py:544-595``).
    """
    B, H, Qb, tk = selected.shape
    dev = selected.device
    counts = torch.empty((B, H, key_blocks), device=dev, dtype=torch.int32)
    offsets = torch.empty_like(counts)
    cursor = torch.empty_like(counts)
    inverse = torch.empty((B, H, Qb * tk), device=dev, dtype=torch.int32)
    call("vsa_route_invert", selected.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(),
         cursor.data_ptr(), B * H, Qb, key_blocks, tk, _stream(dev))
    return inverse, offsets, counts


def invert_routes_edges(selected: Tensor, key_blocks: int):
    """``invert_routes`` with every in-edge recorded as ``(query_block << 11) | slot`` (slot = position of the
    key block in that query block's row of ``selected``), which names the edge for the stored-dS backward."""
    B, H, Qb, tk = selected.shape
    dev = selected.device
    counts = torch.empty((B, H, key_blocks), device=dev, dtype=torch.int32)
    offsets = torch.empty_like(counts)
    cursor = torch.empty_like(counts)
    inverse = torch.empty((B, H, Qb * tk), device=dev, dtype=torch.int32)
    call("vsa_route_invert_edges", selected.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(),
         cursor.data_ptr(), B * H, Qb, key_blocks, tk, _stream(dev))
    return inverse, offsets, counts


def _ds_workspace_cap() -> int:
    """Upper bound in bytes for the dS workspace of one group of slices (``VSA_B200_DS_WORKSPACE_GB``, default 16)."""
    return int(float(os.environ.get("VSA_B200_DS_WORKSPACE_GB", "16")) * (1 << 30))


def _sparse_backward_stored_ds(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale, pooled_grads, dt, st):
    """delta, then per group of slices: key-owned dK/dV pass that also stores dS, query-owned dQ = scale * dS K.

    The scores and dP are formed once instead of once per pass; the price is the dS workspace (8 KB per query
    tile x selected key tile), which is why the slices are walked in groups that keep it under a fixed size."""
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    BH, Qb, Kb, tk = B * H, Lq // be, Lkv // be, selected.shape[-1]
    inverse, offsets, counts = invert_routes_edges(selected, Kb)
    delta = torch.empty_like(lse)
    call("vsa_sparse_bwd_delta", out_s.data_ptr(), dout.data_ptr(), delta.data_ptr(), BH, Lq, D, dt, st)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    per_slice = int(_lib.lib.vsa_sparse_bwd_ds_workspace_bytes(1, Lq, be, tk))
    group = max(1, min(BH, _ds_workspace_cap() // max(1, per_slice)))
    ws = torch.empty(group * per_slice, device=q.device, dtype=torch.uint8)
    dqc = dkc = dvc = q_sizes = None
    if pooled_grads is not None:
        dqc, dkc, dvc, q_sizes = pooled_grads

    def at(t, s0, *shape):          # address of slice s0 of a [B, H, ...] tensor
        return None if t is None else t.view(BH, *shape)[s0].data_ptr()

    for s0 in range(0, BH, group):
        n = min(group, BH - s0)
        call("vsa_sparse_bwd_dkdv_ds", at(dout, s0, Lq, D), at(q, s0, Lq, D), at(k, s0, Lkv, D), at(v, s0, Lkv, D),
             at(lse, s0, Lq), at(delta, s0, Lq), at(counts, s0, Kb), at(offsets, s0, Kb), at(inverse, s0, Qb * tk),
             kv_sizes.data_ptr(), at(dk, s0, Lkv, D), at(dv, s0, Lkv, D), at(dkc, s0, Kb, D), at(dvc, s0, Kb, D),
             ws.data_ptr(), n, Lq, Lkv, D, be, tk, scale, dt, st)
        call("vsa_sparse_bwd_dq_from_ds", at(k, s0, Lkv, D), at(selected, s0, Qb, tk), kv_sizes.data_ptr(),
             ws.data_ptr(), at(dq, s0, Lq, D), at(dqc, s0, Qb, D), _ptr(q_sizes), n, Lq, Lkv, D, be, tk, scale, dt, st)
    return dq, dk, dv


def sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be: int, scale: float, pooled_grads=None):
    """dQ, dK, dV of the fine branch.  ``pooled_grads = (dq_mean, dk_mean, dv_mean, q_sizes)`` folds the
    block-mean backward of the pooled branch into the same kernels' stores.

    The default is two independent passes that each recompute the scores and dP (a query-owned dQ pass and a
    key-owned dK/dV pass, like the reference).  ``VSA_B200_BACKWARD=stored_ds`` selects, on the tensor path, the
    variant that forms dS once (``_sparse_backward_stored_ds``): 16 of 56 tensor-core products per pair of edges
    fewer, but 8 KB per edge written and read back; on a B200 the extra write traffic slows the key-owned pass by
    about as much as the dQ pass gains, so it is not the default."""
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    dt = _check_device_dtype(q, k, v)
    st = _stream(q.device)
    tk = selected.shape[-1]
    if os.environ.get("VSA_B200_BACKWARD", "") == "stored_ds" and \
            _lib.lib.vsa_sparse_bwd_ds_supported(D, be, tk, dt):
        return _sparse_backward_stored_ds(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale, pooled_grads,
                                          dt, st)
    inverse, offsets, counts = invert_routes(selected, Lkv // be)
    delta = torch.empty_like(lse)
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    if pooled_grads is not None:
        dqc, dkc, dvc, q_sizes = pooled_grads
        call("vsa_sparse_bwd_dq_fused", dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out_s.data_ptr(),
             lse.data_ptr(), selected.data_ptr(), kv_sizes.data_ptr(), delta.data_ptr(), dq.data_ptr(),
             dqc.data_ptr(), q_sizes.data_ptr(), B * H, Lq, Lkv, D, be, tk, scale, dt, st)
        call("vsa_sparse_bwd_dkdv_fused", dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), lse.data_ptr(),
             delta.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(), kv_sizes.data_ptr(),
             dk.data_ptr(), dv.data_ptr(), dkc.data_ptr(), dvc.data_ptr(), B * H, Lq, Lkv, D, be, tk, scale, dt, st)
        return dq, dk, dv
    call("vsa_sparse_bwd_dq", dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out_s.data_ptr(),
         lse.data_ptr(), selected.data_ptr(), kv_sizes.data_ptr(), delta.data_ptr(), dq.data_ptr(),
         B * H, Lq, Lkv, D, be, tk, scale, dt, st)
    call("vsa_sparse_bwd_dkdv", dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), lse.data_ptr(),
         delta.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(), kv_sizes.data_ptr(),
         dk.data_ptr(), dv.data_ptr(), B * H, Lq, Lkv, D, be, tk, scale, dt, st)
    return dq, dk, dv


def pooled_forward(q, k, v, kv_sizes, q_sizes, be: int, scale: float, topk: int):
    """Block means, pooled scores/probabilities/output and the Top-K routing table."""
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    Qb, Kb = Lq // be, Lkv // be
    dt = _check_device_dtype(q, k, v)
    st = _stream(q.device)
    dev, ty = q.device, q.dtype
    qc = torch.empty((B, H, Qb, D), device=dev, dtype=ty)
    kc = torch.empty((B, H, Kb, D), device=dev, dtype=ty)
    vc = torch.empty((B, H, Kb, D), device=dev, dtype=ty)
    call("vsa_block_mean3_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), q_sizes.data_ptr(), kv_sizes.data_ptr(),
         qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), B * H, Lq, Lkv, D, be, dt, st)
    scores = torch.empty((B, H, Qb, Kb), device=dev, dtype=ty)
    probs = torch.empty_like(scores)
    out_c = torch.empty((B, H, Qb, D), device=dev, dtype=ty)
    call("vsa_coarse_fwd", qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), scores.data_ptr(), probs.data_ptr(),
         out_c.data_ptr(), B * H, Qb, Kb, D, scale, dt, st)
    selected = torch.empty((B, H, Qb, topk), device=dev, dtype=torch.int32)
    call("vsa_topk", scores.data_ptr(), selected.data_ptr(), B * H * Qb, Kb, topk, dt, st)
    return qc, kc, vc, scores, probs, out_c, selected


class _SparseAttention(torch.autograd.Function):
    """Route-explicit fine attention (``vsa/triton_impl.py:1530-1580``)."""

    @staticmethod
    def forward(ctx, q, k, v, selected, kv_sizes, be, scale):
        out, lse = sparse_forward(q, k, v, selected, kv_sizes, be, scale, True)
        ctx.save_for_backward(q, k, v, out, lse, selected, kv_sizes)
        ctx.be, ctx.scale = be, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, selected, kv_sizes = ctx.saved_tensors
        with torch.cuda.device(q.device):
            dq, dk, dv = sparse_backward(_dense(dout), q, k, v, out, lse, selected, kv_sizes, ctx.be, ctx.scale)
        return dq, dk, dv, None, None, None, None


def sparse_attention(q, k, v, selected, variable_block_sizes, *, block_size: BlockSize,
                     sm_scale: Optional[float] = None) -> Tensor:
    """Fine attention on caller-supplied routes ``selected [B,H,Qb,topk]`` (``vsa/triton_impl.py:1583-1652``)."""
    be = as_block_elements(block_size)
    dt = _check_device_dtype(q, k, v)
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, and v must have shape [batch, heads, seq_len, dim]")
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    if Lq % be or Lkv % be:
        raise ValueError(f"q/kv sequence lengths must be divisible by block_elements={be}")
    if tuple(selected.shape[:3]) != (B, H, Lq // be):
        raise ValueError("selected must have shape [batch, heads, query_blocks, topk]")
    tk = selected.shape[-1]
    if not 1 <= tk <= Lkv // be:
        raise ValueError(f"selected topk must be in [1, {Lkv // be}]")
    if variable_block_sizes.numel() != Lkv // be:
        raise ValueError(
            f"variable_block_sizes must have {Lkv // be} entries, got {variable_block_sizes.numel()}")
    scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
    with torch.cuda.device(q.device):
        _warn_if_far_off_the_tensor_path(dt, B, H, Lq, D, be, tk)
        q, k, v = _dense(q), _dense(k), _dense(v)
        selected = selected.to(device=q.device, dtype=torch.int32).contiguous()
        sizes = _sizes(variable_block_sizes, q.device)
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
            return _SparseAttention.apply(q, k, v, selected, sizes, be, scale)
        return sparse_forward(q, k, v, selected, sizes, be, scale, False)[0]


class _VideoSparseAttention(torch.autograd.Function):
    """Whole operator: pooled branch, Top-K, fine branch, gated combine -- and its backward."""

    @staticmethod
    def forward(ctx, q, k, v, gate, kv_sizes, q_sizes, topk, be, scale, need_grad):
        B, H, Lq, D = q.shape
        dt = _check_device_dtype(q, k, v)
        st = _stream(q.device)
        qc, kc, vc, scores, probs, out_c, selected = pooled_forward(q, k, v, kv_sizes, q_sizes, be, scale, topk)
        # the gated combine rides on the store of the fine output (no separate pass over out_s)
        out_s, lse, out = sparse_forward(q, k, v, selected, kv_sizes, be, scale, need_grad, combine_with=(out_c, gate))
        if need_grad:
            saved = [q, k, v, out_s, lse, selected, kv_sizes, q_sizes, qc, kc, vc, probs, out_c]
            if gate is not None:
                saved.append(gate)
            ctx.save_for_backward(*saved)
            ctx.has_gate = gate is not None
            ctx.be, ctx.scale = be, scale
        ctx.mark_non_differentiable(scores, selected, out_c, out_s)
        return out, scores, selected, out_c, out_s

    @staticmethod
    def backward(ctx, dout, _dscores, _dselected, _dout_c, _dout_s):
        saved = ctx.saved_tensors
        q, k, v, out_s, lse, selected, kv_sizes, q_sizes, qc, kc, vc, probs, out_c = saved[:13]
        gate = saved[13] if ctx.has_gate else None
        be, scale = ctx.be, ctx.scale
        B, H, Lq, D = q.shape
        Lkv = k.shape[2]
        Qb, Kb = Lq // be, Lkv // be
        with torch.cuda.device(q.device):
            dt = _check_device_dtype(q, k, v)
            st = _stream(q.device)
            dout = _dense(dout)
            d_out_c = torch.empty_like(out_c)
            dgate = torch.empty_like(gate) if gate is not None else None
            call("vsa_combine_bwd", dout.data_ptr(), _ptr(gate), out_c.data_ptr(), d_out_c.data_ptr(), _ptr(dgate),
                 B * H, Lq, D, be, dt, st)
            ds_ws = torch.empty_like(probs)
            rowdot = torch.empty((B, H, Qb), device=q.device, dtype=torch.float32)
            dqc, dkc, dvc = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
            call("vsa_coarse_bwd", d_out_c.data_ptr(), out_c.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                 probs.data_ptr(), ds_ws.data_ptr(), rowdot.data_ptr(), dqc.data_ptr(), dkc.data_ptr(),
                 dvc.data_ptr(), B * H, Qb, Kb, D, scale, dt, st)
            del ds_ws
            # the block-mean backward of the pooled gradients rides on the stores of the fine backward
            dq, dk, dv = sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale,
                                         pooled_grads=(dqc, dkc, dvc, q_sizes))
        return dq, dk, dv, dgate, None, None, None, None, None, None


class _ShardedVideoSparseAttention(torch.autograd.Function):
    """One rank's part of the sequence-parallel operator: its own queries against the all-gathered K/V, read in the
    shard-major layout the gather leaves (``[W, B, H, L/W, D]``), with the pooled keys/values of ALL blocks given.

    The gradients returned for the gathered K/V are this rank's partial sums over its query blocks, in the same
    shard-major layout (ready for a reduce-scatter); the pooled-branch gradients of the keys/values are folded into
    them by the dK/dV kernel, so the pooled tensors themselves need no gradient path of their own."""

    @staticmethod
    def forward(ctx, q, k_sh, v_sh, gate, kc, vc, kv_sizes, q_sizes, topk, be, scale, need_grad):
        B, H, Lq, D = q.shape
        W, shard = k_sh.shape[0], k_sh.shape[3]
        Lkv = W * shard
        Qb, Kb = Lq // be, Lkv // be
        dt = _check_device_dtype(q, k_sh, v_sh)
        st = _stream(q.device)
        dev, ty = q.device, q.dtype
        qc = torch.empty((B, H, Qb, D), device=dev, dtype=ty)
        call("vsa_block_mean_fwd", q.data_ptr(), q_sizes.data_ptr(), qc.data_ptr(), B * H, Lq, D, be, dt, st)
        scores = torch.empty((B, H, Qb, Kb), device=dev, dtype=ty)
        probs = torch.empty_like(scores)
        out_c = torch.empty((B, H, Qb, D), device=dev, dtype=ty)
        call("vsa_coarse_fwd", qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), scores.data_ptr(), probs.data_ptr(),
             out_c.data_ptr(), B * H, Qb, Kb, D, scale, dt, st)
        selected = torch.empty((B, H, Qb, topk), device=dev, dtype=torch.int32)
        call("vsa_topk", scores.data_ptr(), selected.data_ptr(), B * H * Qb, Kb, topk, dt, st)
        del scores
        out_s, out = torch.empty_like(q), torch.empty_like(q)
        lse = torch.empty((B, H, Lq), device=dev, dtype=torch.float32)
        call("vsa_sparse_fwd_combine_sharded", q.data_ptr(), k_sh.data_ptr(), v_sh.data_ptr(), selected.data_ptr(),
             kv_sizes.data_ptr(), out_s.data_ptr(), lse.data_ptr(), out_c.data_ptr(), _ptr(gate), out.data_ptr(), B * H,
             Lq, Lkv, shard, D, be, topk, scale, dt, st)
        if need_grad:
            saved = [q, k_sh, v_sh, out_s, lse, selected, kv_sizes, q_sizes, qc, kc, vc, probs, out_c]
            if gate is not None:
                saved.append(gate)
            ctx.save_for_backward(*saved)
            ctx.has_gate = gate is not None
            ctx.be, ctx.scale = be, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        saved = ctx.saved_tensors
        q, k_sh, v_sh, out_s, lse, selected, kv_sizes, q_sizes, qc, kc, vc, probs, out_c = saved[:13]
        gate = saved[13] if ctx.has_gate else None
        be, scale = ctx.be, ctx.scale
        B, H, Lq, D = q.shape
        W, shard = k_sh.shape[0], k_sh.shape[3]
        Lkv = W * shard
        Qb, Kb, tk = Lq // be, Lkv // be, selected.shape[-1]
        with torch.cuda.device(q.device):
            dt = _check_device_dtype(q, k_sh, v_sh)
            st = _stream(q.device)
            dout = _dense(dout)
            d_out_c = torch.empty_like(out_c)
            dgate = torch.empty_like(gate) if gate is not None else None
            call("vsa_combine_bwd", dout.data_ptr(), _ptr(gate), out_c.data_ptr(), d_out_c.data_ptr(), _ptr(dgate),
                 B * H, Lq, D, be, dt, st)
            ds_ws = torch.empty_like(probs)
            rowdot = torch.empty((B, H, Qb), device=q.device, dtype=torch.float32)
            dqc, dkc, dvc = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
            call("vsa_coarse_bwd", d_out_c.data_ptr(), out_c.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                 probs.data_ptr(), ds_ws.data_ptr(), rowdot.data_ptr(), dqc.data_ptr(), dkc.data_ptr(),
                 dvc.data_ptr(), B * H, Qb, Kb, D, scale, dt, st)
            del ds_ws
            inverse, offsets, counts = invert_routes(selected, Kb)
            delta = torch.empty_like(lse)
            dq = torch.empty_like(q)
            dk_sh, dv_sh = torch.empty_like(k_sh), torch.empty_like(v_sh)
            call("vsa_sparse_bwd_dq_sharded", dout.data_ptr(), q.data_ptr(), k_sh.data_ptr(), v_sh.data_ptr(),
                 out_s.data_ptr(), lse.data_ptr(), selected.data_ptr(), kv_sizes.data_ptr(), delta.data_ptr(),
                 dq.data_ptr(), dqc.data_ptr(), q_sizes.data_ptr(), B * H, Lq, Lkv, shard, D, be, tk, scale, dt, st)
            # dkc / dvc are this rank's share of the pooled gradients of ALL key blocks: folded into its partial dK/dV
            call("vsa_sparse_bwd_dkdv_sharded", dout.data_ptr(), q.data_ptr(), k_sh.data_ptr(), v_sh.data_ptr(),
                 lse.data_ptr(), delta.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(),
                 kv_sizes.data_ptr(), dk_sh.data_ptr(), dv_sh.data_ptr(), dkc.data_ptr(), dvc.data_ptr(), B * H, Lq, Lkv,
                 shard, D, be, tk, scale, dt, st)
        return dq, dk_sh, dv_sh, dgate, None, None, None, None, None, None, None, None


def sharded_supported(q: Tensor, be: int, topk: int) -> bool:
    """Whether the shard-major kernels cover these tensors (bf16 or fp16, head dim 128, block volume 64, 128 or 256,
    CUDA)."""
    if not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    dt = _lib.VSA_BF16 if q.dtype == torch.bfloat16 else _lib.VSA_F16
    return bool(_lib.lib.vsa_sparse_sharded_supported(q.shape[-1], be, topk, dt))


def vsa_on_gathered_shards(q, k_sh, v_sh, kc, vc, variable_block_sizes, q_variable_block_sizes, topk: int,
                           block_size: BlockSize = 64, compress_attn_weight: Optional[Tensor] = None) -> Tensor:
    """The operator for one rank of a sequence-parallel group: ``q [B,H,l,D]`` (this rank's queries),
    ``k_sh, v_sh [W,B,H,l,D]`` (the all-gathered shards, rank-major, as the collective left them), ``kc, vc
    [B,H,Kb,D]`` (pooled keys/values of all ``Kb = W*l/be`` blocks in global order, no gradient needed),
    ``variable_block_sizes [Kb]``, ``q_variable_block_sizes [l/be]``.  Differentiable in q, k_sh, v_sh and the gate."""
    be = as_block_elements(block_size)
    B, H, Lq, D = q.shape
    W, shard = k_sh.shape[0], k_sh.shape[3]
    if tuple(k_sh.shape) != (W, B, H, shard, D) or v_sh.shape != k_sh.shape:
        raise ValueError("k_sh and v_sh must have shape [world, batch, heads, shard_len, dim]")
    Lkv = W * shard
    if Lq % be or shard % be:
        raise ValueError(f"q/kv sequence lengths must be divisible by block_elements={be}")
    if variable_block_sizes.numel() != Lkv // be:
        raise ValueError(f"variable_block_sizes must have length {Lkv // be}, got {variable_block_sizes.numel()}")
    if q_variable_block_sizes.numel() != Lq // be:
        raise ValueError(f"q_variable_block_sizes must have length {Lq // be}, got {q_variable_block_sizes.numel()}")
    if not 1 <= topk <= Lkv // be:
        raise ValueError(f"topk must be in [1, {Lkv // be}]")
    if tuple(kc.shape) != (B, H, Lkv // be, D) or vc.shape != kc.shape:
        raise ValueError("kc and vc must have shape [batch, heads, key_blocks, dim]")
    gate = compress_attn_weight
    if gate is not None and gate.shape != q.shape:
        raise ValueError("compress_attn_weight must have the same shape as q")
    if not sharded_supported(q, be, topk):
        raise ValueError("the shard-major path needs bfloat16 or float16 CUDA tensors with head dim 128 and block volume 64, 128 or 256")
    scale = 1.0 / math.sqrt(D)
    with torch.cuda.device(q.device):
        q, k_sh, v_sh = _dense(q), _dense(k_sh), _dense(v_sh)
        gate = _dense(gate.to(q.dtype)) if gate is not None else None
        kv_sizes = _sizes(variable_block_sizes, q.device)
        q_sizes = _sizes(q_variable_block_sizes, q.device)
        need_grad = torch.is_grad_enabled() and any(
            t is not None and t.requires_grad for t in (q, k_sh, v_sh, gate))
        return _ShardedVideoSparseAttention.apply(q, k_sh, v_sh, gate, _dense(kc.detach()), _dense(vc.detach()),
                                                  kv_sizes, q_sizes, int(topk), be, scale, need_grad)


def vsa_forward_full(q, k, v, variable_block_sizes, q_variable_block_sizes, topk: int, block_size: BlockSize = 64,
                     compress_attn_weight: Optional[Tensor] = None, sm_scale: Optional[float] = None
                     ) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Run the operator; returns (out, pooled scores, routing table, pooled output, fine output)."""
    be = as_block_elements(block_size)
    validate_vsa_inputs(q, k, v, variable_block_sizes, q_variable_block_sizes, topk, be)
    if compress_attn_weight is not None and compress_attn_weight.shape != q.shape:
        raise ValueError("compress_attn_weight must have the same shape as q")
    dt = _check_device_dtype(q, k, v)
    gate = compress_attn_weight
    if gate is not None and (gate.device != q.device or gate.dtype != q.dtype):
        gate = gate.to(device=q.device, dtype=q.dtype)
    scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    with torch.cuda.device(q.device):
        _warn_if_far_off_the_tensor_path(dt, q.shape[0], q.shape[1], q.shape[2], q.shape[3], be, int(topk))
        q, k, v = _dense(q), _dense(k), _dense(v)
        gate = _dense(gate) if gate is not None else None
        kv_sizes = _sizes(variable_block_sizes, q.device)
        q_sizes = _sizes(q_variable_block_sizes, q.device)
        need_grad = torch.is_grad_enabled() and any(
            t is not None and t.requires_grad for t in (q, k, v, gate))
        return _VideoSparseAttention.apply(q, k, v, gate, kv_sizes, q_sizes, int(topk), be, scale, need_grad)


class _BlockMean(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sizes, be):
        B, H, L, D = x.shape
        dt = {torch.bfloat16: _lib.VSA_BF16, torch.float32: _lib.VSA_F32, torch.float16: _lib.VSA_F16}[x.dtype]
        out = torch.empty((B, H, L // be, D), device=x.device, dtype=x.dtype)
        call("vsa_block_mean_fwd", x.data_ptr(), sizes.data_ptr(), out.data_ptr(), B * H, L, D, be, dt,
             _stream(x.device))
        ctx.save_for_backward(sizes)
        ctx.shape, ctx.be, ctx.dt = x.shape, be, dt
        return out

    @staticmethod
    def backward(ctx, dmean):
        (sizes,) = ctx.saved_tensors
        B, H, L, D = ctx.shape
        with torch.cuda.device(dmean.device):
            dmean = _dense(dmean)
            dx = torch.empty(ctx.shape, device=dmean.device, dtype=dmean.dtype)
            call("vsa_block_mean_bwd", dx.data_ptr(), dmean.data_ptr(), sizes.data_ptr(), B * H, L, D, ctx.be,
                 ctx.dt, _stream(dmean.device))
        return dx, None, None


def block_mean(x: Tensor, variable_block_sizes: Tensor, block_elements: int) -> Tensor:
    """Padding-aware block means ``[B,H,L,D] -> [B,H,L/be,D]`` (``vsa/common.py:55-82``), differentiable."""
    if not x.is_cuda:
        raise ValueError("the B200 implementation requires CUDA tensors")
    if x.dtype not in (torch.bfloat16, torch.float32, torch.float16):
        raise ValueError("the B200 path supports bfloat16, float16 and float32")
    if x.ndim != 4 or x.shape[2] % block_elements:
        raise ValueError(f"sequence length must be divisible by block_elements={block_elements}")
    with torch.cuda.device(x.device):
        return _BlockMean.apply(_dense(x), _sizes(variable_block_sizes, x.device), int(block_elements))
