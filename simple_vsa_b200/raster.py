"""The operator on raster-order activations: the tiling front end folded into the kernels.

A DiT layer holds q, k, v, the gate and the attention output as ``[B, S, H, D]`` with the ``S = T*H*W`` tokens in
raster order.  The reference path around the operator is ``tile`` (index gather into zero-padded tile order,
``vsa/fastvideo_tiling.py:128-140``), a transpose to ``[B, H, L, D]``, the operator, a transpose back and ``untile``
(``:143-145``): two tensor-sized copies per input and two per output, and as many again for the gradients.

Here every operand is made in ONE pass (``vsa_gather_rows_heads``: gather + head transpose + zero padding, needed
because TMA reads 64-token tiles as contiguous rows), and nothing is moved back: the forward kernel reads the gate and
writes the combined output at each token's raster row, and the dQ and dK/dV kernels write the gradients there too.
The backward's first kernel (combine backward) reads dout and the gate at raster rows, writes dgate there and leaves
the tile-order copy of dout the TMA loads need as a by-product.  Per training step that is 3 layout passes (q, k,
v) and no other tensor-sized copy, instead of 18; for inference 3 instead of 10.

Tensor path only (bf16/fp16, head dim 128, block volume 64, 128 or 256); other CUDA shapes take the two-step form
with the same numbers.
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch
from torch import Tensor

from . import _lib, ops
from ._lib import call


def _gather_heads(x: Tensor, row_map: Tensor, dst_rows: int, to_tiled: bool) -> Tensor:
    """``[B,S,H,D] -> [B,H,L,D]`` (``to_tiled``) or ``[B,H,L,D] -> [B,S,H,D]``, one kernel."""
    x = ops._dense(x)
    if to_tiled:
        B, src_rows, H, D = x.shape
        out = torch.empty((B, H, dst_rows, D), device=x.device, dtype=x.dtype)
    else:
        B, H, src_rows, D = x.shape
        out = torch.empty((B, dst_rows, H, D), device=x.device, dtype=x.dtype)
    call("vsa_gather_rows_heads", x.data_ptr(), row_map.data_ptr(), out.data_ptr(), B, H, src_rows, dst_rows,
         D * x.element_size(), 1 if to_tiled else 0, ops._stream(x.device))
    return out


def raster_supported(q: Tensor, be: int, topk: int) -> bool:
    """Whether the kernels with raster-order stores cover these tensors."""
    if not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    dt = _lib.VSA_BF16 if q.dtype == torch.bfloat16 else _lib.VSA_F16
    return bool(_lib.lib.vsa_sparse_raster_supported(q.shape[-1], be, topk, dt))


class _RasterVideoSparseAttention(torch.autograd.Function):
    """Whole operator on ``[B,S,H,D]`` raster-order tensors (self-attention over one token grid)."""

    @staticmethod
    def forward(ctx, q, k, v, gate, tile_map, untile_map, sizes, topk, be, scale, need_grad):
        B, S, H, D = q.shape
        L = tile_map.numel()
        dt = ops._check_device_dtype(q, k, v)
        st = ops._stream(q.device)
        qt, kt, vt = (_gather_heads(t, tile_map, L, True) for t in (q, k, v))
        qc, kc, vc, scores, probs, out_c, selected = ops.pooled_forward(qt, kt, vt, sizes, sizes, be, scale, topk)
        out_s = torch.empty_like(qt)
        lse = torch.empty((B, H, L), device=q.device, dtype=torch.float32)
        out = torch.empty_like(q)
        call("vsa_sparse_fwd_combine_raster", qt.data_ptr(), kt.data_ptr(), vt.data_ptr(), selected.data_ptr(),
             sizes.data_ptr(), out_s.data_ptr(), lse.data_ptr(), out_c.data_ptr(), ops._ptr(gate), out.data_ptr(),
             tile_map.data_ptr(), S, H, B * H, L, L, D, be, topk, scale, dt, st)
        if need_grad:
            saved = [qt, kt, vt, out_s, lse, selected, sizes, qc, kc, vc, probs, out_c, tile_map, untile_map]
            if gate is not None:
                saved.append(gate)
            ctx.save_for_backward(*saved)
            ctx.has_gate = gate is not None
            ctx.be, ctx.scale, ctx.raster_shape = be, scale, (B, S, H, D)
        return out

    @staticmethod
    def backward(ctx, dout):
        saved = ctx.saved_tensors
        qt, kt, vt, out_s, lse, selected, sizes, qc, kc, vc, probs, out_c, tile_map, untile_map = saved[:14]
        gate = saved[14] if ctx.has_gate else None
        be, scale = ctx.be, ctx.scale
        B, S, H, D = ctx.raster_shape
        L = tile_map.numel()
        nb = L // be
        tk = selected.shape[-1]
        with torch.cuda.device(qt.device):
            dt = ops._check_device_dtype(qt, kt, vt)
            st = ops._stream(qt.device)
            # one pass: dout and the gate read at raster rows, dgate written there, dout stored in tile order for TMA
            dout = ops._dense(dout)
            dout_t = torch.empty_like(qt)
            d_out_c = torch.empty_like(out_c)
            dgate = torch.empty_like(gate) if gate is not None else None
            call("vsa_combine_bwd_raster", dout.data_ptr(), ops._ptr(gate), out_c.data_ptr(), d_out_c.data_ptr(),
                 ops._ptr(dgate), dout_t.data_ptr(), tile_map.data_ptr(), S, H, B * H, L, D, be, dt, st)
            ds_ws = torch.empty_like(probs)
            rowdot = torch.empty((B, H, nb), device=qt.device, dtype=torch.float32)
            dqc, dkc, dvc = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
            call("vsa_coarse_bwd", d_out_c.data_ptr(), out_c.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                 probs.data_ptr(), ds_ws.data_ptr(), rowdot.data_ptr(), dqc.data_ptr(), dkc.data_ptr(),
                 dvc.data_ptr(), B * H, nb, nb, D, scale, dt, st)
            del ds_ws
            inverse, offsets, counts = ops.invert_routes(selected, nb)
            delta = torch.empty_like(lse)
            dq, dk, dv = (torch.empty((B, S, H, D), device=qt.device, dtype=qt.dtype) for _ in range(3))
            call("vsa_sparse_bwd_dq_raster", dout_t.data_ptr(), qt.data_ptr(), kt.data_ptr(), vt.data_ptr(),
                 out_s.data_ptr(), lse.data_ptr(), selected.data_ptr(), sizes.data_ptr(), delta.data_ptr(),
                 dq.data_ptr(), dqc.data_ptr(), sizes.data_ptr(), tile_map.data_ptr(), S, H, B * H, L, L, D, be, tk,
                 scale, dt, st)
            call("vsa_sparse_bwd_dkdv_raster", dout_t.data_ptr(), qt.data_ptr(), kt.data_ptr(), vt.data_ptr(),
                 lse.data_ptr(), delta.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(),
                 sizes.data_ptr(), dk.data_ptr(), dv.data_ptr(), dkc.data_ptr(), dvc.data_ptr(), tile_map.data_ptr(),
                 S, H, B * H, L, L, D, be, tk, scale, dt, st)
        return dq, dk, dv, dgate, None, None, None, None, None, None, None


def video_sparse_attn_raster(q: Tensor, k: Tensor, v: Tensor, meta: Dict[str, object], topk: int,
                             compress_attn_weight: Optional[Tensor] = None) -> Tensor:
    """Video sparse self-attention of raster-order tokens.

    ``q, k, v`` (and the optional gate) are ``[batch, seq_len, heads, head_dim]`` with ``seq_len = T*H*W`` tokens in
    raster order; ``meta`` comes from ``build_vsa_metadata((T, H, W), tile_size, device)``.  Returns the attention
    output in the same layout.  Same numbers as ``untile(video_sparse_attn(tile(q).transpose(1, 2), ...))``: the same
    kernels do the same arithmetic, only the addresses of their stores differ.
    """
    if q.ndim != 4 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, and v must share the shape [batch, seq_len, heads, head_dim]")
    ops._check_device_dtype(q, k, v)
    be = int(meta["max_block_size"])
    tile_map, untile_map = meta["tile_map"], meta["untile_map"]
    B, S, H, D = q.shape
    if untile_map.numel() != S:
        raise ValueError(f"the metadata describes {untile_map.numel()} tokens, the tensors hold {S}")
    gate = compress_attn_weight
    if gate is not None and gate.shape != q.shape:
        raise ValueError("compress_attn_weight must have the same shape as q")
    nb = tile_map.numel() // be
    if not 1 <= topk <= nb:
        raise ValueError(f"topk must be in [1, {nb}]")
    with torch.cuda.device(q.device):
        tile_map = tile_map.to(device=q.device, dtype=torch.int32).contiguous()
        untile_map = untile_map.to(device=q.device, dtype=torch.int32).contiguous()
        sizes = ops._sizes(meta["variable_block_sizes"], q.device)
        if gate is not None and (gate.device != q.device or gate.dtype != q.dtype):
            gate = gate.to(device=q.device, dtype=q.dtype)
        if not raster_supported(q, be, int(topk)):
            # other shapes: the layout passes as separate kernels around the ordinary operator, same numbers
            from . import b200_vsa
            qt, kt, vt = (_tiled_with_grad(t, tile_map, untile_map) for t in (q, k, v))
            gt = _tiled_with_grad(gate, tile_map, untile_map) if gate is not None else None
            out_t = b200_vsa(qt, kt, vt, sizes, sizes, int(topk), (1, 1, be), gt)
            return _raster_with_grad(out_t, tile_map, untile_map)
        q, k, v = ops._dense(q), ops._dense(k), ops._dense(v)
        gate = ops._dense(gate) if gate is not None else None
        need_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, gate))
        return _RasterVideoSparseAttention.apply(q, k, v, gate, tile_map, untile_map, sizes, int(topk), be,
                                                 1.0 / math.sqrt(D), need_grad)


class _GatherHeads(torch.autograd.Function):
    """Differentiable ``_gather_heads``: no source row is read twice, so the gradient is the opposite gather."""

    @staticmethod
    def forward(ctx, x, row_map, back_map, to_tiled):
        ctx.save_for_backward(back_map)
        ctx.to_tiled = to_tiled
        return _gather_heads(x, row_map, row_map.numel(), to_tiled)

    @staticmethod
    def backward(ctx, grad):
        (back_map,) = ctx.saved_tensors
        return _gather_heads(grad, back_map, back_map.numel(), not ctx.to_tiled), None, None, None


def _tiled_with_grad(x: Tensor, tile_map: Tensor, untile_map: Tensor) -> Tensor:
    return _GatherHeads.apply(x, tile_map, untile_map, True)


def _raster_with_grad(x: Tensor, tile_map: Tensor, untile_map: Tensor) -> Tensor:
    return _GatherHeads.apply(x, untile_map, tile_map, False)


def tile_heads(x: Tensor, meta: Dict[str, object]) -> Tensor:
    """``[B,S,H,D]`` raster order -> ``[B,H,L,D]`` zero-padded tile order in one pass (differentiable)."""
    tile_map = meta["tile_map"].to(device=x.device, dtype=torch.int32).contiguous()
    untile_map = meta["untile_map"].to(device=x.device, dtype=torch.int32).contiguous()
    with torch.cuda.device(x.device):
        return _tiled_with_grad(x, tile_map, untile_map)


def untile_heads(x: Tensor, meta: Dict[str, object]) -> Tensor:
    """Inverse of :func:`tile_heads`."""
    tile_map = meta["tile_map"].to(device=x.device, dtype=torch.int32).contiguous()
    untile_map = meta["untile_map"].to(device=x.device, dtype=torch.int32).contiguous()
    with torch.cuda.device(x.device):
        return _raster_with_grad(x, tile_map, untile_map)
