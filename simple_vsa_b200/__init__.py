"""B200-native Video Sparse Attention behind the reference project's operator API.

Drop-in names (same positional order as ``vsa/__init__.py`` of the reference):

* ``video_sparse_attn(q, k, v, variable_block_sizes, q_variable_block_sizes, topk,
  block_size, compress_attn_weight)`` and its aliases ``b200_vsa``, ``triton_vsa``,
  ``helion_vsa`` -- the whole operator, differentiable in q, k, v and the gate;
* ``b200_sparse_attention(q, k, v, selected, variable_block_sizes, *, block_size,
  sm_scale=None)`` and its aliases ``triton_sparse_attention``,
  ``helion_sparse_attention`` -- the fine branch on caller-supplied routes;
* ``block_mean``, ``topk_block_mask``, ``CompressionGate``.

Everything runs in hand-written CUDA kernels for sm_100a loaded from
``libvsa_b200.so``; importing this package without that library raises.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor, nn

from . import _lib  # noqa: F401  (fails loudly when the CUDA library is absent)
from .tiling import build_vsa_metadata, tile, tile_with, untile, untile_with
from .raster import tile_heads, untile_heads, video_sparse_attn_raster
from .ops import (
    BlockSize,
    as_block_elements,
    block_mean,
    invert_routes,
    sparse_attention,
    validate_vsa_inputs,
    vsa_forward_full,
)

__all__ = [
    "video_sparse_attn", "b200_vsa", "triton_vsa", "helion_vsa",
    "b200_sparse_attention", "triton_sparse_attention", "helion_sparse_attention",
    "block_mean", "topk_block_mask", "CompressionGate", "invert_routes",
    "as_block_elements", "validate_vsa_inputs",
    "build_vsa_metadata", "tile", "untile", "tile_with", "untile_with",
    "video_sparse_attn_raster", "tile_heads", "untile_heads",
]


def video_sparse_attn(q: Tensor, k: Tensor, v: Tensor, variable_block_sizes: Tensor,
                      q_variable_block_sizes: Tensor, topk: int, block_size: BlockSize = 64,
                      compress_attn_weight: Optional[Tensor] = None, *, sm_scale: Optional[float] = None,
                      return_aux: bool = False):
    """Video Sparse Attention over ``[batch, heads, seq_len, dim]`` CUDA tensors.

    ``out = pooled_attention(block means)[block] * compress_attn_weight + fine_attention``
    where the fine branch of each query block attends to the valid tokens of its
    ``topk`` best key blocks under the pooled scores.  ``block_size`` is a tile shape
    whose product is the block volume (an int is cubed).  With ``return_aux`` the
    dict holds ``coarse_scores``, ``block_mask``, ``selected``, ``out_compress``
    (per query block) and ``out_sparse``.
    """
    out, scores, selected, out_c, out_s = vsa_forward_full(
        q, k, v, variable_block_sizes, q_variable_block_sizes, topk, block_size, compress_attn_weight, sm_scale)
    if not return_aux:
        return out
    mask = torch.zeros_like(scores, dtype=torch.bool).scatter_(-1, selected.long(), True)
    be = as_block_elements(block_size)
    return out, {"coarse_scores": scores, "block_mask": mask, "selected": selected,
                 "out_compress": out_c.repeat_interleave(be, dim=2), "out_compress_blocks": out_c,
                 "out_sparse": out_s}


def b200_vsa(q, k, v, variable_block_sizes, q_variable_block_sizes, topk, block_size: BlockSize = 64,
             compress_attn_weight: Optional[Tensor] = None) -> Tensor:
    """Eight-argument form shared by every backend of the reference (``vsa/triton_impl.py:1734-1743``)."""
    return vsa_forward_full(q, k, v, variable_block_sizes, q_variable_block_sizes, topk, block_size,
                            compress_attn_weight)[0]


triton_vsa = b200_vsa
helion_vsa = b200_vsa


def b200_sparse_attention(q, k, v, selected, variable_block_sizes, *, block_size: BlockSize,
                          sm_scale: Optional[float] = None) -> Tensor:
    """Fine attention on an externally supplied routing table (``vsa/triton_impl.py:1626-1652``)."""
    return sparse_attention(q, k, v, selected, variable_block_sizes, block_size=block_size, sm_scale=sm_scale)


triton_sparse_attention = b200_sparse_attention
helion_sparse_attention = b200_sparse_attention


def topk_block_mask(scores: Tensor, topk: int) -> Tensor:
    """Boolean ``[..., Kb]`` mask with exactly ``topk`` True per row, chosen by the Top-K kernel."""
    if not scores.is_cuda:
        raise ValueError("the B200 implementation requires CUDA tensors")
    kb = scores.shape[-1]
    topk = min(int(topk), kb)
    flat = scores.contiguous()
    if flat.dtype not in (torch.bfloat16, torch.float32, torch.float16):
        flat = flat.float()
    rows = flat.numel() // kb
    sel = torch.empty((rows, topk), device=scores.device, dtype=torch.int32)
    with torch.cuda.device(scores.device):
        _lib.call("vsa_topk", flat.data_ptr(), sel.data_ptr(), rows, kb, topk,
                  {torch.bfloat16: _lib.VSA_BF16, torch.float32: _lib.VSA_F32, torch.float16: _lib.VSA_F16}[flat.dtype],
                  torch.cuda.current_stream(scores.device).cuda_stream)
    mask = torch.zeros((rows, kb), device=scores.device, dtype=torch.bool).scatter_(-1, sel.long(), True)
    return mask.view(scores.shape)


class _HeadMajorLinear(torch.autograd.Function):
    """``y[b, h, s, :] = x[b, s, :] @ W[h*D:(h+1)*D, :]^T + bias[h*D:(h+1)*D]`` written straight into a dense
    ``[B, H, S, D]`` tensor: one library GEMM per batch entry, batched over the heads (the hidden states are the
    shared left operand, broadcast with a zero batch stride; every head's slice of the weight is a right operand).
    The reference's layer (``vsa/common.py:317-328``) returns ``Linear(x).view(B,S,H,D).transpose(1,2)``, a strided
    view that the attention operator has to copy into the dense layout its kernels read; here the GEMM's own
    store does the re-layout.  The backward brings the gate gradient back to ``[B, S, H*D]`` once (the copy
    autograd makes on the reference path too) and runs the two usual GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, bias, heads):
        B, S, dim_in = x.shape
        dim_out = weight.shape[0]
        D = dim_out // heads
        wt = weight.view(heads, D, dim_in).transpose(1, 2)                 # [H, dim_in, D], a view
        out = torch.empty((B, heads, S, D), device=x.device, dtype=x.dtype)
        for b in range(B):
            xb = x[b].unsqueeze(0).expand(heads, S, dim_in)
            if bias is None:
                torch.bmm(xb, wt, out=out[b])
            else:
                torch.baddbmm(bias.view(heads, 1, D), xb, wt, out=out[b])
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return out

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        B, S, dim_in = x.shape
        dyt = dy.transpose(1, 2).reshape(B * S, weight.shape[0])            # [B*S, H*D]: the one re-layout copy
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = (dyt @ weight).view(B, S, dim_in)
        if ctx.needs_input_grad[1]:
            dw = dyt.t() @ x.reshape(B * S, dim_in)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dyt.sum(0)
        return dx, dw, db, None


class CompressionGate(nn.Module):
    """Produces ``compress_attn_weight``: a bias-optional ``Linear(dim, dim)`` on the hidden states (no
    activation), returned as ``[batch, heads, seq_len, head_dim]`` -- same parameters (``to_gate_compress``), same
    numbers and same ``ValueError`` as the reference's layer (``vsa/common.py:288-328``).  The result is DENSE in
    that layout: the GEMM writes every head's ``[seq_len, head_dim]`` panel where the attention kernels read it,
    so no transposing copy sits between this layer and the operator."""

    def __init__(self, dim: int, num_heads: int, bias: bool = True) -> None:
        super().__init__()
        if dim % num_heads:
            raise ValueError(f"dim={dim} must be divisible by num_heads={num_heads}")
        self.num_heads = num_heads
        self.to_gate_compress = nn.Linear(dim, dim, bias=bias)

    def forward(self, hidden_states: Tensor) -> Tensor:
        if hidden_states.ndim != 3:
            raise ValueError("hidden_states must have shape [batch, seq_len, dim]")
        layer = self.to_gate_compress
        return _HeadMajorLinear.apply(hidden_states, layer.weight, layer.bias, self.num_heads)
