"""3-D tiling front end: raster (t, h, w) token order <-> zero-padded, tile-contiguous order.

Same names, arguments and returned keys as the reference's ``vsa/fastvideo_tiling.py``
(``build_vsa_metadata`` :92-125, ``tile`` :128-140, ``untile`` :143-145), so a DiT layer written
against it keeps working.  The index tensors are built with closed-form arithmetic (no Python loop
over tiles); on CUDA tensors the moves themselves run in one gather kernel of the library
(``vsa_gather_rows``), which also writes the zero padding, instead of an index-put into a zeroed
buffer plus two advanced-indexing gathers.  The moves are differentiable (the backward is the same
kernel with the opposite map); tensors that are not on a GPU take the reference's index expressions.
"""

from __future__ import annotations

import functools
import math
from typing import Dict, Tuple

import torch
from torch import Tensor

VSA_TILE_SIZE = (4, 4, 4)


def _axis(n: int, t: int, device):
    """Per position of one axis: its tile, its offset inside the tile, the (clipped) extent of that tile."""
    pos = torch.arange(n, device=device)
    tile = pos // t
    extent = torch.clamp(n - tile * t, max=t)
    return tile, pos - tile * t, extent


@functools.lru_cache(maxsize=32)
def _maps(shape: Tuple[int, int, int], tile_size: Tuple[int, int, int], device: torch.device):
    T, H, W = shape
    ts, hs, ws = tile_size
    nt, nh, nw = math.ceil(T / ts), math.ceil(H / hs), math.ceil(W / ws)
    be = ts * hs * ws
    tt, to, te = _axis(T, ts, device)
    ht, ho, he = _axis(H, hs, device)
    wt, wo, we = _axis(W, ws, device)
    # padded slot of every raster token: tile id * volume + row-major offset inside the CLIPPED tile
    block = (tt[:, None, None] * nh + ht[None, :, None]) * nw + wt[None, None, :]
    inside = (to[:, None, None] * he[None, :, None] + ho[None, :, None]) * we[None, None, :] + wo[None, None, :]
    slot_of_raster = (block * be + inside).reshape(-1)                     # [T*H*W] -> padded slot
    non_pad_index, order = torch.sort(slot_of_raster)                       # real slots ascending; raster id per slot
    reverse = torch.empty_like(order)
    reverse[order] = torch.arange(order.numel(), device=device)
    sizes = (torch.clamp(T - torch.arange(nt, device=device) * ts, max=ts)[:, None, None]
             * torch.clamp(H - torch.arange(nh, device=device) * hs, max=hs)[None, :, None]
             * torch.clamp(W - torch.arange(nw, device=device) * ws, max=ws)[None, None, :]).reshape(-1)
    tile_map = torch.full((nt * nh * nw * be,), -1, dtype=torch.int32, device=device)
    tile_map[non_pad_index] = order.to(torch.int32)                         # padded slot -> raster id or -1
    return order, reverse, sizes, non_pad_index, (nt, nh, nw), be, tile_map, slot_of_raster.to(torch.int32)


def build_vsa_metadata(dit_seq_shape: Tuple[int, int, int], tile_size: Tuple[int, int, int] = VSA_TILE_SIZE,
                       device="cpu") -> Dict[str, object]:
    """Every tiling tensor for a ``(T, H, W)`` latent grid; the reference's keys plus the two int32 row
    maps (``tile_map``: padded slot -> raster id or -1, ``untile_map``: raster id -> padded slot)."""
    order, reverse, sizes, npi, num_tiles, be, tile_map, untile_map = _maps(
        tuple(dit_seq_shape), tuple(tile_size), torch.device(device))
    return {"tile_partition_indices": order, "reverse_tile_partition_indices": reverse,
            "variable_block_sizes": sizes, "non_pad_index": npi, "num_tiles": num_tiles, "max_block_size": be,
            "tile_map": tile_map, "untile_map": untile_map}


def _gather_cuda(x: Tensor, row_map: Tensor, dst_rows: int) -> Tensor:
    from . import _lib
    x = x.contiguous()
    batch, src_rows = x.shape[0], x.shape[1]
    row_bytes = (x.numel() // max(1, batch * src_rows)) * x.element_size()
    out = torch.empty((batch, dst_rows) + tuple(x.shape[2:]), device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        _lib.call("vsa_gather_rows", x.data_ptr(), row_map.data_ptr(), out.data_ptr(), batch, src_rows, dst_rows,
                  row_bytes, torch.cuda.current_stream(x.device).cuda_stream)
    return out


class _GatherRows(torch.autograd.Function):
    """``out[:, r] = x[:, row_map[r]]`` (zero where ``row_map[r] < 0``).  No source row is read twice, so the
    gradient is the same kernel with the opposite map: the gradient of tiling is an un-tiling, and the gradient of
    un-tiling is a tiling that zero-fills the padding rows."""

    @staticmethod
    def forward(ctx, x, row_map, back_map):
        ctx.save_for_backward(back_map)
        return _gather_cuda(x, row_map, row_map.numel())

    @staticmethod
    def backward(ctx, grad):
        (back_map,) = ctx.saved_tensors
        return _gather_cuda(grad, back_map, back_map.numel()), None, None


def _inverse_map(row_map: Tensor, src_rows: int) -> Tensor:
    inv = torch.full((src_rows,), -1, dtype=torch.int32, device=row_map.device)
    live = (row_map >= 0).nonzero().flatten()
    inv[row_map[live].long()] = live.to(torch.int32)
    return inv


def _gather(x: Tensor, row_map: Tensor, back_map: Tensor = None) -> Tensor:
    """Row gather along dim 1 with zero fill.  CUDA tensors go through ``vsa_gather_rows`` (differentiable);
    tensors elsewhere use the reference's index expressions (``vsa/fastvideo_tiling.py:128-145``), so metadata
    and layout code can be exercised without a GPU."""
    row_map = row_map.to(device=x.device, dtype=torch.int32).contiguous()
    if not x.is_cuda:
        live = row_map >= 0
        out = x.new_zeros((x.shape[0], row_map.numel()) + tuple(x.shape[2:]))
        out[:, live] = x[:, row_map[live].long()]
        return out
    if back_map is None:
        back_map = _inverse_map(row_map, x.shape[1])
    back_map = back_map.to(device=x.device, dtype=torch.int32).contiguous()
    if torch.is_grad_enabled() and x.requires_grad:
        return _GatherRows.apply(x, row_map, back_map)
    return _gather_cuda(x, row_map, row_map.numel())


def tile(x: Tensor, tile_partition_indices: Tensor, non_pad_index: Tensor, num_blocks: int,
         max_block_size: int) -> Tensor:
    """``[batch, seq_len, ...]`` raster order -> ``[batch, num_blocks*max_block_size, ...]`` tile order, zero padded."""
    rows = num_blocks * max_block_size
    row_map = torch.full((rows,), -1, dtype=torch.int32, device=x.device)
    row_map[non_pad_index.to(x.device)] = tile_partition_indices.to(device=x.device, dtype=torch.int32)
    return _gather(x, row_map)


def untile(x: Tensor, non_pad_index: Tensor, reverse_tile_partition_indices: Tensor) -> Tensor:
    """Inverse of :func:`tile`."""
    row_map = non_pad_index.to(x.device)[reverse_tile_partition_indices.to(x.device)]
    return _gather(x, row_map)


def tile_with(meta: Dict[str, object], x: Tensor) -> Tensor:
    """:func:`tile` with the cached row maps of ``build_vsa_metadata`` (no index arithmetic per call)."""
    return _gather(x, meta["tile_map"], meta["untile_map"])


def untile_with(meta: Dict[str, object], x: Tensor) -> Tensor:
    """:func:`untile` with the cached row maps of ``build_vsa_metadata``."""
    return _gather(x, meta["untile_map"], meta["tile_map"])
