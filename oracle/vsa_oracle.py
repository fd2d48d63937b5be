"""CPU oracle for the Video Sparse Attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the arithmetic of the
reference project's readable implementation so that the CUDA kernels can be
checked against it on identical seeded inputs.  It is imported only by the
test-suite, by the smoke check and by the CPU-baseline leg of the benchmark;
the product package never imports it and has no CPU fallback.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference
package itself (``vsa.torch_vsa``, ``vsa.video_sparse_attn``,
``vsa.common.block_mean`` ...) in the build container, runs it on seeded
inputs and stores inputs' seeds plus outputs under ``tests/golden``;
``tests/test_oracle_golden.py`` checks every function here against those
stored vectors.

Reference lines followed (paths inside the reference project):
  * block volume from ``block_size``            vsa/common.py:39-42
  * valid-token mask                             vsa/common.py:45-52
  * padding-aware block mean                     vsa/common.py:55-82
  * coarse scores / softmax / pooled output      vsa/common.py:137-167
  * Top-K routing                                vsa/torch_impl.py:85
  * gathered fine attention                      vsa/torch_impl.py:33-46,86-106
  * gated combine                                vsa/torch_impl.py:108-113
  * argument checks                              vsa/common.py:97-134
  * KV->query inverse routing (CSR)              vsa/triton_impl.py:544-595
  * base-2 log-sum-exp convention                vsa/triton_impl.py:113-115,189-192
"""

from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch
from torch import Tensor

LOG2E = 1.4426950408889634


def block_elements(block_size: Union[int, Sequence[int]]) -> int:
    """An int block size is a cube edge; a tuple is multiplied out."""
    if isinstance(block_size, int):
        return block_size ** 3
    return int(math.prod(block_size))


def valid_mask(sizes: Tensor, be: int) -> Tensor:
    """[nb, be] bool, True on the first ``sizes[b]`` slots of block ``b``."""
    return torch.arange(be, device=sizes.device)[None, :] < sizes[:, None]


def check_inputs(q, k, v, kv_sizes, q_sizes, topk: int, be: int) -> None:
    """Same conditions and message fragments as the reference validator."""
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, and v must have shape [batch, heads, seq_len, dim]")
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    if (k.shape[0], k.shape[1]) != (B, H) or (v.shape[0], v.shape[1]) != (B, H):
        raise ValueError("q, k, and v must share batch and head dimensions")
    if v.shape[2] != Lkv:
        raise ValueError("k and v must have the same sequence length")
    if k.shape[3] != D or v.shape[3] != D:
        raise ValueError("q, k, and v must have the same head dimension")
    if Lq % be or Lkv % be:
        raise ValueError(f"q/kv sequence lengths must be divisible by block_elements={be}")
    if kv_sizes.numel() != Lkv // be:
        raise ValueError(
            f"variable_block_sizes must have length {Lkv // be}, got {kv_sizes.numel()}")
    if q_sizes.numel() != Lq // be:
        raise ValueError(
            f"q_variable_block_sizes must have length {Lq // be}, got {q_sizes.numel()}")
    if not 1 <= topk <= Lkv // be:
        raise ValueError(f"topk must be in [1, {Lkv // be}]")


def block_mean(x: Tensor, sizes: Tensor, be: int) -> Tensor:
    """fp32 sum of the valid tokens of each block / max(size, 1), in x's dtype."""
    B, H, L, D = x.shape
    nb = L // be
    xb = x.reshape(B, H, nb, be, D).float()
    keep = valid_mask(sizes, be).view(1, 1, nb, be, 1)
    total = (xb * keep).sum(dim=3)
    denom = sizes.clamp(min=1).to(total.dtype).view(1, 1, nb, 1)
    return (total / denom).to(x.dtype)


def coarse_compact(q, k, v, kv_sizes, q_sizes, be: int, scale: float) -> Tuple[Tensor, Tensor]:
    """Pooled scores [B,H,Qb,Kb] and pooled output [B,H,Qb,D], both in the input dtype.

    Every intermediate keeps the input dtype (bf16 stays bf16): the product is
    rounded, then scaled and rounded again, and the softmax output is rounded
    before it multiplies the pooled values.
    """
    qc = block_mean(q, q_sizes, be)
    kc = block_mean(k, kv_sizes, be)
    vc = block_mean(v, kv_sizes, be)
    scores = torch.matmul(qc, kc.transpose(-2, -1)) * scale
    probs = torch.softmax(scores, dim=-1)
    return scores, torch.matmul(probs, vc)


def select_topk(scores: Tensor, topk: int) -> Tensor:
    """Indices of the ``topk`` largest pooled scores per query block (no gradient)."""
    return scores.topk(topk, dim=-1).indices


def sparse_attention(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    selected: Tensor,
    kv_sizes: Tensor,
    be: int,
    scale: Optional[float] = None,
    *,
    q_blocks_per_chunk: Optional[int] = None,
    return_lse2: bool = False,
):
    """Fine attention of every query block over the valid tokens of its selected key blocks.

    fp32 math throughout; the result is fp32 [B,H,Lq,D].  Query sizes play no
    part here: padded query rows are computed like any other row.  The work is
    cut into chunks of query blocks so that the gathered K/V stay small; the
    chunks are independent in the forward pass and autograd sums their K/V
    gradients.  ``return_lse2`` also returns row_max + log2(row_sum) of the
    scores multiplied by scale*log2(e), the convention of the saved statistic.
    """
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    Qb, Kb = Lq // be, Lkv // be
    tk = selected.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    selected = selected.long()
    kb = k.reshape(B, H, Kb, be, D)
    vb = v.reshape(B, H, Kb, be, D)
    keep = valid_mask(kv_sizes.to(q.device), be)                      # [Kb, be]
    step = q_blocks_per_chunk or Qb
    outs, lses = [], []
    bi = torch.arange(B)[:, None, None, None]
    hi = torch.arange(H)[None, :, None, None]
    for start in range(0, Qb, step):
        stop = min(Qb, start + step)
        ids = selected[:, :, start:stop]                              # [B,H,c,tk]
        kg = kb[bi, hi, ids].float()                                  # [B,H,c,tk,be,D]
        vg = vb[bi, hi, ids].float()
        ok = keep[ids]                                                # [B,H,c,tk,be]
        qq = q[:, :, start * be:stop * be].reshape(B, H, stop - start, be, D).float()
        s = torch.einsum("bhctd,bhcksd->bhctks", qq, kg) * scale      # [B,H,c,be,tk,be]
        s = s.masked_fill(~ok[:, :, :, None], float("-inf")).flatten(-2)
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("bhctn,bhcnd->bhctd", p, vg.flatten(3, 4))
        outs.append(o.reshape(B, H, (stop - start) * be, D))
        if return_lse2:
            lses.append((torch.logsumexp(s, dim=-1) * LOG2E).reshape(B, H, -1))
    out = torch.cat(outs, dim=2)
    if return_lse2:
        return out, torch.cat(lses, dim=2)
    return out


def combine(out_s: Tensor, out_c_blocks: Tensor, gate: Optional[Tensor], be: int, dtype) -> Tensor:
    """out = sparse + pooled[block] * gate in fp32, one rounding at the end."""
    B, H, L, D = out_s.shape
    spread = out_c_blocks.float().repeat_interleave(be, dim=2)
    if gate is not None:
        spread = spread * gate.float()
    return (spread + out_s.float()).to(dtype)


def vsa(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    kv_sizes: Tensor,
    q_sizes: Tensor,
    topk: int,
    block_size: Union[int, Sequence[int]] = 64,
    gate: Optional[Tensor] = None,
    *,
    selected: Optional[Tensor] = None,
    q_blocks_per_chunk: Optional[int] = None,
    return_aux: bool = False,
):
    """Whole operator: pooled branch + Top-K routed fine branch + gated sum.

    ``selected`` overrides the Top-K choice (used to compare the fine branch on
    identical routes when pooled scores tie).  Differentiable with autograd.
    """
    be = block_elements(block_size)
    check_inputs(q, k, v, kv_sizes, q_sizes, topk, be)
    scale = 1.0 / math.sqrt(q.shape[-1])
    kv_sizes = kv_sizes.to(q.device)
    q_sizes = q_sizes.to(q.device)
    scores, out_c_blocks = coarse_compact(q, k, v, kv_sizes, q_sizes, be, scale)
    if selected is None:
        selected = select_topk(scores, topk)
    out_s = sparse_attention(q, k, v, selected, kv_sizes, be, scale,
                             q_blocks_per_chunk=q_blocks_per_chunk)
    out = combine(out_s, out_c_blocks, gate, be, q.dtype)
    if return_aux:
        return out, {"scores": scores, "selected": selected,
                     "out_c_blocks": out_c_blocks, "out_s": out_s}
    return out


def invert_routes(selected: Tensor, key_blocks: int):
    """CSR of key block -> query blocks that selected it, per (batch, head).

    Returns numpy int32 ``counts [B,H,Kb]``, exclusive ``offsets [B,H,Kb]`` and
    ``inverse [B,H,Qb*tk]`` with the query ids of each key row in ascending
    order (the GPU builder may emit any order inside a row).
    """
    sel = selected.cpu().numpy().astype(np.int64)
    B, H, Qb, tk = sel.shape
    counts = np.zeros((B, H, key_blocks), np.int32)
    offsets = np.zeros((B, H, key_blocks), np.int32)
    inverse = np.zeros((B, H, Qb * tk), np.int32)
    qid = np.repeat(np.arange(Qb, dtype=np.int32), tk)
    for b in range(B):
        for h in range(H):
            flat = sel[b, h].reshape(-1)
            counts[b, h] = np.bincount(flat, minlength=key_blocks)
            offsets[b, h] = np.cumsum(counts[b, h]) - counts[b, h]
            order = np.argsort(flat, kind="stable")
            inverse[b, h] = qid[order]
    return counts, offsets, inverse


def topk_mismatch_report(scores: Tensor, selected: Tensor, topk: int):
    """Compare a routing table against the oracle's pooled scores as sets.

    For each row, ids chosen by ``selected`` but not by the oracle's Top-K (and
    vice versa) are acceptable only when their oracle scores equal the row's
    k-th largest score (an exact tie).  Returns (rows_differing, rows_not_explained).
    """
    s = scores.float()
    ref = s.topk(topk, dim=-1)
    kth = ref.values[..., -1:]
    ref_mask = torch.zeros_like(s, dtype=torch.bool).scatter_(-1, ref.indices, True)
    got_mask = torch.zeros_like(s, dtype=torch.bool).scatter_(-1, selected.long().cpu(), True)
    differ = ref_mask != got_mask
    unexplained = differ & (s != kth)
    return int(differ.any(-1).sum()), int(unexplained.any(-1).sum())
