"""Parity at the sizes the benchmark configurations name, on a few (batch, head) slices.

The kernels run the real shapes (92,160 tokens x topk 180 at block 64; 40,960 tokens x topk 20 at block 256
with ragged blocks; 16,384 tokens x topk 32 with a gate) and the CPU oracle recomputes SAMPLED blocks of them:

* output, saved statistic and dQ of a handful of query blocks (first, last, random) -- each depends on that
  block's own routes only, so the oracle runs on those rows against the full K/V;
* dK/dV of a handful of key blocks (the hottest and the coldest row of the inverse routing, plus random ones):
  the oracle runs every query block that routes to them (the same chunked gather as ``vsa/torch_impl.py:86-106``
  of the reference) and autograd sums their contributions;
* for the whole operator the pooled branch is cheap and is recomputed in full, so that the sampled gradients
  contain the pooled terms too; Top-K is compared as sets with exact-tie classification on the sampled rows.

Tolerances are the stated ones: forward 2e-2 abs/rel, gradients 3e-2.
"""

import math

import numpy as np
import pytest
import torch

from oracle import vsa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _V():
    import simple_vsa_b200 as V
    return V


@pytest.fixture(autouse=True)
def _no_device_timeouts():
    yield
    from simple_vsa_b200 import _lib
    assert _lib.device_status() == 0


_DT = torch.bfloat16      # element type of the generated tensors; one test switches it to fp16


def _randn(shape, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, device=DEV, generator=g) * scale).to(_DT)


def _rows(blocks, be):
    return torch.cat([torch.arange(b * be, (b + 1) * be) for b in blocks])


def _close(got, want, atol, rtol, what):
    got, want = got.float().cpu(), want.float().cpu()
    bad = (got - want).abs() > atol + rtol * want.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} elements off, max abs err " \
                          f"{float((got - want).abs().max()):.4f}"


def _zipf_routes(H, Qb, Kb, tk, seed):
    """Per query block, tk distinct key blocks from a Zipf(1.1) law over a random ranking (Gumbel top-k)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    perm = torch.randperm(Kb, device=DEV, generator=g)
    logw = -1.1 * torch.log(torch.arange(1, Kb + 1, device=DEV).float())
    out = torch.empty(1, H, Qb, tk, dtype=torch.int32, device=DEV)
    for h in range(H):
        u = torch.rand(Qb, Kb, device=DEV, generator=g).clamp_min(1e-12)
        out[0, h] = perm[(logw - torch.log(-torch.log(u))).topk(tk, dim=-1).indices].to(torch.int32)
    return out


def _pick_blocks(n, count, seed):
    g = torch.Generator().manual_seed(seed)
    picks = {0, n - 1}
    while len(picks) < min(count, n):
        picks.add(int(torch.randint(0, n, (1,), generator=g)))
    return sorted(picks)


def _key_block_sample(selected_cpu, Kb, head, extra, seed):
    """Hottest, coldest (but used) and `extra` random key blocks of one head, with the query blocks that use them."""
    counts = np.bincount(selected_cpu[0, head].reshape(-1).numpy(), minlength=Kb)
    used = np.nonzero(counts)[0]
    picks = {int(counts.argmax()), int(used[counts[used].argmin()])}
    g = np.random.default_rng(seed)
    while len(picks) < min(2 + extra, len(used)):
        picks.add(int(g.choice(used)))
    picks = sorted(picks)
    users = torch.isin(selected_cpu[0, head], torch.tensor(picks, dtype=selected_cpu.dtype)).any(-1).nonzero().flatten()
    return picks, users.tolist(), counts


def _check_fine_branch(q, k, v, dout, selected, kv_sizes, be, got_out, got_lse, got_dq, got_dk, got_dv, *,
                       q_blocks, key_head, key_extra, seed):
    """Sampled comparison of the fine branch.  All `got_*` are device tensors of the full shape."""
    B, H, Lq, D = q.shape
    Kb = k.shape[2] // be
    sel_cpu = selected.cpu()
    kc, vc = k.cpu(), v.cpu()
    # ---- output, statistic and dQ on sampled query blocks (all heads) ----
    rows = _rows(q_blocks, be)
    qs = q[:, :, rows.to(DEV)].cpu().float().requires_grad_()
    want, want_lse = O.sparse_attention(qs, kc, vc, sel_cpu[:, :, q_blocks], kv_sizes, be, q_blocks_per_chunk=16,
                                        return_lse2=True)
    want.backward(dout[:, :, rows.to(DEV)].cpu().float())
    _close(got_out[:, :, rows.to(DEV)], want.detach(), 2e-2, 2e-2, "fine output")
    if got_lse is not None:
        _close(got_lse[:, :, rows.to(DEV)], want_lse.detach(), 5e-2, 1e-3, "log-sum-exp")
    if got_dq is not None:
        _close(got_dq[:, :, rows.to(DEV)], qs.grad, 3e-2, 3e-2, "dQ")
    if got_dk is None:
        return
    # ---- dK/dV on sampled key blocks of one head: every query block that routes to them takes part ----
    picks, users, counts = _key_block_sample(sel_cpu[:, key_head:key_head + 1], Kb, 0, key_extra, seed)
    urows = _rows(users, be)
    kl = kc[:, key_head:key_head + 1].float().requires_grad_()
    vl = vc[:, key_head:key_head + 1].float().requires_grad_()
    qu = q[:, key_head:key_head + 1, urows.to(DEV)].cpu().float()
    wu = O.sparse_attention(qu, kl, vl, sel_cpu[:, key_head:key_head + 1, users], kv_sizes, be, q_blocks_per_chunk=16)
    wu.backward(dout[:, key_head:key_head + 1, urows.to(DEV)].cpu().float())
    krows = _rows(picks, be)
    for name, got, leaf in (("dK", got_dk, kl), ("dV", got_dv, vl)):
        w = leaf.grad[:, :, krows]
        # a key block with hundreds of in-edges sums that many 64-row products: tolerance relative to the sum's scale
        scale = max(1.0, float(w.abs().max()) / 8.0)
        _close(got[:, key_head:key_head + 1, krows.to(DEV)], w, 3e-2 * scale, 3e-2, f"{name} (in-degrees "
               f"{[int(counts[p]) for p in picks]})")


def _run_fine(q, k, v, dout, selected, kv_sizes, be):
    from simple_vsa_b200 import ops
    scale = 1.0 / math.sqrt(q.shape[-1])
    sizes_dev = kv_sizes.to(DEV, torch.int32)
    out, lse = ops.sparse_forward(q, k, v, selected, sizes_dev, be, scale, True)
    dq, dk, dv = ops.sparse_backward(dout, q, k, v, out, lse, selected, sizes_dev, be, scale)
    torch.cuda.synchronize()
    return out, lse, dq, dk, dv


def test_explicit_zipf_routes_92k_tokens_block64_topk180():
    """[1,2,92160,128], 1440 blocks of 64, topk 180, Zipf(1.1) routes: 90 tile pairs per query CTA, key rows with
    in-degree from a handful up to all 1440 query blocks."""
    B, H, L, D, be, tk = 1, 2, 92160, 128, 64, 180
    nb = L // be
    q, k, v, dout = (_randn((B, H, L, D), 100 + i) for i in range(4))
    selected = _zipf_routes(H, nb, nb, tk, 7)
    kv_sizes = torch.full((nb,), be)
    out, lse, dq, dk, dv = _run_fine(q, k, v, dout, selected, kv_sizes, be)
    assert torch.isfinite(out.float()).all() and torch.isfinite(dq.float()).all()
    assert torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()
    _check_fine_branch(q, k, v, dout, selected, kv_sizes, be, out, lse, dq, dk, dv,
                       q_blocks=_pick_blocks(nb, 6, 1), key_head=1, key_extra=1, seed=3)
    # CSR bookkeeping at 518,400 edges per slice
    V = _V()
    inverse, offsets, counts = V.invert_routes(selected, nb)
    assert int(counts.sum()) == H * nb * tk
    wc = torch.stack([torch.bincount(selected[0, h].reshape(-1).long(), minlength=nb) for h in range(H)])
    assert torch.equal(counts[0].long(), wc)
    assert torch.equal(offsets[0].long(), wc.cumsum(-1) - wc)


@pytest.mark.parametrize("be,tk,dtype", [(64, 180, torch.float16), (128, 90, torch.bfloat16)])
def test_explicit_zipf_routes_92k_tokens_fp16_and_128_token_blocks(be, tk, dtype, monkeypatch):
    """The same size through the other instantiations of the tensor path: fp16 inputs (90 pairs per query CTA with P
    kept inside fp16's range by the redo rule), and blocks of 128 tokens (two 64-token tiles per block, 720 blocks)."""
    import sys
    monkeypatch.setattr(sys.modules[__name__], "_DT", dtype)
    B, H, L, D = 1, 2, 92160, 128
    nb = L // be
    q, k, v, dout = (_randn((B, H, L, D), 500 + i) for i in range(4))
    selected = _zipf_routes(H, nb, nb, tk, 17)
    kv_sizes = torch.full((nb,), be)
    kv_sizes[3], kv_sizes[nb // 2] = be // 3, be - 1
    out, lse, dq, dk, dv = _run_fine(q, k, v, dout, selected, kv_sizes, be)
    assert out.dtype == dtype
    for t in (out, dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    _check_fine_branch(q, k, v, dout, selected, kv_sizes, be, out, lse, dq, dk, dv,
                       q_blocks=_pick_blocks(nb, 5, 2), key_head=0, key_extra=1, seed=4)


def test_whole_operator_92k_tokens_block64_topk180():
    """The headline shape on two slices: the operator's own Top-K routes, pooled branch recomputed in full by the
    oracle, fine branch and all gradients on sampled blocks."""
    V = _V()
    B, H, L, D, be, tk = 1, 2, 92160, 128, 64, 180
    _whole_operator_sampled(V, B, H, L, D, be, tk, block_size=(4, 4, 4), ragged_frac=0.0, with_gate=False, seed=200,
                            n_q_blocks=5, key_extra=1, oracle_heads=[0, 1])


def test_whole_operator_40k_tokens_block256_topk20_ragged():
    """[1,2,40960,128], 160 logical blocks of 256, topk 20; a tenth of the blocks hold 1..255 valid tokens and the
    padded positions are zero in q, k and v."""
    V = _V()
    _whole_operator_sampled(V, 1, 2, 40960, 128, 256, 20, block_size=(4, 8, 8), ragged_frac=0.1, with_gate=False,
                            seed=300, n_q_blocks=6, key_extra=2, oracle_heads=[0, 1])


def test_whole_operator_16k_tokens_12_heads_topk32_gate():
    """[1,12,16384,128] block 64 topk 32 with a sigmoid gate at full size on the GPU; the oracle follows two heads."""
    V = _V()
    _whole_operator_sampled(V, 1, 12, 16384, 128, 64, 32, block_size=(4, 4, 4), ragged_frac=0.0, with_gate=True,
                            seed=400, n_q_blocks=8, key_extra=2, oracle_heads=[3, 11])


def _whole_operator_sampled(V, B, H, L, D, be, tk, *, block_size, ragged_frac, with_gate, seed, n_q_blocks,
                            key_extra, oracle_heads):
    nb = L // be
    q, k, v, dout = (_randn((B, H, L, D), seed + i) for i in range(4))
    gate = torch.sigmoid(_randn((B, H, L, D), seed + 9).float()).to(torch.bfloat16) if with_gate else None
    sizes = torch.full((nb,), be)
    if ragged_frac > 0:
        g = torch.Generator().manual_seed(seed)
        ragged = torch.randperm(nb, generator=g)[:max(1, int(ragged_frac * nb))]
        sizes[ragged] = torch.randint(1, be, (ragged.numel(),), generator=g)
        pad = (torch.arange(be)[None, :] >= sizes[:, None]).reshape(L).to(DEV)
        for t in (q, k, v):
            t[:, :, pad] = 0
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    gl = gate.clone().requires_grad_() if with_gate else None
    out, aux = V.video_sparse_attn(*leaves, sizes, sizes, tk, block_size, gl, return_aux=True)
    out.backward(dout)
    torch.cuda.synchronize()
    selected = aux["selected"]
    assert torch.isfinite(out.float()).all()
    for t in leaves:
        assert torch.isfinite(t.grad.float()).all()

    hs = oracle_heads
    qc_, kc_, vc_, dc_ = (t[:, hs].cpu() for t in (q, k, v, dout))
    gc_ = gate[:, hs].cpu() if with_gate else None
    sel = selected[:, hs].cpu()
    scale = 1.0 / math.sqrt(D)
    # ---- Top-K against the oracle's pooled scores (bf16 roundings as the reference makes them) ----
    with torch.no_grad():
        w_scores, w_out_c = O.coarse_compact(qc_, kc_, vc_, sizes, sizes, be, scale)
    got_scores = aux["coarse_scores"][:, hs].cpu()
    ulp = 2.0 ** -7
    assert float((got_scores.float() - w_scores.float()).abs().max()) <= 2 * ulp * float(w_scores.float().abs().max())
    differ, unexplained = O.topk_mismatch_report(w_scores, sel, tk)
    # a pooled score that lands one bf16 unit away from the CPU's (fp32 sums in another order) may swap a block at
    # the k-th place; such rows must stay rare, and the kernel's choice must be exact on ITS OWN scores
    assert unexplained <= 0.03 * len(hs) * nb, (differ, unexplained)
    d2, u2 = O.topk_mismatch_report(got_scores, sel, tk)
    assert u2 == 0, f"{u2} rows are not a Top-K of the kernel's own scores"

    # ---- sampled oracle with the pooled branch in full ----
    q_blocks = _pick_blocks(nb, n_q_blocks, seed)
    picks, users, counts = _key_block_sample(sel, nb, 0, key_extra, seed)      # key blocks of the first oracle head
    for h_local in range(len(hs)):
        follow = sorted(set(q_blocks) | (set(users) if h_local == 0 else set()))
        rows = _rows(follow, be)
        ql = qc_[:, h_local:h_local + 1].clone().requires_grad_()
        kl = kc_[:, h_local:h_local + 1].clone().requires_grad_()
        vl = vc_[:, h_local:h_local + 1].clone().requires_grad_()
        gl_o = gc_[:, h_local:h_local + 1].clone().requires_grad_() if with_gate else None
        d_h = dc_[:, h_local:h_local + 1]
        _, out_c = O.coarse_compact(ql, kl, vl, sizes, sizes, be, scale)
        out_s = O.sparse_attention(ql[:, :, rows], kl, vl, sel[:, h_local:h_local + 1, follow], sizes, be, scale,
                                   q_blocks_per_chunk=16)
        want = O.combine(out_s, out_c[:, :, follow], gl_o[:, :, rows] if with_gate else None, be, torch.bfloat16)
        # the rest of the query blocks reach k and v through the pooled branch only
        d_out_c = d_h.float() * (gc_[:, h_local:h_local + 1].float() if with_gate else 1.0)
        d_out_c = d_out_c.reshape(1, 1, nb, be, D).sum(3)
        d_out_c[:, :, follow] = 0
        loss = (want.float() * d_h[:, :, rows].float()).sum() + (out_c.float() * d_out_c).sum()
        loss.backward()
        h = hs[h_local]
        qrows = _rows(q_blocks, be)
        sub = torch.isin(rows, qrows)
        _close(out[:, h:h + 1, qrows.to(DEV)], want.detach()[:, :, sub], 2e-2, 2e-2, f"output (head {h})")
        _close(leaves[0].grad[:, h:h + 1, qrows.to(DEV)], ql.grad[:, :, qrows], 3e-2, 3e-2, f"dQ (head {h})")
        if with_gate:
            _close(gl.grad[:, h:h + 1, qrows.to(DEV)], gl_o.grad[:, :, qrows], 3e-2, 3e-2, f"dgate (head {h})")
        if h_local == 0:
            krows = _rows(picks, be)
            for name, leaf, oleaf in (("dK", leaves[1], kl), ("dV", leaves[2], vl)):
                w = oleaf.grad[:, :, krows]
                s = max(1.0, float(w.float().abs().max()) / 8.0)
                _close(leaf.grad[:, h:h + 1, krows.to(DEV)], w, 3e-2 * s, 3e-2,
                       f"{name} (head {h}, in-degrees {[int(counts[p]) for p in picks]})")


def test_shard_major_layout_at_92k_tokens_eight_shards():
    """The long-sequence layout of the sequence-parallel mode at its real proportions: 92,160 key tokens in eight
    rank-major shards of 11,520, one rank's 11,520 queries, topk 180 -- against the ordinary layout on the same
    numbers (itself checked against the oracle above).  Output and dQ must be bit-identical (same routes, same tiles,
    same order); dK/dV agree up to the order of the fp32 sums."""
    V = _V()
    from simple_vsa_b200 import ops
    B, H, L, D, be, tk, W = 1, 2, 92160, 128, 64, 180, 8
    l, nb = L // W, L // be
    k, v = (_randn((B, H, L, D), 500 + i) for i in range(2))
    sizes = torch.full((nb,), be)
    rank = 5
    q = _randn((B, H, l, D), 510)
    dout = _randn((B, H, l, D), 511)
    q_sizes = sizes[rank * (nb // W):(rank + 1) * (nb // W)]
    a = [t.clone().requires_grad_() for t in (q, k, v)]
    out_a = V.b200_vsa(a[0], a[1], a[2], sizes, q_sizes, tk, (4, 4, 4))
    out_a.backward(dout)
    k_sh = k.view(B, H, W, l, D).permute(2, 0, 1, 3, 4).contiguous().requires_grad_()
    v_sh = v.view(B, H, W, l, D).permute(2, 0, 1, 3, 4).contiguous().requires_grad_()
    kc, vc = V.block_mean(k, sizes, be), V.block_mean(v, sizes, be)
    qb_ = q.clone().requires_grad_()
    out_b = ops.vsa_on_gathered_shards(qb_, k_sh, v_sh, kc, vc, sizes, q_sizes, tk, (4, 4, 4))
    out_b.backward(dout)
    torch.cuda.synchronize()
    assert torch.isfinite(out_b.float()).all()
    assert torch.equal(out_b, out_a) and torch.equal(qb_.grad, a[0].grad)
    for got_sh, want in ((k_sh.grad, a[1].grad), (v_sh.grad, a[2].grad)):
        got = got_sh.permute(1, 2, 0, 3, 4).reshape(B, H, L, D)
        _close(got, want, 2e-2, 2e-2, "shard-major dK/dV")
