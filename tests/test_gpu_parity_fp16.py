"""fp16 on the tensor path: the tcgen05 kernels exist once per 16-bit element type (other input format in the
instruction descriptor and the tensor maps, other conversions in the epilogues).  The cases below repeat, in
fp16, the checks that pin the bf16 kernels: the CPU oracle, the three kernel families against one another,
the exact recomputation of out-of-range tiles (fp16 overflows at 2^16, so it is reached much earlier than in
bf16), the stored-dS backward, the shard-major layout, the two forward schedules and the pooled GEMMs.
Tolerances are those stated for 16-bit inputs: 2e-2 for outputs, 3e-2 for gradients."""

import math

import pytest
import torch

from oracle import vsa_oracle as O
from tests.test_gpu_parity import _assert_close, _zipf_routes

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F16 = torch.float16


def _V():
    import simple_vsa_b200 as V
    return V


@pytest.fixture(autouse=True)
def _no_device_timeouts():
    yield
    from simple_vsa_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("be,nb,tk,ragged", [(64, 24, 6, False), (64, 24, 7, True), (256, 8, 3, True), (128, 12, 5, True)])
def test_fp16_fine_attention_matches_oracle_on_every_kernel_family(be, nb, tk, ragged, monkeypatch):
    V = _V()
    torch.manual_seed(141)
    B, H, D = 1, 3, 128
    L = be * nb
    q, k, v, dout = (torch.randn(B, H, L, D).to(F16) for _ in range(4))
    sizes = torch.full((nb,), be)
    if ragged:
        sizes[1], sizes[nb // 2], sizes[-1] = 1, be // 2 + 3, be - 1
    selected = _zipf_routes(B, H, nb, nb, tk, 7)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    want = O.sparse_attention(*ol, selected, sizes, be, q_blocks_per_chunk=8)
    want.backward(dout.float())
    for mode in ("auto", "mma", "scalar"):
        monkeypatch.setenv("VSA_B200_KERNELS", mode)
        leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
        out = V.b200_sparse_attention(*leaves, selected.to(DEV), sizes, block_size=(1, 1, be))
        out.backward(dout.to(DEV))
        assert out.dtype == F16 and all(x.grad.dtype == F16 for x in leaves)
        _assert_close(out, want, atol=2e-2, rtol=2e-2)
        for leaf, oleaf in zip(leaves, ol):
            _assert_close(leaf.grad, oleaf.grad, atol=3e-2, rtol=3e-2)
        if ragged and mode == "auto":      # padded key rows receive exactly zero gradient
            assert leaves[1].grad[0, :, be + 1:2 * be].abs().max() == 0


def test_fp16_whole_operator_with_gate_matches_oracle():
    """Pooled branch (tcgen05 GEMMs in fp16), Top-K, fine branch, fused gated combine, and the whole backward."""
    V = _V()
    torch.manual_seed(147)
    B, H, L, D, be, tk = 1, 2, 2048, 128, 64, 4
    q, k, v, dout = (torch.randn(B, H, L, D).to(F16) for _ in range(4))
    gate = torch.sigmoid(torch.randn(B, H, L, D)).to(F16)
    sizes = torch.full((L // be,), be)
    sizes[3], sizes[-1] = 17, 40
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    g = gate.to(DEV).requires_grad_()
    out, aux = V.video_sparse_attn(*leaves, sizes, sizes, tk, (4, 4, 4), g, return_aux=True)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    og = gate.clone().requires_grad_()
    _, waux = O.vsa(*ol, sizes, sizes, tk, (4, 4, 4), og, return_aux=True)
    differ, unexplained = O.topk_mismatch_report(waux["scores"], aux["selected"], tk)
    assert unexplained <= 0.02 * B * H * (L // be), (differ, unexplained)
    want = O.vsa(*ol, sizes, sizes, tk, (4, 4, 4), og, selected=aux["selected"].cpu(), q_blocks_per_chunk=8)
    want.backward(dout)
    out.backward(dout.to(DEV))
    assert out.dtype == F16
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    for leaf, oleaf in zip(leaves + [g], ol + [og]):
        _assert_close(leaf.grad, oleaf.grad, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("factor", [3.5, 6.0, 40.0])
def test_fp16_forward_out_of_range_tiles_are_recomputed_exactly(factor):
    """A later key block scores far above the first pair.  Factor 3.5 gives a gap of ~18 binades: above 2^16, inside
    the 20 binades the fp16 forward leaves above the first pair's maximum (its softmax shift is biased by four
    binades).  With factor 6 the gap (~30-40 binades) fits bf16 and fp32 but not fp16; with factor 40 it overflows
    everything.  Whatever the tile's route through the kernels, it must match the oracle, log-sum-exp included."""
    torch.manual_seed(161)
    be, nb, D = 64, 8, 128
    q, k, v = (torch.randn(1, 1, be * nb, D).to(F16) for _ in range(3))
    k[:, :, 5 * be:6 * be] *= factor
    sizes = torch.full((nb,), be)
    selected = torch.tensor([[0, 1, 5, 2], [3, 4, 6, 7], [1, 0, 2, 5], [5, 1, 2, 3]] * 2, dtype=torch.int32)[None, None]
    want, want_lse = O.sparse_attention(q, k, v, selected, sizes, be, return_lse2=True)
    from simple_vsa_b200 import ops
    out, lse = ops.sparse_forward(q.to(DEV), k.to(DEV), v.to(DEV), selected.to(DEV), sizes.to(DEV, torch.int32),
                                  be, 1.0 / math.sqrt(D), True)
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    _assert_close(lse, want_lse, atol=5e-2, rtol=1e-3)


def test_fp16_rows_of_very_different_scale_in_one_query_tile():
    torch.manual_seed(162)
    be, nb, D, tk = 64, 8, 128, 4
    q, k, v = (torch.randn(1, 2, be * nb, D).to(F16) for _ in range(3))
    q[:, :, 3::be] *= 30.0
    sizes = torch.full((nb,), be)
    selected = torch.stack([torch.randperm(nb)[:tk] for _ in range(2 * nb)]).to(torch.int32).view(1, 2, nb, tk)
    want, want_lse = O.sparse_attention(q, k, v, selected, sizes, be, return_lse2=True)
    from simple_vsa_b200 import ops
    out, lse = ops.sparse_forward(q.to(DEV), k.to(DEV), v.to(DEV), selected.to(DEV), sizes.to(DEV, torch.int32),
                                  be, 1.0 / math.sqrt(D), True)
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    _assert_close(lse, want_lse, atol=5e-2, rtol=1e-3)


@pytest.mark.parametrize("be,nb,tk", [(64, 24, 6), (256, 8, 3)])
def test_fp16_backward_that_stores_ds_equals_the_recomputing_backward(be, nb, tk, monkeypatch):
    from simple_vsa_b200 import ops
    torch.manual_seed(193)
    B, H, D = 1, 3, 128
    L = be * nb
    q, k, v, dout = (torch.randn(B, H, L, D, device=DEV).to(F16) for _ in range(4))
    kv_sizes = torch.full((nb,), be, dtype=torch.int32, device=DEV)
    q_sizes = kv_sizes.clone()
    kv_sizes[1], kv_sizes[nb // 2], kv_sizes[-1] = 1, be // 2 + 3, 0
    q_sizes[2] = be - 5
    selected = _zipf_routes(B, H, nb, nb, tk, 19).to(DEV)
    scale = 1.0 / math.sqrt(D)
    out_s, lse = ops.sparse_forward(q, k, v, selected, kv_sizes, be, scale, True)
    pooled = tuple(torch.randn(B, H, nb, D, device=DEV).to(F16) for _ in range(3)) + (q_sizes,)
    for pg in (None, pooled):
        monkeypatch.delenv("VSA_B200_BACKWARD", raising=False)
        want = ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale, pooled_grads=pg)
        monkeypatch.setenv("VSA_B200_BACKWARD", "stored_ds")
        got = ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale, pooled_grads=pg)
        for name, g, w in zip(("dq", "dk", "dv"), got, want):
            assert g.dtype == F16 and torch.isfinite(g.float()).all(), name
            _assert_close(g, w, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("be,nb,tk,W", [(64, 16, 5, 2), (256, 8, 3, 2)])
def test_fp16_shard_major_kv_layout_equals_the_ordinary_layout(be, nb, tk, W):
    V = _V()
    from simple_vsa_b200 import ops
    torch.manual_seed(199)
    B, H, D = 1, 3, 128
    L = be * nb
    l = L // W
    q_all, k, v = (torch.randn(B, H, L, D, device=DEV).to(F16) for _ in range(3))
    k[:, :, 5 * 64:6 * 64] *= 8.0
    sizes = torch.full((nb,), be)
    sizes[1], sizes[nb - 2] = be // 2 + 3, 7
    rank = W - 1
    q = q_all[:, :, rank * l:(rank + 1) * l].contiguous()
    gate = torch.randn(B, H, l, D, device=DEV).to(F16)
    dout = torch.randn(B, H, l, D, device=DEV).to(F16)
    q_sizes = sizes[rank * (nb // W):(rank + 1) * (nb // W)]
    a = [t.clone().requires_grad_() for t in (q, k, v, gate)]
    out_a = V.b200_vsa(a[0], a[1], a[2], sizes, q_sizes, tk, (1, 1, be), a[3])
    out_a.backward(dout)
    k_sh = k.view(B, H, W, l, D).permute(2, 0, 1, 3, 4).contiguous().requires_grad_()
    v_sh = v.view(B, H, W, l, D).permute(2, 0, 1, 3, 4).contiguous().requires_grad_()
    kc, vc = V.block_mean(k, sizes, be), V.block_mean(v, sizes, be)
    b = [q.clone().requires_grad_(), gate.clone().requires_grad_()]
    out_b = ops.vsa_on_gathered_shards(b[0], k_sh, v_sh, kc, vc, sizes, q_sizes, tk, (1, 1, be), b[1])
    out_b.backward(dout)
    assert torch.isfinite(out_b.float()).all()
    assert torch.equal(out_b, out_a)
    assert torch.equal(b[0].grad, a[0].grad) and torch.equal(b[1].grad, a[3].grad)
    for got_sh, want in ((k_sh.grad, a[1].grad), (v_sh.grad, a[2].grad)):
        _assert_close(got_sh.permute(1, 2, 0, 3, 4).reshape(B, H, L, D), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("be,nb,tk", [(64, 40, 7), (256, 6, 3)])
def test_fp16_two_schedules_of_the_forward_give_the_same_bits(be, nb, tk, monkeypatch):
    from simple_vsa_b200 import ops
    torch.manual_seed(211)
    B, H, D = 1, 5, 128
    L = be * nb
    q, k, v = (torch.randn(B, H, L, D, device=DEV).to(F16) for _ in range(3))
    sizes = torch.full((nb,), be, dtype=torch.int32, device=DEV)
    sizes[2], sizes[-1] = 9, be - 1
    selected = _zipf_routes(B, H, nb, nb, tk, 23).to(DEV)
    res = {}
    for sched in ("classic", "persistent"):
        monkeypatch.setenv("VSA_B200_FWD", sched)
        res[sched] = ops.sparse_forward(q, k, v, selected, sizes, be, 1.0 / math.sqrt(D), True)
    assert torch.equal(res["classic"][0], res["persistent"][0])
    assert torch.equal(res["classic"][1], res["persistent"][1])


@pytest.mark.parametrize("Qb,Kb", [(200, 136), (8, 8)])
def test_fp16_pooled_attention_tensor_core_path_matches_scalar_path(Qb, Kb, monkeypatch):
    from simple_vsa_b200 import _lib
    torch.manual_seed(155)
    BH, D = 3, 128
    scale = D ** -0.5
    qc, kc, vc, dco = (torch.randn(n, device=DEV).to(F16) for n in
                       ((BH, Qb, D), (BH, Kb, D), (BH, Kb, D), (BH, Qb, D)))
    st = torch.cuda.current_stream().cuda_stream

    def run():
        scores = torch.empty(BH, Qb, Kb, device=DEV, dtype=F16)
        probs, ds = torch.empty_like(scores), torch.empty_like(scores)
        out_c = torch.empty(BH, Qb, D, device=DEV, dtype=F16)
        _lib.call("vsa_coarse_fwd", qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), scores.data_ptr(), probs.data_ptr(),
                  out_c.data_ptr(), BH, Qb, Kb, D, scale, _lib.VSA_F16, st)
        rowdot = torch.empty(BH, Qb, device=DEV)
        dq, dk, dv = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
        _lib.call("vsa_coarse_bwd", dco.data_ptr(), out_c.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                  probs.data_ptr(), ds.data_ptr(), rowdot.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                  BH, Qb, Kb, D, scale, _lib.VSA_F16, st)
        torch.cuda.synchronize()
        return scores, probs, out_c, dq, dk, dv

    fast = run()
    monkeypatch.setenv("VSA_B200_KERNELS", "scalar")
    slow = run()
    # scores: identical roundings, fp32 sums in a different order -> at most one fp16 unit apart
    assert (fast[0].float() - slow[0].float()).abs().max() <= 2 ** -10 * slow[0].float().abs().max()
    for a, b in zip(fast[1:], slow[1:]):
        torch.testing.assert_close(a.float(), b.float(), atol=2e-2, rtol=2e-2)
    ql, kl, vl = (t.float().requires_grad_() for t in (qc, kc, vc))
    ref = torch.softmax(torch.matmul(ql, kl.transpose(-2, -1)) * scale, -1) @ vl
    ref.backward(dco.float())
    torch.testing.assert_close(fast[2].float(), ref, atol=2e-2, rtol=2e-2)
    for got, leaf in zip(fast[3:], (ql, kl, vl)):
        torch.testing.assert_close(got.float(), leaf.grad, atol=3e-2, rtol=3e-2)


def test_fp16_is_closer_to_the_oracle_than_bf16_on_the_same_numbers():
    """A sanity check that the fp16 kernels really compute in fp16 (11-bit significands) and not through a bf16
    round trip: on inputs representable in both types the fp16 result has the smaller error."""
    V = _V()
    torch.manual_seed(171)
    be, nb, tk, D = 64, 16, 4, 128
    base = [torch.randn(1, 2, be * nb, D).to(torch.bfloat16) for _ in range(3)]      # exact in fp16 as well
    sizes = torch.full((nb,), be)
    selected = _zipf_routes(1, 2, nb, nb, tk, 5)
    want = O.sparse_attention(*[t.float() for t in base], selected, sizes, be)
    err = {}
    for dt in (torch.bfloat16, F16):
        out = V.b200_sparse_attention(*[t.to(dt).to(DEV) for t in base], selected.to(DEV), sizes, block_size=(1, 1, be))
        err[dt] = float((out.float().cpu() - want).abs().max())
    assert err[F16] < 0.5 * err[torch.bfloat16], err
