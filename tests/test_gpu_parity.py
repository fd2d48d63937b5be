"""Parity of the CUDA kernels (called through the C ABI via the package) with the CPU oracle
and with the golden vectors the reference produced.  Everything here needs a B200."""

import math
import os

import numpy as np
import pytest
import torch

from oracle import vsa_oracle as O
from tests.golden.cases import SPARSE_CASES, VSA_CASES, sparse_inputs, to_np, vsa_inputs

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


def _V():
    import simple_vsa_b200 as V
    return V


def _load(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def _fwd_tol(dtype):
    # stated tolerances of the task: 2e-2 abs/rel in bf16, 1e-5 in the fp32 validation mode
    return dict(atol=2e-2, rtol=2e-2) if dtype != "f32" else dict(atol=1e-5, rtol=1e-5)


def _grad_tol(dtype):
    # dQ/dK/dV within 3e-2 in bf16; fp32 validation mode at 1e-4 relative of the gradient scale
    return dict(atol=3e-2, rtol=3e-2) if dtype != "f32" else dict(atol=2e-5, rtol=1e-4)


def _assert_close(got, want, **tol):
    np.testing.assert_allclose(to_np(got), want if isinstance(want, np.ndarray) else to_np(want), **tol)


@pytest.fixture(autouse=True)
def _no_device_timeouts():
    """Every test must leave the device status word clear (no bounded wait ran out)."""
    yield
    from simple_vsa_b200 import _lib
    assert _lib.device_status() == 0


# ---------------------------------------------------------------------------------------------
# tcgen05 building blocks
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode", [0, 1])
def test_umma_building_blocks(mode):
    """TMA boxes + shared-memory operand descriptors + tensor-memory read-out give A*B."""
    from simple_vsa_b200 import _lib
    torch.manual_seed(60 + mode)
    a = torch.randn(128, 128, device=DEV).to(torch.bfloat16)
    if mode == 0:
        b = torch.randn(64, 128, device=DEV).to(torch.bfloat16)
        want = a.float() @ b.float().t()
    else:
        b = torch.randn(128, 64, device=DEV).to(torch.bfloat16)
        want = a.float().t() @ b.float()
    out = torch.full((128, 64), float("nan"), device=DEV)
    _lib.call("vsa_selftest_umma", a.data_ptr(), b.data_ptr(), out.data_ptr(), mode,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    torch.testing.assert_close(out, want, atol=1e-3, rtol=1e-3)


def test_forward_fixed_shift_out_of_range_is_recomputed_exactly():
    """Later key blocks score ~200 (log2 units) above the first pair: the tcgen05 forward must hand those
    tiles to the exact kernel, and the result must still match the oracle."""
    V = _V()
    torch.manual_seed(61)
    be, nb, D = 64, 8, 128
    q, k, v = (torch.randn(1, 1, be * nb, D).to(torch.bfloat16) for _ in range(3))
    k[:, :, 5 * be:6 * be] *= 40.0          # block 5 dominates whenever it is selected
    sizes = torch.full((nb,), be)
    selected = torch.tensor([[0, 1, 5, 2], [3, 4, 6, 7], [1, 0, 2, 5], [5, 1, 2, 3]] * 2, dtype=torch.int32)[None, None]
    want, want_lse = O.sparse_attention(q, k, v, selected, sizes, be, return_lse2=True)
    from simple_vsa_b200 import ops
    out, lse = ops.sparse_forward(q.to(DEV), k.to(DEV), v.to(DEV), selected.to(DEV), sizes.to(DEV, torch.int32),
                                  be, 1.0 / math.sqrt(D), True)
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    _assert_close(lse, want_lse, atol=5e-2, rtol=1e-3)


@pytest.mark.parametrize("factor", [30.0, 300.0])
def test_forward_rows_of_very_different_scale_in_one_query_tile(factor):
    """One row of every 64-row query tile has scores `factor` times larger than its neighbours (~100 and
    ~1000 binades): the softmax shift of the tcgen05 forward must be per row, or the small rows lose their
    precision (or their sum) to the large one.  Every row matches the oracle."""
    torch.manual_seed(62)
    be, nb, D, tk = 64, 8, 128, 4
    q, k, v = (torch.randn(1, 2, be * nb, D).to(torch.bfloat16) for _ in range(3))
    q[:, :, 3::be] *= factor                 # row 3 of every query tile
    sizes = torch.full((nb,), be)
    selected = torch.stack([torch.randperm(nb)[:tk] for _ in range(2 * nb)]).to(torch.int32).view(1, 2, nb, tk)
    want, want_lse = O.sparse_attention(q, k, v, selected, sizes, be, return_lse2=True)
    from simple_vsa_b200 import ops
    out, lse = ops.sparse_forward(q.to(DEV), k.to(DEV), v.to(DEV), selected.to(DEV), sizes.to(DEV, torch.int32),
                                  be, 1.0 / math.sqrt(D), True)
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    _assert_close(lse, want_lse, atol=5e-2, rtol=1e-3)


# ---------------------------------------------------------------------------------------------
# bandwidth kernels
# ---------------------------------------------------------------------------------------------
def test_block_mean_known_answer_forward_backward():
    V = _V()
    gold = _load("block_mean_64_37_11")
    torch.manual_seed(11)
    x = torch.randn(1, 2, 3 * 64, 128).to(torch.bfloat16)
    sizes = torch.tensor([64, 37, 11])
    grad = torch.randn(1, 2, 3, 128).to(torch.bfloat16)
    leaf = x.to(DEV).requires_grad_()
    out = V.block_mean(leaf, sizes, 64)
    out.backward(grad.to(DEV))
    _assert_close(out, gold["out"], atol=2e-2, rtol=2e-2)
    # same fp32 sum and one rounding: expect at most one bf16 ulp of difference
    assert np.abs(to_np(out) - gold["out"]).max() <= 2 ** -7 * np.abs(gold["out"]).max()
    _assert_close(leaf.grad, gold["dx"], atol=2e-2, rtol=2e-2)
    # padding values never reach the mean
    y = x.clone()
    y[:, :, 64 + 37:128] = float("nan")
    _assert_close(V.block_mean(y.to(DEV), sizes, 64), to_np(out), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("with_gate", [False, True])
def test_combine_forward_backward(dtype, with_gate):
    from simple_vsa_b200 import _lib
    torch.manual_seed(13)
    be, nb, D = 64, 3, 128
    sparse = torch.randn(1, 2, be * nb, D).to(dtype)
    coarse = torch.randn(1, 2, nb, D).to(dtype)
    gate = torch.randn(1, 2, be * nb, D).to(dtype) if with_gate else None
    dout = torch.randn(1, 2, be * nb, D).to(dtype)
    want = O.combine(sparse, coarse, gate, be, dtype)
    spread = coarse.float().repeat_interleave(be, dim=2)
    want_dgate = (dout.float() * spread).to(dtype) if with_gate else None
    want_dc = ((dout.float() * (gate.float() if with_gate else 1.0)).reshape(1, 2, nb, be, D).sum(3)).to(dtype)
    dt = _lib.VSA_BF16 if dtype == torch.bfloat16 else _lib.VSA_F32
    s, c, d = sparse.to(DEV), coarse.to(DEV), dout.to(DEV)
    g = gate.to(DEV) if with_gate else None
    out = torch.empty_like(s)
    st = torch.cuda.current_stream().cuda_stream
    _lib.call("vsa_combine_fwd", s.data_ptr(), c.data_ptr(), g.data_ptr() if g is not None else None, out.data_ptr(),
              2, be * nb, D, be, dt, st)
    dc = torch.empty_like(c)
    dg = torch.empty_like(s) if with_gate else None
    _lib.call("vsa_combine_bwd", d.data_ptr(), g.data_ptr() if g is not None else None, c.data_ptr(), dc.data_ptr(),
              dg.data_ptr() if dg is not None else None, 2, be * nb, D, be, dt, st)
    tol = dict(atol=2e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)
    _assert_close(out, want, **tol)
    _assert_close(dc, want_dc, atol=6e-2 if dtype == torch.bfloat16 else 1e-4, rtol=3e-2)
    if with_gate:
        _assert_close(dg, want_dgate, **tol)


def test_route_inversion_matches_cpu_sets():
    V = _V()
    torch.manual_seed(17)
    key_blocks = 13
    selected = torch.randn(2, 3, 7, key_blocks).topk(5, dim=-1).indices.to(torch.int32)
    inverse, offsets, counts = V.invert_routes(selected.to(DEV), key_blocks)
    assert inverse.shape == (2, 3, 35)
    want_counts, want_offsets, want_inverse = O.invert_routes(selected, key_blocks)
    np.testing.assert_array_equal(counts.cpu().numpy(), want_counts)
    np.testing.assert_array_equal(offsets.cpu().numpy(), want_offsets)
    inv = inverse.cpu().numpy()
    for b in range(2):
        for h in range(3):
            for kb in range(key_blocks):
                lo, n = want_offsets[b, h, kb], want_counts[b, h, kb]
                assert sorted(inv[b, h, lo:lo + n].tolist()) == want_inverse[b, h, lo:lo + n].tolist()


def test_route_inversion_large_and_skewed():
    V = _V()
    g = torch.Generator().manual_seed(5)
    Qb, Kb, tk = 300, 700, 40
    w = torch.arange(1, Kb + 1).float().pow(-1.1)
    selected = torch.stack([torch.multinomial(w, tk, generator=g) for _ in range(Qb)]).to(torch.int32)[None, None]
    selected = selected.expand(1, 3, Qb, tk).contiguous()
    inverse, offsets, counts = V.invert_routes(selected.to(DEV), Kb)
    wc, wo, wi = O.invert_routes(selected, Kb)
    np.testing.assert_array_equal(counts.cpu().numpy(), wc)
    np.testing.assert_array_equal(offsets.cpu().numpy(), wo)
    inv = inverse.cpu().numpy()
    for kb in (0, 1, 5, 100, Kb - 1):
        lo, n = wo[0, 2, kb], wc[0, 2, kb]
        assert sorted(inv[0, 2, lo:lo + n].tolist()) == wi[0, 2, lo:lo + n].tolist()
    assert int(counts.sum()) == 3 * Qb * tk


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_topk_kernel_with_ties(dtype):
    V = _V()
    torch.manual_seed(3)
    rows, n, k = 64, 1440, 180
    scores = (torch.randn(rows, n) * 0.016).to(dtype)      # bf16 at this scale ties heavily
    mask = V.topk_block_mask(scores.to(DEV), k).cpu()
    assert mask.sum(-1).eq(k).all()
    s = scores.float()
    kth = s.topk(k, dim=-1).values[:, -1:]
    assert (s[mask].reshape(rows, k) >= kth).all()          # nothing below the k-th value is chosen
    assert ((s > kth) <= mask).all()                        # everything above it is chosen
    # ties go to the lowest ids
    for r in range(rows):
        tied = (s[r] == kth[r]).nonzero().flatten()
        taken = mask[r][tied]
        n_taken = int(taken.sum())
        assert taken[:n_taken].all() and not taken[n_taken:].any()


@pytest.mark.parametrize("n,k", [(1440, 180), (256, 32), (40, 1), (8, 8)])
def test_topk_routes_start_with_the_best_block(n, k):
    """Order of a route: the best-scoring block (lowest id among equals), then the rest by ascending id.  The fine
    forward takes its softmax shift from the first pair of tiles it meets, so the best block leads."""
    from simple_vsa_b200 import _lib
    torch.manual_seed(4)
    rows = 37
    scores = (torch.randn(rows, n) * 0.05).to(torch.bfloat16).to(DEV)
    scores[5, :] = 0.25                                      # a row of equal scores
    sel = torch.empty(rows, k, dtype=torch.int32, device=DEV)
    _lib.call("vsa_topk", scores.data_ptr(), sel.data_ptr(), rows, n, k, _lib.VSA_BF16,
              torch.cuda.current_stream().cuda_stream)
    sel = sel.cpu().long()
    s = scores.float().cpu()
    for r in range(rows):
        assert len(set(sel[r].tolist())) == k
        assert int(sel[r, 0]) == int((s[r] == float(s[r].max())).nonzero()[0])
        tail = sel[r, 1:]
        assert torch.equal(tail, tail.sort().values)


# ---------------------------------------------------------------------------------------------
# route-explicit fine attention against the reference's vectors
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(SPARSE_CASES))
@pytest.mark.parametrize("kernels", ["auto", "mma", "scalar"])
def test_route_explicit_against_reference_vectors(name, kernels, monkeypatch):
    V = _V()
    monkeypatch.setenv("VSA_B200_KERNELS", kernels)
    case = SPARSE_CASES[name]
    gold = _load("sparse_" + name)
    q, k, v, dout, sizes, selected = sparse_inputs(case)
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    out = V.b200_sparse_attention(*leaves, selected.to(DEV), sizes, block_size=(1, 1, case["be"]))
    _assert_close(out, gold["out_s"], **_fwd_tol(case["dtype"]))
    out.backward(dout.to(DEV))
    for tag, leaf in zip(("dq", "dk", "dv"), leaves):
        _assert_close(leaf.grad, gold[tag], **_grad_tol(case["dtype"]))
    # the saved statistic is row_max + log2(row_sum) of scores * scale * log2(e)
    from simple_vsa_b200 import ops
    _, lse = ops.sparse_forward(leaves[0].detach(), leaves[1].detach(), leaves[2].detach(),
                                selected.to(DEV), sizes.to(DEV, torch.int32), case["be"],
                                1.0 / math.sqrt(q.shape[-1]), True)
    _assert_close(lse, gold["lse2"], atol=2e-2 if case["dtype"] != "f32" else 1e-4, rtol=1e-3)
    # no gradient path: forward-only call gives the same numbers
    with torch.no_grad():
        again = V.triton_sparse_attention(*[t.detach() for t in leaves], selected.to(DEV), sizes,
                                          block_size=(1, 1, case["be"]))
    assert torch.equal(again, out.detach())


# ---------------------------------------------------------------------------------------------
# the whole operator against the reference's vectors
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(VSA_CASES))
def test_whole_operator_against_reference_vectors(name):
    V = _V()
    case = VSA_CASES[name]
    gold = _load("vsa_" + name)
    q, k, v, gate, dout, sizes = vsa_inputs(case)
    leaves = [t.to(DEV).requires_grad_(case["grad"]) for t in (q, k, v)]
    g = gate.to(DEV).requires_grad_(case["grad"]) if gate is not None else None
    out, aux = V.video_sparse_attn(*leaves, sizes, sizes, case["topk"], case["block_size"], g, return_aux=True)
    # pooled scores: same roundings as the reference; allow one unit in the last place
    ulp = {"bf16": 2 ** -7, "f16": 2 ** -10, "f32": 2 ** -20}[case["dtype"]]
    sc = to_np(aux["coarse_scores"])
    assert np.abs(sc - gold["scores"]).max() <= ulp * max(1e-6, np.abs(gold["scores"]).max())
    # routing: identical sets, except where the reference's own scores tie at the k-th place
    differ, unexplained = O.topk_mismatch_report(torch.from_numpy(gold["scores"]), aux["selected"], case["topk"])
    assert unexplained == 0, f"{unexplained} rows pick a block the reference scores exclude"
    same_routes = differ == 0
    _assert_close(aux["out_compress_blocks"], gold["out_c_blocks"], **_fwd_tol(case["dtype"]))
    # the reference's own key holds the same values repeated on the tokens of each query block
    assert aux["out_compress"].shape == out.shape
    assert torch.equal(aux["out_compress"][:, :, ::O.block_elements(case["block_size"])], aux["out_compress_blocks"])
    if same_routes:
        _assert_close(out, gold["out"], **_fwd_tol(case["dtype"]))
    # against the oracle on the routes the kernel chose (removes tie ambiguity)
    ol = [t.clone().requires_grad_(case["grad"]) for t in (q, k, v)]
    og = gate.clone().requires_grad_(case["grad"]) if gate is not None else None
    want = O.vsa(*ol, sizes, sizes, case["topk"], case["block_size"], og, selected=aux["selected"].cpu())
    _assert_close(out, want, **_fwd_tol(case["dtype"]))
    if case["grad"]:
        out.backward(dout.to(DEV))
        want.backward(dout)
        stride = int(gold["grad_row_stride"])
        for tag, leaf, oleaf in zip(("dq", "dk", "dv"), leaves, ol):
            _assert_close(leaf.grad, oleaf.grad, **_grad_tol(case["dtype"]))
            if same_routes:
                np.testing.assert_allclose(to_np(leaf.grad)[:, :, ::stride], gold[tag], **_grad_tol(case["dtype"]))
        if g is not None:
            _assert_close(g.grad, og.grad, **_grad_tol(case["dtype"]))
            if same_routes:
                np.testing.assert_allclose(to_np(g.grad)[:, :, ::stride], gold["dgate"], **_grad_tol(case["dtype"]))


def test_whole_operator_unselected_blocks_get_gradient_from_pooled_branch():
    V = _V()
    torch.manual_seed(9)
    be, nb = 64, 6
    q, k, v = (torch.randn(1, 1, be * nb, 128, device=DEV, dtype=torch.bfloat16).requires_grad_() for _ in range(3))
    sizes = torch.full((nb,), be)
    out, aux = V.video_sparse_attn(q, k, v, sizes, sizes, 1, (4, 4, 4), return_aux=True)
    out.float().square().mean().backward()
    chosen = set(aux["selected"].flatten().tolist())
    skipped = [b for b in range(nb) if b not in chosen]
    assert skipped, "every block was selected; pick another seed"
    for b in skipped:
        assert k.grad[0, 0, b * be:(b + 1) * be].abs().sum() > 0
        assert v.grad[0, 0, b * be:(b + 1) * be].abs().sum() > 0


# ---------------------------------------------------------------------------------------------
# mid-size cases: tensor-core kernels vs oracle, and vs the scalar kernels
# ---------------------------------------------------------------------------------------------
def _zipf_routes(B, H, Qb, Kb, tk, seed):
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(Kb, generator=g)
    logw = -1.1 * torch.log(torch.arange(1, Kb + 1).float())
    gumbel = -torch.log(-torch.log(torch.rand(B, H, Qb, Kb, generator=g).clamp_min(1e-12)))
    return perm[(logw + gumbel).topk(tk, dim=-1).indices].to(torch.int32)


@pytest.mark.parametrize("be,nb,tk,ragged", [(64, 24, 6, False), (64, 24, 6, True), (256, 8, 3, True), (128, 12, 5, True)])
def test_fine_attention_midsize_matches_oracle(be, nb, tk, ragged, monkeypatch):
    V = _V()
    torch.manual_seed(41)
    B, H, D = 1, 3, 128
    L = be * nb
    q, k, v, dout = (torch.randn(B, H, L, D).to(torch.bfloat16) for _ in range(4))
    sizes = torch.full((nb,), be)
    if ragged:
        sizes[1], sizes[nb // 2], sizes[-1] = 1, be // 2 + 3, be - 1
    selected = _zipf_routes(B, H, nb, nb, tk, 7)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    want = O.sparse_attention(*ol, selected, sizes, be, q_blocks_per_chunk=8)
    want.backward(dout.float())
    results = {}
    for mode in ("auto", "mma", "scalar"):
        monkeypatch.setenv("VSA_B200_KERNELS", mode)
        leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
        out = V.b200_sparse_attention(*leaves, selected.to(DEV), sizes, block_size=(1, 1, be))
        out.backward(dout.to(DEV))
        _assert_close(out, want, atol=2e-2, rtol=2e-2)
        for leaf, oleaf in zip(leaves, ol):
            _assert_close(leaf.grad, oleaf.grad, atol=3e-2, rtol=3e-2)
        results[mode] = (out, [x.grad for x in leaves])
    # padded key rows receive exactly zero gradient
    if ragged:
        dk = results["auto"][1][1]
        assert dk[0, :, be + 1:2 * be].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("be,nb,tk", [(64, 20, 6), (128, 10, 4), (256, 6, 3)])
def test_head_dim_64_runs_on_the_warp_level_tensor_kernels(be, nb, tk, dtype, monkeypatch):
    """Head dim 64 (bf16 / fp16, blocks of 64, 128, 256): the mma.sync kernels instantiated for 64-wide tiles, against
    the oracle and against the CUDA-core kernels, ragged blocks included; the whole operator (pooled branch on the
    CUDA-core GEMMs at this head dim) with a gate as well."""
    from simple_vsa_b200 import _lib
    V = _V()
    torch.manual_seed(81)
    B, H, D = 1, 3, 64
    L = be * nb
    dt_code = _lib.VSA_BF16 if dtype == torch.bfloat16 else _lib.VSA_F16
    assert _lib.lib.vsa_sparse_kernel_family(D, be, tk, dt_code) == 1
    assert _lib.lib.vsa_sparse_kernel_family(128, be, tk, dt_code) == 2
    assert _lib.lib.vsa_sparse_kernel_family(D, be, tk, _lib.VSA_F32) == 0
    q, k, v, dout = (torch.randn(B, H, L, D).to(dtype) for _ in range(4))
    sizes = torch.full((nb,), be)
    sizes[1], sizes[nb // 2], sizes[-1] = 1, be // 2 + 3, be - 1
    selected = _zipf_routes(B, H, nb, nb, tk, 9)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    want = O.sparse_attention(*ol, selected, sizes, be, q_blocks_per_chunk=8)
    want.backward(dout.float())
    for mode in ("auto", "scalar"):
        monkeypatch.setenv("VSA_B200_KERNELS", mode)
        leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
        out = V.b200_sparse_attention(*leaves, selected.to(DEV), sizes, block_size=(1, 1, be))
        out.backward(dout.to(DEV))
        _assert_close(out, want, atol=2e-2, rtol=2e-2)
        for leaf, oleaf in zip(leaves, ol):
            _assert_close(leaf.grad, oleaf.grad, atol=3e-2, rtol=3e-2)
        if mode == "auto":
            assert leaves[1].grad[0, :, be + 1:2 * be].abs().max() == 0      # padded key rows: exactly zero
    monkeypatch.delenv("VSA_B200_KERNELS")
    gate = torch.sigmoid(torch.randn(B, H, L, D)).to(dtype)
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v, gate)]
    out, aux = V.video_sparse_attn(leaves[0], leaves[1], leaves[2], sizes, sizes, tk, (1, 1, be), leaves[3], return_aux=True)
    out.backward(dout.to(DEV))
    ol = [t.clone().requires_grad_() for t in (q, k, v, gate)]
    want = O.vsa(ol[0], ol[1], ol[2], sizes, sizes, tk, (1, 1, be), ol[3], selected=aux["selected"].cpu(), q_blocks_per_chunk=8)
    want.backward(dout)
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    for leaf, oleaf in zip(leaves, ol):
        _assert_close(leaf.grad, oleaf.grad, atol=3e-2, rtol=3e-2)


def test_hot_key_block_all_queries_route_to_block_zero():
    V = _V()
    torch.manual_seed(43)
    be, nb, D = 64, 40, 128
    q, k, v, dout = (torch.randn(1, 2, be * nb, D).to(torch.bfloat16) for _ in range(4))
    sizes = torch.full((nb,), be)
    sizes[0] = 51
    selected = torch.zeros(1, 2, nb, 1, dtype=torch.int32)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    want = O.sparse_attention(*ol, selected, sizes, be)
    want.backward(dout.float())
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    out = V.b200_sparse_attention(*leaves, selected.to(DEV), sizes, block_size=(4, 4, 4))
    out.backward(dout.to(DEV))
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    # 40 query blocks x 64 rows accumulate into one key block: tolerance relative to that sum
    for leaf, oleaf in zip(leaves, ol):
        scale = max(1.0, float(oleaf.grad.abs().max()))
        _assert_close(leaf.grad, oleaf.grad, atol=3e-2 * scale, rtol=3e-2)
    assert leaves[1].grad[0, :, be:].abs().max() == 0       # unselected key blocks: zero


def test_query_and_key_lengths_may_differ():
    V = _V()
    torch.manual_seed(45)
    be, D = 64, 128
    q = torch.randn(1, 2, 4 * be, D).to(torch.bfloat16)
    k, v = (torch.randn(1, 2, 10 * be, D).to(torch.bfloat16) for _ in range(2))
    dout = torch.randn_like(q)
    kv_sizes = torch.full((10,), be)
    kv_sizes[3] = 20
    q_sizes = torch.full((4,), be)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    want, waux = O.vsa(*ol, kv_sizes, q_sizes, 3, (4, 4, 4), None, return_aux=True)
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    out, aux = V.video_sparse_attn(*leaves, kv_sizes, q_sizes, 3, (4, 4, 4), return_aux=True)
    differ, unexplained = O.topk_mismatch_report(waux["scores"], aux["selected"], 3)
    assert unexplained == 0
    want = O.vsa(*ol, kv_sizes, q_sizes, 3, (4, 4, 4), None, selected=aux["selected"].cpu())
    want.backward(dout)
    out.backward(dout.to(DEV))
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    for leaf, oleaf in zip(leaves, ol):
        _assert_close(leaf.grad, oleaf.grad, atol=3e-2, rtol=3e-2)


def test_downscaled_headline_config_with_gate():
    """[1,12,16384,128] be 64 topk 32 with a sigmoid gate, cut to 2 heads and 2048 tokens (topk 4)."""
    V = _V()
    torch.manual_seed(47)
    B, H, L, D, be, tk = 1, 2, 2048, 128, 64, 4
    q, k, v, dout = (torch.randn(B, H, L, D).to(torch.bfloat16) for _ in range(4))
    gate = torch.sigmoid(torch.randn(B, H, L, D)).to(torch.bfloat16)
    sizes = torch.full((L // be,), be)
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    g = gate.to(DEV).requires_grad_()
    out, aux = V.video_sparse_attn(*leaves, sizes, sizes, tk, (4, 4, 4), g, return_aux=True)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    og = gate.clone().requires_grad_()
    want, waux = O.vsa(*ol, sizes, sizes, tk, (4, 4, 4), og, return_aux=True)
    differ, unexplained = O.topk_mismatch_report(waux["scores"], aux["selected"], tk)
    # pooled scores may differ from the CPU's by one bf16 unit where the fp32 sums round differently;
    # such rows are allowed only while they stay rare
    assert unexplained <= 0.02 * B * H * (L // be), (differ, unexplained)
    ol = [t.clone().requires_grad_() for t in (q, k, v)]
    og = gate.clone().requires_grad_()
    want = O.vsa(*ol, sizes, sizes, tk, (4, 4, 4), og, selected=aux["selected"].cpu(), q_blocks_per_chunk=8)
    want.backward(dout)
    out.backward(dout.to(DEV))
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    for leaf, oleaf in zip(leaves + [g], ol + [og]):
        _assert_close(leaf.grad, oleaf.grad, atol=3e-2, rtol=3e-2)


# ---------------------------------------------------------------------------------------------
# size-independent properties at a larger shape
# ---------------------------------------------------------------------------------------------
def test_properties_full_topk_is_dense_attention_and_linearity_in_v():
    V = _V()
    torch.manual_seed(49)
    B, H, L, D, be = 1, 4, 4096, 128, 64
    nb = L // be
    q, k, v1, v2 = (torch.randn(B, H, L, D, device=DEV, dtype=torch.bfloat16) for _ in range(4))
    sizes = torch.full((nb,), be)
    every = torch.arange(nb, dtype=torch.int32, device=DEV).expand(B, H, nb, nb).contiguous()
    got = V.b200_sparse_attention(q, k, v1, every, sizes, block_size=(4, 4, 4))
    want = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v1.float())
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
    # fixed routes: the output is linear in V
    routes = _zipf_routes(B, H, nb, nb, 8, 11).to(DEV)
    a = V.b200_sparse_attention(q, k, v1, routes, sizes, block_size=(4, 4, 4)).float()
    b = V.b200_sparse_attention(q, k, v2, routes, sizes, block_size=(4, 4, 4)).float()
    ab = V.b200_sparse_attention(q, k, (v1.float() + v2.float()).to(torch.bfloat16), routes, sizes,
                                 block_size=(4, 4, 4)).float()
    torch.testing.assert_close(ab, a + b, atol=6e-2, rtol=3e-2)
    # routing order does not matter
    shuffled = routes[..., torch.randperm(8, device=DEV)]
    c = V.b200_sparse_attention(q, k, v1, shuffled, sizes, block_size=(4, 4, 4)).float()
    torch.testing.assert_close(c, a, atol=1e-2, rtol=1e-2)
    # deterministic: two runs give the same bits
    assert torch.equal(V.b200_sparse_attention(q, k, v1, routes, sizes, block_size=(4, 4, 4)).float(), a)


def test_host_resident_step_equals_one_big_call():
    """The chunked, copy-overlapped step for host tensors gives the bits of a single device call."""
    V = _V()
    from simple_vsa_b200.host import vsa_step_from_host
    torch.manual_seed(51)
    B, H, L, D, be, tk = 1, 5, 1024, 128, 64, 4
    q, k, v, dout = (torch.randn(B, H, L, D).to(torch.bfloat16).pin_memory() for _ in range(4))
    sizes = torch.full((L // be,), be)
    sizes[5] = 33
    out = {n: torch.empty(B, H, L, D, dtype=torch.bfloat16).pin_memory() for n in ("out", "dq", "dk", "dv")}
    vsa_step_from_host(q, k, v, dout, sizes, sizes, tk, (4, 4, 4), out=out, device=DEV, slices_per_chunk=2)
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    want = V.b200_vsa(*leaves, sizes, sizes, tk, (4, 4, 4))
    want.backward(dout.to(DEV))
    assert torch.equal(out["out"], want.detach().cpu())
    assert torch.equal(out["dq"], leaves[0].grad.cpu())
    # dK/dV sum over in-edges whose order inside a CSR row is not fixed: equal up to fp32 summation order
    for n, leaf in zip(("dk", "dv"), leaves[1:]):
        torch.testing.assert_close(out[n].float(), leaf.grad.cpu().float(), atol=2e-2, rtol=2e-2)


def test_more_tiles_than_the_tcgen05_list_holds_uses_the_warp_level_kernels():
    """topk above 1024 tiles is outside the tcgen05 kernels' tile list: the dispatcher must fall back to the
    warp-level kernels and stay correct (checked against dense attention with every block selected)."""
    V = _V()
    torch.manual_seed(53)
    be, nb, D = 64, 1040, 128
    q, k, v = (torch.randn(1, 1, be * nb, D, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    sizes = torch.full((nb,), be)
    # 8 query blocks only (Lq != Lkv), each attending to all 1040 key blocks
    ql = q[:, :, :8 * be].contiguous().requires_grad_()
    kl, vl = k.clone().requires_grad_(), v.clone().requires_grad_()
    every = torch.arange(nb, dtype=torch.int32, device=DEV).expand(1, 1, 8, nb).contiguous()
    got = V.b200_sparse_attention(ql, kl, vl, every, sizes, block_size=(4, 4, 4))
    dout = torch.randn_like(got)
    got.backward(dout)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (ql, kl, vl))
    want = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr)
    want.backward(dout.float())
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(ql.grad.float(), qr.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(kl.grad.float(), kr.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(vl.grad.float(), vr.grad, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("Qb,Kb,D", [(200, 136, 128), (8, 8, 128), (264, 1448, 128), (200, 136, 64), (256, 256, 64)])
def test_pooled_attention_tensor_core_path_matches_scalar_path(Qb, Kb, D, monkeypatch):
    """The tcgen05 pooled GEMMs (ragged M/N/K edges filled by TMA; head dim 64 as half-empty 128-wide tiles) against
    the CUDA-core GEMMs and torch."""
    from simple_vsa_b200 import _lib
    torch.manual_seed(55)
    BH = 3
    scale = D ** -0.5
    qc, kc, vc, dco = (torch.randn(n, device=DEV).to(torch.bfloat16) for n in
                       ((BH, Qb, D), (BH, Kb, D), (BH, Kb, D), (BH, Qb, D)))
    st = torch.cuda.current_stream().cuda_stream

    def run():
        scores = torch.empty(BH, Qb, Kb, device=DEV, dtype=torch.bfloat16)
        probs, ds = torch.empty_like(scores), torch.empty_like(scores)
        out_c = torch.empty(BH, Qb, D, device=DEV, dtype=torch.bfloat16)
        _lib.call("vsa_coarse_fwd", qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), scores.data_ptr(), probs.data_ptr(),
                  out_c.data_ptr(), BH, Qb, Kb, D, scale, 0, st)
        rowdot = torch.empty(BH, Qb, device=DEV)
        dq, dk, dv = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
        _lib.call("vsa_coarse_bwd", dco.data_ptr(), out_c.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                  probs.data_ptr(), ds.data_ptr(), rowdot.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                  BH, Qb, Kb, D, scale, 0, st)
        torch.cuda.synchronize()
        return scores, probs, out_c, dq, dk, dv

    fast = run()
    monkeypatch.setenv("VSA_B200_KERNELS", "scalar")
    slow = run()
    # scores: identical roundings, fp32 sums in a different order -> at most one bf16 unit apart
    assert (fast[0].float() - slow[0].float()).abs().max() <= 2 ** -7 * slow[0].float().abs().max()
    for a, b in zip(fast[1:], slow[1:]):
        torch.testing.assert_close(a.float(), b.float(), atol=2e-2, rtol=2e-2)
    # and against torch on the same roundings
    want_scores = (torch.matmul(qc.float(), kc.float().transpose(-2, -1)).to(torch.bfloat16).float() * scale)
    assert (fast[0].float() - want_scores).abs().max() <= 2 ** -6 * want_scores.abs().max()
    ql, kl, vl = (t.float().requires_grad_() for t in (qc, kc, vc))
    ref = torch.softmax(torch.matmul(ql, kl.transpose(-2, -1)) * scale, -1) @ vl
    ref.backward(dco.float())
    torch.testing.assert_close(fast[2].float(), ref, atol=2e-2, rtol=2e-2)
    for got, leaf in zip(fast[3:], (ql, kl, vl)):
        torch.testing.assert_close(got.float(), leaf.grad, atol=3e-2, rtol=3e-2)


def test_fused_block_mean_backward_equals_the_two_step_form():
    """vsa_sparse_bwd_dq_fused / _dkdv_fused = plain backward + vsa_block_mean_bwd_accumulate, up to the one
    rounding the fusion saves; ragged sizes, an unselected key block and a wholly padded tail included."""
    from simple_vsa_b200 import ops
    torch.manual_seed(77)
    B, H, nb, be, D, tk = 1, 2, 12, 64, 128, 3
    L = nb * be
    q, k, v, dout = (torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16) for _ in range(4))
    kv_sizes = torch.full((nb,), be, dtype=torch.int32, device=DEV)
    kv_sizes[2], kv_sizes[5], kv_sizes[11] = 37, 1, 0
    q_sizes = torch.full((nb,), be, dtype=torch.int32, device=DEV)
    q_sizes[1], q_sizes[7] = 50, 3
    # block 9 is never selected: its dK/dV come from the pooled gradients alone; block 11 (all padding) is selected
    pool = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 8, 10, 11], device=DEV)
    selected = torch.stack([pool[torch.randperm(pool.numel(), device=DEV)[:tk]] for _ in range(B * H * nb)])
    selected = selected.view(B, H, nb, tk).to(torch.int32)
    scale = 1.0 / math.sqrt(D)
    out_s, lse = ops.sparse_forward(q, k, v, selected, kv_sizes, be, scale, True)
    dqc, dkc, dvc = (torch.randn(B, H, nb, D, device=DEV).to(torch.bfloat16) for _ in range(3))
    fused = ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale,
                                pooled_grads=(dqc, dkc, dvc, q_sizes))
    plain = ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale)
    st = torch.cuda.current_stream().cuda_stream
    from simple_vsa_b200 import _lib
    for g, m, sizes in zip(plain, (dqc, dkc, dvc), (q_sizes, kv_sizes, kv_sizes)):
        _lib.call("vsa_block_mean_bwd_accumulate", g.data_ptr(), m.data_ptr(), sizes.data_ptr(), B * H, L, D, be,
                  _lib.VSA_BF16, st)
    for name, f, p_ in zip(("dq", "dk", "dv"), fused, plain):
        # dK/dV sums run in a different order from launch to launch (unordered CSR), hence not bitwise
        _assert_close(f, p_, atol=2e-2, rtol=2e-2)
        assert torch.isfinite(f.float()).all(), name
    # rows beyond a block's size receive nothing from the pooled gradient: same values as the plain backward
    plain2 = ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale)
    pad_q = (torch.arange(be, device=DEV)[None, :] >= q_sizes[:, None]).reshape(L)
    assert torch.equal(fused[0][:, :, pad_q], plain2[0][:, :, pad_q])
    pad_k = (torch.arange(be, device=DEV)[None, :] >= kv_sizes[:, None]).reshape(L)
    assert float(fused[1][:, :, pad_k].float().abs().max()) == 0.0
    assert float(fused[2][:, :, pad_k].float().abs().max()) == 0.0


def test_compression_gate_trains_through_the_operator():
    """The gate layer sits outside the operator; its weights must receive gradient through the pooled branch
    (mirrors tests/test_common.py:33-55 of the reference; block of 4 tokens, D = 8: the CUDA-core path)."""
    V = _V()
    torch.manual_seed(1)
    batch, heads, head_dim, be, nb = 1, 2, 8, 4, 3
    seq, dim = be * nb, heads * head_dim
    hidden = torch.randn(batch, seq, dim, device=DEV)
    q, k, v = (torch.randn(batch, heads, seq, head_dim, device=DEV) for _ in range(3))
    vbs = torch.full((nb,), be, dtype=torch.long, device=DEV)
    layer = V.CompressionGate(dim=dim, num_heads=heads).to(DEV)
    out = V.video_sparse_attn(q, k, v, vbs, vbs, 2, (1, 1, be), layer(hidden))
    out.square().mean().backward()
    grad = layer.to_gate_compress.weight.grad
    assert grad is not None and torch.isfinite(grad).all() and float(grad.abs().sum()) > 0
    # same value as the oracle on the CPU
    layer_c = V.CompressionGate(dim=dim, num_heads=heads)
    layer_c.load_state_dict({n: t.cpu() for n, t in layer.state_dict().items()})
    want = O.vsa(q.cpu(), k.cpu(), v.cpu(), vbs.cpu(), vbs.cpu(), 2, (1, 1, be), layer_c(hidden.cpu()))
    want.square().mean().backward()
    _assert_close(out.detach(), want.detach(), atol=1e-5, rtol=1e-5)
    _assert_close(grad, layer_c.to_gate_compress.weight.grad, atol=1e-5, rtol=1e-4)


def test_a_large_problem_off_the_tensor_path_warns_once():
    """fp32 (the validation mode) is served by the CUDA-core kernels only; a problem of 1e11 useful FLOPs or more says so
    once per process; tensor-core shapes (head dim 128 on tcgen05, head dim 64 on the warp-level kernels) and small
    validation-size problems never do."""
    import warnings

    from simple_vsa_b200 import ops
    V = _V()
    torch.manual_seed(7)
    be, tk = 64, 32
    sizes = torch.full((256,), be)
    small = [torch.randn(1, 1, 4 * be, 64, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    big64 = [torch.randn(1, 4, 256 * be, 64, device=DEV, dtype=torch.float32) for _ in range(3)]
    big64_bf16 = [t.to(torch.bfloat16) for t in big64]
    big128 = [torch.randn(1, 2, 256 * be, 128, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    ops._warned_slow_path = False
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        with torch.no_grad():
            V.video_sparse_attn(*small, sizes[:4], sizes[:4], 2, (4, 4, 4))
            V.video_sparse_attn(*big128, sizes, sizes, tk, (4, 4, 4))
            V.video_sparse_attn(*big64_bf16, sizes, sizes, tk, (4, 4, 4))
    with pytest.warns(RuntimeWarning, match="CUDA-core validation kernels"), torch.no_grad():
        out = V.video_sparse_attn(*big64, sizes, sizes, tk, (4, 4, 4))
    assert torch.isfinite(out.float()).all()
    with warnings.catch_warnings():
        warnings.simplefilter("error")                      # the second large call stays quiet
        with torch.no_grad():
            V.video_sparse_attn(*big64, sizes, sizes, tk, (4, 4, 4))
    ops._warned_slow_path = False


def test_compression_gate_writes_the_operator_layout_without_a_transposing_copy():
    """bf16, 8 heads of 128: the gate comes out dense in [B,H,S,D] (the operator's ``_dense`` then copies nothing),
    equals the reference form Linear(x).view(B,S,H,D).transpose(1,2) up to one bf16 rounding of the same fp32 sums,
    and the batched GEMM does not materialise the hidden states once per head."""
    V = _V()
    torch.manual_seed(5)
    B, H, S, D = 2, 8, 16384, 128
    dim = H * D
    layer = V.CompressionGate(dim, H).to(DEV).to(torch.bfloat16)
    x = (torch.randn(B, S, dim, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    gate = layer(x)
    torch.cuda.synchronize()
    grown = torch.cuda.max_memory_allocated() - before
    assert gate.is_contiguous() and gate.shape == (B, H, S, D)
    # the output (64 MB) and at most a library workspace -- not the hidden states once per head (256 MB per batch entry)
    assert grown < 2 * gate.numel() * 2 + (40 << 20), grown
    want = layer.to_gate_compress(x).view(B, S, H, D).transpose(1, 2)
    _assert_close(gate.detach(), want.detach(), atol=2e-2, rtol=2e-2)
    w = torch.randn_like(gate)
    params = [x, layer.to_gate_compress.weight, layer.to_gate_compress.bias]
    got = torch.autograd.grad((gate.float() * w.float()).sum(), params)
    ref = torch.autograd.grad((want.float() * w.float()).sum(), params)
    for a, b in zip(got, ref):
        scale = max(1.0, float(b.float().abs().max()))
        _assert_close(a, b, atol=2e-2 * scale, rtol=2e-2)


@pytest.mark.parametrize("kernels", ["auto", "mma", "scalar"])
def test_route_ids_outside_the_key_table_count_as_empty_blocks(kernels, monkeypatch):
    """A caller-supplied routing table may hold ids that are not key blocks (negative, or >= Kb).  Every consumer
    treats them like a block with no valid token -- the same way route inversion drops them -- so forward, dQ and
    dK/dV stay finite and agree with the table that points those entries at an all-padding block instead."""
    V = _V()
    monkeypatch.setenv("VSA_B200_KERNELS", kernels)
    torch.manual_seed(91)
    be, nb, D, tk = 64, 10, 128, 4
    q, k, v, dout = (torch.randn(1, 2, be * nb, D, device=DEV).to(torch.bfloat16) for _ in range(4))
    sizes = torch.full((nb,), be)
    sizes[nb - 1] = 0                                   # an all-padding block that nothing below selects by itself
    pool = torch.arange(nb - 1)
    good = torch.stack([pool[torch.randperm(nb - 1)[:tk]] for _ in range(2 * nb)]).view(1, 2, nb, tk).to(torch.int32)
    bad = good.clone()
    bad[0, 0, 3, 1] = -7
    bad[0, 1, 5, 0] = nb + 3
    bad[0, 1, 0, 3] = 2 ** 30
    stand_in = bad.clone()
    stand_in[(bad < 0) | (bad >= nb)] = nb - 1
    results = []
    for table in (bad, stand_in):
        leaves = [t.clone().requires_grad_() for t in (q, k, v)]
        out = V.b200_sparse_attention(*leaves, table.to(DEV), sizes, block_size=(1, 1, be))
        out.backward(dout)
        results.append([out.detach()] + [t.grad for t in leaves])
    for a, b in zip(*results):
        assert torch.isfinite(a.float()).all()
        torch.testing.assert_close(a.float(), b.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("be,nb,tk,ragged", [(64, 24, 6, True), (64, 33, 5, False), (256, 8, 3, True), (128, 14, 4, True)])
def test_backward_that_stores_ds_equals_the_recomputing_backward(be, nb, tk, ragged, monkeypatch):
    """``VSA_B200_BACKWARD=stored_ds`` forms dS once (key-owned pass stores it, query-owned pass multiplies it by K);
    the default backward forms it twice, once per pass.  Same dQ up to the rounding point of the scale (before or
    after bf16), same dK/dV, with the pooled gradients folded in and without, and with the slices walked in groups
    smaller than the batch."""
    from simple_vsa_b200 import ops
    torch.manual_seed(93)
    B, H, D = 1, 3, 128
    L = be * nb
    q, k, v, dout = (torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16) for _ in range(4))
    kv_sizes = torch.full((nb,), be, dtype=torch.int32, device=DEV)
    q_sizes = kv_sizes.clone()
    if ragged:
        kv_sizes[1], kv_sizes[nb // 2], kv_sizes[-1] = 1, be // 2 + 3, 0
        q_sizes[2] = be - 5
    selected = _zipf_routes(B, H, nb, nb, tk, 19).to(DEV)
    scale = 1.0 / math.sqrt(D)
    out_s, lse = ops.sparse_forward(q, k, v, selected, kv_sizes, be, scale, True)
    pooled = tuple(torch.randn(B, H, nb, D, device=DEV).to(torch.bfloat16) for _ in range(3)) + (q_sizes,)
    for pg in (None, pooled):
        monkeypatch.delenv("VSA_B200_BACKWARD", raising=False)
        want = ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale, pooled_grads=pg)
        monkeypatch.setenv("VSA_B200_BACKWARD", "stored_ds")
        for cap in ("16", "1e-9"):                 # one group of slices, then one slice per group
            monkeypatch.setenv("VSA_B200_DS_WORKSPACE_GB", cap)
            got = ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale, pooled_grads=pg)
            for name, g, w in zip(("dq", "dk", "dv"), got, want):
                assert torch.isfinite(g.float()).all(), name
                _assert_close(g, w, atol=2e-2, rtol=2e-2)
    # and against the oracle
    ol = [t.cpu().float().requires_grad_() for t in (q, k, v)]
    O.sparse_attention(*ol, selected.cpu(), kv_sizes.cpu(), be, scale).backward(dout.cpu().float())
    for g, leaf in zip(got if pg is None else ops.sparse_backward(dout, q, k, v, out_s, lse, selected, kv_sizes, be, scale),
                       ol):
        _assert_close(g, leaf.grad, atol=3e-2, rtol=3e-2)


def test_a_bounded_wait_that_runs_out_is_reported_and_later_kernels_drain():
    """The failure path of the tcgen05 kernels, walked without making anything fail: a self-test warp waits 1 ms on
    a barrier nothing arrives at and gives up.  The code must reach the status word, kernels launched while the
    word is set must return without writing, the Python check must raise, and after the clear the same launch works."""
    from simple_vsa_b200 import _lib
    torch.manual_seed(95)
    be, nb, D, tk = 64, 6, 128, 2
    q, k, v = (torch.randn(1, 1, be * nb, D).to(torch.bfloat16) for _ in range(3))
    sizes = torch.full((nb,), be)
    selected = torch.stack([torch.randperm(nb)[:tk] for _ in range(nb)]).view(1, 1, nb, tk).to(torch.int32)
    want = O.sparse_attention(q, k, v, selected, sizes, be)
    qd, kd, vd, sd, zd = q.to(DEV), k.to(DEV), v.to(DEV), selected.to(DEV), sizes.to(DEV, torch.int32)
    st = torch.cuda.current_stream().cuda_stream

    def forward(out, lse):
        _lib.call("vsa_sparse_fwd", qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), sd.data_ptr(), zd.data_ptr(),
                  out.data_ptr(), lse.data_ptr(), 1, be * nb, be * nb, D, be, tk, 1.0 / math.sqrt(D), _lib.VSA_BF16, st)

    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    _lib.call("vsa_selftest_wait_timeout", 1_000_000, gave_up.data_ptr(), st)
    torch.cuda.synchronize()
    assert int(gave_up) == 1
    out = torch.full((1, 1, be * nb, D), 7.0, device=DEV, dtype=torch.bfloat16)
    lse = torch.zeros((1, 1, be * nb), device=DEV)
    forward(out, lse)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()) and bool((lse == 0).all())      # drained: nothing was written
    with pytest.raises(_lib.VsaError, match="code 201"):
        _lib.raise_on_device_timeout("test")
    assert _lib.device_status() == 0                                  # the check cleared the word
    forward(out, lse)
    torch.cuda.synchronize()
    _assert_close(out, want, atol=2e-2, rtol=2e-2)
    with pytest.raises(ValueError, match="limit"):
        _lib.call("vsa_selftest_wait_timeout", 10, gave_up.data_ptr(), st)


@pytest.mark.parametrize("kernels", ["auto", "mma", "scalar"])
@pytest.mark.parametrize("with_gate", [False, True])
def test_forward_with_the_combine_folded_in_equals_the_two_step_form(kernels, with_gate, monkeypatch):
    """vsa_sparse_fwd_combine = vsa_sparse_fwd followed by vsa_combine_fwd, bit for bit: block 64 and 256, ragged
    sizes, and a key block scaled so that the tcgen05 forward hands some tiles to the exact redo kernel (which must
    then redo their combined rows as well)."""
    from simple_vsa_b200 import _lib, ops
    monkeypatch.setenv("VSA_B200_KERNELS", kernels)
    torch.manual_seed(97)
    st = torch.cuda.current_stream().cuda_stream
    for be, nb, tk in ((64, 12, 4), (256, 5, 2)):
        B, H, D = 1, 2, 128
        L = be * nb
        q, k, v = (torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16) for _ in range(3))
        k[:, :, 5 * 64:6 * 64] *= 40.0            # scores far above the first pair's maximum whenever selected late
        out_c = torch.randn(B, H, nb, D, device=DEV).to(torch.bfloat16)
        gate = torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16) if with_gate else None
        sizes = torch.full((nb,), be, dtype=torch.int32, device=DEV)
        sizes[1], sizes[nb - 1] = be // 2 + 1, 3
        selected = torch.stack([torch.randperm(nb)[:tk] for _ in range(B * H * nb)]).view(B, H, nb, tk).to(torch.int32).to(DEV)
        scale = 1.0 / math.sqrt(D)
        out_s, lse = ops.sparse_forward(q, k, v, selected, sizes, be, scale, True)
        want = torch.empty_like(q)
        _lib.call("vsa_combine_fwd", out_s.data_ptr(), out_c.data_ptr(), gate.data_ptr() if with_gate else None,
                  want.data_ptr(), B * H, L, D, be, _lib.VSA_BF16, st)
        out_s2, lse2, got = ops.sparse_forward(q, k, v, selected, sizes, be, scale, True, combine_with=(out_c, gate))
        assert torch.equal(out_s2, out_s) and torch.equal(lse2, lse)
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)
        _assert_close(want, O.combine(out_s.cpu(), out_c.cpu(), gate.cpu() if with_gate else None, be, torch.bfloat16),
                      atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("be,nb,tk,W", [(64, 16, 5, 2), (64, 24, 6, 4), (256, 8, 3, 2), (128, 12, 4, 2)])
def test_shard_major_kv_layout_equals_the_ordinary_layout(be, nb, tk, W):
    """The kernels of the sequence-parallel mode read K/V (and write dK/dV) in the rank-major layout an all-gather
    leaves, ``[W,B,H,L/W,D]``.  One GPU, no collective: the same operator on the same numbers in both layouts, a
    rank's share of the queries against all keys, ragged blocks, a gate, and a scaled key block so that the exact
    redo kernel takes part."""
    V = _V()
    from simple_vsa_b200 import ops
    torch.manual_seed(99)
    B, H, D = 1, 3, 128
    L = be * nb
    l = L // W
    q_all, k, v = (torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16) for _ in range(3))
    k[:, :, 5 * 64:6 * 64] *= 30.0
    sizes = torch.full((nb,), be)
    sizes[1], sizes[nb - 2] = be // 2 + 3, 7
    for rank in (0, W - 1):
        sl = slice(rank * l, (rank + 1) * l)
        q = q_all[:, :, sl].contiguous()
        gate = torch.randn(B, H, l, D, device=DEV).to(torch.bfloat16)
        dout = torch.randn(B, H, l, D, device=DEV).to(torch.bfloat16)
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
        assert torch.equal(out_b, out_a)                       # same routes, same tiles, same order
        assert torch.equal(b[0].grad, a[0].grad) and torch.equal(b[1].grad, a[3].grad)
        for got_sh, want in ((k_sh.grad, a[1].grad), (v_sh.grad, a[2].grad)):
            got = got_sh.permute(1, 2, 0, 3, 4).reshape(B, H, L, D)
            _assert_close(got, want, atol=2e-2, rtol=2e-2)     # CSR rows are unordered: fp32 sums in another order
    with pytest.raises(ValueError, match="shard-major"):
        ops.vsa_on_gathered_shards(q.float(), k_sh.detach().float(), v_sh.detach().float(), kc.float(), vc.float(),
                                   sizes, q_sizes, tk, (1, 1, be))


@pytest.mark.parametrize("be,nb,tk", [(64, 40, 7), (64, 24, 24), (256, 6, 3), (128, 10, 6)])
def test_the_two_schedules_of_the_forward_give_the_same_bits(be, nb, tk, monkeypatch):
    """One CTA per query tile and the persistent form (one CTA per SM walking the query tiles, chosen for short
    routes) run the same arithmetic in the same order: outputs, statistics and combined outputs are bit-identical,
    with ragged blocks, an odd number of live tiles, an empty route and more query tiles than SMs."""
    from simple_vsa_b200 import ops
    torch.manual_seed(101)
    B, H, D = 1, 5, 128
    L = be * nb
    q, k, v = (torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16) for _ in range(3))
    out_c = torch.randn(B, H, nb, D, device=DEV).to(torch.bfloat16)
    gate = torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16)
    sizes = torch.full((nb,), be, dtype=torch.int32, device=DEV)
    sizes[1], sizes[3], sizes[nb - 1] = be // 2 + 1, 0, 5
    selected = torch.stack([torch.randperm(nb)[:tk] for _ in range(B * H * nb)]).view(B, H, nb, tk).to(torch.int32).to(DEV)
    selected[0, 2, 4, :] = 3                       # a query block whose whole route is the empty block
    scale = 1.0 / math.sqrt(D)
    results = {}
    for mode in ("classic", "persistent"):
        monkeypatch.setenv("VSA_B200_FWD", mode)
        results[mode] = ops.sparse_forward(q, k, v, selected, sizes, be, scale, True, combine_with=(out_c, gate))
    for a, b in zip(results["classic"], results["persistent"]):
        assert torch.equal(torch.nan_to_num(a.float(), nan=7.0), torch.nan_to_num(b.float(), nan=7.0))
    out_s = results["persistent"][0]
    live = torch.ones(B, H, L, dtype=torch.bool)
    live[0, 2, 4 * be:5 * be] = False                # the rows of the empty route are NaN in both, as in the oracle
    want = O.sparse_attention(q.cpu(), k.cpu(), v.cpu(), selected.cpu(), sizes.cpu(), be)
    _assert_close(out_s.cpu()[live], want[live], atol=2e-2, rtol=2e-2)
    assert torch.isnan(out_s.float().cpu()[~live]).all()


@pytest.mark.parametrize("seed", list(range(24)))
def test_random_shapes_tensor_path_matches_cuda_core_path(seed, monkeypatch):
    """Seeded random problems (block 64, 128 or 256, 1..40 blocks, any topk, query length != key length, random ragged
    and empty blocks, with and without a gate): the whole operator on the tcgen05 kernels against the same call on
    the CUDA-core kernels, forward and every gradient; seeds 10-13 and 21-23 run in fp16, the others in bf16; seeds 14-17 use blocks of 128 tokens; seeds from 18 up
    have head dim 64 (the warp-level tensor-core kernels).  The routes are fixed by the first run's Top-K (pooled scores
    are computed by the same kernels in both runs)."""
    V = _V()
    dt = torch.float16 if 10 <= seed < 14 or seed >= 21 else torch.bfloat16
    g = torch.Generator().manual_seed(1000 + seed)
    ri = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    be = 64 if ri(0, 3) else 256
    if 14 <= seed < 18:
        be = 128
    Kb = ri(1, {64: 40, 128: 20, 256: 10}[be])
    Qb = ri(1, {64: 24, 128: 12, 256: 6}[be])
    tk = ri(1, Kb)
    B, H, D = ri(1, 2), ri(1, 3), (64 if seed >= 18 else 128)
    q = torch.randn(B, H, Qb * be, D, generator=g).to(dt)
    k, v = (torch.randn(B, H, Kb * be, D, generator=g).to(dt) for _ in range(2))
    dout = torch.randn(B, H, Qb * be, D, generator=g).to(dt)
    gate = torch.randn(B, H, Qb * be, D, generator=g).to(dt) if ri(0, 1) else None
    kv_sizes = torch.full((Kb,), be)
    q_sizes = torch.full((Qb,), be)
    for sizes in (kv_sizes, q_sizes):
        for _ in range(ri(0, 3)):
            sizes[ri(0, sizes.numel() - 1)] = ri(0, be)
    if int(kv_sizes.sum()) == 0:
        kv_sizes[0] = 1
    results = {}
    for mode in ("auto", "scalar"):
        monkeypatch.setenv("VSA_B200_KERNELS", mode)
        leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
        gl = gate.to(DEV).requires_grad_() if gate is not None else None
        out, aux = V.video_sparse_attn(*leaves, kv_sizes, q_sizes, tk, (1, 1, be), gl, return_aux=True)
        out.backward(dout.to(DEV))
        results[mode] = [out.detach(), aux["selected"]] + [t.grad for t in leaves] + ([gl.grad] if gl is not None else [])
    a, b = results["auto"], results["scalar"]
    same_routes = torch.equal(a[1], b[1])
    assert same_routes, "the pooled branch must not depend on the fine kernels' path"
    # a query block whose selected blocks are all empty has no defined output (NaN in both paths, as in the reference)
    finite = torch.isfinite(b[0].float())
    assert torch.equal(finite, torch.isfinite(a[0].float()))
    _assert_close(torch.where(finite, a[0].float(), torch.zeros(())), torch.where(finite, b[0].float(), torch.zeros(())),
                  atol=2e-2, rtol=2e-2)
    if bool(finite.all()):
        for x, y in zip(a[2:], b[2:]):
            _assert_close(x, y, atol=3e-2, rtol=3e-2)


def test_whole_step_replays_from_a_cuda_graph():
    """Forward + backward of the operator captured once into a CUDA graph and replayed on new numbers in the same
    buffers: no launch of the path synchronises, allocates outside torch's capturable pool, or keeps host-side state
    that a replay would miss.  The replay must give what an eager call gives on the same inputs."""
    V = _V()
    torch.manual_seed(301)
    B, H, L, D, be, tk = 1, 4, 4096, 128, 64, 8
    sizes = torch.full((L // be,), be, dtype=torch.int32, device=DEV)
    sizes[5], sizes[-1] = 33, 1
    static = [torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16).requires_grad_() for _ in range(4)]   # q, k, v, gate
    dout = torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16)

    def step():
        out = V.b200_vsa(static[0], static[1], static[2], sizes, sizes, tk, (4, 4, 4), static[3])
        grads = torch.autograd.grad(out, static, dout)
        return (out,) + grads

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                      # warm-up outside the capture: attributes, tensor maps, allocator
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    fresh = [torch.randn(B, H, L, D, device=DEV).to(torch.bfloat16) for _ in range(4)]
    with torch.no_grad():
        for s, f in zip(static, fresh):
            s.copy_(f)
    graph.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in captured]
    want = step()
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]) and torch.equal(got[4], want[4])   # out, dq, dgate
    for g, w in zip(got[2:4], want[2:4]):                                                                 # dk, dv: CSR row order
        _assert_close(g, w, atol=2e-2, rtol=2e-2)
