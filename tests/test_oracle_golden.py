"""The CPU oracle against the vectors the reference project produced (tests/golden)."""

import os

import numpy as np
import pytest
import torch

from oracle import vsa_oracle as O
from tests.golden.cases import SPARSE_CASES, VSA_CASES, sparse_inputs, to_np, vsa_inputs

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def _tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == "f32" else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("name", list(VSA_CASES))
def test_vsa_oracle_matches_reference_vectors(name):
    case = VSA_CASES[name]
    gold = _load("vsa_" + name)
    q, k, v, gate, dout, sizes = vsa_inputs(case)
    fingerprint = float(q.double().sum() + 2 * k.double().sum() + 3 * v.double().sum())
    assert fingerprint == pytest.approx(float(gold["input_sum"]), rel=0, abs=1e-9), "seeded inputs drifted"
    leaves = [t.clone().requires_grad_(case["grad"]) for t in (q, k, v)]
    g = gate.clone().requires_grad_(case["grad"]) if gate is not None else None
    out, aux = O.vsa(*leaves, sizes, sizes, case["topk"], case["block_size"], g, return_aux=True)
    be = O.block_elements(case["block_size"])
    # pooled means, scores and routing are the same torch calls: expect identical bits
    for tag, x in (("q", q), ("k", k), ("v", v)):
        np.testing.assert_array_equal(to_np(O.block_mean(x, sizes, be)), gold["mean_" + tag])
    np.testing.assert_array_equal(to_np(aux["scores"]), gold["scores"])
    np.testing.assert_array_equal(np.sort(aux["selected"].numpy(), -1), np.sort(gold["selected"], -1))
    np.testing.assert_allclose(to_np(aux["out_c_blocks"]), gold["out_c_blocks"], **_tol(case["dtype"]))
    np.testing.assert_allclose(to_np(out), gold["out"], **_tol(case["dtype"]))
    if "out_dense" in gold:           # the dense masked-fill form the reference pins its gather form to
        np.testing.assert_allclose(to_np(out), gold["out_dense"], atol=1e-5, rtol=1e-5)
        np.testing.assert_allclose(to_np(aux["out_s"]), gold["out_sparse"], atol=1e-5, rtol=1e-5)
    if case["grad"]:
        out.backward(dout)
        stride = int(gold["grad_row_stride"])
        gtol = dict(atol=1e-5, rtol=1e-4) if case["dtype"] == "f32" else dict(atol=3e-2, rtol=3e-2)
        for tag, leaf in zip(("dq", "dk", "dv"), leaves):
            np.testing.assert_allclose(to_np(leaf.grad)[:, :, ::stride], gold[tag], **gtol)
        if g is not None:
            np.testing.assert_allclose(to_np(g.grad)[:, :, ::stride], gold["dgate"], **gtol)


@pytest.mark.parametrize("name", list(SPARSE_CASES))
@pytest.mark.parametrize("chunk", [None, 1])
def test_route_explicit_oracle_matches_reference_vectors(name, chunk):
    case = SPARSE_CASES[name]
    gold = _load("sparse_" + name)
    q, k, v, dout, sizes, selected = sparse_inputs(case)
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    out, lse2 = O.sparse_attention(*leaves, selected, sizes, case["be"],
                                   q_blocks_per_chunk=chunk, return_lse2=True)
    np.testing.assert_allclose(to_np(out), gold["out_s"], atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(to_np(lse2), gold["lse2"], atol=1e-4, rtol=1e-5)
    out.backward(dout.float())
    for tag, leaf in zip(("dq", "dk", "dv"), leaves):
        np.testing.assert_allclose(to_np(leaf.grad), gold[tag], atol=2e-2 if case["dtype"] != "f32" else 1e-5, rtol=1e-2)


def test_block_mean_known_answer():
    gold = _load("block_mean_64_37_11")
    torch.manual_seed(11)
    x = torch.randn(1, 2, 3 * 64, 128).to(torch.bfloat16)
    sizes = torch.tensor([64, 37, 11])
    grad = torch.randn(1, 2, 3, 128).to(torch.bfloat16)
    assert float(x.double().sum()) == pytest.approx(float(gold["input_sum"]), abs=1e-9)
    leaf = x.clone().requires_grad_()
    out = O.block_mean(leaf, sizes, 64)
    out.backward(grad)
    np.testing.assert_array_equal(to_np(out), gold["out"])
    np.testing.assert_allclose(to_np(leaf.grad), gold["dx"], atol=1e-6)
    # padding values must not leak into the mean
    y = x.clone()
    y[:, :, 64 + 37:128] = 1e4
    np.testing.assert_array_equal(to_np(O.block_mean(y, sizes, 64)), gold["out"])


def test_full_topk_is_dense_attention():
    torch.manual_seed(7)
    q, k, v = (torch.randn(1, 2, 32, 16) for _ in range(3))
    sizes = torch.full((4,), 8)
    sel = torch.arange(4).expand(1, 2, 4, 4)
    got = O.sparse_attention(q, k, v, sel, sizes, 8)
    want = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_argument_errors_carry_reference_substrings():
    q = torch.randn(1, 1, 12, 8)
    s3 = torch.full((3,), 4)
    with pytest.raises(ValueError, match="divisible"):
        O.vsa(q[:, :, :10], q[:, :, :10], q[:, :, :10], s3, s3, 1, (1, 1, 4))
    with pytest.raises(ValueError, match="variable_block_sizes"):
        O.vsa(q, q, q, s3[:2], s3, 1, (1, 1, 4))
    with pytest.raises(ValueError, match="topk"):
        O.vsa(q, q, q, s3, s3, 4, (1, 1, 4))


def test_invert_routes_small():
    sel = torch.tensor([[[[0, 2], [1, 2], [0, 1]]]])
    counts, offsets, inverse = O.invert_routes(sel, 3)
    assert counts[0, 0].tolist() == [2, 2, 2]
    assert offsets[0, 0].tolist() == [0, 2, 4]
    assert inverse[0, 0].tolist() == [0, 2, 1, 2, 0, 1]
