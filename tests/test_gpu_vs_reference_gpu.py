"""Parity with the reference project's own GPU implementation (its Triton kernels), where an installed copy of
the unmodified reference package is available under ``baseline/_ref`` (put there by ``__graft_entry__.build()``;
never part of this repository's sources).  Skipped when the package or Triton cannot be imported."""

import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _reference():
    if not os.path.isdir(os.path.join(REF, "vsa")):
        pytest.skip("no installed copy of the reference package")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    try:
        from vsa import triton_sparse_attention, triton_vsa
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"reference package not importable: {exc}")
    return triton_vsa, triton_sparse_attention


def _grads(fn, tensors, dout):
    for t in tensors:
        t.grad = None
    out = fn()
    out.backward(dout)
    return [out.detach().float()] + [t.grad.detach().float().clone() for t in tensors]


@pytest.mark.parametrize("shape,tk,ragged,with_gate", [
    ((1, 4, 64 * 32, 128), 8, False, True),        # full blocks, gate
    ((2, 2, 64 * 24, 128), 5, True, False),        # ragged blocks, no gate
])
def test_whole_operator_matches_the_reference_gpu_kernels(shape, tk, ragged, with_gate):
    triton_vsa, _ = _reference()
    import simple_vsa_b200 as V
    torch.manual_seed(70)
    dev = "cuda:0"
    B, H, L, D = shape
    nb = L // 64
    q, k, v = (torch.randn(shape, device=dev, dtype=torch.bfloat16).requires_grad_() for _ in range(3))
    dout = torch.randn(shape, device=dev, dtype=torch.bfloat16)
    gate = torch.sigmoid(torch.randn(shape, device=dev)).to(torch.bfloat16).requires_grad_() if with_gate else None
    sizes = torch.full((nb,), 64, dtype=torch.long, device=dev)
    if ragged:
        sizes[3], sizes[7], sizes[nb - 1] = 41, 19, 1
        pad = (torch.arange(64, device=dev)[None, :] >= sizes[:, None]).reshape(L)
        with torch.no_grad():
            for t in (q, k, v):
                t[:, :, pad] = 0
    leaves = [q, k, v] + ([gate] if with_gate else [])
    want = _grads(lambda: triton_vsa(q, k, v, sizes, sizes, tk, (4, 4, 4), gate), leaves, dout)
    got = _grads(lambda: V.b200_vsa(q, k, v, sizes, sizes, tk, (4, 4, 4), gate), leaves, dout)
    names = ["out", "dq", "dk", "dv", "dgate"]
    for name, g, w in zip(names, got, want):
        # both sides round P and dS to bf16 before their second GEMM: they agree far inside the stated budget
        np.testing.assert_allclose(g.cpu().numpy(), w.cpu().numpy(), atol=1e-2, rtol=2e-2, err_msg=name)


def test_route_explicit_matches_the_reference_gpu_kernels():
    _, triton_sparse_attention = _reference()
    import simple_vsa_b200 as V
    torch.manual_seed(71)
    dev = "cuda:0"
    shape, nb, tk = (1, 3, 64 * 16, 128), 16, 6
    q, k, v = (torch.randn(shape, device=dev, dtype=torch.bfloat16).requires_grad_() for _ in range(3))
    dout = torch.randn(shape, device=dev, dtype=torch.bfloat16)
    sizes = torch.full((nb,), 64, dtype=torch.long, device=dev)
    sizes[5] = 23
    selected = torch.stack([torch.randperm(nb, device=dev)[:tk] for _ in range(3 * nb)]).view(1, 3, nb, tk).to(torch.int32)
    want = _grads(lambda: triton_sparse_attention(q, k, v, selected, sizes, block_size=(4, 4, 4)), [q, k, v], dout)
    got = _grads(lambda: V.b200_sparse_attention(q, k, v, selected, sizes, block_size=(4, 4, 4)), [q, k, v], dout)
    for name, g, w in zip(["out", "dq", "dk", "dv"], got, want):
        np.testing.assert_allclose(g.cpu().numpy(), w.cpu().numpy(), atol=1e-2, rtol=2e-2, err_msg=name)
