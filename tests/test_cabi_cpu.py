"""CPU-side checks: the C ABI library loads and exports what the header declares; host-side
argument checks behave like the reference's; nothing here launches a kernel."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "vsa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vsa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import simple_vsa_b200._lib as L
    lib = ctypes.CDLL(L.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/vsa_b200.h but not exported"
    for name in list(L.SIGNATURES) + list(L.PLAIN):
        assert name in names, f"{name} bound in _lib.py but not declared in the header"
    assert L.lib.vsa_version() >= 100
    assert L.last_error() == ""


def test_bad_arguments_are_refused_before_any_launch():
    import simple_vsa_b200._lib as L
    # null pointers and a topk out of range come back as status codes with a message, no CUDA call made
    rc = L.lib.vsa_topk(None, None, 4, 8, 2, 0, None)
    assert rc == L.ERR_BAD_ARGUMENT and "null" in L.last_error()
    rc = L.lib.vsa_topk(1, 1, 4, 8, 9, 0, None)
    assert rc == L.ERR_BAD_ARGUMENT and "topk" in L.last_error()
    rc = L.lib.vsa_sparse_fwd(1, 1, 1, 1, 1, 1, None, 1, 100, 128, 128, 64, 1, 0.1, 0, None)
    assert rc == L.ERR_BAD_ARGUMENT and "divisible" in L.last_error()
    rc = L.lib.vsa_sparse_fwd(1, 1, 1, 1, 1, 1, None, 1, 128, 128, 128, 64, 1, 0.1, 7, None)
    assert rc == L.ERR_UNSUPPORTED
    with pytest.raises(ValueError, match="topk"):
        L.call("vsa_topk", 1, 1, 4, 8, 0, 0, None)


def test_operator_validation_matches_reference_messages():
    import simple_vsa_b200 as V
    q = torch.randn(1, 1, 12, 8)
    s3 = torch.full((3,), 4)
    with pytest.raises(ValueError, match="divisible"):
        V.b200_vsa(q[:, :, :10], q[:, :, :10], q[:, :, :10], s3, s3, 1, (1, 1, 4))
    with pytest.raises(ValueError, match="variable_block_sizes"):
        V.b200_vsa(q, q, q, s3[:2], s3, 1, (1, 1, 4))
    with pytest.raises(ValueError, match="topk"):
        V.b200_vsa(q, q, q, s3, s3, 4, (1, 1, 4))
    with pytest.raises(ValueError, match="same shape as q"):
        V.b200_vsa(q, q, q, s3, s3, 1, (1, 1, 4), torch.randn(1, 1, 12, 4))
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        V.b200_vsa(q, q, q, s3, s3, 1, (1, 1, 4))
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        V.b200_sparse_attention(q, q, q, torch.zeros(1, 1, 3, 1, dtype=torch.int32), s3, block_size=(1, 1, 4))
    assert V.as_block_elements(2) == 8 and V.as_block_elements((4, 4, 4)) == 64
    assert V.triton_vsa is V.b200_vsa and V.helion_sparse_attention is V.b200_sparse_attention


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    import importlib
    import simple_vsa_b200._lib as L
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no other compute path"):
        L._load()
    importlib.reload(L)


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "simple_vsa_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("oracle form", ""), f"{f} mentions the oracle"


def test_compression_gate_shape_layout_and_argument_check():
    """Mirrors the reference's CompressionGate tests (tests/test_common.py:24-61): [B,S,dim] -> [B,H,S,D],
    and a ``ValueError`` containing "divisible" for a head count that does not divide dim."""
    import torch

    import simple_vsa_b200 as V
    torch.manual_seed(0)
    batch, heads, seq, head_dim = 2, 3, 12, 8
    layer = V.CompressionGate(dim=heads * head_dim, num_heads=heads)
    hidden = torch.randn(batch, seq, heads * head_dim)
    gate = layer(hidden)
    assert gate.shape == (batch, heads, seq, head_dim)
    # head h, token s, channel d of the gate is channel h*head_dim + d of the linear layer's output
    want = layer.to_gate_compress(hidden)
    assert torch.equal(gate[1, 2, 5], want[1, 5, 2 * head_dim:3 * head_dim])
    with pytest.raises(ValueError, match="divisible"):
        V.CompressionGate(dim=10, num_heads=3)


@pytest.mark.parametrize("bias", [True, False])
def test_compression_gate_is_dense_head_major_and_equals_the_linear_layer(bias):
    """The layer writes the gate in the dense [B,H,S,D] layout the kernels read (the reference returns a
    transposed view of Linear's output, vsa/common.py:326-328); values and all three gradients are those of the
    plain Linear + view + transpose."""
    import torch

    import simple_vsa_b200 as V
    torch.manual_seed(3)
    B, H, S, D = 2, 3, 10, 8
    layer = V.CompressionGate(H * D, H, bias=bias).double()
    x = torch.randn(B, S, H * D, dtype=torch.double, requires_grad=True)
    gate = layer(x)
    assert gate.is_contiguous() and gate.shape == (B, H, S, D)
    want = layer.to_gate_compress(x).view(B, S, H, D).transpose(1, 2)
    torch.testing.assert_close(gate, want, atol=1e-12, rtol=1e-12)
    w = torch.randn_like(gate)
    params = [x, layer.to_gate_compress.weight] + ([layer.to_gate_compress.bias] if bias else [])
    got = torch.autograd.grad((gate * w).sum(), params)
    ref = torch.autograd.grad((want * w).sum(), params)
    for a, b in zip(got, ref):
        torch.testing.assert_close(a, b, atol=1e-12, rtol=1e-12)
    # the parameters keep the reference's names, so its checkpoints load
    assert set(layer.state_dict()) == {"to_gate_compress.weight"} | ({"to_gate_compress.bias"} if bias else set())


def test_workspace_sizes_and_support_queries_need_no_gpu():
    import simple_vsa_b200._lib as L
    lib = L.lib
    BH, Lq, Lkv, D, be, tk = 80, 92160, 92160, 128, 64, 180
    Qb = Kb = Lq // be
    assert lib.vsa_workspace_bytes(0, BH, Lq, Lkv, D, be, tk, L.VSA_BF16) == BH * Qb * Kb * 2
    assert lib.vsa_workspace_bytes(1, BH, Lq, Lkv, D, be, tk, L.VSA_BF16) == BH * Qb * 4
    assert lib.vsa_workspace_bytes(2, BH, Lq, Lkv, D, be, tk, L.VSA_F32) == BH * Lq * 4
    assert lib.vsa_workspace_bytes(3, BH, Lq, Lkv, D, be, tk, L.VSA_BF16) == BH * Kb * 4
    assert lib.vsa_workspace_bytes(4, BH, Lq, Lkv, D, be, tk, L.VSA_BF16) == BH * Qb * tk * 4
    assert lib.vsa_workspace_bytes(5, BH, Lq, Lkv, D, be, tk, L.VSA_F16) == BH * Qb * D * 2
    assert lib.vsa_workspace_bytes(6, BH, Lq, Lkv, D, be, tk, L.VSA_BF16) == BH * Qb * tk * 8192 == \
        lib.vsa_sparse_bwd_ds_workspace_bytes(BH, Lq, be, tk)
    assert lib.vsa_workspace_bytes(6, 1, 1024, 1024, D, 256, 3, L.VSA_BF16) == 4 * 3 * 16 * 8192
    assert lib.vsa_workspace_bytes(9, BH, Lq, Lkv, D, be, tk, L.VSA_BF16) == -1
    assert lib.vsa_workspace_bytes(0, BH, Lq, Lkv, D, be, tk, 7) == -1
    assert lib.vsa_sparse_bwd_ds_workspace_bytes(1, 1024, 48, 3) == -1
    # the tensor path covers bf16 and fp16, head dim 128, block volume 64, 128 or 256
    assert lib.vsa_sparse_sharded_supported(128, 64, 180, L.VSA_BF16) == 1
    assert lib.vsa_sparse_sharded_supported(128, 128, 90, L.VSA_F16) == 1
    assert lib.vsa_sparse_sharded_supported(128, 192, 4, L.VSA_BF16) == 0
    assert lib.vsa_sparse_sharded_supported(128, 128, 513, L.VSA_BF16) == 0      # 1026 tiles: beyond the tile list
    assert lib.vsa_sparse_sharded_supported(64, 64, 4, L.VSA_BF16) == 0
    assert lib.vsa_sparse_bwd_ds_supported(128, 256, 20, L.VSA_BF16) == 1
    # kernel families: tcgen05 (2), warp-level tensor cores (1), CUDA cores (0)
    assert lib.vsa_sparse_kernel_family(128, 64, 180, L.VSA_BF16) == 2
    assert lib.vsa_sparse_kernel_family(128, 64, 1025, L.VSA_BF16) == 1      # more tiles than the tcgen05 list holds
    assert lib.vsa_sparse_kernel_family(64, 128, 8, L.VSA_F16) == 1
    assert lib.vsa_sparse_kernel_family(64, 64, 8, L.VSA_F32) == 0
    assert lib.vsa_sparse_kernel_family(128, 32, 8, L.VSA_BF16) == 0
    assert lib.vsa_sparse_bwd_ds_supported(128, 64, 180, L.VSA_F32) == 0


def test_host_step_helpers():
    from simple_vsa_b200.host import _chunk_spans, _parse_cpulist
    for total, per in ((80, 4), (10, 4), (1, 8), (7, 3), (40, 40)):
        spans = _chunk_spans(total, per)
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(hi - lo for lo, hi in spans) <= max(1, min(per, total))
    assert _parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert _parse_cpulist("") == set()
