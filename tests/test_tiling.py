"""Tiling front end: metadata against the reference's vectors (CPU), the gather kernel on a GPU."""

import glob
import math
import os
import re

import numpy as np
import pytest
import torch

from oracle import tiling_oracle as TO

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
FILES = sorted(glob.glob(os.path.join(GOLDEN, "tiling_*.npz")))


def _case(path):
    m = re.search(r"tiling_(\d+)x(\d+)x(\d+)_(\d+)x(\d+)x(\d+)", path)
    v = [int(g) for g in m.groups()]
    return tuple(v[:3]), tuple(v[3:]), dict(np.load(path))


@pytest.mark.parametrize("path", FILES)
def test_metadata_matches_reference_vectors(path):
    from simple_vsa_b200 import build_vsa_metadata
    shape, tsz, gold = _case(path)
    meta = build_vsa_metadata(shape, tile_size=tsz, device="cpu")
    ora = TO.metadata(shape, tsz)
    for key in ("tile_partition_indices", "reverse_tile_partition_indices", "variable_block_sizes", "non_pad_index"):
        np.testing.assert_array_equal(ora[key], gold[key])
        np.testing.assert_array_equal(meta[key].numpy(), gold[key])
    assert tuple(meta["num_tiles"]) == tuple(gold["num_tiles"].tolist()) == tuple(ora["num_tiles"])
    assert meta["max_block_size"] == int(gold["max_block_size"]) == ora["max_block_size"]
    seq = math.prod(shape)
    x = np.arange(2 * seq * 3, dtype=np.float32).reshape(2, seq, 3)
    np.testing.assert_array_equal(TO.tile(x, ora), gold["tiled"])
    np.testing.assert_array_equal(TO.untile(gold["tiled"], ora), gold["untiled"])
    # the int32 row maps are consistent with the index tensors
    tm = meta["tile_map"].numpy()
    assert (tm >= 0).sum() == seq and np.array_equal(tm[gold["non_pad_index"]], gold["tile_partition_indices"])
    assert np.array_equal(meta["untile_map"].numpy(), gold["non_pad_index"][gold["reverse_tile_partition_indices"]])
    assert int(meta["variable_block_sizes"].sum()) == seq


@pytest.mark.gpu
@pytest.mark.parametrize("path", FILES)
@pytest.mark.parametrize("dtype,width", [(torch.float32, 3), (torch.bfloat16, 128), (torch.bfloat16, 5)])
def test_tile_untile_kernel(path, dtype, width):
    from simple_vsa_b200 import build_vsa_metadata, tile, tile_with, untile, untile_with
    shape, tsz, gold = _case(path)
    meta = build_vsa_metadata(shape, tile_size=tsz, device="cuda:0")
    ora = TO.metadata(shape, tsz)
    seq = math.prod(shape)
    torch.manual_seed(3)
    x = torch.randn(2, seq, width).to(dtype)
    want = TO.tile(x.float().numpy(), ora)
    nb = math.prod(meta["num_tiles"])
    got = tile(x.cuda(), meta["tile_partition_indices"], meta["non_pad_index"], nb, meta["max_block_size"])
    np.testing.assert_array_equal(got.float().cpu().numpy(), want)
    assert torch.equal(tile_with(meta, x.cuda()), got)
    back = untile(got, meta["non_pad_index"], meta["reverse_tile_partition_indices"])
    assert torch.equal(back.cpu(), x) and torch.equal(untile_with(meta, got).cpu(), x)
    if width == 3 and dtype == torch.float32:
        y = torch.arange(2 * seq * 3, dtype=torch.float32).reshape(2, seq, 3).cuda()
        np.testing.assert_array_equal(tile_with(meta, y).cpu().numpy(), gold["tiled"])


@pytest.mark.parametrize("path", FILES[:2])
def test_tile_untile_on_cpu_tensors_follow_the_reference_expressions(path):
    """Tensors that are not on a GPU go through plain index operations: same values as the reference-made
    vectors, and autograd flows through them."""
    from simple_vsa_b200 import build_vsa_metadata, tile, tile_with, untile, untile_with
    shape, tsz, gold = _case(path)
    meta = build_vsa_metadata(shape, tile_size=tsz, device="cpu")
    seq = math.prod(shape)
    x = torch.arange(2 * seq * 3, dtype=torch.float32).reshape(2, seq, 3).requires_grad_()
    nb = math.prod(meta["num_tiles"])
    tiled = tile(x, meta["tile_partition_indices"], meta["non_pad_index"], nb, meta["max_block_size"])
    np.testing.assert_array_equal(tiled.detach().numpy(), gold["tiled"])
    assert torch.equal(tile_with(meta, x), tiled)
    back = untile(tiled, meta["non_pad_index"], meta["reverse_tile_partition_indices"])
    np.testing.assert_array_equal(back.detach().numpy(), gold["untiled"])
    assert torch.equal(untile_with(meta, tiled), back)
    w = torch.randn_like(tiled)
    (tiled * w).sum().backward()
    assert torch.equal(x.grad, untile_with(meta, w))


@pytest.mark.gpu
@pytest.mark.parametrize("path", FILES)
def test_gradient_flows_through_tile_and_untile(path):
    """tile -> (anything) -> untile stays attached to the graph, and the gradients equal those of the index-op form
    (``vsa/fastvideo_tiling.py:128-145`` of the reference); padding rows receive no gradient from untile."""
    from simple_vsa_b200 import build_vsa_metadata, tile, tile_with, untile, untile_with
    shape, tsz, _ = _case(path)
    meta = build_vsa_metadata(shape, tile_size=tsz, device="cuda:0")
    seq = math.prod(shape)
    nb = math.prod(meta["num_tiles"])
    torch.manual_seed(5)
    x = torch.randn(2, seq, 2, 16, device="cuda:0")
    w = torch.randn(2, nb * meta["max_block_size"], 2, 16, device="cuda:0")
    tpi, npi, rev = meta["tile_partition_indices"], meta["non_pad_index"], meta["reverse_tile_partition_indices"]

    def reference_form(x_):
        buf = torch.zeros_like(w)
        buf[:, npi] = x_[:, tpi]
        y = (buf * w).tanh()
        return y[:, npi][:, rev]

    for variant in ("explicit", "cached"):
        a = x.clone().requires_grad_()
        if variant == "explicit":
            y = untile((tile(a, tpi, npi, nb, meta["max_block_size"]) * w).tanh(), npi, rev)
        else:
            y = untile_with(meta, (tile_with(meta, a) * w).tanh())
        b = x.clone().requires_grad_()
        z = reference_form(b)
        assert torch.equal(y, z)
        g = torch.randn_like(y)
        y.backward(g)
        z.backward(g)
        assert torch.equal(a.grad, b.grad)
    # the gradient of untile alone puts zeros on the padding rows
    t = torch.randn_like(w).requires_grad_()
    untile_with(meta, t).sum().backward()
    pad = torch.ones(w.shape[1], dtype=torch.bool, device="cuda:0")
    pad[npi] = False
    assert float(t.grad[:, pad].abs().sum()) == 0.0 and float(t.grad[:, ~pad].min()) == 1.0


# ---------------------------------------------------------------------------------------------
# the operator on raster-order [B,S,H,D] tensors (layout moves folded into the kernels' stores)
# ---------------------------------------------------------------------------------------------
def _two_step(V, meta, q, k, v, gate, topk, tile_size):
    """tile -> transpose -> operator -> transpose -> untile, the form a DiT layer writes around the operator."""
    to_tiles = lambda x: V.tile_with(meta, x).transpose(1, 2).contiguous()
    sizes = meta["variable_block_sizes"]
    out_t = V.b200_vsa(to_tiles(q), to_tiles(k), to_tiles(v), sizes, sizes, topk, tile_size,
                       to_tiles(gate) if gate is not None else None)
    return V.untile_with(meta, out_t.transpose(1, 2).contiguous())


@pytest.mark.gpu
@pytest.mark.parametrize("grid,tile_size,dtype", [((6, 10, 9), (4, 4, 4), torch.bfloat16),
                                                  ((8, 8, 8), (4, 4, 4), torch.float16),
                                                  ((5, 16, 12), (4, 8, 8), torch.bfloat16),
                                                  ((4, 9, 16), (2, 8, 8), torch.bfloat16)])
@pytest.mark.parametrize("with_gate", [False, True])
def test_raster_order_operator_equals_the_two_step_form(grid, tile_size, dtype, with_gate):
    """Clipped tiles on every axis, full tiles, blocks of 64 / 128 / 256 tokens: out, dq and dgate bit for bit (same
    kernels, same arithmetic, other store addresses); dk/dv up to the order of the fp32 sums over CSR rows."""
    import simple_vsa_b200 as V
    dev = "cuda:0"
    torch.manual_seed(11)
    B, H, D, topk = 2, 3, 128, 3
    S = grid[0] * grid[1] * grid[2]
    meta = V.build_vsa_metadata(grid, tile_size, device=dev)
    make = lambda: torch.randn(B, S, H, D, device=dev).to(dtype)
    q, k, v, dout = make(), make(), make(), make()
    gate = make() if with_gate else None
    a = [t.clone().requires_grad_() for t in (q, k, v)] + ([gate.clone().requires_grad_()] if with_gate else [])
    b = [t.clone().requires_grad_() for t in (q, k, v)] + ([gate.clone().requires_grad_()] if with_gate else [])
    out_a = V.video_sparse_attn_raster(a[0], a[1], a[2], meta, topk, a[3] if with_gate else None)
    out_b = _two_step(V, meta, b[0], b[1], b[2], b[3] if with_gate else None, topk, tile_size)
    assert out_a.shape == (B, S, H, D) and torch.isfinite(out_a.float()).all()
    assert torch.equal(out_a, out_b)
    out_a.backward(dout)
    out_b.backward(dout)
    assert torch.equal(a[0].grad, b[0].grad)
    if with_gate:
        assert torch.equal(a[3].grad, b[3].grad)
    for x, y in zip(a[1:3], b[1:3]):
        torch.testing.assert_close(x.grad.float(), y.grad.float(), atol=2e-2, rtol=2e-2)
    with torch.no_grad():                                    # the inference path (nothing saved) gives the same bits
        assert torch.equal(V.video_sparse_attn_raster(q, k, v, meta, topk, gate), out_a)


@pytest.mark.gpu
def test_raster_order_operator_other_shapes_take_the_two_step_form():
    """Head dim 64 is off the tensor path: the raster-order entry point still answers, through separate layout passes."""
    import simple_vsa_b200 as V
    dev = "cuda:0"
    torch.manual_seed(12)
    grid, tile_size, B, H, D, topk = (5, 6, 7), (4, 4, 4), 1, 2, 64, 2
    S = grid[0] * grid[1] * grid[2]
    meta = V.build_vsa_metadata(grid, tile_size, device=dev)
    q, k, v = (torch.randn(B, S, H, D, device=dev).to(torch.bfloat16).requires_grad_() for _ in range(3))
    out = V.video_sparse_attn_raster(q, k, v, meta, topk)
    ref = _two_step(V, meta, q.detach(), k.detach(), v.detach(), None, topk, tile_size)
    assert torch.equal(out, ref)
    out.float().square().mean().backward()
    assert all(t.grad is not None and torch.isfinite(t.grad.float()).all() for t in (q, k, v))


@pytest.mark.gpu
@pytest.mark.parametrize("D", [8, 24, 128])          # rows of 1, 3 (not a power of two: the general kernel) and 16 words
def test_tile_heads_is_tile_plus_transpose_in_one_pass(D):
    import simple_vsa_b200 as V
    dev = "cuda:0"
    torch.manual_seed(13)
    grid = (3, 5, 6)
    meta = V.build_vsa_metadata(grid, (2, 2, 4), device=dev)
    x = torch.randn(2, 90, 3, D, device=dev).to(torch.bfloat16).requires_grad_()
    got = V.tile_heads(x, meta)
    want = V.tile_with(meta, x.detach()).transpose(1, 2)
    assert got.is_contiguous() and torch.equal(got, want)
    assert torch.equal(V.untile_heads(got, meta), x)
    w = torch.randn_like(got)
    (got.float() * w.float()).sum().backward()
    assert torch.equal(x.grad, V.untile_heads(w, meta))
