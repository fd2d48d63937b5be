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
