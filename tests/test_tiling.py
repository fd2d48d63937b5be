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
