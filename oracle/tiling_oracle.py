"""CPU restatement of the reference's 3-D tiling metadata.  TEST INFRASTRUCTURE ONLY.

Follows vsa/fastvideo_tiling.py of the reference: tile-contiguous ordering of raster token ids
(:22-43), its inverse (:46-53), valid tokens per tile (:56-79), flat indices of the real slots in
the padded layout (:82-89), and the tile / untile moves (:128-145).  Plain numpy loops; pinned by
tests/golden/tiling_*.npz, which tests/golden/make_golden.py produced with the reference itself.
"""

import math

import numpy as np


def metadata(shape, tile):
    T, H, W = shape
    ts, hs, ws = tile
    ids = np.arange(T * H * W).reshape(T, H, W)
    order, sizes = [], []
    for t in range(math.ceil(T / ts)):
        for h in range(math.ceil(H / hs)):
            for w in range(math.ceil(W / ws)):
                block = ids[t * ts:(t + 1) * ts, h * hs:(h + 1) * hs, w * ws:(w + 1) * ws].reshape(-1)
                order.append(block)
                sizes.append(block.size)
    order = np.concatenate(order)
    sizes = np.array(sizes, dtype=np.int64)
    be = ts * hs * ws
    non_pad = np.concatenate([b * be + np.arange(n) for b, n in enumerate(sizes)])
    return {"tile_partition_indices": order, "reverse_tile_partition_indices": np.argsort(order),
            "variable_block_sizes": sizes, "non_pad_index": non_pad,
            "num_tiles": (math.ceil(T / ts), math.ceil(H / hs), math.ceil(W / ws)), "max_block_size": be}


def tile(x, meta):
    nb = int(np.prod(meta["num_tiles"]))
    out = np.zeros((x.shape[0], nb * meta["max_block_size"]) + x.shape[2:], dtype=x.dtype)
    out[:, meta["non_pad_index"]] = x[:, meta["tile_partition_indices"]]
    return out


def untile(x, meta):
    return x[:, meta["non_pad_index"]][:, meta["reverse_tile_partition_indices"]]
