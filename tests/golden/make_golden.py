"""Generate the golden vectors under tests/golden from the reference project itself.

Run once in a container where the reference checkout is importable:

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

It imports the reference's own ``vsa`` package (never this repository's code
for the values it stores), runs it on the seeded inputs of ``cases.py`` and
writes one compressed ``.npz`` per case.  The tests then check the oracle, and
on a GPU the CUDA kernels, against these files; the reference checkout is not
needed at test time.
"""

from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import vsa as ref                                      # the reference package
from vsa import common as ref_common
from vsa import torch_impl as ref_torch

from tests.golden.cases import SPARSE_CASES, VSA_CASES, sparse_inputs, to_np, vsa_inputs

ROW_STRIDE_BIG = 8      # gradients of the 1024-token case are stored every 8th row


def _be(block_size):
    return ref_common._as_block_elements(block_size)


def make_vsa(name, case):
    q, k, v, gate, dout, sizes = vsa_inputs(case)
    be = _be(case["block_size"])
    scale = 1.0 / math.sqrt(q.shape[-1])
    leaves = [t.clone().requires_grad_(case["grad"]) for t in (q, k, v)]
    g = gate.clone().requires_grad_(case["grad"]) if gate is not None else None
    out = ref.torch_vsa(*leaves, sizes, sizes, case["topk"], case["block_size"], g)
    rec = {"out": to_np(out)}
    scores, out_c_blocks = ref_common.coarse_branch_compact(q, k, v, sizes, sizes, be, scale)
    rec["scores"] = to_np(scores)
    rec["out_c_blocks"] = to_np(out_c_blocks)
    rec["selected"] = scores.topk(case["topk"], dim=-1).indices.numpy().astype(np.int32)
    for tag, x in (("q", q), ("k", k), ("v", v)):
        rec["mean_" + tag] = to_np(ref_common.block_mean(x, sizes, be))
    if q.shape[2] <= 32 or name.startswith("c1"):
        dense, aux = ref.video_sparse_attn(q, k, v, sizes, sizes, case["topk"],
                                           block_size=case["block_size"],
                                           compress_attn_weight=gate, return_aux=True)
        rec["out_dense"] = to_np(dense)
        rec["out_sparse"] = to_np(aux["out_sparse"])
    if case["grad"]:
        out.backward(dout)
        stride = ROW_STRIDE_BIG if q.shape[2] >= 1024 else 1
        rec["grad_row_stride"] = np.int32(stride)
        for tag, leaf in zip(("dq", "dk", "dv"), leaves):
            rec[tag] = to_np(leaf.grad)[:, :, ::stride]
        if g is not None:
            rec["dgate"] = to_np(g.grad)[:, :, ::stride]
    # fingerprint of the inputs so that a drift of the random generator is detected
    rec["input_sum"] = np.float64(q.double().sum() + 2 * k.double().sum() + 3 * v.double().sum())
    np.savez_compressed(os.path.join(HERE, f"vsa_{name}.npz"), **rec)
    print("wrote", name, {k_: getattr(v_, "shape", None) for k_, v_ in rec.items()})


def make_sparse(name, case):
    q, k, v, dout, sizes, selected = sparse_inputs(case)
    be = case["be"]
    B, H, L, D = q.shape
    Qb = L // be
    scale = 1.0 / math.sqrt(D)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    ql, kl, vl = leaves
    ids = selected.long()
    # the reference's own gather + mask helpers, composed as its fine branch composes them
    kg = ref_torch._gather_blocks(kl, ids, be).float()
    vg = ref_torch._gather_blocks(vl, ids, be).float()
    ok = ref_common._valid_token_mask(sizes, be)[ids]
    qq = ql.reshape(B, H, Qb, be, D).float()
    s = torch.einsum("bhqtd,bhqksd->bhqtks", qq, kg) * scale
    s = s.masked_fill(~ok[:, :, :, None, :, :], float("-inf"))
    p = torch.softmax(s.flatten(-2), dim=-1)
    out = torch.einsum("bhqtn,bhqnd->bhqtd", p, vg.flatten(3, 4)).reshape(B, H, L, D)
    out.backward(dout.float())
    rec = {"out_s": to_np(out),
           "lse2": to_np(torch.logsumexp(s.flatten(-2), dim=-1).reshape(B, H, L) * 1.4426950408889634),
           "dq": to_np(ql.grad), "dk": to_np(kl.grad), "dv": to_np(vl.grad),
           "input_sum": np.float64(q.double().sum() + 2 * k.double().sum() + 3 * v.double().sum())}
    np.savez_compressed(os.path.join(HERE, f"sparse_{name}.npz"), **rec)
    print("wrote", name)


def make_block_mean():
    torch.manual_seed(11)
    x = torch.randn(1, 2, 3 * 64, 128).to(torch.bfloat16)
    sizes = torch.tensor([64, 37, 11])
    grad = torch.randn(1, 2, 3, 128).to(torch.bfloat16)
    leaf = x.clone().requires_grad_()
    out = ref_common.block_mean(leaf, sizes, 64)
    out.backward(grad)
    np.savez_compressed(os.path.join(HERE, "block_mean_64_37_11.npz"),
                        out=to_np(out), dx=to_np(leaf.grad),
                        input_sum=np.float64(x.double().sum()))
    print("wrote block_mean")


if __name__ == "__main__" and "--tiling-only" not in sys.argv:
    torch.set_num_threads(8)
    for n, c in VSA_CASES.items():
        make_vsa(n, c)
    for n, c in SPARSE_CASES.items():
        make_sparse(n, c)
    make_block_mean()


def make_tiling():
    from vsa import build_vsa_metadata, tile as ref_tile, untile as ref_untile
    for shape, tsz in (((3, 5, 5), (2, 4, 4)), ((2, 6, 6), (2, 3, 3)), ((5, 9, 7), (4, 4, 4))):
        meta = build_vsa_metadata(shape, tile_size=tsz, device="cpu")
        seq = math.prod(shape)
        x = torch.arange(2 * seq * 3, dtype=torch.float32).reshape(2, seq, 3)
        nb = math.prod(meta["num_tiles"])
        tiled = ref_tile(x, meta["tile_partition_indices"], meta["non_pad_index"], nb, meta["max_block_size"])
        back = ref_untile(tiled, meta["non_pad_index"], meta["reverse_tile_partition_indices"])
        name = "tiling_%dx%dx%d_%dx%dx%d.npz" % (shape + tsz)
        np.savez_compressed(os.path.join(HERE, name),
                            tile_partition_indices=meta["tile_partition_indices"].numpy(),
                            reverse_tile_partition_indices=meta["reverse_tile_partition_indices"].numpy(),
                            variable_block_sizes=meta["variable_block_sizes"].numpy(),
                            non_pad_index=meta["non_pad_index"].numpy(),
                            num_tiles=np.array(meta["num_tiles"]), max_block_size=np.int64(meta["max_block_size"]),
                            tiled=tiled.numpy(), untiled=back.numpy())
        print("wrote", name)


if __name__ == "__main__":
    make_tiling()
