"""Seeded input generators shared by the fixture maker and the tests.

Every case names its seed, shapes, block volume, per-block sizes and routing so
that the fixture maker (which runs the reference project) and the parity tests
(which run the oracle and the CUDA kernels) see bit-identical inputs.  Inputs
come from ``torch.manual_seed(seed)`` + ``torch.randn`` on the CPU generator.
"""

from __future__ import annotations

import numpy as np
import torch

_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}

# name -> dict(seed, shape [B,H,L,D], dtype, block_size, sizes (None = all full), topk, gate, grad)
VSA_CASES = {
    # the four tiny fp32 agreements the reference keeps between its gather and dense forms
    "ref_full_be4":   dict(seed=1, shape=(2, 2, 16, 16), dtype="f32", block_size=(1, 1, 4), sizes=None, topk=2, gate=False, grad=False),
    "ref_padded_be4": dict(seed=2, shape=(1, 2, 12, 16), dtype="f32", block_size=(1, 1, 4), sizes=[4, 2, 3], topk=2, gate=False, grad=False),
    "ref_gate_be4":   dict(seed=3, shape=(1, 2, 16, 16), dtype="f32", block_size=(1, 1, 4), sizes=None, topk=2, gate=True, grad=False),
    "ref_cube_be8":   dict(seed=4, shape=(1, 1, 24, 8), dtype="f32", block_size=2, sizes=None, topk=2, gate=False, grad=False),
    # the CPU-runnable headline configuration: fp32, 16 full blocks of 64, topk 4, forward + backward
    "c1_fp32_be64":   dict(seed=100, shape=(1, 2, 1024, 64), dtype="f32", block_size=(1, 1, 64), sizes=None, topk=4, gate=False, grad=True),
    # bf16, block 64, head dim 128, ragged blocks and a gate, forward + backward
    "bf16_be64_ragged_gate": dict(seed=21, shape=(1, 2, 256, 128), dtype="bf16", block_size=(1, 1, 64), sizes=[64, 41, 64, 19], topk=2, gate=True, grad=True),
    # bf16, logical block 256, ragged, forward + backward
    "bf16_be256_ragged": dict(seed=23, shape=(1, 1, 768, 128), dtype="bf16", block_size=(4, 8, 8), sizes=[256, 191, 73], topk=2, gate=False, grad=True),
    # fp16, tiny blocks of 8, head dim 64, ragged, gate: the shape of the reference's own fp16 GPU tests
    "f16_be8_ragged_gate": dict(seed=37, shape=(1, 2, 48, 64), dtype="f16", block_size=2, sizes=[8, 5, 8, 3, 8, 8], topk=2, gate=True, grad=True),
    # fp32 with head dim 128 and a gate, for the fp32 validation mode of the kernels
    "f32_be64_gate":  dict(seed=29, shape=(1, 1, 512, 128), dtype="f32", block_size=(4, 4, 4), sizes=[64, 64, 17, 64, 1, 64, 40, 64], topk=3, gate=True, grad=True),
}

# explicit-route fine attention: name -> dict(seed, shape, dtype, be, sizes, selected)
SPARSE_CASES = {
    "routes_be64": dict(seed=15, shape=(1, 2, 192, 128), dtype="bf16", be=64, sizes=None,
                        selected=[[0, 2], [1, 2], [0, 1]]),
    # every query block reads key block 0 only: the whole in-degree lands on one key row
    "hot_block0_be256": dict(seed=31, shape=(1, 1, 768, 128), dtype="bf16", be=256, sizes=[256, 173, 91],
                             selected=[[0], [0], [0]]),
    "routes_f32_be64": dict(seed=33, shape=(1, 1, 256, 64), dtype="f32", be=64, sizes=[64, 5, 64, 33],
                            selected=[[3, 1, 0], [2, 3, 1], [0, 1, 2], [1, 0, 3]]),
}


def torch_dtype(name: str) -> torch.dtype:
    return _DT[name]


def vsa_inputs(case: dict):
    """q, k, v, gate-or-None, upstream grad, kv sizes (int64) for a VSA case."""
    from oracle.vsa_oracle import block_elements

    torch.manual_seed(case["seed"])
    dt = _DT[case["dtype"]]
    shape = case["shape"]
    q = torch.randn(shape).to(dt)
    k = torch.randn(shape).to(dt)
    v = torch.randn(shape).to(dt)
    gate = torch.randn(shape).to(dt) if case["gate"] else None
    dout = torch.randn(shape).to(dt)
    be = block_elements(case["block_size"])
    nb = shape[2] // be
    sizes = torch.full((nb,), be, dtype=torch.long) if case["sizes"] is None \
        else torch.tensor(case["sizes"], dtype=torch.long)
    return q, k, v, gate, dout, sizes


def sparse_inputs(case: dict):
    """q, k, v, upstream grad, sizes and the [B,H,Qb,tk] routing table of a route-explicit case."""
    torch.manual_seed(case["seed"])
    dt = _DT[case["dtype"]]
    shape = case["shape"]
    B, H, L, D = shape
    q = torch.randn(shape).to(dt)
    k = torch.randn(shape).to(dt)
    v = torch.randn(shape).to(dt)
    dout = torch.randn(shape).to(dt)
    be = case["be"]
    nb = L // be
    sizes = torch.full((nb,), be, dtype=torch.long) if case["sizes"] is None \
        else torch.tensor(case["sizes"], dtype=torch.long)
    sel = torch.tensor(case["selected"], dtype=torch.int32)          # [Qb, tk]
    selected = sel[None, None].expand(B, H, -1, -1).contiguous()
    return q, k, v, dout, sizes, selected


def to_np(t: torch.Tensor) -> np.ndarray:
    """fp32 numpy copy (bf16/fp16 widen exactly)."""
    return t.detach().float().cpu().numpy()
