"""Sequence-parallel VSA over NCCL on two (and, where four GPUs are visible, four) ranks against the single-GPU
operator.  NVLS is switched off for these child processes and no kernel reads a peer's memory."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import simple_vsa_b200 as V
        from simple_vsa_b200 import _lib
        from simple_vsa_b200.parallel import sequence_parallel_vsa
        torch.manual_seed(77)
        B, H, L, D, be, tk = 1, 3, 2048, 128, 64, 6
        q, k, v, gate, dout = (torch.randn(B, H, L, D).to(torch.bfloat16) for _ in range(5))
        sizes = torch.full((L // be,), be)
        sizes[7] = 21
        l = L // world
        sl = slice(rank * l, (rank + 1) * l)
        nbl = l // be
        leaves = [t[:, :, sl].to(dev).requires_grad_() for t in (q, k, v, gate)]
        out = sequence_parallel_vsa(leaves[0], leaves[1], leaves[2], sizes, sizes[rank * nbl:(rank + 1) * nbl], tk,
                                    (4, 4, 4), leaves[3])
        out.backward(dout[:, :, sl].to(dev))
        full = [t.to(dev).requires_grad_() for t in (q, k, v, gate)]
        want = V.b200_vsa(full[0], full[1], full[2], sizes, sizes, tk, (4, 4, 4), full[3])
        want.backward(dout.to(dev))
        torch.testing.assert_close(out.float(), want[:, :, sl].float(), atol=1e-2, rtol=1e-2)
        for got, ref in zip(leaves, full):
            torch.testing.assert_close(got.grad.float(), ref.grad[:, :, sl].float(), atol=3e-2, rtol=3e-2)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sequence_parallel_matches_single_gpu(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
