"""Fused tensor-parallel FFN (peer stores over NVLink) against the NCCL path, on two GPUs.
Skipped on boxes with a single GPU.  Ranks leave only between steps; no kernel waits on a peer."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from sparseflow_b200 import ops, parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        H, I, M = 1024, 2816, 1000          # ragged M: the last owner's block is partly empty

        def seeded(shape, seed, sigma):
            g = torch.Generator().manual_seed(seed)
            return (torch.randn(shape, generator=g) * sigma).to(torch.bfloat16).to(dev)
        wg, wu, wd = seeded((I, H), 1, 0.02), seeded((I, H), 2, 0.02), seeded((H, I), 3, 0.02)
        x = seeded((M, H), 4, 1.0)
        ref = parallel.TensorParallelFFN(wg, wu, wd).forward(x).clone()
        fused = parallel.FusedTensorParallelFFN(wg, wu, wd, max_tokens=M, use_switch_stores=True)   # if the fabric has them
        a = fused.forward(x).clone()
        b = fused.forward(x).clone()
        plain = parallel.FusedTensorParallelFFN(wg, wu, wd, max_tokens=M)
        c = plain.forward(x).clone()
        torch.cuda.synchronize()
        assert ops.device_status() == 0 and plain.switch_out == 0
        err = (a.float() - ref.float()).abs().max().item()
        ret[rank] = (err <= 2.0 ** -7 * ref.float().abs().max().item(), torch.equal(a, b) and torch.equal(a, c))
        ret[f"switch{rank}"] = bool(fused.switch_out)
    finally:
        dist.destroy_process_group()


def test_fused_tp_matches_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        got = dict(ret)
        print("switch-replicated output mapping in use:", got.pop("switch0"), got.pop("switch1"))
        assert got == {0: (True, True), 1: (True, True)}
