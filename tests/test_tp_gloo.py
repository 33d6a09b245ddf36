"""Host logic of the tensor-parallel FFN, run as two gloo ranks on the CPU: sharding commutes
with pruning, padded shards are inert, and the all-reduced partial products equal the unsharded
oracle."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as o
from sparseflow_b200 import parallel


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dt = "bf16"
        H, I, M = 128, 208, 24                        # I/2 = 104: a multiple of 4 but not of 64 -> padded to 128
        g = torch.Generator().manual_seed(0)
        wg, wu = (torch.randn(I, H, generator=g) * 0.1 for _ in range(2))
        wd = torch.randn(H, I, generator=g) * 0.1
        x = torch.randn(M, H, generator=g)
        bits = lambda t: o.from_f32(t.numpy(), dt)
        g_r, u_r, d_r = parallel.shard_ffn_weights(wg, wu, wd, world, rank)
        lo, hi = parallel.shard_bounds(I, world, rank)
        assert g_r.shape == (128, H) and d_r.shape == (H, 128)
        # prune(shard) == shard(prune) for all three weights
        pg, pu, pd = (o.prune_24(bits(w), dt)["pruned"] for w in (wg, wu, wd))
        pg_r, pu_r, pd_r = (o.prune_24(bits(w), dt)["pruned"] for w in (g_r, u_r, d_r))
        w = hi - lo
        assert (pg_r[:w] == pg[lo:hi]).all() and (pu_r[:w] == pu[lo:hi]).all()
        assert (pd_r[:, :w] == pd[:, lo:hi]).all()
        assert (pg_r[w:] == 0).all() and (pd_r[:, w:] == 0).all()
        # local hidden slice and partial output, then the one exchange step
        xb = bits(x)
        h_r = o.from_f32(o.silu_mul_ref(o.gemm_ref(xb, pg_r, dt), o.gemm_ref(xb, pu_r, dt)), dt)
        part = torch.from_numpy(o.gemm_ref(h_r, pd_r, dt))
        dist.all_reduce(part)
        full = o.ffn_ref(xb, pg, pu, pd, dt, round_gate_up=False)
        np.testing.assert_allclose(part.numpy(), full["out_f32"], rtol=1e-4, atol=1e-4)
        # hidden slices reassemble to the unsharded hidden
        parts = [torch.zeros(M, 128, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(h_r.astype(np.int32)))
        hid = parallel.unshard_hidden(parts, I).numpy().astype(np.uint16)
        assert (hid == full["hidden"]).all()
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_tp_sharding_two_gloo_ranks():
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}


def test_shard_bounds_errors():
    import pytest
    with pytest.raises(ValueError):
        parallel.shard_bounds(11008, 3, 0)
    with pytest.raises(ValueError):
        parallel.shard_bounds(24, 4, 0)          # shards of 6 are not multiples of 4
    assert parallel.shard_bounds(11008, 8, 7) == (9632, 11008)
    assert parallel.padded_width(1376) == 1408 and parallel.padded_width(3584) == 3584


def test_token_blocks_partition_the_batch():
    """Owner blocks of the exchange step: multiples of 16 rows, consecutive, covering [0, M) exactly once."""
    for tp in (2, 4, 8):
        for M in (1, 15, 16, 17, 40, 100, 1000, 4096, 8191):
            mo = parallel.block_rows(M, tp)
            assert mo % 16 == 0 and mo * tp >= M and (mo - 16) * tp < M
            spans = [parallel.owned_rows(M, tp, r) for r in range(tp)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b and c <= d
