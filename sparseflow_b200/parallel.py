"""Tensor-parallel gated FFN: column-parallel gate/up, row-parallel down, one all-reduce.

The reference has no distributed code; this is the sharding its FFN admits.  Rank r of tp keeps
rows [r*I/tp, (r+1)*I/tp) of W_gate and W_up and the matching COLUMNS of W_down (a K slice).  2:4
groups run along K: for gate/up K = H is untouched by the split; for down the slice boundaries are
multiples of 4, so pruning a shard equals sharding the pruned matrix.  Each rank produces a partial
out_r[M, H]; their sum (NCCL all-reduce over NVLink) is the FFN output.  Shards whose width is not
a multiple of 64 are zero-padded (zero gate/up rows give hidden == 0, zero down columns add 0).

One process per GPU; torch.distributed carries the collective.  With ``chunks > 1`` the token
dimension is split and the all-reduce of chunk i overlaps the GEMMs of chunk i+1 on a second stream.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

PAD_TO = 64


def shard_bounds(I: int, tp: int, rank: int) -> Tuple[int, int]:
    """Half-open range of intermediate features owned by `rank`.  I must split into multiples of 4."""
    if I % tp != 0 or (I // tp) % 4 != 0:
        raise ValueError(f"intermediate size {I} does not split into {tp} shards that are multiples of 4")
    w = I // tp
    return rank * w, (rank + 1) * w


def padded_width(width: int) -> int:
    return -(-width // PAD_TO) * PAD_TO


def shard_ffn_weights(gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, tp: int, rank: int):
    """Return this rank's (gate_r, up_r, down_r), zero-padded to a multiple of 64 features.
    gate, up: [I, H]; down: [H, I]."""
    I, H = gate.shape
    lo, hi = shard_bounds(I, tp, rank)
    w, wp = hi - lo, padded_width(hi - lo)
    g = gate.new_zeros((wp, H))
    u = up.new_zeros((wp, H))
    d = down.new_zeros((H, wp))
    g[:w] = gate[lo:hi]
    u[:w] = up[lo:hi]
    d[:, :w] = down[:, lo:hi]
    return g, u, d


def unshard_hidden(parts: List[torch.Tensor], I: int) -> torch.Tensor:
    """Concatenate per-rank hidden slices (dropping padding) back to [M, I]."""
    tp = len(parts)
    w = I // tp
    return torch.cat([p[:, :w] for p in parts], dim=1)


class TensorParallelFFN:
    """Per-rank state of the TP FFN on the CUDA kernels."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, group=None,
                 chunks: int = 1, down_bias: Optional[torch.Tensor] = None):
        from . import ops
        self.ops = ops
        self.group = group
        self.tp = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.I, self.H = gate.shape
        g, u, d = shard_ffn_weights(gate, up, down, self.tp, self.rank)
        self.Ip = g.shape[0]
        self.gu = ops.compress_gate_up(g, u)
        self.dn = ops.compress_weight(d)
        self.down_bias = down_bias
        self.chunks = max(1, chunks)
        self.comm_stream = torch.cuda.Stream() if self.chunks > 1 else None
        self.kernel_launches = 0

    def forward(self, x: torch.Tensor, hidden: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops = self.ops
        M = x.shape[0]
        if hidden is None:
            hidden = torch.empty((M, self.Ip), dtype=x.dtype, device=x.device)
        if out is None:
            out = torch.empty((M, self.H), dtype=x.dtype, device=x.device)
        bias = self.down_bias if self.rank == 0 else None      # added once across the sum
        if self.chunks == 1 or self.tp == 1:
            ops.sparse_gemm_swiglu(x, self.gu, out=hidden)
            ops.sparse_gemm(hidden, self.dn, bias=bias, out=out)
            self.kernel_launches += 2
            if self.tp > 1:
                dist.all_reduce(out, group=self.group)
            return out
        main = torch.cuda.current_stream()
        step = -(-M // self.chunks)
        step = -(-step // 256) * 256
        for lo in range(0, M, step):
            hi = min(M, lo + step)
            ops.sparse_gemm_swiglu(x[lo:hi], self.gu, out=hidden[lo:hi])
            ops.sparse_gemm(hidden[lo:hi], self.dn, bias=bias, out=out[lo:hi])
            self.kernel_launches += 2
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                dist.all_reduce(out[lo:hi], group=self.group)
        main.wait_stream(self.comm_stream)
        return out
