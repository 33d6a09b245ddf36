"""Tensor-parallel gated FFN: column-parallel gate/up, row-parallel down, one all-reduce.

The reference has no distributed code; this is the sharding its FFN admits.  Rank r of tp keeps
rows [r*I/tp, (r+1)*I/tp) of W_gate and W_up and the matching COLUMNS of W_down (a K slice).  2:4
groups run along K: for gate/up K = H is untouched by the split; for down the slice boundaries are
multiples of 4, so pruning a shard equals sharding the pruned matrix.  Each rank produces a partial
out_r[M, H]; their sum (NCCL all-reduce over NVLink) is the FFN output.  Shards whose width is not
a multiple of 64 are zero-padded (zero gate/up rows give hidden == 0, zero down columns add 0).

Two implementations of the exchange step:
* ``TensorParallelFFN``: down GEMM, then NCCL all-reduce (the baseline);
* ``FusedTensorParallelFFN``: the down GEMM's epilogue TMA-stores each partial token block straight
  into the owning rank's receive slot over NVLink (reduce-scatter fused into the GEMM), then one
  kernel sums the slots in fp32 and writes the finished block into every rank's output (all-gather
  fused into the reduction).  Buffers are torch symmetric memory; ranks are ordered by its
  stream-ordered barrier between the two kernels, so no kernel ever waits on another GPU.

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


class FusedTensorParallelFFN:
    """TP FFN whose exchange step is fused into the kernels (peer stores over NVLink)."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, max_tokens: int, group=None,
                 down_bias: Optional[torch.Tensor] = None, use_switch_stores: bool = False):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib, ops
        self.C, self.ops, self.L = C, ops, _lib.lib()
        self.group = group if group is not None else dist.group.WORLD
        self.tp = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if not 2 <= self.tp <= 8:
            raise ValueError("fused tensor-parallel FFN needs 2..8 ranks")
        self.I, self.H = gate.shape
        g, u, d = shard_ffn_weights(gate, up, down, self.tp, self.rank)
        self.Ip = g.shape[0]
        self.gu = ops.compress_gate_up(g, u)
        self.dn = ops.compress_weight(d)
        self.down_bias = down_bias
        self.dtype = gate.dtype
        dev = gate.device
        self.tok_per_owner = -(-(-(-max_tokens // self.tp)) // 16) * 16
        self.max_tokens = max_tokens
        Mo, H = self.tok_per_owner, self.H
        # receive slots [source rank][tok_per_owner, H] and the replicated output [tp * tok_per_owner, H]
        self.recv = symm_mem.empty((self.tp, Mo, H), dtype=self.dtype, device=dev)
        self.out = symm_mem.empty((self.tp * Mo, H), dtype=self.dtype, device=dev)
        self.h_recv = symm_mem.rendezvous(self.recv, self.group)
        self.h_out = symm_mem.rendezvous(self.out, self.group)
        blk = Mo * H * self.recv.element_size()
        VP = C.c_void_p * 8
        recv_ptrs = [int(p) for p in self.h_recv.buffer_ptrs]
        out_ptrs = [int(p) for p in self.h_out.buffer_ptrs]
        # rank o's slot for my partial sums; rank d's output rows of my token block
        self.peer_slots = VP(*[(recv_ptrs[o] + self.rank * blk) if o < self.tp else None for o in range(8)])
        self.peer_out = VP(*[(out_ptrs[d] + self.rank * blk) if d < self.tp else None for d in range(8)])
        # Optional: NVSwitch-replicated mapping of the output, when the fabric offers one; the all-gather then sends
        # each finished block once (multimem.st) instead of once per peer.  Off by default: the 16-byte switch
        # stores measured slower than plain peer stores at 2 ranks (0.059 vs 0.037 ms) and at 4 (0.057 vs 0.051 ms).
        mc = int(getattr(self.h_out, "multicast_ptr", 0) or 0) if use_switch_stores else 0
        self.switch_out = (mc + self.rank * blk) if mc else 0
        self.hidden = torch.empty((max_tokens, self.Ip), dtype=self.dtype, device=dev)
        self.kernel_launches = 0

    def forward(self, x: torch.Tensor, phase_events=None) -> torch.Tensor:
        """``phase_events``: optional list that receives six CUDA events bracketing the five phases of the step
        (gate|up GEMM, down GEMM + scatter, barrier, reduce + all-gather, barrier) for per-phase timing."""
        from . import _lib
        ops, L, C = self.ops, self.L, self.C
        M = x.shape[0]
        if M > self.max_tokens:
            raise ValueError(f"{M} tokens exceed the {self.max_tokens} this instance was built for")
        st = ops._stream()
        dt = ops._dt(x)
        hidden = self.hidden[:M]

        def mark():
            if phase_events is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                phase_events.append(e)
        mark()
        ops.sparse_gemm_swiglu(x, self.gu, out=hidden)
        mark()
        _lib.check("sfb200_sparse_gemm_scatter", L.sfb200_sparse_gemm_scatter(
            hidden.data_ptr(), hidden.stride(0), self.dn.values.data_ptr(), self.dn.meta.data_ptr(),
            C.cast(self.peer_slots, C.POINTER(C.c_void_p)), self.tp, self.tok_per_owner, M, self.H, self.Ip, dt, st))
        mark()
        self.h_recv.barrier(channel=0)            # every rank's partial sums have landed
        mark()
        bias = self.down_bias.data_ptr() if self.down_bias is not None else None
        if self.switch_out:
            _lib.check("sfb200_reduce_allgather_switch", L.sfb200_reduce_allgather_switch(
                self.recv.data_ptr(), self.tp, self.tok_per_owner, self.H, self.switch_out, dt, bias, st))
        else:
            _lib.check("sfb200_reduce_allgather", L.sfb200_reduce_allgather(
                self.recv.data_ptr(), self.tp, self.tok_per_owner, self.H,
                C.cast(self.peer_out, C.POINTER(C.c_void_p)), dt, bias, st))
        mark()
        self.h_out.barrier(channel=0)             # every rank's finished block has landed everywhere
        mark()
        self.kernel_launches += 3
        return self.out[:M]
