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


def block_rows(M: int, tp: int) -> int:
    """Token rows per owner in a step of M tokens: ceil(M / tp) rounded up to 16 (the GEMM epilogue's store box)."""
    return -(-(-(-M // tp)) // 16) * 16


def owned_rows(M: int, tp: int, rank: int) -> Tuple[int, int]:
    """Half-open range of the token rows whose finished values `rank` computes in a step of M tokens
    (consecutive blocks of ``block_rows(M, tp)``; trailing ranks may own nothing when M is small)."""
    mo = block_rows(M, tp)
    return min(M, rank * mo), min(M, (rank + 1) * mo)


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
    """TP FFN whose exchange step runs in this library's own kernels over NVLink / NVSwitch.

    ``exchange="switch"`` (the default where the fabric offers switch-replicated mappings of symmetric memory):
    the down GEMM writes this rank's partial sums into its own copy of a symmetric buffer, then ONE kernel per
    rank does barrier -> in-switch reduction of its own token block (``multimem.ld_reduce``, fp32 accumulation) ->
    bias -> ``multimem.st`` of the finished block into every rank's output -> barrier.  Three launches per step.

    ``exchange="scatter"``: the down GEMM's epilogue TMA-stores each partial token block into the owning rank's
    receive slot (reduce-scatter fused into the GEMM), a second kernel sums the slots and writes the finished block
    to every rank with peer stores; two stream-ordered symmetric-memory barriers order them.  Needs no multicast
    mapping; kept for fabrics without one.

    The result of ``forward`` is a view of a symmetric buffer that peers write into: see ``forward``.
    """

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, max_tokens: int, group=None,
                 down_bias: Optional[torch.Tensor] = None, use_switch_stores: bool = False, exchange: str = "auto"):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib, ops
        self.C, self.ops, self.L = C, ops, _lib.lib()
        self.group = group if group is not None else dist.group.WORLD
        self.tp = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if not 2 <= self.tp <= 8:
            raise ValueError("fused tensor-parallel FFN needs 2..8 ranks")
        if exchange not in ("auto", "switch", "scatter"):
            raise ValueError("exchange must be 'auto', 'switch' or 'scatter'")
        self.I, self.H = gate.shape
        g, u, d = shard_ffn_weights(gate, up, down, self.tp, self.rank)
        self.Ip = g.shape[0]
        self.gu = ops.compress_gate_up(g, u)
        self.dn = ops.compress_weight(d)
        self.down_bias = down_bias
        self.dtype = gate.dtype
        dev = gate.device
        self.tok_per_owner = block_rows(max_tokens, self.tp)
        self.max_tokens = max_tokens
        Mo, H = self.tok_per_owner, self.H
        self.row_bytes = H * 2
        VP = C.c_void_p * 8
        self._VP = VP
        # the replicated output [tp * tok_per_owner, H]
        self.out = symm_mem.empty((self.tp * Mo, H), dtype=self.dtype, device=dev)
        self.h_out = symm_mem.rendezvous(self.out, self.group)
        self.out_ptrs = [int(p) for p in self.h_out.buffer_ptrs]
        self.mc_out = int(getattr(self.h_out, "multicast_ptr", 0) or 0)
        self.exchange = exchange
        if exchange == "auto":
            self.exchange = "switch" if self.mc_out else "scatter"
        if self.exchange == "switch":
            # partial sums of every rank (same offsets), the gathered activations, and the flag words
            self.partial = symm_mem.empty((self.tp * Mo, H), dtype=self.dtype, device=dev)
            self.h_partial = symm_mem.rendezvous(self.partial, self.group)
            self.mc_partial = int(getattr(self.h_partial, "multicast_ptr", 0) or 0)
            if not self.mc_out or not self.mc_partial:
                raise RuntimeError("exchange='switch' needs switch-replicated (multicast) symmetric memory")
            self.flags = symm_mem.empty((self.L.sfb200_tp_flag_words(),), dtype=torch.int32, device=dev)
            self.flags.zero_()
            self.h_flags = symm_mem.rendezvous(self.flags, self.group)
            self.peer_flags = VP(*[int(self.h_flags.buffer_ptrs[r]) if r < self.tp else None for r in range(8)])
            self.epoch = 0
            self.x_full = None       # symmetric copy of the activations, created by forward_from_shards
            torch.cuda.synchronize(dev)
            dist.barrier(self.group)           # every rank's flags are zero before anyone signals
        else:
            # receive slots [source rank][tok_per_owner, H]
            self.recv = symm_mem.empty((self.tp, Mo, H), dtype=self.dtype, device=dev)
            self.h_recv = symm_mem.rendezvous(self.recv, self.group)
            self.recv_ptrs = [int(p) for p in self.h_recv.buffer_ptrs]
            # Optional: the all-gather half through NVSwitch-replicated stores.  Off by default: the 16-byte
            # switch stores measured slower than plain peer stores at 2 ranks (0.059 vs 0.037 ms) and at 4.
            self.switch_out_base = self.mc_out if use_switch_stores else 0
        self.switch_out = self.mc_out if (self.exchange == "switch" or use_switch_stores) else 0
        self.hidden = torch.empty((max_tokens, self.Ip), dtype=self.dtype, device=dev)
        self.kernel_launches = 0

    def owned_rows(self, M: int) -> Tuple[int, int]:
        """Half-open range of the token rows whose finished values THIS rank computes in a step of M tokens."""
        return owned_rows(M, self.tp, self.rank)

    def forward_from_shards(self, x_rows: torch.Tensor, M: int) -> torch.Tensor:
        """Like ``forward``, but every rank passes only the rows ``owned_rows(M)`` of the activations (e.g. the
        part of the batch it uploaded itself); the rows are replicated to all ranks through the switch
        (``multimem.st``) inside this call.  ``exchange="switch"`` only."""
        if self.exchange != "switch":
            raise RuntimeError("forward_from_shards needs exchange='switch'")
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        if self.x_full is None:
            self.x_full = symm_mem.empty((self.tp * self.tok_per_owner, self.H), dtype=self.dtype, device=self.out.device)
            self.h_x = symm_mem.rendezvous(self.x_full, self.group)
            self.mc_x = int(getattr(self.h_x, "multicast_ptr", 0) or 0)
            if not self.mc_x:
                raise RuntimeError("no switch-replicated mapping for the activations")
        if M > self.max_tokens:
            raise ValueError(f"{M} tokens exceed the {self.max_tokens} this instance was built for")
        lo, hi = self.owned_rows(M)
        if x_rows.shape != (hi - lo, self.H) or not x_rows.is_contiguous():
            raise ValueError(f"rank {self.rank} must pass its rows [{lo}, {hi}) as a contiguous [{hi - lo}, {self.H}] tensor")
        mo = block_rows(M, self.tp)
        self.epoch += 1
        # every rank launches, also one whose block is empty (M much smaller than tp * 16): the kernel's two
        # barriers are part of the protocol
        src = x_rows.data_ptr() if hi > lo else self.x_full.data_ptr()
        rc = self.L.sfb200_tp_allgather_switch(src, self.mc_x + self.rank * mo * self.row_bytes, hi - lo, self.H,
                                               self.C.cast(self.peer_flags, self.C.POINTER(self.C.c_void_p)),
                                               self.tp, self.rank, self.epoch, self.ops._stream())
        _lib.check("sfb200_tp_allgather_switch", rc)
        self.kernel_launches += 1
        return self.forward(self.x_full[:M])

    def forward(self, x: torch.Tensor, phase_events=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns the FFN output [M, H] (identical on every rank).

        Without ``out`` the result is a VIEW of this instance's symmetric output buffer: it is valid until
        the next ``forward`` of this instance on ANY rank (peers write into it through NVLink), so consume
        it on the same stream before calling again, or pass ``out`` (a tensor of shape [M, H]) to receive a
        private copy.  ``phase_events``: optional list that receives CUDA events bracketing the phases of
        the step for per-phase timing (gate|up GEMM, down GEMM, then the exchange: one phase with
        ``exchange="switch"``, barrier / reduce + all-gather / barrier with ``"scatter"``)."""
        from . import _lib
        ops, L, C = self.ops, self.L, self.C
        M = x.shape[0]
        if M > self.max_tokens:
            raise ValueError(f"{M} tokens exceed the {self.max_tokens} this instance was built for")
        st = ops._stream()
        dt = ops._dt(x)
        hidden = self.hidden[:M]
        # rows per owner for THIS call: with the switch exchange a small batch pays a small exchange; the scatter
        # path keeps the receive slots' fixed pitch
        mo = block_rows(M, self.tp) if self.exchange == "switch" else self.tok_per_owner
        blk = mo * self.row_bytes

        def mark():
            if phase_events is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                phase_events.append(e)
        bias = self.down_bias.data_ptr() if self.down_bias is not None else None
        mark()
        ops.sparse_gemm_swiglu(x, self.gu, out=hidden)
        mark()
        if self.exchange == "switch":
            ops.sparse_gemm(hidden, self.dn, out=self.partial[:M])
            mark()
            self.epoch += 1
            _lib.check("sfb200_tp_allreduce_switch", L.sfb200_tp_allreduce_switch(
                self.mc_partial + self.rank * blk, self.mc_out + self.rank * blk, mo, self.H, dt, bias,
                C.cast(self.peer_flags, C.POINTER(C.c_void_p)), self.tp, self.rank, self.epoch, st))
            mark()
        else:
            VP = self._VP
            # rank o's slot for my partial sums; rank d's output rows of my token block
            slot = self.tok_per_owner * self.row_bytes
            peer_slots = VP(*[(self.recv_ptrs[o] + self.rank * slot) if o < self.tp else None for o in range(8)])
            peer_out = VP(*[(self.out_ptrs[d] + self.rank * blk) if d < self.tp else None for d in range(8)])
            _lib.check("sfb200_sparse_gemm_scatter", L.sfb200_sparse_gemm_scatter(
                hidden.data_ptr(), hidden.stride(0), self.dn.values.data_ptr(), self.dn.meta.data_ptr(),
                C.cast(peer_slots, C.POINTER(C.c_void_p)), self.tp, mo, M, self.H, self.Ip, dt, st))
            mark()
            self.h_recv.barrier(channel=0)            # every rank's partial sums have landed
            mark()
            if self.switch_out_base:
                _lib.check("sfb200_reduce_allgather_switch", L.sfb200_reduce_allgather_switch(
                    self.recv.data_ptr(), self.tp, mo, self.H, self.switch_out_base + self.rank * blk, dt, bias, st))
            else:
                _lib.check("sfb200_reduce_allgather", L.sfb200_reduce_allgather(
                    self.recv.data_ptr(), self.tp, mo, self.H, C.cast(peer_out, C.POINTER(C.c_void_p)), dt, bias, st))
            mark()
            self.h_out.barrier(channel=0)             # every rank's finished block has landed everywhere
            mark()
        self.kernel_launches += 3      # own kernels per step (the scatter path's two barriers are torch's)
        res = self.out[:M]
        if out is not None:
            out.copy_(res)
            return out
        return res
