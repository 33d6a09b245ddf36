"""Tensor-parallel gated FFN: column-parallel gate/up, row-parallel down, one all-reduce.

The reference has no distributed code; this is the sharding its FFN admits.  Rank r of tp keeps
rows [r*I/tp, (r+1)*I/tp) of W_gate and W_up and the matching COLUMNS of W_down (a K slice).  2:4
groups run along K: for gate/up K = H is untouched by the split; for down the slice boundaries are
multiples of 4, so pruning a shard equals sharding the pruned matrix.  Each rank produces a partial
out_r[M, H]; their sum (NCCL all-reduce over NVLink) is the FFN output.  Shards whose width is not
a multiple of 64 are zero-padded (zero gate/up rows give hidden == 0, zero down columns add 0).

Two implementations of the exchange step:
* ``TensorParallelFFN``: down GEMM, then NCCL all-reduce (the baseline);
* ``FusedTensorParallelFFN``: the down GEMM's epilogue stores each partial token block straight into the
  owning rank's receive slot over NVLink (reduce-scatter fused into the GEMM), then one kernel per rank
  sums the slots in fp32 and writes the finished block into every rank's output (all-gather fused into
  the reduction), with the ordering across ranks inside that kernel (flag words in symmetric memory,
  bounded polls).  Buffers are torch symmetric memory.

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
    """Per-rank state of the TP FFN on the CUDA kernels, the exchange being one NCCL all-reduce of the down GEMM's
    output: of the 16-bit output (``partial_dtype="16bit"``, the usual baseline: every rank's partial sum is rounded
    before the sum) or, unchunked, of fp32 partial sums that are rounded once after the sum (``"fp32"``: twice the bytes
    on the wire, the single-GPU error bound)."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, group=None,
                 chunks: int = 1, down_bias: Optional[torch.Tensor] = None, partial_dtype: str = "16bit"):
        from . import ops
        if partial_dtype not in ("16bit", "fp32"):
            raise ValueError("partial_dtype must be '16bit' or 'fp32'")
        if partial_dtype == "fp32" and chunks > 1:
            raise ValueError("fp32 partial sums are not chunked")
        self.partial_f32 = partial_dtype == "fp32"
        self._partial = None
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
        if self.partial_f32 and self.tp > 1:
            from . import _lib
            ops.sparse_gemm_swiglu(x, self.gu, out=hidden)
            if self._partial is None or self._partial.shape[0] < M:
                self._partial = torch.empty((M, self.H), dtype=torch.float32, device=x.device)
            part = self._partial[:M]
            _lib.check("sfb200_sparse_gemm_f32out", _lib.lib().sfb200_sparse_gemm_f32out(
                hidden.data_ptr(), hidden.stride(0), self.dn.values.data_ptr(), self.dn.meta.data_ptr(), part.data_ptr(),
                self.H, M, self.H, self.Ip, ops._dt(x), bias.data_ptr() if bias is not None else None, 0, ops._stream()))
            self.kernel_launches += 2
            dist.all_reduce(part, group=self.group)
            out.copy_(part)                       # the one rounding to 16 bits
            return out
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

    ``exchange="push"`` (default): the down GEMM's epilogue stores every partial token block straight into the owning
    rank's receive slot over NVLink while the GEMM runs (reduce-scatter fused into the GEMM, tile by tile); then ONE
    kernel per rank waits for all ranks' GEMMs, adds the slots in fp32, adds the bias, rounds once and stores the
    finished block into every rank's output (all-gather fused into the reduction), and returns when every rank is
    done.  Three launches per step, plain peer stores only, no multicast needed.

    ``exchange="pipeline"``: the same data movement, scheduled for overlap instead of fused into the GEMM: tokens are
    cut into ``chunks``; the down GEMM of a chunk writes its partial sums locally at full speed, and ONE light kernel
    per chunk on a side stream (128 threads per SM, it fits beside a GEMM CTA) pushes them to the owners' slots, waits
    for all ranks, reduces its own slots and stores the finished block to every rank -- while the main stream already
    runs the GEMMs of the next chunk.  Pays where the pushes would otherwise make the down GEMM wait for NVLink
    (four and more ranks).

    ``exchange="switch"``: the down GEMM writes this rank's partial sums into its own copy of a symmetric buffer; one
    kernel per rank sums its token block across ranks INSIDE NVSwitch (``multimem.ld_reduce``) and writes the finished
    block to every rank with ``multimem.st``.  Needs switch-replicated (multicast) symmetric memory.  ``chunks`` cuts
    the down GEMM and this exchange into token chunks, the exchange of chunk c running on a side stream beside the
    GEMM of chunk c + 1.

    ``partial_dtype``: ``"fp32"`` (default) keeps every rank's partial sums in fp32 until they have been added, so the
    output is rounded to 16 bits once, as on one GPU, and meets the single-GPU error bound; ``"16bit"`` (the weight
    dtype) halves the bytes of the reduction, but every partial then carries its own rounding and a few outputs per
    million end up just outside that bound (measured 1.0e-2 .. 1.3e-2 against 1e-2); ``"fp16"`` (push exchange) sends
    the partial sums as fp16 whatever the weight dtype, clamped to the finite fp16 range: the bytes of ``"16bit"`` with
    eight times finer rounding than bf16, for models whose down-projection outputs stay below 65504.

    The result of ``forward`` is a view of a symmetric buffer that peers write into: see ``forward``.
    """

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, max_tokens: int, group=None,
                 down_bias: Optional[torch.Tensor] = None, exchange: str = "push", partial_dtype: str = "fp32",
                 chunks: int = 1, out_multicast: bool = False):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib, ops
        self.C, self.ops, self.L = C, ops, _lib.lib()
        self.group = group if group is not None else dist.group.WORLD
        self.tp = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if not 2 <= self.tp <= 8:
            raise ValueError("fused tensor-parallel FFN needs 2..8 ranks")
        if exchange not in ("push", "pipeline", "switch"):
            raise ValueError("exchange must be 'push', 'pipeline' or 'switch'")
        if partial_dtype not in ("fp32", "16bit", "fp16"):
            raise ValueError("partial_dtype must be 'fp32', 'fp16' or '16bit'")
        if partial_dtype == "fp16" and exchange != "push" and gate.dtype != torch.float16:
            raise ValueError("partial_dtype='fp16' on a bf16 model needs exchange='push'")
        self.exchange = exchange
        self.partial_f32 = partial_dtype == "fp32"
        # element type of the receive slots as the C calls name it: 0 weight dtype, 1 float, 2 fp16 whatever the weights are
        self.slot_kind = 1 if self.partial_f32 else (2 if partial_dtype == "fp16" else 0)
        self.chunks = max(1, int(chunks)) if exchange != "push" else 1
        self.I, self.H = gate.shape
        g, u, d = shard_ffn_weights(gate, up, down, self.tp, self.rank)
        self.Ip = g.shape[0]
        self.gu = ops.compress_gate_up(g, u)
        self.dn = ops.compress_weight(d)
        self.down_bias = down_bias
        self.dtype = gate.dtype
        dev = gate.device
        self.device = dev
        self.tok_per_owner = block_rows(max_tokens, self.tp)
        self.max_tokens = max_tokens
        Mo, H, tp = self.tok_per_owner, self.H, self.tp
        self.row_bytes = H * 2
        self.pbytes = H * (4 if self.partial_f32 else 2)          # bytes per row of a partial-sum buffer
        VP = C.c_void_p * 8
        self._VP = VP
        pdtype = torch.float32 if self.partial_f32 else (torch.float16 if self.slot_kind == 2 else self.dtype)
        self._symm = symm_mem

        def ptrs(handle):
            return [int(p) for p in handle.buffer_ptrs]
        # the replicated output [tp * tok_per_owner, H]
        self.out = symm_mem.empty((tp * Mo, H), dtype=self.dtype, device=dev)
        self.h_out = symm_mem.rendezvous(self.out, self.group)
        self.out_ptrs = ptrs(self.h_out)
        self.mc_out = int(getattr(self.h_out, "multicast_ptr", 0) or 0)
        self.out_multicast = bool(out_multicast and self.mc_out)
        if exchange == "switch":
            # every rank's partial sums, same offsets on every rank
            self.partial = symm_mem.empty((tp * Mo, H), dtype=pdtype, device=dev)
            self.h_partial = symm_mem.rendezvous(self.partial, self.group)
            self.mc_partial = int(getattr(self.h_partial, "multicast_ptr", 0) or 0)
            if not self.mc_out or not self.mc_partial:
                raise RuntimeError("exchange='switch' needs switch-replicated (multicast) symmetric memory")
        else:
            # receive slots [source rank][slot_rows, H]: rank s stores its partial sums of MY token blocks into slot s
            # (one block per token chunk, one after the other; 16 spare rows per possible chunk for rounding)
            self.slot_rows = Mo + 16 * 8
            self.recv = symm_mem.empty((tp, self.slot_rows, H), dtype=pdtype, device=dev)
            self.h_recv = symm_mem.rendezvous(self.recv, self.group)
            self.recv_ptrs = ptrs(self.h_recv)
            if exchange == "pipeline":      # the down GEMM writes its partial sums here, locally
                self.partial = torch.empty((tp * Mo, H), dtype=pdtype, device=dev)
        # flag words: one array for the exchange kernels (which may run on the side stream), one for the all-gather of
        # the activations (main stream); each has its own epoch counter
        nflag = self.L.sfb200_tp_flag_words()
        self.flags = symm_mem.empty((2 * nflag,), dtype=torch.int32, device=dev)
        self.flags.zero_()
        self.h_flags = symm_mem.rendezvous(self.flags, self.group)
        fp = ptrs(self.h_flags)
        self.peer_flags = VP(*[fp[r] if r < tp else None for r in range(8)])
        self.peer_flags_x = VP(*[fp[r] + 4 * nflag if r < tp else None for r in range(8)])
        self.epoch = 0
        self.epoch_x = 0
        self.comm_stream = torch.cuda.Stream(device=dev) if self.chunks > 1 else None
        self.x_full = None       # symmetric copy of the activations, created by forward_from_shards
        self.hidden = torch.empty((max_tokens, self.Ip), dtype=self.dtype, device=dev)
        self.kernel_launches = 0
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)           # every rank's flags are zero before anyone signals

    # ------------------------------------------------------------------ who computes what
    def _chunk_spans(self, M: int):
        """Token ranges of the down GEMM / exchange pipeline.  Chunks are multiples of 256 tokens (whole GEMM tiles)
        and of 16 * tp (so that every chunk splits into whole owner blocks); otherwise one span."""
        n = self.chunks
        if n > 1:
            step = -(-(-(-M // n)) // 256) * 256
            if step % (16 * self.tp) == 0 and step < M:
                return [(lo, min(M, lo + step)) for lo in range(0, M, step)]
        return [(0, M)]

    def finished_rows(self, M: int):
        """The token ranges whose finished values THIS rank produces in a step of M tokens (one per chunk)."""
        out = []
        for lo, hi in self._chunk_spans(M):
            mo_c = block_rows(hi - lo, self.tp)
            a, b = min(hi, lo + self.rank * mo_c), min(hi, lo + (self.rank + 1) * mo_c)
            if b > a:
                out.append((a, b))
        return out

    def owned_rows(self, M: int) -> Tuple[int, int]:
        """Half-open range of the token rows that THIS rank contributes in ``forward_from_shards``."""
        return owned_rows(M, self.tp, self.rank)

    def _cast(self, arr):
        return self.C.cast(arr, self.C.POINTER(self.C.c_void_p))

    # ------------------------------------------------------------------ steps
    def forward_from_shards(self, x_rows: torch.Tensor, M: int) -> torch.Tensor:
        """Like ``forward``, but every rank passes only the rows ``owned_rows(M)`` of the activations (e.g. the
        part of the batch it uploaded itself); the rows are replicated to all ranks over NVLink inside this call
        (one kernel: barrier, peer stores or ``multimem.st``, barrier)."""
        from . import _lib
        if self.x_full is None:
            self.x_full = self._symm.empty((self.tp * self.tok_per_owner, self.H), dtype=self.dtype, device=self.device)
            self.h_x = self._symm.rendezvous(self.x_full, self.group)
            self.x_ptrs = [int(p) for p in self.h_x.buffer_ptrs]
            self.mc_x = int(getattr(self.h_x, "multicast_ptr", 0) or 0) if self.out_multicast else 0
        if M > self.max_tokens:
            raise ValueError(f"{M} tokens exceed the {self.max_tokens} this instance was built for")
        lo, hi = self.owned_rows(M)
        if x_rows.shape != (hi - lo, self.H) or not x_rows.is_contiguous():
            raise ValueError(f"rank {self.rank} must pass its rows [{lo}, {hi}) as a contiguous [{hi - lo}, {self.H}] tensor")
        off = self.rank * block_rows(M, self.tp) * self.row_bytes
        self.epoch_x += 1
        # every rank launches, also one whose block is empty (M much smaller than tp * 16): the kernel's two
        # barriers are part of the protocol
        src = x_rows.data_ptr() if hi > lo else self.x_full.data_ptr()
        peer_dst = self._VP(*[self.x_ptrs[d] + off if d < self.tp else None for d in range(8)])
        rc = self.L.sfb200_tp_allgather(src, (self.mc_x + off) if self.mc_x else None, self._cast(peer_dst), hi - lo, self.H,
                                        self._cast(self.peer_flags_x), self.tp, self.rank, self.epoch_x, self.ops._stream())
        _lib.check("sfb200_tp_allgather", rc)
        self.kernel_launches += 1
        return self.forward(self.x_full[:M])

    def forward(self, x: torch.Tensor, phase_events=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns the FFN output [M, H] (identical on every rank).

        Without ``out`` the result is a VIEW of this instance's symmetric output buffer: it is valid until
        the next ``forward`` of this instance on ANY rank (peers write into it through NVLink), so consume
        it on the same stream before calling again, or pass ``out`` (a tensor of shape [M, H]) to receive a
        private copy.  ``phase_events``: optional list that receives four CUDA events bracketing three phases
        of the step for per-phase timing: gate|up GEMM, down GEMM (of the first chunk), exchange (and the
        remaining chunks)."""
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
        bias = self.down_bias.data_ptr() if self.down_bias is not None else None
        flags = self._cast(self.peer_flags)
        mark()
        ops.sparse_gemm_swiglu(x, self.gu, out=hidden)
        mark()
        if self.exchange == "push":
            # rows per owner for THIS call: a small batch pays a small exchange; slots keep their fixed pitch
            mo = block_rows(M, self.tp)
            slot = self.slot_rows * self.pbytes
            blk = mo * self.row_bytes
            peer_slots = self._VP(*[(self.recv_ptrs[o] + self.rank * slot) if o < self.tp else None for o in range(8)])
            _lib.check("sfb200_sparse_gemm_scatter", L.sfb200_sparse_gemm_scatter(
                hidden.data_ptr(), hidden.stride(0), self.dn.values.data_ptr(), self.dn.meta.data_ptr(),
                self._cast(peer_slots), self.tp, self.rank, mo, self.slot_kind, M, self.H, self.Ip, dt, st))
            mark()
            self.epoch += 1
            peer_out = self._VP(*[(self.out_ptrs[d] + self.rank * blk) if d < self.tp else None for d in range(8)])
            mc = (self.mc_out + self.rank * blk) if self.out_multicast else None
            _lib.check("sfb200_tp_reduce_slots", L.sfb200_tp_reduce_slots(
                self.recv.data_ptr(), self.slot_rows, self.slot_kind, mc, self._cast(peer_out), mo,
                self.H, dt, bias, flags, self.tp, self.rank, self.epoch, st))
            mark()
            self.kernel_launches += 3
        elif self.exchange == "pipeline":
            main = torch.cuda.current_stream()
            spans = self._chunk_spans(M)
            side = len(spans) > 1
            f32 = 1 if self.partial_f32 else 0
            slot = self.slot_rows * self.pbytes
            soff = 0                                   # row offset of this chunk's block inside every slot
            for ci, (lo, hi) in enumerate(spans):
                rows_c = hi - lo
                if self.partial_f32:
                    _lib.check("sfb200_sparse_gemm_f32out", L.sfb200_sparse_gemm_f32out(
                        hidden.data_ptr() + lo * hidden.stride(0) * 2, hidden.stride(0), self.dn.values.data_ptr(),
                        self.dn.meta.data_ptr(), self.partial.data_ptr() + lo * self.pbytes, self.H, rows_c, self.H,
                        self.Ip, dt, None, 0, st))
                else:
                    ops.sparse_gemm(hidden[lo:hi], self.dn, out=self.partial[lo:hi])
                if ci == 0:
                    mark()
                mo_c = block_rows(rows_c, self.tp)
                valid = (C.c_int * 8)(*[max(0, min(mo_c, rows_c - o * mo_c)) if o < self.tp else 0 for o in range(8)])
                peer_slots = self._VP(*[(self.recv_ptrs[o] + self.rank * slot + soff * self.pbytes) if o < self.tp else None
                                        for o in range(8)])
                peer_out = self._VP(*[(self.out_ptrs[d] + (lo + self.rank * mo_c) * self.row_bytes) if d < self.tp else None
                                      for d in range(8)])
                self.epoch += 1
                if side:        # the exchange of this chunk runs beside the next chunk's GEMMs
                    ev = torch.cuda.Event()
                    ev.record(main)
                    self.comm_stream.wait_event(ev)
                _lib.check("sfb200_tp_push_reduce", L.sfb200_tp_push_reduce(
                    self.partial.data_ptr() + lo * self.pbytes, mo_c, valid, self._cast(peer_slots),
                    self.recv.data_ptr() + soff * self.pbytes, self.slot_rows, f32, self._cast(peer_out), valid[self.rank],
                    self.H, dt, bias, flags, self.tp, self.rank, self.epoch, 1 if side else 0,
                    self.comm_stream.cuda_stream if side else st))
                soff += mo_c
            if side:
                main.wait_stream(self.comm_stream)
            mark()
            self.kernel_launches += 1 + 2 * len(spans)
        else:
            main = torch.cuda.current_stream()
            spans = self._chunk_spans(M)
            side = len(spans) > 1
            for ci, (lo, hi) in enumerate(spans):
                rows_c = hi - lo
                if self.partial_f32:
                    _lib.check("sfb200_sparse_gemm_f32out", L.sfb200_sparse_gemm_f32out(
                        hidden.data_ptr() + lo * hidden.stride(0) * 2, hidden.stride(0), self.dn.values.data_ptr(),
                        self.dn.meta.data_ptr(), self.partial.data_ptr() + lo * self.pbytes, self.H, rows_c, self.H,
                        self.Ip, dt, None, 0, st))
                else:
                    ops.sparse_gemm(hidden[lo:hi], self.dn, out=self.partial[lo:hi])
                if ci == 0:
                    mark()
                mo_c = block_rows(rows_c, self.tp)
                row0 = lo + self.rank * mo_c
                self.epoch += 1
                if side:        # the exchange of this chunk runs beside the next chunk's GEMM
                    ev = torch.cuda.Event()
                    ev.record(main)
                    self.comm_stream.wait_event(ev)
                _lib.check("sfb200_tp_allreduce_switch", L.sfb200_tp_allreduce_switch(
                    self.mc_partial + row0 * self.pbytes, self.mc_out + row0 * self.row_bytes, mo_c, self.H, dt,
                    1 if self.partial_f32 else 0, bias, flags, self.tp, self.rank, self.epoch,
                    self.comm_stream.cuda_stream if side else st))
            if side:
                main.wait_stream(self.comm_stream)
            mark()
            self.kernel_launches += 1 + 2 * len(spans)
        res = self.out[:M]
        if out is not None:
            out.copy_(res)
            return out
        return res
