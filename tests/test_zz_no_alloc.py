"""The allocation-free FFN entry point, through the C ABI.

Some callers of this library are not allowed to allocate device memory where they run the FFN (they
sit inside an arena that forbids side allocations, or in a latency-critical loop): for them
``sfb200_ffn_forward_noalloc`` keeps the hidden tensor in a fixed array inside the library.  It
launches the same kernels as ``sfb200_ffn_forward``, so its output must equal that entry point's
bit for bit, also on a second call (the array keeps the previous call's contents), and it must
refuse a problem that does not fit.  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from sparseflow_b200 import _lib, ops
from tests.util import seeded_act, seeded_weight, to_dev

pytestmark = pytest.mark.gpu


def _setup(H, I, dt="bf16"):
    gu = ops.compress_gate_up(to_dev(seeded_weight(I, H, dt, 1), dt), to_dev(seeded_weight(I, H, dt, 2), dt))
    dn = ops.compress_weight(to_dev(seeded_weight(H, I, dt, 3), dt))
    W = _lib.FFNWeights(H, I, ops.BF16, gu.values.data_ptr(), gu.meta.data_ptr(), dn.values.data_ptr(),
                        dn.meta.data_ptr(), None)
    return W, (gu, dn)


def test_noalloc_matches_regular_entry_point_twice():
    ops.force_token_tile(0)
    H, I = 1024, 2816
    W, keep = _setup(H, I)
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    for M, seed in ((300, 11), (77, 12)):          # two calls in a row, second one smaller: stale scratch beyond it
        x = to_dev(seeded_act(M, H, "bf16", seed), "bf16")
        hidden = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
        want = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
        got = torch.zeros(M, H, device="cuda", dtype=torch.bfloat16)
        assert L.sfb200_ffn_forward(C.byref(W), x.data_ptr(), H, hidden.data_ptr(), want.data_ptr(), H, M, st) == 0
        assert L.sfb200_ffn_forward_noalloc(C.byref(W), x.data_ptr(), H, got.data_ptr(), H, M, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)              # same kernels, same bits: tolerance 0
        # this entry point reports device-side failures in a word of its own, read without allocating
        word = C.c_int(-1)
        assert L.sfb200_noalloc_device_status(C.byref(word)) == 0 and word.value == 0
    assert ops.device_status() == 0


def test_noalloc_rejects_oversized_problem():
    H, I = 1024, 2816
    W, keep = _setup(H, I)
    L = _lib.lib()
    M = (16 << 20) // (I * 2) + 1                  # one row past the 16 MiB static scratch
    x = torch.zeros(M, H, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(M, H, device="cuda", dtype=torch.bfloat16)
    rc = L.sfb200_ffn_forward_noalloc(C.byref(W), x.data_ptr(), H, out.data_ptr(), H, M, None)
    assert rc == 10
    assert b"static scratch" in L.sfb200_status_string(rc)
