"""The allocation-free GEMV entry point (`iq_linear_static`) against `iq_linear`.

Collected last on purpose (the file name sorts after every other test file), so a run
that stops at the first failure has already run the rest.

`iq_linear_static` serves callers that cannot allocate device memory at the call site --
a plugin invoked while its host application is capturing a stream, a server that gave
all of its memory away at start-up -- by keeping the kernel's work area in a device
array inside the library.  It must give exactly what `iq_linear` gives with a caller
scratch buffer (same kernel, same fixed summation order: bit-identical bf16), also on a
second call that finds the first call's leftovers in the shared array."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(n, k, m, seed):
    from iquestrt_b200 import synth
    return synth.make_linear_case(n, k, m, device="cuda", seed=seed)


def test_static_work_area_matches_caller_scratch_twice_in_a_row():
    from iquestrt_b200 import ops
    scratch = ops.Scratch("cuda")
    # stream-K split tiles (the scratch's partial sums and counters are exercised), then a
    # different shape on the same shared array
    shapes = [(6144, 6144, 1, 41), (6144, 8192, 4, 42)]
    for call, (n, k, m, seed) in enumerate(shapes):
        x, w, s = _case(n, k, m, seed)
        want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.linear(x, w, s, scratch=scratch, out=want)
        assert scratch.status() == 0
        ops.linear_static(x, w, s, got)
        assert ops.linear_static_status() == 0, f"call {call}"     # synchronises the stream
        assert torch.isfinite(got.float()).all(), f"call {call}"
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}"
    # and the same shape again right away: counters and ticket were left clean
    x, w, s = _case(6144, 6144, 1, 41)
    again = torch.empty(1, 6144, dtype=torch.bfloat16, device="cuda")
    first = torch.empty_like(again)
    ops.linear_static(x, w, s, first)
    ops.linear_static(x, w, s, again)
    torch.cuda.synchronize()
    assert torch.equal(first.view(torch.int16), again.view(torch.int16))


def test_static_work_area_rejects_oversize_and_tail():
    from iquestrt_b200 import _lib, ops
    import ctypes as C
    a = _lib.LinearArgs()
    a.n, a.k, a.m = 65536 + 16, 1024, 1
    assert _lib.load().iq_linear_static(C.byref(a), None) == _lib.IQ_ERR_UNSUPPORTED
    x, w, s = _case(256, 1024, 1, 3)
    out = torch.empty(1, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.linear_static(x, w, s, out[:, :128])
