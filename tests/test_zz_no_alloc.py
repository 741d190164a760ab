"""GPU tier, collected last: ``fm_w4a8_linear_static`` — the W4A8 decode layer for callers
that may not allocate device memory at the call site (code inside a foreign stream
capture, server plugins with a fixed memory plan, real-time loops).  It keeps the
quantised activations in a fixed array of the library instead of a caller buffer.

The test calls it through the C ABI twice in a row with different inputs and compares
each result with the regular entry points (quant_act + gemv_w4a8 by name, scratch
allocated by the caller) to the tolerance of the GEMV tests, 1e-5 relative; the second
call shows that what the first left in the shared array does no harm.  The input and
output buffers here come from ``fm_alloc`` only because the test needs some device
memory; the entry point itself is handed plain pointers."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import W4Runner, synth

pytestmark = pytest.mark.gpu
REL = 1e-5


def _static(rt, pwq, pws, px, py, m, n, k):
    return rt._lib.fm_w4a8_linear_static(ctypes.c_void_p(pwq), ctypes.c_void_p(pws), ctypes.c_void_p(px),
                                         ctypes.c_void_p(py), m, n, k, None, 1)


def test_static_scratch_linear_matches_regular_path(rt):
    runner = W4Runner(rt)
    try:
        for call, (n, k, m, seed) in enumerate([(1000, 5120, 3, 21), (520, 2048, 1, 22)]):
            L = synth.rt4_layer(n, k, m, seed=seed)
            with Bufs(rt) as b:
                pwq, pws, px = b.put(L["wq"]), b.put(L["ws"]), b.put(L["x"])
                py = b.zeros(m * n, np.float32, np.nan)
                rt.sync()
                assert _static(rt, pwq, pws, px, py, m, n, k) == 0, rt.last_error()
                got = rt.download(py, m * n, np.float32).reshape(m, n)
                want = runner.gemv("w4a8", pwq, pws, L["x"], n, k)
            assert O.rel_err(got, want) < REL, f"call {call}"
            q = O.quant_act(L["x"])
            assert O.rel_err(got, O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"]) < REL
    finally:
        runner.close()


def _cudart():
    for name in ("libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so.12", "libcudart.so"):
        try:
            return ctypes.CDLL(name)
        except OSError:
            continue
    return None


def test_static_scratch_linear_largest_shape_decode_shape_and_caller_stream(rt):
    """The shapes at the edges of the entry point: four tokens at K = 16384 fill the built-in array and take
    the large shared-memory configuration of the GEMV; one token at K = 5120 is the decode default (codes
    held in registers).  The last call runs on a stream made by the caller, without waiting inside the call."""
    rt_lib = _cudart()
    stream = ctypes.c_void_p()
    if rt_lib is not None and rt_lib.cudaStreamCreate(ctypes.byref(stream)) != 0:
        stream = ctypes.c_void_p()
    for n, k, m, seed, own_stream in [(96, 16384, 4, 23, False), (700, 5120, 1, 24, False), (300, 5120, 2, 25, True)]:
        L = synth.rt4_layer(n, k, m, seed=seed)
        with Bufs(rt) as b:
            pwq, pws, px = b.put(L["wq"]), b.put(L["ws"]), b.put(L["x"])
            py = b.zeros(m * n, np.float32, np.nan)
            rt.sync()
            if own_stream and stream.value:
                rc = rt._lib.fm_w4a8_linear_static(ctypes.c_void_p(pwq), ctypes.c_void_p(pws), ctypes.c_void_p(px),
                                                   ctypes.c_void_p(py), m, n, k, stream, 0)
                assert rc == 0, rt.last_error()
                assert rt_lib.cudaStreamSynchronize(stream) == 0
            else:
                assert _static(rt, pwq, pws, px, py, m, n, k) == 0, rt.last_error()
            got = rt.download(py, m * n, np.float32).reshape(m, n)
        q = O.quant_act(L["x"])
        assert O.rel_err(got, O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"]) < REL, (n, k, m)
    if stream.value:
        rt_lib.cudaStreamDestroy(stream)


def test_static_scratch_linear_refuses_oversize(rt):
    with Bufs(rt) as b:
        p = b.zeros(1024)
        assert _static(rt, p, p, p, p, 5, 8, 1024) == -4 and "M=5" in rt.last_error()
        assert _static(rt, p, p, p, p, 1, 8, 16384 + 128) == -4 and "16384" in rt.last_error()
        assert _static(rt, p, p, p, p, 1, 8, 1000) == -4
