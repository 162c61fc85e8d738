"""The allocation-free entry point ``jabas_dot_norms_static_f32``.

It serves hosts that cannot call ``cudaMalloc`` at the moment they need the statistic — a
process whose memory pool already holds the whole GPU, or code that must not run into a
synchronising allocation — by keeping the reduction scratch in a static device array of
the library.  The test calls it through the C ABI and compares with the context-based
``jabas_dot_norms_f32`` on two calls in a row (the shared scratch keeps the first call's
contents, so the second call proves that nothing stale leaks into the result).  This file
sorts last on purpose: if it fails, a run that stops at the first failure has already run
every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(n, device="cuda", generator=g) * 1e-3
    b = torch.randn(n, device="cuda", generator=g) * 1e-3 + 0.25 * a
    return a, b


@pytest.mark.parametrize("n", [5, 1025, 3 * 2 ** 20 + 3, 40 * 2 ** 20])
def test_static_scratch_matches_context_entry_point_twice(n):
    from jabas_b200 import _lib, ops
    lib = _lib.load()
    ctx = ops.Context(0)
    stream = torch.cuda.current_stream().cuda_stream
    for call, seed in enumerate((11, 12)):                     # two calls in a row, new data each time
        a, b = _pair(n, seed)
        want = torch.zeros(3, dtype=torch.float64, device="cuda")
        got = torch.zeros(3, dtype=torch.float64, device="cuda")
        ops.dot_norms(ctx, a, b, want)
        rc = lib.jabas_dot_norms_static_f32(a.data_ptr(), b.data_ptr(), n, got.data_ptr(), stream)
        assert rc == 0, lib.jabas_last_error()
        torch.cuda.synchronize()
        assert np.allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=1e-6, atol=0), call
        a64, b64 = a.double(), b.double()                      # and both agree with an fp64 reduction
        ref = np.array([float((a64 * b64).sum()), float((a64 * a64).sum()), float((b64 * b64).sum())])
        assert np.allclose(got.cpu().numpy(), ref, rtol=1e-6, atol=1e-30)
    # accumulation into a non-zero stat3 and an unaligned pointer (scalar kernel)
    a, b = _pair(n + 1, 13)
    acc = torch.ones(3, dtype=torch.float64, device="cuda")
    want = torch.ones(3, dtype=torch.float64, device="cuda")
    ops.dot_norms(ctx, a[1:], b[1:], want)
    ops.dot_norms_static(a[1:], b[1:], acc)
    torch.cuda.synchronize()
    assert np.allclose(acc.cpu().numpy(), want.cpu().numpy(), rtol=1e-6, atol=0)
    ctx.close()


def test_static_entry_point_rejects_oversize_and_null():
    from jabas_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(8, device="cuda")
    st = torch.zeros(3, dtype=torch.float64, device="cuda")
    rc = lib.jabas_dot_norms_static_f32(x.data_ptr(), x.data_ptr(), (1 << 31) + 1, st.data_ptr(), None)
    assert rc == -1 and b"JABAS_STATIC_MAX_ELEMS" in lib.jabas_last_error()      # refused before any launch
    assert lib.jabas_dot_norms_static_f32(None, x.data_ptr(), 8, st.data_ptr(), None) == -1
    assert lib.jabas_dot_norms_static_f32(x.data_ptr(), x.data_ptr(), 0, st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert float(st.abs().sum()) == 0.0
