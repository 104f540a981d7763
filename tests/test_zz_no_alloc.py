"""The allocation-free host-buffer GEMM entry point, `pto_b200_gemm_f16f32_host_static`.

It serves callers that are not allowed to allocate device memory when they call in (another allocator owns
all of the device's memory, or allocation calls are barred after start-up): its device staging and its
status record live in an array built into the library.  The check is against the regular host-buffer entry
point, `pto_b200_gemm_f16f32_host`, through the C ABI with plain host arrays: the same kernel runs on the
same bytes, so the outputs must be identical bit for bit.  Two calls in a row with different operands show
that nothing left in the shared array by the first call leaks into the second.

This file is collected last on purpose, so that a run that stops at the first failure has already run
every other test; it also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _operands(m, n, k, b_layout, seed):
    r = np.random.default_rng(seed)
    a = r.uniform(-1, 1, (m, k)).astype(np.float16)
    b = r.uniform(-1, 1, (k, n) if b_layout == 0 else (n, k)).astype(np.float16)
    return a, b


def test_static_scratch_gemm_matches_allocating_entry_point_twice_in_a_row():
    from pto_isa_b200 import _lib
    lib = _lib.lib()
    # two calls in a row: a larger problem first, then a smaller one of another layout whose staging
    # overlaps what the first call left behind
    for (m, n, k, b_layout, seed) in ((512, 768, 448, 1, 1), (384, 256, 320, 0, 2)):
        a, b = _operands(m, n, k, b_layout, seed)
        want = np.full((m, n), np.nan, np.float32)
        got = np.full((m, n), np.nan, np.float32)
        rc = lib.pto_b200_gemm_f16f32_host(_p(a), _p(b), _p(want), m, n, k, b_layout)
        assert rc == 0, lib.pto_b200_last_error()
        rc = lib.pto_b200_gemm_f16f32_host_static(_p(a), _p(b), _p(got), m, n, k, b_layout)
        assert rc == 0, lib.pto_b200_last_error()
        assert np.isfinite(got).all()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # same kernel, same bytes: bit-exact
        # and both agree with a float64 product (tolerance of the GEMM tests: 2e-3 of max(|x|, rms))
        bf = b.astype(np.float64) if b_layout == 0 else b.astype(np.float64).T
        exact = a.astype(np.float64) @ bf
        floor = np.sqrt(np.mean(exact ** 2))
        assert (np.abs(got - exact) <= 2e-3 * np.maximum(np.abs(exact), floor)).all()


def test_static_scratch_gemm_rejects_problems_beyond_its_capacity():
    from pto_isa_b200 import _lib
    lib = _lib.lib()
    m = n = k = 4096  # 32 MiB + 32 MiB + 64 MiB of staging: more than the built-in 36 MiB
    a = np.zeros((8, 8), np.float16)  # never read: the size check comes first
    c = np.zeros((8, 8), np.float32)
    rc = lib.pto_b200_gemm_f16f32_host_static(_p(a), _p(a), _p(c), m, n, k, 1)
    assert rc == 5  # PTO_B200_ERR_TOO_LARGE
    msg = lib.pto_b200_last_error().decode()
    assert "scratch" in msg and "pto_b200_gemm_f16f32_host" in msg
    assert lib.pto_b200_gemm_f16f32_host_static(None, None, None, 128, 256, 64, 1) == 1
