"""The allocation-free host-buffer GEMM entry point, `pto_b200_gemm_f16f32_host_static`.

It serves callers that are not allowed to allocate device memory when they call in (another allocator owns
all of the device's memory, or allocation calls are barred after start-up): its device staging and its
status record live in an array built into the library.  The check is against the regular host-buffer entry
point, `pto_b200_gemm_f16f32_host`, through the C ABI with plain host arrays.  The two entry points run
different kernels (the regular one hands a tile to a pair of thread blocks, this one to a single block), but
both feed the tensor core the same 16-wide k steps in the same order, so every output element is the same
sequence of accumulations and the results are identical bit for bit.  Consecutive calls with different
operands (one of them ragged in m, n and k) show that nothing left in the shared array by one call leaks into
the next, and the device's free memory is compared across the calls: they must not allocate.

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
    import torch

    from pto_isa_b200 import _lib
    lib = _lib.lib()
    # calls in a row: a larger problem first, then a smaller one of another layout whose staging overlaps what
    # the first call left behind, then one that is ragged in every extent (tile 128 x 256, k step 64)
    for (m, n, k, b_layout, seed) in ((512, 768, 448, 1, 1), (384, 256, 320, 0, 2), (200, 264, 72, 1, 3)):
        a, b = _operands(m, n, k, b_layout, seed)
        want = np.full((m, n), np.nan, np.float32)
        got = np.full((m, n), np.nan, np.float32)
        rc = lib.pto_b200_gemm_f16f32_host(_p(a), _p(b), _p(want), m, n, k, b_layout)
        assert rc == 0, lib.pto_b200_last_error()
        rc = lib.pto_b200_gemm_f16f32_host_static(_p(a), _p(b), _p(got), m, n, k, b_layout)
        assert rc == 0, lib.pto_b200_last_error()
        # the first call on a device makes CUDA load the array (the one moment memory is taken); every later call
        # must leave the device's free memory exactly where it was
        free_before = torch.cuda.mem_get_info()[0]
        got2 = np.full((m, n), np.nan, np.float32)
        assert lib.pto_b200_gemm_f16f32_host_static(_p(a), _p(b), _p(got2), m, n, k, b_layout) == 0
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed free device memory"
        assert np.array_equal(got2.view(np.uint32), got.view(np.uint32))
        assert np.isfinite(got).all()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # same accumulation order: bit-exact
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
