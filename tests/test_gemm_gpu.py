"""GPU parity of the fp16 -> fp32 GEMM against the CPU oracle (the reference's tile program arithmetic).

Tolerance: max relative error <= 2e-3 with the denominator floored at rms(expected), i.e.
|got - want| <= 2e-3 * max(|want|, rms(want)) for every element (outputs that cancel to ~0 are judged
against the typical magnitude).  The reference's own self-check rule (ResultCmp eps 1e-3,
kernels/manual/a2a3/gemm_performance/main.cpp:72) is applied as well."""
import os

import numpy as np
import pytest
import torch

import oracle
import pto_isa_b200 as pto
from util import dev, host, rel_err_ok, result_cmp

pytestmark = pytest.mark.gpu
port = oracle.port


def make(m, n, k, b_layout, seed):
    r = np.random.default_rng(seed)
    a = r.uniform(-1, 1, (m, k)).astype(np.float32).astype(np.float16)
    b = r.uniform(-1, 1, (k, n) if b_layout == 0 else (n, k)).astype(np.float32).astype(np.float16)
    return a, b


@pytest.mark.parametrize("b_layout", [1, 0])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (128, 256, 256), (256, 512, 320), (384, 256, 1024),
                                 (1536, 1536, 1536)])
def test_gemm_matches_oracle(mnk, b_layout):
    m, n, k = mnk
    a, b = make(m, n, k, b_layout, seed=0)
    want = port.gemm_f16f32(a, b, b_layout)
    got = host(pto.gemm(dev(a), dev(b), b_layout))
    ok, worst = rel_err_ok(got, want, 2e-3, label=f"gemm {m}x{n}x{k} b_layout={b_layout}")
    assert ok, f"max relative error {worst:.3e}"
    assert result_cmp(want, got, 1e-3)
    assert pto.device_status() == 0


@pytest.mark.parametrize("b_layout", [1, 0])
@pytest.mark.parametrize("mnk", [(100, 200, 72), (129, 264, 520), (1, 8, 8), (300, 40, 136)])
def test_gemm_ragged_shapes(mnk, b_layout):
    """m, n not multiples of the 128 x 256 tile and k not a multiple of 64: edges are zero-filled by TMA
    on the way in and masked on the way out."""
    m, n, k = mnk
    a, b = make(m, n, k, b_layout, seed=1)
    bf = b.astype(np.float64) if b_layout == 0 else b.astype(np.float64).T
    want = a.astype(np.float64) @ bf
    c = torch.full((m + 1, n), 7.0, device="cuda")  # guard row must stay untouched
    pto.gemm(dev(a), dev(b), b_layout, out=c[:m])
    got = host(c)
    ok, worst = rel_err_ok(got[:m], want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"
    assert (got[m] == 7.0).all()


def test_gemm_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "gemm.npz"))
    got = host(pto.gemm(dev(z["a"]), dev(z["b_dn"]), 1))
    assert result_cmp(z["golden"], got, 1e-3)


def test_gemm_unsupported_shapes_are_errors():
    a = torch.zeros(128, 68, dtype=torch.float16, device="cuda")  # k not a multiple of 8
    b = torch.zeros(256, 68, dtype=torch.float16, device="cuda")
    with pytest.raises(pto.PtoB200Error):
        pto.gemm(a, b, 1)


def test_gemm_batched_and_linearity():
    a, b = make(256, 256, 128, 1, seed=3)
    a2, _ = make(256, 256, 128, 1, seed=4)
    da = torch.stack([dev(a), dev(a2)])
    db = torch.stack([dev(b), dev(b)])
    c = host(pto.gemm(da, db, 1))
    assert np.array_equal(c[0], host(pto.gemm(dev(a), dev(b), 1)))
    assert np.array_equal(c[1], host(pto.gemm(dev(a2), dev(b), 1)))
    # exactness property: scaling A by 2 scales C by exactly 2 (powers of two commute with rounding)
    c2 = host(pto.gemm(dev((a.astype(np.float32) * 2).astype(np.float16)), dev(b), 1))
    assert np.array_equal(c2, 2 * c[0])


@pytest.mark.parametrize("size", [3072, 6144, 7680])
def test_gemm_full_size_sampled_tiles(size):
    """The square sweep (6144^3 is the headline size): the whole product runs on the GPU; sampled 128 x 256 C tiles
    are recomputed by the oracle at full K, and a row/column checksum identity is checked on everything."""
    m = n = k = size
    a, b = make(m, n, k, 1, seed=size)
    da, db = dev(a), dev(b)
    c = pto.gemm(da, db, 1)
    assert pto.device_status() == 0
    r = np.random.default_rng(0)
    for _ in range(4):
        ti, tj = int(r.integers(0, m // 128)), int(r.integers(0, n // 256))
        r0, c0 = ti * 128, tj * 256
        want = np.zeros((128, 256), np.float32)
        import ctypes
        P = lambda x: x.ctypes.data_as(ctypes.c_void_p)
        asub = np.ascontiguousarray(a[r0:r0 + 128])
        bsub = np.ascontiguousarray(b[c0:c0 + 256])
        assert port.lib.pto_oracle_gemm_f16f32(P(asub), P(bsub), P(want), 128, 256, k, 1) == 0
        got = host(c[r0:r0 + 128, c0:c0 + 256])
        ok, worst = rel_err_ok(got, want, 2e-3)
        assert ok, f"tile ({ti},{tj}) max relative error {worst:.3e}"
    # checksum of checksums: sum_j C[i, j] == A[i, :] . (sum_j B[j, :]) for every row i (float64 on host)
    colsum_b = b.astype(np.float64).sum(axis=0)
    want_rows = a.astype(np.float64) @ colsum_b
    got_rows = host(c.double().sum(dim=1))
    assert np.abs(got_rows - want_rows).max() <= 1e-3 * np.sqrt(n * k / 9.0)


def test_host_batched_pipeline_equals_device_path():
    """Pipelined host-buffer entry point: every problem of the batch (odd count: both staging sets, a tail) equals the
    device-pointer entry point bit for bit; pinned and pageable host memory."""
    g = torch.Generator().manual_seed(8)
    batch, m, n, k = 5, 256, 384, 512
    a = (torch.rand(batch, m, k, generator=g) * 2 - 1).half()
    b = (torch.rand(batch, n, k, generator=g) * 2 - 1).half()
    for pin in (False, True):
        ha, hb = (a.pin_memory(), b.pin_memory()) if pin else (a, b)
        hc = torch.zeros(batch, m, n)
        hc = hc.pin_memory() if pin else hc
        pto.gemm_host_batched(ha, hb, hc, 1)
        for i in range(batch):
            assert torch.equal(hc[i], pto.gemm(a[i].cuda(), b[i].cuda(), 1).cpu()), (pin, i)
    assert pto.gemm_host_batched(a[:0], b[:0], torch.zeros(0, m, n), 1).shape[0] == 0
    assert pto.device_status() == 0


@pytest.mark.parametrize("mnk", [(256, 512, 320), (129, 264, 520), (16, 16, 16)])
def test_gemm_bias_form(mnk):
    """TMATMUL_BIAS (include/pto/cpu/TMatmul.hpp:99-116): the product plus one bias value per column; against the
    oracle's product with the bias added in fp32, and exactly equal to the plain kernel's output plus the bias."""
    m, n, k = mnk
    a, b = make(m, n, k, 1, seed=11)
    bias = np.random.default_rng(5).uniform(-10, 10, n).astype(np.float32)
    got = host(pto.gemm(dev(a), dev(b), 1, bias=dev(bias)))
    plain = host(pto.gemm(dev(a), dev(b), 1))
    assert np.array_equal(got, plain + bias[None, :])
    want = a.astype(np.float64) @ b.astype(np.float64).T + bias[None, :]
    ok, worst = rel_err_ok(got, want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"


@pytest.mark.parametrize("mnk", [(128, 256, 64), (256, 512, 320), (300, 200, 112), (1, 4, 16), (1024, 768, 2048)])
def test_gemm_int8_exact(mnk):
    """TMATMUL's (int8, int8 -> int32) form on kind::i8: bit-exact against the oracle over the full int8 range, ragged
    m and n included, with a guard row."""
    m, n, k = mnk
    r = np.random.default_rng(m + k)
    a = r.integers(-128, 128, (m, k)).astype(np.int8)
    b = r.integers(-128, 128, (n, k)).astype(np.int8)
    want = port.tmatmul_i8i32(a, np.ascontiguousarray(b.T))
    c = torch.full((m + 1, n), 7, device="cuda", dtype=torch.int32)
    pto.gemm_i8(dev(a), dev(b), out=c[:m])
    got = host(c)
    assert np.array_equal(got[:m], want) and (got[m] == 7).all()
    assert pto.device_status() == 0


def test_gemm_int8_reference_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "tmatmul_i8.npz"))
    for name in ("small", "mid"):
        got = host(pto.gemm_i8(dev(z[name + "_a"]), dev(np.ascontiguousarray(z[name + "_b"].T))))
        assert np.array_equal(got, z[name + "_golden"])
    with pytest.raises(pto.PtoB200Error):
        pto.gemm_i8(torch.zeros(16, 24, dtype=torch.int8, device="cuda"), torch.zeros(16, 24, dtype=torch.int8, device="cuda"))


def test_gemm_bias_reference_golden(golden_dir):
    """The bias case of the reference's tmatmul generator (integer-valued operands: the result is exact)."""
    z = np.load(os.path.join(golden_dir, "tmatmul_bias.npz"))
    got = host(pto.gemm(dev(z["a"]), dev(z["b"]), 0, bias=dev(z["bias"])))
    assert np.array_equal(got, z["golden"])


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mnk_layout", [((256, 512, 320), 1), ((129, 264, 520), 1), ((300, 40, 136), 0), ((1, 8, 8), 1),
                                        ((130, 36, 64), 1)])
def test_gemm_16bit_output(mnk_layout, out_dtype):
    """C rounded to fp16 / bf16 in the epilogue (TSTORE's conversion out of the accumulator): bit-equal to the fp32
    kernel's output rounded by torch (same accumulator, round to nearest even), ragged shapes and an output whose rows
    are not 16-byte multiples (n = 36) included; a guard row stays untouched."""
    (m, n, k), b_layout = mnk_layout
    a, b = make(m, n, k, b_layout, seed=21)
    want = pto.gemm(dev(a), dev(b), b_layout).to(out_dtype)
    c = torch.full((m + 1, n), 7.0, device="cuda", dtype=out_dtype)
    pto.gemm_out16(dev(a), dev(b), b_layout, out_dtype, out=c[:m])
    assert torch.equal(c[:m], want) and bool((c[m] == 7.0).all())
    assert pto.device_status() == 0


def test_gemm_16bit_output_full_size():
    a, b = make(6144, 6144, 6144, 1, seed=6)
    da, db = dev(a), dev(b)
    assert torch.equal(pto.gemm_out16(da, db, 1, torch.bfloat16), pto.gemm(da, db, 1).bfloat16())


@pytest.mark.parametrize("b_layout", [1, 0])
@pytest.mark.parametrize("mnk", [(256, 512, 320), (129, 264, 520), (1024, 768, 2048)])
def test_gemm_bf16_operands(mnk, b_layout):
    """bfloat16 operands, fp32 accumulate: against the exact (float64) product of the same bf16 values, tolerance 2e-3 of
    max(|want|, rms(want)) as for fp16."""
    m, n, k = mnk
    g = torch.Generator().manual_seed(m + b_layout)
    a = (torch.rand(m, k, generator=g) * 2 - 1).bfloat16()
    b = (torch.rand((k, n) if b_layout == 0 else (n, k), generator=g) * 2 - 1).bfloat16()
    bd = b.double() if b_layout == 0 else b.double().t()
    want = (a.double() @ bd).numpy()
    got = host(pto.gemm_bf16(a.cuda(), b.cuda(), b_layout))
    ok, worst = rel_err_ok(got, want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"
    assert pto.device_status() == 0


_WIDTH_SCRIPT = r"""
import random, sys, torch
import pto_isa_b200 as pto
random.seed(11)
for it in range(36):
    m = random.choice([1, 7, 64, 100, 128, 129, 200, 256, 257, 384, 500, 777, 1024])
    n = random.choice([8, 16, 64, 72, 120, 128, 136, 192, 256, 264, 400, 512, 1000])
    k = random.choice([8, 16, 64, 72, 128, 136, 248, 256, 264, 512, 520, 1032])
    lay = random.choice([0, 1])
    a = (torch.rand(m, k, device="cuda") * 2 - 1).half()
    b = ((torch.rand(k, n, device="cuda") if lay == 0 else torch.rand(n, k, device="cuda")) * 2 - 1).half()
    c = torch.full((m, n), float("nan"), device="cuda")
    pto.gemm(a, b, lay, out=c)
    ref = a.double() @ (b.double() if lay == 0 else b.double().t())
    err = float(((c.double() - ref).abs().max() / max(float(ref.abs().max()), 1e-6)))
    assert err < 2e-3 and not bool(torch.isnan(c).any()), (m, n, k, lay, err)
# 16-bit output, bias and int8 go through the same launcher
a = (torch.rand(300, 264, device="cuda") * 2 - 1).half(); b = (torch.rand(200, 264, device="cuda") * 2 - 1).half()
c16 = pto.gemm_out16(a, b, 1)
assert torch.equal(c16, pto.gemm(a, b, 1).half())
bias = torch.rand(200, device="cuda")
assert torch.allclose(pto.gemm(a, b, 1, bias=bias), pto.gemm(a, b, 1) + bias, rtol=0, atol=1e-5)
ai = torch.randint(-128, 128, (130, 272), device="cuda", dtype=torch.int8); bi = torch.randint(-128, 128, (72, 272), device="cuda", dtype=torch.int8)
assert torch.equal(pto.gemm_i8(ai, bi).cpu().long(), ai.cpu().long() @ bi.cpu().long().t())
assert pto.device_status() == 0
print("ok")
"""


@pytest.mark.parametrize("width", ["128", "256"])
def test_gemm_both_tile_widths_on_ragged_shapes(width):
    """The block-pair kernel chooses 256- or 128-column tiles by problem size (launch_pair in csrc/gemm_2cta.cu).
    PTO_B200_GEMM2_BN, read once per process, forces one: 36 seeded shapes with ragged m, n, k in both layouts of B, plus
    the 16-bit output, the bias form and int8, run in a child process on each width against a float64 product."""
    import subprocess
    import sys
    env = dict(os.environ, PTO_B200_GEMM2_BN=width)
    env["PYTHONPATH"] = os.pathsep.join([os.path.dirname(os.path.dirname(os.path.abspath(__file__))), env.get("PYTHONPATH", "")])
    r = subprocess.run([sys.executable, "-c", _WIDTH_SCRIPT], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout[-2000:] + r.stderr[-2000:]
