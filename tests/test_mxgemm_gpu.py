"""MX block-scaled fp8 GEMM (the reference's MxMatmul, kernels/manual/a5/matmul_mxfp8_performance) on the GPU through
the C ABI against the CPU oracle and the reference generator's golden.

Tolerance.  The oracle sums the scaled products exactly; the tensor core accumulates in fp32.  With float output the
bar is the GEMM's: |got - want| <= 2e-3 * max(|want|, rms(want)).  With bfloat16 output (the reference's type) both
sides are rounded to bfloat16: every element within one bfloat16 ulp (or, for sums that cancel to almost nothing,
within 2e-5 of rms(want), the size of the fp32 accumulation error), and at most 0.5 % of the elements different at
all (a difference needs the exact sum within fp32 accumulation error of a rounding boundary).  The reference's own
ResultCmp rule (eps 1e-3, main.cpp:26) is applied as well."""
import os

import numpy as np
import pytest
import torch

import oracle
import pto_isa_b200 as pto
from util import dev, host, rel_err_ok, result_cmp

pytestmark = pytest.mark.gpu
port = oracle.port


def to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def make(m, n, k, fmt, seed):
    """fp8 bytes of uniform(-5, 5) values and scales in {2^0, 2^1, 2^2} as the reference generator draws them
    (scripts/gen_data.py:33-40), plus a wider scale range in the second half of k."""
    r = np.random.default_rng(seed)
    tdt = torch.float8_e5m2 if fmt == 1 else torch.float8_e4m3fn
    a = torch.from_numpy(r.uniform(-5, 5, (m, k)).astype(np.float32)).to(tdt).view(torch.uint8).numpy()
    b = torch.from_numpy(r.uniform(-5, 5, (n, k)).astype(np.float32)).to(tdt).view(torch.uint8).numpy()
    sa = r.integers(127, 130, (m, k // 32)).astype(np.uint8)
    sb = r.integers(127, 130, (n, k // 32)).astype(np.uint8)
    sa[:, (k // 64):] = r.integers(120, 134, sa[:, (k // 64):].shape).astype(np.uint8)
    return a, b, sa, sb


def check_bf16(got_bits, want_f32):
    want_bits = to_bf16_bits(want_f32)
    got, want = bf16_bits_to_f32(got_bits), bf16_bits_to_f32(want_bits)
    ulp = np.abs(got_bits.astype(np.int32) - want_bits.astype(np.int32))  # same sign assumed away below
    same_sign = (got_bits >> 15) == (want_bits >> 15)
    floor = 2e-5 * np.sqrt(np.mean(want.astype(np.float64) ** 2))  # fp32 accumulation error of a sum that cancels
    one_ulp = np.where(same_sign, ulp <= 1, False) | (np.abs(got - want) <= floor)
    assert one_ulp.all(), f"{(~one_ulp).sum()} elements differ by more than one bfloat16 ulp"
    assert (got_bits != want_bits).mean() <= 5e-3
    assert result_cmp(want, got, 1e-3)


@pytest.mark.parametrize("fmt", [1, 0])
@pytest.mark.parametrize("mnk", [(256, 256, 128), (256, 256, 640), (128, 256, 256), (512, 768, 1024), (384, 512, 96)])
def test_mxgemm_matches_oracle(mnk, fmt):
    m, n, k = mnk
    a, b, sa, sb = make(m, n, k, fmt, seed=m + n + k + fmt)
    want = port.mxgemm_fp8(a, b, sa, sb, fmt, fmt)
    got32 = host(pto.mx_gemm(dev(a), dev(b), dev(sa), dev(sb), torch.float32, fmt=fmt))
    ok, worst = rel_err_ok(got32, want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"
    got16 = host(pto.mx_gemm(dev(a), dev(b), dev(sa), dev(sb), torch.bfloat16, fmt=fmt).view(torch.int16)).view(np.uint16)
    check_bf16(got16, want)
    assert pto.device_status() == 0


@pytest.mark.parametrize("mnk", [(100, 200, 64), (129, 264, 160), (1, 8, 32), (300, 40, 416)])
def test_mxgemm_ragged_shapes(mnk):
    """m, n not multiples of the 256 x 256 tile, k not a multiple of the 128 stage: data edges are zero-filled by TMA,
    scale edges padded with 2^0, output edges masked; a guard row stays untouched."""
    m, n, k = mnk
    a, b, sa, sb = make(m, n, k, 1, seed=7 + m)
    want = port.mxgemm_fp8(a, b, sa, sb, 1, 1)
    for dt in (torch.float32, torch.bfloat16):
        c = torch.full((m + 1, n), 7.0, device="cuda", dtype=dt)
        pto.mx_gemm(dev(a), dev(b), dev(sa), dev(sb), dt, out=c[:m])
        got = host(c.float())
        assert (got[m] == 7.0).all()
        if dt == torch.float32:
            ok, worst = rel_err_ok(got[:m], want, 2e-3)
            assert ok, f"max relative error {worst:.3e}"
        else:
            check_bf16(host(c[:m].contiguous().view(torch.int16)).view(np.uint16), want)
    assert pto.device_status() == 0


def test_mxgemm_reference_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "mxgemm.npz"))
    for tag, fmt in (("e5m2", 1), ("e4m3", 0)):
        got = pto.mx_gemm(dev(z[f"{tag}_a"]), dev(z[f"{tag}_b"]), dev(z[f"{tag}_scale_a"]), dev(z[f"{tag}_scale_b"]),
                          torch.bfloat16, fmt=fmt)
        bits = host(got.view(torch.int16)).view(np.uint16)
        gold = z[f"{tag}_golden_bf16_bits"]
        assert result_cmp(bf16_bits_to_f32(gold), bf16_bits_to_f32(bits), 1e-3)
        assert (bits != gold).mean() <= 5e-3


def test_mxgemm_torch_fp8_dtypes_and_scale_identity():
    """float8 tensors select the format by dtype; multiplying every scale of A by 2 doubles C exactly."""
    a, b, sa, sb = make(256, 256, 256, 1, seed=3)
    ta, tb = dev(a).view(torch.float8_e5m2), dev(b).view(torch.float8_e5m2)
    c1 = pto.mx_gemm(ta, tb, dev(sa), dev(sb), torch.float32)
    c2 = pto.mx_gemm(ta, tb, dev(sa + 1), dev(sb), torch.float32)
    assert torch.equal(c2, 2 * c1)
    assert torch.equal(c1, pto.mx_gemm(dev(a), dev(b), dev(sa), dev(sb), torch.float32, fmt=pto.ops.FP8_E5M2))


def test_mxgemm_bad_arguments():
    a, b, sa, sb = make(128, 256, 128, 1, seed=4)
    with pytest.raises(pto.PtoB200Error):
        pto.mx_gemm(dev(a[:, :48]), dev(b[:, :48]), dev(sa[:, :1]), dev(sb[:, :1]))  # k not a multiple of 32
    with pytest.raises(pto.PtoB200Error):
        pto.mx_gemm(dev(a), dev(b), dev(sa[:, :2]), dev(sb))


def test_mxgemm_full_size_sampled_tiles():
    """6144^3, the reference's configuration: sampled 128 x 128 windows of C against the oracle at full k, and the
    scale identity on the whole output."""
    m = n = k = 6144
    a, b, sa, sb = make(m, n, k, 1, seed=6144)
    da, db, dsa, dsb = dev(a), dev(b), dev(sa), dev(sb)
    c = pto.mx_gemm(da, db, dsa, dsb, torch.bfloat16)
    assert pto.device_status() == 0
    r = np.random.default_rng(1)
    for _ in range(3):
        r0, c0 = int(r.integers(0, m // 128)) * 128, int(r.integers(0, n // 128)) * 128
        want = port.mxgemm_fp8(a, b, sa, sb, 1, 1, window=(r0, r0 + 128, c0, c0 + 128))[r0:r0 + 128, c0:c0 + 128]
        got = host(c[r0:r0 + 128, c0:c0 + 128].contiguous().view(torch.int16)).view(np.uint16)
        check_bf16(got, want)
    c32 = pto.mx_gemm(da, db, dsa, dsb, torch.float32)
    assert torch.equal(pto.mx_gemm(da, db, dsa, dev(sb + 1), torch.float32), 2 * c32)
    assert torch.equal(c32.bfloat16(), c)


# ---------------------------------------------------------------- packed fp4 (float4_e2m1) operands
def make_fp4(m, n, k, seed, full_range=True):
    """Packed e2m1 bytes.  full_range: all 16 codes; otherwise the reference generator's values {-1, 0, 1}
    (kernels/manual/a5/matmul_mxfp4_performance/scripts/gen_data.py:44-45)."""
    r = np.random.default_rng(seed)
    if full_range:
        a = r.integers(0, 256, (m, k // 2)).astype(np.uint8)
        b = r.integers(0, 256, (n, k // 2)).astype(np.uint8)
    else:
        code = np.array([0xA, 0x0, 0x2], np.uint8)  # -1, 0, 1
        ea, eb = code[r.integers(0, 3, (m, k))], code[r.integers(0, 3, (n, k))]
        a = (ea[:, 0::2] | (ea[:, 1::2] << 4)).astype(np.uint8)
        b = (eb[:, 0::2] | (eb[:, 1::2] << 4)).astype(np.uint8)
    sa = r.integers(127, 130, (m, k // 32)).astype(np.uint8)
    sb = r.integers(127, 130, (n, k // 32)).astype(np.uint8)
    sa[:, (k // 64):] = r.integers(120, 134, sa[:, (k // 64):].shape).astype(np.uint8)
    return a, b, sa, sb


@pytest.mark.parametrize("full_range", [False, True])
@pytest.mark.parametrize("mnk", [(256, 256, 512), (256, 256, 256), (128, 256, 1024), (512, 768, 2048), (300, 200, 1184), (1, 8, 32)])
def test_mxgemm_fp4_matches_oracle(mnk, full_range):
    """Positions matter here: every k block carries its own pair of scales, so a wrong nibble order, scale byte or
    scale atom shows as an error far above the tolerance."""
    m, n, k = mnk
    a, b, sa, sb = make_fp4(m, n, k, seed=m + n + k, full_range=full_range)
    want = port.mxgemm_fp4(a, b, sa, sb)
    got32 = host(pto.mx_gemm_fp4(dev(a), dev(b), dev(sa), dev(sb), torch.float32))
    ok, worst = rel_err_ok(got32, want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"
    got16 = host(pto.mx_gemm_fp4(dev(a), dev(b), dev(sa), dev(sb), torch.bfloat16).view(torch.int16)).view(np.uint16)
    check_bf16(got16, want)
    assert pto.device_status() == 0


def test_mxgemm_fp4_full_size_sampled_tiles():
    """6144^3 (the reference's MXFP4 configuration): sampled 64 x 64 windows against the oracle at full k."""
    m = n = k = 6144
    a, b, sa, sb = make_fp4(m, n, k, seed=61, full_range=True)
    c = pto.mx_gemm_fp4(dev(a), dev(b), dev(sa), dev(sb), torch.bfloat16)
    assert pto.device_status() == 0
    r = np.random.default_rng(2)
    for _ in range(3):
        r0, c0 = int(r.integers(0, m // 64)) * 64, int(r.integers(0, n // 64)) * 64
        want = port.mxgemm_fp4(a, b, sa, sb, window=(r0, r0 + 64, c0, c0 + 64))[r0:r0 + 64, c0:c0 + 64]
        got = host(c[r0:r0 + 64, c0:c0 + 64].contiguous().view(torch.int16)).view(np.uint16)
        check_bf16(got, want)


def test_mxgemm_fp4_reference_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "mxgemm_fp4.npz"))
    got = pto.mx_gemm_fp4(dev(z["a"]), dev(z["b"]), dev(z["scale_a"]), dev(z["scale_b"]), torch.bfloat16)
    bits = host(got.view(torch.int16)).view(np.uint16)
    assert result_cmp(bf16_bits_to_f32(z["golden_bf16_bits"]), bf16_bits_to_f32(bits), 1e-3)
    assert (bits != z["golden_bf16_bits"]).mean() <= 5e-3


def test_mxgemm_fp4_reference_shape_sampled_windows():
    """m 2040, k 8192, n 8100: the ragged configuration of the reference's MXFP4 example (scripts/gen_data.py:100);
    windows that include the last rows and columns, and a guard row."""
    m, k, n = 2040, 8192, 8100
    a, b, sa, sb = make_fp4(m, n, k, seed=2040, full_range=False)
    c = torch.full((m + 1, n), 7.0, device="cuda", dtype=torch.bfloat16)
    pto.mx_gemm_fp4(dev(a), dev(b), dev(sa), dev(sb), torch.bfloat16, out=c[:m])
    assert pto.device_status() == 0 and bool((c[m] == 7.0).all())
    for r0, c0 in ((0, 0), (m - 40, n - 36), (1024, 4096)):
        r1, c1 = min(m, r0 + 40), min(n, c0 + 36)
        want = port.mxgemm_fp4(a, b, sa, sb, window=(r0, r1, c0, c1))[r0:r1, c0:c1]
        got = host(c[r0:r1, c0:c1].contiguous().view(torch.int16)).view(np.uint16)
        check_bf16(got, want)


@pytest.mark.parametrize("mnk", [(130, 36, 160), (64, 7, 64), (257, 260, 96)])
def test_mxgemm_unaligned_output_rows(mnk):
    """Output rows that are not multiples of 16 bytes (bf16 n = 36, 7; fp32 n = 7) leave through element stores instead
    of TMA stores; an output that starts at an odd element too."""
    m, n, k = mnk
    a, b, sa, sb = make(m, n, k, 0, seed=n)
    want = port.mxgemm_fp8(a, b, sa, sb, 0, 0)
    for dt in (torch.bfloat16, torch.float32):
        flat = torch.full(((m + 1) * n + 1,), 7.0, device="cuda", dtype=dt)
        out = flat[1:1 + m * n].view(m, n)  # starts one element into the allocation
        pto.mx_gemm(dev(a), dev(b), dev(sa), dev(sb), dt, out=out, fmt=0)
        assert float(flat[0]) == 7.0 and bool((flat[1 + m * n:] == 7.0).all())
        if dt == torch.float32:
            ok, worst = rel_err_ok(host(out), want, 2e-3)
            assert ok, f"max relative error {worst:.3e}"
        else:
            check_bf16(host(out.contiguous().view(torch.int16)).view(np.uint16), want)
    assert pto.device_status() == 0
