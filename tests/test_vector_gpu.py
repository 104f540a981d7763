"""GPU parity of the vector tile ops against the CPU oracle and the reference's golden vectors.
Bit-exact for TCVT, TGATHER (both forms) and TROWMAX; TROWSUM / TEXP within the reference's own
test tolerance (eps 1e-3 with its ResultCmp rule) and within 2e-6 relative of the oracle."""
import os

import numpy as np
import pytest
import torch

import oracle
import pto_isa_b200 as pto
from util import dev, host, result_cmp

pytestmark = pytest.mark.gpu
port = oracle.port


def rng(seed):
    return np.random.default_rng(seed)


def bits16(t):
    return host(t.view(torch.int16)).view(np.uint16)


@pytest.mark.parametrize("n", [0, 1, 7, 8, 1000, 4096 * 33 + 5, 1 << 22])
def test_tcvt_f16_bf16_bit_exact(n):
    r = rng(n)
    x = r.standard_normal(n).astype(np.float32)
    if n >= 1000:
        special = np.array([0, -0.0, np.inf, -np.inf, np.nan, -np.nan, 65504, 65520, 65519.99, 1e-8, 6e-8, 5.96e-8,
                            2.98e-8, 2.9802322e-8, 3e-8, 6.1e-5, 6.1035156e-5, 1e5, -1e5, 1e-45], np.float32)
        x[:special.size] = special
        x[100:600] = r.integers(0, 2 ** 32, 500, dtype=np.uint32).view(np.float32)  # arbitrary bit patterns
    d = dev(x)
    assert np.array_equal(bits16(pto.TCVT(d, torch.float16)), port.tcvt_f32_f16(x).view(np.uint16))
    assert np.array_equal(bits16(pto.TCVT(d, torch.bfloat16)), port.tcvt_f32_bf16(x))


def test_tcvt_unaligned_pointers():
    x = rng(5).standard_normal(5001).astype(np.float32)
    d = dev(x)
    out = torch.empty(5003, dtype=torch.float16, device="cuda")
    pto.TCVT(d[1:], torch.float16, out=out[3:])  # 4-byte / 2-byte aligned only
    assert np.array_equal(bits16(out[3:]), port.tcvt_f32_f16(x[1:]).view(np.uint16))


def test_tcvt_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "tcvt.npz"))
    got = pto.TCVT(dev(z["case8_src"]), torch.float16)
    assert np.array_equal(bits16(got), z["case8_golden"].view(np.uint16))
    for c in ("case1", "case4", "case6"):
        assert np.array_equal(host(pto.TCVT(dev(z[f"{c}_src"]), torch.int32)), z[f"{c}_golden"])


def test_tcvt_i32_round_modes():
    x = (rng(6).standard_normal(10000) * 1000).astype(np.float32)
    x[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5, -3.5]
    d = dev(x)
    for mode in range(1, 7):
        assert np.array_equal(host(pto.TCVT(d, torch.int32, round_mode=mode)), port.tcvt_f32_i32(x, mode)), mode


def test_tgather_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "tgather.npz"))
    names = sorted({k.split("__")[0] for k in z.files})
    for n in names:
        if n.startswith("1D_"):
            src0, idx, g = z[f"{n}__src0"], z[f"{n}__idx"], z[f"{n}__golden"]
            ut = np.uint32 if src0.itemsize == 4 else np.uint16
            tt = torch.int32 if src0.itemsize == 4 else torch.int16
            got = pto.TGATHER(dev(src0.view(ut).view(np.int32 if src0.itemsize == 4 else np.int16)), dev(idx))
            assert got.dtype == tt
            assert np.array_equal(host(got).view(ut), g.view(ut)), n
        else:
            src, g, pat = z[f"{n}__src"], z[f"{n}__golden"], int(z[f"{n}__pattern"])
            st = np.int32 if src.itemsize == 4 else np.int16
            got = pto.TGATHER_MASK(dev(src.view(st)), pat)
            assert np.array_equal(host(got).view(st), g.view(st)), n


@pytest.mark.parametrize("n", [0, 3, 4097, 1 << 20])
def test_tgather_index_bit_exact(n):
    r = rng(7 + n)
    src = r.standard_normal((512, 2048)).astype(np.float32)
    idx = r.integers(-1000, src.size + 1000, n).astype(np.int32)  # out-of-range on both sides -> 0
    if n > 100:
        idx[:50] = [-1, src.size, src.size - 1, 0, -(2 ** 31)] * 10
        idx[50:100] = idx[:50][::-1]  # duplicates
    got = pto.TGATHER(dev(src), dev(idx))
    assert np.array_equal(host(got).view(np.uint32), port.tgather(src, idx).view(np.uint32))
    s16 = r.integers(0, 65536, (1024, 1024)).astype(np.uint16)
    i16 = r.integers(-5, s16.size + 5, n).astype(np.int32)
    got = pto.TGATHER(dev(s16.view(np.int16)), dev(i16))
    assert np.array_equal(host(got).view(np.uint16), port.tgather(s16, i16))


def test_tgather_16m_with_duplicates():
    """The benchmark configuration: 16M fp32 table, 16M int32 indices with >= 10% duplicates."""
    n = 1 << 24
    r = rng(2)
    src = r.standard_normal(n).astype(np.float32).reshape(4096, 4096)
    idx = r.integers(0, n, n).astype(np.int32)
    pos = r.integers(0, n, n // 10)
    idx[pos] = idx[(pos * 2654435761) % n]
    got = pto.TGATHER(dev(src), dev(idx))
    assert np.array_equal(host(got).view(np.uint32), port.tgather(src, idx).view(np.uint32))


@pytest.mark.parametrize("shape", [(16, 64), (64, 256), (7, 1024), (3, 1056), (5, 130)])
def test_tgather_mask_bit_exact(shape):
    r = rng(sum(shape))
    for pat in range(1, 8):
        s = r.standard_normal(shape).astype(np.float32)
        assert np.array_equal(host(pto.TGATHER_MASK(dev(s), pat)), port.tgather_mask(s, pat)), pat
        h = r.integers(0, 65536, shape).astype(np.uint16)
        got = pto.TGATHER_MASK(dev(h.view(np.int16)), pat)
        assert np.array_equal(host(got).view(np.uint16), port.tgather_mask(h, pat)), pat


@pytest.mark.parametrize("shape", [(1, 1), (37, 1000), (64, 64), (77, 81), (4096, 4096), (5, 8191)])
def test_row_reductions(shape):
    x = rng(shape[1]).standard_normal(shape).astype(np.float32)
    d = dev(x)
    assert np.array_equal(host(pto.TROWMAX(d)), port.trowmax_f32(x))
    want = port.trowsum_f32(x)
    got = host(pto.TROWSUM(d))
    # tree reduction vs the reference's sequential fp32 sum: bound by the row's absolute mass
    bound = 2e-6 * np.abs(x).sum(axis=1) + 1e-30
    assert (np.abs(got - want) <= bound).all()


def test_rowops_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "rowops.npz"))
    for i in (0, 3, 4):
        src, g, (vr, vc) = z[f"trowmax{i}_src"], z[f"trowmax{i}_golden"], z[f"trowmax{i}_valid"]
        assert np.array_equal(host(pto.TROWMAX(dev(src[:vr, :vc]))), g)
    assert result_cmp(z["trowsum0_golden"], host(pto.TROWSUM(dev(z["trowsum0_src"]))), 1e-3)
    for i in (0, 3, 4):
        assert result_cmp(z[f"texp{i}_golden"], host(pto.TEXP(dev(z[f"texp{i}_src"]))), 1e-3)


def test_texp_close_to_oracle():
    x = (rng(9).standard_normal(1 << 20) * 5).astype(np.float32)
    want = port.texp_f32(x)
    got = host(pto.TEXP(dev(x)))
    assert (np.abs(got - want) <= 2e-6 * want).all()  # the oracle rounds a double exp; expf is within 2 ulp


def test_softmax_vector_ops_compose():
    """The vector instruction sequence of the attention softmax, op by op against numpy fp32."""
    r = rng(11)
    x = r.standard_normal((128, 256)).astype(np.float32)
    d = dev(x)
    m = pto.TROWMAX(d)
    c = pto.TROWEXPANDSUB(d, m)
    c = pto.TMULS(c, 0.125)
    e = pto.TEXP(c)
    s = pto.TROWSUM(e)
    p = pto.TROWEXPANDDIV(e, s)
    xm = (x - x.max(axis=1, keepdims=True)) * np.float32(0.125)
    assert np.array_equal(host(c), xm)
    want = np.exp(xm.astype(np.float64))
    want = want / want.sum(axis=1, keepdims=True)
    assert np.abs(host(p) - want).max() < 1e-6
    assert np.array_equal(host(pto.TADD(d, d)), x + x)
    assert np.array_equal(host(pto.TSUB(d, e)), x - host(e))
    assert np.array_equal(host(pto.TMAX(d, e)), np.maximum(x, host(e)))
    assert np.array_equal(host(pto.TADDS(d, 1.5)), x + np.float32(1.5))
    assert np.array_equal(host(pto.TROWEXPANDMUL(d, m)), x * host(m)[:, None])
