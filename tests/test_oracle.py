"""The CPU restatement (oracle/pto_oracle.c) against (1) the golden vectors produced by the reference's
own generator scripts and (2) the reference's CPU-simulation headers compiled as oracle/_ref/libpto_ref.so.

Comparison rule for the reference's goldens is its own `ResultCmp` (tests/common/test_common.h:211-300):
an element is wrong when |diff| > eps and |diff / expected| > eps; a case passes while the number of
wrong elements is <= size * eps.  eps values are the ones the reference's test mains use.
"""
import os

import numpy as np
import pytest

import oracle

port, ref = oracle.port, oracle.ref
needs_ref = pytest.mark.skipif(ref is None, reason="reference CPU-simulation build (oracle/_ref) not present")


def result_cmp(golden, actual, eps):
    g = np.asarray(golden, np.float64).ravel()
    a = np.asarray(actual, np.float64).ravel()
    diff = np.abs(g - a)
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.where(g != 0, diff / np.abs(g), np.inf)
    bad = (diff > eps) & (rel > eps)
    return int(bad.sum()) <= g.size * eps


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


# ------------------------------------------------------------------ golden vectors (reference generators)

def test_tcvt_golden(golden_dir):
    z = load(golden_dir, "tcvt.npz")
    # tcvt case8: fp32 -> fp16 64x64, exact (tests/cpu/st/testcase/tcvt/main.cpp:126-129)
    assert np.array_equal(port.tcvt_f32_f16(z["case8_src"]).view(np.uint16), z["case8_golden"].view(np.uint16))
    for c in ("case1", "case4", "case6"):  # fp32 -> int32, CAST_RINT
        assert np.array_equal(port.tcvt_f32_i32(z[f"{c}_src"], 1), z[f"{c}_golden"])


def test_tgather_golden(golden_dir):
    z = load(golden_dir, "tgather.npz")
    names = sorted({k.split("__")[0] for k in z.files})
    assert len(names) == 23
    for n in names:
        if n.startswith("1D_"):
            src0, idx, g = z[f"{n}__src0"], z[f"{n}__idx"], z[f"{n}__golden"]
            bits = src0.view(np.uint32 if src0.itemsize == 4 else np.uint16)
            out = port.tgather(bits.view(np.float32) if src0.itemsize == 4 else bits, idx)
            assert np.array_equal(out.view(bits.dtype), g.view(bits.dtype)), n
        else:
            src, g, pat = z[f"{n}__src"], z[f"{n}__golden"], int(z[f"{n}__pattern"])
            bits = src.view(np.uint32 if src.itemsize == 4 else np.uint16)
            out = port.tgather_mask(bits.view(np.float32) if src.itemsize == 4 else bits, pat)
            assert np.array_equal(out.view(bits.dtype), g.view(bits.dtype)), n


def test_rowops_golden(golden_dir):
    z = load(golden_dir, "rowops.npz")
    for i in (0, 3, 4):  # fp32 TROWMAX cases
        src, g, (vr, vc) = z[f"trowmax{i}_src"], z[f"trowmax{i}_golden"], z[f"trowmax{i}_valid"]
        assert np.array_equal(port.trowmax_f32(src[:vr, :vc]), g)
    src, g = z["trowsum0_src"], z["trowsum0_golden"]  # fp32 TROWSUM 64x64, eps 1e-3
    assert result_cmp(g, port.trowsum_f32(src), 1e-3)
    for i in (0, 3, 4):  # fp32 TEXP cases, eps 1e-3
        assert result_cmp(z[f"texp{i}_golden"], port.texp_f32(z[f"texp{i}_src"]), 1e-3)


def test_tmatmul_golden(golden_dir):
    z = load(golden_dir, "tmatmul.npz")
    import ctypes
    P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    # case1: 40x50x60 fp16 -> fp32
    a, b, g = z["case1_a"][0], z["case1_b"][0], z["case1_golden"]
    c = np.empty(g.shape, np.float32)
    port.lib.pto_oracle_tmatmul_f16f32(P(np.ascontiguousarray(a)), P(np.ascontiguousarray(b)), P(c), 40, 50, 60)
    assert result_cmp(g, c, 1e-3)
    # case3: split-K, five 128x128x64 products accumulated == one GEMM with k = 5*128 in 64-wide steps
    a = np.concatenate(list(z["case3_a"]), axis=1)  # (128, 640)
    b = np.concatenate(list(z["case3_b"]), axis=0)  # (640, 64)
    c = np.zeros((128, 64), np.float32)
    assert port.lib.pto_oracle_gemm_f16f32_window(P(a), P(b), P(c), 128, 64, 640, 0, 0, 128, 0, 64) == 0
    assert result_cmp(z["case3_golden"], c, 1e-3)
    # case4: 120x110x50 fp32
    a, b, g = z["case4_a"][0], z["case4_b"][0], z["case4_golden"]
    c = np.empty(g.shape, np.float32)
    port.lib.pto_oracle_tmatmul_f32(P(np.ascontiguousarray(a)), P(np.ascontiguousarray(b)), P(c), 120, 110, 50)
    assert result_cmp(g, c, 1e-3)


def test_gemm_golden(golden_dir):
    # generator of kernels/manual/a2a3/gemm_performance (B handed over as n x k); kernel self-check eps 1e-3
    z = load(golden_dir, "gemm.npz")
    c = port.gemm_f16f32(z["a"], z["b_dn"], 1)
    assert result_cmp(z["golden"], c, 1e-3)
    # same product with B given k x n
    c2 = port.gemm_f16f32(z["a"], np.ascontiguousarray(z["b_dn"].T), 0)
    assert np.array_equal(c, c2)


def test_attention_golden(golden_dir):
    z = load(golden_dir, "attention.npz")
    import ctypes
    P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    # reference unit test: 64x32 fp32 head against a float64 model, eps 2e-4 (tflashattn/main.cpp:42-44)
    q, k, v, g = (np.ascontiguousarray(z[f"tflashattn_{n}"]) for n in ("q", "k", "v", "golden"))
    o = np.empty_like(g)
    port.lib.pto_oracle_attn_head_f32_plain(P(q), P(k), P(v), P(o), 64, 32)
    assert result_cmp(g, o, 2e-4)
    # streaming-softmax model of the flash-attention kernel (TILE_S1 = 256), kernel self-check eps 1e-3
    scale = 1.0 / np.sqrt(128.0)
    for name, causal in (("fa_nc_128x512", 0), ("fa_causal_128x512", 1)):
        q, k, v, g = (z[f"{name}_{n}"] for n in ("q", "k", "v", "o"))
        o = port.fa_tiled_f16(q, k, v, causal, scale, 256)
        assert result_cmp(g, o, 1e-3), name
        assert np.abs(o - g).max() < 2e-3 * max(1.0, np.abs(g).max()), name
        o_plain = port.attn_head_f16(q, k, v, causal, scale)
        assert result_cmp(g, o_plain, 1e-3), name


# ------------------------------------------------------------------ bit-exact against the reference build

def _rng(seed):
    return np.random.default_rng(seed)


@needs_ref
def test_tcvt_matches_reference_bits():
    r = _rng(1)
    special = np.array([0, -0.0, np.inf, -np.inf, np.nan, 65504, 65520, 65519.99, 1e-8, 6e-8, 5.96e-8, 2.98e-8,
                        2.9802322e-8, 3e-8, 6.1e-5, 6.1035156e-5, 1e5, -1e5, 1e-45], np.float32)
    x = np.concatenate([r.standard_normal(1 << 18).astype(np.float32), special,
                        r.integers(0, 2 ** 32, 1 << 18, dtype=np.uint32).view(np.float32)])
    assert np.array_equal(port.tcvt_f32_f16(x).view(np.uint16), ref.tcvt_f32_f16(x).view(np.uint16))
    assert np.array_equal(port.tcvt_f32_bf16(x), ref.tcvt_f32_bf16(x))
    xi = (r.standard_normal(4096) * 1000).astype(np.float32)
    xi[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5, -3.5]
    for mode in range(1, 7):
        assert np.array_equal(port.tcvt_f32_i32(xi, mode), ref.tcvt_f32_i32(xi, mode)), mode


@needs_ref
def test_bf16_rne_bit_trick():
    # the reference has no bf16 case; pin round-to-nearest-even on ties and near-ties with the integer identity
    r = _rng(2)
    u = r.integers(0, 2 ** 32, 1 << 16, dtype=np.uint32)
    u[:4096] = (u[:4096] & 0xFFFF0000) | 0x8000  # exact ties
    u[4096:8192] = (u[4096:8192] & 0xFFFF0000) | 0x7FFF
    u[8192:12288] = (u[8192:12288] & 0xFFFF0000) | 0x8001
    x = u.view(np.float32)
    finite = np.isfinite(x)
    want = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    got = ref.tcvt_f32_bf16(x)
    assert np.array_equal(got[finite], want[finite])
    assert np.array_equal(port.tcvt_f32_bf16(x), got)


@needs_ref
def test_vector_ops_match_reference_bits():
    r = _rng(3)
    x = (r.standard_normal(50000) * 4).astype(np.float32)
    assert np.array_equal(port.texp_f32(x), ref.texp_f32(x))
    m = r.standard_normal((37, 1000)).astype(np.float32)
    assert np.array_equal(port.trowmax_f32(m), ref.trowmax_f32(m))
    assert np.array_equal(port.trowsum_f32(m), ref.trowsum_f32(m))
    src = r.standard_normal((32, 1024)).astype(np.float32)
    idx = r.integers(-100, 32 * 1024 + 100, 5000).astype(np.int32)  # includes negative / too-large -> 0
    assert np.array_equal(port.tgather(src, idx), ref.tgather(src, idx))
    s16 = r.integers(0, 65536, (16, 1024)).astype(np.uint16)
    idx = r.integers(-5, 16 * 1024 + 5, 3000).astype(np.int32)
    assert np.array_equal(port.tgather(s16, idx), ref.tgather(s16, idx))
    for pat in range(1, 8):
        s = r.standard_normal((64, 256)).astype(np.float32)
        assert np.array_equal(port.tgather_mask(s, pat), ref.tgather_mask(s, pat))
        s = r.integers(0, 65536, (16, 64)).astype(np.uint16)
        assert np.array_equal(port.tgather_mask(s, pat), ref.tgather_mask(s, pat))


@needs_ref
@pytest.mark.parametrize("b_layout", [0, 1])
def test_gemm_matches_reference_bits(b_layout):
    r = _rng(4 + b_layout)
    m, n, k = 256, 512, 320
    a = r.uniform(-1, 1, (m, k)).astype(np.float16)
    b = r.uniform(-1, 1, (k, n) if b_layout == 0 else (n, k)).astype(np.float16)
    assert np.array_equal(port.gemm_f16f32(a, b, b_layout), ref.gemm_f16f32(a, b, b_layout))


@needs_ref
def test_tmatmul_unit_cases_match_reference_bits(golden_dir):
    import ctypes
    P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    z = load(golden_dir, "tmatmul.npz")
    a, b = np.ascontiguousarray(z["case1_a"][0]), np.ascontiguousarray(z["case1_b"][0])
    c1 = np.empty((40, 60), np.float32)
    c2 = np.empty((40, 60), np.float32)
    assert ref.lib.pto_ref_tmatmul_case(1, P(a), P(b), P(c1)) == 0
    port.lib.pto_oracle_tmatmul_f16f32(P(a), P(b), P(c2), 40, 50, 60)
    assert np.array_equal(c1, c2)
    assert result_cmp(z["case1_golden"], c1, 1e-3)


@needs_ref
@pytest.mark.parametrize("shape", [(128, 128, 128), (128, 512, 128), (256, 256, 128), (128, 256, 64)])
@pytest.mark.parametrize("causal", [0, 1])
def test_attention_matches_reference_bits(shape, causal):
    s0, s1, d = shape
    r = _rng(10 + s1 + causal)
    q = (r.standard_normal((s0, d)) / np.sqrt(np.sqrt(d))).astype(np.float16)
    k = (r.standard_normal((s1, d)) / np.sqrt(np.sqrt(d))).astype(np.float16)
    v = r.standard_normal((s1, d)).astype(np.float16)
    scale = 1.0 / np.sqrt(d)
    o_ref = ref.attn_head_f16(q, k, v, causal, scale)
    assert np.array_equal(port.attn_head_f16(q, k, v, causal, scale), o_ref)
    # the streaming recurrence agrees with the plain sequence to fp32 rounding
    o_t = port.fa_tiled_f16(q, k, v, causal, scale, 128)
    assert np.abs(o_t - o_ref).max() <= 2e-3 * max(np.abs(o_ref).max(), 1e-3)


@needs_ref
def test_reference_unit_test_kernel(golden_dir):
    """The unmodified reference test kernel (64x32 fp32 head) against its golden and the restatement."""
    import ctypes
    P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    z = load(golden_dir, "attention.npz")
    q, k, v, g = (np.ascontiguousarray(z[f"tflashattn_{n}"]) for n in ("q", "k", "v", "golden"))
    o1 = np.empty_like(g)
    o2 = np.empty_like(g)
    assert ref.lib.pto_ref_tflashattn_64x32(P(q), P(k), P(v), P(o1)) == 0
    port.lib.pto_oracle_attn_head_f32_plain(P(q), P(k), P(v), P(o2), 64, 32)
    assert result_cmp(g, o1, 2e-4)
    assert np.array_equal(o1, o2)


# ------------------------------------------------------------------ second batch of vector ops

OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5, "expdif": 6}


def test_vector2_golden(golden_dir):
    """Goldens of the reference's generators (numpy): exact for copies, selections and comparisons; the
    arithmetic ones within the reference test mains' eps 1e-3 (ResultCmp), in practice bit-equal except expdif."""
    z = load(golden_dir, "vector2.npz")
    x = z["trowexpand_src"]
    assert np.array_equal(port.trowexpand_f32(np.zeros_like(x), x[:, 0].copy(), 7), z["trowexpand_golden"])
    for name, op in OPS.items():
        got = port.trowexpand_f32(z[f"trowexpandop_{name}_a"], z[f"trowexpandop_{name}_s"], op)
        if name == "expdif":
            assert result_cmp(z[f"trowexpandop_{name}_golden"], got, 1e-3)
        else:
            assert np.array_equal(got, z[f"trowexpandop_{name}_golden"]), name
    for i in (0, 3, 4):  # float32 cases; 3 and 4: the tile is narrower than the tensor, the golden covers min(tile, valid)
        src, golden = z[f"trowmin{i}_src"], z[f"trowmin{i}_golden"]
        assert np.array_equal(port.trowmin_f32(src)[: golden.size], golden)
    assert np.array_equal(port.tcolreduce_f32(z["tcolmax_src"], 4), z["tcolmax_golden"])
    assert np.array_equal(port.tcolreduce_f32(z["tcolsum_src"], 0), z["tcolsum_golden"])  # small integers: exact
    for i in (0, 2):
        src, golden = z[f"tcolmin{i}_src"], z[f"tcolmin{i}_golden"]
        assert np.array_equal(port.tcolreduce_f32(src, 5)[: golden.size], golden)
    assert np.array_equal(port.ttrans(z["ttrans_src"]), z["ttrans_golden"])
    for i in range(3):
        assert np.array_equal(port.tsel(z[f"tsel{i}_mask"], z[f"tsel{i}_a"], z[f"tsel{i}_b"]), z[f"tsel{i}_golden"])
    n_cmps = 0
    for i in range(8):
        if f"tcmps{i}_src" in z:
            got = port.tcmps_f32(z[f"tcmps{i}_src"], float(z[f"tcmps{i}_scalar"][0]), int(z[f"tcmps{i}_mode"]))
            assert np.array_equal(got, z[f"tcmps{i}_golden"]), i
            n_cmps += 1
    assert n_cmps == 4
    assert np.array_equal(port.tcmp_f32(z["tcmp_a"], z["tcmp_b"], 0), z["tcmp_golden"])


@needs_ref
def test_vector2_matches_reference_bits():
    r = np.random.default_rng(77)
    bits = lambda a: np.ascontiguousarray(a).view(np.uint32)
    for rows, cols in ((64, 256), (37, 200), (1, 8), (64, 1)):
        a = r.standard_normal((rows, cols)).astype(np.float32) * 3
        s = (r.standard_normal(rows).astype(np.float32) + 2.5)
        for op in range(8):
            assert np.array_equal(bits(port.trowexpand_f32(a, s, op)), bits(ref.trowexpand_f32(a, s, op))), (rows, cols, op)
        assert np.array_equal(bits(port.trowmin_f32(a)), bits(ref.trowmin_f32(a)))
        for op in (0, 4, 5):
            assert np.array_equal(bits(port.tcolreduce_f32(a, op)), bits(ref.tcolreduce_f32(a, op))), (rows, cols, op)
        b = np.round(a)
        c = np.round(r.standard_normal((rows, cols)).astype(np.float32) * 3)
        for mode in range(6):
            assert np.array_equal(port.tcmp_f32(b, c, mode), ref.tcmp_f32(b, c, mode))
    t = r.standard_normal((64, 256)).astype(np.float32)
    for kind in (1, 2, 3):
        for vr, vc in ((64, 256), (40, 100), (1, 1)):
            assert np.array_equal(bits(port.tfillpad_f32(t, vr, vc, kind)), bits(ref.tfillpad_f32(t, vr, vc, kind)))
    u = r.standard_normal((64, 128)).astype(np.float32)
    assert np.array_equal(port.ttrans(u), ref.ttrans(u))
    for rows in (1, 50, 64):
        m = r.integers(0, 256, rows * 256 // 8, dtype=np.uint8)
        a = r.standard_normal((rows, 256)).astype(np.float32)
        b = r.standard_normal((rows, 256)).astype(np.float32)
        assert np.array_equal(port.tsel(m, a, b), ref.tsel(m, a, b))
    t2 = np.round(t * 2) / 2
    for mode in range(6):
        assert np.array_equal(port.tcmps_f32(t2, 0.5, mode), ref.tcmps_f32(t2, 0.5, mode))
        # EQ / NE use a 1e-9 window in double (include/pto/cpu/TCmps.hpp:27-33): values 1e-10 apart count as equal
    near = np.full((64, 256), 1.0, np.float32)
    assert np.array_equal(port.tcmps_f32(near, float(np.nextafter(np.float32(1.0), np.float32(2.0))), 0),
                          ref.tcmps_f32(near, float(np.nextafter(np.float32(1.0), np.float32(2.0))), 0))


def test_mxgemm_oracle_matches_reference_generator(golden_dir):
    """The restatement of the MX block-scaled fp8 GEMM reproduces, bit for bit after rounding to bfloat16, the golden
    the reference's own generator wrote (kernels/manual/a5/matmul_mxfp8_performance/scripts/gen_data.py)."""
    z = np.load(os.path.join(golden_dir, "mxgemm.npz"))
    for tag, fmt in (("e5m2", 1), ("e4m3", 0)):
        c = port.mxgemm_fp8(z[f"{tag}_a"], z[f"{tag}_b"], z[f"{tag}_scale_a"], z[f"{tag}_scale_b"], fmt, fmt)
        u = c.view(np.uint32).astype(np.uint64)
        bits = ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        assert np.array_equal(bits, z[f"{tag}_golden_bf16_bits"]), tag


def test_mxgemm_oracle_fp8_decoding_against_torch():
    """All 256 codes of both fp8 formats, through a one-element product with unit scales."""
    import torch
    codes = np.arange(256, dtype=np.uint8)
    one = {1: 0x3c, 0: 0x38}  # 1.0 in e5m2 / e4m3
    for fmt, tdt in ((1, torch.float8_e5m2), (0, torch.float8_e4m3fn)):
        a = np.zeros((256, 32), np.uint8)
        a[:, 0] = codes
        b = np.zeros((1, 32), np.uint8)
        b[0, 0] = one[fmt]
        s = np.full((256, 1), 127, np.uint8)
        got = port.mxgemm_fp8(a, b, s, s[:1], fmt, fmt)[:, 0]
        want = torch.from_numpy(codes).view(tdt).float().numpy()
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got[ok], want[ok])


def test_mxgemm_fp4_oracle_matches_reference_generator(golden_dir):
    """Packed fp4 form: nibble order, e2m1 decoding and scale handling of the restatement against the golden of the
    reference's generator (kernels/manual/a5/matmul_mxfp4_performance/scripts/gen_data.py), bit for bit in bfloat16."""
    z = np.load(os.path.join(golden_dir, "mxgemm_fp4.npz"))
    c = port.mxgemm_fp4(z["a"], z["b"], z["scale_a"], z["scale_b"])
    u = c.view(np.uint32).astype(np.uint64)
    bits = ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(bits, z["golden_bf16_bits"])


def test_mxgemm_fp4_oracle_decodes_all_codes():
    """All 16 e2m1 codes in both nibble positions against ml_dtypes' float4_e2m1fn."""
    ml_dtypes = pytest.importorskip("ml_dtypes")
    codes = np.arange(16, dtype=np.uint8)
    want = codes.view(ml_dtypes.float4_e2m1fn).astype(np.float32)
    one = np.zeros((1, 16), np.uint8)
    s = np.full((16, 1), 127, np.uint8)
    for pos in (0, 1):
        a = np.zeros((16, 16), np.uint8)
        a[:, 0] = codes << (4 * pos)
        one[0, 0] = 0x2 << (4 * pos)  # 1.0 in the same position
        got = port.mxgemm_fp4(a, one, s, s[:1])[:, 0]
        assert np.array_equal(got, want), pos


@pytest.mark.parametrize("diagonal", [-70, -2, 0, 1, 5, 300])
@pytest.mark.parametrize("upper", [0, 1])
def test_ttri_restatement_against_reference_build_and_numpy(diagonal, upper):
    """TTRI (include/pto/cpu/TTRI.hpp:30-77): the restatement equals numpy's tril / triu of ones and, where the
    reference build is present, the reference's own implementation on a 64 x 256 tile and a 40 x 100 corner."""
    for rows, cols in ((64, 256), (40, 100), (1, 1)):
        got = port.ttri_f32(rows, cols, diagonal, upper)
        ones = np.ones((rows, cols), np.float32)
        want = np.triu(ones, diagonal) if upper else np.tril(ones, diagonal)
        assert np.array_equal(got, want)
        if oracle.ref is not None:
            assert np.array_equal(oracle.ref.ttri_f32(rows, cols, diagonal, upper), want), (rows, cols)


def test_tmatmul_i8_oracle_matches_reference_generator(golden_dir):
    """(int8, int8 -> int32): exact equality with the golden of tests/cpu/st/testcase/tmatmul/gen_data.py."""
    z = np.load(os.path.join(golden_dir, "tmatmul_i8.npz"))
    for name in ("small", "mid"):
        assert np.array_equal(port.tmatmul_i8i32(z[name + "_a"], z[name + "_b"]), z[name + "_golden"])
