"""Tile programs written against this repository's PTO headers (pto_isa_b200/csrc/pto_programs/programs.cu),
run on the GPU and checked against the CPU oracle: TGATHER (index and mask forms), the softmax instruction
chain, TMATMUL with a k x n (Layout::ND) second operand, and a whole attention head built from PTO
instructions (TLOAD / TMOV / TMATMUL / TROWMAX / TROWEXPANDSUB / TMULS / TEXP / TROWSUM / TCVT / TROWEXPANDDIV /
TSTORE)."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle
from util import attn_err_ok, dev, host, rel_err_ok

pytestmark = pytest.mark.gpu
port = oracle.port
_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "pto_isa_b200",
                   "libpto_b200_programs.so")


@pytest.fixture(scope="module")
def prog():
    lib = ctypes.CDLL(_SO)  # built by pto_isa_b200.build; its absence is an error, not a skip
    return lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_tgather_index_program(prog):
    r = np.random.default_rng(1)
    src = r.standard_normal((32, 1024)).astype(np.float32)
    idx = r.integers(-50, 32 * 1024 + 50, (16, 64)).astype(np.int32)
    out = torch.full((16, 64), 7.0, device="cuda")
    assert prog.pto_prog_tgather_index_f32(_ptr(out), _ptr(dev(src)), _ptr(dev(idx)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out), port.tgather(src, idx))
    s16 = r.integers(0, 65536, (16, 1024)).astype(np.uint16)
    i16 = r.integers(-5, 16 * 1024 + 5, (16, 128)).astype(np.int32)
    o16 = torch.zeros(16, 128, dtype=torch.int16, device="cuda")
    assert prog.pto_prog_tgather_index_b16(_ptr(o16), _ptr(dev(s16.view(np.int16))), _ptr(dev(i16)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(o16).view(np.uint16), port.tgather(s16, i16))


def test_tgather_mask_program(prog):
    r = np.random.default_rng(2)
    src = r.standard_normal((64, 256)).astype(np.float32)
    d = dev(src)
    for pat in range(1, 8):
        want = port.tgather_mask(src, pat)
        out = torch.zeros(want.size, device="cuda")
        assert prog.pto_prog_tgather_mask_f32(_ptr(out), _ptr(d), pat, _stream()) == 0
        torch.cuda.synchronize()
        assert np.array_equal(host(out), want), pat


def test_row_softmax_program(prog):
    r = np.random.default_rng(3)
    x = (r.standard_normal((64, 256)) * 3).astype(np.float32)
    out = torch.zeros(64, 256, device="cuda")
    mx = torch.zeros(64, device="cuda")
    sm = torch.zeros(64, device="cuda")
    scale = np.float32(0.125)
    assert prog.pto_prog_row_softmax_64x256(_ptr(out), _ptr(mx), _ptr(sm), _ptr(dev(x)), ctypes.c_float(scale),
                                            _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(mx), port.trowmax_f32(x))
    p = port.texp_f32(((x - x.max(axis=1, keepdims=True)) * scale).astype(np.float32))
    s = port.trowsum_f32(p)
    assert np.abs(host(sm) - s).max() <= 1e-5 * s.max()
    assert np.abs(host(out) - p / s[:, None]).max() <= 1e-6


def test_matmul_nd_program(prog):
    r = np.random.default_rng(4)
    a = r.uniform(-1, 1, (128, 128)).astype(np.float16)
    b = r.uniform(-1, 1, (128, 256)).astype(np.float16)
    out = torch.full((128, 256), float("nan"), device="cuda")
    assert prog.pto_prog_matmul_nd_128x128x256(_ptr(out), _ptr(dev(a)), _ptr(dev(b)), _stream()) == 0
    torch.cuda.synchronize()
    want = port.gemm_f16f32(a, b, 0)
    ok, worst = rel_err_ok(host(out), want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"


def test_attention_head_program(prog):
    r = np.random.default_rng(5)
    s0, s1, d = 128, 128, 64
    q = r.standard_normal((s0, d)).astype(np.float16)
    k = r.standard_normal((s1, d)).astype(np.float16)
    v = r.standard_normal((s1, d)).astype(np.float16)
    scale = 1.0 / np.sqrt(d)
    o = torch.full((s0, d), float("nan"), device="cuda")
    assert prog.pto_prog_attention_head_128x128x64(_ptr(o), _ptr(dev(q)), _ptr(dev(k)), _ptr(dev(v)),
                                                   ctypes.c_float(scale), _stream()) == 0
    torch.cuda.synchronize()
    want = port.attn_head_f16(q, k, v, 0, scale)
    ok, worst, frac = attn_err_ok(host(o), want)
    assert ok, f"max relative error {worst:.3e}, {frac:.5f} within tolerance"


def test_row_softmax_tutorial_program(prog):
    """The tutorial's decomposition (TROWMAX, TROWEXPAND + TSUB, TEXP, TROWSUM, TROWEXPAND + TDIV)."""
    r = np.random.default_rng(21)
    x = (r.standard_normal((64, 256)) * 4).astype(np.float32)
    out = torch.zeros(64, 256, device="cuda")
    assert prog.pto_prog_row_softmax_tutorial_64x256(_ptr(out), _ptr(dev(x)), _stream()) == 0
    torch.cuda.synchronize()
    mx = port.trowmax_f32(x)
    e = port.texp_f32(port.trowexpand_f32(x, mx, 1))
    want = e / port.trowsum_f32(e)[:, None]
    ok, worst = rel_err_ok(host(out), want, 2e-6)  # expf and the row sum's order differ from the CPU's in the last bits
    assert ok, worst
    assert np.allclose(host(out).sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("valid", [(64, 128), (40, 100), (1, 1)])
def test_vector2_program(prog, valid):
    """TFILLPAD, TROWMIN, TCOLMAX / TCOLSUM / TCOLMIN, TTRANS, TCMPS + TSEL, TROWEXPAND{MAX,MIN,EXPDIF}, TROWEXPAND, TCMP
    issued as PTO instructions on shared-memory tiles: bit-equal to the oracle (EXPDIF: one ulp)."""
    vr, vc = valid
    r = np.random.default_rng(22)
    a = r.standard_normal((64, 128)).astype(np.float32)
    b = r.standard_normal((64, 128)).astype(np.float32)
    s = (r.standard_normal(64) * 0.5).astype(np.float32)
    names = ["fill", "rowmin", "colmax", "colsum", "colmin", "trans", "sel", "emax", "emin", "edif", "expand", "cmp"]
    shapes = {"rowmin": (64,), "colmax": (128,), "colsum": (128,), "colmin": (128,), "trans": (128, 64)}
    outs = {n: torch.full(shapes.get(n, (64, 128)), -7.0, device="cuda") for n in names}
    bits = torch.zeros(64 * 128 // 8, dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_void_p * 13)(*[outs[n].data_ptr() for n in names], bits.data_ptr())
    assert prog.pto_prog_vector2_64x128(ptrs, _ptr(dev(a)), _ptr(dev(b)), _ptr(dev(s)), vr, vc, _stream()) == 0
    torch.cuda.synchronize()
    u32 = lambda x: np.ascontiguousarray(x).view(np.uint32)
    fill = port.tfillpad_f32(a, vr, vc, 2)
    assert np.array_equal(u32(host(outs["fill"])), u32(fill))
    assert np.array_equal(u32(host(outs["rowmin"])), u32(port.trowmin_f32(fill)))
    assert np.array_equal(u32(host(outs["colmax"])), u32(port.tcolreduce_f32(a, 4)))
    assert np.array_equal(u32(host(outs["colsum"])), u32(port.tcolreduce_f32(a, 0)))  # same top-to-bottom order
    assert np.array_equal(u32(host(outs["colmin"])), u32(port.tcolreduce_f32(a, 5)))
    assert np.array_equal(host(outs["trans"]), port.ttrans(a))
    want_bits = port.tcmps_f32(a, 0.25, 4)
    assert np.array_equal(host(bits), want_bits)
    assert np.array_equal(host(outs["sel"]), port.tsel(want_bits, a, b))
    assert np.array_equal(u32(host(outs["emax"])), u32(port.trowexpand_f32(a, s, 4)))
    assert np.array_equal(u32(host(outs["emin"])), u32(port.trowexpand_f32(a, s, 5)))
    got, want = u32(host(outs["edif"])).astype(np.int64), u32(port.trowexpand_f32(a, s, 6)).astype(np.int64)
    assert np.all(np.abs(got - want) <= 1)
    assert np.array_equal(u32(host(outs["expand"])), u32(port.trowexpand_f32(a, s, 7)))
    assert np.array_equal(host(outs["cmp"]), port.tcmp_f32(a, b, 2))


def test_tmatmul_bias_program(prog, golden_dir):
    """TMATMUL_BIAS as a PTO instruction (bias row in a TileType::Bias tile, written into tensor memory under the
    product) in the sequence of the reference's unit-test kernel, against the golden of the reference's generator
    (integer-valued operands: exact) and against the oracle product plus bias on random operands."""
    z = np.load(os.path.join(golden_dir, "tmatmul_bias.npz"))
    out = torch.zeros(128, 256, device="cuda")
    assert prog.pto_prog_tmatmul_bias_128x64x256(_ptr(out), _ptr(dev(z["a"].view(np.int16))), _ptr(dev(z["b"].view(np.int16))),
                                                 _ptr(dev(z["bias"])), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out), z["golden"])
    r = np.random.default_rng(3)
    a = r.uniform(-1, 1, (128, 64)).astype(np.float16)
    b = r.uniform(-1, 1, (64, 256)).astype(np.float16)
    bias = r.uniform(-10, 10, 256).astype(np.float32)
    assert prog.pto_prog_tmatmul_bias_128x64x256(_ptr(out), _ptr(dev(a.view(np.int16))), _ptr(dev(b.view(np.int16))),
                                                 _ptr(dev(bias)), _stream()) == 0
    torch.cuda.synchronize()
    want = a.astype(np.float64) @ b.astype(np.float64) + bias[None, :]
    ok, worst = rel_err_ok(host(out), want, 2e-3)
    assert ok, worst


@pytest.mark.parametrize("diagonal", [1, 0, -5, 40, 200])
def test_tri_reshape_program(prog, diagonal):
    """TTRI (upper, times the lowest float, added to the logits: the causal mask of the reference's streaming softmax),
    TTRI (lower), TRESHAPE 64 x 128 -> 128 x 64 and the row maxima of the reshaped tile, as PTO instructions."""
    r = np.random.default_rng(7)
    x = r.standard_normal((64, 128)).astype(np.float32)
    masked = torch.full((64, 128), 5.0, device="cuda")
    tril = torch.full((64, 128), 5.0, device="cuda")
    rowmax = torch.full((128,), 5.0, device="cuda")
    assert prog.pto_prog_tri_reshape_64x128(_ptr(masked), _ptr(tril), _ptr(rowmax), _ptr(dev(x)), diagonal, _stream()) == 0
    torch.cuda.synchronize()
    mask = port.ttri_f32(64, 128, diagonal, 1) * np.float32(-3.40282e38)
    want = x + mask
    u32 = lambda a: np.ascontiguousarray(a).view(np.uint32)
    assert np.array_equal(u32(host(masked)), u32(want))
    assert np.array_equal(host(tril), port.ttri_f32(64, 128, -2, 0))
    assert np.array_equal(host(rowmax), want.reshape(128, 64).max(axis=1))


def test_mla_head_program(prog, golden_dir):
    """The instruction sequence of the reference's multi-latent-attention demo (latent projections, TTRANS of K_lat,
    scaled scores, row softmax, context, output projection) on the GPU against the same sequence run by the
    reference's CPU simulation (tests/golden/mla.npz).  Five chained fp16 products with fp16 hand-offs: tolerance 2e-3
    of max(|x|, rms), as for the GEMM and attention."""
    import os
    z = np.load(os.path.join(golden_dir, "mla.npz"))
    out = torch.zeros(128, 64, device="cuda")
    h = lambda name: dev(z[name].view(np.int16))
    ops = [h(n) for n in ("q", "k", "v", "wq", "wk", "wv", "wo")]
    rc = prog.pto_prog_mla_head_128x64x64(_ptr(out), *[_ptr(t) for t in ops], ctypes.c_float(float(z["scale"])), _stream())
    assert rc == 0
    torch.cuda.synchronize()
    ok, worst = rel_err_ok(host(out), z["o"], 2e-3)
    assert ok, worst
    if oracle.ref is not None:  # the reference build itself, when it travelled along
        P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        o2 = np.zeros((128, 64), np.float32)
        arrs = [np.ascontiguousarray(z[n]) for n in ("q", "k", "v", "wq", "wk", "wv", "wo")]
        assert oracle.ref.lib.pto_ref_mla_head_f16_128x64x64(*[P(a) for a in arrs], P(o2), ctypes.c_float(float(z["scale"]))) == 0
        assert np.array_equal(o2, z["o"])


@pytest.mark.parametrize("fmt", [1, 0], ids=["e5m2", "e4m3"])
def test_tmatmul_mx_tile_program(prog, fmt):
    """TMATMUL_MX as a tile instruction (include/pto/common/pto_instr.hpp:403-460 in the reference): TLOAD of fp8 data and
    e8m0 scale tiles, TEXTRACT of the k block of each (the scale tiles become the tensor core's atoms), the product
    with block scaling and its accumulating form, TSTORE with conversion to bfloat16.  Checked like the C-ABI MX GEMM:
    against the oracle's exact sums, within one bfloat16 ulp."""
    from test_mxgemm_gpu import check_bf16, make
    m, n, k = 128, 256, 256
    a, b, sa, sb = make(m, n, k, fmt, seed=31 + fmt)
    want = port.mxgemm_fp8(a, b, sa, sb, fmt, fmt)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert prog.pto_prog_mx_matmul_128x256x256(_ptr(out), _ptr(dev(a)), _ptr(dev(b)), _ptr(dev(sa)), _ptr(dev(sb)), fmt,
                                               _stream(), _ptr(status)) == 0
    torch.cuda.synchronize()
    assert host(status).tolist() == [0, 0, 0, 0]
    check_bf16(host(out.view(torch.int16)).view(np.uint16), want)
