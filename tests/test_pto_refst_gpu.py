"""The reference's unit-test tile programs and flash-attention macro headers, compiled unchanged against this
repository's PTO headers (pto_isa_b200/csrc/refkernels/wrappers.cu.in lists them), run on the GPU.

tests/cpu/st/testcase/{tload,tstore,tgather,tmatmul,trowmax,trowsum,texp}/*_kernel.cpp are checked at the reference's
own tolerances: eps 0 for TLOAD / TSTORE / TGATHER (tload/main.cpp:123, tstore/main.cpp:88), the goldens of the
reference's generators for TMATMUL (tests/golden/tmatmul.npz, ResultCmp eps 1e-3) with the CUDA-core forms (fp32, int8)
bit-exact against the simulation's sum order.  TEXTRACT windows are read back bit for bit.  One attention head is built
from pto_macro_matmul / pto_macro_fa_softmax / pto_macro_fa_gu and three TPipe rings (TPUSH / TPOP) and compared with
the oracle's streaming formulation.  A wait that nothing satisfies must give up, report and leave the GPU usable.

The library under test is built where the reference tree is available; the tests skip when it is absent."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle
from util import dev, host, rel_err_ok, result_cmp

pytestmark = pytest.mark.gpu
port = oracle.port
_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(os.path.dirname(_HERE), "pto_isa_b200", "libpto_b200_refkernels.so")


@pytest.fixture(scope="module")
def refk():
    if not os.path.exists(_SO):
        pytest.skip("libpto_b200_refkernels.so has not been built (needs the reference tree at build time)")
    lib = ctypes.CDLL(_SO)
    lib.pto_refk_wait_that_runs_out.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_void_p,
                                                ctypes.c_void_p]
    return lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _bytes_dev(a):
    return torch.from_numpy(np.frombuffer(a.tobytes(), np.uint8).copy()).cuda()


# ---------------------------------------------------------------- TLOAD: the reference's ten cases, its own goldens
@pytest.mark.parametrize("key", range(1, 11))
def test_reference_tload_cases(refk, key):
    inp = np.zeros(1 << 20, np.uint8)
    gold = np.zeros(1 << 20, np.uint8)
    n = refk.pto_refk_tload_golden(key, inp.ctypes.data_as(ctypes.c_void_p), gold.ctypes.data_as(ctypes.c_void_p))
    assert n > 0
    src = torch.from_numpy(inp).cuda()
    out = torch.full((n,), 0xA5, dtype=torch.uint8, device="cuda")
    assert refk.pto_refk_tload(key, _ptr(out), _ptr(src), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out), gold[:n]), f"TLOAD case {key}"


# ---------------------------------------------------------------- TSTORE: sub-block of a larger tensor, eps 0
_TSTORE_CASES = [
    (0, "ND", np.float32, (1, 1, 1, 2, 128), (1, 1, 1, 2, 128)),
    (1, "ND", np.int16, (1, 2, 1, 23, 121), (3, 2, 2, 35, 125)),
    (2, "ND", np.int8, (2, 2, 3, 23, 47), (3, 3, 4, 32, 50)),
    (3, "DN", np.float32, (1, 1, 1, 4, 21), (1, 1, 1, 8, 32)),
    (4, "DN", np.int16, (3, 1, 1, 1, 124), (5, 1, 1, 2, 128)),
    (5, "DN", np.int8, (2, 1, 2, 32, 32), (3, 4, 3, 64, 35)),
    (6, "ND", np.int64, (1, 1, 1, 2, 128), (1, 1, 1, 2, 128)),
    (7, "ND", np.uint64, (1, 2, 1, 23, 121), (3, 2, 2, 35, 125)),
    (8, "DN", np.int64, (1, 1, 1, 4, 21), (1, 1, 1, 8, 32)),
]


@pytest.mark.parametrize("case", _TSTORE_CASES, ids=lambda c: f"{c[1]}_{np.dtype(c[2]).name}_{c[0]}")
def test_reference_tstore_cases(refk, case):
    """The data rule of tests/cpu/st/testcase/tstore/gen_data.py:19-46."""
    key, fmt, dt, g, w = case
    r = np.random.default_rng(19 + key)
    if fmt == "ND":
        shape = w
        sub = tuple(slice(0, n) for n in g)
    else:
        shape = (w[0], w[1], w[2], w[4], w[3])
        sub = (slice(0, g[0]), slice(0, g[1]), slice(0, g[2]), slice(0, g[4]), slice(0, g[3]))
    inp = r.integers(-5, 5, size=shape).astype(dt)
    want = np.zeros(shape, dt)
    want[sub] = inp[sub]
    out = _bytes_dev(np.zeros(shape, dt))
    assert refk.pto_refk_tstore(key, _ptr(out), _ptr(_bytes_dev(inp)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out).view(dt).reshape(shape), want)


# ---------------------------------------------------------------- TGATHER
_MASK_CASES = {  # key: (dtype, rows, cols, pattern)  -- tgather_common.h:14-61
    1: (np.float32, 4, 64, 1), 2: (np.float32, 7, 1024, 2), 3: (np.float32, 3, 1056, 3), 4: (np.float32, 4, 128, 4),
    5: (np.float32, 5, 256, 5), 6: (np.float32, 6, 288, 6), 7: (np.float32, 7, 320, 7),
    11: (np.float16, 5, 128, 1), 12: (np.float16, 7, 1024, 2), 13: (np.float16, 3, 1056, 3),
    15: (np.float16, 5, 256, 5), 16: (np.float16, 6, 288, 6),
    21: (np.uint16, 5, 128, 1), 22: (np.uint16, 7, 1024, 2), 23: (np.int16, 3, 1056, 3), 24: (np.int16, 4, 128, 4),
    25: (np.uint32, 5, 256, 5), 26: (np.int32, 6, 288, 6), 27: (np.int32, 7, 320, 7),
}


@pytest.mark.parametrize("key", sorted(_MASK_CASES))
def test_reference_tgather_mask_cases(refk, key):
    dt, rows, cols, pattern = _MASK_CASES[key]
    r = np.random.default_rng(key)
    raw = r.integers(0, 1 << (8 * np.dtype(dt).itemsize - 2), (rows, cols)).astype(
        np.uint16 if np.dtype(dt).itemsize == 2 else np.uint32)
    want = port.tgather_mask(raw, pattern)  # packed selection, as the program's dst tile holds it from offset 0
    out = _bytes_dev(np.zeros((rows, cols), raw.dtype))
    assert refk.pto_refk_tgather_mask(key, _ptr(out), _ptr(_bytes_dev(raw)), _stream()) == 0
    torch.cuda.synchronize()
    got = host(out).view(raw.dtype)
    assert np.array_equal(got[:want.size], want.ravel()), f"TGATHER mask case {key}"


@pytest.mark.parametrize("key,dt,src_shape,idx_shape", [(0, np.float32, (32, 1024), (16, 64)),
                                                       (1, np.int32, (32, 512), (16, 256)),
                                                       (2, np.int16, (16, 1024), (16, 128)),
                                                       (3, np.int16, (32, 256), (32, 64))])
def test_reference_tgather_index_cases(refk, key, dt, src_shape, idx_shape):
    r = np.random.default_rng(100 + key)
    src = r.integers(-30000, 30000, src_shape).astype(dt)
    if dt == np.float32:
        src = r.standard_normal(src_shape).astype(np.float32)
    n = src_shape[0] * src_shape[1]
    idx = r.integers(-20, n + 20, idx_shape).astype(np.int32)
    raw = src.view(np.uint32 if src.itemsize == 4 else np.uint16)
    want = port.tgather(raw, idx)
    out = _bytes_dev(np.zeros(idx_shape, raw.dtype))
    assert refk.pto_refk_tgather_index(key, _ptr(out), _ptr(_bytes_dev(raw)), _ptr(dev(idx)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out).view(raw.dtype).reshape(idx_shape), want)


# ---------------------------------------------------------------- TMATMUL
def _seq_matmul(a, b, acc_dtype):
    """One sum over k per element, products and sums rounded separately (include/pto/cpu/TMatmul.hpp:22-37)."""
    c = np.zeros((a.shape[0], b.shape[1]), acc_dtype)
    for k in range(a.shape[1]):
        c = (c + (a[:, k:k + 1].astype(acc_dtype) * b[k:k + 1, :].astype(acc_dtype)).astype(acc_dtype)).astype(acc_dtype)
    return c


def test_reference_tmatmul_cases(refk, golden_dir):
    z = np.load(os.path.join(golden_dir, "tmatmul.npz"))
    # key 1: half 40 x 50 x 60 (ragged, tensor core); key 3: five accumulated 128 x 128 x 64 products
    for key, name in ((1, "case1"), (3, "case3")):
        a, b, g = z[f"{name}_a"], z[f"{name}_b"], z[f"{name}_golden"]
        out = torch.full(g.shape, float("nan"), device="cuda")
        assert refk.pto_refk_tmatmul(key, _ptr(out), _ptr(dev(a)), _ptr(dev(b)), _stream()) == 0
        torch.cuda.synchronize()
        assert result_cmp(g, host(out), 1e-3), name
        ok, worst = rel_err_ok(host(out), g, 2e-3, label=f"reference tmatmul {name}")
        assert ok, f"{name}: max relative error {worst:.3e}"
    # key 4: fp32 120 x 110 x 50 on the CUDA cores, bit-exact against the simulation's sum order
    a, b, g = z["case4_a"][0], z["case4_b"][0], z["case4_golden"]
    out = torch.full(g.shape, float("nan"), device="cuda")
    assert refk.pto_refk_tmatmul(4, _ptr(out), _ptr(dev(a)), _ptr(dev(b)), _stream()) == 0
    torch.cuda.synchronize()
    assert result_cmp(g, host(out), 1e-3)
    assert np.array_equal(host(out), _seq_matmul(a, b, np.float32))
    # key 2: int8 6 x 7 x 8
    r = np.random.default_rng(2)
    a8 = r.integers(-128, 128, (6, 7)).astype(np.int8)
    b8 = r.integers(-128, 128, (7, 8)).astype(np.int8)
    out = torch.zeros(6, 8, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_tmatmul(2, _ptr(out), _ptr(dev(a8)), _ptr(dev(b8)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out), a8.astype(np.int32) @ b8.astype(np.int32))


def test_reference_tmatmul_bias_cases(refk):
    r = np.random.default_rng(5)
    # key 1: int8 8 x 7 x 6 with an int32 bias
    a8 = r.integers(-128, 128, (8, 7)).astype(np.int8)
    b8 = r.integers(-128, 128, (7, 6)).astype(np.int8)
    bias = r.integers(-1000, 1000, 6).astype(np.int32)
    out = torch.zeros(8, 6, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_tmatmul_bias(1, _ptr(out), _ptr(dev(a8)), _ptr(dev(b8)), _ptr(dev(bias)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out), a8.astype(np.int32) @ b8.astype(np.int32) + bias)
    # key 2: half 16 x 15 x 16 with an fp32 bias (tensor core)
    a = r.uniform(-1, 1, (16, 15)).astype(np.float16)
    b = r.uniform(-1, 1, (15, 16)).astype(np.float16)
    fb = r.uniform(-1, 1, 16).astype(np.float32)
    out = torch.full((16, 16), float("nan"), device="cuda")
    assert refk.pto_refk_tmatmul_bias(2, _ptr(out), _ptr(dev(a)), _ptr(dev(b)), _ptr(dev(fb)), _stream()) == 0
    torch.cuda.synchronize()
    want = a.astype(np.float64) @ b.astype(np.float64) + fb
    ok, worst = rel_err_ok(host(out), want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"
    # key 5: fp32 127 x 128 x 63 with bias, bit-exact against the simulation's order (sum over k, then + bias)
    a = r.standard_normal((127, 128)).astype(np.float32)
    b = r.standard_normal((128, 63)).astype(np.float32)
    fb = r.standard_normal(63).astype(np.float32)
    out = torch.full((127, 63), float("nan"), device="cuda")
    assert refk.pto_refk_tmatmul_bias(5, _ptr(out), _ptr(dev(a)), _ptr(dev(b)), _ptr(dev(fb)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out), (_seq_matmul(a, b, np.float32) + fb).astype(np.float32))


# ---------------------------------------------------------------- TROWMAX / TROWSUM / TEXP
def test_reference_row_and_exp_programs(refk):
    r = np.random.default_rng(7)
    x = r.standard_normal((64, 64)).astype(np.float32)
    out = torch.zeros(64, device="cuda")
    assert refk.pto_refk_trowmax(0, _ptr(out), _ptr(dev(x)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out), port.trowmax_f32(x))
    xh = r.standard_normal((64, 64)).astype(np.float16)
    outh = torch.zeros(64, dtype=torch.float16, device="cuda")
    assert refk.pto_refk_trowmax(1, _ptr(outh), _ptr(dev(xh)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(outh), xh.max(axis=1))
    x2 = r.standard_normal((32, 16)).astype(np.float32)
    out2 = torch.zeros(32, device="cuda")
    assert refk.pto_refk_trowmax(2, _ptr(out2), _ptr(dev(x2)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(out2), x2.max(axis=1))
    outs = torch.full((64, 64), 9.0, device="cuda")  # the program stores its whole destination tile; sums in column 0
    assert refk.pto_refk_trowsum_f32_64x64(_ptr(outs), _ptr(dev(x)), _stream()) == 0
    torch.cuda.synchronize()
    want = port.trowsum_f32(x)
    assert np.abs(host(outs)[:, 0] - want).max() <= 2e-6 * np.abs(x).sum(axis=1).max()  # tree sum / sequential sum
    assert not host(outs)[:, 1:].any()  # the rest of the tile is what the program's std::fill left there
    oute = torch.zeros(64, 64, device="cuda")
    assert refk.pto_refk_texp(0, _ptr(oute), _ptr(dev(x)), _stream()) == 0
    torch.cuda.synchronize()
    assert result_cmp(port.texp_f32(x), host(oute), 1e-3)
    ok, worst = rel_err_ok(host(oute), port.texp_f32(x), 1e-6)
    assert ok, f"TEXP max relative error {worst:.3e}"


# ---------------------------------------------------------------- the flash-attention unit-test program
def test_reference_tflashattn_program(refk, golden_dir):
    """tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp unchanged: a 64 x 32 fp32 head in fifteen instructions
    with no TASSIGN (every tile keeps the storage it was constructed with) and no flags.  Checked against the golden of
    the reference's generator at the unit test's eps (tflashattn/main.cpp:42-44, 2e-4) and against the oracle's
    restatement of the same instruction sequence, from which it may differ only by the exponential's last bits and
    the row sum's order."""
    z = np.load(os.path.join(golden_dir, "attention.npz"))
    q, k, v, g = (np.ascontiguousarray(z[f"tflashattn_{n}"]) for n in ("q", "k", "v", "golden"))
    out = torch.full((64, 32), 7.0, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_tflashattn_64x32(_ptr(out), _ptr(dev(q)), _ptr(dev(k)), _ptr(dev(v)), _stream(), _ptr(status)) == 0
    torch.cuda.synchronize()
    assert host(status).tolist() == [0, 0, 0, 0]
    assert result_cmp(g, host(out), 2e-4)
    want = np.empty_like(g)
    P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    port.lib.pto_oracle_attn_head_f32_plain(P(q), P(k), P(v), P(want), 64, 32)
    ok, worst = rel_err_ok(host(out), want, 1e-5, label="tflashattn unit-test program 64x32 f32")
    assert ok, f"max relative error {worst:.3e}"


# ---------------------------------------------------------------- TEXTRACT, bit for bit
@pytest.mark.parametrize("which,kstep", [(0, 0), (1, 0), (2, 0), (3, 0), (3, 3), (4, 0), (4, 2), (5, 0), (6, 0)])
def test_textract_windows_bit_exact(refk, which, kstep):
    """The window is fed through TMATMUL with an identity operand: each output is one source element times one plus
    exact zeros, so the result equals the window exactly.  Golden rule of tests/cpu/st/testcase/textract/gen_data.py:
    golden = src[idx_row:, idx_col:]."""
    r = np.random.default_rng(40 + which)
    if which <= 2:
        vr, vc = (31, 31) if which == 2 else (32, 32)
        ir, ic = (0, 0) if which == 0 else (8, 16)
        src = np.arange(1, vr * vc + 1).reshape(vr, vc).astype(np.float16)  # the reference generator's input
        out_shape, ident_n, cdt = (32, 32 - ic), 32 - ic, np.float32
    elif which == 3:
        vr, vc, ir, ic = 128, 256, 0, 64 * kstep
        src = r.uniform(-1, 1, (vr, vc)).astype(np.float16)
        src[1, ic:ic + 4] = [6.1e-5, 5.96e-8, 65504.0, -65504.0]  # smallest normal, smallest subnormal, largest
        out_shape, ident_n, cdt = (128, 64), 64, np.float32
    elif which == 4:
        vr, vc, ir, ic = 256, 256, 64 * kstep, 0
        src = r.uniform(-1, 1, (vr, vc)).astype(np.float16)
        out_shape, ident_n, cdt = (64, 256), 64, np.float32
    elif which == 5:
        vr, vc, ir, ic = 125, 93, 8, 16
        src = r.standard_normal((vr, vc)).astype(np.float32)
        out_shape, ident_n, cdt = (128, 80), 80, np.float32
    else:
        vr, vc, ir, ic = 125, 61, 8, 16
        src = r.integers(-128, 128, (vr, vc)).astype(np.int8)
        out_shape, ident_n, cdt = (128, 48), 48, np.int32
    ident = np.eye(ident_n, dtype=src.dtype)
    out = _bytes_dev(np.full(out_shape, 77, cdt))
    assert refk.pto_refk_textract(which, kstep, _ptr(out), _ptr(_bytes_dev(src)), _ptr(_bytes_dev(ident)), _stream()) == 0
    torch.cuda.synchronize()
    got = host(out).view(cdt).reshape(out_shape)
    window = src[ir:, ic:]
    want = np.zeros(out_shape, cdt)  # outside the source's valid region the operand is zero
    h, w = min(window.shape[0], out_shape[0]), min(window.shape[1], out_shape[1])
    want[:h, :w] = window[:h, :w].astype(cdt)
    assert np.array_equal(got, want), f"TEXTRACT case {which} kstep {kstep}"


# ---------------------------------------------------------------- the flash-attention macros and pipes
def _newton_inv_sqrt(x):
    """constexpr_inv_sqrt of kernels/manual/common/flash_atten/pto_macro_fa_softmax.hpp:31-45 in fp32."""
    x = np.float32(x)
    g = x
    for _ in range(8):
        g = np.float32(0.5) * (g + x / g)
    return np.float32(1.0) / g


@pytest.fixture(scope="module")
def refk_pw():
    so = _SO.replace("refkernels.so", "refkernels_pw.so")
    if not os.path.exists(so):
        pytest.skip("libpto_b200_refkernels_pw.so has not been built (needs the reference tree at build time)")
    return ctypes.CDLL(so)


@pytest.mark.parametrize("pipe_warps", [0, 1], ids=["one_stream", "pipe_warps"])
@pytest.mark.parametrize("fifo", [0, 1], ids=["gm_fifo", "smem_fifo"])
@pytest.mark.parametrize("causal", [0, 1])
@pytest.mark.parametrize("s0,s1", [(32, 64), (64, 256), (128, 128)])
def test_reference_fa_macros_one_head(refk, refk_pw, s0, s1, causal, fifo, pipe_warps):
    """One attention head built from pto_macro_matmul / pto_macro_fa_softmax / pto_macro_fa_gu and three TPipe rings
    (TPUSH / TPOP with cross-core flags), once with every thread on one instruction stream and once with the pipes on
    warps of their own (the cross-core flags are then counts that each team of warps waits on)."""
    if causal and s0 != s1:
        pytest.skip("the causal mask of the macros assumes a square problem")
    entry = refk_pw.pto_refk_pw_fa_head if pipe_warps else refk.pto_refk_fa_head
    d = 128
    r = np.random.default_rng(s0 + s1 + causal)
    q = r.standard_normal((s0, d)).astype(np.float16)
    k = r.standard_normal((s1, d)).astype(np.float16)
    v = r.standard_normal((s1, d)).astype(np.float16)
    blocks = s0 // 32
    o = torch.full((s0, d), float("nan"), device="cuda")
    qk_ws = torch.zeros(blocks * 2 * 32 * 64, device="cuda")
    p_ws = torch.zeros(blocks * 2 * 32 * 64, dtype=torch.float16, device="cuda")
    pv_ws = torch.zeros(blocks * 2 * 32 * 128, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert entry(_ptr(o), _ptr(dev(q)), _ptr(dev(k)), _ptr(dev(v)), s0, s1, causal, fifo, _ptr(qk_ws), _ptr(p_ws),
                 _ptr(pv_ws), _stream(), _ptr(status)) == 0
    assert refk.pto_refk_status(_stream(), _ptr(status)) == 0, host(status)
    scale = float(_newton_inv_sqrt(d))
    # non-causal: the oracle's streaming formulation with the program's key tile; causal: its plain formulation (the
    # streaming one models the reference kernel's 128-row query blocks, which this program's 32-row blocks are not)
    want = port.attn_head_f16(q, k, v, 1, scale) if causal else port.fa_tiled_f16(q, k, v, 0, scale, tile_s1=64)
    ok, worst = rel_err_ok(host(o), want, 2e-3,
                           label=f"fa macros + pipes s0={s0} s1={s1} causal={causal} fifo={fifo} pipe_warps={pipe_warps}")
    assert ok, f"max relative error {worst:.3e}"


# ---------------------------------------------------------------- bounded waits, typed events
def test_wait_that_runs_out_reports_and_returns(refk):
    """wait_flag on a flag no pipe raises, limit 5 ms: the kernel returns, the status record holds
    PTO_B200_ERR_DEVICE_WAIT_TIMEOUT (4), the block and the flag; the record of libpto_b200.so is used so that
    pto_b200_device_status reports it; the next launch on the stream works."""
    import pto_isa_b200 as pto
    lib = pto.lib()
    record = lib.pto_b200_status_record()
    assert record
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert refk.pto_refk_wait_that_runs_out(_ptr(out), 5_000_000, 3, ctypes.c_void_p(record), _stream()) == 0
    t1.record()
    torch.cuda.synchronize()
    assert 4.0 <= t0.elapsed_time(t1) < 500.0  # gave up after the limit, not after the default two seconds
    assert int(out.item()) == 1234  # the program ran on after the wait
    rec = (ctypes.c_int * 4)()
    assert lib.pto_b200_device_status_ex(_stream(), rec) == 4  # PTO_B200_ERR_DEVICE_WAIT_TIMEOUT
    assert rec[0] == 4 and 0 <= rec[1] < 3
    assert rec[2] == ((1 * 8 + 4) * 8 + 5)  # flag (PIPE_V -> PIPE_MTE3, EVENT_ID5)
    assert rec[3] == 1 * 16 + 4
    assert "gave up" in lib.pto_b200_last_error().decode()
    assert pto.device_status() == 0  # the record was cleared by the read
    # the context is intact: the next launches succeed
    x = torch.randn(64, 64, device="cuda")
    y = torch.zeros(64, 64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_typed_events(_ptr(y), _ptr(x), _stream(), _ptr(status)) == 0
    assert refk.pto_refk_status(_stream(), _ptr(status)) == 0
    assert np.array_equal(host(y), host(x) + np.float32(3.0))


def test_tile_assigned_beyond_the_arena_is_reported_not_written(refk):
    """A staged tile whose storage would end past the block's shared memory: TLOAD checks before it copies, the block
    reports {4, block, 602} and runs on; the next launch on the same context works."""
    import pto_isa_b200 as pto
    lib = pto.lib()
    record = lib.pto_b200_status_record()
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    src = torch.ones(128, 128, dtype=torch.float16, device="cuda")
    refk.pto_refk_tile_beyond_arena.argtypes = [ctypes.c_void_p] * 4
    assert refk.pto_refk_tile_beyond_arena(_ptr(out), _ptr(src), _stream(), ctypes.c_void_p(record)) == 0
    rec = (ctypes.c_int * 4)()
    assert lib.pto_b200_device_status_ex(_stream(), rec) == 4
    assert rec[0] == 4 and rec[1] == 0 and rec[2] == 602, list(rec)
    torch.cuda.synchronize()
    assert int(out[0]) == 4321  # the program ran to its end
    assert pto.device_status() == 0
    x = torch.randn(64, 64, device="cuda")
    y = torch.zeros(64, 64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_typed_events(_ptr(y), _ptr(x), _stream(), _ptr(status)) == 0
    assert refk.pto_refk_status(_stream(), _ptr(status)) == 0
    assert np.array_equal(host(y), host(x) + np.float32(3.0))


def test_typed_events_program(refk):
    """Event<SrcOp, DstOp>: `event = TXXX(...)` records, TXXX(..., event) waits (include/pto/common/event.hpp:110-152)."""
    x = torch.randn(64, 64, device="cuda")
    y = torch.zeros(64, 64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_typed_events(_ptr(y), _ptr(x), _stream(), _ptr(status)) == 0
    assert refk.pto_refk_status(_stream(), _ptr(status)) == 0
    assert np.array_equal(host(y), host(x) + np.float32(3.0))
