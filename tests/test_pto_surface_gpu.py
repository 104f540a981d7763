"""The reference's own tile programs, compiled against this repository's PTO headers (include/pto/) with
only their Ascend launch statements rewritten, run on the GPU and are checked against the CPU oracle.

The library under test, pto_isa_b200/libpto_b200_refkernels.so, is built by pto_isa_b200/refkernels.py where
the reference tree is available; the tests skip when it is absent."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle
from util import dev, host, rel_err_ok

pytestmark = pytest.mark.gpu
port = oracle.port
_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "pto_isa_b200",
                   "libpto_b200_refkernels.so")


class _Libs:
    """Entry points of the two libraries built from the reference's sources: `..._pw_...` names live in the one compiled
    with the core's pipes on warps of their own (PTO_B200_PIPE_WARPS is a property of a translation unit)."""

    def __init__(self):
        self.plain = ctypes.CDLL(_SO)
        self.pw = ctypes.CDLL(_SO.replace("refkernels.so", "refkernels_pw.so"))

    def __getattr__(self, name):
        return getattr(self.pw if "_pw_" in name else self.plain, name)


@pytest.fixture(scope="module")
def refk():
    if not os.path.exists(_SO) or not os.path.exists(_SO.replace("refkernels.so", "refkernels_pw.so")):
        pytest.skip("libpto_b200_refkernels*.so have not been built (they need the reference tree at build time)")
    return _Libs()


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("name,m,k,n", [("pto_refk_gemm_256x128x512", 256, 128, 512),
                                        ("pto_refk_gemm_1536", 1536, 1536, 1536),
                                        ("pto_refk_gemm_pw_256x128x512", 256, 128, 512),
                                        ("pto_refk_gemm_pw_256x128x512_copies", 256, 128, 512),
                                        ("pto_refk_gemm_pw_1536", 1536, 1536, 1536)])
def test_reference_gemm_tile_program(refk, name, m, k, n):
    """RunGemmE2E (TLOAD / TEXTRACT / TMATMUL / TMATMUL_ACC / TSTORE with its set_flag / wait_flag ping-pong),
    base tile 128 x 256, k step 64, B stored n x k.  The `pw` instances run the core's pipes on warps of their own
    (loads, products and stores overlap as the program's flags allow; TEXTRACT hands out views); `_copies` is that mode's
    fallback through every instruction: nothing registered (cp.async loads by the copying warp), copying TEXTRACT, TSTORE
    from registers."""
    r = np.random.default_rng(m + n)
    a = r.uniform(-1, 1, (m, k)).astype(np.float16)
    b = r.uniform(-1, 1, (n, k)).astype(np.float16)
    da, db = dev(a), dev(b)
    c = torch.full((m, n), float("nan"), device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert getattr(refk, name)(_ptr(c), _ptr(da), _ptr(db), _stream(), _ptr(status)) == 0
    assert refk.pto_refk_status(_stream(), _ptr(status)) == 0
    want = port.gemm_f16f32(a, b, 1)
    ok, worst = rel_err_ok(host(c), want, 2e-3)
    assert ok, f"max relative error {worst:.3e}"


@pytest.mark.parametrize("name", ["pto_refk_gemm_6144", "pto_refk_gemm_pw_6144", "pto_refk_gemm_pw_6144_k128",
                                  "pto_refk_gemm_pw_6144_x2"])
def test_reference_gemm_tile_program_6144(refk, name):
    import pto_isa_b200 as pto
    m = n = k = 6144
    g = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).half()
    b = (torch.rand(n, k, device="cuda", generator=g) * 2 - 1).half()
    c = torch.full((m, n), float("nan"), device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert getattr(refk, name)(_ptr(c), _ptr(a), _ptr(b), _stream(), _ptr(status)) == 0
    assert refk.pto_refk_status(_stream(), _ptr(status)) == 0
    # against the hand-written kernel (itself checked against the oracle): same tensor-core arithmetic
    want = pto.gemm(a, b, 1)
    ok, worst = rel_err_ok(host(c), host(want), 1e-5)
    assert ok, f"max relative error {worst:.3e}"


def test_reference_tcvt_tile_program(refk):
    """runTCVT of tests/cpu/st/testcase/tcvt/tcvt_kernel.cpp: TLOAD -> TCVT(CAST_RINT) -> TSTORE."""
    r = np.random.default_rng(19)
    x = (r.random((64, 64)) * 4.41).astype(np.float32)
    x[0, :6] = [np.nan, np.inf, -np.inf, 65520.0, 1e-8, -0.0]
    d = torch.zeros(64, 64, dtype=torch.float16, device="cuda")
    assert refk.pto_refk_tcvt_f32_f16_64x64(_ptr(d), _ptr(dev(x)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(d.view(torch.int16)).view(np.uint16), port.tcvt_f32_f16(x).view(np.uint16))
    xi = (r.standard_normal((128, 128)) * 100).astype(np.float32)
    di = torch.zeros(128, 128, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_tcvt_f32_i32_128x128(_ptr(di), _ptr(dev(xi)), _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host(di), port.tcvt_f32_i32(xi, 1))


def test_vector_program_with_typed_events_on_pipe_warps(refk):
    """TLOAD -> TADDS -> TSTORE ordered by three typed events, with the pipes on warps of their own: the load on the
    loading thread and the copying warp, the vector instruction and the store on the vector / store warps (three blocks
    run the same program: they write the same values)."""
    x = torch.randn(64, 64, device="cuda")
    y = torch.zeros(64, 64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert refk.pto_refk_pw_typed_events(_ptr(y), _ptr(x), _stream(), _ptr(status)) == 0
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert np.array_equal(host(y), host(x) + np.float32(3.0))
