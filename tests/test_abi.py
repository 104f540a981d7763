"""The C ABI boundary, checked without a GPU: the shared library loads, exports every symbol that
include/pto_b200.h declares, the Python signature table matches the header, and argument errors are
reported as status codes before anything touches a device."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "pto_b200.h")


def header_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pto_b200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built_lib():
    from pto_isa_b200 import build
    return build.build()


def test_header_declares_expected_entry_points():
    syms = header_symbols()
    for must in ("pto_b200_gemm_f16f32", "pto_b200_flash_attn_fwd_f16", "pto_b200_tcvt_f32_f16",
                 "pto_b200_tcvt_f32_bf16", "pto_b200_tgather", "pto_b200_trowmax_f32", "pto_b200_trowsum_f32",
                 "pto_b200_texp_f32", "pto_b200_gemm_call_kernel", "pto_b200_fa_call_kernel"):
        assert must in syms


def test_library_exports_every_declared_symbol(built_lib):
    handle = ctypes.CDLL(built_lib)
    for name in header_symbols():
        assert hasattr(handle, name), f"{name} is declared in pto_b200.h but not exported"


def test_only_the_c_abi_is_exported(built_lib):
    out = subprocess.check_output(["nm", "-D", "--defined-only", built_lib], text=True)
    exported = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert exported and all(s.startswith("pto_b200_") for s in exported), exported


def test_python_signature_table_matches_header(built_lib):
    from pto_isa_b200 import _lib
    assert sorted(_lib.SIGNATURES) == header_symbols()
    import re
    header = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "pto_b200.h")).read()
    assert _lib.lib().pto_b200_version() == int(re.search(r"#define PTO_B200_ABI_VERSION (\d+)", header).group(1)) == 4


def test_call_kernel_shims_export_the_reference_symbol(built_lib):
    d = os.path.dirname(built_lib)
    for so in ("libpto_b200_gemm_jit.so", "libpto_b200_flash_jit.so"):
        out = subprocess.check_output(["nm", "-D", "--defined-only", os.path.join(d, so)], text=True)
        assert any(l.split()[-1] == "call_kernel" for l in out.splitlines())


def test_argument_errors_are_status_codes(built_lib):
    from pto_isa_b200 import _lib
    l = _lib.lib()
    assert l.pto_b200_tcvt_f32_f16(None, None, 16, None) == 1
    assert l.pto_b200_tcvt_f32_f16(None, None, 0, None) == 0  # empty input is a no-op
    assert l.pto_b200_tgather(None, 0, None, None, 0, 4, None) == 0
    assert l.pto_b200_tgather(None, 0, None, None, 0, 3, None) == 1
    assert l.pto_b200_tgather_mask(None, None, 4, 4, 9, 4, None) == 1
    assert l.pto_b200_trowmax_f32(None, None, 4, 0, 0, None) == 1
    assert l.pto_b200_gemm_f16f32(None, None, None, 128, 256, 64, 1, None) == 1
    assert b"gemm" in l.pto_b200_last_error()
    assert l.pto_b200_flash_attn_fwd_f16(None, None, None, None, 1, 128, 128, 128, 0, 1.0, 0, None) == 1


def test_missing_library_fails_loudly(monkeypatch):
    from pto_isa_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_NAME", "libpto_b200_absent.so")
    with pytest.raises(_lib.PtoB200Error):
        _lib.lib()


def test_cpu_tensors_are_rejected():
    import torch
    import pto_isa_b200 as p
    with pytest.raises(p.PtoB200Error):
        p.TCVT(torch.zeros(8), torch.float16)
    with pytest.raises(p.PtoB200Error):
        p.gemm(torch.zeros(128, 64, dtype=torch.float16), torch.zeros(256, 64, dtype=torch.float16))


def test_ascend_launch_statements_are_rewritten():
    """The one non-C++-for-nvcc construct of the reference kernels: `k<<<blocks, l2ctrl, stream>>>(args)`."""
    from pto_isa_b200.refkernels import rewrite_launches
    src = ("void f() {\n    Kern<T, a,\n         b><<<blockDim, nullptr, stream>>>(out, src0, src1);\n"
           "    warm<<<24, nullptr, stream>>>();\n    g(x);\n}\n")
    out = rewrite_launches(src)
    assert "<<<" not in out
    assert "PTO_B200_LAUNCH((Kern<T, a,\n         b>), blockDim, stream, out, src0, src1);" in out
    assert "PTO_B200_LAUNCH((warm), 24, stream);" in out
    assert out.endswith("    g(x);\n}\n")
    assert rewrite_launches("no launches here;") == "no launches here;"


def test_build_entry_version_check():
    """The check build() ends with (library version == header version) holds for the library in the tree."""
    import __graft_entry__
    __graft_entry__.check_library_version()
