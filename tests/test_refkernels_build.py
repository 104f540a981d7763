"""What the build of the reference's own sources leaves behind (pto_isa_b200/refkernels.py): the two libraries of tile
programs and the compile check of the flash-attention kernel file.  These tests look at build output only (no GPU); they
skip where the reference tree was not available at build time."""
import os
import re
import subprocess

import pytest

from pto_isa_b200 import refkernels

_BUILD = os.path.join(os.path.dirname(refkernels.OUT), "build", "refkernels")


def _symbols(path):
    return subprocess.run(["nm", "-C", path], capture_output=True, text=True, check=True).stdout


def test_rewrite_launches_keeps_preprocessor_and_comment_lines_in_place():
    src = ("void host(void *stream)\n{\n    prepare();\n#if defined(A)\n    // warm up\n"
           "    warm<1><<<24, nullptr, stream>>>();\n#endif\n    run<2, 3><<<blocks, nullptr, stream>>>(a, (int)b);\n}\n")
    out = refkernels.rewrite_launches(src)
    assert "#if defined(A)\n    // warm up\n    PTO_B200_LAUNCH((warm<1>), 24, stream)" in out
    assert "#endif\n    PTO_B200_LAUNCH((run<2, 3>), blocks, stream, a, (int)b)" in out
    assert "<<<" not in out


def test_rewrite_core_statics_only_touches_function_locals():
    src = "static int file_scope = 3;\nAICORE inline void f()\n{\n    static uint64_t pingpong = 0;\n    pingpong ^= 1;\n}\n"
    out = refkernels.rewrite_core_statics(src)
    assert "static int file_scope = 3;" in out
    assert "PTO_B200_CORE_STATIC(uint64_t, pingpong, 0, 0);" in out


@pytest.mark.parametrize("flavour", ["cube", "vec"])
def test_flash_attention_kernel_file_compiled_for_both_core_kinds(flavour):
    obj = os.path.join(_BUILD, f"fa_kernel_check_{flavour}.o")
    if not os.path.exists(obj):
        pytest.skip("the reference tree was not available when the libraries were built")
    syms = _symbols(obj)
    # every case of the reference's default case list has its launcher (with and without the profile buffer)
    launchers = set(re.findall(r"void LaunchTFA<([^>]*)>", syms))
    assert len(launchers) >= 6, launchers
    assert any(l.startswith("128, 128, 8192, 128, 128") for l in launchers)
    assert any(l.startswith("512, 128, 1024, 128, 128") for l in launchers)


def test_both_libraries_export_the_gemm_program():
    if not (os.path.exists(refkernels.OUT) and os.path.exists(refkernels.OUT_PW)):
        pytest.skip("libpto_b200_refkernels*.so have not been built")
    assert "pto_refk_gemm_6144" in _symbols(refkernels.OUT)
    pw = _symbols(refkernels.OUT_PW)
    assert "pto_refk_gemm_pw_6144_k128" in pw and "pto_refk_gemm_pw_1536" in pw and "pto_refk_pw_fa_head" in pw


def test_launcher_library_defines_the_declared_templates():
    """include/pto_b200_launchers.hpp declares the reference hosts' launcher templates; libpto_b200_launchers.so holds
    the instances a host links against (checked by name, nothing is launched)."""
    lib = os.path.join(os.path.dirname(refkernels.OUT), "libpto_b200_launchers.so")
    if not os.path.exists(lib):
        pytest.skip("libpto_b200_launchers.so has not been built")
    syms = subprocess.run(["nm", "-DC", lib], capture_output=True, text=True, check=True).stdout
    for name in ("void LaunchGEMME2E<unsigned short>(", "void LaunchTFA<", "LaunchTMATMUL<1>(", "LaunchTMATMUL<4>(",
                 "LaunchTMATMULBIAS<5>(", "LaunchTROWMAX<", "LaunchTROWSUM<", "LaunchTExp<", "launchTCVT<",
                 "LaunchTFLASHATTN(", "pto_b200_launcher_status"):
        assert name in syms, name
