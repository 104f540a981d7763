"""The C++ half of the boundary: a C++ host in the shape of the reference's kernel hosts (pto_isa_b200/csrc/host/
host_main.cpp; kernels/manual/a2a3/gemm_performance/main.cpp:22-98 in the reference) calls the reference's launcher
templates (include/pto_b200_launchers.hpp: LaunchGEMME2E<uint16_t>, LaunchTFA<...>, LaunchTMATMUL<key>) on .bin files
written the way the reference's generators write them, and compares with the goldens by the ResultCmp rule."""
import os
import subprocess

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_HOST = os.path.join(_ROOT, "pto_isa_b200", "pto_b200_host")


def _run(*args):
    assert os.path.exists(_HOST), "pto_isa_b200/pto_b200_host is built by pto_isa_b200.build"
    p = subprocess.run([_HOST, *map(str, args)], capture_output=True, text=True, timeout=300)
    return p.returncode, p.stdout + p.stderr


def test_gemm_host_reads_launches_and_compares(tmp_path):
    """Files as kernels/manual/a2a3/gemm_performance/scripts/gen_data.py:18-45 writes them: x1 m x k, x2 n x k (B
    transposed), golden = fp32 product."""
    m, k, n = 384, 256, 512
    r = np.random.default_rng(0)
    os.makedirs(tmp_path / "input")
    os.makedirs(tmp_path / "output")
    a = r.uniform(-1, 1, (m, k)).astype(np.float16)
    b = r.uniform(-1, 1, (k, n)).astype(np.float16)
    a.tofile(tmp_path / "input" / "x1_gm.bin")
    np.ascontiguousarray(b.T).tofile(tmp_path / "input" / "x2_gm.bin")
    golden = np.matmul(a.astype(np.float32), b.astype(np.float32)).astype(np.float32)
    golden.tofile(tmp_path / "output" / "golden.bin")
    rc, out = _run("gemm", tmp_path, m, k, n)
    assert rc == 0 and "test success" in out, out
    got = np.fromfile(tmp_path / "output" / "output_z.bin", np.float32).reshape(m, n)
    assert np.array_equal(got, oracle.port.gemm_f16f32(a, np.ascontiguousarray(b.T), 1)) or \
        np.abs(got - golden).max() <= 2e-3 * np.abs(golden).max()
    # a corrupted golden must be reported as a failure
    golden[:, ::2] += 1.0
    golden.tofile(tmp_path / "output" / "golden.bin")
    rc, out = _run("gemm", tmp_path, m, k, n)
    assert rc == 1 and "test failed" in out, out


@pytest.mark.parametrize("s0,s1,causal", [(128, 1024, 0), (1024, 1024, 1)])
def test_flash_attention_host(tmp_path, s0, s1, causal):
    """Files as kernels/manual/common/flash_atten/scripts/gen_data.py writes them (q, kt, v as fp16; o as fp32 from its
    tiled model, which the oracle's streaming formulation restates)."""
    d = 128
    r = np.random.default_rng(s0 + s1)
    q = r.standard_normal((s0, d)).astype(np.float16)
    k = r.standard_normal((s1, d)).astype(np.float16)
    v = r.standard_normal((s1, d)).astype(np.float16)
    q.tofile(tmp_path / "q.bin")
    k.tofile(tmp_path / "kt.bin")
    v.tofile(tmp_path / "v.bin")
    o = oracle.port.fa_tiled_f16(q, k, v, causal, 1.0 / np.sqrt(d), tile_s1=256)
    o.astype(np.float32).tofile(tmp_path / "o.bin")
    rc, out = _run("fa", tmp_path, s0, s1, causal)
    assert rc == 0 and "test success" in out, out


def test_tmatmul_launcher_runs_the_reference_cases(tmp_path, golden_dir):
    if not os.path.exists(os.path.join(_ROOT, "pto_isa_b200", "libpto_b200_refkernels.so")):
        pytest.skip("LaunchTMATMUL runs the reference's tile programs; their library was not built")
    z = np.load(os.path.join(golden_dir, "tmatmul.npz"))
    for key, name in ((1, "case1"), (3, "case3"), (4, "case4")):
        d = tmp_path / name
        os.makedirs(d)
        z[f"{name}_a"].tofile(d / "x1_gm.bin")
        z[f"{name}_b"].tofile(d / "x2_gm.bin")
        z[f"{name}_golden"].tofile(d / "golden.bin")
        rc, out = _run("tmatmul", d, key)
        assert rc == 0 and "test success" in out, (name, out)
