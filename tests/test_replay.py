"""The reference harnesses' on-disk formats (raw .bin tensors, generated_cases.json / .h, report.csv) as read and
written by pto_isa_b200/replay.py: byte-for-byte against files produced by the reference's own generator
(tests/golden/harness_*), and a replay of golden cases on the GPU."""
import os

import numpy as np
import pytest

from pto_isa_b200 import replay

DEFAULT_CASES = [(128, 128, 1024, 128), (128, 128, 2048, 128), (128, 128, 8192, 128), (128, 512, 1024, 128),
                 (128, 512, 2048, 128), (128, 512, 8192, 128)]  # scripts/generate_cases.py:36-43


def _text(golden_dir, name):
    with open(os.path.join(golden_dir, name)) as f:
        return f.read()


def test_case_list_files_match_the_reference_generator(golden_dir, tmp_path):
    cases = [replay.make_case(h, s0, s1, c0) for (h, s0, s1, c0) in DEFAULT_CASES]
    replay.write_cases(cases, str(tmp_path / "generated_cases.json"), str(tmp_path / "generated_cases.h"))
    assert (tmp_path / "generated_cases.json").read_text() == _text(golden_dir, "harness_default_generated_cases.json")
    assert (tmp_path / "generated_cases.h").read_text() == _text(golden_dir, "harness_default_generated_cases.h")
    explicit = [replay.make_case(128, 128, 512, 128, qk_preload=2), replay.make_case(128, 512, 2048, 128, 512, qk_preload=2)]
    replay.write_cases(explicit, str(tmp_path / "e.json"), str(tmp_path / "e.h"))
    assert (tmp_path / "e.json").read_text() == _text(golden_dir, "harness_explicit_generated_cases.json")
    assert (tmp_path / "e.h").read_text() == _text(golden_dir, "harness_explicit_generated_cases.h")


def test_case_list_reader(golden_dir):
    cases = replay.load_cases(os.path.join(golden_dir, "harness_explicit_generated_cases.json"))
    assert [c["name"] for c in cases] == ["case_float_H_128_S0_128_S1_512", "case_float_H_128_S0_512_S1_2048"]
    assert cases[1]["tile_s1"] == 512 and cases[1]["qk_preload"] == 2 and cases[0]["causal_mask"] == 0
    with pytest.raises(ValueError):
        replay.make_case(128, 128, 500, 128)  # S1 not a multiple of 128
    assert replay.make_case(128, 96, 512, 128)["cube_s0"] == 96  # cube_s0 larger than s0 becomes s0


def test_bin_tensors_and_comparison(tmp_path):
    a = np.arange(12, dtype=np.float16).reshape(3, 4)
    replay.write_bin(str(tmp_path / "x" / "a.bin"), a)
    assert (tmp_path / "x" / "a.bin").read_bytes() == a.astype("<f2").tobytes()
    assert np.array_equal(replay.read_bin(str(tmp_path / "x" / "a.bin"), np.float16, (3, 4)), a)
    with pytest.raises(ValueError):
        replay.read_bin(str(tmp_path / "x" / "a.bin"), np.float16, (3, 5))
    g = np.ones(1000, np.float32)
    bad = g.copy()
    bad[0] = 2.0
    assert replay.result_cmp(g, bad, 1e-3)          # one wrong element of 1000 is within size * eps
    bad[1] = 2.0
    assert not replay.result_cmp(g, bad, 1e-3)
    assert replay.result_cmp(g, g + 5e-4, 1e-3)


def test_report_rows(tmp_path):
    path = str(tmp_path / "report.csv")
    replay.append_report_row(path, "case_float_H_128_S0_128_S1_512", 128, 128, 512, 128, 128, 256, 0, 12345, 12.345, 12.345,
                             33.554, 2.718, True)
    replay.append_report_row(path, "c2", 128, 128, 512, 128, 128, 256, 0, 0, 0.0, 0.0, 33.554, None, False)
    lines = open(path).read().splitlines()
    assert lines[0] == ("case,HEAD,S0,S1,CUBE_S0,CUBE_S1,TILE_S1,start_time,end_time,duration_us,avg_block_us,GOPS,"
                        "TFLOPS,result")  # kernels/manual/common/flash_atten/main.cpp:98-99
    assert lines[1] == "case_float_H_128_S0_128_S1_512,128,128,512,128,128,256,0,12345,12.345,12.345,33.554,2.718,OK"
    assert lines[2].endswith(",NA,NOK")
    rows = replay.read_report(path)
    assert rows[0]["result"] == "OK" and rows[1]["TFLOPS"] == "NA"


@pytest.mark.gpu
def test_replay_of_reference_cases(golden_dir, tmp_path):
    z = np.load(os.path.join(golden_dir, "attention.npz"))
    build = tmp_path / "build"
    cases = []
    for tag, causal in (("fa_nc_128x512", False), ("fa_causal_128x512", True)):
        case = replay.make_case(128, 128, 512, 128, causal_mask=causal)
        case["name"] = replay.case_name(case) + ("_causal" if causal else "")
        d = build / case["name"]
        replay.write_bin(str(d / "q.bin"), z[f"{tag}_q"])
        replay.write_bin(str(d / "kt.bin"), np.ascontiguousarray(z[f"{tag}_k"].T))  # the harness reads kt.bin
        replay.write_bin(str(d / "v.bin"), z[f"{tag}_v"])
        replay.write_bin(str(d / "o.bin"), z[f"{tag}_o"])
        ok, us = replay.replay_flash_case(str(d), case, str(build / "report.csv"))
        assert ok and us > 0
        out = replay.read_bin(str(d / "o_out.bin"), np.float32, (128, 128))
        assert replay.result_cmp(z[f"{tag}_o"], out, 1e-3)
        cases.append(case)
    rows = replay.read_report(str(build / "report.csv"))
    assert [r["result"] for r in rows] == ["OK", "OK"] and rows[0]["GOPS"] == f"{128 * 512 * 128 * 4 / 1e6:.3f}"
    g = np.load(os.path.join(golden_dir, "gemm.npz"))
    gd = tmp_path / "gemm"
    replay.write_bin(str(gd / "input" / "x1_gm.bin"), g["a"])
    replay.write_bin(str(gd / "input" / "x2_gm.bin"), g["b_dn"])
    replay.write_bin(str(gd / "output" / "golden.bin"), g["golden"])
    ok, us = replay.replay_gemm_case(str(gd), 128, 192, 256)
    assert ok and os.path.getsize(gd / "output" / "output_z.bin") == 128 * 256 * 4
    assert replay.main(["gemm", str(gd), "128", "192", "256"]) == 0
