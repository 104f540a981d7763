#!/usr/bin/env python3
"""Regenerate the golden fixtures in this directory from the reference's own generator scripts.

Run where the reference tree is available:

    python tests/golden/make_golden.py [--reference /path/to/pto-isa]

Each reference `gen_data.py` is loaded as a module *from where it lies* (nothing is copied), its
generator function is called with the case list its own `__main__` block uses (restated below with
the file:line it comes from, because those lists live under `if __name__ == "__main__"` and two of
the scripts would otherwise try to create directories inside the reference tree), in the same
order and after the same `np.random.seed(...)`, so the bytes are the ones the reference's test
drivers would feed to its kernels.  Inputs and goldens of the cases on the GEMM / attention /
vector hot path are packed into compressed .npz files here.

The fixtures travel with the repository; the reference tree does not have to exist where the
tests run.
"""
import argparse
import importlib.util
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)  # runs the module-level np.random.seed(...)
    return mod


def read(path, dtype, shape=None):
    a = np.fromfile(path, dtype=dtype)
    return a.reshape(shape) if shape is not None else a


def in_case_dir(tmp, name):
    d = os.path.join(tmp, name)
    os.makedirs(d, exist_ok=True)
    os.chdir(d)
    return d


def gen_tcvt(ref, tmp, out):
    # tests/cpu/st/testcase/tcvt/gen_data.py:62-72 (case list), :20-38 (generator)
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/tcvt/gen_data.py"), "ref_tcvt_gen")
    P = mod.TCvtParams
    rint = "RoundMode::CAST_RINT"
    cases = [
        P(np.float32, np.int32, 128, 128, rint), P(np.int32, np.float32, 256, 64, rint),
        P(np.float32, np.int16, 16, 32, rint), P(np.float32, np.int32, 32, 512, rint),
        P(np.int16, np.int32, 2, 512, rint), P(np.float32, np.int32, 4, 4096, rint),
        P(np.int16, np.float32, 64, 64, rint), P(np.float32, np.float16, 64, 64, rint),
        P(np.float16, np.uint8, 64, 64, rint),
    ]
    keep = {}
    for i, p in enumerate(cases, start=1):
        d = in_case_dir(tmp, f"tcvt_case{i}")
        mod.gen_golden(p)
        if i in (1, 4, 6, 8):  # f32->i32 (three shapes) and f32->f16
            keep[f"case{i}_src"] = read(os.path.join(d, "x1_gm.bin"), p.srctype, (p.m, p.n))
            keep[f"case{i}_golden"] = read(os.path.join(d, "golden.bin"), p.dsttype, (p.m, p.n))
    np.savez_compressed(os.path.join(out, "tcvt.npz"), **keep)


def gen_tgather(ref, tmp, out):
    # tests/cpu/st/testcase/tgather/gen_data.py:132-173 (case list), :92-129 (generator)
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/tgather/gen_data.py"), "ref_tgather_gen")
    M, D = mod.TGatherParamsMasked, mod.TGatherParams1D
    f32, f16 = np.float32, np.half
    cases = [
        M("float_P0101", f32, f32, 4, 64, 1), M("float_P1010", f32, f32, 7, 1024, 2),
        M("float_P0001", f32, f32, 3, 1056, 3), M("float_P0010", f32, f32, 4, 128, 4),
        M("float_P0100", f32, f32, 5, 256, 5), M("float_P1000", f32, f32, 6, 288, 6),
        M("float_P1111", f32, f32, 7, 320, 7),
        M("half_P0101", f16, f16, 5, 128, 1), M("half_P1010", f16, f16, 7, 1024, 2),
        M("half_P0001", f16, f16, 3, 1056, 3), M("half_P0100", f16, f16, 5, 256, 5),
        M("half_P1000", f16, f16, 6, 288, 6),
        M("U16_P0101", np.uint16, np.uint16, 5, 128, 1), M("U16_P1010", np.uint16, np.uint16, 7, 1024, 2),
        M("I16_P0001", np.int16, np.int16, 3, 1056, 3), M("I16_P0010", np.int16, np.int16, 4, 128, 4),
        M("U32_P0100", np.uint32, np.uint32, 5, 256, 5), M("I32_P1000", np.int32, np.int32, 6, 288, 6),
        M("I32_P1111", np.int32, np.int32, 7, 320, 7),
        D("1D_float_32x1024_16x64", f32, 32, 1024, 16, 64), D("1D_int32_32x512_16x256", np.int32, 32, 512, 16, 256),
        D("1D_half_16x1024_16x128", np.float16, 16, 1024, 16, 128), D("1D_int16_32x256_32x64", np.int16, 32, 256, 32, 64),
    ]
    keep = {}
    for p in cases:
        d = in_case_dir(tmp, "tgather_" + p.testname)
        mod.original_dir = tmp  # the generator chdir()s back to this global after a masked case
        mod.gen_golden_data(p)
        if isinstance(p, M):
            keep[f"{p.testname}__src"] = read(os.path.join(d, "x1_gm.bin"), p.src_type, (p.row, p.col))
            keep[f"{p.testname}__golden"] = read(os.path.join(d, "golden.bin"), p.dst_type)
            keep[f"{p.testname}__pattern"] = np.array(p.pattern)
        else:
            keep[f"{p.testname}__src0"] = read(os.path.join(d, "src0.bin"), p.src_type, (p.src_row, p.src_col))
            keep[f"{p.testname}__idx"] = read(os.path.join(d, "src1.bin"), np.int32, (p.dst_row, p.dst_col))
            keep[f"{p.testname}__golden"] = read(os.path.join(d, "golden.bin"), p.src_type, (p.dst_row, p.dst_col))
    np.savez_compressed(os.path.join(out, "tgather.npz"), **keep)


def gen_tmatmul(ref, tmp, out):
    # tests/cpu/st/testcase/tmatmul/gen_data.py:86-96 (case list), :34-59 (generator)
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/tmatmul/gen_data.py"), "ref_tmatmul_gen")
    P = mod.tmatmulParams
    cases = [
        ("case1", P(np.float16, np.float16, np.float32, 40, 50, 60, False)),
        ("case2", P(np.int8, np.int8, np.int32, 6, 7, 8, False)),
        ("case3", P(np.float16, np.float16, np.float32, 128, 128, 64, False, repeats=5)),
        ("case4", P(np.float32, np.float32, np.float32, 120, 110, 50, False)),
    ]
    keep = {}
    for name, p in cases:
        d = in_case_dir(tmp, "tmatmul_" + name)
        mod.gen_golden_data(name, p)
        if name == "case2":
            continue
        keep[f"{name}_a"] = read(os.path.join(d, "x1_gm.bin"), p.atype, (p.repeats, p.m, p.k))
        keep[f"{name}_b"] = read(os.path.join(d, "x2_gm.bin"), p.btype, (p.repeats, p.k, p.n))
        keep[f"{name}_golden"] = read(os.path.join(d, "golden.bin"), p.ctype, (p.m, p.n))
    np.savez_compressed(os.path.join(out, "tmatmul.npz"), **keep)


def gen_tmatmul_i8(ref, tmp, out):
    """The int8 -> int32 case of the same generator (tests/cpu/st/testcase/tmatmul/gen_data.py:34-59; its own case2 is
    6 x 7 x 8) at 128 x 64 x 256 and 256 x 320 x 512, shapes whose rows a TMA descriptor accepts."""
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/tmatmul/gen_data.py"), "ref_tmatmul_gen_i8")
    keep = {}
    for name, (m, k, n) in (("small", (128, 64, 256)), ("mid", (256, 320, 512))):
        p = mod.tmatmulParams(np.int8, np.int8, np.int32, m, k, n, False)
        d = in_case_dir(tmp, "tmatmul_i8_" + name)
        mod.gen_golden_data(name, p)
        keep[f"{name}_a"] = read(os.path.join(d, "x1_gm.bin"), np.int8, (m, k))
        keep[f"{name}_b"] = read(os.path.join(d, "x2_gm.bin"), np.int8, (k, n))
        keep[f"{name}_golden"] = read(os.path.join(d, "golden.bin"), np.int32, (m, n))
    np.savez_compressed(os.path.join(out, "tmatmul_i8.npz"), **keep)


def gen_tmatmul_bias(ref, tmp, out):
    """The bias form of the tmatmul generator (tests/cpu/st/testcase/tmatmul/gen_data.py:34-59 with is_bias; the
    reference's own case_bias_2 is fp16 16 x 15 x 16) at 128 x 64 x 256: A m x k, B k x n fp16, bias n fp32."""
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/tmatmul/gen_data.py"), "ref_tmatmul_gen_bias")
    m, k, n = 128, 64, 256
    p = mod.tmatmulParams(np.float16, np.float16, np.float32, m, k, n, True, np.float32)
    d = in_case_dir(tmp, "tmatmul_bias")
    mod.gen_golden_data("bias", p)
    np.savez_compressed(os.path.join(out, "tmatmul_bias.npz"),
                        a=read(os.path.join(d, "x1_gm.bin"), np.float16, (m, k)),
                        b=read(os.path.join(d, "x2_gm.bin"), np.float16, (k, n)),
                        bias=read(os.path.join(d, "bias_gm.bin"), np.float32, (n,)),
                        golden=read(os.path.join(d, "golden.bin"), np.float32, (m, n)))


def gen_rowops(ref, tmp, out):
    keep = {}
    # tests/cpu/st/testcase/trowmax/gen_data.py:79-85 (case list), :17-35 (generator)
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/trowmax/gen_data.py"), "ref_trowmax_gen")
    P = mod.TRowmaxParams
    for i, p in enumerate([P(np.float32, 64, 64, 64, 64, 64, 64), P(np.float16, 64, 64, 64, 64, 64, 64),
                           P(np.float16, 161, 161, 32, 32, 161, 161), P(np.float32, 77, 81, 32, 16, 77, 81),
                           P(np.float32, 32, 32, 32, 16, 32, 32)]):
        in_case_dir(tmp, f"trowmax_{i}")
        src, golden = mod.gen_golden_data_trowmax("", p)
        keep[f"trowmax{i}_src"] = src
        keep[f"trowmax{i}_golden"] = golden
        keep[f"trowmax{i}_valid"] = np.array([min(p.tile_row, p.valid_row), min(p.tile_col, p.valid_col)])
    # tests/cpu/st/testcase/trowsum/gen_data.py:69-72 (case list), :17-43 (generator)
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/trowsum/gen_data.py"), "ref_trowsum_gen")
    P = mod.trowsumParams
    for i, p in enumerate([P(np.float32, 64, 64, 64, 64, 64, 64), P(np.float16, 16, 256, 16, 256, 16, 256)]):
        in_case_dir(tmp, f"trowsum_{i}")
        _, src, golden = mod.gen_golden_data_trowsum("", p)
        keep[f"trowsum{i}_src"] = src
        keep[f"trowsum{i}_golden"] = golden[:, 0].copy()
    # tests/cpu/st/testcase/texp/gen_data.py:79-85 (case list), :17-41 (generator)
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/texp/gen_data.py"), "ref_texp_gen")
    P = mod.TExpParams
    for i, p in enumerate([P(np.float32, 64, 64, 64, 64, 64, 64), P(np.float16, 64, 64, 64, 64, 64, 64),
                           P(np.float16, 32, 32, 32, 32, 32, 32), P(np.float32, 32, 32, 32, 32, 32, 32),
                           P(np.float32, 32, 16, 32, 16, 32, 16)]):
        in_case_dir(tmp, f"texp_{i}")
        _, src, golden = mod.gen_golden_data_texp("", p)
        keep[f"texp{i}_src"] = src
        keep[f"texp{i}_golden"] = golden
    np.savez_compressed(os.path.join(out, "rowops.npz"), **keep)


def gen_attention(ref, tmp, out):
    keep = {}
    # tests/cpu/st/testcase/tflashattn/gen_data.py:62-73: 64 x 32 fp32 head, float64 golden
    mod = load(os.path.join(ref, "tests/cpu/st/testcase/tflashattn/gen_data.py"), "ref_tflashattn_gen")
    d = os.path.join(tmp, "tflashattn_case1")
    mod.gen_case(d, seq_len=64, head_dim=32, seed=20251220, init_scale=0.02)
    for key, f in (("q", "x1_gm.bin"), ("k", "x2_gm.bin"), ("v", "x3_gm.bin"), ("golden", "golden.bin")):
        keep[f"tflashattn_{key}"] = read(os.path.join(d, f), np.float32, (64, 32))
    # kernels/manual/common/flash_atten/scripts/gen_data.py:32-149: the streaming-softmax NumPy model of
    # the flash-attention kernel (TILE_S1 = 256, fp16 P, fp32 O), seeded np.random.seed(7) at import.
    # S1 = 512 gives two key tiles: with a single tile the generator never divides by the row sum (:141-147).
    mod = load(os.path.join(ref, "kernels/manual/common/flash_atten/scripts/gen_data.py"), "ref_fa_gen")
    for name, s0, s1, causal in (("fa_nc_128x512", 128, 512, False), ("fa_causal_128x512", 128, 512, True)):
        d = os.path.join(tmp, name)
        os.makedirs(d, exist_ok=True)
        mod.gen_case(d, s0, s1, 128, 128, 256, causal)
        keep[f"{name}_q"] = read(os.path.join(d, "q.bin"), np.float16, (s0, 128))
        keep[f"{name}_k"] = read(os.path.join(d, "kt.bin"), np.float16, (s1, 128))  # K rows: s1 x head
        keep[f"{name}_v"] = read(os.path.join(d, "v.bin"), np.float16, (s1, 128))
        keep[f"{name}_o"] = read(os.path.join(d, "o.bin"), np.float32, (s0, 128))
    np.savez_compressed(os.path.join(out, "attention.npz"), **keep)


def gen_gemm(ref, tmp, out):
    # kernels/manual/a2a3/gemm_performance/scripts/gen_data.py:18-45: A m x k and B k x n fp16 drawn
    # uniform(-5, 5) after np.random.seed(19), golden = fp32 np.matmul, B written transposed (n x k, the
    # Layout::DN operand).  The reference calls it for 6144^3 (:62-66); the same generator is called here for
    # a 128 x 256 x 192 problem (m, n multiples of the 128 x 256 base tile, k of the 64 step).
    mod = load(os.path.join(ref, "kernels/manual/a2a3/gemm_performance/scripts/gen_data.py"), "ref_gemm_gen")
    m, k, n = 128, 192, 256
    d = in_case_dir(tmp, "gemm_small")
    mod.gen_golden_data(mod.GemmParams(np.float16, np.float16, np.float32, m, k, n, False, np.float32))
    np.savez_compressed(os.path.join(out, "gemm.npz"),
                        a=read(os.path.join(d, "input/x1_gm.bin"), np.float16, (m, k)),
                        b_dn=read(os.path.join(d, "input/x2_gm.bin"), np.float16, (n, k)),
                        golden=read(os.path.join(d, "output/golden.bin"), np.float32, (m, n)))


def gen_vector2(ref, tmp, out):
    """Row-expand family, TROWMIN, column reductions, TTRANS, TSEL, TCMPS, TCMP: the float32 cases of the
    reference's generators (each module seeds np.random with 19 when it is loaded; cases run in its own order,
    the non-float32 ones too, so that the random stream matches)."""
    keep = {}
    base = os.path.join(ref, "tests/cpu/st/testcase")

    # trowexpand/gen_data.py:61-63 (case list), :19-25 (generator)
    mod = load(os.path.join(base, "trowexpand/gen_data.py"), "ref_trowexpand_gen")
    d = in_case_dir(tmp, "trowexpand_0")
    mod.gen_expand()
    keep["trowexpand_src"] = read(os.path.join(d, "input.bin"), np.float32, (64, 64))
    keep["trowexpand_golden"] = read(os.path.join(d, "golden.bin"), np.float32, (64, 64))

    # trowexpandop/gen_data.py:66-73 (case list x operations), :19-45 (generator)
    mod = load(os.path.join(base, "trowexpandop/gen_data.py"), "ref_trowexpandop_gen")
    P = mod.TRowExpandOpParams
    for pi, prm in enumerate([P(np.float32, 64, 64), P(np.float16, 16, 256)]):
        for op in ["div", "mul", "sub", "add", "min", "max", "expdif"]:
            d = in_case_dir(tmp, f"trowexpandop_{pi}_{op}")
            mod.gen_golden_data_trowexpandop(prm, op)
            if prm.dtype == np.float32:
                keep[f"trowexpandop_{op}_a"] = read(os.path.join(d, "input1.bin"), np.float32, (64, 64))
                keep[f"trowexpandop_{op}_s"] = read(os.path.join(d, "input2.bin"), np.float32, (64,))
                keep[f"trowexpandop_{op}_golden"] = read(os.path.join(d, "golden.bin"), np.float32, (64, 64))

    # trowmin/gen_data.py:59-65 (case list), :19-31 (generator)
    mod = load(os.path.join(base, "trowmin/gen_data.py"), "ref_trowmin_gen")
    P = mod.TRowminParams
    for i, prm in enumerate([P(np.float32, 64, 64, 64, 64, 64, 64), P(np.float16, 64, 64, 64, 64, 64, 64),
                             P(np.float16, 161, 161, 32, 32, 161, 161), P(np.float32, 77, 81, 32, 16, 77, 81),
                             P(np.float32, 32, 32, 32, 16, 32, 32)]):
        d = in_case_dir(tmp, f"trowmin_{i}")
        mod.gen_golden_data_trowmin(prm)
        if prm.dtype == np.float32:
            keep[f"trowmin{i}_src"] = read(os.path.join(d, "input1.bin"), np.float32, (prm.tile_row, prm.tile_col))
            keep[f"trowmin{i}_golden"] = read(os.path.join(d, "golden.bin"), np.float32)

    # tcolmax/gen_data.py:80-83 (case list), :17-43; tcolsum/gen_data.py:72-75, :17-36; tcolmin/gen_data.py:59-63, :19-31
    mod = load(os.path.join(base, "tcolmax/gen_data.py"), "ref_tcolmax_gen")
    P = mod.tcolmaxParams
    for i, prm in enumerate([P(np.float32, 64, 64, 64, 64, 64, 64), P(np.float16, 16, 256, 16, 256, 16, 256)]):
        in_case_dir(tmp, f"tcolmax_{i}")
        _, src, golden = mod.gen_golden_data_tcolmax("", prm)
        if prm.dtype == np.float32:
            keep["tcolmax_src"], keep["tcolmax_golden"] = src, golden[0].copy()
    mod = load(os.path.join(base, "tcolsum/gen_data.py"), "ref_tcolsum_gen")
    P = mod.TColsumParams
    for i, prm in enumerate([P(np.float32, 64, 64, 64, 64, 64, 64), P(np.float16, 16, 256, 16, 256, 16, 256)]):
        in_case_dir(tmp, f"tcolsum_{i}")
        src, golden = mod.gen_golden_data_tcolsum("", prm)
        if prm.dtype == np.float32:
            keep["tcolsum_src"], keep["tcolsum_golden"] = src, golden[0].copy()
    mod = load(os.path.join(base, "tcolmin/gen_data.py"), "ref_tcolmin_gen")
    P = mod.TColminParams
    for i, prm in enumerate([P(np.float32, 64, 64, 64, 64, 64, 64), P(np.float16, 64, 64, 64, 64, 64, 64),
                             P(np.float32, 32, 32, 32, 16, 32, 32)]):
        d = in_case_dir(tmp, f"tcolmin_{i}")
        mod.gen_golden_data_tcolmin(prm)
        if prm.dtype == np.float32:
            keep[f"tcolmin{i}_src"] = read(os.path.join(d, "input1.bin"), np.float32, (prm.tile_row, prm.tile_col))
            keep[f"tcolmin{i}_golden"] = read(os.path.join(d, "golden.bin"), np.float32)

    # ttrans/gen_data.py:41-43 (case list), :19-27 (generator)
    mod = load(os.path.join(base, "ttrans/gen_data.py"), "ref_ttrans_gen")
    d = in_case_dir(tmp, "ttrans_0")
    mod.gen_golden("", mod.TTransParams(np.float32, 128, 128))
    keep["ttrans_src"] = read(os.path.join(d, "x1_gm.bin"), np.float32, (128, 128))
    keep["ttrans_golden"] = read(os.path.join(d, "golden.bin"), np.float32, (128, 128))

    # tsel/gen_data.py:62-72 (case list), :28-51 (generator); the float32 cases come first
    mod = load(os.path.join(base, "tsel/gen_data.py"), "ref_tsel_gen")
    P = mod.TSelParams
    for i, prm in enumerate([P("c1", np.float32, 2, 128, 2, 128), P("c2", np.float32, 2, 32, 2, 32),
                             P("c3", np.float32, 2, 160, 2, 160)]):
        d = in_case_dir(tmp, f"tsel_{i}")
        mod.gen_golden_data_tsel(prm)
        shape = (prm.validRows, prm.validCols)
        keep[f"tsel{i}_a"] = read(os.path.join(d, "input0.bin"), np.float32, shape)
        keep[f"tsel{i}_b"] = read(os.path.join(d, "input1.bin"), np.float32, shape)
        keep[f"tsel{i}_mask"] = read(os.path.join(d, "mask.bin"), np.uint8)
        keep[f"tsel{i}_golden"] = read(os.path.join(d, "golden.bin"), np.float32, shape)

    # tcmps/gen_data.py:95-106 (case list), :17-64 (generator); float32 cases whose tile is the whole tensor
    mod = load(os.path.join(base, "tcmps/gen_data.py"), "ref_tcmps_gen")
    P = mod.tcmpsParams
    modes = {"CmpMode::EQ": 0, "CmpMode::NE": 1, "CmpMode::LT": 2, "CmpMode::LE": 3, "CmpMode::GT": 4, "CmpMode::GE": 5}
    cases = [P(np.float16, 32, 32, 32, 32, 32, 32, "CmpMode::GE"), P(np.float32, 1, 64, 1, 64, 1, 64, "CmpMode::EQ"),
             P(np.float32, 8, 64, 8, 64, 8, 64, "CmpMode::GT"), P(np.float32, 4, 64, 4, 64, 4, 64, "CmpMode::NE"),
             P(np.float32, 128, 128, 64, 64, 128, 128, "CmpMode::LT"), P(np.int32, 64, 64, 32, 32, 64, 64, "CmpMode::EQ"),
             P(np.int32, 16, 32, 16, 32, 16, 32, "CmpMode::EQ"), P(np.float32, 128, 128, 128, 128, 128, 128, "CmpMode::LE")]
    for i, prm in enumerate(cases):
        d = in_case_dir(tmp, f"tcmps_{i}")
        mod.gen_golden_data_tcmps("", prm)
        if prm.dtype == np.float32 and prm.tile_row == prm.global_row:
            keep[f"tcmps{i}_src"] = read(os.path.join(d, "input1.bin"), np.float32, (prm.tile_row, prm.tile_col))
            keep[f"tcmps{i}_scalar"] = read(os.path.join(d, "input2.bin"), np.float32)
            keep[f"tcmps{i}_mode"] = np.array(modes[prm.mode])
            keep[f"tcmps{i}_golden"] = read(os.path.join(d, "golden.bin"), np.uint8)

    # tcmp/gen_data.py:92-97 (case list), :18-56 (generator)
    mod = load(os.path.join(base, "tcmp/gen_data.py"), "ref_tcmp_gen")
    _, a, b, golden = mod.gen_golden_data_tcmp("", mod.TCmpParams(np.float32, 64, 64, 64, 64, 64, 64, "EQ")) \
        if in_case_dir(tmp, "tcmp_0") else (None, None, None, None)
    keep["tcmp_a"], keep["tcmp_b"], keep["tcmp_golden"] = a, b, golden
    np.savez_compressed(os.path.join(out, "vector2.npz"), **keep)


def gen_harness(ref, tmp, out):
    """The case list files of the flash-attention harness, written by the reference's own generator
    (kernels/manual/common/flash_atten/scripts/generate_cases.py:168-232) for its default cases and for an explicit
    list: kept as text fixtures so that the B200 replay tool's reader / writer can be compared byte for byte."""
    import subprocess
    script = os.path.join(ref, "kernels/manual/common/flash_atten/scripts/generate_cases.py")
    for tag, extra in (("default", []), ("explicit", ["--cases", "128,128,512,128", "--cases", "128,512,2048,128,512",
                                                      "--qk-preload", "2"])):
        d = in_case_dir(tmp, f"harness_{tag}")
        subprocess.check_call([sys.executable, script, "--output-header", os.path.join(d, "generated_cases.h"),
                               "--output-json", os.path.join(d, "generated_cases.json")] + extra,
                              stdout=subprocess.DEVNULL)
        for name in ("generated_cases.h", "generated_cases.json"):
            with open(os.path.join(d, name)) as f:
                text = f.read()
            with open(os.path.join(out, f"harness_{tag}_{name}"), "w") as f:
                f.write(text)


def gen_mla(ref, tmp, out):
    """One multi-latent-attention head (S 128, D 64, R 64, fp16 operands): seeded inputs and the output of the
    reference's CPU simulation running the instruction sequence of demos/cpu/mla_attention_demo/mla_attention_demo.cpp:326-376
    (oracle/ref_mla.cpp, compiled against the reference headers as oracle/_ref/libpto_ref.so)."""
    import ctypes
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    import oracle
    if oracle.ref is None:
        raise SystemExit("oracle/_ref/libpto_ref.so is needed for the MLA fixture")
    r = np.random.default_rng(20260)
    S, D, R = 128, 64, 64
    q, k, v = (r.standard_normal((S, D)).astype(np.float16) for _ in range(3))
    wq, wk, wv = ((r.standard_normal((D, R)) / np.sqrt(D)).astype(np.float16) for _ in range(3))
    wo = (r.standard_normal((R, D)) / np.sqrt(R)).astype(np.float16)
    o = np.zeros((S, D), np.float32)
    P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    scale = 1.0 / np.sqrt(R)
    rc = oracle.ref.lib.pto_ref_mla_head_f16_128x64x64(P(q), P(k), P(v), P(wq), P(wk), P(wv), P(wo), P(o), ctypes.c_float(scale))
    assert rc == 0
    np.savez_compressed(os.path.join(out, "mla.npz"), q=q, k=k, v=v, wq=wq, wk=wk, wv=wv, wo=wo, o=o, scale=np.float32(scale))


def gen_mxgemm(ref, tmp, out):
    """MX block-scaled fp8 GEMM: inputs, e8m0 scales and golden written by the reference's own generator
    (kernels/manual/a5/matmul_mxfp8_performance/scripts/gen_data.py:27-70; it needs ml_dtypes), called for two small
    problems instead of its 6144^3: float8_e5m2 at 256 x 384 x 256 (m, k, n) and float8_e4m3fn at 128 x 128 x 256.
    Files as the generator writes them: A m x k, B transposed to n x k, scaleA m x k/32, scaleB transposed to n x k/32,
    golden m x n bfloat16 (stored here as its 16-bit patterns)."""
    mod = load(os.path.join(ref, "kernels/manual/a5/matmul_mxfp8_performance/scripts/gen_data.py"), "ref_mx_gen")
    saved = {}
    for tag, dtype, (m, k, n) in (("e5m2", mod.fp8_e5m2, (256, 384, 256)), ("e4m3", mod.fp8_e4m3fn, (128, 128, 256))):
        d = in_case_dir(tmp, f"mxgemm_{tag}")
        mod.gen_golden_data(mod.MxMatmulParams(dtype, dtype, mod.bfloat16, m, k, n, False))
        saved[f"{tag}_a"] = read(os.path.join(d, "input/x1_gm.bin"), np.uint8, (m, k))
        saved[f"{tag}_b"] = read(os.path.join(d, "input/x2_gm.bin"), np.uint8, (n, k))
        saved[f"{tag}_scale_a"] = read(os.path.join(d, "input/x1_scale_gm.bin"), np.uint8, (m, k // 32))
        saved[f"{tag}_scale_b"] = read(os.path.join(d, "input/x2_scale_gm.bin"), np.uint8, (n, k // 32))
        saved[f"{tag}_golden_bf16_bits"] = read(os.path.join(d, "output/golden.bin"), np.uint16, (m, n))
    np.savez_compressed(os.path.join(out, "mxgemm.npz"), **saved)


def gen_mxgemm_fp4(ref, tmp, out):
    """MXFP4 form: packed inputs, scales and golden written by the reference's generator
    (kernels/manual/a5/matmul_mxfp4_performance/scripts/gen_data.py:24-80) for a 128 x 512 x 256 (m, k, n) problem.
    The generator imports the `en_dtypes` package for its float4 types; that package is not in this image, so the
    module name is bound to a stand-in whose float4_e2m1 is ml_dtypes.float4_e2m1fn - the same E2M1 format, one value
    per byte in the low four bits, which is all pack_two_fp4 (:24-34) relies on."""
    import types

    import ml_dtypes
    sys.modules.setdefault("en_dtypes", types.SimpleNamespace(float4_e2m1=ml_dtypes.float4_e2m1fn,
                                                              float4_e1m2=ml_dtypes.float4_e2m1fn))
    mod = load(os.path.join(ref, "kernels/manual/a5/matmul_mxfp4_performance/scripts/gen_data.py"), "ref_mx4_gen")
    m, k, n = 128, 512, 256
    d = in_case_dir(tmp, "mxgemm_fp4")
    mod.gen_golden_data(mod.MxMatmulParams(mod.fp4_e2m1x2, mod.fp4_e2m1x2, mod.bfloat16, m, k, n, False))
    np.savez_compressed(os.path.join(out, "mxgemm_fp4.npz"),
                        a=read(os.path.join(d, "input/x1_gm.bin"), np.uint8, (m, k // 2)),
                        b=read(os.path.join(d, "input/x2_gm.bin"), np.uint8, (n, k // 2)),
                        scale_a=read(os.path.join(d, "input/x1_scale_gm.bin"), np.uint8, (m, k // 32)),
                        scale_b=read(os.path.join(d, "input/x2_scale_gm.bin"), np.uint8, (n, k // 32)),
                        golden_bf16_bits=read(os.path.join(d, "output/golden.bin"), np.uint16, (m, n)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("PTO_REFERENCE_ROOT") or
                    os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"),
                    help="root of the reference tree (default: $PTO_REFERENCE_ROOT, else `reference` beside the repository)")
    args = ap.parse_args()
    cwd = os.getcwd()
    with tempfile.TemporaryDirectory() as tmp:
        try:
            for fn in (gen_tcvt, gen_tgather, gen_tmatmul, gen_rowops, gen_attention, gen_gemm, gen_vector2, gen_harness, gen_mla, gen_mxgemm, gen_mxgemm_fp4, gen_tmatmul_i8, gen_tmatmul_bias):
                os.chdir(tmp)
                fn(args.reference, tmp, HERE)
        finally:
            os.chdir(cwd)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz") or f.startswith("harness_"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    sys.exit(main())
