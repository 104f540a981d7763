"""Builds the reference's own tile programs against this repository's PTO headers (include/pto/) with nvcc.

The device code of the reference kernels is compiled unchanged, with two exceptions that CUDA cannot express as
written.  (1) Ascend's launch statement `kernel<<<blocks, l2ctrl, stream>>>(args)` (the second launch argument is
an L2 control pointer there, a block shape in CUDA): `rewrite_launches` turns exactly those statements into
`PTO_B200_LAUNCH((kernel), blocks, stream, args)`.  (2) A function-local `static T name = init;` in device code:
in CUDA that is one variable for the whole grid, where the reference means one per core; `rewrite_core_statics`
turns the declaration into `PTO_B200_CORE_STATIC(T, name, init, slot)` (a per-block value, include/pto/b200/
runtime.hpp).  Nothing else in the files is touched, and the rewritten text only ever exists in the build directory.
Unit-test kernels and headers that contain neither construct are included straight from the reference tree.

The result, pto_isa_b200/libpto_b200_refkernels.so, is built where the reference tree is available and
travels with the package; tests that need it skip when it is absent.
"""
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "libpto_b200_refkernels.so")
WRAPPER = os.path.join(HERE, "csrc", "refkernels", "wrappers.cu.in")
# the same reference sources compiled with the core's pipes on warps of their own (PTO_B200_PIPE_WARPS is a property of a
# translation unit, and of its library: the two must not be linked into one)
OUT_PW = os.path.join(HERE, "libpto_b200_refkernels_pw.so")
WRAPPER_PW = os.path.join(HERE, "csrc", "refkernels", "wrappers_pw.cu.in")

_LAUNCH = re.compile(r"<<<\s*([^,<>]+?)\s*,\s*nullptr\s*,\s*([^,<>]+?)\s*>>>\s*\(")


def rewrite_launches(text):
    """`callee<<<blocks, nullptr, stream>>>(args);` -> `PTO_B200_LAUNCH((callee), blocks, stream, args);`"""
    out = []
    pos = 0
    while True:
        m = _LAUNCH.search(text, pos)
        if not m:
            out.append(text[pos:])
            break
        # the callee expression runs back to the previous statement / block boundary
        start = max(text.rfind(";", pos, m.start()), text.rfind("{", pos, m.start()), text.rfind("}", pos, m.start())) + 1
        callee = text[start:m.start()]
        # preprocessor and comment lines between the previous statement and the callee stay where they are
        while True:
            stripped = callee.lstrip()
            if not (stripped.startswith("#") or stripped.startswith("//")):
                break
            cut = len(callee) - len(stripped) + (stripped.index("\n") + 1 if "\n" in stripped else len(stripped))
            start += cut
            callee = callee[cut:]
        lead = callee[: len(callee) - len(callee.lstrip())]
        # the argument list runs to the matching parenthesis
        depth, i = 1, m.end()
        while depth:
            depth += {"(": 1, ")": -1}.get(text[i], 0)
            i += 1
        args = text[m.end(): i - 1].strip()
        out.append(text[pos:start])
        out.append(f"{lead}PTO_B200_LAUNCH(({callee.strip()}), {m.group(1)}, {m.group(2)}"
                   + (f", {args}" if args else "") + ")")
        pos = i
    return "".join(out)


_STATIC = re.compile(r"^(\s*)static\s+([A-Za-z_][\w:]*)\s+([A-Za-z_]\w*)\s*=\s*([^;]+);", re.M)


def rewrite_core_statics(text):
    """`static T name = init;` (indented, i.e. inside a function) -> `PTO_B200_CORE_STATIC(T, name, init, slot);`"""
    slot = [0]

    def rep(m):
        if not m.group(1):  # file scope: not a function-local static
            return m.group(0)
        out = f"{m.group(1)}PTO_B200_CORE_STATIC({m.group(2)}, {m.group(3)}, {m.group(4).strip()}, {slot[0]});"
        slot[0] += 1
        return out

    return _STATIC.sub(rep, text)


def fa_kernel_check(reference, build_dir, nvcc, verbose=False):
    """Compiles the reference's flash-attention kernel file for sm_100a in both of its flavours (cube core / vector
    cores) against include/pto/: objects only, see csrc/refkernels/fa_kernel_check.cu.in.  The case list header is
    produced by the reference's own generator with its default cases."""
    fa = os.path.join(reference, "kernels", "manual", "common", "flash_atten")
    with open(os.path.join(fa, "fa_performance_kernel.cpp")) as f:
        text = rewrite_core_statics(rewrite_launches(f.read()))
    with open(os.path.join(build_dir, "fa_performance_kernel.inc"), "w") as f:
        f.write(text)
    # the kernel file includes its matmul macro header by name: the rewritten copy beside it is found first
    with open(os.path.join(fa, "pto_macro_matmul.hpp")) as f:
        macro = rewrite_core_statics(rewrite_launches(f.read()))
    with open(os.path.join(build_dir, "pto_macro_matmul.hpp"), "w") as f:
        f.write(macro)
    subprocess.check_call([sys.executable, os.path.join(fa, "scripts", "generate_cases.py"), "--output-header",
                           os.path.join(build_dir, "generated_cases.h"), "--output-json",
                           os.path.join(build_dir, "generated_cases.json")], stdout=subprocess.DEVNULL)
    with open(os.path.join(HERE, "csrc", "refkernels", "fa_kernel_check.cu.in")) as f:
        template = f.read()
    objects = []
    for flavour in ("CUBE", "VEC"):
        tu = os.path.join(build_dir, f"fa_kernel_check_{flavour.lower()}.cu")
        with open(tu, "w") as f:
            f.write(template.replace("@FLAVOUR@", flavour))
        obj = tu[:-3] + ".o"
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++20", "--extended-lambda",
               "--expt-relaxed-constexpr", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "include", "pto", "b200", "compat"),
               "-I", build_dir, "-I", fa, "-c", "-o", obj, tu]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
        objects.append(obj)
    return objects


def default_reference():
    """The reference tree: $PTO_REFERENCE_ROOT, else a `reference` directory beside the repository."""
    return os.environ.get("PTO_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


def build(reference=None, force=False, verbose=False):
    """Returns the path of the built library, or None when the reference tree is not present."""
    reference = reference or default_reference()
    if not os.path.isdir(os.path.join(reference, "kernels")):
        return OUT if os.path.exists(OUT) else None
    newest = max(max(os.path.getmtime(os.path.join(dp, f)) for dp, _, fs in os.walk(os.path.join(ROOT, "include", "pto"))
                     for f in fs), os.path.getmtime(WRAPPER), os.path.getmtime(WRAPPER_PW),
                 os.path.getmtime(os.path.join(HERE, "csrc", "refkernels", "ref_fa_head.inc")))
    if not force and all(os.path.exists(o) and os.path.getmtime(o) >= newest for o in (OUT, OUT_PW)):
        return OUT
    build_dir = os.path.join(HERE, "build", "refkernels")
    os.makedirs(build_dir, exist_ok=True)
    sources = {
        "gemm_performance_kernel.inc": "kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp",
        "pto_macro_matmul.inc": "kernels/manual/common/flash_atten/pto_macro_matmul.hpp",
    }
    for name, rel in sources.items():
        with open(os.path.join(reference, rel)) as f:
            text = rewrite_core_statics(rewrite_launches(f.read()))
        with open(os.path.join(build_dir, name), "w") as f:
            f.write(text)
    shutil.copyfile(os.path.join(HERE, "csrc", "refkernels", "ref_fa_head.inc"), os.path.join(build_dir, "ref_fa_head.inc"))
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    fa_kernel_check(reference, build_dir, nvcc, verbose)
    extra = os.environ.get("PTO_B200_REFK_NVCC_FLAGS", "").split()  # e.g. -DPTO_B200_TIMELINE, -DPTO_B200_TRACE_WAITS
    for wrapper, out in ((WRAPPER, OUT), (WRAPPER_PW, OUT_PW)):
        tu = os.path.join(build_dir, os.path.basename(wrapper)[:-3])
        with open(wrapper) as f:
            body = f.read().replace("@REFERENCE@", reference)
        with open(tu, "w") as f:
            f.write(body)
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++20", "--extended-lambda",
               "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", build_dir,
               *extra, "-shared", "-o", out, tu]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return OUT


_CODES = {0x1: "wait_flag entered", 0x2: "wait_flag passed", 0x3: "set_flag", 0x4: "TLOAD", 0x5: "TEXTRACT", 0x6: "TMATMUL",
          0x7: "TSTORE"}


def timeline(name="pto_refk_gemm_pw_6144_k128", first=400, count=48):
    """Prints the stamps of block 0 of one 6144^3 launch of a GEMM entry point (`name`), from libraries built with
    PTO_B200_REFK_NVCC_FLAGS=-DPTO_B200_TIMELINE (include/pto/b200/runtime.hpp explains the codes): per stamping thread
    the cycles between consecutive stamps, `count` of them from entry `first`, and the mean cycles per k iteration."""
    import ctypes

    import numpy as np
    import torch
    lib = ctypes.CDLL(OUT_PW if "_pw_" in name else OUT)
    m = n = k = 6144
    g = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).half()
    b = (torch.rand(n, k, device="cuda", generator=g) * 2 - 1).half()
    c = torch.zeros(m, n, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fn = getattr(lib, name)
    fn(ptr(c), ptr(a), ptr(b), stream(), ptr(st))
    torch.cuda.synchronize()
    lib.pto_refk_timeline(None, None, 1)
    fn(ptr(c), ptr(a), ptr(b), stream(), ptr(st))
    torch.cuda.synchronize()
    out = np.zeros((3, 4096), np.uint64)
    counts = np.zeros(3, np.uint32)
    cap = lib.pto_refk_timeline(out.ctypes.data_as(ctypes.c_void_p), counts.ctypes.data_as(ctypes.c_void_p), 0)
    print("status", st.tolist(), "stamps per thread", counts.tolist())
    for row, who in enumerate(("thread 0 (MTE2, or the whole block)", "thread of MTE1 / M", "first thread of the vector / store warps")):
        used = min(int(counts[row]), cap)
        if used < 2:
            continue
        codes = (out[row, :used] >> np.uint64(48)).astype(np.int64)
        clk = (out[row, :used] & np.uint64((1 << 48) - 1)).astype(np.int64)
        issues = np.flatnonzero(codes == 0x6000)
        per_iter = f", {(clk[issues[-1]] - clk[issues[0]]) / max(1, len(issues) - 1):.0f} cycles per TMATMUL" if len(issues) > 1 else ""
        print(f"--- {who}: {used} stamps{per_iter}")
        for i in range(min(first, used - 1), min(used, first + count)):
            kind = _CODES.get(int(codes[i]) >> 12, "?")
            print(f"  {i:5d} {int(codes[i]):#06x} {kind:18s} +{int(clk[i] - clk[i - 1]) if i else 0:6d}")


def run(name="pto_refk_gemm_pw_6144_k128", launches=12):
    """Launches a 6144^3 GEMM entry point `launches` times and prints the CUDA-event time of the last ten."""
    import ctypes

    import torch
    lib = ctypes.CDLL(OUT_PW if "_pw_" in name else OUT)
    m = n = k = 6144
    g = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).half()
    b = (torch.rand(n, k, device="cuda", generator=g) * 2 - 1).half()
    c = torch.zeros(m, n, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fn = getattr(lib, name)
    timed = min(10, launches)
    for _ in range(launches - timed):
        fn(ptr(c), ptr(a), ptr(b), stream, ptr(st))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(timed):
        fn(ptr(c), ptr(a), ptr(b), stream, ptr(st))
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / timed
    print(f"{name}: {ms:.3f} ms per launch, {2.0 * m * n * k / ms / 1e9:.1f} TFLOP/s, status record {st.tolist()}")
    if st.tolist() != [0, 0, 0, 0]:
        raise SystemExit(1)


if __name__ == "__main__":
    import sys
    if "--run" in sys.argv:
        i = sys.argv.index("--run")
        run(sys.argv[i + 1], int(sys.argv[i + 2]) if len(sys.argv) > i + 2 else 12)
    elif "--timeline" in sys.argv:
        i = sys.argv.index("--timeline")
        timeline(*(sys.argv[i + 1:i + 2]))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
