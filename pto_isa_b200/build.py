"""Compiles the CUDA sources under csrc/ into libpto_b200.so (sm_100a only), in-tree next to this file.

`python -m pto_isa_b200.build` or `pto_isa_b200.build.build()`.  nvcc cross-compiles without a GPU.
The two `call_kernel` shim libraries carry the exact symbol name the reference's ctypes loaders bind
(demos/torch_jit/gemm/jit_util_gemm.py:66-73, demos/torch_jit/flash_atten/jit_util_flash.py:76-94).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpto_b200.so")
SHIMS = {
    "libpto_b200_gemm_jit.so": "shim_gemm_call_kernel.cpp",
    "libpto_b200_flash_jit.so": "shim_fa_call_kernel.cpp",
}
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return nvcc


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    flags = list(NVCC_FLAGS)
    deps = _sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "pto_b200.h"))
    if force or _stale(LIB, deps):
        cmd = [_nvcc()] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-shared", "-o", LIB] + _sources()
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    # tile programs written against include/pto/ (the PTO surface on this backend)
    prog_src = os.path.join(CSRC, "pto_programs", "programs.cu")
    prog_out = os.path.join(HERE, "libpto_b200_programs.so")
    pto_headers = [os.path.join(dp, f) for dp, _, fs in os.walk(os.path.join(HERE, "..", "include", "pto")) for f in fs]
    if force or _stale(prog_out, [prog_src] + pto_headers):
        subprocess.check_call([_nvcc()] + flags + ["--extended-lambda", "-I", os.path.join(HERE, "..", "include"),
                                                  "-shared", "-o", prog_out, prog_src])
    build_host(force)
    for so, src in SHIMS.items():
        src_path = os.path.join(CSRC, src)
        out = os.path.join(HERE, so)
        if os.path.exists(src_path) and (force or _stale(out, [src_path, LIB])):
            subprocess.check_call(["g++", "-O2", "-fPIC", "-shared", "-o", out, src_path, "-L" + HERE, "-lpto_b200",
                                   "-Wl,-rpath,$ORIGIN"])
    return LIB


def build_host(force=False):
    """The C++ half of the boundary: the reference's host launcher templates over the C ABI
    (libpto_b200_launchers.so, include/pto_b200_launchers.hpp) and a C++ host program in the shape of the
    reference's kernel hosts (pto_b200_host).  Plain g++; the CUDA runtime supplies memory and streams."""
    host_dir = os.path.join(CSRC, "host")
    hdrs = [os.path.join(HERE, "..", "include", "pto_b200_launchers.hpp"), os.path.join(HERE, "..", "include", "pto_b200.h")]
    lib_out = os.path.join(HERE, "libpto_b200_launchers.so")
    refk = os.path.join(HERE, "libpto_b200_refkernels.so")
    src = os.path.join(host_dir, "launchers.cpp")
    deps = [src, LIB] + hdrs + ([refk] if os.path.exists(refk) else [])
    if force or _stale(lib_out, deps):
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", lib_out, src, "-L" + HERE, "-lpto_b200",
               "-Wl,-rpath,$ORIGIN"]
        if os.path.exists(refk):  # LaunchTMATMUL<key> runs the reference's tile programs compiled for B200
            cmd += ["-Wl,--no-as-needed", "-lpto_b200_refkernels", "-Wl,--as-needed"]  # (weak references only)
        subprocess.check_call(cmd)
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    exe = os.path.join(HERE, "pto_b200_host")
    main_src = os.path.join(host_dir, "host_main.cpp")
    if force or _stale(exe, [main_src, lib_out] + hdrs):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-o", exe, main_src, "-I" + os.path.join(cuda_home, "include"),
                               "-L" + HERE, "-lpto_b200_launchers", "-lpto_b200", "-L" + os.path.join(cuda_home, "lib64"),
                               "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda_home, "lib64")])
    return exe


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
