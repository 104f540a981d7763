"""Host callers shaped like the reference's torch demos, over CUDA tensors.

* `load_lib()` / `load_flash_lib()` return the callables that demos/torch_jit/gemm/jit_util_gemm.py:60-95 and
  demos/torch_jit/flash_atten/jit_util_flash.py:70-135 return - `gemm(c, a, b, block_dim, stream_ptr)` and
  `flash(q, k, v, o_out, <seven workspaces>, stream_ptr, is_causal)` - bound with ctypes to the exported symbol
  `call_kernel` of libpto_b200_gemm_jit.so / libpto_b200_flash_jit.so.  Nothing is compiled at call time: the
  libraries are built ahead (`python -m pto_isa_b200.build`), so the reference's `compile_cpp` step has no twin.
* `torch.ops.pto_b200.pto_gemm_basic(a, b_dn)` is the operator of demos/baseline/gemm_basic
  (csrc/host/my_gemm_basic.cpp:43-53, schema "pto_gemm_basic(Tensor a, Tensor b_dn) -> Tensor") for CUDA tensors:
  a is [m, k] fp16, b_dn is [n, k] fp16 (b.t().contiguous()), the result is [m, n] fp32.  The reference fixes
  m, k, n = 512, 2048, 1536; any shape the kernel accepts works here.
* `attn_flops_matmul_softmax_scale` / `tflops` are the flop accounting of
  demos/torch_jit/flash_atten/fa_benchmark.py:30-66.
"""
import ctypes
import os

import torch

from . import _lib, ops

_HERE = os.path.dirname(os.path.abspath(__file__))
GEMM_JIT_LIB = os.path.join(_HERE, "libpto_b200_gemm_jit.so")
FLASH_JIT_LIB = os.path.join(_HERE, "libpto_b200_flash_jit.so")

BLOCK_DIM = 24  # the reference passes its core count; the B200 kernel sizes its own grid and ignores it
GEMM_JIT_M = GEMM_JIT_N = GEMM_JIT_K = 6144  # the problem `call_kernel` of the GEMM library is built for


def torch_to_ctypes(t):
    return ctypes.c_void_p(t.data_ptr())


def _current_stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _open(path):
    if not os.path.exists(path):
        raise _lib.PtoB200Error(f"{path} is missing: build it with `python -m pto_isa_b200.build`")
    _lib.lib()  # the shim forwards into libpto_b200.so: load it first so that the dependency resolves
    return ctypes.CDLL(os.path.abspath(path))


def _check_status(what):
    rc = _lib.lib().pto_b200_last_status()
    _lib.check(rc, what)


def load_lib(lib_path=None, check_type=True):
    """Returns gemm(c, a, b, block_dim=24, stream_ptr=None): c [6144, 6144] fp32 = a [6144, 6144] fp16 times
    b stored n x k, through `call_kernel(blockDim, stream, out, src0, src1)`."""
    lib = _open(lib_path or GEMM_JIT_LIB)
    if check_type:
        lib.call_kernel.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                    ctypes.c_void_p]
        lib.call_kernel.restype = None

    def gemm(c, a, b, block_dim=BLOCK_DIM, stream_ptr=None):
        for t, shape, dtype in ((c, (GEMM_JIT_M, GEMM_JIT_N), torch.float32), (a, (GEMM_JIT_M, GEMM_JIT_K), torch.float16),
                                (b, (GEMM_JIT_N, GEMM_JIT_K), torch.float16)):
            if not t.is_cuda or tuple(t.shape) != shape or t.dtype != dtype or not t.is_contiguous():
                raise _lib.PtoB200Error(f"gemm (call_kernel): expected a contiguous CUDA {dtype} tensor of shape {shape}")
        with torch.cuda.device(a.device):
            lib.call_kernel(block_dim, stream_ptr if stream_ptr is not None else _current_stream_ptr(),
                            torch_to_ctypes(c), torch_to_ctypes(a), torch_to_ctypes(b))
        _check_status("call_kernel (gemm)")

    return gemm


def load_flash_lib(lib_path=None, check_type=True):
    """Returns flash(q, k, v, o_out, out_device, xexp_device, p_out_fp32_device, out_2device, g_sum_device,
    exp_max_device, o_parts_device, stream_ptr=None, is_causal=False) for one head: q [s0, d], k / v [s1, d] fp16,
    o_out [s0, d] fp32.  The seven workspace tensors are the reference's global-memory FIFOs and snapshots; they are
    accepted for signature compatibility and left untouched (None is allowed)."""
    lib = _open(lib_path or FLASH_JIT_LIB)
    if check_type:
        lib.call_kernel.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_bool] + \
                                   [ctypes.c_void_p] * 11
        lib.call_kernel.restype = None

    def ptr_or_null(t):
        return ctypes.c_void_p(0) if t is None else torch_to_ctypes(t)

    def flash(q, k, v, o_out, out_device=None, xexp_device=None, p_out_fp32_device=None, out_2device=None,
              g_sum_device=None, exp_max_device=None, o_parts_device=None, stream_ptr=None, is_causal=False):
        for t, dtype in ((q, torch.float16), (k, torch.float16), (v, torch.float16), (o_out, torch.float32)):
            if not t.is_cuda or t.dtype != dtype or t.dim() != 2 or not t.is_contiguous():
                raise _lib.PtoB200Error(f"flash (call_kernel): expected contiguous 2-D CUDA tensors, {dtype} here")
        with torch.cuda.device(q.device):
            lib.call_kernel(stream_ptr if stream_ptr is not None else _current_stream_ptr(), q.shape[1], q.shape[0],
                            k.shape[0], bool(is_causal), torch_to_ctypes(q), torch_to_ctypes(k), torch_to_ctypes(v),
                            torch_to_ctypes(o_out), ptr_or_null(out_device), ptr_or_null(xexp_device),
                            ptr_or_null(p_out_fp32_device), ptr_or_null(out_2device), ptr_or_null(g_sum_device),
                            ptr_or_null(exp_max_device), ptr_or_null(o_parts_device))
        _check_status("call_kernel (flash attention)")

    return flash


# ---------------------------------------------------------------- flop accounting of the reference's benchmark

def attn_flops_matmul_softmax_scale(batch_size, s_q, s_k, h, include_scale=True, count_exp_as_flop=True,
                                    count_max_as_flop=True):
    flops_matmul = 4 * batch_size * s_q * s_k * h
    flops_scale = (batch_size * s_q * s_k) if include_scale else 0
    rows = batch_size * s_q
    softmax_ops = 0
    if count_max_as_flop:
        softmax_ops += rows * (s_k - 1)
    softmax_ops += rows * s_k
    if count_exp_as_flop:
        softmax_ops += rows * s_k
    softmax_ops += rows * (s_k - 1)
    softmax_ops += rows * s_k
    return {"total": flops_matmul + flops_scale + softmax_ops, "matmul": flops_matmul, "scale": flops_scale,
            "softmax": softmax_ops}


def tflops(flops, ms):
    return flops / (ms * 1e-3) / 1e12


# ---------------------------------------------------------------- torch operator

_OP_NS = "pto_b200"
_lib_def = torch.library.Library(_OP_NS, "FRAGMENT")
_lib_def.define("pto_gemm_basic(Tensor a, Tensor b_dn) -> Tensor")


def _pto_gemm_basic_cuda(a, b_dn):
    if a.dim() != 2 or b_dn.dim() != 2 or a.shape[1] != b_dn.shape[1]:
        raise _lib.PtoB200Error("pto_gemm_basic: a must be [m, k] and b_dn [n, k] (b.t().contiguous())")
    if not a.is_contiguous() or not b_dn.is_contiguous():
        raise _lib.PtoB200Error("pto_gemm_basic: a and b_dn must be contiguous")
    return ops.gemm(a, b_dn, b_layout=1)


def _pto_gemm_basic_meta(a, b_dn):
    return a.new_empty((a.shape[0], b_dn.shape[0]), dtype=torch.float32)


_lib_def.impl("pto_gemm_basic", _pto_gemm_basic_cuda, "CUDA")
_lib_def.impl("pto_gemm_basic", _pto_gemm_basic_meta, "Meta")


def pto_gemm_basic(a, b_dn):
    return torch.ops.pto_b200.pto_gemm_basic(a, b_dn)
