"""ctypes binding of libpto_b200.so; every symbol declared in include/pto_b200.h gets its signature here."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "libpto_b200.so"


class PtoB200Error(RuntimeError):
    pass


def lib_path():
    return os.path.join(_HERE, _LIB_NAME)


_vp, _i, _i64, _f, _u32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_uint32

# name -> (restype, argtypes); mirrors include/pto_b200.h one to one
SIGNATURES = {
    "pto_b200_version": (_i, []),
    "pto_b200_last_error": (ctypes.c_char_p, []),
    "pto_b200_last_status": (_i, []),
    "pto_b200_device_status": (_i, [_vp]),
    "pto_b200_device_status_ex": (_i, [_vp, _vp]),
    "pto_b200_status_record": (_vp, []),
    "pto_b200_set_profile_buffer": (_i, [_vp, _i64, _vp]),
    "pto_b200_probe_random_reads": (_i, [_vp, _i64, _i64, _vp, _vp]),
    "pto_b200_tcvt_f32_f16": (_i, [_vp, _vp, _i64, _vp]),
    "pto_b200_tcvt_f32_bf16": (_i, [_vp, _vp, _i64, _vp]),
    "pto_b200_tcvt_f32_i32": (_i, [_vp, _vp, _i64, _i, _vp]),
    "pto_b200_tgather": (_i, [_vp, _i64, _vp, _vp, _i64, _i, _vp]),
    "pto_b200_tgather_mask": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "pto_b200_trowmax_f32": (_i, [_vp, _vp, _i, _i, _i64, _vp]),
    "pto_b200_trowsum_f32": (_i, [_vp, _vp, _i, _i, _i64, _vp]),
    "pto_b200_texp_f32": (_i, [_vp, _vp, _i64, _vp]),
    "pto_b200_tbinary_f32": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "pto_b200_tscalar_f32": (_i, [_vp, _f, _vp, _i64, _i, _vp]),
    "pto_b200_trowexpand_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "pto_b200_trowmin_f32": (_i, [_vp, _vp, _i, _i, _i64, _vp]),
    "pto_b200_tcolreduce_workspace_bytes": (_i64, [_i, _i]),
    "pto_b200_tcolreduce_f32": (_i, [_vp, _vp, _i, _i, _i64, _i, _vp, _i64, _vp]),
    "pto_b200_tfillpad": (_i, [_vp, _vp, _i, _i, _i, _i, _u32, _i, _vp]),
    "pto_b200_ttrans": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "pto_b200_tsel": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _vp]),
    "pto_b200_tcmps_f32": (_i, [_vp, _f, _vp, _i64, _i, _vp]),
    "pto_b200_tcmp_f32": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "pto_b200_gemm_f16f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pto_b200_mxgemm_workspace_bytes": (_i64, [_i, _i, _i]),
    "pto_b200_mxgemm_fp8": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _i64, _vp]),
    "pto_b200_ttri": (_i, [_vp, _i, _i, _i, _i, _i, _vp]),
    "pto_b200_mxgemm_fp4": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i64, _vp]),
    "pto_b200_gemm_bf16f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pto_b200_gemm_f16_out16": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "pto_b200_gemm_i8i32": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "pto_b200_gemm_f16f32_bias": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pto_b200_gemm_f16f32_batched": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i64, _i64, _i64, _vp]),
    "pto_b200_gemm_f16f32_host": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "pto_b200_gemm_f16f32_host_batched": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i64, _i64, _i64]),
    "pto_b200_gemm_f16f32_host_static": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "pto_b200_flash_attn_fwd_f16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp]),
    "pto_b200_flash_attn_fwd_f16_ex": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp]),
    "pto_b200_flash_attn_fwd_f16_host": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i]),
    "pto_b200_gemm_call_kernel": (None, [_u32, _vp, _vp, _vp, _vp]),
    "pto_b200_fa_call_kernel": (None, [_vp, _i, _i, _i, ctypes.c_bool] + [_vp] * 11),
}

_lib = None


def lib():
    """The loaded library.  Raises PtoB200Error when it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise PtoB200Error(f"{path} is missing: build it with `python -m pto_isa_b200.build` "
                               "(the CUDA kernels are the only implementation; there is no fallback)")
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the ABI and this table drift apart
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().pto_b200_last_error().decode("utf-8", "replace")
        raise PtoB200Error(f"{what} failed with status {rc}: {msg}")
