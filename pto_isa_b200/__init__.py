"""pto_isa_b200 - host side of the B200 (sm_100a) backend for the PTO tile-ISA hot path.

The product is libpto_b200.so (hand-written CUDA behind the C ABI of include/pto_b200.h).  This package
is the thin Python host layer over that ABI, in the role the reference's ctypes loaders play
(demos/torch_jit/gemm/jit_util_gemm.py, demos/torch_jit/flash_atten/jit_util_flash.py): it passes
torch CUDA tensors' device pointers and the current stream.  There is no CPU or PyTorch fallback:
if the library is missing or a call fails, an exception is raised.
"""
from ._lib import PtoB200Error, lib, lib_path  # noqa: F401
from . import ops  # noqa: F401
from .ops import (  # noqa: F401
    TCVT, TGATHER, TGATHER_MASK, TROWMAX, TROWSUM, TEXP, TROWEXPANDSUB, TROWEXPANDMUL, TROWEXPANDDIV,
    TROWEXPAND, TROWEXPANDADD, TROWEXPANDMAX, TROWEXPANDMIN, TROWEXPANDEXPDIF, TROWMIN, TCOLSUM, TCOLMAX, TCOLMIN,
    TFILLPAD, TTRANS, TTRI, TRESHAPE, TSEL, TCMPS, TCMP, TADD, TSUB, TMUL, TDIV, TMAX, TMIN, TMULS, TADDS, gemm, gemm_i8, gemm_out16, gemm_bf16, gemm_host, gemm_host_batched, mx_gemm, mx_gemm_fp4, flash_attn_fwd, flash_attn_fwd_host, device_status,
    device_status_record, set_profile_buffer, probe_random_reads,
)
