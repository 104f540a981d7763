"""The PTO operator names of the hot path over torch CUDA tensors (host side of the C ABI).

Names and argument meaning follow the reference's instruction surface (include/pto/common/pto_instr.hpp,
paths relative to the reference root): TCVT :864, TGATHER :800/:824, TROWMAX :990, TROWSUM :942, TEXP :1129,
TROWEXPAND :1049 and TROWEXPANDSUB/MUL/DIV/ADD/MAX/MIN/EXPDIF :1057-1108, TROWMIN :1007, TCOLSUM/TCOLMAX/TCOLMIN
:959-988/:1305, TFILLPAD :754, TTRANS :1032, TSEL :1024, TCMPS :143, TCMP :151, TADD/TSUB/TMUL/TDIV/TMAX/TMIN :56-120
and :238, TMULS :1188, TADDS :1161; `gemm` stands for
LaunchGEMME2E (kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:243) and `flash_attn_fwd` for
LaunchTFA (kernels/manual/common/flash_atten/fa_performance_kernel.cpp:970).  A whole tensor plays the role of
the tile: destination first is replaced by a returned (or `out=`) tensor.  Everything runs on the current
CUDA stream of the tensors' device; nothing is computed by torch.
"""
import ctypes

import torch

from ._lib import PtoB200Error, check, lib

CAST_RINT, CAST_ROUND, CAST_FLOOR, CAST_CEIL, CAST_TRUNC, CAST_ODD = 1, 2, 3, 4, 5, 6
P0101, P1010, P0001, P0010, P0100, P1000, P1111 = 1, 2, 3, 4, 5, 6, 7
OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_MAX, OP_MIN, OP_EXPDIF, OP_EXPAND = 0, 1, 2, 3, 4, 5, 6, 7
CMP_EQ, CMP_NE, CMP_LT, CMP_LE, CMP_GT, CMP_GE = 0, 1, 2, 3, 4, 5
PAD_ZERO, PAD_MAX, PAD_MIN = 1, 2, 3  # PadValue::Zero / Max / Min (include/pto/common/type.hpp:204-210)


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _need_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise PtoB200Error("operands must be CUDA tensors (there is no CPU path)")
        if not t.is_contiguous():
            raise PtoB200Error("operands must be contiguous")


def _out(out, shape, dtype, device, what):
    """A fresh result tensor, or the caller's `out=` once it is known to be exactly what the kernel will write:
    the C ABI takes raw pointers, so a wrong shape, type or device here would be an out-of-bounds device write."""
    shape = tuple(int(x) for x in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
    if out is None:
        return torch.empty(shape, dtype=dtype, device=device)
    if not isinstance(out, torch.Tensor):
        raise PtoB200Error(f"{what}: out= must be a tensor")
    if tuple(out.shape) != shape or out.dtype != dtype:
        raise PtoB200Error(f"{what}: out= must have shape {shape} and dtype {dtype}, got {tuple(out.shape)} {out.dtype}")
    want = torch.device(device)
    if not out.is_cuda or (want.index is not None and out.device != want):
        raise PtoB200Error(f"{what}: out= must be a CUDA tensor on {want}")
    if not out.is_contiguous():
        raise PtoB200Error(f"{what}: out= must be contiguous")
    return out


def _same_device(what, *ts):
    for t in ts[1:]:
        if t.device != ts[0].device:
            raise PtoB200Error(f"{what}: operands must be on the same device")


def TCVT(src, dtype, round_mode=CAST_RINT, out=None):
    """Elementwise cast of an fp32 tensor to torch.float16, torch.bfloat16 or torch.int32."""
    _need_cuda(src)
    if src.dtype != torch.float32:
        raise PtoB200Error("TCVT: source must be float32")
    out = _out(out, src.shape, dtype, src.device, "TCVT")
    _need_cuda(out)
    with torch.cuda.device(src.device):
        if dtype == torch.float16:
            rc = lib().pto_b200_tcvt_f32_f16(_ptr(src), _ptr(out), src.numel(), _stream(src))
        elif dtype == torch.bfloat16:
            rc = lib().pto_b200_tcvt_f32_bf16(_ptr(src), _ptr(out), src.numel(), _stream(src))
        elif dtype == torch.int32:
            rc = lib().pto_b200_tcvt_f32_i32(_ptr(src), _ptr(out), src.numel(), int(round_mode), _stream(src))
        else:
            raise PtoB200Error(f"TCVT: unsupported destination type {dtype}")
    check(rc, "TCVT")
    return out


def TGATHER(src0, idx, out=None):
    """out[i] = src0.flatten()[idx[i]]; an index outside [0, src0.numel()) gives 0.  4- or 2-byte elements."""
    _need_cuda(src0, idx)
    _same_device("TGATHER", src0, idx)
    if idx.dtype != torch.int32:
        raise PtoB200Error("TGATHER: indices must be int32")
    if src0.element_size() not in (2, 4):
        raise PtoB200Error("TGATHER: 16- or 32-bit elements only")
    out = _out(out, idx.shape, src0.dtype, src0.device, "TGATHER")
    with torch.cuda.device(src0.device):
        rc = lib().pto_b200_tgather(_ptr(src0), src0.numel(), _ptr(idx), _ptr(out), idx.numel(), src0.element_size(),
                                    _stream(src0))
    check(rc, "TGATHER")
    return out


def TGATHER_MASK(src, pattern, out=None):
    """Keeps the columns of a 2-D tensor that `pattern` selects, packed contiguously (1-D result)."""
    _need_cuda(src)
    if src.dim() != 2:
        raise PtoB200Error("TGATHER_MASK: expects a 2-D tensor")
    rows, cols = src.shape
    div, off = {1: (2, 0), 2: (2, 1), 3: (4, 0), 4: (4, 1), 5: (4, 2), 6: (4, 3), 7: (1, 0)}[int(pattern)]
    out_cols = (cols - off + div - 1) // div
    out = _out(out, rows * out_cols, src.dtype, src.device, "TGATHER_MASK")
    with torch.cuda.device(src.device):
        rc = lib().pto_b200_tgather_mask(_ptr(src), _ptr(out), rows, cols, int(pattern), src.element_size(),
                                         _stream(src))
    check(rc, "TGATHER_MASK")
    return out


def _row_reduce(fn_name, src, out):
    _need_cuda(src)
    if src.dim() != 2 or src.dtype != torch.float32:
        raise PtoB200Error(f"{fn_name}: expects a 2-D float32 tensor")
    rows, cols = src.shape
    out = _out(out, rows, torch.float32, src.device, "_row_reduce")
    with torch.cuda.device(src.device):
        rc = getattr(lib(), fn_name)(_ptr(src), _ptr(out), rows, cols, cols, _stream(src))
    check(rc, fn_name)
    return out


def TROWMAX(src, out=None):
    return _row_reduce("pto_b200_trowmax_f32", src, out)


def TROWSUM(src, out=None):
    return _row_reduce("pto_b200_trowsum_f32", src, out)


def TEXP(src, out=None):
    _need_cuda(src)
    if src.dtype != torch.float32:
        raise PtoB200Error("TEXP: source must be float32")
    out = _out(out, src.shape, src.dtype, src.device, "TEXP")
    with torch.cuda.device(src.device):
        rc = lib().pto_b200_texp_f32(_ptr(src), _ptr(out), src.numel(), _stream(src))
    check(rc, "TEXP")
    return out


def _binary(a, b, op, out):
    _need_cuda(a, b)
    if a.shape != b.shape or a.dtype != torch.float32 or b.dtype != torch.float32:
        raise PtoB200Error("binary tile op: operands must be float32 of the same shape")
    out = _out(out, a.shape, a.dtype, a.device, "_binary")
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_tbinary_f32(_ptr(a), _ptr(b), _ptr(out), a.numel(), op, _stream(a))
    check(rc, "binary tile op")
    return out


def TADD(a, b, out=None):
    return _binary(a, b, OP_ADD, out)


def TSUB(a, b, out=None):
    return _binary(a, b, OP_SUB, out)


def TMAX(a, b, out=None):
    return _binary(a, b, OP_MAX, out)


def TMUL(a, b, out=None):
    return _binary(a, b, OP_MUL, out)


def TDIV(a, b, out=None):
    return _binary(a, b, OP_DIV, out)


def TMIN(a, b, out=None):
    return _binary(a, b, OP_MIN, out)


def _scalar(a, s, op, out):
    _need_cuda(a)
    out = _out(out, a.shape, a.dtype, a.device, "_scalar")
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_tscalar_f32(_ptr(a), float(s), _ptr(out), a.numel(), op, _stream(a))
    check(rc, "scalar tile op")
    return out


def TMULS(a, s, out=None):
    return _scalar(a, s, OP_MUL, out)


def TADDS(a, s, out=None):
    return _scalar(a, s, OP_ADD, out)


def _rowexpand(a, row_scalar, op, out):
    _need_cuda(a, row_scalar)
    if a.dim() != 2 or row_scalar.numel() != a.shape[0]:
        raise PtoB200Error("row-expand tile op: expects a 2-D tile and one scalar per row")
    out = _out(out, a.shape, a.dtype, a.device, "_rowexpand")
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_trowexpand_f32(_ptr(a), _ptr(row_scalar), _ptr(out), a.shape[0], a.shape[1], op,
                                           _stream(a))
    check(rc, "row-expand tile op")
    return out


def TROWEXPANDSUB(a, row_scalar, out=None):
    return _rowexpand(a, row_scalar, OP_SUB, out)


def TROWEXPANDMUL(a, row_scalar, out=None):
    return _rowexpand(a, row_scalar, OP_MUL, out)


def TROWEXPANDDIV(a, row_scalar, out=None):
    return _rowexpand(a, row_scalar, OP_DIV, out)


def TROWEXPANDADD(a, row_scalar, out=None):
    return _rowexpand(a, row_scalar, OP_ADD, out)


def TROWEXPANDMAX(a, row_scalar, out=None):
    return _rowexpand(a, row_scalar, OP_MAX, out)


def TROWEXPANDMIN(a, row_scalar, out=None):
    return _rowexpand(a, row_scalar, OP_MIN, out)


def TROWEXPANDEXPDIF(a, row_scalar, out=None):
    return _rowexpand(a, row_scalar, OP_EXPDIF, out)


def TROWEXPAND(row_scalar, cols, out=None):
    """dst[r, c] = row_scalar[r] for `cols` columns."""
    _need_cuda(row_scalar)
    if row_scalar.dtype != torch.float32:
        raise PtoB200Error("TROWEXPAND: expects float32")
    rows = row_scalar.numel()
    out = _out(out, (rows, cols), torch.float32, row_scalar.device, "TROWEXPAND")
    with torch.cuda.device(row_scalar.device):
        rc = lib().pto_b200_trowexpand_f32(None, _ptr(row_scalar), _ptr(out), rows, cols, OP_EXPAND, _stream(row_scalar))
    check(rc, "TROWEXPAND")
    return out


def TROWMIN(src, out=None):
    return _row_reduce("pto_b200_trowmin_f32", src, out)


def _col_reduce(src, op, out, what, workspace=None):
    _need_cuda(src)
    if src.dim() != 2 or src.dtype != torch.float32:
        raise PtoB200Error(f"{what}: expects a 2-D float32 tensor")
    rows, cols = src.shape
    out = _out(out, cols, torch.float32, src.device, "_col_reduce")
    ws_bytes = lib().pto_b200_tcolreduce_workspace_bytes(rows, cols) if workspace is None else workspace.numel() * workspace.element_size()
    if workspace is None and ws_bytes > 0:
        workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=src.device)  # torch's caching allocator
    with torch.cuda.device(src.device):
        rc = lib().pto_b200_tcolreduce_f32(_ptr(src), _ptr(out), rows, cols, cols, op,
                                           _ptr(workspace) if workspace is not None else None, ws_bytes, _stream(src))
    check(rc, what)
    return out


def TCOLSUM(src, out=None, workspace=None):
    return _col_reduce(src, OP_ADD, out, "TCOLSUM", workspace)


def TCOLMAX(src, out=None, workspace=None):
    return _col_reduce(src, OP_MAX, out, "TCOLMAX", workspace)


def TCOLMIN(src, out=None, workspace=None):
    return _col_reduce(src, OP_MIN, out, "TCOLMIN", workspace)


def _pad_bits(dtype, pad):
    """The bit pattern PadValue::Zero / Max / Min mean for `dtype` (include/pto/cpu/TFillPad.hpp:24-36): infinities
    for floating types, the type's max / min for integers."""
    if pad == PAD_ZERO:
        return 0
    if dtype.is_floating_point:
        bits = {torch.float32: 0x7f800000, torch.float16: 0x7c00, torch.bfloat16: 0x7f80}[dtype]  # +infinity
        return bits | ((0x80000000 if dtype.itemsize == 4 else 0x8000) if pad == PAD_MIN else 0)
    info = torch.iinfo(dtype)
    return int(info.max if pad == PAD_MAX else info.min) & (0xffffffff if dtype.itemsize == 4 else 0xffff)


def TFILLPAD(src, valid_rows, valid_cols, pad=PAD_ZERO, out=None):
    """Copies the valid_rows x valid_cols corner of the 2-D tile `src` and fills the rest with the pad value."""
    _need_cuda(src)
    if src.dim() != 2 or src.dtype.itemsize not in (2, 4):
        raise PtoB200Error("TFILLPAD: expects a 2-D tensor of 2- or 4-byte elements")
    out = _out(out, src.shape, src.dtype, src.device, "TFILLPAD")
    with torch.cuda.device(src.device):
        rc = lib().pto_b200_tfillpad(_ptr(src), _ptr(out), src.shape[0], src.shape[1], int(valid_rows), int(valid_cols),
                                     _pad_bits(src.dtype, pad), src.dtype.itemsize, _stream(src))
    check(rc, "TFILLPAD")
    return out


def TTRANS(src, out=None):
    _need_cuda(src)
    if src.dim() != 2 or src.dtype.itemsize not in (2, 4):
        raise PtoB200Error("TTRANS: expects a 2-D tensor of 2- or 4-byte elements")
    out = _out(out, (src.shape[1], src.shape[0]), src.dtype, src.device, "TTRANS")
    with torch.cuda.device(src.device):
        rc = lib().pto_b200_ttrans(_ptr(src), _ptr(out), src.shape[0], src.shape[1], src.dtype.itemsize, _stream(src))
    check(rc, "TTRANS")
    return out


def TSEL(mask, src0, src1, out=None):
    """mask: uint8 tensor, one bit per element of the operands in row-major order, least significant bit first."""
    _need_cuda(mask, src0, src1)
    if src0.shape != src1.shape or src0.dtype != src1.dtype or src0.dtype.itemsize not in (2, 4):
        raise PtoB200Error("TSEL: operands must have the same shape and a 2- or 4-byte element type")
    if mask.dtype != torch.uint8 or mask.numel() * 8 < src0.numel():
        raise PtoB200Error("TSEL: the mask must be uint8 with one bit per element")
    out = _out(out, src0.shape, src0.dtype, src0.device, "TSEL")
    with torch.cuda.device(src0.device):
        rc = lib().pto_b200_tsel(_ptr(mask), _ptr(src0), _ptr(src1), _ptr(out), src0.numel(), src0.dtype.itemsize,
                                 _stream(src0))
    check(rc, "TSEL")
    return out


def TCMPS(src, scalar, mode, out=None):
    """Packed comparison bits of `src` against a scalar: numel / 8 bytes, least significant bit first."""
    _need_cuda(src)
    if src.dtype != torch.float32 or src.numel() % 8 != 0:
        raise PtoB200Error("TCMPS: expects float32 with a multiple of 8 elements")
    out = _out(out, src.numel() // 8, torch.uint8, src.device, "TCMPS")
    with torch.cuda.device(src.device):
        rc = lib().pto_b200_tcmps_f32(_ptr(src), float(scalar), _ptr(out), src.numel(), int(mode), _stream(src))
    check(rc, "TCMPS")
    return out


def TCMP(a, b, mode, out=None):
    """1.0 / 0.0 per element, the form the reference's CPU simulation gives TCMP."""
    _need_cuda(a, b)
    if a.shape != b.shape or a.dtype != torch.float32 or b.dtype != torch.float32:
        raise PtoB200Error("TCMP: operands must be float32 of the same shape")
    out = _out(out, a.shape, a.dtype, a.device, "TCMP")
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_tcmp_f32(_ptr(a), _ptr(b), _ptr(out), a.numel(), int(mode), _stream(a))
    check(rc, "TCMP")
    return out


_TRI_DTYPES = {torch.float32: 0, torch.int32: 1, torch.float16: 2, torch.int16: 3}


def TTRI(rows, cols, diagonal=0, upper=False, dtype=torch.float32, device="cuda", out=None):
    """rows x cols tile of ones inside the lower (c <= r + diagonal) or upper (c >= r + diagonal) triangle, zeros outside."""
    if dtype not in _TRI_DTYPES:
        raise PtoB200Error("TTRI: float32, int32, float16 or int16")
    out = _out(out, (rows, cols), dtype, device, "TTRI")
    _need_cuda(out)
    with torch.cuda.device(out.device):
        rc = lib().pto_b200_ttri(_ptr(out), int(rows), int(cols), int(diagonal), 1 if upper else 0, _TRI_DTYPES[dtype],
                                 _stream(out))
    check(rc, "TTRI")
    return out


def TRESHAPE(src, rows, cols):
    """The same bytes under another 2-D shape (include/pto/cpu/TReshape.hpp:18-56): a view, no kernel."""
    _need_cuda(src)
    if src.numel() != rows * cols:
        raise PtoB200Error("TRESHAPE: the total size must match")
    return src.view(rows, cols)


FP8_E4M3, FP8_E5M2 = 0, 1
_mx_workspaces = {}


def _fp8_format(t, fmt):
    if t.dtype == torch.float8_e5m2:
        return FP8_E5M2
    if t.dtype == torch.float8_e4m3fn:
        return FP8_E4M3
    if t.dtype == torch.uint8 and fmt in (FP8_E4M3, FP8_E5M2):
        return fmt
    raise PtoB200Error("mx_gemm: operands must be float8_e5m2 / float8_e4m3fn, or uint8 with fmt=FP8_E4M3 / FP8_E5M2")


def mx_gemm(a, b, scale_a, scale_b, out_dtype=torch.bfloat16, out=None, fmt=FP8_E5M2, workspace=None):
    """C[m,n] = (scale_a (x) A[m,k]) @ (scale_b (x) B[n,k])^T, the reference's MxMatmul
    (kernels/manual/a5/matmul_mxfp8_performance): fp8 operands, one float8_e8m0 scale (uint8 bytes, 2^(byte - 127)) per
    32 consecutive k of a row: scale_a (m, k/32), scale_b (n, k/32).  Output bfloat16 (the reference's) or float32."""
    _need_cuda(a, b, scale_a, scale_b)
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise PtoB200Error("mx_gemm: a is (m, k) and b is (n, k)")
    (m, k), n = a.shape, b.shape[0]
    if k % 32 != 0 or tuple(scale_a.shape) != (m, k // 32) or tuple(scale_b.shape) != (n, k // 32):
        raise PtoB200Error("mx_gemm: k must be a multiple of 32 and the scales (m, k/32) and (n, k/32)")
    if scale_a.dtype.itemsize != 1 or scale_b.dtype.itemsize != 1:
        raise PtoB200Error("mx_gemm: scales are one byte each (float8_e8m0)")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise PtoB200Error("mx_gemm: the output is bfloat16 or float32")
    fa, fb = _fp8_format(a, fmt), _fp8_format(b, fmt)
    out = _out(out, (m, n), out_dtype, a.device, "mx_gemm")
    _need_cuda(out)
    need = lib().pto_b200_mxgemm_workspace_bytes(m, n, k)
    if workspace is None:
        key = (a.device.index, torch.cuda.current_stream(a.device).cuda_stream)
        workspace = _mx_workspaces.get(key)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
            _mx_workspaces[key] = workspace
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_mxgemm_fp8(_ptr(a), _ptr(b), _ptr(scale_a), _ptr(scale_b), _ptr(out), m, n, k, fa, fb,
                                       1 if out_dtype == torch.float32 else 0, _ptr(workspace), workspace.numel(),
                                       _stream(a))
    check(rc, "mx_gemm")
    return out


def mx_gemm_fp4(a, b, scale_a, scale_b, out_dtype=torch.bfloat16, out=None, workspace=None):
    """C[m,n] = (scale_a (x) A[m,k]) @ (scale_b (x) B[n,k])^T with packed float4_e2m1 operands: a is (m, k/2) and b is
    (n, k/2) uint8, two values per byte, the lower k index in the low nibble (the reference's MXFP4 MxMatmul,
    kernels/manual/a5/matmul_mxfp4_performance); scales as for mx_gemm."""
    _need_cuda(a, b, scale_a, scale_b)
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1] or a.dtype.itemsize != 1 or b.dtype.itemsize != 1:
        raise PtoB200Error("mx_gemm_fp4: a is (m, k/2) and b is (n, k/2) bytes")
    m, n, k = a.shape[0], b.shape[0], 2 * a.shape[1]
    if k % 32 != 0 or tuple(scale_a.shape) != (m, k // 32) or tuple(scale_b.shape) != (n, k // 32):
        raise PtoB200Error("mx_gemm_fp4: k must be a multiple of 32 and the scales (m, k/32) and (n, k/32)")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise PtoB200Error("mx_gemm_fp4: the output is bfloat16 or float32")
    out = _out(out, (m, n), out_dtype, a.device, "mx_gemm_fp4")
    _need_cuda(out)
    need = lib().pto_b200_mxgemm_workspace_bytes(m, n, k)
    if workspace is None:
        key = (a.device.index, torch.cuda.current_stream(a.device).cuda_stream)
        workspace = _mx_workspaces.get(key)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
            _mx_workspaces[key] = workspace
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_mxgemm_fp4(_ptr(a), _ptr(b), _ptr(scale_a), _ptr(scale_b), _ptr(out), m, n, k,
                                       1 if out_dtype == torch.float32 else 0, _ptr(workspace), workspace.numel(),
                                       _stream(a))
    check(rc, "mx_gemm_fp4")
    return out


def gemm(a, b, b_layout=1, out=None, bias=None):
    """C[m,n] fp32 = A[m,k] fp16 @ B.  b_layout 0: b is (k, n); 1: b is (n, k), the reference kernel's layout.
    A 3-D `a` (batch, m, k) with 3-D `b` runs `batch` independent problems.  `bias` (n floats, 2-D problems only) is
    added to every row: TMATMUL_BIAS."""
    _need_cuda(a, b)
    if a.dtype != torch.float16 or b.dtype != torch.float16:
        raise PtoB200Error("gemm: operands must be float16")
    _same_device("gemm", a, b)
    batched = a.dim() == 3
    if a.dim() not in (2, 3) or b.dim() != a.dim() or (batched and a.shape[0] != b.shape[0]):
        raise PtoB200Error("gemm: a and b are both 2-D, or both 3-D with the same batch")
    if b_layout not in (0, 1):
        raise PtoB200Error("gemm: b_layout is 0 (b is k x n) or 1 (b is n x k)")
    if a.shape[-1] != (b.shape[-2] if b_layout == 0 else b.shape[-1]):
        raise PtoB200Error(f"gemm: the k extents of a {tuple(a.shape)} and b {tuple(b.shape)} differ (b_layout {b_layout})")
    if bias is not None:
        _need_cuda(bias)
        _same_device("gemm", a, bias)
        n_ = b.shape[-1] if b_layout == 0 else b.shape[-2]
        if batched or bias.dtype != torch.float32 or bias.numel() != n_:
            raise PtoB200Error("gemm: bias is n float32 values, for a single problem")
        out = _out(out, (a.shape[0], n_), torch.float32, a.device, "gemm")
        with torch.cuda.device(a.device):
            rc = lib().pto_b200_gemm_f16f32_bias(_ptr(a), _ptr(b), _ptr(bias), _ptr(out), a.shape[0], n_, a.shape[1],
                                                 int(b_layout), _stream(a))
        check(rc, "gemm (bias)")
        return out
    m, k = a.shape[-2:]
    n = b.shape[-1] if b_layout == 0 else b.shape[-2]
    shape = (a.shape[0], m, n) if batched else (m, n)
    out = _out(out, shape, torch.float32, a.device, "gemm")
    with torch.cuda.device(a.device):
        if batched:
            rc = lib().pto_b200_gemm_f16f32_batched(_ptr(a), _ptr(b), _ptr(out), m, n, k, int(b_layout), a.shape[0],
                                                    m * k, n * k, m * n, _stream(a))
        else:
            rc = lib().pto_b200_gemm_f16f32(_ptr(a), _ptr(b), _ptr(out), m, n, k, int(b_layout), _stream(a))
    check(rc, "gemm")
    return out


def gemm_bf16(a, b, b_layout=1, out=None):
    """C[m,n] fp32 = A[m,k] bfloat16 @ B (layouts as gemm)."""
    _need_cuda(a, b)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.dim() != 2 or b.dim() != 2:
        raise PtoB200Error("gemm_bf16: operands are 2-D bfloat16")
    _same_device("gemm_bf16", a, b)
    if b_layout not in (0, 1) or a.shape[1] != (b.shape[0] if b_layout == 0 else b.shape[1]):
        raise PtoB200Error(f"gemm_bf16: the k extents of a {tuple(a.shape)} and b {tuple(b.shape)} differ (b_layout {b_layout})")
    m, k = a.shape
    n = b.shape[1] if b_layout == 0 else b.shape[0]
    out = _out(out, (m, n), torch.float32, a.device, "gemm_bf16")
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_gemm_bf16f32(_ptr(a), _ptr(b), _ptr(out), m, n, k, int(b_layout), _stream(a))
    check(rc, "gemm_bf16")
    return out


def gemm_out16(a, b, b_layout=1, out_dtype=torch.float16, out=None):
    """The fp16 product with C rounded to float16 or bfloat16 on the way out of the accumulator (TSTORE's conversion)."""
    _need_cuda(a, b)
    if a.dtype != torch.float16 or b.dtype != torch.float16 or a.dim() != 2 or b.dim() != 2:
        raise PtoB200Error("gemm_out16: operands are 2-D float16")
    _same_device("gemm_out16", a, b)
    if b_layout not in (0, 1) or a.shape[1] != (b.shape[0] if b_layout == 0 else b.shape[1]):
        raise PtoB200Error(f"gemm_out16: the k extents of a {tuple(a.shape)} and b {tuple(b.shape)} differ (b_layout {b_layout})")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise PtoB200Error("gemm_out16: the output is float16 or bfloat16")
    m, k = a.shape
    n = b.shape[1] if b_layout == 0 else b.shape[0]
    out = _out(out, (m, n), out_dtype, a.device, "gemm_out16")
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_gemm_f16_out16(_ptr(a), _ptr(b), _ptr(out), m, n, k, int(b_layout),
                                           2 if out_dtype == torch.float16 else 4, _stream(a))
    check(rc, "gemm_out16")
    return out


def gemm_i8(a, b, out=None):
    """C[m,n] int32 = A[m,k] int8 @ B[n,k]^T int8, exact (TMATMUL's int8 form).  k a multiple of 16."""
    _need_cuda(a, b)
    if a.dtype != torch.int8 or b.dtype != torch.int8 or a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise PtoB200Error("gemm_i8: a is (m, k) and b is (n, k), both int8")
    _same_device("gemm_i8", a, b)
    m, k = a.shape
    n = b.shape[0]
    out = _out(out, (m, n), torch.int32, a.device, "gemm_i8")
    with torch.cuda.device(a.device):
        rc = lib().pto_b200_gemm_i8i32(_ptr(a), _ptr(b), _ptr(out), m, n, k, _stream(a))
    check(rc, "gemm_i8")
    return out


def gemm_host(a, b, c, b_layout=1):
    """Same product over HOST tensors (pinned or pageable): copies in, computes, copies out, synchronises."""
    if any(t.is_cuda or not t.is_contiguous() for t in (a, b, c)) or a.dim() != 2 or b.dim() != 2:
        raise PtoB200Error("gemm_host: expects contiguous 2-D host tensors")
    if a.dtype != torch.float16 or b.dtype != torch.float16 or c.dtype != torch.float32 or b_layout not in (0, 1):
        raise PtoB200Error("gemm_host: a and b are float16, c is float32, b_layout is 0 or 1")
    if a.shape[1] != (b.shape[0] if b_layout == 0 else b.shape[1]):
        raise PtoB200Error("gemm_host: the k extents of a and b differ")
    if tuple(c.shape) != (a.shape[0], b.shape[1] if b_layout == 0 else b.shape[0]):
        raise PtoB200Error("gemm_host: c must be (m, n)")
    m, k = a.shape
    n = b.shape[1] if b_layout == 0 else b.shape[0]
    rc = lib().pto_b200_gemm_f16f32_host(_ptr(a), _ptr(b), _ptr(c), m, n, k, int(b_layout))
    check(rc, "gemm_host")
    return c


def gemm_host_batched(a, b, c, b_layout=1):
    """`batch` products over HOST tensors a (batch, m, k), b (batch, n, k) or (batch, k, n), c (batch, m, n): copies in,
    kernels and copies out of consecutive problems overlap (pin the tensors for that)."""
    if a.dim() != 3 or b.dim() != 3 or c.dim() != 3 or a.is_cuda or b.is_cuda or c.is_cuda:
        raise PtoB200Error("gemm_host_batched: expects 3-D host tensors")
    if not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
        raise PtoB200Error("gemm_host_batched: operands must be contiguous")
    if a.dtype != torch.float16 or b.dtype != torch.float16 or c.dtype != torch.float32 or b_layout not in (0, 1):
        raise PtoB200Error("gemm_host_batched: a and b are float16, c is float32, b_layout is 0 or 1")
    batch, m, k = a.shape
    n = b.shape[2] if b_layout == 0 else b.shape[1]
    if b.shape[0] != batch or k != (b.shape[1] if b_layout == 0 else b.shape[2]) or tuple(c.shape) != (batch, m, n):
        raise PtoB200Error("gemm_host_batched: a (batch, m, k), b (batch, n, k) or (batch, k, n) and c (batch, m, n) disagree")
    rc = lib().pto_b200_gemm_f16f32_host_batched(_ptr(a), _ptr(b), _ptr(c), m, n, k, int(b_layout), batch, m * k, n * k, m * n)
    check(rc, "gemm_host_batched")
    return c


def flash_attn_fwd(q, k, v, causal=False, scale=None, out_dtype=torch.float16, out=None, defer_rescale=None):
    """q: (..., sq, d), k / v: (..., sk, d) fp16 with the same leading (batch, heads) dims.  Returns O like q.
    defer_rescale: False = the reference's recurrence (the row maximum moves at every key tile where it grows), True =
    it moves only after growing 256-fold (fewer rescales of O); None = False for float32 output, True for float16."""
    _need_cuda(q, k, v)
    if q.dtype != torch.float16 or k.dtype != torch.float16 or v.dtype != torch.float16:
        raise PtoB200Error("flash_attn_fwd: operands must be float16")
    _same_device("flash_attn_fwd", q, k, v)
    if out_dtype not in (torch.float16, torch.float32):
        raise PtoB200Error("flash_attn_fwd: the output is float16 or float32")
    if q.dim() < 2 or k.shape != v.shape or k.dim() != q.dim() or k.shape[:-2] != q.shape[:-2] or k.shape[-1] != q.shape[-1]:
        raise PtoB200Error(f"flash_attn_fwd: q {tuple(q.shape)}, k {tuple(k.shape)} and v {tuple(v.shape)} must share "
                           "their leading (batch, heads) extents and the head size, and k and v their shape")
    sq, d = q.shape[-2:]
    sk = k.shape[-2]
    bh = q.numel() // (sq * d)
    scale = (1.0 / d ** 0.5) if scale is None else float(scale)
    out = _out(out, q.shape, out_dtype, q.device, "flash_attn_fwd")
    with torch.cuda.device(q.device):
        if defer_rescale is None:
            rc = lib().pto_b200_flash_attn_fwd_f16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), bh, sq, sk, d, int(bool(causal)),
                                                   scale, 1 if out_dtype == torch.float16 else 0, _stream(q))
        else:
            rc = lib().pto_b200_flash_attn_fwd_f16_ex(_ptr(q), _ptr(k), _ptr(v), _ptr(out), bh, sq, sk, d,
                                                      int(bool(causal)), scale, 1 if out_dtype == torch.float16 else 0,
                                                      int(bool(defer_rescale)), _stream(q))
    check(rc, "flash_attn_fwd")
    return out


def flash_attn_fwd_host(q, k, v, o, causal=False, scale=None):
    """The same over HOST tensors: copies in, computes, copies out, synchronises.  o is float16 or float32, shaped like q."""
    if any(t.is_cuda or not t.is_contiguous() for t in (q, k, v, o)):
        raise PtoB200Error("flash_attn_fwd_host: expects contiguous host tensors")
    if q.dtype != torch.float16 or k.dtype != torch.float16 or v.dtype != torch.float16 or \
            o.dtype not in (torch.float16, torch.float32):
        raise PtoB200Error("flash_attn_fwd_host: q, k, v are float16, o is float16 or float32")
    if k.shape != v.shape or k.shape[:-2] != q.shape[:-2] or k.shape[-1] != q.shape[-1] or o.shape != q.shape:
        raise PtoB200Error("flash_attn_fwd_host: shapes of q, k, v and o disagree")
    sq, d = q.shape[-2:]
    sk = k.shape[-2]
    bh = q.numel() // (sq * d)
    scale = (1.0 / d ** 0.5) if scale is None else float(scale)
    rc = lib().pto_b200_flash_attn_fwd_f16_host(_ptr(q), _ptr(k), _ptr(v), _ptr(o), bh, sq, sk, d,
                                                int(bool(causal)), scale, 1 if o.dtype == torch.float16 else 0)
    check(rc, "flash_attn_fwd_host")
    return o


def device_status(device=None):
    """Reads and clears the device-side status record (synchronises the current stream)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        return lib().pto_b200_device_status(ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))


def device_status_record(device=None):
    """Reads and clears the status record; returns (code, block, where, detail)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    rec = (ctypes.c_int * 4)()
    with torch.cuda.device(dev):
        lib().pto_b200_device_status_ex(ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream), rec)
    return tuple(rec)


def set_profile_buffer(stamps):
    """Per-block profile stamps: `stamps` is a CUDA int64 tensor of shape (blocks, 4) that the GEMM and attention
    kernels fill with {timer ns at block start, at block end, SM cycle counter at start, at end}; None switches them off."""
    if stamps is None:
        check(lib().pto_b200_set_profile_buffer(None, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
              "set_profile_buffer")
        return
    _need_cuda(stamps)
    if stamps.dtype != torch.int64 or stamps.dim() != 2 or stamps.shape[1] != 4:
        raise PtoB200Error("set_profile_buffer: expects an int64 tensor of shape (blocks, 4)")
    with torch.cuda.device(stamps.device):
        check(lib().pto_b200_set_profile_buffer(_ptr(stamps), stamps.shape[0], _stream(stamps)), "set_profile_buffer")


def probe_random_reads(table, reads, table_bytes=None):
    """Launches `reads` random 4-byte reads over the first `table_bytes` of `table` (measurement helper for TGATHER)."""
    _need_cuda(table)
    table_bytes = table.numel() * table.element_size() if table_bytes is None else int(table_bytes)
    if table_bytes > table.numel() * table.element_size():
        raise PtoB200Error("probe_random_reads: table_bytes exceeds the tensor")
    sink = torch.zeros(1, dtype=torch.int32, device=table.device)
    with torch.cuda.device(table.device):
        check(lib().pto_b200_probe_random_reads(_ptr(table), table_bytes, int(reads), _ptr(sink), _stream(table)),
              "probe_random_reads")
    return sink
