"""ctypes front-end of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

`port` wraps liboracle.so (the C restatement, pto_oracle.c) and is always available; `ref` wraps
_ref/libpto_ref.so (tile programs compiled against the reference's own CPU-simulation headers) and
is None where that library was never built.  Nothing in the product package imports this module:
only the tests, the smoke check and the benchmark's CPU-baseline leg do.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_i64 = ctypes.c_int64


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def reference_root():
    """The reference tree: $PTO_REFERENCE_ROOT, else a directory named `reference` beside the repository."""
    return os.environ.get("PTO_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(force=False):
    """Compile liboracle.so (and _ref/libpto_ref.so when the reference tree is present)."""
    so = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(_HERE, "pto_oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    ref_so = os.path.join(_HERE, "_ref", "libpto_ref.so")
    ref_srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.startswith("ref_") and f.endswith(".cpp")]
    stale = os.path.exists(ref_so) and any(os.path.getmtime(f) > os.path.getmtime(ref_so) for f in ref_srcs)
    reference = reference_root()
    if os.path.isdir(os.path.join(reference, "include", "pto")) and (force or stale or not os.path.exists(ref_so)):
        subprocess.check_call(["make", "-C", _HERE, "ref", "REFERENCE=" + reference], stdout=subprocess.DEVNULL)


class _Lib:
    """Thin numpy wrapper; `prefix` is 'pto_oracle_' (restatement) or 'pto_ref_' (reference build)."""

    def __init__(self, path, prefix):
        self.lib = ctypes.CDLL(path)
        self.prefix = prefix
        self.path = path

    def _f(self, name):
        return getattr(self.lib, self.prefix + name)

    def has(self, name):
        return hasattr(self.lib, self.prefix + name)

    # -- vector ops
    def tcvt_f32_f16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self._f("tcvt_f32_f16")(_p(x), _p(out), _i64(x.size))
        return out.view(np.float16)

    def tcvt_f32_bf16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self._f("tcvt_f32_bf16")(_p(x), _p(out), _i64(x.size))
        return out  # raw bf16 bits

    def tcvt_f32_i32(self, x, mode=1):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.int32)
        self._f("tcvt_f32_i32")(_p(x), _p(out), _i64(x.size), int(mode))
        return out

    def texp_f32(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        self._f("texp_f32")(_p(x), _p(out), _i64(x.size))
        return out

    def tgather(self, src0, idx):
        src0 = np.ascontiguousarray(src0)
        idx = np.ascontiguousarray(idx, np.int32)
        assert src0.ndim == 2 and src0.itemsize in (2, 4)
        out = np.empty(idx.shape, src0.dtype)
        name = "tgather_f32" if src0.itemsize == 4 else "tgather_b16"
        rc = self._f(name)(_p(src0), src0.shape[0], src0.shape[1], _p(idx), _p(out), _i64(idx.size))
        if rc != 0:
            raise ValueError(f"{self.prefix}{name}: unsupported shape {src0.shape}")
        return out

    def tgather_mask(self, src, pattern):
        src = np.ascontiguousarray(src)
        div, off = {1: (2, 0), 2: (2, 1), 3: (4, 0), 4: (4, 1), 5: (4, 2), 6: (4, 3), 7: (1, 0)}[int(pattern)]
        out = np.empty(src.shape[0] * ((src.shape[1] - off + div - 1) // div), src.dtype)
        name = "tgather_mask_f32" if src.itemsize == 4 else "tgather_mask_b16"
        rc = self._f(name)(_p(src), _p(out), src.shape[0], src.shape[1], int(pattern))
        if rc != 0:
            raise ValueError(f"{self.prefix}{name}: unsupported shape {src.shape}")
        return out

    def trowmax_f32(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[0], np.float32)
        rc = self._f("trowmax_f32")(_p(x), _p(out), x.shape[0], x.shape[1])
        assert rc == 0
        return out

    def trowsum_f32(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[0], np.float32)
        rc = self._f("trowsum_f32")(_p(x), _p(out), x.shape[0], x.shape[1])
        assert rc == 0
        return out

    # -- second batch of vector ops (op codes as in include/pto_b200.h)
    def trowexpand_f32(self, a, s, op):
        """dst[r, c] = a[r, c] op s[r]; op 7 ignores `a` (plain TROWEXPAND, pass the wanted shape as zeros)."""
        a = np.ascontiguousarray(a, np.float32)
        s = np.ascontiguousarray(s, np.float32)
        out = np.empty_like(a)
        rc = self._f("trowexpand_f32")(_p(a), _p(s), _p(out), a.shape[0], a.shape[1], int(op))
        if rc != 0:
            raise ValueError("trowexpand: unsupported shape or operator")
        return out

    def trowmin_f32(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[0], np.float32)
        rc = self._f("trowmin_f32")(_p(x), _p(out), x.shape[0], x.shape[1])
        if rc != 0:
            raise ValueError("trowmin: unsupported shape")
        return out

    def tcolreduce_f32(self, x, op):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[1], np.float32)
        rc = self._f("tcolreduce_f32")(_p(x), _p(out), x.shape[0], x.shape[1], int(op))
        if rc != 0:
            raise ValueError("tcolreduce: unsupported shape or operator")
        return out

    def tfillpad_f32(self, src, valid_rows, valid_cols, pad_kind):
        """pad_kind 1 zero, 2 max (+inf), 3 min (-inf).  The reference build takes dense 64 x 256 tiles only."""
        src = np.ascontiguousarray(src, np.float32)
        out = np.empty_like(src)
        if self.prefix == "pto_ref_":
            assert src.shape == (64, 256)
            rc = self._f("tfillpad_f32")(_p(src), _p(out), int(valid_rows), int(valid_cols), int(pad_kind))
        else:
            pad = {1: 0, 2: 0x7f800000, 3: 0xff800000}[int(pad_kind)]
            rc = self._f("tfillpad_b32")(_p(src), _p(out), src.shape[0], src.shape[1], int(valid_rows),
                                         int(valid_cols), ctypes.c_uint32(pad))
        if rc != 0:
            raise ValueError("tfillpad: unsupported shape")
        return out

    def ttrans(self, src):
        src = np.ascontiguousarray(src)
        out = np.empty((src.shape[1], src.shape[0]), src.dtype)
        if self.prefix == "pto_ref_":
            assert src.shape == (64, 128) and src.dtype == np.float32
            rc = self._f("ttrans_f32_64x128")(_p(src), _p(out))
        else:
            name = "ttrans_b32" if src.itemsize == 4 else "ttrans_b16"
            rc = self._f(name)(_p(src), _p(out), src.shape[0], src.shape[1])
        assert rc == 0
        return out

    def tsel(self, mask, a, b):
        """mask: uint8, one bit per element of the row-major operands, least significant bit first."""
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        mask = np.ascontiguousarray(mask, np.uint8)
        out = np.empty_like(a)
        name = "tsel_f32" if self.prefix == "pto_ref_" else "tsel_b32"
        rc = self._f(name)(_p(mask), _p(a), _p(b), _p(out), a.shape[0], a.shape[1])
        if rc != 0:
            raise ValueError("tsel: unsupported shape")
        return out

    def tcmps_f32(self, x, scalar, mode):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.size // 8, np.uint8)
        if self.prefix == "pto_ref_":
            assert x.shape == (64, 256)
            rc = self._f("tcmps_f32")(_p(x), ctypes.c_float(scalar), _p(out), int(mode))
        else:
            rc = self._f("tcmps_f32")(_p(x), ctypes.c_float(scalar), _p(out), x.shape[0], x.shape[1], int(mode))
        if rc != 0:
            raise ValueError("tcmps: unsupported shape")
        return out

    def tcmp_f32(self, a, b, mode):
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        out = np.empty_like(a)
        if self.prefix == "pto_ref_":
            rc = self._f("tcmp_f32")(_p(a), _p(b), _p(out), a.shape[0], a.shape[1], int(mode))
        else:
            rc = self._f("tcmp_f32")(_p(a), _p(b), _p(out), _i64(a.size), int(mode))
        if rc != 0:
            raise ValueError("tcmp: unsupported shape")
        return out

    def ttri_f32(self, rows, cols, diagonal, upper):
        out = np.empty((rows, cols), np.float32)
        if self.prefix == "pto_ref_":
            rc = self._f("ttri_f32")(_p(out), rows, cols, int(diagonal), int(upper))
        else:
            rc = self._f("ttri_b32")(_p(out), rows, cols, int(diagonal), int(upper), ctypes.c_uint32(0x3f800000))
        if rc != 0:
            raise ValueError("ttri: unsupported shape")
        return out

    # -- GEMM
    def gemm_f16f32(self, a, b, b_layout):
        """a: (m,k) fp16; b: (k,n) fp16 when b_layout == 0, (n,k) when 1.  Returns (m,n) fp32."""
        a = np.ascontiguousarray(a, np.float16)
        b = np.ascontiguousarray(b, np.float16)
        m, k = a.shape
        n = b.shape[1] if b_layout == 0 else b.shape[0]
        c = np.empty((m, n), np.float32)
        rc = self._f("gemm_f16f32")(_p(a), _p(b), _p(c), m, n, k, int(b_layout))
        if rc != 0:
            raise ValueError("gemm: unsupported shape")
        return c

    def gemm_f16f32_window(self, a, b, b_layout, r0, r1, c0, c1):
        """Restatement only: computes C[r0:r1, c0:c1] of the full product and returns that window."""
        a = np.ascontiguousarray(a, np.float16)
        b = np.ascontiguousarray(b, np.float16)
        m, k = a.shape
        n = b.shape[1] if b_layout == 0 else b.shape[0]
        c = np.zeros((m, n), np.float32) if (m * n <= (1 << 26)) else None
        if c is None:
            raise ValueError("window helper is for matrices up to 64M outputs")
        rc = self._f("gemm_f16f32_window")(_p(a), _p(b), _p(c), m, n, k, int(b_layout), r0, r1, c0, c1)
        assert rc == 0
        return c[r0:r1, c0:c1].copy()

    # -- MX block-scaled fp8 GEMM
    def mxgemm_fp8(self, a, b, sfa, sfb, a_fmt=1, b_fmt=1, window=None):
        """a: (m,k), b: (n,k) fp8 bytes; sfa: (m,k/32), sfb: (n,k/32) e8m0 bytes.  Returns the exact sums as fp32 (m,n);
        with window=(r0, r1, c0, c1) only that part of C is computed (the rest stays 0)."""
        a, b = np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(b, np.uint8)
        sfa, sfb = np.ascontiguousarray(sfa, np.uint8), np.ascontiguousarray(sfb, np.uint8)
        (m, k), n = a.shape, b.shape[0]
        assert b.shape[1] == k and sfa.shape == (m, k // 32) and sfb.shape == (n, k // 32)
        r0, r1, c0, c1 = window if window is not None else (0, m, 0, n)
        c = np.zeros((m, n), np.float32)
        rc = self._f("mxgemm_fp8_window")(_p(a), _p(b), _p(sfa), _p(sfb), _p(c), m, n, k, int(a_fmt), int(b_fmt), r0, r1,
                                          c0, c1)
        if rc != 0:
            raise ValueError("mxgemm: unsupported shape or format")
        return c

    def mxgemm_fp4(self, a, b, sfa, sfb, window=None):
        """a: (m,k/2), b: (n,k/2) bytes of packed float4_e2m1 (low nibble first); scales as mxgemm_fp8.  Exact sums, fp32."""
        a, b = np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(b, np.uint8)
        sfa, sfb = np.ascontiguousarray(sfa, np.uint8), np.ascontiguousarray(sfb, np.uint8)
        m, n, k = a.shape[0], b.shape[0], 2 * a.shape[1]
        assert b.shape[1] == a.shape[1] and sfa.shape == (m, k // 32) and sfb.shape == (n, k // 32)
        r0, r1, c0, c1 = window if window is not None else (0, m, 0, n)
        c = np.zeros((m, n), np.float32)
        rc = self._f("mxgemm_fp4_window")(_p(a), _p(b), _p(sfa), _p(sfb), _p(c), m, n, k, r0, r1, c0, c1)
        if rc != 0:
            raise ValueError("mxgemm_fp4: unsupported shape")
        return c

    def tmatmul_i8i32(self, a, b):
        """a: (m,k) int8, b: (k,n) int8 -> (m,n) int32, exact."""
        a, b = np.ascontiguousarray(a, np.int8), np.ascontiguousarray(b, np.int8)
        (m, k), n = a.shape, b.shape[1]
        c = np.empty((m, n), np.int32)
        assert self._f("tmatmul_i8i32")(_p(a), _p(b), _p(c), m, k, n) == 0
        return c

    # -- attention (one head)
    def attn_head_f16(self, q, k, v, causal, scale):
        q = np.ascontiguousarray(q, np.float16)
        k = np.ascontiguousarray(k, np.float16)
        v = np.ascontiguousarray(v, np.float16)
        o = np.empty(q.shape, np.float32)
        rc = self._f("attn_head_f16")(_p(q), _p(k), _p(v), _p(o), q.shape[0], k.shape[0], q.shape[1], int(causal),
                                      ctypes.c_float(scale))
        if rc != 0:
            raise ValueError("attn_head: unsupported shape")
        return o

    def fa_tiled_f16(self, q, k, v, causal, scale, tile_s1=256):
        q = np.ascontiguousarray(q, np.float16)
        k = np.ascontiguousarray(k, np.float16)
        v = np.ascontiguousarray(v, np.float16)
        o = np.empty(q.shape, np.float32)
        rc = self._f("fa_tiled_f16")(_p(q), _p(k), _p(v), _p(o), q.shape[0], k.shape[0], q.shape[1], int(causal),
                                     ctypes.c_float(scale), int(tile_s1))
        assert rc == 0
        return o


def _load():
    build()
    port = _Lib(os.path.join(_HERE, "liboracle.so"), "pto_oracle_")
    ref_path = os.path.join(_HERE, "_ref", "libpto_ref.so")
    ref = _Lib(ref_path, "pto_ref_") if os.path.exists(ref_path) else None
    return port, ref


port, ref = _load()
