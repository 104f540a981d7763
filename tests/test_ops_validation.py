"""Argument checks of the Python host layer (pto_isa_b200/ops.py), without a GPU.

The C ABI takes raw pointers and sizes: a tensor that is smaller than the sizes claim would be read or written out
of bounds on the device.  The wrappers therefore refuse mismatched operands before anything reaches the library.
Here the device check is switched off and the library replaced by a recorder, so that the checks themselves can be
exercised on CPU tensors; no kernel runs."""
import pytest
import torch

from pto_isa_b200 import ops
from pto_isa_b200._lib import PtoB200Error


class _Recorder:
    """Stands in for the loaded library: every entry point reports success and counts the call."""

    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        def fn(*args):
            self.calls.append(name)
            return 0
        return fn


@pytest.fixture()
def rec(monkeypatch):
    r = _Recorder()
    monkeypatch.setattr(ops, "lib", lambda: r)
    monkeypatch.setattr(ops, "_need_cuda", lambda *ts: None)
    monkeypatch.setattr(ops, "_stream", lambda t: None)
    # result tensors are made on the operands' (CPU) device here
    real_out = ops._out

    def out_on_cpu(out, shape, dtype, device, what):
        if out is None:
            return torch.empty(tuple(shape) if not isinstance(shape, int) else (shape,), dtype=dtype)
        return real_out(out, shape, dtype, device, what)
    monkeypatch.setattr(ops, "_out", out_on_cpu)
    monkeypatch.setattr(torch.cuda, "device", lambda d: __import__("contextlib").nullcontext())
    return r


def h(*shape):
    return torch.zeros(*shape, dtype=torch.float16)


def test_gemm_rejects_mismatched_k_rank_and_batch(rec):
    ops.gemm(h(128, 64), h(256, 64), 1)
    ops.gemm(h(128, 64), h(64, 256), 0)
    assert rec.calls == ["pto_b200_gemm_f16f32"] * 2
    with pytest.raises(PtoB200Error, match="k extents"):
        ops.gemm(h(128, 64), h(256, 32), 1)
    with pytest.raises(PtoB200Error, match="k extents"):
        ops.gemm(h(128, 64), h(256, 64), 0)
    with pytest.raises(PtoB200Error, match="both 2-D, or both 3-D"):
        ops.gemm(h(2, 128, 64), h(256, 64), 1)
    with pytest.raises(PtoB200Error, match="same batch"):
        ops.gemm(h(2, 128, 64), h(3, 256, 64), 1)
    with pytest.raises(PtoB200Error, match="b_layout"):
        ops.gemm(h(128, 64), h(256, 64), 2)
    assert len(rec.calls) == 2  # nothing reached the library


def test_gemm_variants_reject_mismatched_k(rec):
    b16 = lambda *s: torch.zeros(*s, dtype=torch.bfloat16)
    with pytest.raises(PtoB200Error, match="k extents"):
        ops.gemm_bf16(b16(128, 64), b16(256, 48), 1)
    with pytest.raises(PtoB200Error, match="k extents"):
        ops.gemm_out16(h(128, 64), h(256, 48), 1)
    with pytest.raises(PtoB200Error, match="float16 or bfloat16"):
        ops.gemm_out16(h(128, 64), h(256, 64), 1, out_dtype=torch.float32)
    i8 = lambda *s: torch.zeros(*s, dtype=torch.int8)
    with pytest.raises(PtoB200Error):
        ops.gemm_i8(i8(128, 64), i8(256, 32))
    assert rec.calls == []


def test_out_tensors_are_checked(rec):
    with pytest.raises(PtoB200Error, match="must have shape"):
        ops.gemm(h(128, 64), h(256, 64), 1, out=torch.zeros(128, 128))
    with pytest.raises(PtoB200Error, match="must have shape"):
        ops.gemm(h(128, 64), h(256, 64), 1, out=torch.zeros(128, 256, dtype=torch.float16))
    with pytest.raises(PtoB200Error, match="CUDA tensor"):
        ops.gemm(h(128, 64), h(256, 64), 1, out=torch.zeros(128, 256))  # right shape and type, wrong device
    with pytest.raises(PtoB200Error, match="contiguous|must have shape|CUDA"):
        ops.TEXP(torch.zeros(8, 8), out=torch.zeros(16, 8)[::2])
    with pytest.raises(PtoB200Error, match="must have shape"):
        ops.TGATHER(torch.zeros(4, 4), torch.zeros(8, dtype=torch.int32), out=torch.zeros(4))
    with pytest.raises(PtoB200Error, match="must have shape"):
        ops.TROWMAX(torch.zeros(4, 8), out=torch.zeros(8))
    with pytest.raises(PtoB200Error, match="must have shape"):
        ops.TADD(torch.zeros(4, 8), torch.zeros(4, 8), out=torch.zeros(4, 8, dtype=torch.float16))
    assert rec.calls == []


def test_texp_needs_float32(rec):
    with pytest.raises(PtoB200Error, match="float32"):
        ops.TEXP(h(8, 8))
    assert rec.calls == []


def test_flash_attention_checks_shapes_and_output_type(rec):
    q, k = h(2, 4, 128, 128), h(2, 4, 256, 128)
    ops.flash_attn_fwd(q, k, k.clone())
    assert rec.calls == ["pto_b200_flash_attn_fwd_f16"]
    with pytest.raises(PtoB200Error, match="float16 or float32"):
        ops.flash_attn_fwd(q, k, k, out_dtype=torch.bfloat16)
    with pytest.raises(PtoB200Error, match="must share"):
        ops.flash_attn_fwd(q, h(2, 3, 256, 128), h(2, 3, 256, 128))
    with pytest.raises(PtoB200Error, match="must share"):
        ops.flash_attn_fwd(q, k, h(2, 4, 128, 128))
    with pytest.raises(PtoB200Error, match="must share"):
        ops.flash_attn_fwd(q, h(2, 4, 256, 64), h(2, 4, 256, 64))
    with pytest.raises(PtoB200Error, match="must have shape"):
        ops.flash_attn_fwd(q, k, k, out_dtype=torch.float32, out=torch.zeros(2, 4, 128, 128, dtype=torch.float16))
    assert len(rec.calls) == 1


def test_host_variants_check_their_operands(rec):
    a, b, c = h(128, 64), h(256, 64), torch.zeros(128, 256)
    ops.gemm_host(a, b, c)
    with pytest.raises(PtoB200Error, match="k extents"):
        ops.gemm_host(a, h(256, 32), c)
    with pytest.raises(PtoB200Error, match=r"\(m, n\)"):
        ops.gemm_host(a, b, torch.zeros(128, 128))
    with pytest.raises(PtoB200Error, match="float16"):
        ops.gemm_host(a.float(), b, c)
    with pytest.raises(PtoB200Error, match="disagree"):
        ops.gemm_host_batched(h(2, 128, 64), h(2, 256, 64), torch.zeros(2, 128, 128))
    with pytest.raises(PtoB200Error, match="disagree"):
        ops.gemm_host_batched(h(2, 128, 64), h(3, 256, 64), torch.zeros(2, 128, 256))
    q, k = h(1, 128, 128), h(1, 256, 128)
    with pytest.raises(PtoB200Error, match="disagree"):
        ops.flash_attn_fwd_host(q, k, k, torch.zeros(1, 256, 128))
    with pytest.raises(PtoB200Error, match="float16 or float32"):
        ops.flash_attn_fwd_host(q, k, k, torch.zeros(1, 128, 128, dtype=torch.bfloat16))
    assert rec.calls == ["pto_b200_gemm_f16f32_host"]
