"""Host callers shaped like the reference's torch demos (demos/torch_jit/*/jit_util_*.py, demos/baseline/gemm_basic)."""
import pytest
import torch

from pto_isa_b200 import jit_util

from util import dev


def test_flop_accounting_matches_the_reference_formula():
    # demos/torch_jit/flash_atten/fa_benchmark.py:30-66
    b, sq, sk, h = 2, 128, 256, 128
    f = jit_util.attn_flops_matmul_softmax_scale(b, sq, sk, h)
    rows = b * sq
    assert f["matmul"] == 4 * b * sq * sk * h
    assert f["scale"] == b * sq * sk
    assert f["softmax"] == rows * (sk - 1) + rows * sk + rows * sk + rows * (sk - 1) + rows * sk
    assert f["total"] == f["matmul"] + f["scale"] + f["softmax"]
    f2 = jit_util.attn_flops_matmul_softmax_scale(b, sq, sk, h, include_scale=False, count_exp_as_flop=False,
                                                  count_max_as_flop=False)
    assert f2["scale"] == 0 and f2["softmax"] == rows * sk + rows * (sk - 1) + rows * sk
    assert jit_util.tflops(2e12, 1000.0) == pytest.approx(2.0)


def test_operator_schema_is_the_reference_one():
    # demos/baseline/gemm_basic/csrc/host/my_gemm_basic.cpp:43-46
    schema = torch.ops.pto_b200.pto_gemm_basic.default._schema
    assert str(schema) == "pto_b200::pto_gemm_basic(Tensor a, Tensor b_dn) -> Tensor"


def test_operator_shape_inference_and_no_cpu_kernel():
    a = torch.empty(512, 2048, dtype=torch.float16, device="meta")
    b_dn = torch.empty(1536, 2048, dtype=torch.float16, device="meta")
    out = torch.ops.pto_b200.pto_gemm_basic(a, b_dn)
    assert out.shape == (512, 1536) and out.dtype == torch.float32
    with pytest.raises(NotImplementedError):
        torch.ops.pto_b200.pto_gemm_basic(torch.zeros(8, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16))


def test_loaders_reject_cpu_tensors():
    gemm = jit_util.load_lib()
    z = torch.zeros(4, 4)
    with pytest.raises(Exception):
        gemm(z, z, z)
    flash = jit_util.load_flash_lib()
    with pytest.raises(Exception):
        flash(z, z, z, z)


@pytest.mark.gpu
def test_operator_on_the_reference_shape():
    import pto_isa_b200 as pto
    g = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.rand(512, 2048, device="cuda", generator=g) * 2 - 1).half()
    b_dn = (torch.rand(1536, 2048, device="cuda", generator=g) * 2 - 1).half()
    out = jit_util.pto_gemm_basic(a, b_dn)
    assert out.shape == (512, 1536) and out.dtype == torch.float32
    assert torch.equal(out, pto.gemm(a, b_dn, 1))
    ref = a.float() @ b_dn.float().t()
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


@pytest.mark.gpu
def test_gemm_loader_equals_the_abi_entry_point():
    import pto_isa_b200 as pto
    g = torch.Generator(device="cuda").manual_seed(4)
    n = jit_util.GEMM_JIT_M
    a = (torch.rand(n, n, device="cuda", generator=g) * 2 - 1).half()
    b = (torch.rand(n, n, device="cuda", generator=g) * 2 - 1).half()
    c = torch.zeros(n, n, device="cuda")
    gemm = jit_util.load_lib()
    gemm(c, a, b)
    torch.cuda.synchronize()
    assert torch.equal(c, pto.gemm(a, b, 1))
    assert pto.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
def test_flash_loader_equals_the_abi_entry_point(causal):
    import pto_isa_b200 as pto
    g = torch.Generator(device="cuda").manual_seed(5)
    s0, s1, d = 512, 512, 128
    q = torch.randn(s0, d, device="cuda", generator=g).half()
    k = torch.randn(s1, d, device="cuda", generator=g).half()
    v = torch.randn(s1, d, device="cuda", generator=g).half()
    o = torch.zeros(s0, d, device="cuda")
    flash = jit_util.load_flash_lib()
    flash(q, k, v, o, is_causal=causal)
    torch.cuda.synchronize()
    expect = pto.flash_attn_fwd(q, k, v, causal=causal, out_dtype=torch.float32)  # internal scale 1/sqrt(d)
    assert torch.equal(o, expect)
    assert pto.device_status() == 0
