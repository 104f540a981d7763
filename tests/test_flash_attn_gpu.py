"""GPU parity of flash-attention forward against the CPU oracle (the reference's instruction sequence with
fp16 operands, fp32 softmax, fp16 P) and the golden output of the reference's NumPy model of its kernel.

Tolerance (util.attn_err_ok): relative error |got - want| / max(|want|, rms(want)) <= 2e-3 for EVERY element; only the
causal rows that see fewer than 128 keys get, on top, one flipped fp16 ulp of their largest weight
(util.few_key_allowance, derived there).
A half-precision output must be the round-to-nearest-even of the fp32 output bit for bit; where only the
half-precision output exists it is compared with the oracle's fp32 output with half an fp16 ulp added for
that rounding.  Every test prints its worst error (pytest -s, or the captured output of a failure)."""
import os

import numpy as np
import pytest
import torch

import oracle
import pto_isa_b200 as pto
from util import attn_err_ok, dev, few_key_allowance, host, result_cmp

pytestmark = pytest.mark.gpu
port = oracle.port


def make_qkv(bh, sq, sk, d, seed):
    r = np.random.default_rng(seed)
    q = (r.standard_normal((bh, sq, d)) / np.sqrt(d)).astype(np.float32).astype(np.float16)  # Q pre-scaled by 1/sqrt(d)
    k = r.standard_normal((bh, sk, d)).astype(np.float16)
    v = r.standard_normal((bh, sk, d)).astype(np.float16)
    return q, k, v


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 128, 128), (1, 256, 256), (2, 128, 512), (3, 384, 384), (1, 1024, 1024),
                                   (2, 512, 256)])
def test_attention_matches_oracle(shape, causal):
    bh, sq, sk = shape
    d = 128
    q, k, v = make_qkv(bh, sq, sk, d, seed=sq + sk + int(causal))
    scale = 1.0  # logits already carry 1/sqrt(d) through Q: the softmax scale argument is exercised below
    o = host(pto.flash_attn_fwd(dev(q), dev(k), dev(v), causal=causal, scale=scale, out_dtype=torch.float32))
    assert pto.device_status() == 0
    for h in range(bh):
        want = port.attn_head_f16(q[h], k[h], v[h], int(causal), scale)
        ok, worst, _ = attn_err_ok(o[h], want, label=f"{shape} causal={causal} head {h}",
                                   allowance=few_key_allowance(q[h], k[h], v[h], scale, causal))
        assert ok, f"head {h}: max relative error {worst:.3e}"


@pytest.mark.parametrize("causal", [False, True])
def test_attention_internal_scale_and_fp16_output(causal):
    r = np.random.default_rng(5)
    bh, s, d = 2, 512, 128
    q = r.standard_normal((bh, s, d)).astype(np.float16)
    k = r.standard_normal((bh, s, d)).astype(np.float16)
    v = r.standard_normal((bh, s, d)).astype(np.float16)
    scale = 1.0 / np.sqrt(d)
    o32 = host(pto.flash_attn_fwd(dev(q), dev(k), dev(v), causal=causal, out_dtype=torch.float32))
    o16 = host(pto.flash_attn_fwd(dev(q), dev(k), dev(v), causal=causal, out_dtype=torch.float16))
    # the same computation (here: both with the deferred rescale) differs only by the rounding on store
    o32d = host(pto.flash_attn_fwd(dev(q), dev(k), dev(v), causal=causal, out_dtype=torch.float32, defer_rescale=True))
    assert np.array_equal(o16, o32d.astype(np.float16))
    o16e = host(pto.flash_attn_fwd(dev(q), dev(k), dev(v), causal=causal, out_dtype=torch.float16, defer_rescale=False))
    assert np.array_equal(o16e, o32.astype(np.float16))
    for h in range(bh):
        want = port.attn_head_f16(q[h], k[h], v[h], int(causal), scale)
        ok, worst, _ = attn_err_ok(o32[h], want, label=f"internal scale causal={causal} head {h}",
                                   allowance=few_key_allowance(q[h], k[h], v[h], scale, causal))
        assert ok, f"head {h}: max relative error {worst:.3e}"
        ok, worst, _ = attn_err_ok(o16[h].astype(np.float32), want, half_output=True,
                                   allowance=few_key_allowance(q[h], k[h], v[h], scale, causal))
        assert ok, f"head {h} (fp16 out): max relative error {worst:.3e}"


def test_attention_golden(golden_dir):
    """Outputs of the reference's own NumPy model of its kernel (TILE_S1 = 256), self-check eps 1e-3."""
    z = np.load(os.path.join(golden_dir, "attention.npz"))
    for name, causal in (("fa_nc_128x512", False), ("fa_causal_128x512", True)):
        q, k, v, g = (z[f"{name}_{n}"] for n in ("q", "k", "v", "o"))
        o = host(pto.flash_attn_fwd(dev(q[None]), dev(k[None]), dev(v[None]), causal=causal,
                                    out_dtype=torch.float32))[0]
        assert result_cmp(g, o, 1e-3), name
        ok, worst, _ = attn_err_ok(o, g, label=name)
        assert ok, f"{name}: max relative error {worst:.3e}"


def test_attention_large_logits_rescale_path():
    """Rows whose running max keeps growing across key tiles (forces the rescale of O in tensor memory)."""
    r = np.random.default_rng(9)
    s, d = 1024, 128
    q = r.standard_normal((1, s, d)).astype(np.float16)
    k = r.standard_normal((1, s, d)).astype(np.float32)
    k *= np.linspace(0.5, 4.0, s)[None, :, None]  # later keys give larger logits
    k = k.astype(np.float16)
    v = r.standard_normal((1, s, d)).astype(np.float16)
    scale = 1.0 / np.sqrt(d)
    for causal in (False, True):
        o = host(pto.flash_attn_fwd(dev(q), dev(k), dev(v), causal=causal, out_dtype=torch.float32))
        want = port.attn_head_f16(q[0], k[0], v[0], int(causal), scale)
        ok, worst, _ = attn_err_ok(o[0], want, label=f"growing maxima causal={causal}",
                                   allowance=few_key_allowance(q[0], k[0], v[0], scale, causal))
        assert ok, f"causal={causal}: max relative error {worst:.3e}"


def test_attention_unsupported_shapes_are_errors():
    q = torch.zeros(1, 128, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(pto.PtoB200Error):
        pto.flash_attn_fwd(q, q, q)
    q = torch.zeros(1, 100, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(pto.PtoB200Error):
        pto.flash_attn_fwd(q, q, q)


@pytest.mark.parametrize("causal", [False, True])
def test_attention_full_size_sampled_heads(causal):
    """B=4, H=32, S=4096, D=128 (the benchmark configuration): all 128 heads run on the GPU; three sampled
    heads are recomputed by the oracle; every output row is a convex combination of V rows (bounded by the
    per-column min/max of V over the visible keys), checked on all heads."""
    bh, s, d = 128, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(1234)
    q = (torch.randn(bh, s, d, device="cuda", generator=g) / d ** 0.5).half()
    k = torch.randn(bh, s, d, device="cuda", generator=g).half()
    v = torch.randn(bh, s, d, device="cuda", generator=g).half()
    o = pto.flash_attn_fwd(q, k, v, causal=causal, scale=1.0, out_dtype=torch.float16)
    assert pto.device_status() == 0
    for h in (0, 77, 127):
        want = port.attn_head_f16(host(q[h]), host(k[h]), host(v[h]), int(causal), 1.0)
        ok, worst, _ = attn_err_ok(host(o[h]).astype(np.float32), want, half_output=True,
                                   label=f"B4 H32 S4096 causal={causal} head {h}",
                                   allowance=few_key_allowance(host(q[h]), host(k[h]), host(v[h]), 1.0, causal))
        assert ok, f"head {h}: max relative error {worst:.3e}"
    if causal:
        vmax = torch.cummax(v.float(), dim=1).values
        vmin = torch.cummin(v.float(), dim=1).values
    else:
        vmax = v.float().amax(dim=1, keepdim=True)
        vmin = v.float().amin(dim=1, keepdim=True)
    of = o.float()
    assert bool((of <= vmax + 2e-3 * vmax.abs() + 1e-3).all()) and bool((of >= vmin - 2e-3 * vmin.abs() - 1e-3).all())
    assert bool(torch.isfinite(of).all())


def test_attention_long_sequence_causal_sampled_rows():
    """S = 8192, causal (the sequence length of the multi-GPU sharding configuration), 6 heads: the last 128 queries
    (they see all 8192 keys, 64 key tiles) and the first 256 of two heads are recomputed by the oracle, which is
    given the same rows as a rectangular problem (s0 rows against the keys they may see)."""
    bh, s, d = 6, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(8192)
    q = (torch.randn(bh, s, d, device="cuda", generator=g) / d ** 0.5).half()
    k = torch.randn(bh, s, d, device="cuda", generator=g).half()
    v = torch.randn(bh, s, d, device="cuda", generator=g).half()
    o = pto.flash_attn_fwd(q, k, v, causal=True, scale=1.0, out_dtype=torch.float32)
    assert pto.device_status() == 0
    for h in (0, 5):
        # first 256 queries: a square causal problem of its own
        want = port.attn_head_f16(host(q[h, :256]), host(k[h, :256]), host(v[h, :256]), 1, 1.0)
        ok, worst, _ = attn_err_ok(host(o[h, :256]), want, label=f"S8192 head {h} first 256 rows",
                                   allowance=few_key_allowance(host(q[h, :256]), host(k[h, :256]), host(v[h, :256]), 1.0, True))
        assert ok, f"head {h} first rows: max relative error {worst:.3e}"
        # last 128 queries against all keys: row i of the block may see keys 0 .. s - 128 + i; the oracle's causal mask
        # works on square problems, so every row is checked as the last row of the problem made of keys 0 .. its own
        for row in (s - 128, s - 65, s - 1):
            qi = host(q[h, row:row + 1]).repeat(128, axis=0)  # 128 copies: the oracle's tile height
            want_row = port.attn_head_f16(qi, host(k[h, :row + 1]), host(v[h, :row + 1]), 0, 1.0)[0]
            got_row = host(o[h, row])
            ok, worst, _ = attn_err_ok(got_row, want_row, label=f"S8192 head {h} row {row}")
            assert ok, f"head {h} row {row}: max relative error {worst:.3e}"
    assert bool(torch.isfinite(o).all())
