"""Row-expand family, TROWMIN, column reductions, TFILLPAD, TTRANS, TSEL, TCMPS, TCMP on the GPU through the C ABI,
against the CPU restatement (oracle.port), the golden vectors of the reference's generators, and size-independent
properties at 16 M elements.  Bit-exact except where stated (TCOLSUM: summation order; EXPDIF: exp of the device)."""
import os

import numpy as np
import pytest
import torch

import oracle
import pto_isa_b200 as pto
from pto_isa_b200 import ops
from util import dev, host

pytestmark = pytest.mark.gpu
port = oracle.port

SHAPES = [(64, 256), (37, 200), (5, 7), (1, 8), (129, 1), (300, 1028)]


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_rowexpand_family(rows, cols):
    r = np.random.default_rng(rows * 1000 + cols)
    a = (r.standard_normal((rows, cols)) * 3).astype(np.float32)
    s = (r.standard_normal(rows) + 2.5).astype(np.float32)
    fns = {0: pto.TROWEXPANDADD, 1: pto.TROWEXPANDSUB, 2: pto.TROWEXPANDMUL, 3: pto.TROWEXPANDDIV, 4: pto.TROWEXPANDMAX,
           5: pto.TROWEXPANDMIN}
    for op, fn in fns.items():
        got = host(fn(cuda(a), cuda(s)))
        assert np.array_equal(bits(got), bits(port.trowexpand_f32(a, s, op))), op
    got = host(pto.TROWEXPAND(cuda(s), cols))
    assert np.array_equal(bits(got), bits(port.trowexpand_f32(np.zeros_like(a), s, 7)))
    # exp(a - s): the device's double-precision exp rounded to float; at most one float ulp from the reference's
    got = host(pto.TROWEXPANDEXPDIF(cuda(a), cuda(s)))
    want = port.trowexpand_f32(a, s, 6)
    assert np.all(np.abs(bits(got).astype(np.int64) - bits(want).astype(np.int64)) <= 1)
    assert np.mean(bits(got) == bits(want)) > 0.999


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_rowmin_and_column_reductions(rows, cols):
    r = np.random.default_rng(rows * 7 + cols)
    a = (r.standard_normal((rows, cols)) * 10).astype(np.float32)
    assert np.array_equal(bits(host(pto.TROWMIN(cuda(a)))), bits(port.trowmin_f32(a)))
    assert np.array_equal(bits(host(pto.TCOLMAX(cuda(a)))), bits(port.tcolreduce_f32(a, 4)))
    assert np.array_equal(bits(host(pto.TCOLMIN(cuda(a)))), bits(port.tcolreduce_f32(a, 5)))
    # the sum is a fixed-order tree: tolerance 2e-6 of the column's absolute mass (the reference sums top to bottom)
    got, want = host(pto.TCOLSUM(cuda(a))), port.tcolreduce_f32(a, 0)
    assert np.all(np.abs(got - want) <= 2e-6 * np.abs(a).sum(axis=0) + 1e-30)
    # small integers sum exactly in any order
    ai = r.integers(-16, 16, (rows, cols)).astype(np.float32)
    assert np.array_equal(host(pto.TCOLSUM(cuda(ai))), port.tcolreduce_f32(ai, 0))


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_fillpad_trans_sel_cmp(rows, cols):
    r = np.random.default_rng(rows * 31 + cols)
    a = r.standard_normal((rows, cols)).astype(np.float32)
    b = r.standard_normal((rows, cols)).astype(np.float32)
    for kind in (ops.PAD_ZERO, ops.PAD_MAX, ops.PAD_MIN):
        for vr, vc in ((rows, cols), (rows // 2, cols // 3), (0, 0), (rows, 1)):
            got = host(pto.TFILLPAD(cuda(a), vr, vc, kind))
            assert np.array_equal(bits(got), bits(port.tfillpad_f32(a, vr, vc, kind))), (kind, vr, vc)
    h = a.astype(np.float16)
    got = host(pto.TFILLPAD(cuda(h), rows // 2, cols // 3, ops.PAD_MIN))
    want = np.full_like(h, -np.inf)
    want[: rows // 2, : cols // 3] = h[: rows // 2, : cols // 3]
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    assert np.array_equal(host(pto.TTRANS(cuda(a))), port.ttrans(a))
    assert np.array_equal(host(pto.TTRANS(cuda(h))).view(np.uint16), port.ttrans(h.view(np.uint16)))
    n = rows * cols
    mask = r.integers(0, 256, (n + 7) // 8, dtype=np.uint8)
    want = np.where(np.unpackbits(mask, bitorder="little")[:n].reshape(rows, cols) == 1, a, b)
    assert np.array_equal(host(pto.TSEL(cuda(mask), cuda(a), cuda(b))), want)
    if n % 8 == 0:
        assert np.array_equal(want, port.tsel(mask, a, b))
    assert np.array_equal(host(pto.TSEL(cuda(mask), cuda(h), cuda(b.astype(np.float16)))).view(np.uint16),
                          np.where(np.unpackbits(mask, bitorder="little")[:n].reshape(rows, cols) == 1, h,
                                   b.astype(np.float16)).view(np.uint16))
    ai, bi = np.round(a * 2), np.round(b * 2)
    for mode in range(6):
        assert np.array_equal(host(pto.TCMP(cuda(ai), cuda(bi), mode)), port.tcmp_f32(ai, bi, mode)), mode
        if cols % 8 == 0:  # the reference packs cols / 8 bytes per row
            assert np.array_equal(host(pto.TCMPS(cuda(ai), 1.0, mode)), port.tcmps_f32(ai, 1.0, mode)), mode


def test_column_reduction_forms_agree():
    """The two-pass form (caller workspace) and the single-pass form give the same max / min and sums within the
    order tolerance; a workspace that is too small falls back to the single pass."""
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(1000, 2052, device="cuda", generator=g)
    need = pto.lib().pto_b200_tcolreduce_workspace_bytes(1000, 2052)
    assert need > 0 and pto.lib().pto_b200_tcolreduce_workspace_bytes(100, 2052) == 0
    small = torch.empty(4, device="cuda")
    for fn in (pto.TCOLMAX, pto.TCOLMIN):
        assert torch.equal(fn(a), fn(a, workspace=small))
        assert torch.equal(fn(a), getattr(a, "max" if fn is pto.TCOLMAX else "min")(dim=0).values)
    s2, s1 = pto.TCOLSUM(a), pto.TCOLSUM(a, workspace=small)
    assert (s2 - s1).abs().max().item() <= 2e-6 * a.abs().sum(dim=0).max().item()
    want = port.tcolreduce_f32(host(a), 0)
    assert np.all(np.abs(host(s2) - want) <= 2e-6 * np.abs(host(a)).sum(axis=0))


def test_tcmps_equality_window():
    # EQ / NE compare |a - b| in double against 1e-9 (include/pto/cpu/TCmps.hpp:27-33)
    x = np.array([1.0, 1.0 + 2 ** -23, 1e-10, -1e-10, 0.0, 5e-10, 2e-9, 3.0], np.float32)
    for mode in (0, 1):
        assert np.array_equal(host(pto.TCMPS(cuda(x), 0.0, mode)), port.tcmps_f32(x.reshape(1, 8), 0.0, mode))
        assert np.array_equal(host(pto.TCMPS(cuda(x), 1.0, mode)), port.tcmps_f32(x.reshape(1, 8), 1.0, mode))


def test_goldens_of_the_reference_generators(golden_dir):
    z = np.load(os.path.join(golden_dir, "vector2.npz"))
    x = z["trowexpand_src"]
    assert np.array_equal(host(pto.TROWEXPAND(cuda(x[:, 0].copy()), 64)), z["trowexpand_golden"])
    fns = {"div": pto.TROWEXPANDDIV, "mul": pto.TROWEXPANDMUL, "sub": pto.TROWEXPANDSUB, "add": pto.TROWEXPANDADD,
           "min": pto.TROWEXPANDMIN, "max": pto.TROWEXPANDMAX}
    for name, fn in fns.items():
        got = host(fn(cuda(z[f"trowexpandop_{name}_a"]), cuda(z[f"trowexpandop_{name}_s"])))
        assert np.array_equal(got, z[f"trowexpandop_{name}_golden"]), name
    got = host(pto.TROWEXPANDEXPDIF(cuda(z["trowexpandop_expdif_a"]), cuda(z["trowexpandop_expdif_s"])))
    assert np.allclose(got, z["trowexpandop_expdif_golden"], rtol=1e-3, atol=0)  # the reference test's eps
    assert np.array_equal(host(pto.TROWMIN(cuda(z["trowmin0_src"]))), z["trowmin0_golden"])
    assert np.array_equal(host(pto.TCOLMAX(cuda(z["tcolmax_src"]))), z["tcolmax_golden"])
    assert np.array_equal(host(pto.TCOLSUM(cuda(z["tcolsum_src"]))), z["tcolsum_golden"])
    assert np.array_equal(host(pto.TCOLMIN(cuda(z["tcolmin0_src"]))), z["tcolmin0_golden"])
    assert np.array_equal(host(pto.TTRANS(cuda(z["ttrans_src"]))), z["ttrans_golden"])
    for i in range(3):
        got = host(pto.TSEL(cuda(z[f"tsel{i}_mask"]), cuda(z[f"tsel{i}_a"]), cuda(z[f"tsel{i}_b"])))
        assert np.array_equal(got, z[f"tsel{i}_golden"])
    for i in range(8):
        if f"tcmps{i}_src" in z:
            got = host(pto.TCMPS(cuda(z[f"tcmps{i}_src"]), float(z[f"tcmps{i}_scalar"][0]), int(z[f"tcmps{i}_mode"])))
            assert np.array_equal(got, z[f"tcmps{i}_golden"]), i
    assert np.array_equal(host(pto.TCMP(cuda(z["tcmp_a"]), cuda(z["tcmp_b"]), 0)), z["tcmp_golden"])


@pytest.mark.parametrize("rows,cols", [(4, 4), (64, 64), (68, 132), (1024, 192), (260, 64), (8, 4100)])
def test_ttrans_vector_path_shapes(rows, cols):
    """Shapes the 16-byte path takes (rows and cols multiples of 4), with partial 64 x 64 edge tiles."""
    a = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols)
    guard = torch.full((cols + 1, rows), -1.0, device="cuda")
    pto.TTRANS(cuda(a), out=guard[:cols])
    got = host(guard)
    assert np.array_equal(got[:cols], port.ttrans(a)) and (got[cols] == -1.0).all()


def test_full_size_properties():
    """4096 x 4096 (the vector-op config's 16 M elements): identities that need no CPU pass."""
    g = torch.Generator(device="cuda").manual_seed(11)
    n = 4096
    a = torch.randn(n, n, device="cuda", generator=g)
    t = pto.TTRANS(a)
    assert torch.equal(pto.TTRANS(t), a) and torch.equal(t[17], a[:, 17])
    rmin, cmin, cmax = pto.TROWMIN(a), pto.TCOLMIN(a), pto.TCOLMAX(a)
    assert torch.equal(rmin, pto.TCOLMIN(t)) and torch.equal(pto.TROWMAX(a), pto.TCOLMAX(t))
    assert torch.equal(rmin.min(), cmin.min()) and torch.equal(cmax.max(), pto.TROWMAX(a).max())
    s = pto.TROWMAX(a)
    d = pto.TROWEXPANDSUB(a, s)
    assert torch.equal(pto.TROWMAX(d), torch.zeros(n, device="cuda"))
    assert torch.equal(pto.TROWEXPANDADD(d, s), a) or (pto.TROWEXPANDADD(d, s) - a).abs().max().item() < 1e-6
    csum = pto.TCOLSUM(a)
    assert (csum.double().sum() - pto.TROWSUM(a).double().sum()).abs().item() < 1e-2
    bits_gt = pto.TCMPS(a, 0.0, ops.CMP_GT)
    zero = torch.zeros_like(a)
    relu = pto.TSEL(bits_gt, a, zero)
    assert torch.equal(relu, pto.TMAX(a, zero))
    assert torch.equal(pto.TCMP(a, zero, ops.CMP_GT), (relu > 0).float())
    pad = pto.TFILLPAD(a, 1000, 3000, ops.PAD_MIN)
    assert torch.equal(pad[:1000, :3000], a[:1000, :3000]) and bool(torch.isinf(pad[1000:]).all()) and \
        bool(torch.isinf(pad[:, 3000:]).all())
    assert pto.device_status() == 0


def test_argument_errors():
    a = torch.zeros(8, 8, device="cuda")
    with pytest.raises(pto.PtoB200Error):
        pto.TCMPS(torch.zeros(7, device="cuda"), 0.0, 0)
    with pytest.raises(pto.PtoB200Error):
        pto.TFILLPAD(a, 9, 8)
    with pytest.raises(pto.PtoB200Error):
        pto.TSEL(torch.zeros(1, dtype=torch.uint8, device="cuda"), a, a)
    with pytest.raises(pto.PtoB200Error):
        pto.TCOLSUM(torch.zeros(0, 8, device="cuda"))
    assert pto.TROWMIN(torch.zeros(0, 8, device="cuda")).numel() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.int32, torch.float16, torch.int16])
def test_ttri_and_treshape(dtype):
    """TTRI against the oracle for lower / upper triangles, diagonals outside the tile included; TRESHAPE is a view."""
    for rows, cols in ((64, 256), (37, 200), (1, 1), (300, 1028)):
        for diagonal in (-400, -3, 0, 1, 7, 2000):
            for upper in (False, True):
                got = pto.TTRI(rows, cols, diagonal, upper, dtype)
                want = port.ttri_f32(rows, cols, diagonal, int(upper))
                assert np.array_equal(host(got.float()), want), (rows, cols, diagonal, upper)
    t = pto.TTRI(64, 256, 3, True, dtype)
    r = pto.TRESHAPE(t, 128, 128)
    assert r.data_ptr() == t.data_ptr() and torch.equal(r.reshape(-1), t.reshape(-1))
    with pytest.raises(pto.PtoB200Error):
        pto.TRESHAPE(t, 100, 100)
