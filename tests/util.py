"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def rel_err_ok(actual, expected, tol=2e-3):
    """Max relative error with a denominator floor: |a - e| <= tol * max(|e|, rms(e)) everywhere.
    The floor keeps outputs that cancel to ~0 from dominating; it is stated with every use."""
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    floor = np.sqrt(np.mean(e * e))
    bound = tol * np.maximum(np.abs(e), floor)
    diff = np.abs(a - e)
    worst = float((diff / np.maximum(np.abs(e), floor)).max())
    return bool((diff <= bound).all()), worst


def result_cmp(golden, actual, eps):
    """The reference's ResultCmp (tests/common/test_common.h:211-300)."""
    g = np.asarray(golden, np.float64).ravel()
    a = np.asarray(actual, np.float64).ravel()
    diff = np.abs(g - a)
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.where(g != 0, diff / np.abs(g), np.inf)
    bad = (diff > eps) & (rel > eps)
    return int(bad.sum()) <= g.size * eps


def attn_err_ok(actual, expected, tol=2e-3, hard=5e-3, quantile_ok=0.9999):
    """Attention tolerance.  The relative error of an element is |a - e| / max(|e|, rms(e)).

    P is rounded to fp16 before the second product, by the oracle as well as by the kernel.  The kernel's
    logits come from a tensor-core sum in a different order and its exponentials from ex2.approx, so about
    0.2 % of the P values fall on the other side of an fp16 rounding boundary (one fp16 ulp, 2^-10 relative).
    In rows that see only a few keys a single such flip moves an output by more than 2e-3 of its own size.
    The bar is therefore: at least 99.99 % of the elements within `tol`, every element within `hard`.
    The reference's own streaming formulation differs from its plain one by the same mechanism."""
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    floor = np.sqrt(np.mean(e * e))
    rel = np.abs(a - e) / np.maximum(np.abs(e), floor)
    frac_ok = float((rel <= tol).mean())
    worst = float(rel.max())
    return bool(frac_ok >= quantile_ok and worst <= hard), worst, frac_ok
