"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


# (label, worst relative error, bar) of every labelled parity check of this run; tests/conftest.py prints the list in
# pytest's terminal summary, so that the margins are in the log of a passing run too
PARITY_LOG = []


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def rel_err_ok(actual, expected, tol=2e-3, label=None):
    """Max relative error with a denominator floor: |a - e| <= tol * max(|e|, rms(e)) everywhere.
    The floor keeps outputs that cancel to ~0 from dominating; it is stated with every use."""
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    floor = np.sqrt(np.mean(e * e))
    bound = tol * np.maximum(np.abs(e), floor)
    diff = np.abs(a - e)
    worst = float((diff / np.maximum(np.abs(e), floor)).max())
    if label is not None:
        PARITY_LOG.append((label, worst, tol))
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


def few_key_allowance(q, k, v, scale, causal, keys_below=128):
    """Extra absolute allowance for causal rows that see fewer than `keys_below` keys (the first query tile).

    Where it comes from: P is rounded to fp16 by the oracle and by the kernel, whose logits are summed in another
    order.  A weight whose two roundings fall on different sides moves by one fp16 ulp, at most 2^-10 of itself, and
    the output by 2^-10 * w_j * |v_jc| (w_j: the weight after normalisation).  In a row with thousands of keys no
    weight is large enough for that to matter; in a row with a handful, one such flip of the largest contributor alone
    can exceed 2e-3 of the output.  The allowance is exactly that: one flipped ulp of the largest contributor,
    2^-10 * max_j (w_j |v_jc|), for rows with fewer than `keys_below` keys, zero for every other row.
    `keys_below` = 128, one key tile: with 128 or more N(0, 1)-like logits the largest weight stays below the 0.08
    at which 2^-10 * w * |v| (|v| up to 4.5) reaches 2e-3 of the outputs' rms."""
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    v = np.asarray(v, np.float32)
    allow = np.zeros((q.shape[0], v.shape[1]), np.float64)
    if not causal:
        return allow
    for r in range(min(keys_below - 1, q.shape[0], k.shape[0])):
        x = (k[:r + 1] @ q[r]).astype(np.float64) * scale
        w = np.exp(x - x.max())
        w /= w.sum()
        allow[r] = 2.0 ** -10 * (w[:, None] * np.abs(v[:r + 1].astype(np.float64))).max(axis=0)
    return allow


def attn_err_ok(actual, expected, tol=2e-3, half_output=False, label=None, allowance=None):
    """Attention tolerance: every element within `tol` (2e-3, the bar this backend is held to) of the oracle, the
    relative error of an element being |a - e| / max(|e|, rms(e)).

    What the measured error consists of: the oracle and the kernel both round P to fp16 before the second product,
    but relative to different row maxima (the kernel's running maximum at that key tile, the oracle's maximum of the
    whole row), so the two roundings are independent: each output carries the difference of two sums of fp16
    rounding errors, about 4e-4 of its size (rms), 1.3e-3 to 1.5e-3 at the worst element of a head.
    The reference's own streaming formulation differs from its plain one by the same mechanism.

    `half_output`: `actual` is the kernel's output after its own rounding to fp16 (tested separately to be the
    round-to-nearest-even of its fp32 output) and `expected` the oracle's unrounded fp32 output; half an fp16 ulp of
    the value (2^-11 of it, 2^-25 absolute below the normal range) is allowed on top for that rounding.
    `allowance`: see few_key_allowance().
    Returns (ok, worst relative error, fraction of elements within tol); prints the worst error when given a label."""
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    floor = np.sqrt(np.mean(e * e))
    den = np.maximum(np.abs(e), floor)
    diff = np.abs(a - e)
    if half_output:
        diff = np.maximum(diff - np.maximum(np.abs(a) * 2.0 ** -11, 2.0 ** -25), 0.0)
    if allowance is not None:  # few_key_allowance(): one flipped fp16 ulp of the largest weight, short causal rows only
        diff = np.maximum(diff - np.asarray(allowance, np.float64), 0.0)
    rel = diff / den
    worst = float(rel.max())
    frac_ok = float((rel <= tol).mean())
    if label is not None:
        PARITY_LOG.append((label, worst, tol))
        print(f"attention parity {label}: worst relative error {worst:.3e} (bar {tol:.0e}), rms of the oracle {floor:.3f}")
    return bool(worst <= tol), worst, frac_ok
