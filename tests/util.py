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
