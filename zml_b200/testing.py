"""Test helpers: closeness check with an error report, random inputs, layer comparison.

`expect_close` has the contract of the reference's `zml.testing.expectClose`
(zml/testing.zig:51-286): a value is close when |l - r| <= atol + rtol * |r|, and
the check passes when at least `min_close` of the values are close; on failure the
message carries max / mean / RMSE and error percentiles.
"""
from __future__ import annotations

import torch


class NotClose(AssertionError):
    pass


def error_report(left: torch.Tensor, right: torch.Tensor) -> dict:
    l, r = left.detach().double().flatten().cpu(), right.detach().double().flatten().cpu()
    err = (l - r).abs()
    finite = torch.isfinite(err)
    e = err[finite] if finite.any() else torch.zeros(1, dtype=torch.double)
    qs = torch.tensor([0.5, 0.9, 0.99, 0.999], dtype=torch.double)
    if e.numel() > 1_000_000:
        idx = torch.randperm(e.numel())[:1_000_000]
        pct = torch.quantile(e[idx], qs)
    else:
        pct = torch.quantile(e, qs)
    return {
        "max": float(e.max()), "mean": float(e.mean()), "rmse": float(e.pow(2).mean().sqrt()),
        "p50": float(pct[0]), "p90": float(pct[1]), "p99": float(pct[2]), "p99.9": float(pct[3]),
        "non_finite": int((~finite).sum()),
    }


def close_fraction(left, right, atol=1e-3, rtol=1e-2) -> float:
    l, r = left.detach().double(), right.detach().double()
    same_inf = torch.isinf(l) & torch.isinf(r) & (torch.sign(l) == torch.sign(r))
    both_nan = torch.isnan(l) & torch.isnan(r)
    ok = ((l - r).abs() <= atol + rtol * r.abs()) | same_inf | both_nan
    return float(ok.double().mean()) if ok.numel() else 1.0


def expect_close(left, right, atol: float = 1e-3, rtol: float = 1e-2, min_close: float = 0.999):
    if tuple(left.shape) != tuple(right.shape):
        raise NotClose(f"shape mismatch: {tuple(left.shape)} vs {tuple(right.shape)}")
    frac = close_fraction(left, right, atol, rtol)
    if frac < min_close:
        rep = error_report(left, right)
        raise NotClose(
            f"only {frac * 100:.3f}% of values are close (need {min_close * 100:.3f}%), "
            f"atol={atol} rtol={rtol}; errors: {rep}")


def expect_equal_shapes(expected, actual):
    if tuple(expected) != tuple(actual):
        raise AssertionError(f"expected shape {tuple(expected)}, got {tuple(actual)}")
