"""Test helpers: closeness check with an error report, random inputs, layer comparison.

`expect_close` has the contract of the reference's `zml.testing.expectClose`
(zml/testing.zig:51-286): a value is close when |l - r| <= atol + rtol * |r|, and
the check passes when at least `min_close` of the values are close; on failure the
message carries max / mean / RMSE and error percentiles.
"""
from __future__ import annotations

from dataclasses import dataclass

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


def _to_torch(x) -> torch.Tensor:
    """Buffers, Slices and tagged Tensors are brought to a host torch tensor; Buffers are gathered (the reference's
    `expectClose` accepts both, zml/testing.zig:42-57)."""
    if torch.is_tensor(x):
        return x
    if hasattr(x, "to_tensor"):          # Buffer
        return x.to_tensor()
    if hasattr(x, "to_torch"):           # Slice
        return x.to_torch()
    if hasattr(x, "data") and torch.is_tensor(getattr(x, "data")):      # Tensor
        return x.data
    return torch.as_tensor(x)


def approx_eq(l: float, r: float, tolerance: float) -> bool:
    """Close relatively (|l - r| <= tolerance * max(|l|, |r|)) or absolutely (|l - r| <= tolerance / 2): near zero the
    relative precision matters less (zml/testing.zig:36-40)."""
    d = abs(l - r)
    return d <= tolerance * max(abs(l), abs(r)) or d <= tolerance / 2


@dataclass
class CompareOpts:
    """zml/testing.zig:120-132."""
    absolute_tolerance: float = 1e-3
    relative_tolerance: float = 1e-2
    epsilon_relative: float = 1e-6
    minimum_close_fraction: float = 0.999

    @staticmethod
    def exact_match() -> "CompareOpts":
        return CompareOpts(0.0, 0.0, 0.0, 1.0)


@dataclass
class CompareReport:
    """zml/testing.zig:134-160."""
    nan_or_inf: bool
    max_absolute_error: float
    mean_absolute_error: float
    rmse: float
    close_fraction: float
    p50_absolute_error: float
    p90_absolute_error: float
    p99_absolute_error: float
    p999_absolute_error: float
    p99_relative_error: float = 0.0

    def ok(self, opts: "CompareOpts") -> bool:
        return not self.nan_or_inf and self.close_fraction >= opts.minimum_close_fraction


def compare_slices(left, right, opts: CompareOpts = CompareOpts()) -> CompareReport:
    """The reference's element-wise comparison (zml/testing.zig:222-284): a pair is close when
    |l - r| <= absolute_tolerance + relative_tolerance * max(|l|, |r|); pairs with a non-finite member set
    `nan_or_inf` and count as not close; quantiles are picked at round((n - 1) * q) of the sorted errors."""
    l = _to_torch(left).detach().double().flatten().cpu()
    r = _to_torch(right).detach().double().flatten().cpu()
    if l.numel() != r.numel():
        raise NotClose(f"{l.numel()} values against {r.numel()}")
    n = l.numel()
    if n == 0:
        return CompareReport(False, 0.0, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0, 0.0)
    finite = torch.isfinite(l) & torch.isfinite(r)
    err = torch.where(finite, (l - r).abs(), torch.zeros_like(l))
    scale = torch.maximum(l.abs(), r.abs())
    close = finite & (err <= opts.absolute_tolerance + opts.relative_tolerance * scale)
    rel = torch.where(finite, err / torch.clamp(scale, min=max(opts.epsilon_relative, 1e-300)), torch.zeros_like(l))
    srt, srel = torch.sort(err).values, torch.sort(rel).values

    def q(v, frac):
        return float(v[int(round((n - 1) * frac))])

    return CompareReport(bool((~finite).any()), float(err.max()), float(err.sum() / n), float((err.pow(2).sum() / n).sqrt()),
                         float(close.sum()) / n, q(srt, 0.5), q(srt, 0.9), q(srt, 0.99), q(srt, 0.999), q(srel, 0.99))


def auto_call(exe, *inputs):
    """Calls a compiled executable on `inputs` (Buffers or pytrees of them) and waits for the results: the
    argument / result bookkeeping of zml/testing.zig:302-316 in one line."""
    return exe.call_opts(*inputs, wait=True)


def env():
    """The platform tests run on: CUDA when a GPU is visible, else CPU, with the `model` sharding the attention
    back-ends expect registered (zml/testing.zig:14-32)."""
    global _ENV
    if _ENV is None:
        from .platform import Platform
        from .sharding import LogicalMesh
        _ENV = Platform.auto()
        try:
            _ENV.sharding("model")
        except KeyError:
            _ENV.register_sharding("model", LogicalMesh.mesh({"model": "high_bandwidth"}))
    return _ENV


_ENV = None


def test_layer(*args, **kwargs):
    """`utils.activations.test_layer` under the reference's name (zml/testing.zig:341)."""
    from .utils.activations import test_layer as impl
    return impl(*args, **kwargs)


test_layer.__test__ = False      # not a pytest test despite the name


def expect_close(left, right, atol: float = 1e-3, rtol: float = 1e-2, min_close: float = 0.999):
    left, right = _to_torch(left), _to_torch(right)
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
