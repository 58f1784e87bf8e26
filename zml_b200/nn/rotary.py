"""Rotary position embedding: layouts, frequency scalings and the HF config parser.

Behaviour follows the reference (zml/nn.zig:536-880): three layouts for how the
head dimension splits into real / imaginary / pass-through parts, five ways to
derive ``inv_freq`` (default, llama3, yarn, linear, proportional) read from the
``rope_scaling`` / ``rope_parameters`` object of a HF ``config.json``, partial rotary
dimensions and the yarn attention factor.  ``inv_freq`` is computed on the host in
float32/float64 exactly as the reference does and handed to the RoPE kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Optional

import torch

from ..ops import reference as _ref


class Layout(Enum):
    real_im_pass = 0
    interleaved = 1
    real_pass_im_pass = 2


@dataclass
class Scaling:
    """`kind` is one of default, llama3, yarn, linear, proportional."""
    kind: str = "default"
    rope_theta: float = 10000.0
    factor: Optional[float] = None
    high_freq_factor: float = 4.0
    low_freq_factor: float = 1.0
    original_max_position_embeddings: int = 8192
    truncate: bool = True
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: Optional[float] = None
    mscale_all_dim: Optional[float] = None
    attention_factor: Optional[float] = None
    partial_rotary_factor: float = 1.0

    @staticmethod
    def from_hf(obj: Optional[dict], rope_theta: Optional[float] = None) -> "Scaling":
        """Parses HF `rope_scaling`; None -> default.  Unknown types fall back to default
        (the reference warns and does the same)."""
        if obj is None:
            s = Scaling()
        else:
            kind = obj.get("rope_type", obj.get("type"))
            if kind is None:
                raise ValueError("rope_scaling needs a 'rope_type'")
            if kind not in ("default", "llama3", "yarn", "linear", "proportional"):
                kind = "default"
            known = {f for f in Scaling.__dataclass_fields__ if f != "kind"}
            s = Scaling(kind=kind, **{k: v for k, v in obj.items() if k in known and v is not None})
            if kind in ("llama3", "linear") and s.factor is None:
                raise ValueError(f"rope scaling {kind} needs 'factor'")
        if rope_theta is not None and (obj is None or "rope_theta" not in obj):
            s.rope_theta = float(rope_theta)
        return s

    def partial_rotary_dim(self, head_dim: int) -> int:
        if self.kind in ("yarn", "proportional"):
            return int(math.floor(head_dim * min(max(self.partial_rotary_factor, 0.0), 1.0)))
        return int(head_dim)

    def attention_scaling(self) -> float:
        if self.kind != "yarn":
            return 1.0
        if self.attention_factor is not None:
            return float(self.attention_factor)

        def get_mscale(factor, mscale):
            return 1.0 if mscale < 1.0 else 0.1 * mscale * math.log(factor) + 1.0
        if self.mscale is not None and self.mscale_all_dim is not None:
            return get_mscale(self.factor, self.mscale) / get_mscale(self.factor, self.mscale_all_dim)
        return get_mscale(self.factor, 1.0)


@dataclass
class RopeOpts:
    layout: Layout = Layout.real_im_pass
    scaling: Scaling = field(default_factory=Scaling)


def inv_freq(head_dim: int, opts: RopeOpts) -> torch.Tensor:
    """float32 [rotary_dim / 2] inverse frequencies (zml/nn.zig:797-880)."""
    import numpy as np
    s = opts.scaling
    half = head_dim // 2
    n = s.partial_rotary_dim(half)
    theta = np.float32(s.rope_theta)
    log_theta = np.log(theta, dtype=np.float32)
    idx = np.arange(n, dtype=np.float32)
    f = np.exp(-log_theta * (idx / np.float32(n)), dtype=np.float32)
    if s.kind == "proportional":
        f = np.exp(-log_theta * (idx / np.float32(half)), dtype=np.float32)
    elif s.kind == "linear":
        f = (f / np.float32(s.factor)).astype(np.float32)
    elif s.kind == "llama3":
        m = float(s.original_max_position_embeddings)
        f_high = s.high_freq_factor * (2 * math.pi) / m
        f_low = s.low_freq_factor * (2 * math.pi) / m
        down = 1.0 / s.factor
        out = f.copy()
        for i in range(n):
            v = float(f[i])
            if v > f_high:
                continue
            if v < f_low:
                out[i] = np.float32(v * down)
            else:
                lerp = (v - f_low) / (f_high - f_low)
                out[i] = np.float32(f[i] * np.float32(lerp + (1 - lerp) * down))
        f = out
    elif s.kind == "yarn":
        m = float(s.original_max_position_embeddings)
        f_high = s.beta_fast * (2 * math.pi) / m
        f_low = s.beta_slow * (2 * math.pi) / m
        down = 1.0 / s.factor
        n_low = -math.log(f_high) / math.log(s.rope_theta) * n
        n_high = -math.log(f_low) / math.log(s.rope_theta) * n
        if s.truncate:
            n_high, n_low = math.ceil(n_high), math.floor(n_low)
        out = f.copy()
        for i in range(n):
            v = float(f[i])
            if v > f_high:
                continue
            if v < f_low:
                out[i] = np.float32(v * down)
            else:
                lerp = (n_high - i) / (n_high - n_low)
                out[i] = np.float32(f[i] * np.float32(lerp + (1 - lerp) * down))
        f = out
    return torch.from_numpy(np.ascontiguousarray(f, dtype=np.float32))


def rope(x: torch.Tensor, positions: Optional[torch.Tensor] = None, opts: RopeOpts = RopeOpts()):
    """Rotates x[..., s, h, hd] (or [..., s, hd]) at `positions` (default 0..s-1)."""
    squeeze = False
    if x.dim() == 2:
        x = x[:, None, :]
        squeeze = True
    hd = x.shape[-1]
    if positions is None:
        positions = torch.arange(x.shape[-3], device=x.device)
    rot = opts.scaling.partial_rotary_dim(hd)
    freqs = inv_freq(hd, opts).to(x.device)
    y = _ref.rope_rotate(x, positions, freqs, opts.layout.value, rot, opts.scaling.attention_scaling())
    return y[:, 0, :] if squeeze else y


# ---- how a head vector splits into real / imaginary / pass-through parts (zml/nn.zig:718-790) ----------------
def split_real_img(x: torch.Tensor, layout: Layout) -> tuple[torch.Tensor, torch.Tensor]:
    """(real, imaginary) halves of the last axis: first / second half for the sequential layouts, even / odd entries
    for the interleaved one."""
    n = x.shape[-1]
    if layout is Layout.interleaved:
        return x[..., 0::2], x[..., 1::2]
    return x[..., : n // 2], x[..., n // 2:]


def merge_real_img(real: torch.Tensor, imag: torch.Tensor, layout: Layout) -> torch.Tensor:
    if layout is Layout.interleaved:
        return torch.stack([real, imag], dim=-1).flatten(-2)
    return torch.cat([real, imag], dim=-1)


def split_real_img_pass(x: torch.Tensor, layout: Layout, rotary_dim: int):
    """(real, imaginary, pass-through) when only `rotary_dim` of the head dimension rotates; the pass-through is
    None, one tensor, or for `real_pass_im_pass` the pair (after the real part, after the imaginary part)."""
    hd = x.shape[-1]
    if rotary_dim == hd:
        return (*split_real_img(x, layout), None)
    half, hr = hd // 2, rotary_dim // 2
    if layout is Layout.real_im_pass:
        return x[..., :hr], x[..., hr:rotary_dim], x[..., rotary_dim:]
    if layout is Layout.real_pass_im_pass:
        return x[..., :hr], x[..., half:half + hr], (x[..., hr:half], x[..., half + hr:])
    return x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2], x[..., rotary_dim:]


def merge_real_img_pass(real: torch.Tensor, imag: torch.Tensor, passthrough, layout: Layout) -> torch.Tensor:
    if passthrough is None:
        return merge_real_img(real, imag, layout)
    if layout is Layout.real_im_pass:
        return torch.cat([real, imag, passthrough], dim=-1)
    if layout is Layout.real_pass_im_pass:
        return torch.cat([real, passthrough[0], imag, passthrough[1]], dim=-1)
    return torch.cat([merge_real_img(real, imag, layout), passthrough], dim=-1)
