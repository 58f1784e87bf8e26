"""Ops of the hybrid decoder layers: depthwise causal conv with a rolling cache, the gated
delta rule scan, and the sigmoid output gate (libzb_cuda.so: linear_attn.cu).

All three run over the flattened varlen token batch the engine uses everywhere else:
`q_start[S+1]` gives every sequence's token range in this launch, `seq_lens[S]` its length
including those tokens (so `seq_lens - count == 0` marks a sequence that starts here and
takes a zero state), `slots[S]` its row in the state pool.  On CPU tensors the functions
below evaluate the same math with plain torch in float32 - that is also the test oracle.

Reference: zml/nn.zig:1749-1874 (GatedDeltaNet), examples/llm/models/qwen3_5/model.zig:824-980,
examples/llm/models/lfm2/model.zig:441-500.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

_p, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
_lib.register_signature("zb_causal_conv1d", _i, [_p, _ll, _p, _ll, _p, _ll, _p, _p, _ll, _p, _p, _p, _p, _i, _i,
                                                _i, _i, _p])
_lib.register_signature("zb_gated_delta_scan", _i, [_p, _ll, _p, _ll, _p, _p, _ll, _p, _p, _p, _f, _p, _p, _ll,
                                                   _p, _p, _p, _i, _i, _i, _i, _i, _p])
_lib.register_signature("zb_sigmoid_gate_mul", _i, [_p, _ll, _p, _ll, _i, _i, _p])


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


# ---------------------------------------------------------------------------- conv
def causal_conv1d_reference(x, w, state, q_start, seq_lens, slots, pre=None, post=None, silu=False):
    t, c = x.shape
    k = w.shape[1]
    out = torch.empty((t, c), dtype=x.dtype, device=x.device)
    wf = w.float()
    qs, sl, so = q_start.tolist(), seq_lens.tolist(), slots.tolist()
    for s in range(len(sl)):
        a, b = qs[s], qs[s + 1]
        if b <= a:
            continue
        xin = x[a:b].float()
        if pre is not None:
            xin = _bf16_round(xin * pre[a:b].float())
        hist = torch.zeros((k - 1, c)) if sl[s] - (b - a) <= 0 else state[so[s]].float()
        full = torch.cat([hist.to(xin.device), xin], 0)                     # [K-1+n, C]
        win = full.unfold(0, k, 1)                                           # [n, C, K]
        y = _bf16_round((win * wf[None]).sum(-1))
        if silu:
            y = y * torch.sigmoid(y)
        if post is not None:
            y = _bf16_round(y) * post[a:b].float()
        out[a:b] = y.to(x.dtype)
        state[so[s]] = full[-(k - 1):].to(state.dtype)
    return out


def causal_conv1d(x, w, state, q_start, seq_lens, slots, pre=None, post=None, silu: bool = False, out=None):
    """x [T, C] (row stride free), w [C, K] taps (tap K-1 on the current token), state
    [slots, K-1, C] updated in place.  Returns [T, C]."""
    if not x.is_cuda:
        return causal_conv1d_reference(x, w, state, q_start, seq_lens, slots, pre, post, silu)
    t, c = x.shape
    k = w.shape[1]
    assert w.is_contiguous() and state.is_contiguous() and state.shape[1:] == (k - 1, c)
    if out is None:
        out = torch.empty((t, c), dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().zb_causal_conv1d(
        _ptr(x), x.stride(0), _ptr(pre), pre.stride(0) if pre is not None else 0, _ptr(post),
        post.stride(0) if post is not None else 0, _ptr(w), _ptr(out), out.stride(0), _ptr(state),
        _ptr(q_start), _ptr(seq_lens), _ptr(slots), seq_lens.shape[0], c, k, 1 if silu else 0, _lib.stream_ptr())
    _lib.check(rc, "zb_causal_conv1d")
    return out


# ---------------------------------------------------------------------------- gated delta rule
def gated_delta_scan_reference(mix, z, a, b, a_log, dt_bias, norm_w, eps, state, q_start, seq_lens, slots,
                               hk, hv, dk, dv):
    t = mix.shape[0]
    key_dim = hk * dk
    rep = hv // hk
    out = torch.empty((t, hv * dv), dtype=mix.dtype, device=mix.device)
    q = mix[:, :key_dim].float().reshape(t, hk, dk).repeat_interleave(rep, 1)
    k = mix[:, key_dim:2 * key_dim].float().reshape(t, hk, dk).repeat_interleave(rep, 1)
    v = mix[:, 2 * key_dim:2 * key_dim + hv * dv].float().reshape(t, hv, dv)
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * (dk ** -0.5)
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    alpha = torch.exp(-torch.exp(a_log.float())[None] * torch.nn.functional.softplus(a.float() + dt_bias.float()[None]))
    beta = torch.sigmoid(b.float())
    qs, sl, so = q_start.tolist(), seq_lens.tolist(), slots.tolist()
    for s in range(len(sl)):
        t0, t1 = qs[s], qs[s + 1]
        if t1 <= t0:
            continue
        st = torch.zeros((hv, dk, dv)) if sl[s] - (t1 - t0) <= 0 else state[so[s]].float().clone()
        st = st.to(mix.device)
        for i in range(t0, t1):
            vh = torch.einsum("hkv,hk->hv", st, k[i]) * alpha[i][:, None]
            delta = (v[i] - vh) * beta[i][:, None]
            st = st * alpha[i][:, None, None] + k[i][:, :, None] * delta[:, None, :]
            y = _bf16_round(torch.einsum("hkv,hk->hv", st, q[i]))
            inv = torch.rsqrt((y * y).mean(-1, keepdim=True) + eps)
            zg = z[i].float().reshape(hv, dv)
            out[i] = (y * inv * norm_w.float()[None] * (zg * torch.sigmoid(zg))).reshape(-1).to(mix.dtype)
        state[so[s]] = st.to(state.dtype)
    return out


def gated_delta_scan(mix, z, a, b, a_log, dt_bias, norm_w, eps, state, q_start, seq_lens, slots,
                     hk: int, hv: int, dk: int, dv: int, out=None):
    """mix [T, 2*hk*dk + hv*dv] = q | k | v after the conv; z [T, hv*dv]; a, b [T, hv] (same row
    stride); a_log, dt_bias float32 [hv]; norm_w [dv]; state float32 [slots, hv, dk, dv] updated
    in place.  Returns the gated, normalised output [T, hv*dv]."""
    if not mix.is_cuda:
        return gated_delta_scan_reference(mix, z, a, b, a_log, dt_bias, norm_w, eps, state, q_start, seq_lens,
                                          slots, hk, hv, dk, dv)
    t = mix.shape[0]
    assert a.stride(0) == b.stride(0) and state.dtype == torch.float32 and state.is_contiguous()
    assert a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32
    if out is None:
        out = torch.empty((t, hv * dv), dtype=torch.bfloat16, device=mix.device)
    rc = _lib.lib().zb_gated_delta_scan(
        _ptr(mix), mix.stride(0), _ptr(z), z.stride(0), _ptr(a), _ptr(b), a.stride(0), _ptr(a_log), _ptr(dt_bias),
        _ptr(norm_w), float(eps), _ptr(state), _ptr(out), out.stride(0), _ptr(q_start), _ptr(seq_lens),
        _ptr(slots), seq_lens.shape[0], hk, hv, dk, dv, _lib.stream_ptr())
    _lib.check(rc, "zb_gated_delta_scan")
    return out


# ---------------------------------------------------------------------------- output gate
def sigmoid_gate_mul(x, gate):
    """x[r, c] * sigmoid(gate[r, c]); in place on CUDA tensors."""
    if not x.is_cuda:
        return (x.float() * torch.sigmoid(gate.float())).to(x.dtype)
    rows, cols = x.shape
    rc = _lib.lib().zb_sigmoid_gate_mul(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), rows, cols,
                                        _lib.stream_ptr())
    _lib.check(rc, "zb_sigmoid_gate_mul")
    return x
