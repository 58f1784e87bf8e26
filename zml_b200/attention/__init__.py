"""Attention front-end: one `attention()` entry point over interchangeable back-ends, with
per-backend `Parameters` / `Metadata` objects, as in zml/attention.zig:17-191 of the reference.

Back-ends here:

* ``vanilla``  - causal mask gathered at `token_index` + `nn.sdpa` (the reference's fallback,
  attention.zig:174-184); runs anywhere, used as the oracle.
* ``b200``     - the sm_100a flash kernels of this package (libzb_cuda.so: attention.cu), taking
  the dense K/V as a paged cache whose block table is the identity.  It takes the place of the
  reference's `cuda_fa2` / `cuda_fa3` (FlashAttention binaries reached through XLA FFI).
* ``attnd``    - per-token UDP offload to a remote attention daemon (zml/attention/attnd.zig).

Tensors follow the reference's tags: q {q, h, hd}, k / v {k, h, hd}; `token_index` is the
position of the first query token inside the K/V sequence.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Optional, Union

import torch

from ..nn import attention_ref
from ..tensor import Tensor
from . import attnd, paged  # noqa: F401


class Backend(enum.Enum):
    vanilla = "vanilla"
    attnd = "attnd"
    b200 = "b200"

    @staticmethod
    def auto(platform=None) -> "Backend":
        """The flash kernels on a CUDA platform, the tensor formulation elsewhere."""
        target = getattr(platform, "target", None)
        name = getattr(target, "name", target)
        if name is None:
            return Backend.b200 if torch.cuda.is_available() else Backend.vanilla
        return Backend.b200 if name == "cuda" else Backend.vanilla

    def is_available(self, platform=None) -> bool:
        if self is Backend.b200:
            target = getattr(platform, "target", None)
            name = getattr(target, "name", target)
            return (name == "cuda") if name is not None else torch.cuda.is_available()
        return True


@dataclass
class FlashParameters:
    """Options of the `b200` back-end: sliding window (0 = none) and softmax scale."""
    sliding_window: int = 0
    scale: Optional[float] = None


@dataclass
class FlashMetadata:
    """Shapes the `b200` back-end is planned for (the reference sizes its FA2 scratch buffers from
    the same two numbers, zml/attention/flashattn.zig:146-172)."""
    seqlen: int = 0
    num_heads: int = 0


@dataclass
class Parameters:
    backend: Backend = Backend.vanilla
    value: object = None

    @staticmethod
    def from_backend(backend: Backend) -> "Parameters":
        if backend is Backend.attnd:
            raise ValueError("attnd parameters must be initialised manually (attnd.Parameters.init)")
        return Parameters(backend, FlashParameters() if backend is Backend.b200 else None)

    @staticmethod
    def init(backend_or_value) -> "Parameters":
        if isinstance(backend_or_value, Backend):
            return Parameters.from_backend(backend_or_value)
        if isinstance(backend_or_value, attnd.Parameters):
            return Parameters(Backend.attnd, backend_or_value)
        if isinstance(backend_or_value, FlashParameters):
            return Parameters(Backend.b200, backend_or_value)
        raise TypeError(type(backend_or_value))


@dataclass
class Metadata:
    backend: Backend = Backend.vanilla
    value: object = None

    @staticmethod
    def from_backend(backend: Backend, seqlen: int = 0, num_heads: int = 0) -> "Metadata":
        if backend is Backend.b200:
            return Metadata(backend, FlashMetadata(seqlen, num_heads))
        if backend is Backend.attnd:
            return Metadata(backend, attnd.Metadata())
        return Metadata(backend, None)

    init = from_backend

    def init_buffer(self, platform=None, sharding=None) -> "Metadata":
        """Device-side state of the metadata (only attnd has any: conversation id, layer id, count)."""
        return self

    def deinit_buffer(self) -> None:
        pass


def _token_index_value(token_index) -> int:
    if isinstance(token_index, Tensor):
        return int(token_index.to_torch().reshape(-1)[0])
    if torch.is_tensor(token_index):
        return int(token_index.reshape(-1)[0])
    return int(token_index)


def _vanilla(q: Tensor, k: Tensor, v: Tensor, token_index) -> Tensor:
    seq = k.dim("k")
    dev = q.to_torch().device
    mask = attention_ref.causal_attn_mask({"q": seq, "k": seq}, q.dtype(), None, device=dev)
    t0 = _token_index_value(token_index)
    rows = mask.to_torch()[t0:t0 + q.dim("q")]
    mask_q = Tensor(rows, mask.shape().set_dim("q", q.dim("q")))
    out = attention_ref.sdpa(q.transpose(("h", "q", "hd")), k.transpose(("h", "k", "hd")), v.transpose(("h", "k", "hd")),
                             attn_mask=mask_q)
    return out.transpose(q.shape().tags)


def _flash(q: Tensor, k: Tensor, v: Tensor, token_index, params: FlashParameters) -> Tensor:
    """Dense K/V through the paged kernels: the K/V rows are viewed as pages of 64 tokens and the
    block table is 0, 1, 2, ...  Rows past `token_index + q` are never read (seq_lens bounds them)."""
    from .. import ops
    qt = q.transpose(("q", "h", "hd")).to_torch().contiguous()
    kt = k.transpose(("k", "h", "hd")).to_torch()
    vt = v.transpose(("k", "h", "hd")).to_torch()
    nq, t0 = qt.shape[0], _token_index_value(token_index)
    page = 64
    seq = kt.shape[0]
    pad = (-seq) % page
    if pad:
        kt = torch.nn.functional.pad(kt, (0, 0, 0, 0, 0, pad))
        vt = torch.nn.functional.pad(vt, (0, 0, 0, 0, 0, pad))
    pages = (seq + pad) // page
    kc = kt.contiguous().view(pages, page, kt.shape[1], kt.shape[2])
    vc = vt.contiguous().view(pages, page, vt.shape[1], vt.shape[2])
    dev = qt.device
    bt = torch.arange(pages, dtype=torch.int32, device=dev)[None]
    sl = torch.tensor([t0 + nq], dtype=torch.int32, device=dev)
    if nq == 1:
        o = ops.paged_decode(qt, kc, vc, bt, sl, scale=params.scale, window=params.sliding_window)
    else:
        qs = torch.tensor([0, nq], dtype=torch.int32, device=dev)
        o = ops.paged_prefill(qt, kc, vc, bt, sl, qs, scale=params.scale, window=params.sliding_window)
    return Tensor(o, q.transpose(("q", "h", "hd")).shape()).transpose(q.shape().tags)


def _token_indices(token_index, batch: int) -> list[int]:
    if isinstance(token_index, Tensor):
        token_index = token_index.to_torch()
    if torch.is_tensor(token_index):
        vals = [int(x) for x in token_index.reshape(-1).tolist()]
    elif isinstance(token_index, (list, tuple)):
        vals = [int(x) for x in token_index]
    else:
        vals = [int(token_index)]
    if len(vals) == 1:
        vals = vals * batch
    if len(vals) != batch:
        raise ValueError(f"token_index has {len(vals)} entries for a batch of {batch}")
    return vals


def attention(q: Tensor, k: Tensor, v: Tensor, token_index, metadata: Metadata, parameters: Parameters) -> Tensor:
    """Causal attention of q {q, h, hd} at positions token_index.. over k, v {k, h, hd}.  With a leading batch axis
    `b` on q, k and v, `token_index` holds one position per batch entry (or one for all), as in the reference
    (zml/attention.zig:172-191, its tests use b = 4 with different positions)."""
    if q.shape().has_tag("b") is not None:
        nb = q.dim("b")
        outs = [attention(q.choose1d("b", i), k.choose1d("b", i), v.choose1d("b", i), t, metadata, parameters)
                for i, t in enumerate(_token_indices(token_index, nb))]
        return Tensor.stack(outs, q.axis("b"), "b")
    be = parameters.backend
    if be is Backend.vanilla:
        return _vanilla(q, k, v, token_index)
    if be is Backend.b200:
        return _flash(q, k, v, token_index, parameters.value or FlashParameters())
    if be is Backend.attnd:
        return attnd.causal_attention(q, k, v, token_index, metadata.value, parameters.value)
    raise ValueError(be)
