from __future__ import annotations

import ctypes as C
import enum
from typing import Optional

import torch

from ..ops import _lib

_lib.register_signature("zb_moe_router_topk", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                                         C.c_longlong, C.c_int, C.c_void_p], optional=False)
_lib.register_signature("zb_moe_align", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                   C.c_int, C.c_void_p], optional=False)
_lib.register_signature("zb_moe_gather", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                    C.c_int, C.c_int, C.c_void_p], optional=False)
_lib.register_signature("zb_moe_finalize", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                      C.c_int, C.c_void_p], optional=False)
_lib.register_signature("zb_moe_grouped_gemm", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                          C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p],
                        optional=False)


class Backend(enum.Enum):
    """b200: the tcgen05 grouped-GEMM path; reference: per-expert torch matmuls (CPU / oracle)."""
    b200 = "b200"
    reference = "reference"

    @staticmethod
    def auto(x: torch.Tensor) -> "Backend":
        return Backend.b200 if x.is_cuda else Backend.reference


# ---------------------------------------------------------------------- router
def _baseline_on() -> bool:
    from ..ops import baseline as _baseline
    return _baseline.enabled()


def router_topk(logits: torch.Tensor, k: int, renormalize: bool = True):
    """float32 logits [T, E] -> (ids int32 [T, k], weights float32 [T, k]): top-k experts and the
    softmax over the selected logits (`renormalize`) or the softmax over all experts."""
    if not logits.is_cuda or _baseline_on():
        lf = logits.float()
        v, i = torch.topk(lf, k, dim=-1)
        w = torch.softmax(v, -1) if renormalize else torch.softmax(lf, -1).gather(1, i)
        return i.to(torch.int32), w
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    t, e = logits.shape
    ids = torch.empty((t, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((t, k), dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().zb_moe_router_topk(logits.data_ptr(), ids.data_ptr(), w.data_ptr(), t, e, k,
                                             logits.stride(0), int(renormalize), _lib.stream_ptr()), "zb_moe_router_topk")
    return ids, w


# ---------------------------------------------------------------------- permutation
def moe_align(ids: torch.Tensor, e0: int, e_local: int):
    """Groups the (token, expert) pairs of the local experts [e0, e0 + e_local) by expert.
    Returns (meta, sorted_pair, pair_pos): meta[:e_local + 1] are the row offsets of each
    expert in the permuted order, sorted_pair[pos] is the pair index t * k + j at row `pos`,
    pair_pos[pair] is the row of a pair (-1: expert not local)."""
    pairs = ids.numel()
    dev = ids.device
    if not ids.is_cuda:
        flat = ids.reshape(-1).long() - e0
        local = (flat >= 0) & (flat < e_local)
        order = torch.argsort(torch.where(local, flat, torch.full_like(flat, e_local)), stable=True)
        n = int(local.sum())
        sorted_pair = order[:n].to(torch.int32)
        counts = torch.bincount(flat[local], minlength=e_local)
        meta = torch.zeros(2 * e_local + 2, dtype=torch.int32)
        meta[1:e_local + 1] = torch.cumsum(counts, 0).to(torch.int32)
        pair_pos = torch.full((pairs,), -1, dtype=torch.int32)
        pair_pos[sorted_pair.long()] = torch.arange(n, dtype=torch.int32)
        full = torch.zeros(pairs, dtype=torch.int32)
        full[:n] = sorted_pair
        return meta, full, pair_pos
    meta = torch.empty(2 * e_local + 2, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(pairs, dtype=torch.int32, device=dev)
    pair_pos = torch.empty(pairs, dtype=torch.int32, device=dev)
    _lib.check(_lib.lib().zb_moe_align(ids.data_ptr(), meta.data_ptr(), sorted_pair.data_ptr(), pair_pos.data_ptr(),
                                       pairs, e0, e_local, _lib.stream_ptr()), "zb_moe_align")
    return meta, sorted_pair, pair_pos


def gather(x: torch.Tensor, sorted_pair: torch.Tensor, meta: torch.Tensor, e_local: int, k: int, cap: int):
    """xs[pos] = x[sorted_pair[pos] // k] for the rows in use; xs has `cap` rows."""
    d = x.shape[1]
    if not x.is_cuda:
        n = int(meta[e_local])
        xs = torch.zeros((cap, d), dtype=x.dtype)
        xs[:n] = x[(sorted_pair[:n].long() // k)]
        return xs
    xs = torch.empty((cap, d), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().zb_moe_gather(x.data_ptr(), sorted_pair.data_ptr(), meta.data_ptr(), xs.data_ptr(), e_local,
                                        k, d, cap, _lib.stream_ptr()), "zb_moe_gather")
    return xs


def nvfp4_roundtrip(w: torch.Tensor) -> torch.Tensor:
    """Quantises expert weights [..., N, K] to NVFP4 (e2m1 values, one f8e4m3fn scale per 16, one
    fp32 scale per matrix) and returns them de-quantised to the input dtype: the values an NVFP4
    checkpoint holds, in the layout the bf16 grouped GEMM consumes."""
    from ..nn import quant as Q
    out = torch.empty_like(w)
    flat_in, flat_out = w.reshape(-1, w.shape[-2], w.shape[-1]), out.reshape(-1, w.shape[-2], w.shape[-1])
    for e in range(flat_in.shape[0]):                      # one matrix at a time bounds the fp32 temporaries
        packed, scales, gs = Q.quantize_weight_nvfp4(flat_in[e])
        flat_out[e] = Q.dequantize_nvfp4(Q.unpack_e2m1(packed), scales, gs, w.dtype)
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[E, F, D] x 2 -> [E, 2F, D] with rows laid out [64 gate | 64 up] per 128-row block, the
    layout the grouped GEMM's SwiGLU epilogue expects (F must be a multiple of 64)."""
    e, f, d = gate.shape
    assert f % 64 == 0 and up.shape == gate.shape
    g = gate.reshape(e, f // 64, 64, d)
    u = up.reshape(e, f // 64, 64, d)
    return torch.cat([g, u], 2).reshape(e, 2 * f, d).contiguous()


def deinterleave_gate_up(w: torch.Tensor):
    e, f2, d = w.shape
    b = w.reshape(e, f2 // 128, 2, 64, d)
    return b[:, :, 0].reshape(e, f2 // 2, d), b[:, :, 1].reshape(e, f2 // 2, d)


# Activations of the expert MLP (zml/moe/cutlass_flashinfer.zig:24-28 of the reference): the gated ones take an
# interleaved gate|up weight, `relu2` a plain up projection.  The code is what the kernels' `swiglu` argument carries.
ACTIVATIONS = {"none": 0, "swiglu": 1, "geglu": 2, "geglu_tanh": 3, "relu2": 4}


def activation_code(swiglu) -> int:
    """False / True (SwiGLU) / an activation name -> kernel code."""
    if isinstance(swiglu, str):
        return ACTIVATIONS[swiglu]
    return 1 if swiglu else 0


def _gate_act(g: torch.Tensor, code: int) -> torch.Tensor:
    if code == 2:
        return torch.nn.functional.gelu(g)
    if code == 3:
        return torch.nn.functional.gelu(g, approximate="tanh")
    return torch.nn.functional.silu(g)


def grouped_gemm(xs: torch.Tensor, w: torch.Tensor, meta: torch.Tensor, swiglu=False, avg_tokens: int = 8):
    """Per local expert e: out[rows_e] = xs[rows_e] @ w[e]^T.  `swiglu` True or "swiglu" / "geglu" / "geglu_tanh": w is
    the interleaved gate/up weight [E, 2F, K] and out is act(gate) * up, [cap, F]; "relu2": relu(x w^T)^2."""
    e_local, n, k = w.shape
    cap = xs.shape[0]
    code = activation_code(swiglu)
    gated = 1 <= code <= 3
    n_out = n // 2 if gated else n
    if not xs.is_cuda:
        out = torch.zeros((cap, n_out), dtype=xs.dtype)
        gate_up = deinterleave_gate_up(w) if gated else None
        for e in range(e_local):
            a, b = int(meta[e]), int(meta[e + 1])
            if b <= a:
                continue
            x = xs[a:b].float()
            if gated:
                g, u = gate_up
                out[a:b] = (_gate_act(x @ g[e].float().t(), code) * (x @ u[e].float().t())).to(xs.dtype)
            elif code == 4:
                out[a:b] = torch.relu(x @ w[e].float().t()).square().to(xs.dtype)
            else:
                out[a:b] = (x @ w[e].float().t()).to(xs.dtype)
        return out
    assert xs.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and xs.is_contiguous() and w.is_contiguous()
    out = torch.empty((cap, n_out), dtype=xs.dtype, device=xs.device)
    _lib.check(_lib.lib().zb_moe_grouped_gemm(xs.data_ptr(), w.data_ptr(), out.data_ptr(), meta.data_ptr(), e_local, n, k,
                                              cap, n_out, code, int(avg_tokens), _lib.stream_ptr()),
               "zb_moe_grouped_gemm")
    return out


_KERNEL_NIBBLE_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)     # nibble position p of a 32-bit word holds weight _KERNEL_NIBBLE_ORDER[p]


def nvfp4_codes_to_kernel_order(codes: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 codes [R, K / 2] (two per byte, low nibble first) -> the same codes with the 8
    nibbles of every 4 bytes re-ordered to (w0 w2 w4 w6 w1 w3 w5 w7), the order the grouped GEMM
    de-quantises with one shift and one mask per weight pair (csrc/moe_w4.cu)."""
    r, kb = codes.shape
    assert kb % 4 == 0
    b = codes.reshape(r, kb // 4, 4)
    nib = torch.stack([b & 0xF, b >> 4], dim=-1).reshape(r, kb // 4, 8)        # weight order
    nib = nib[..., list(_KERNEL_NIBBLE_ORDER)].reshape(r, kb // 4, 4, 2)
    return (nib[..., 0] | (nib[..., 1] << 4)).reshape(r, kb).contiguous()


def nvfp4_codes_from_kernel_order(codes: torch.Tensor) -> torch.Tensor:
    r, kb = codes.shape
    b = codes.reshape(r, kb // 4, 4)
    nib = torch.stack([b & 0xF, b >> 4], dim=-1).reshape(r, kb // 4, 8)        # kernel order
    inv = [0] * 8
    for pos, w in enumerate(_KERNEL_NIBBLE_ORDER):
        inv[w] = pos
    nib = nib[..., inv].reshape(r, kb // 4, 4, 2)
    return (nib[..., 0] | (nib[..., 1] << 4)).reshape(r, kb).contiguous()


W4_K_MULTIPLE = 256         # NVFP4 kernel: one load stage is 4 k-blocks of 64 (16 bytes of block scales per weight row)
W4_BLOCK_BYTES = 128 * 128 + 128 * 16      # one (128 rows x 256 K) block: 16 KB of codes + 2 KB of block scales


def nvfp4_pack_blocks(codes: torch.Tensor, scales: torch.Tensor, e: int, n: int, k: int) -> torch.Tensor:
    """Checkpoint-order codes [E * N, K / 2] and f8e4m3fn scales [E * N, K / 16] -> the tile-major
    layout the grouped GEMM streams (csrc/moe_w4.cu): uint8 [E, N / 128, K / 256, 18432], each block
    [8 chunks][128 rows][16 bytes] of nibble-re-ordered codes, then [128 rows][16] scales."""
    assert n % 128 == 0 and k % 256 == 0
    c = nvfp4_codes_to_kernel_order(codes.reshape(e * n, k // 2)).reshape(e, n // 128, 128, k // 256, 8, 16)
    c = c.permute(0, 1, 3, 4, 2, 5).reshape(e, n // 128, k // 256, 128 * 128)
    sc = scales.reshape(e * n, k // 16).view(torch.uint8).reshape(e, n // 128, 128, k // 256, 16)
    sc = sc.permute(0, 1, 3, 2, 4).reshape(e, n // 128, k // 256, 128 * 16)
    return torch.cat([c, sc], -1).contiguous()


def nvfp4_pack_blocks_mma(codes: torch.Tensor, scales: torch.Tensor, e: int, n: int, k: int) -> torch.Tensor:
    """Checkpoint-order codes [E * N, K / 2] and f8e4m3fn scales [E * N, K / 16] -> the tile-major layout of the
    block-scaled tensor-core kernel (csrc/moe_fp4.cu): uint8 [E, N / 128, K / 256, 18432].  Each block is the
    shared-memory image of its (128 rows x 256 K) tile: 16 KB of codes with the 128-byte swizzle (16-byte chunk j
    of row r at chunk j ^ (r % 8) of the row's 128 bytes), then four 512-byte scale images (one per K = 64):
    [32 rows r % 32][4 row groups r / 32][4 scales]."""
    assert n % 128 == 0 and k % 256 == 0
    dev = codes.device
    c = codes.reshape(e, n // 128, 128, k // 256, 8, 16)                       # [e, tile, r, kchunk, j, b]
    r = torch.arange(128, device=dev)
    j = torch.arange(8, device=dev)
    src = (j[None, :] ^ (r[:, None] % 8))                                      # position p holds chunk p ^ (r % 8)
    c = torch.gather(c, 4, src[None, None, :, None, :, None].expand(e, n // 128, 128, k // 256, 8, 16))
    c = c.permute(0, 1, 3, 2, 4, 5).reshape(e, n // 128, k // 256, 128 * 128)
    sc = scales.reshape(e * n, k // 16).view(torch.uint8).reshape(e, n // 128, 4, 32, k // 256, 4, 4)   # [e, tile, r/32, r%32, kchunk, j, s]
    sc = sc.permute(0, 1, 4, 5, 3, 2, 6).reshape(e, n // 128, k // 256, 128 * 16)                       # [.., kchunk, j, r%32, r/32, s]
    return torch.cat([c, sc], -1).contiguous()


def nvfp4_unpack_blocks(blocks: torch.Tensor, e: int, n: int, k: int):
    """Inverse of `nvfp4_pack_blocks`: (codes [E * N, K / 2] in checkpoint order, scales [E * N, K / 16])."""
    c = blocks[..., :128 * 128].reshape(e, n // 128, k // 256, 8, 128, 16).permute(0, 1, 4, 2, 3, 5).reshape(e * n, k // 2)
    sc = blocks[..., 128 * 128:].reshape(e, n // 128, k // 256, 128, 16).permute(0, 1, 3, 2, 4).reshape(e * n, k // 16)
    return nvfp4_codes_from_kernel_order(c.contiguous()), sc.contiguous().view(torch.float8_e4m3fn)


class Nvfp4Experts:
    """Expert weights [E, N, K] in NVFP4: e2m1 codes, one f8e4m3fn scale per 16 values along K, and
    float32 matrix scales [E, P]: P = 1, or P = 2 for an interleaved gate|up matrix whose gate and up
    halves were quantised separately (rows 0-63 of every 128 take scale 0, rows 64-127 scale 1).
    Held as `blocks` (`nvfp4_pack_blocks`, what the kernel streams) when N is a multiple of 128 and K
    of 256; otherwise as checkpoint-order `codes` [E * N, K / 2] and `scales` [E * N, K / 16], which
    only the de-quantising fallback reads."""

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, gscale: torch.Tensor, e: int, n: int, k: int):
        self.e, self.n, self.k = e, n, k
        self.gscale = gscale.reshape(e, -1).float().contiguous()
        assert self.gscale.shape[1] in (1, 2)
        codes = codes.reshape(e * n, k // 2)
        scales = scales.reshape(e * n, k // 16)
        self.kernel_ready = n % 128 == 0 and k % W4_K_MULTIPLE == 0
        if self.kernel_ready:
            self.blocks, self.codes, self.scales = nvfp4_pack_blocks(codes, scales, e, n, k), None, None
        else:
            self.blocks, self.codes, self.scales = None, codes.contiguous(), scales.contiguous()

    # kept for callers that name where the data comes from
    from_checkpoint = classmethod(lambda cls, codes, scales, gscale, e, n, k: cls(codes, scales, gscale, e, n, k))

    @staticmethod
    def from_checkpoint_gate_up(gate, up) -> "Nvfp4Experts":
        """gate, up: (codes [E, F, K / 2], scales [E, F, K / 16], gscale [E]) of separately quantised
        projections -> one interleaved gate|up matrix [E, 2F, K] with two matrix scales per expert."""
        (gc, gs, gg), (uc, us, ug) = gate, up
        e, f, kb = gc.shape
        codes = interleave_gate_up(gc, uc)
        scales = interleave_gate_up(gs.view(torch.uint8), us.view(torch.uint8)).view(torch.float8_e4m3fn)
        gscale = torch.stack([gg.reshape(e).float(), ug.reshape(e).float()], 1)
        return Nvfp4Experts(codes, scales, gscale, e, 2 * f, kb * 2)

    @staticmethod
    def quantize(w: torch.Tensor) -> "Nvfp4Experts":
        from ..nn import quant as Q
        e, n, k = w.shape
        codes, scales, gs = Q.quantize_weight_nvfp4(w)
        return Nvfp4Experts(codes, scales, gs, e, n, k)

    def checkpoint_arrays(self):
        """(codes [E * N, K / 2] low nibble = even K index, scales [E * N, K / 16])."""
        if self.blocks is not None:
            return nvfp4_unpack_blocks(self.blocks, self.e, self.n, self.k)
        return self.codes, self.scales

    def row_scales(self, i: int) -> torch.Tensor:
        """Matrix scale of every row of expert i, [N, 1]."""
        g = self.gscale[i]
        if g.numel() == 1:
            return g.reshape(1, 1).expand(self.n, 1)
        part = (torch.arange(self.n, device=g.device) // 64) % 2
        return g[part].reshape(self.n, 1)

    def dequantize(self, dtype=torch.bfloat16) -> torch.Tensor:
        from ..nn import quant as Q
        codes, scales = self.checkpoint_arrays()
        out = torch.empty((self.e, self.n, self.k), dtype=dtype, device=codes.device)
        one = torch.ones((), dtype=torch.float32, device=codes.device)
        for i in range(self.e):
            sl = slice(i * self.n, (i + 1) * self.n)
            w = Q.dequantize_nvfp4(Q.unpack_e2m1(codes[sl]), scales[sl], one, torch.float32)
            out[i] = (w * self.row_scales(i)).to(dtype)
        return out

    def mma_blocks(self) -> torch.Tensor:
        """The weights in the layout of the block-scaled tensor-core kernel (made once, on first use)."""
        if getattr(self, "_mma_blocks", None) is None:
            codes, scales = self.checkpoint_arrays()
            self._mma_blocks = nvfp4_pack_blocks_mma(codes, scales, self.e, self.n, self.k)
        return self._mma_blocks

    def nbytes(self) -> int:
        body = self.blocks.numel() if self.blocks is not None else self.codes.numel() + self.scales.numel()
        return body + self.gscale.numel() * 4


def grouped_gemm_w4(xs: torch.Tensor, w: Nvfp4Experts, meta: torch.Tensor, swiglu=False, avg_tokens: int = 8):
    """`grouped_gemm` with NVFP4 expert weights de-quantised inside the kernel (few tokens per
    expert; libzb_cuda.so: zb_moe_grouped_gemm_w4).  CPU tensors: de-quantise, then the float path."""
    if not xs.is_cuda or not w.kernel_ready:
        return grouped_gemm(xs, w.dequantize(xs.dtype), meta, swiglu, avg_tokens)
    cap = xs.shape[0]
    code = activation_code(swiglu)
    n_out = w.n // 2 if 1 <= code <= 3 else w.n
    assert xs.dtype == torch.bfloat16 and xs.is_contiguous() and xs.shape[1] == w.k
    out = torch.empty((cap, n_out), dtype=xs.dtype, device=xs.device)
    _lib.check(_lib.lib().zb_moe_grouped_gemm_w4(xs.data_ptr(), w.blocks.data_ptr(), w.gscale.data_ptr(),
                                                 int(w.gscale.shape[1]), out.data_ptr(), meta.data_ptr(), w.e, w.n, w.k, cap, n_out,
                                                 code,
                                                 int(avg_tokens), _lib.stream_ptr()), "zb_moe_grouped_gemm_w4")
    return out


class Fp4Activations:
    """Activation rows in NVFP4: packed e2m1 codes [rows, K / 2] and f8e4m3fn block scales [rows, K / 16]."""
    __slots__ = ("codes", "scales", "k")

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor):
        self.codes, self.scales, self.k = codes, scales, codes.shape[1] * 2

    @staticmethod
    def quantize(xs: torch.Tensor) -> "Fp4Activations":
        from ..ops import quant as opsq
        return Fp4Activations(*opsq.nvfp4_quantize(xs.to(torch.bfloat16)))

    def dequantize(self, dtype=torch.bfloat16) -> torch.Tensor:
        from ..nn import quant as Q
        return Q.dequantize_nvfp4(Q.unpack_e2m1(self.codes), self.scales, None, dtype)


def gather_fp4(x: torch.Tensor, sorted_pair: torch.Tensor, meta: torch.Tensor, e_local: int, k: int, cap: int) -> Fp4Activations:
    """`gather` with the NVFP4 activation quantiser behind it (one kernel): the rows leave as codes + block scales."""
    d = x.shape[1]
    if not x.is_cuda:
        return Fp4Activations.quantize(gather(x, sorted_pair, meta, e_local, k, cap))
    # rows past the last pair stay unwritten: the GEMM computes their columns too but never stores them
    xq = torch.empty((cap, d // 2), dtype=torch.uint8, device=x.device)
    xsf = torch.empty((cap, d // 16), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib().zb_moe_gather_fp4(x.data_ptr(), sorted_pair.data_ptr(), meta.data_ptr(), xq.data_ptr(), xsf.data_ptr(),
                                            e_local, k, d, cap, _lib.stream_ptr()), "zb_moe_gather_fp4")
    return Fp4Activations(xq, xsf.view(torch.float8_e4m3fn))


def grouped_gemm_fp4(xs, w: Nvfp4Experts, meta: torch.Tensor, swiglu=False, avg_tokens: int = 8,
                     quantize_out: bool = False):
    """`grouped_gemm` with NVFP4 weights AND NVFP4 activations (one f8e4m3 scale per 16 values on both sides),
    multiplied by the block-scaled tensor-core instruction (libzb_cuda.so: zb_moe_grouped_gemm_fp4).  `xs` is an
    `Fp4Activations` or a bf16 tensor (quantised first).  `quantize_out` (with `swiglu`): the result is returned as
    `Fp4Activations`, quantised in the kernel's epilogue.  CPU tensors: de-quantise both sides, then the float path."""
    if not isinstance(xs, Fp4Activations):
        xs = Fp4Activations.quantize(xs)
    if not xs.codes.is_cuda or not w.kernel_ready:
        out = grouped_gemm(xs.dequantize(torch.float32), w.dequantize(torch.float32), meta, swiglu, avg_tokens).to(torch.bfloat16)
        return Fp4Activations.quantize(out) if quantize_out else out
    cap = xs.codes.shape[0]
    code = activation_code(swiglu)
    gated = 1 <= code <= 3
    n_out = w.n // 2 if gated else w.n
    assert xs.k == w.k and xs.codes.is_contiguous() and xs.scales.is_contiguous()
    dev = xs.codes.device
    out = oq = osf = None
    if quantize_out:
        assert gated and n_out % 64 == 0
        oq = torch.empty((cap, n_out // 2), dtype=torch.uint8, device=dev)
        osf = torch.empty((cap, n_out // 16), dtype=torch.uint8, device=dev)
    else:
        out = torch.empty((cap, n_out), dtype=torch.bfloat16, device=dev)
    ptr = lambda t: t.data_ptr() if t is not None else None
    _lib.check(_lib.lib().zb_moe_grouped_gemm_fp4(xs.codes.data_ptr(), xs.scales.data_ptr(), None, w.mma_blocks().data_ptr(),
                                                  w.gscale.data_ptr(), int(w.gscale.shape[1]), ptr(out), ptr(oq), ptr(osf),
                                                  meta.data_ptr(), w.e, w.n, w.k, cap, n_out, code, int(avg_tokens),
                                                  _lib.stream_ptr()), "zb_moe_grouped_gemm_fp4")
    return Fp4Activations(oq, osf.view(torch.float8_e4m3fn)) if quantize_out else out


def finalize(o: torch.Tensor, pair_pos: torch.Tensor, weights: torch.Tensor, tokens: int, k: int):
    """y[t] = sum_j weights[t, j] * o[pair_pos[t * k + j]] over the pairs that are local."""
    d = o.shape[1]
    if not o.is_cuda:
        pos = pair_pos.reshape(tokens, k).long()
        valid = pos >= 0
        rows = o[pos.clamp_min(0)].float() * (weights.float() * valid)[..., None]
        return rows.sum(1).to(o.dtype)
    y = torch.empty((tokens, d), dtype=o.dtype, device=o.device)
    _lib.check(_lib.lib().zb_moe_finalize(o.data_ptr(), pair_pos.data_ptr(), weights.data_ptr(), y.data_ptr(), tokens, k, d,
                                          _lib.stream_ptr()), "zb_moe_finalize")
    return y


def combine(o: torch.Tensor, pair_pos: torch.Tensor, weights: torch.Tensor, tokens: int, k: int, extra=None, residual=None,
            fused=None):
    """residual + [sum over the ranks of `fused`] (extra + finalize(o, pair_pos, weights)) in one kernel
    (libzb_cuda.so: zb_moe_combine); `fused` is a SymmetricContext whose slot area holds the exchange."""
    if not o.is_cuda:
        assert fused is None
        y = finalize(o, pair_pos, weights, tokens, k)
        if extra is not None:
            y = y + extra
        return y + residual if residual is not None else y
    if fused is not None:
        return fused.moe_combine(o, pair_pos, weights, tokens, k, extra, residual)
    d = o.shape[1]
    y = torch.empty((tokens, d), dtype=o.dtype, device=o.device)
    _lib.check(_lib.lib().zb_moe_combine(o.data_ptr(), pair_pos.data_ptr(), weights.data_ptr(),
                                         extra.data_ptr() if extra is not None else None,
                                         residual.data_ptr() if residual is not None else None, y.data_ptr(), tokens, k, d,
                                         None, 0, 0, _lib.stream_ptr()), "zb_moe_combine")
    return y


# ---------------------------------------------------------------------- fused experts
W4_MAX_AVG_TOKENS = 32      # NVFP4 kernel: tiles of at most 64 tokens per expert


FP4_MAX_AVG_TOKENS = 128


def fp4_activations() -> bool:
    """NVFP4 expert weights are multiplied with NVFP4 activations on the block-scaled tensor-core path (`ZB_MOE_FP4=a4`,
    the default) or with bf16 activations after de-quantising the weights inside the kernel (`ZB_MOE_FP4=a16`)."""
    import os
    return os.environ.get("ZB_MOE_FP4", "a4") != "a16"


def fused_experts(x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, w_gate_up_il: torch.Tensor,
                  w_down: torch.Tensor, e0: int = 0, num_experts_total: Optional[int] = None,
                  w4: Optional[tuple] = None, extra=None, residual=None, fused=None, activation: str = "swiglu") -> torch.Tensor:
    """Mixture output of the LOCAL experts for all tokens: permute -> grouped GEMM (+ `activation`: swiglu | geglu |
    geglu_tanh on an interleaved gate|up weight, relu2 on a plain up projection [E_local, F, D]) ->
    grouped GEMM -> un-permute x routing weight.  x [T, D] bf16; w_gate_up_il [E_local, 2F, D]
    (interleaved, see `interleave_gate_up`); w_down [E_local, D, F].  `extra`, `residual` and `fused`
    go to `combine`: with `fused` the result is the sum over the expert-parallel group."""
    t, d = x.shape
    k = topk_ids.shape[1]
    e_local = w_gate_up_il.shape[0]
    total_e = num_experts_total or e_local
    cap = t * k
    avg = max(1, (t * k) // max(total_e, 1))
    meta, sorted_pair, pair_pos = moe_align(topk_ids, e0, e_local)
    if w4 is not None and fp4_activations() and avg <= FP4_MAX_AVG_TOKENS and w4[0].kernel_ready and w4[1].kernel_ready:
        # NVFP4 on both sides: the gather quantises the activations, the gate|up GEMM applies SwiGLU and quantises its
        # output, and both GEMMs run on the block-scaled tensor-core instruction.  Up to FP4_MAX_AVG_TOKENS per expert:
        # with 128 x 128 tiles the kernel is bound by operand traffic into shared memory, and at prefill sizes the
        # bf16 grouped GEMM on de-quantised weights is faster (787 against 559 TFLOP/s at 512 tokens per expert)
        xq = gather_fp4(x, sorted_pair, meta, e_local, k, cap)
        hq = grouped_gemm_fp4(xq, w4[0], meta, swiglu=activation, avg_tokens=avg, quantize_out=activation != "relu2")
        o = grouped_gemm_fp4(hq, w4[1], meta, swiglu=False, avg_tokens=avg)
        if extra is None and residual is None and fused is None:
            return finalize(o, pair_pos, topk_w, t, k)
        return combine(o, pair_pos, topk_w, t, k, extra, residual, fused)
    xs = gather(x, sorted_pair, meta, e_local, k, cap)
    if w4 is not None and avg <= W4_MAX_AVG_TOKENS and w4[0].kernel_ready and w4[1].kernel_ready:
        # few tokens per expert: the step is bound by reading expert weights - read them as NVFP4
        h = grouped_gemm_w4(xs, w4[0], meta, swiglu=activation, avg_tokens=avg)
        o = grouped_gemm_w4(h, w4[1], meta, swiglu=False, avg_tokens=avg)
    else:
        h = grouped_gemm(xs, w_gate_up_il, meta, swiglu=activation, avg_tokens=avg)
        o = grouped_gemm(h, w_down, meta, swiglu=False, avg_tokens=avg)
    if extra is None and residual is None and fused is None:
        return finalize(o, pair_pos, topk_w, t, k)
    return combine(o, pair_pos, topk_w, t, k, extra, residual, fused)


def reference_fused_experts(x, topk_ids, topk_w, gate, up, down, e0: int = 0):
    """Oracle: for every token, sum over its experts that are local (dense per-expert matmuls in f32)."""
    t, d = x.shape
    y = torch.zeros((t, d), dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(gate.shape[0]):
        sel = (topk_ids == (e + e0))
        tok = sel.any(1).nonzero()[:, 0]
        if tok.numel() == 0:
            continue
        w = (topk_w.float() * sel).sum(1)[tok]
        h = torch.nn.functional.silu(xf[tok] @ gate[e].float().t()) * (xf[tok] @ up[e].float().t())
        h = h.to(x.dtype).float()
        y[tok] += w[:, None] * (h @ down[e].float().t()).to(x.dtype).float()
    return y.to(x.dtype)


def library_experts(x, topk_ids, topk_w, w_gate_up_il, w_down, e0: int = 0):
    """Comparison path built from library pieces only: torch sort / gather for the permutation,
    the library grouped GEMM (`torch._grouped_mm`) for both expert GEMMs, unfused SwiGLU, and an
    index_add for the weighted combine.  No host synchronisation, so it can be graph-captured."""
    t, d = x.shape
    k = topk_ids.shape[1]
    e_local = w_gate_up_il.shape[0]
    flat = topk_ids.reshape(-1).long() - e0
    local = (flat >= 0) & (flat < e_local)
    key = torch.where(local, flat, torch.full_like(flat, e_local))        # foreign pairs sort last
    order = torch.argsort(key, stable=True)
    counts = (key[:, None] == torch.arange(e_local, device=x.device)[None, :]).sum(0)
    offs = torch.cumsum(counts, 0).to(torch.int32)
    tok = torch.div(order, k, rounding_mode="floor")
    xs = x[tok]                                                            # [T*k, D]; rows past offs[-1] unused
    h = torch._grouped_mm(xs, w_gate_up_il.transpose(-2, -1), offs=offs)
    f2 = h.shape[1]
    h = h.reshape(-1, f2 // 128, 2, 64)
    h = (torch.nn.functional.silu(h[:, :, 0].float()) * h[:, :, 1].float()).to(x.dtype).reshape(-1, f2 // 2)
    o = torch._grouped_mm(h, w_down.transpose(-2, -1), offs=offs)
    w = (topk_w.reshape(-1).float() * local.float())[order]
    valid = (torch.arange(t * k, device=x.device) < offs[-1]).float()
    y = torch.zeros((t, d), dtype=torch.float32, device=x.device)
    y.index_add_(0, tok, torch.nan_to_num(o.float()) * (w * valid)[:, None])
    return y.to(x.dtype)


def forward_moe(x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, comm=None, num_experts_total: Optional[int] = None, residual=None,
                extra_partial=None, w4: Optional[tuple] = None):
    """Routed mixture with expert parallelism.  `w_gate_up` / `w_down` hold this rank's experts
    (rank r owns experts [r * E_local, (r + 1) * E_local)); partial outputs are summed across
    ranks (in-kernel over peer memory when `comm.fused` is set, NCCL otherwise) and `residual`
    is added once.  `extra_partial` is another per-rank partial sum (a tensor-parallel shared
    expert) that rides on the same all-reduce."""
    e_local = w_gate_up.shape[0]
    world = comm.world if comm is not None else 1
    rank = comm.rank if comm is not None else 0
    from ..ops import baseline as _baseline
    if _baseline.enabled():
        y = library_experts(x, topk_ids, topk_weights, w_gate_up, w_down, rank * e_local)
        if extra_partial is not None:
            y = y + extra_partial
        if world > 1:
            y = comm.all_reduce_(y)
        return y + residual if residual is not None else y
    total = num_experts_total or e_local * world
    fused_ctx = getattr(comm, "fused", None) if world > 1 else None
    if world == 1 and x.is_cuda and x.dtype == torch.bfloat16:
        return fused_experts(x, topk_ids, topk_weights, w_gate_up, w_down, 0, total, w4, extra=extra_partial, residual=residual)
    if fused_ctx is not None and x.is_cuda and x.dtype == torch.bfloat16 and fused_ctx.can_combine(x.shape[0], x.shape[1]):
        return fused_experts(x, topk_ids, topk_weights, w_gate_up, w_down, rank * e_local, total, w4, extra=extra_partial,
                             residual=residual, fused=fused_ctx)
    y = fused_experts(x, topk_ids, topk_weights, w_gate_up, w_down, rank * e_local, total, w4)
    if extra_partial is not None:
        y = y + extra_partial
    if world > 1:
        fz = getattr(comm, "fused", None)
        if fz is not None and y.is_cuda and y.dim() == 2 and fz.can_all_reduce_mm(y.shape[0], y.shape[1]):
            # prefill-sized: the partial outputs go through the symmetric heap and are added up inside NVSwitch
            # (multimem load-reduce), the residual rides along
            part = fz.partial_buffer(y.shape[0], y.shape[1])
            part.copy_(y)
            return fz.all_reduce_mm(part, residual)
        if fz is not None and y.is_cuda and fz.staging is not None and y.numel() <= fz.staging.numel():
            y = fz.all_reduce(y)
        else:
            y = comm.all_reduce_(y)
    if residual is not None:
        y = y + residual
    return y
