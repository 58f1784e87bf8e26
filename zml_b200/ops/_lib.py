"""ctypes binding of ``libzb_cuda.so`` (the hand-written sm_100a kernels).

The library exports a plain C ABI: raw device pointers, sizes and a stream
handle.  On a machine with a GPU the library MUST load - an op never falls back
to PyTorch silently; `lib()` raises instead.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB = None
# ZB_CUDA_LIB: path of another build of the library (kernel experiments: same ABI, different code)
_PATH = Path(os.environ["ZB_CUDA_LIB"]) if os.environ.get("ZB_CUDA_LIB") else \
    Path(__file__).resolve().parent.parent / "_C" / "libzb_cuda.so"

c_p = C.c_void_p
c_i = C.c_int
c_ll = C.c_longlong
c_f = C.c_float
c_sz = C.c_size_t
c_ull = C.c_ulonglong


class KernelError(RuntimeError):
    """A kernel of libzb_cuda.so returned a non-zero code or recorded a device status."""


class CollectiveTimeout(KernelError):
    """A bounded device-side wait (on an mbarrier, a flag or a peer) ran out.  The kernel returned
    cleanly and the CUDA context is still usable; `kernel`, `phase` and `detail` say where it gave up."""

    def __init__(self, msg: str, kernel: str = "", phase: int = 0, detail: int = 0, rank: int = 0):
        super().__init__(msg)
        self.kernel, self.phase, self.detail, self.rank = kernel, phase, detail, rank


_SIGS = {
    "zb_init": (c_i, [c_i]),
    "zb_num_sms": (c_i, []),
    "zb_status_read": (c_i, [c_p]),
    "zb_status_reset": (c_i, []),
    "zb_status_ptr": (c_p, []),
    "zb_bc_enabled": (c_i, []),
    "zb_bc_set_extents": (c_i, [c_ll, c_ll]),
    "zb_launch_count": (c_ull, []),
    "zb_launch_count_reset": (None, []),
    "zb_launch_count_add": (None, [c_ull]),
    "zb_moe_grouped_gemm_w4": (c_i, [c_p, c_p, c_p, c_i, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p]),
    "zb_moe_grouped_gemm_fp4": (c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p]),
    "zb_moe_gather_fp4": (c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p]),
    "zb_allreduce_ll": (c_i, [c_p, c_p, c_p, c_p, C.c_longlong, c_sz, c_sz, c_p]),
    "zb_argmax_tp": (c_i, [c_p, c_p, c_p, c_i, c_i, c_ll, c_i, c_sz, c_p]),
    "zb_argmax_tp_slot_bytes": (c_sz, [c_i]),
    "zb_moe_combine": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_sz, c_sz, c_p]),
    "zb_wait_probe": (c_i, [c_p, C.c_uint, c_ull, C.c_uint, c_p, c_p]),
    "zb_decode_advance": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p]),
    "zb_moe_w4_set_timeline": (None, [c_p]),
    "zb_gemm_describe_plan": (c_i, [c_i, c_i, c_i, c_p]),
    "zb_gemm_cluster_capacity": (c_i, [c_i, c_i]),
    "zb_gemm_plan": (c_i, [c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_p]),
    "zb_gemm_workspace_bytes": (c_sz, [c_i, c_i, c_i, c_i]),
    "zb_gemm_bf16": (c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p]),
    "zb_gemm_bf16_ex": (c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i,
                              c_p, c_sz, c_p, c_i, c_p, c_i, c_p]),
    "zb_gemm_bf16_epi": (c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_i, c_i, c_f, c_f,
                               c_i, c_p, c_i, c_p, c_p, c_ull, c_p]),
    "zb_gemm_scratch_needed": (c_sz, [c_i, c_i, c_i, c_i]),
    "zb_row_sumsq": (c_i, [c_p, c_i, c_i, c_ll, c_p, c_p]),
    "zb_rmsnorm": (c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_ll, c_ll, c_f, c_i, c_p]),
    "zb_rope_kvwrite": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_ll, c_i, c_i, c_i, c_i,
                              c_i, c_i, c_i, c_ll, c_f, c_f, c_i, c_p]),
    "zb_swiglu": (c_i, [c_p, c_p, c_ll, c_i, c_p]),
    "zb_embedding": (c_i, [c_p, c_p, c_p, c_i, c_i, c_i, c_p]),
    "zb_argmax_f32": (c_i, [c_p, c_p, c_i, c_i, c_ll, c_p]),
    "zb_topk_sample": (c_i, [c_p, c_p, c_p, c_p, c_i, c_i, c_ll, c_i, c_f, c_ull, c_ull, c_p]),
    "zb_topk_sample_rng": (c_i, [c_p, c_p, c_p, c_p, c_i, c_i, c_ll, c_i, c_f, c_ull, c_ull, c_p, c_p]),
    "zb_u64_add": (c_i, [c_p, c_ull, c_p]),
    "zb_decode_advance_rng": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_p]),
    "zb_decode_plan_splits": (c_i, [c_i, c_i, c_i, c_i]),
    "zb_decode_scratch_bytes": (c_sz, [c_i, c_i, c_i, c_i]),
    "zb_paged_decode": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_ll, c_f,
                              c_i, c_i, c_p]),
    "zb_paged_prefill_tc_supported": (c_i, [c_i, c_i, c_i, c_i]),
    "zb_paged_prefill_tc": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_ll, c_f, c_i,
                                  C.c_uint, C.c_uint, c_p]),
    "zb_paged_prefill": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i,
                               c_ll, c_f, c_i, c_p]),
}

# Symbols added by later source files; bound only if the library exports them.
_OPTIONAL_SIGS: dict[str, tuple] = {}


def register_signature(name: str, restype, argtypes, optional: bool = True) -> None:
    """Lets other modules of the package declare the C signature of their entry points."""
    (_OPTIONAL_SIGS if optional else _SIGS)[name] = (restype, argtypes)
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.restype, fn.argtypes = restype, argtypes


def available() -> bool:
    return _PATH.exists()


def path() -> Path:
    return _PATH


def lib():
    """Loads the library once.  Raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _PATH.exists():
        if os.environ.get("ZB_AUTOBUILD", "1") != "0":
            from .. import _build
            _build.build_cuda()
    if not _PATH.exists():
        raise KernelError(
            f"{_PATH} is missing: run `python -m zml_b200._build` (needs nvcc); "
            "ops on CUDA tensors never fall back to PyTorch")
    l = C.CDLL(str(_PATH))
    for name, (res, args) in _SIGS.items():
        fn = getattr(l, name)
        fn.restype, fn.argtypes = res, args
    for name, (res, args) in _OPTIONAL_SIGS.items():
        if hasattr(l, name):
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
    _LIB = l
    return l


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "flag wait timed out",
                3: "index out of bounds", 4: "bad argument"}
KERNEL_NAMES = {1: "gemm_bf16", 2: "paged_decode", 3: "paged_prefill", 4: "gemm_ar_fused",
                5: "comm_barrier", 6: "moe_grouped_gemm", 7: "moe_a2a", 8: "wait_probe", 9: "moe_grouped_gemm_w4",
                10: "moe_combine", 11: "allreduce_ll", 12: "allreduce_mm", 13: "paged_prefill_tc", 14: "gemm_2cta", 15: "argmax_tp",
                20: "rope_kvwrite", 21: "embedding", 22: "decode_advance", 24: "causal_conv1d", 25: "gated_delta_scan"}


class BoundsError(KernelError):
    """The bounds-checking build of the library saw an index outside its extent (`kernel`, `site`, `index`); the
    access was skipped."""

    def __init__(self, msg: str, kernel: str, site: int, index: int):
        super().__init__(msg)
        self.kernel, self.site, self.index = kernel, site, index


def bounds_check_build() -> bool:
    """True when the loaded library is the bounds-checking build (`ZB_CUDA_LIB=.../libzb_cuda_bc.so`)."""
    return bool(lib().zb_bc_enabled())


def set_bounds_extents(num_pages: int = 0, num_state_slots: int = 0) -> None:
    """Declares the extents that kernel arguments do not carry (checked by the bounds-checking build only)."""
    check(lib().zb_bc_set_extents(int(num_pages), int(num_state_slots)), "zb_bc_set_extents")


def read_status() -> tuple[int, int, int, int]:
    """Synchronises the device and returns (code, kernel, where, detail)."""
    buf = (C.c_uint32 * 4)()
    check(lib().zb_status_read(C.cast(buf, c_p)), "zb_status_read")
    return tuple(int(v) for v in buf)  # type: ignore[return-value]


def raise_on_status() -> None:
    """Raises KernelError if any kernel recorded a failure since the last reset."""
    code, kernel, where, detail = read_status()
    if code != 0:
        lib().zb_status_reset()
        msg = (f"device status: {STATUS_NAMES.get(code, code)} in kernel "
               f"{KERNEL_NAMES.get(kernel, kernel)} (where={where}, detail={detail})")
        if code in (1, 2):
            import os
            raise CollectiveTimeout(msg, str(KERNEL_NAMES.get(kernel, kernel)), where, detail,
                                    int(os.environ.get("RANK", "0")))
        if code == 3:
            raise BoundsError(msg, str(KERNEL_NAMES.get(kernel, kernel)), where, detail if detail < 2 ** 31 else detail - 2 ** 32)
        raise KernelError(msg)


def stream_ptr(stream=None) -> int:
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


def launch_count() -> int:
    return int(lib().zb_launch_count())
