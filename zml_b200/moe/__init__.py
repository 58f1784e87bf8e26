"""Mixture of experts (zml/moe/* of the reference): router, fused experts, expert parallelism.

`forward_moe` has the reference's contract (zml/moe/moe.zig:186-302): given the input
activations, the top-k expert ids and weights of every token, and the stacked expert
weights, it returns the mixture output; when the experts are partitioned over ranks
(`comm.world > 1`) each rank runs its local experts and the partial outputs are summed
across ranks.  The B200 path differs from the reference in what it computes: only the
(token, expert) pairs routed to a local expert are gathered and multiplied (the reference
runs every token through the local experts with masked weights), the gate/up projection
and SwiGLU are one grouped tcgen05 GEMM, and the cross-rank sum is done from inside a
kernel over NVLink peer memory when symmetric memory is set up.
"""
from .ops import (Backend, Fp4Activations, Nvfp4Experts, combine, fp4_activations, gather_fp4, grouped_gemm_fp4, grouped_gemm_w4, deinterleave_gate_up, finalize, forward_moe, fused_experts, gather, grouped_gemm, interleave_gate_up,  # noqa: F401
                  nvfp4_roundtrip,
                  moe_align, reference_fused_experts, router_topk)
