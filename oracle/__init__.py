"""CPU oracle for the MoE routing / dispatch hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module;
only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may call it, and only as the checker (or as the timed CPU arm), never as a
stand-in for a CUDA kernel.

Every function restates, in numpy / CPU-torch, the algorithm of one piece of
santiweide/moe-routers; the docstrings cite the reference file and lines they
follow.  Parity status: the routers, the pack and the MoE block are pinned by
golden vectors produced by importing the reference's own Python classes
(tests/golden/make_golden.py).  The grouped expert GEMM arithmetic of the
reference lives in CUTLASS (an empty, un-pinned submodule: third_party/cutlass)
and the reference holds no test for it: for that piece the oracle is an fp32
matmul rounded to fp16 and its parity is "unpinned".
"""
from .routing import (  # noqa: F401
    router_logits,
    topk_select,
    fused_select_gates,
    counts_offsets,
    pack_canonical,
    fused_select_forward,
    sinkhorn_assign,
    sinkhorn_route,
    combine,
    load_skew,
)
from .experts import (  # noqa: F401
    gelu_ffn,
    swiglu_ffn,
    grouped_gemm,
    moe_layer,
    masked_matmul_layer,
    ep_owner,
    ep_send_splits,
    ep_layer,
)
