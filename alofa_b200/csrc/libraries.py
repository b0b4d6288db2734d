"""The list of every native library of the package, for building ahead of use."""
from __future__ import annotations


def all_libraries() -> list:
    """Keyword dicts of :func:`alofa_b200.csrc.build.compile_library`."""
    return [
        {"name": "alofa_cache_manager", "sources": ["host/cache_manager.cpp"], "cuda": False},
        {"name": "alofa_scheduler", "sources": ["host/scheduler.cpp"], "cuda": False},
        {"name": "alofa_generic", "sources": ["kernels/generic.cu"]},
        {"name": "alofa_sampling", "sources": ["kernels/sampling.cu"]},
        {"name": "alofa_gemm_tc", "sources": ["kernels/gemm_tc.cu"]},
        {"name": "alofa_elementwise_bf16", "sources": ["kernels/elementwise_bf16.cu"]},
        *[{"name": f"alofa_attention_hd{hd}", "sources": ["kernels/attention_bf16.cu"], "defines": {"HEAD_DIM": hd}} for hd in (16, 32, 48, 64, 128)],
    ]
