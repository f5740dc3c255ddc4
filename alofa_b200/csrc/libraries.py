"""The list of every native library of the package, for building ahead of use."""
from __future__ import annotations


def all_libraries() -> list:
    """Keyword dicts of :func:`alofa_b200.csrc.build.compile_library`."""
    return [
        {"name": "alofa_cache_manager", "sources": ["host/cache_manager.cpp"], "cuda": False},
        {"name": "alofa_scheduler", "sources": ["host/scheduler.cpp"], "cuda": False},
        {"name": "alofa_generic", "sources": ["kernels/generic.cu"]},
        {"name": "alofa_latent", "sources": ["kernels/latent.cu", "kernels/gemm_batched_bf16.cu"]},
        {"name": "alofa_recurrent", "sources": ["kernels/recurrent.cu"]},
        {"name": "alofa_delta", "sources": ["kernels/delta.cu"]},
        {"name": "alofa_gated_lru", "sources": ["kernels/gated_lru.cu"]},
        {"name": "alofa_hyper", "sources": ["kernels/hyper.cu"]},
        {"name": "alofa_sampling", "sources": ["kernels/sampling.cu"]},
        {"name": "alofa_gemm_tc", "sources": ["kernels/gemm_tc.cu"]},
        {"name": "alofa_elementwise_bf16", "sources": ["kernels/elementwise_bf16.cu"]},
        # latent attention on tensor cores is built per latent size at first use; the size of the tests' model is built ahead
        {"name": "alofa_latent_attention_kv64_r32", "sources": ["kernels/latent_attention_bf16.cu"], "defines": {"KV_RANK": 64, "ROT": 32}},
        {"name": "alofa_latent_attention_kv96_r16", "sources": ["kernels/latent_attention_bf16.cu"], "defines": {"KV_RANK": 96, "ROT": 16}},
        *[{"name": f"alofa_attention_hd{hd}", "sources": ["kernels/attention_bf16.cu"], "defines": {"HEAD_DIM": hd}} for hd in (16, 32, 48, 64, 80, 96, 128)],
        # the build whose scores are capped (softcap * tanh(score / softcap)), likewise per head size at first use; two sizes ahead
        *[{"name": f"alofa_attention_hd{hd}_cap", "sources": ["kernels/attention_bf16.cu"], "defines": {"HEAD_DIM": hd, "SOFTCAP": 1}} for hd in (64, 128)],
    ]
