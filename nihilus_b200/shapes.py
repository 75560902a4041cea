"""LLaMA-3-8B projection shapes (reference: include/nihilus-incl/infra/model_traits.hpp:49-65,
weight dims infra/core_traits.hpp:145-182) and the algorithmic work of a Q8_0 mul_mat."""
from __future__ import annotations

E, FF, KV, V, L = 4096, 14336, 1024, 128256, 32

# name -> (N rows, K)
LLAMA3_8B = {
    "attn_q": (E, E),
    "attn_k": (KV, E),
    "attn_v": (KV, E),
    "attn_output": (E, E),
    "ffn_gate": (FF, E),
    "ffn_up": (FF, E),
    "ffn_down": (E, FF),
    "output": (V, E),
}

# per layer, in execution order; each inner tuple shares one input activation and has no internal dependency
LAYER_STAGES = (("attn_q", "attn_k", "attn_v"), ("attn_output",), ("ffn_gate", "ffn_up"), ("ffn_down",))


def mul_mat_bytes(N: int, K: int, M: int = 1) -> int:
    """Weights once as 34-byte Q8_0 blocks + f32 activations in + f32 outputs out."""
    return N * (K // 32) * 34 + 4 * M * K + 4 * M * N


def mul_mat_flops(N: int, K: int, M: int = 1) -> int:
    return 2 * M * N * K


def decode_set(layers: int = L, lm_head: bool = True):
    """The full per-token matmul list: `layers` x 7 projections (+ lm_head) as (name, layer, N, K)."""
    out = []
    for layer in range(layers):
        for stage in LAYER_STAGES:
            for name in stage:
                n, k = LLAMA3_8B[name]
                out.append((name, layer, n, k))
    if lm_head:
        n, k = LLAMA3_8B["output"]
        out.append(("output", -1, n, k))
    return out
