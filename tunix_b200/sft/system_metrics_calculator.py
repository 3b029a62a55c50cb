"""Step FLOPs estimates (tunix/sft/system_metrics_calculator.py:23-76): 6 * params * tokens / dt."""
from __future__ import annotations


def approximate_tflops_per_step(num_params: int, tokens_per_step: int, step_time_s: float) -> float:
    if step_time_s <= 0:
        return 0.0
    return 6.0 * num_params * tokens_per_step / step_time_s / 1e12


def transformer_flops_per_token(cfg, seq_len: int, backward: bool = True) -> float:
    """Dense matmul FLOPs per token including causal attention (2 * T/2 * D_attn per matmul)."""
    D, N, K, H = cfg.embed_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    attn_proj = 2 * D * (N * H) * 2 + 2 * D * (K * H) * 2
    if cfg.is_moe:
        mlp = 2 * 3 * D * cfg.moe_hidden_dim * cfg.num_experts_per_tok + 2 * D * cfg.num_experts
    else:
        mlp = 2 * 3 * D * cfg.hidden_dim
    attn = 2 * 2 * N * H * (seq_len / 2)
    per_layer = attn_proj + mlp + attn
    total = cfg.num_layers * per_layer + 2 * D * cfg.vocab_size
    return total * (3.0 if backward else 1.0)
