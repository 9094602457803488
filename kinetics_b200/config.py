"""Model-shape configs for the decoder-layer benchmarks.

The reference reads ``transformers.AutoConfig.from_pretrained(args.model)``
(benchmark/blocktopk.py:65); the shapes below are the public Qwen3 ones, so the layers can be
built without network access.  Any object with the same attributes (an HF config) works too.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class LayerConfig:
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    num_hidden_layers: int
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    hidden_act: str = "silu"
    rope_theta: float = 1e6
    max_position_embeddings: int = 40960
    eos_token_id: int = 151645
    vocab_size: int = 151936


PRESETS = {
    "Qwen3-8B": LayerConfig(4096, 32, 8, 12288, 36),
    "Qwen3-32B": LayerConfig(5120, 64, 8, 25600, 64),
    "Qwen3-1.7B": LayerConfig(2048, 16, 8, 6144, 28),
    # the attention shape of the CPU-runnable case (one KV head, four query heads) inside a small layer
    "cfg1": LayerConfig(512, 4, 1, 1024, 1),
}


def get_config(name: str) -> LayerConfig:
    """`Qwen/Qwen3-8B` or `Qwen3-8B` -> LayerConfig."""
    key = name.split("/")[-1]
    if key not in PRESETS:
        raise KeyError(f"unknown model {name!r}; known: {sorted(PRESETS)}")
    return PRESETS[key]
