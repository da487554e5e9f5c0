"""The Qwen2 / Qwen2.5 dense decoder as a `ModelSpec`.

Every layer is a pre-norm block of grouped-query attention (q, k, v with bias, rotary encoding,
no output bias) and a SwiGLU feed-forward, with RMSNorm before each
(tensorline/paged.py:245-276); the final RMSNorm and an output head that may share the
embedding table follow (paged.py:285-287).  Tensor names are the checkpoint's
(tensorline/paged.py:177-188, tensorline/quant.py:25).  With `use_sliding_window`, the layers
from `max_window_layers` on attend to the last `sliding_window` keys only.
"""
from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..parts import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry


def describe_qwen2(cfg: Qwen2Config) -> ModelSpec:
    norm = PartSpec("rms_norm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    ff = PartSpec("gated_mlp", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size,
                                "activation": cfg.hidden_act})
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec("paged_attention", {
            "hidden": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "qkv_bias": True,
            "window": cfg.layer_window(i),
            "position": PartSpec("rotary_half", {"theta": cfg.rope_theta}),
        })
        block = PartSpec("pre_norm", {"mixer": mixer, "feed_forward": ff, "norm1": norm, "norm2": norm})
        layers.append(LayerSpec(block, f"model.layers.{i}"))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=tuple(layers),
        run=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)), final_norm=norm,
        tie_word_embeddings=cfg.tie_word_embeddings, eos_token_id=cfg.eos_token_id,
        max_position_embeddings=cfg.max_position_embeddings)
