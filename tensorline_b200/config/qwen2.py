"""`Qwen2Config`: the config.json of a Qwen2 / Qwen2.5 dense decoder, typed and validated.

tzar-beep/Tensorline reads these values off the loaded model object
(tensorline/paged.py:113-119, :134-137; tensorline/manager.py:48-54, :65); here they come
straight from config.json.  Keys the engine cannot honour are rejected by name instead of
being ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class Qwen2Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    hidden_act: str
    use_sliding_window: bool
    sliding_window: int | None
    max_window_layers: int
    eos_token_id: int | None
    torch_dtype: str | None

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "Qwen2Config":
        r = ConfigReader(raw, where)
        arch = raw.get("architectures", ["Qwen2ForCausalLM"])[0]
        hidden = r.int("hidden_size", min=1)
        nq = r.int("num_attention_heads", min=1)
        nkv = r.int("num_key_value_heads", nq, min=1)
        head_dim = r.int("head_dim", None, min=1)
        if head_dim is None:                                  # tensorline/manager.py:50
            if hidden % nq:
                raise ConfigError(f"{where}: 'hidden_size' {hidden} is not a multiple of "
                                  f"'num_attention_heads' {nq} and no 'head_dim' is given")
            head_dim = hidden // nq
        layers = r.int("num_hidden_layers", min=1)
        theta = r.float("rope_theta", None, positive=True)
        rope_params = r.any("rope_parameters")
        if isinstance(rope_params, dict):                     # newer files nest the rotary keys
            if theta is None and rope_params.get("rope_theta") is not None:
                theta = float(rope_params["rope_theta"])
            kind = rope_params.get("rope_type", rope_params.get("type", "default"))
            if kind not in (None, "default"):
                raise ConfigError(f"{where}: 'rope_parameters.rope_type' = {kind!r} is not supported "
                                  "(only the default rotary table)")
        scaling = r.any("rope_scaling")
        if scaling not in (None, {}):
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                raise ConfigError(f"{where}: 'rope_scaling' = {scaling!r} is not supported")
        eos = r.any("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int)):
            raise ConfigError(f"{where}: 'eos_token_id' must be an integer, got {eos!r}")
        cfg = cls(
            architecture=arch,
            vocab_size=r.int("vocab_size", min=1),
            hidden_size=hidden,
            intermediate_size=r.int("intermediate_size", min=1),
            num_hidden_layers=layers,
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            rms_norm_eps=r.float("rms_norm_eps", 1e-6, positive=True),
            rope_theta=10000.0 if theta is None else theta,
            tie_word_embeddings=r.bool("tie_word_embeddings", False),
            max_position_embeddings=r.int("max_position_embeddings", 32768, min=1),
            hidden_act=r.str("hidden_act", "silu"),
            use_sliding_window=r.bool("use_sliding_window", False),
            sliding_window=r.int("sliding_window", None, min=1),
            max_window_layers=r.int("max_window_layers", layers, min=0),
            eos_token_id=eos,
            torch_dtype=r.str("torch_dtype", None) or r.str("dtype", None),
        )
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config.json") -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{where}: 'num_attention_heads' {self.num_attention_heads} is not a multiple "
                              f"of 'num_key_value_heads' {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"{where}: 'head_dim' {self.head_dim} must be even for rotary pairs")
        if self.hidden_act != "silu":
            raise ConfigError(f"{where}: 'hidden_act' = {self.hidden_act!r}; this architecture runs 'silu' only")
        if self.use_sliding_window and self.sliding_window is None:
            raise ConfigError(f"{where}: 'use_sliding_window' is true but 'sliding_window' is missing")

    # ------------------------------------------------------------------ derived
    def layer_window(self, layer: int) -> int | None:
        """Window of a layer's attention, or None for all keys: with `use_sliding_window`,
        the layers with index >= `max_window_layers` see the last `sliding_window` keys."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_json_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "qwen2"
        if d["torch_dtype"] is None:
            d.pop("torch_dtype")
        return d

    def num_parameters(self) -> int:
        H, I, V, d = self.hidden_size, self.intermediate_size, self.vocab_size, self.head_dim
        nq, nkv = self.num_attention_heads, self.num_key_value_heads
        per_layer = (nq + 2 * nkv) * d * (H + 1) + nq * d * H + 3 * H * I + 2 * H
        return self.num_hidden_layers * per_layer + V * H * (1 if self.tie_word_embeddings else 2) + H
