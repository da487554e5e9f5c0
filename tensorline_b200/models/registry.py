"""The one registry from an architecture's name (config.json `architectures[0]`) to its model.

An entry is (configuration class, describe function): the class parses config.json into a typed
configuration, `describe(config)` turns it into a `ModelSpec`.  Another architecture is one more
`register_architecture` call; the engine above never names an architecture.
tzar-beep/Tensorline leaves this choice to an installed package (tensorline/engine.py:66).
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from ..config.base import ConfigError, architecture_name, read_config_json
from ..config.qwen2 import Qwen2Config
from ..parts import Runtime
from ..weights import load_weights
from .qwen2 import describe_qwen2
from .spec import Model


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    describe: callable


_ARCHITECTURES: dict = {}


def register_architecture(name: str, config_class, describe) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, describe)


def architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; known: {sorted(_ARCHITECTURES)}")
    return _ARCHITECTURES[name]


def registered_architectures() -> list:
    return sorted(_ARCHITECTURES)


register_architecture("Qwen2ForCausalLM", Qwen2Config, describe_qwen2)


def load_config(folder):
    """(architecture, typed configuration) of a model folder."""
    raw = read_config_json(folder)
    arch = architecture(architecture_name(raw))
    return arch, arch.config_class.from_dict(raw, where=str(Path(folder) / "config.json"))


def build_model(config, rt: Runtime, architecture_name_: str | None = None) -> Model:
    arch = architecture(architecture_name_ or config.architecture)
    return Model(arch.describe(config), rt)


def load_model(folder, rt: Runtime):
    """Model of `folder` on the device with its weights bound; returns (model, config)."""
    arch, cfg = load_config(folder)
    model = Model(arch.describe(cfg), rt)
    expected = model.expected_tensors()
    if model.spec.tie_word_embeddings:
        # A tied head is the embedding table: a stored head is neither loaded nor an error.
        head = f"{model.spec.head_prefix}.weight"
        expected = {k: v for k, v in expected.items() if k != head}
        weights = load_weights(folder, expected, device=rt.device, ignore=(head,))
    else:
        weights = load_weights(folder, expected, device=rt.device)
    model.bind(weights)
    return model, cfg


def expected_tensors(config) -> dict:
    """Names and shapes of a configuration's tensors, without touching a device."""
    rt = Runtime(torch.device("cpu"), torch.float32)
    return build_model(config, rt).expected_tensors()
