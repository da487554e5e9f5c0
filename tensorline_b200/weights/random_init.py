"""Random weights: write a model folder (config.json, model.safetensors) from a configuration
and a seed.

Every weight and bias is drawn from N(0, std); tensors whose part declares them as scales
around one (`TensorSpec.init == "ones"`: norm weights) are 1, or 1 + N(0, norm_std).
Values are generated tensor by tensor with a generator seeded from (seed, tensor name), so a
tensor's values depend neither on the order of generation nor on what else the model holds.
They are stored in bfloat16 (or float32 on request), as published checkpoints of this
architecture are; every reader of the folder sees the same numbers.  tzar-beep/Tensorline has
no generator of its own (its tests download tiny random models, tests/test_batching.py:13).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .safetensors_io import write_safetensors


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest, "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensor(seed: int, name: str, shape, std: float, mean: float = 0.0) -> torch.Tensor:
    t = torch.empty(tuple(shape), dtype=torch.float32)
    if std > 0:
        t.normal_(mean, std, generator=_generator(seed, name))
    else:
        t.fill_(mean)
    return t


def write_random_model(folder, config, expected: dict, *, seed: int = 0, std: float = 0.02,
                       norm_std: float = 0.0, store_dtype: torch.dtype = torch.bfloat16) -> Path:
    """`config`: a typed configuration with `to_json_dict()`; `expected`: name -> TensorSpec
    as the model declares them.  Optional tensors are not written."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = {}
    for name, spec in expected.items():
        if spec.optional:
            continue
        if spec.kind == "int":
            raise ValueError(f"'{name}': no rule to draw an integer table")
        if spec.init == "ones":
            t = random_tensor(seed, name, spec.shape, norm_std, 1.0)
        elif spec.init == "zeros":
            t = torch.zeros(tuple(spec.shape), dtype=torch.float32)
        else:
            t = random_tensor(seed, name, spec.shape, std)
        tensors[name] = t.to(store_dtype)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "seed": seed})
    (folder / "config.json").write_text(json.dumps(config.to_json_dict(), indent=1))
    return folder
