"""Loading weights by tensor name.

The model says which tensors it expects (`name -> TensorSpec`); the loader opens
`model.safetensors` (or the shards named by `model.safetensors.index.json`), compares names and
shapes, and raises ONE `WeightError` that lists every missing tensor, every unexpected tensor
and every wrong shape.  Tensors keep the type they are stored in: bfloat16 stays bfloat16, a
tensor stored in 32 bits stays 32-bit, integer tables become int32.  Widening for the 32-bit
engine, or narrowing a 32-bit matrix for the bfloat16 kernels, is the business of the part that
owns the tensor, not of the loader.

tzar-beep/Tensorline delegates all of this to an installed package
(tensorline/engine.py:63-66); the tensor names are those of its projections
(tensorline/paged.py:177-188, tensorline/quant.py:25).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The weights in the folder are not the ones the model expects."""


@dataclass(frozen=True)
class TensorSpec:
    shape: tuple
    kind: str = "float"           # "float" (bfloat16 / float16 / float32 as stored) or "int"
    optional: bool = False        # absent is fine (e.g. an output head that is tied)
    init: str = "normal"          # how a random model draws it: "normal" N(0, std), "ones" 1 + N(0, norm_std), "zeros"


_FLOATS = (torch.bfloat16, torch.float16, torch.float32, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def _open_folder(folder: Path) -> dict:
    """name -> SafetensorsFile for every tensor of the folder."""
    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    files: dict = {}
    where: dict = {}
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        for name, fname in weight_map.items():
            if fname not in files:
                if not (folder / fname).is_file():
                    raise WeightError(f"{folder}: shard '{fname}' named by the index is missing")
                files[fname] = SafetensorsFile(folder / fname)
            if name not in files[fname].entries:
                raise WeightError(f"{folder}: the index places '{name}' in '{fname}', which does not hold it")
            where[name] = files[fname]
    elif single.is_file():
        f = SafetensorsFile(single)
        where = {name: f for name in f.names()}
    else:
        raise WeightError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")
    return where


def load_weights(folder, expected: dict, device="cpu", ignore: tuple = ()) -> dict:
    """Tensors of `expected` from `folder`, on `device`, or one error naming all faults.
    `ignore`: names that may be present without being expected (reported by the caller)."""
    folder = Path(folder)
    try:
        where = _open_folder(folder)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    missing, wrong = [], []
    for name, spec in expected.items():
        f = where.get(name)
        if f is None:
            if not spec.optional:
                missing.append(name)
            continue
        if tuple(f.shape(name)) != tuple(spec.shape):
            wrong.append(f"{name}: stored {list(f.shape(name))}, expected {list(spec.shape)}")
        elif spec.kind == "float" and f.dtype(name) not in _FLOATS:
            wrong.append(f"{name}: stored as {f.dtype(name)}, expected a floating type")
        elif spec.kind == "int" and f.dtype(name) not in _INTS:
            wrong.append(f"{name}: stored as {f.dtype(name)}, expected an integer type")
    unexpected = sorted(n for n in where if n not in expected and n not in ignore)
    if missing or wrong or unexpected:
        lines = [f"{folder}: the weights do not match the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))
    out = {}
    for name, spec in expected.items():
        f = where.get(name)
        if f is None:
            continue
        t = f.tensor(name)
        if spec.kind == "int":
            t = t.to(torch.int32)
        elif t.dtype in (torch.float16, torch.float64):       # not a type the kernels read
            t = t.to(torch.float32)
        out[name] = t.to(device, copy=True)
    return out
