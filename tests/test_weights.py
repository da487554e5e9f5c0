"""safetensors reading and writing, loading by name, the one error that lists every fault."""
import json

import pytest
import torch

from tensorline_b200.config import Qwen2Config
from tensorline_b200.models import expected_tensors
from tensorline_b200.weights import (SafetensorsFile, TensorSpec, WeightError, load_weights, write_random_model,
                                     write_safetensors)
from tests.plain.qwen2_plain import read_safetensors
from tests.tiny import TINY_A, TINY_B, write_tiny


def test_container_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int64),
         "e": torch.randn(2, 2), "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", t)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.names()) == sorted(t)
    for k, v in t.items():
        assert f.dtype(k) == v.dtype and torch.equal(f.tensor(k), v)
    mine = read_safetensors(tmp_path / "x.safetensors")                 # the tests' own reader agrees
    assert all(torch.equal(mine[k], v) for k, v in t.items())


def test_random_model_is_reproducible_and_seeded(tmp_path):
    a = read_safetensors(write_tiny("A", tmp_path / "a", seed=3) / "model.safetensors")
    b = read_safetensors(write_tiny("A", tmp_path / "b", seed=3) / "model.safetensors")
    c = read_safetensors(write_tiny("A", tmp_path / "c", seed=4) / "model.safetensors")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a                                    # tied: no head stored
    assert a["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert torch.all(a["model.norm.weight"] == 1)
    bb = read_safetensors(write_tiny("B", tmp_path / "d") / "model.safetensors")
    assert 0.05 < float(bb["model.norm.weight"].float().std()) < 0.2 and "lm_head.weight" in bb
    assert json.loads((tmp_path / "d" / "config.json").read_text())["sliding_window"] == 24


def test_loading_keeps_stored_types(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    exp = expected_tensors(cfg)
    folder = write_tiny("A", tmp_path / "m")
    w = load_weights(folder, exp)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    folder32 = write_tiny("A", tmp_path / "m32", store_dtype=torch.float32)
    w32 = load_weights(folder32, exp)
    assert all(t.dtype == torch.float32 for t in w32.values())          # stored in 32 bits: stays so
    exp2 = {"table": TensorSpec((4,), kind="int")}
    write_safetensors(tmp_path / "m" / "model.safetensors", {"table": torch.arange(4, dtype=torch.int64)})
    assert load_weights(tmp_path / "m", exp2)["table"].dtype == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_B)
    exp = expected_tensors(cfg)
    folder = write_tiny("B", tmp_path / "m")
    t = read_safetensors(folder / "model.safetensors")
    del t["model.layers.1.mlp.up_proj.weight"], t["model.layers.2.self_attn.q_proj.bias"]
    t["model.layers.0.extra.weight"] = torch.zeros(2)
    t["model.norm.weight"] = torch.zeros(97, dtype=torch.bfloat16)
    t["lm_head.weight"] = t["lm_head.weight"].T.contiguous()
    write_safetensors(folder / "model.safetensors", t)
    with pytest.raises(WeightError) as e:
        load_weights(folder, exp)
    msg = str(e.value)
    for word in ("missing (2)", "model.layers.1.mlp.up_proj.weight", "model.layers.2.self_attn.q_proj.bias",
                 "unexpected (1)", "model.layers.0.extra.weight", "wrong shape or type (2)",
                 "model.norm.weight: stored [97], expected [96]", "lm_head.weight: stored [96, 384]"):
        assert word in msg, word


def test_missing_files_and_broken_container(tmp_path):
    with pytest.raises(WeightError, match="neither"):
        load_weights(tmp_path, {})
    (tmp_path / "model.safetensors").write_bytes(b"\xff" * 16)
    with pytest.raises(WeightError, match="header"):
        load_weights(tmp_path, {})


def test_sharded_folder_with_index(tmp_path):
    t = read_safetensors(write_tiny("A", tmp_path / "src") / "model.safetensors")
    names = sorted(t)
    half = len(names) // 2
    out = tmp_path / "sharded"
    out.mkdir()
    write_safetensors(out / "s1.safetensors", {k: t[k] for k in names[:half]})
    write_safetensors(out / "s2.safetensors", {k: t[k] for k in names[half:]})
    index = {"weight_map": {k: ("s1.safetensors" if i < half else "s2.safetensors") for i, k in enumerate(names)}}
    (out / "model.safetensors.index.json").write_text(json.dumps(index))
    w = load_weights(out, expected_tensors(Qwen2Config.from_dict(TINY_A)))
    assert all(torch.equal(w[k], t[k]) for k in names)


def test_tied_model_ignores_a_stored_head(tmp_path):
    """A checkpoint of a tied model that also stores lm_head.weight loads; the head is not read."""
    from tensorline_b200.models import load_model
    from tensorline_b200.parts import Runtime
    folder = write_tiny("A", tmp_path / "m")
    t = read_safetensors(folder / "model.safetensors")
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", t)
    model, _ = load_model(folder, Runtime(torch.device("cpu"), torch.float32))
    assert model.head.weight is model.embedding.weight
