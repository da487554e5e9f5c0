"""Compares the plain implementation with tzar-beep/Tensorline's own model code, once, on the CPU,
and writes the small outputs that tests/test_plain.py checks the plain implementation against.

What runs from the reference project: `tensorline.paged.PagedModel.forward` with `SeqChunk`s, its
`BlockAllocator`-style block tables, and the CPU branches of `tensorline.fused.add_rmsnorm` and
`rope_` (tensorline/paged.py:190-287, tensorline/fused.py:58-85).  That code fixes the order of
operations in a layer, the residual folded into the norms, the rotate-half pairing, the K/V write
into pages, the three attention paths (decode, fresh prompt, resumed portion) with their masks, the
scale and the grouping of query heads.

tzar-beep/Tensorline has no model definition of its own; it re-drives the sub-modules of a model
object that ITS OWN loader builds through an installed package (tensorline/engine.py:63-66,
tensorline/paged.py:13-14, :172-188).  Two sets of values are written for every model:

* `as_it_runs`: the reference exactly as it runs.  A model folder with the seeded weights, a
  config.json and a word-level tokenizer is written here; the reference's own `Engine(folder,
  device="cpu", dtype="float32")` loads it (its code, its imports; this script imports no installed
  package's model code and reads none); the loaded object goes to `PagedModel` as the reference's
  `BatchEngine` does (tensorline/batch_engine.py:87-88).  RMSNorm, SwiGLU and the rotary table are
  then whatever the reference really executes, not this repository's reading of them.  For the
  window model (Tiny B) the reference's paged path has no window (tensorline/paged.py:230-237), so
  its one-request engine is used instead: `Engine.stream` (tensorline/engine.py:86-120), greedy,
  through its public interface; the generated token ids are stored.
* `shim`: `PagedModel` over a stand-in object whose sub-modules are written from the formulas in
  float32 (kept as a second, independent entry).

tests/test_plain.py checks the plain implementation against both.

Usage (from the repository root, with the reference project's folder as argument):
    python tests/golden/make_golden.py /path/to/Tensorline
"""
from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path
from types import SimpleNamespace

import torch
from torch import nn

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.plain.qwen2_plain import PlainQwen2, forward, read_safetensors  # noqa: E402
from tests.tiny import CONFIGS, PAGE_SIZE, random_tokens, write_tiny  # noqa: E402


class ShimNorm(nn.Module):
    def __init__(self, w, eps):
        super().__init__()
        self.weight = nn.Parameter(w, requires_grad=False)
        self.variance_epsilon = eps

    def forward(self, x):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.variance_epsilon) * self.weight


class ShimMLP(nn.Module):
    def __init__(self, g, u, d):
        super().__init__()
        self.g, self.u, self.d = (nn.Parameter(t, requires_grad=False) for t in (g, u, d))

    def forward(self, h):
        a = h @ self.g.T
        return ((a / (1 + torch.exp(-a))) * (h @ self.u.T)) @ self.d.T


class ShimRotary(nn.Module):
    def __init__(self, d, theta):
        super().__init__()
        i = torch.arange(0, d, 2, dtype=torch.float64)
        self.inv_freq = (float(theta) ** (-i / d)).to(torch.float32)

    def forward(self, x, pos):                       # pos [1, T] -> cos, sin [1, T, d], halves repeated
        ang = pos[0].to(torch.float32)[:, None] * self.inv_freq[None, :]
        ang = torch.cat((ang, ang), dim=-1)
        return ang.cos()[None], ang.sin()[None]


def _linear(w, b=None):
    lin = nn.Linear(w.shape[1], w.shape[0], bias=b is not None)
    lin.weight = nn.Parameter(w, requires_grad=False)
    if b is not None:
        lin.bias = nn.Parameter(b, requires_grad=False)
    return lin


class ShimModel(nn.Module):
    """The attribute layout that tensorline/paged.py:110-130, :172-188 reads."""

    def __init__(self, folder):
        super().__init__()
        p = PlainQwen2(folder)
        w = {k: v.float() for k, v in read_safetensors(Path(folder) / "model.safetensors").items()}
        self.config = SimpleNamespace(num_attention_heads=p.nq, num_key_value_heads=p.nkv, num_hidden_layers=p.L)
        inner = nn.Module()
        inner.embed_tokens = nn.Embedding.from_pretrained(w["model.embed_tokens.weight"])
        inner.rotary_emb = ShimRotary(p.d, p.theta)
        inner.norm = ShimNorm(w["model.norm.weight"], p.eps)
        layers = []
        for i in range(p.L):
            pre = f"model.layers.{i}."
            attn = nn.Module()
            attn.head_dim, attn.scaling = p.d, p.d ** -0.5
            for n in "qkv":
                setattr(attn, f"{n}_proj", _linear(w[pre + f"self_attn.{n}_proj.weight"], w[pre + f"self_attn.{n}_proj.bias"]))
            attn.o_proj = _linear(w[pre + "self_attn.o_proj.weight"])
            layer = nn.Module()
            layer.self_attn = attn
            layer.input_layernorm = ShimNorm(w[pre + "input_layernorm.weight"], p.eps)
            layer.post_attention_layernorm = ShimNorm(w[pre + "post_attention_layernorm.weight"], p.eps)
            layer.mlp = ShimMLP(w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"], w[pre + "mlp.down_proj.weight"])
            layers.append(layer)
        inner.layers = nn.ModuleList(layers)
        self.model = inner
        head = w["model.embed_tokens.weight"] if p.tied else w["lm_head.weight"]
        self.lm_head = _linear(head)


def add_loader_files(folder, raw: dict) -> None:
    """What the reference's loader needs beside config.json and model.safetensors: a `model_type` key and a
    tokenizer.  The tokenizer is word level: token id i is the word "t<i>", words are split on white space."""
    cfg = json.loads((Path(folder) / "config.json").read_text())
    cfg.update(model_type="qwen2", torch_dtype="float32", bos_token_id=raw["eos_token_id"])
    (Path(folder) / "config.json").write_text(json.dumps(cfg))
    V = raw["vocab_size"]
    tok = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
           "pre_tokenizer": {"type": "WhitespaceSplit"}, "post_processor": None, "decoder": None,
           "model": {"type": "WordLevel", "vocab": {f"t{i}": i for i in range(V)}, "unk_token": "t0"}}
    (Path(folder) / "tokenizer.json").write_text(json.dumps(tok))
    (Path(folder) / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": f"t{raw['eos_token_id']}", "unk_token": "t0",
         "model_max_length": 4096}))


def three_schedules(PagedModel, SeqChunk, model, ids, table, bs) -> dict:
    """Logits at the last position from the reference's paged model: the prompt whole, in portions of three
    tokens (resumed portions through the pages), and 20 tokens then one by one (its decode path)."""
    rows = {}
    pm = PagedModel(model, num_blocks=16, block_size=bs)
    rows["whole"] = pm.forward([SeqChunk(ids, 0, table, True)])[0]
    pm = PagedModel(model, num_blocks=16, block_size=bs)
    for s in range(0, len(ids), 3):
        last = pm.forward([SeqChunk(ids[s:s + 3], s, table, True)])[0]
    rows["chunks_of_3"] = last
    pm = PagedModel(model, num_blocks=16, block_size=bs)
    pm.forward([SeqChunk(ids[:20], 0, table, False)])
    for s in range(20, len(ids)):
        last = pm.forward([SeqChunk(ids[s:s + 1], s, table, True)])[0]
    rows["decode_tail"] = last
    return rows


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from tensorline.engine import Engine as ReferenceEngine    # the reference's own loader and one-request engine
    from tensorline.engine import GenStats, SamplingParams
    from tensorline.paged import PagedModel, SeqChunk          # the reference's own paged model

    out = {}
    for name in ("A", "B_FULL"):                                # the reference's paged path has no window
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_tiny(name, tmp, seed=0)
            plain = PlainQwen2(folder)
            bs = PAGE_SIZE[name]
            ids = random_tokens(CONFIGS[name]["vocab_size"], 29, seed=11)
            table = [5, 2, 7, 0, 9, 11, 3, 1][: -(-len(ids) // bs)]
            ref_all = forward(plain, ids)
            weights = read_safetensors(folder / "model.safetensors")
            checksum = float(sum(v.double().abs().sum() for v in weights.values()))
            rec = {"ids": ids, "weights_abs_sum": checksum, "position": len(ids) - 1, "logits": {}}
            shim = ShimModel(folder).eval()
            add_loader_files(folder, CONFIGS[name])
            loaded = ReferenceEngine(str(folder), device="cpu", dtype="float32")
            for how, model in (("as_it_runs", loaded.model), ("shim", shim)):
                with torch.inference_mode():
                    rows = three_schedules(PagedModel, SeqChunk, model, ids, table, bs)
                for k, v in rows.items():
                    diff = float((v.double() - ref_all[-1]).abs().max())
                    print(f"{name} {how} {k}: reference vs plain max abs diff {diff:.3e} "
                          f"(logit scale {float(ref_all[-1].abs().max()):.3f})")
                    assert diff < 2e-5, "the plain implementation and the reference disagree"
                    rec["logits"][f"{how}/{k}"] = [round(float(x), 7) for x in v.tolist()]
            out[name] = rec
    # The window model: the reference's one-request engine, greedy, through its public interface.
    with tempfile.TemporaryDirectory() as tmp:
        from tests.plain.qwen2_plain import greedy_generate
        folder = write_tiny("B", tmp, seed=0)
        plain = PlainQwen2(folder)
        no_window = PlainQwen2(write_tiny("B_FULL", Path(tmp) / "full", seed=0))      # the same weights, all keys visible
        weights = read_safetensors(folder / "model.safetensors")
        checksum = float(sum(v.double().abs().sum() for v in weights.values()))
        add_loader_files(folder, CONFIGS["B"])
        loaded = ReferenceEngine(str(folder), device="cpu", dtype="float32")
        rec = {"weights_abs_sum": checksum, "window": CONFIGS["B"]["sliding_window"], "greedy": []}
        for n, seed in ((40, 21), (57, 22)):                   # prompts longer than the window of 24
            prompt = random_tokens(CONFIGS["B"]["vocab_size"], n, seed=seed)
            text = "".join(loaded.stream(" ".join(f"t{t}" for t in prompt),
                                         SamplingParams(max_tokens=24, stop_token_ids={-1}), GenStats()))
            got = [int(w[1:]) for w in text.split()]
            mine = greedy_generate(plain, prompt, 24)
            print(f"B window, prompt of {n}: reference {got[:8]}..., plain {mine[:8]}..., equal: {got == mine}")
            assert got == mine, "the plain window model and the reference's engine disagree"
            assert greedy_generate(no_window, prompt, 24) != got, "the window changes nothing here: the comparison pins nothing"
            rec["greedy"].append({"prompt": prompt, "tokens": got})
        out["B"] = rec
    path = Path(__file__).with_name("reference_logits.json")
    path.write_text(json.dumps(out))
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
