"""Compares the plain implementation with tzar-beep/Tensorline's own model code, once, on the CPU,
and writes the small outputs that tests/test_plain.py checks the plain implementation against.

What runs from the reference project: `tensorline.paged.PagedModel.forward` with `SeqChunk`s, its
`BlockAllocator`-style block tables, and the CPU branches of `tensorline.fused.add_rmsnorm` and
`rope_` (tensorline/paged.py:190-287, tensorline/fused.py:58-85).  That code fixes the order of
operations in a layer, the residual folded into the norms, the rotate-half pairing, the K/V write
into pages, the three attention paths (decode, fresh prompt, resumed portion) with their masks, the
scale and the grouping of query heads.

What does NOT come from it: tzar-beep/Tensorline has no model definition of its own; it re-drives
the sub-modules of a model object built by an installed package (tensorline/paged.py:13-14,
:172-188).  No installed package's model code is used here.  The object handed to `PagedModel` is a
shim defined below whose sub-modules (RMSNorm, the rotary table, the SwiGLU feed-forward, the linear
projections) are written from the formulas, in float32.  So the golden values rest on the
reference's code for everything it owns and on the formulas for the rest.

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


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from tensorline.paged import PagedModel, SeqChunk          # the reference's own code

    out = {}
    for name in ("A", "B_FULL"):                                # the reference has no window: full attention only
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_tiny(name, tmp, seed=0)
            plain = PlainQwen2(folder)
            shim = ShimModel(folder).eval()
            bs = PAGE_SIZE[name]
            ids = random_tokens(CONFIGS[name]["vocab_size"], 29, seed=11)
            table = [5, 2, 7, 0, 9, 11, 3, 1][: -(-len(ids) // bs)]
            ref_all = forward(plain, ids)
            rows = {}
            pm = PagedModel(shim, num_blocks=16, block_size=bs)
            rows["whole"] = pm.forward([SeqChunk(ids, 0, table, True)])[0]
            pm = PagedModel(shim, num_blocks=16, block_size=bs)
            for s in range(0, len(ids), 3):                     # resumed portions through the pages
                last = pm.forward([SeqChunk(ids[s:s + 3], s, table, True)])[0]
            rows["chunks_of_3"] = last
            pm = PagedModel(shim, num_blocks=16, block_size=bs)
            pm.forward([SeqChunk(ids[:20], 0, table, False)])
            for s in range(20, len(ids)):                       # then token by token (the decode path)
                last = pm.forward([SeqChunk(ids[s:s + 1], s, table, True)])[0]
            rows["decode_tail"] = last
            weights = read_safetensors(folder / "model.safetensors")
            checksum = float(sum(v.double().abs().sum() for v in weights.values()))
            rec = {"ids": ids, "weights_abs_sum": checksum, "position": len(ids) - 1, "logits": {}}
            for k, v in rows.items():
                diff = float((v.double() - ref_all[-1]).abs().max())
                print(f"{name} {k}: reference vs plain max abs diff {diff:.3e} (logit scale {float(ref_all[-1].abs().max()):.3f})")
                assert diff < 2e-5, "the plain implementation and the reference disagree"
                rec["logits"][k] = [round(float(x), 7) for x in v.tolist()]
            out[name] = rec
    path = Path(__file__).with_name("reference_logits.json")
    path.write_text(json.dumps(out))
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
