"""Toy parts defined HERE show that the other families are as open as the mixers: a feed-forward with a
router and experts, a position encoding that is a learned table added to the embedded tokens, and a norm
with a bias.  They are registered, put into an architecture (different feed-forwards and norms in different
layers, one layer run twice with a cache each, one entry reading an earlier entry's cache), loaded from a
random model folder and stepped in portions; nothing in the package is changed for them.  The reference is
a plain loop over whole sequences written below from the same formulas."""
from dataclasses import dataclass

import pytest
import torch

from tests.gpu_helpers import assert_close

pytestmark = pytest.mark.gpu

H, V, E, HEADS, KV, D, MAXPOS = 32, 90, 3, 2, 1, 16, 64


def _define():
    from tensorline_b200.models import LayerSpec, ModelSpec, RunEntry, register_architecture
    from tensorline_b200.parts import (Part, PartSpec, TensorSpec, register_feed_forward, register_norm,
                                       register_position_encoding)
    from tensorline_b200.parts.linear import matmul, resolve

    @register_feed_forward("toy_top1_experts")
    class Top1Experts(Part):
        """y = w_e * relu(h U_e^T) D_e^T for the expert e with the largest router logit (w_e = its softmax weight);
        router logits and softmax in float32."""
        def __init__(self, rt, hidden, inner, experts):
            super().__init__(rt)
            self.hidden, self.inner, self.experts = hidden, inner, experts

        def expected_tensors(self, prefix):
            out = {f"{prefix}.router.weight": TensorSpec((self.experts, self.hidden))}
            for e in range(self.experts):
                out[f"{prefix}.experts.{e}.up.weight"] = TensorSpec((self.inner, self.hidden))
                out[f"{prefix}.experts.{e}.down.weight"] = TensorSpec((self.hidden, self.inner))
            return out

        def bind(self, weights, prefix):
            self.router = weights[f"{prefix}.router.weight"].float()
            self.up = [self._compute_copy(weights[f"{prefix}.experts.{e}.up.weight"]) for e in range(self.experts)]
            self.down = [self._compute_copy(weights[f"{prefix}.experts.{e}.down.weight"]) for e in range(self.experts)]

        def forward(self, h, ctx):
            probs = torch.softmax(h.float() @ self.router.T, dim=-1)
            weight, pick = probs.max(dim=-1)
            y = torch.zeros((h.shape[0], self.hidden), dtype=h.dtype, device=h.device)
            for e in range(self.experts):                    # tokens grouped by expert
                rows = (pick == e).nonzero().flatten()
                if rows.numel():
                    inner = torch.relu(matmul(h[rows].contiguous(), self.up[e]))
                    y[rows] = (matmul(inner, self.down[e]).float() * weight[rows, None]).to(h.dtype)
            return y

    @register_position_encoding("toy_learned_table")
    class LearnedTable(Part):
        def __init__(self, rt, hidden, positions):
            super().__init__(rt)
            self.hidden, self.positions = hidden, positions
            self._none = torch.zeros(0, dtype=torch.float32, device=rt.device)

        def expected_tensors(self, prefix):
            return {f"{prefix}.weight": TensorSpec((self.positions, self.hidden))}

        def bind(self, weights, prefix):
            self.table = weights[f"{prefix}.weight"].float()

        def rotary(self):
            return self._none, 0                               # nothing to rotate inside the mixer

        def on_embedding(self, x, ctx):
            x += self.table[ctx.pos.long()]                    # x is the float32 residual stream

    @register_norm("toy_layer_norm")
    class LayerNormWithBias(Part):
        def __init__(self, rt, dim, eps):
            super().__init__(rt)
            self.dim, self.eps = dim, eps

        def expected_tensors(self, prefix):
            return {f"{prefix}.weight": TensorSpec((self.dim,), init="ones"), f"{prefix}.bias": TensorSpec((self.dim,))}

        def bind(self, weights, prefix):
            self.w, self.b = weights[f"{prefix}.weight"].float(), weights[f"{prefix}.bias"].float()

        def add_norm(self, x, pending, rows=None):
            pending = resolve(pending)                         # a projection may hand over unsummed pieces
            if rows is None:
                if pending is not None:
                    x += pending.float()
                src = x
            else:
                src = x[rows.long()] + (pending[rows.long()].float() if pending is not None else 0)
            return torch.nn.functional.layer_norm(src, (self.dim,), self.w, self.b, self.eps).to(self.rt.act_dtype)

    @dataclass(frozen=True)
    class ToyConfig:
        architecture: str
        seed_note: str

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            return cls(raw["architectures"][0], raw.get("seed_note", ""))

        def to_json_dict(self):
            return {"architectures": [self.architecture], "seed_note": self.seed_note}

    def describe(cfg):
        rms = PartSpec("rms_norm", {"dim": H, "eps": 1e-5})
        ln = PartSpec("toy_layer_norm", {"dim": H, "eps": 1e-4})
        dense = PartSpec("gated_mlp", {"hidden": H, "intermediate": 48})
        routed = PartSpec("toy_top1_experts", {"hidden": H, "inner": 40, "experts": E})
        attn = PartSpec("paged_attention", {"hidden": H, "num_heads": HEADS, "num_kv_heads": KV, "head_dim": D,
                                            "qkv_bias": True, "position": PartSpec("none", {})})
        blocks = [PartSpec("pre_norm", {"mixer": attn, "feed_forward": routed, "norm1": ln, "norm2": rms}),
                  PartSpec("pre_norm", {"mixer": attn, "feed_forward": dense, "norm1": rms, "norm2": ln})]
        # layer 0 runs twice, each time with keys and values of its own; the last entry runs layer 1 again
        # on the keys and values that entry 2 wrote
        run = (RunEntry(0), RunEntry(0), RunEntry(1), RunEntry(1, reads_cache_of=2))
        return ModelSpec(vocab_size=V, hidden_size=H, layers=tuple(LayerSpec(b, f"model.layers.{i}") for i, b in enumerate(blocks)),
                         run=run, final_norm=ln, tie_word_embeddings=False,
                         embedding_position=PartSpec("toy_learned_table", {"hidden": H, "positions": MAXPOS}),
                         max_position_embeddings=MAXPOS)

    register_architecture("ToyRoutedLM", ToyConfig, describe)
    return ToyConfig


def _plain(w, ids):
    """Whole sequence, float64, from the formulas in the classes above and the attention of the package's
    plain model (causal, no rotation)."""
    f = lambda name: w[name].double()
    n = len(ids)
    x = f("model.embed_tokens.weight")[ids] + f("model.embed_positions.weight")[torch.arange(n)]

    def ln(v, p, eps=1e-4):
        mu, var = v.mean(-1, keepdim=True), v.var(-1, unbiased=False, keepdim=True)
        return (v - mu) / torch.sqrt(var + eps) * f(p + ".weight") + f(p + ".bias")

    def rms(v, p, eps=1e-5):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * f(p + ".weight")

    def attention(h, p, kv=None):
        q = (h @ f(p + ".q_proj.weight").T + f(p + ".q_proj.bias")).view(n, HEADS, D)
        if kv is None:
            k = (h @ f(p + ".k_proj.weight").T + f(p + ".k_proj.bias")).view(n, KV, D)
            v = (h @ f(p + ".v_proj.weight").T + f(p + ".v_proj.bias")).view(n, KV, D)
        else:
            k, v = kv
        out = torch.empty(n, HEADS, D, dtype=torch.float64)
        mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
        for hd in range(HEADS):
            s = (q[:, hd] @ k[:, hd // (HEADS // KV)].T) * D ** -0.5
            out[:, hd] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, hd // (HEADS // KV)]
        return out.reshape(n, HEADS * D) @ f(p + ".o_proj.weight").T, (k, v)

    def routed(h, p):
        probs = torch.softmax(h @ f(p + ".router.weight").T, -1)
        weight, pick = probs.max(-1)
        y = torch.zeros_like(h)
        for t in range(n):
            e = int(pick[t])
            y[t] = weight[t] * (torch.relu(h[t] @ f(f"{p}.experts.{e}.up.weight").T) @ f(f"{p}.experts.{e}.down.weight").T)
        return y

    def dense(h, p):
        g, u = h @ f(p + ".gate_proj.weight").T, h @ f(p + ".up_proj.weight").T
        return (g / (1 + torch.exp(-g)) * u) @ f(p + ".down_proj.weight").T

    kv2 = None
    for entry, (layer, reads) in enumerate(((0, None), (0, None), (1, None), (1, 2))):
        p = f"model.layers.{layer}"
        h = ln(x, p + ".input_layernorm") if layer == 0 else rms(x, p + ".input_layernorm")
        a, kv = attention(h, p + ".self_attn", kv2 if reads is not None else None)
        if entry == 2:
            kv2 = kv
        x = x + a
        h = rms(x, p + ".post_attention_layernorm") if layer == 0 else ln(x, p + ".post_attention_layernorm")
        x = x + (routed(h, p + ".mlp") if layer == 0 else dense(h, p + ".mlp"))
    return ln(x, "model.norm") @ f("lm_head.weight").T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_feed_forward_position_encoding_and_norm(dtype, tmp_path):
    from tensorline_b200.cache import CacheManager
    from tensorline_b200.engine.runner import ModelRunner, StepEntry
    from tensorline_b200.models import expected_tensors, load_model
    from tensorline_b200.parts import Runtime
    from tensorline_b200.weights import write_random_model
    from tensorline_b200.weights.safetensors_io import SafetensorsFile
    ToyConfig = _define()
    cfg = ToyConfig("ToyRoutedLM", "toy")
    expected = expected_tensors(cfg)
    assert "model.embed_positions.weight" in expected and "model.layers.0.mlp.experts.2.down.weight" in expected
    assert "model.layers.1.post_attention_layernorm.bias" in expected and "model.norm.bias" in expected
    folder = write_random_model(tmp_path / "toy", cfg, expected, seed=9, std=0.25, norm_std=0.1)
    model, _ = load_model(folder, Runtime(torch.device("cuda"), dtype, 4))
    needs = model.cache_needs()
    assert sorted(needs) == [0, 1, 2]                         # the fourth entry reads the third's cache
    cache = CacheManager(needs, page_size=4, num_pages=30, max_num_seqs=3, max_model_len=MAXPOS)
    runner = ModelRunner(model, cache)
    st = SafetensorsFile(folder / "model.safetensors")
    weights = {name: st.tensor(name).clone() for name in st.names()}
    g = torch.Generator().manual_seed(1)
    seqs = {"a": torch.randint(0, V, (23,), generator=g).tolist(), "b": torch.randint(0, V, (14,), generator=g).tolist()}
    want = {rid: _plain(weights, torch.tensor(toks)) for rid, toks in seqs.items()}
    for rid in seqs:
        cache.admit(rid); runner.start_request(rid)
    got, done = {"a": [], "b": []}, {"a": 0, "b": 0}
    for step in ([("a", 6)], [("a", 3), ("b", 7)], [("b", 1), ("a", 1)], [("a", 13), ("b", 6)]):
        entries = []
        for rid, n in step:
            cache.grow(rid, done[rid], done[rid] + n)
            entries.append(StepEntry(rid, seqs[rid][done[rid]:done[rid] + n], list(range(n))))
            done[rid] += n
        out = runner.step(entries)
        row = 0
        for rid, n in step:
            got[rid].append(out[row:row + n]); row += n
    # the router's choice is a discontinuity: in bfloat16 a token whose two best experts are nearly tied may
    # take the other one, so compare there only where the float64 router has a clear winner
    for rid in seqs:
        res = torch.cat(got[rid]).double().cpu()
        if dtype == torch.float32:
            assert_close(res, want[rid], f"toy model, request {rid}", rtol=2e-4, atol=2e-4)
        else:
            err = (res - want[rid]).abs().amax(-1) / want[rid].abs().amax()
            assert float(err.median()) < 0.03 and float((err < 0.06).double().mean()) >= 0.8, err


# ------------------------------------------------------------------------------------------------------------------
# A second toy architecture: an embedding that scales its rows, an output head with a bias and a soft cap, a rotary
# encoding over interleaved pairs of half the head's dimensions, and an RMS norm of every q and k head before the
# rotation.  All four are options of other published decoders; none is this engine's architecture.  The embedding,
# the head and the encoding are classes of THIS file; pairing and q/k norm are arguments of the package's fused kernel.

H2, V2, HEADS2, KV2, D2, ROT2, CAP, THETA2 = 48, 70, 4, 2, 16, 8, 5.0, 50.0


def _define_scaled():
    from tensorline_b200 import ops
    from tensorline_b200.models import LayerSpec, ModelSpec, RunEntry, register_architecture
    from tensorline_b200.parts import (Part, PartSpec, Rotary, TensorSpec, register_embedding, register_head,
                                       register_position_encoding)
    from tensorline_b200.parts.linear import matmul

    @register_embedding("toy_scaled_table")
    class ScaledTable(Part):
        graph_capturable = True

        def __init__(self, rt, vocab, dim):
            super().__init__(rt)
            self.vocab, self.dim = vocab, dim

        def expected_tensors(self, prefix):
            return {f"{prefix}.weight": TensorSpec((self.vocab, self.dim))}

        def bind(self, weights, prefix):
            self.weight = self._compute_copy(weights[f"{prefix}.weight"])

        def forward(self, ids):
            x = torch.empty((ids.numel(), self.dim), dtype=torch.float32, device=ids.device)
            ops.embed(x, self.weight, ids)
            return x.mul_(self.dim ** 0.5)

    @register_head("toy_capped")
    class CappedHead(Part):
        graph_capturable = True

        def __init__(self, rt, vocab, dim, tied, cap):
            super().__init__(rt)
            self.vocab, self.dim, self.tied, self.cap = vocab, dim, tied, cap

        def expected_tensors(self, prefix):
            return {f"{prefix}.weight": TensorSpec((self.vocab, self.dim), optional=self.tied),
                    f"{prefix}.bias": TensorSpec((self.vocab,))}

        def bind(self, weights, prefix, embedding=None):
            self.weight = embedding.weight if self.tied else self._compute_copy(weights[f"{prefix}.weight"])
            self.bias = weights[f"{prefix}.bias"].float()

        def forward(self, h):
            z = matmul(h, self.weight, out_dtype=torch.float32) + self.bias
            return self.cap * torch.tanh(z / self.cap)

    @register_position_encoding("toy_rotary_interleaved")
    class RotaryInterleaved(Part):
        graph_capturable = True

        def __init__(self, rt, head_dim, theta, rotary_dim):
            super().__init__(rt)
            i = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
            self.rot = rotary_dim
            self.inv_freq = (float(theta) ** (-i / rotary_dim)).to(torch.float32).to(rt.device)

        def rotary(self):
            return Rotary(self.inv_freq, self.rot, "interleaved")

        def on_embedding(self, x, ctx):
            return None

    @dataclass(frozen=True)
    class ScaledConfig:
        architecture: str

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            return cls(raw["architectures"][0])

        def to_json_dict(self):
            return {"architectures": [self.architecture]}

    def describe(cfg):
        rms = PartSpec("rms_norm", {"dim": H2, "eps": 1e-5})
        ff = PartSpec("gated_mlp", {"hidden": H2, "intermediate": 56})
        attn = PartSpec("paged_attention", {"hidden": H2, "num_heads": HEADS2, "num_kv_heads": KV2, "head_dim": D2,
                                            "qkv_bias": True, "qk_norm_eps": 1e-4,
                                            "position": PartSpec("toy_rotary_interleaved", {"theta": THETA2, "rotary_dim": ROT2})})
        block = PartSpec("pre_norm", {"mixer": attn, "feed_forward": ff, "norm1": rms, "norm2": rms})
        return ModelSpec(vocab_size=V2, hidden_size=H2, layers=tuple(LayerSpec(block, f"model.layers.{i}") for i in range(2)),
                         run=(RunEntry(0), RunEntry(1)), final_norm=rms, tie_word_embeddings=True,
                         embedding=PartSpec("toy_scaled_table"), head=PartSpec("toy_capped", {"cap": CAP}))

    register_architecture("ToyScaledLM", ScaledConfig, describe)
    return ScaledConfig


def _plain_scaled(w, ids):
    f = lambda name: w[name].double()
    n = len(ids)
    x = f("model.embed_tokens.weight")[ids] * H2 ** 0.5

    def rms(v, weight, eps):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight

    i = torch.arange(0, ROT2, 2, dtype=torch.float64)
    inv_freq = (THETA2 ** (-i / ROT2)).to(torch.float32)
    angle = (torch.arange(n, dtype=torch.float32)[:, None] * inv_freq[None, :]).double()
    cos, sin = torch.cos(angle), torch.sin(angle)

    def rotate(t):                                               # [n, heads, D2]: pairs (2i, 2i + 1) of the first ROT2 dims
        out = t.clone()
        a, b = t[..., 0:ROT2:2], t[..., 1:ROT2:2]
        out[..., 0:ROT2:2] = a * cos[:, None, :] - b * sin[:, None, :]
        out[..., 1:ROT2:2] = b * cos[:, None, :] + a * sin[:, None, :]
        return out

    mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
    for layer in range(2):
        p = f"model.layers.{layer}"
        h = rms(x, f(p + ".input_layernorm.weight"), 1e-5)
        a = p + ".self_attn"
        q = (h @ f(a + ".q_proj.weight").T + f(a + ".q_proj.bias")).view(n, HEADS2, D2)
        k = (h @ f(a + ".k_proj.weight").T + f(a + ".k_proj.bias")).view(n, KV2, D2)
        v = (h @ f(a + ".v_proj.weight").T + f(a + ".v_proj.bias")).view(n, KV2, D2)
        q = rotate(rms(q, f(a + ".q_norm.weight"), 1e-4))
        k = rotate(rms(k, f(a + ".k_norm.weight"), 1e-4))
        out = torch.empty(n, HEADS2, D2, dtype=torch.float64)
        for hd in range(HEADS2):
            s = (q[:, hd] @ k[:, hd // (HEADS2 // KV2)].T) * D2 ** -0.5
            out[:, hd] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, hd // (HEADS2 // KV2)]
        x = x + out.reshape(n, HEADS2 * D2) @ f(a + ".o_proj.weight").T
        h = rms(x, f(p + ".post_attention_layernorm.weight"), 1e-5)
        g, u = h @ f(p + ".mlp.gate_proj.weight").T, h @ f(p + ".mlp.up_proj.weight").T
        x = x + (g / (1 + torch.exp(-g)) * u) @ f(p + ".mlp.down_proj.weight").T
    z = rms(x, f("model.norm.weight"), 1e-5) @ f("model.embed_tokens.weight").T + f("lm_head.bias")
    return CAP * torch.tanh(z / CAP)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_embedding_head_pairing_and_qk_norm(dtype, tmp_path):
    """Portions beside single tokens, then the last tokens decoded through CUDA graphs, against the float64 loop."""
    from tensorline_b200.cache import CacheManager
    from tensorline_b200.engine.runner import ModelRunner, StepEntry
    from tensorline_b200.models import expected_tensors, load_model
    from tensorline_b200.parts import Runtime
    from tensorline_b200.weights import write_random_model
    from tensorline_b200.weights.safetensors_io import SafetensorsFile
    ScaledConfig = _define_scaled()
    cfg = ScaledConfig("ToyScaledLM")
    expected = expected_tensors(cfg)
    assert "lm_head.bias" in expected and "model.layers.1.self_attn.k_norm.weight" in expected
    assert expected["lm_head.weight"].optional                  # tied: the table is the embedding's
    folder = write_random_model(tmp_path / "toy2", cfg, expected, seed=11, std=0.15, norm_std=0.2)
    model, _ = load_model(folder, Runtime(torch.device("cuda"), dtype, 4))
    assert model.graph_capturable()
    cache = CacheManager(model.cache_needs(), page_size=4, num_pages=30, max_num_seqs=3, max_model_len=64)
    runner = ModelRunner(model, cache)
    runner.use_graphs = True
    st = SafetensorsFile(folder / "model.safetensors")
    weights = {name: st.tensor(name).clone() for name in st.names()}
    g = torch.Generator().manual_seed(2)
    seqs = {"a": torch.randint(0, V2, (25,), generator=g).tolist(), "b": torch.randint(0, V2, (18,), generator=g).tolist()}
    want = {rid: _plain_scaled(weights, torch.tensor(toks)) for rid, toks in seqs.items()}
    for rid in seqs:
        cache.admit(rid); runner.start_request(rid)
    got, done = {"a": [], "b": []}, {"a": 0, "b": 0}
    plan = [[("a", 7)], [("a", 2), ("b", 9)], [("b", 1), ("a", 1)], [("a", 9), ("b", 2)]] + [[("a", 1), ("b", 1)]] * 6
    for step in plan:
        entries = []
        for rid, n in step:
            cache.grow(rid, done[rid], done[rid] + n)
            entries.append(StepEntry(rid, seqs[rid][done[rid]:done[rid] + n], list(range(n))))
            done[rid] += n
        out = runner.step_graph(entries).clone() if runner.can_replay(entries) else runner.step(entries)
        row = 0
        for rid, n in step:
            got[rid].append(out[row:row + n]); row += n
    assert runner.graph_replays == 7 and done == {"a": 25, "b": 18}
    for rid in seqs:
        res = torch.cat(got[rid]).double().cpu()
        if dtype == torch.float32:
            assert_close(res, want[rid], f"scaled toy model, request {rid}", rtol=1e-4, atol=1e-4)
        else:
            err = float((res - want[rid]).abs().max())
            assert err <= 0.05 * float(want[rid].abs().max()), f"request {rid}: {err:.3e}"
