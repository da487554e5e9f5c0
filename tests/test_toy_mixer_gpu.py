"""A toy mixer with state of its own per request, and an architecture that uses it beside attention
layers, are defined HERE, registered, built and stepped; nothing in the package is changed for them.
The mixer keeps a decaying sum of its inputs in the request's state slot:
    s_t = decay * s_{t-1} + h_t,    y_t = s_t W^T
so its output at a position depends on every earlier token of the same request, across steps."""
from dataclasses import dataclass

import pytest
import torch

from tests.gpu_helpers import assert_close

pytestmark = pytest.mark.gpu


def _define():
    from tensorline_b200.cache import SlotState
    from tensorline_b200.models import LayerSpec, ModelSpec, RunEntry, register_architecture
    from tensorline_b200.parts import Part, PartSpec, TensorSpec, register_mixer
    from tensorline_b200.parts.linear import matmul

    @register_mixer("toy_decaying_sum")
    class DecayingSum(Part):
        graph_capturable = True          # a step of single tokens is served from device tensors only (see forward)

        def __init__(self, rt, hidden, decay):
            super().__init__(rt)
            self.hidden, self.decay = hidden, decay

        def cache_need(self):
            return SlotState((self.hidden,), "float32")

        def expected_tensors(self, prefix):
            return {f"{prefix}.mix.weight": TensorSpec((self.hidden, self.hidden))}

        def bind(self, weights, prefix):
            self.w = self._compute_copy(weights[f"{prefix}.mix.weight"])

        def forward(self, h, ctx, cache):
            if ctx.decode_only:                              # one token a request: all requests at once, by slot, on the
                idx = ctx.slots.long()                       # device (this is what a CUDA graph captures; padding rows
                s = self.decay * cache.state.index_select(0, idx) + h.float()      # carry the spare slot)
                cache.state.index_copy_(0, idx, s)
                return matmul(s.to(h.dtype), self.w)
            sums = torch.empty((h.shape[0], self.hidden), dtype=torch.float32, device=h.device)
            for b in range(ctx.B):                           # tokens of a request in order; state carried on
                slot, s = ctx.h_slots[b], None
                s = cache.state[slot].clone()
                for t in range(ctx.h_q_start[b], ctx.h_q_start[b + 1]):
                    s = self.decay * s + h[t].float()
                    sums[t] = s
                cache.state[slot] = s
            return matmul(sums.to(h.dtype), self.w)

    @dataclass(frozen=True)
    class ToyConfig:
        architecture: str
        vocab_size: int
        hidden_size: int
        decay: float

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            return cls(raw["architectures"][0], raw["vocab_size"], raw["hidden_size"], raw["decay"])

        def to_json_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "decay": self.decay}

    def describe(cfg):
        H = cfg.hidden_size
        norm = PartSpec("rms_norm", {"dim": H, "eps": 1e-5})
        ff = PartSpec("gated_mlp", {"hidden": H, "intermediate": 2 * H + 8})
        attn = PartSpec("paged_attention", {"hidden": H, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                            "qkv_bias": False, "position": PartSpec("rotary_half", {"theta": 100.0})})
        toy = PartSpec("toy_decaying_sum", {"hidden": H, "decay": cfg.decay})
        blocks = [PartSpec("pre_norm", {"mixer": m, "feed_forward": ff, "norm1": norm, "norm2": norm})
                  for m in (toy, attn, toy)]                 # different mixers in different layers
        return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=H,
                         layers=tuple(LayerSpec(b, f"model.layers.{i}") for i, b in enumerate(blocks)),
                         run=tuple(RunEntry(i) for i in range(3)), final_norm=norm, tie_word_embeddings=True)

    register_architecture("ToyStateLM", ToyConfig, describe)
    return ToyConfig


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype, tmp_path):
    from tensorline_b200.cache import CacheManager, PagedKV, SlotState
    from tensorline_b200.engine.runner import ModelRunner, StepEntry
    from tensorline_b200.models import expected_tensors, load_model
    from tensorline_b200.parts import Runtime
    from tensorline_b200.weights import write_random_model
    ToyConfig = _define()
    cfg = ToyConfig("ToyStateLM", 120, 32, 0.9)
    folder = write_random_model(tmp_path / "toy", cfg, expected_tensors(cfg), seed=5, std=0.2)
    model, loaded = load_model(folder, Runtime(torch.device("cuda"), dtype, 4))     # chosen by config.json
    assert loaded == cfg
    needs = model.cache_needs()
    assert isinstance(needs[0], SlotState) and isinstance(needs[1], PagedKV) and isinstance(needs[2], SlotState)
    cache = CacheManager(needs, page_size=4, num_pages=24, max_num_seqs=3, max_model_len=64)
    assert not cache.prefix_caching                          # state cannot be restored from pages
    runner = ModelRunner(model, cache)
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 120, (21,), generator=g).tolist()
    b = torch.randint(0, 120, (13,), generator=g).tolist()

    def whole(rid, toks):
        cache.admit(rid); runner.start_request(rid); cache.grow(rid, 0, len(toks))
        out = runner.step([StepEntry(rid, toks, list(range(len(toks))))])
        cache.release(rid); runner.end_request(rid)
        return out

    want_a, want_b = whole("a", a), whole("b", b)
    # now interleaved in portions: a and b share steps; each one's state lives in its own slot
    for rid in ("a", "b"):
        cache.admit(rid); runner.start_request(rid)
    got = {"a": [], "b": []}
    plan = [[("a", 5)], [("a", 2), ("b", 6)], [("b", 1), ("a", 1)], [("a", 13), ("b", 6)]]
    done = {"a": 0, "b": 0}
    for step in plan:
        entries = []
        for rid, n in step:
            toks = a if rid == "a" else b
            cache.grow(rid, done[rid], done[rid] + n)
            entries.append(StepEntry(rid, toks[done[rid]:done[rid] + n], list(range(n))))
            done[rid] += n
        out = runner.step(entries)
        row = 0
        for rid, n in step:
            got[rid].append(out[row:row + n]); row += n
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=4e-2, atol=4e-2)
    assert_close(torch.cat(got["a"]), want_a, "toy model, request a in portions", **tol)
    assert_close(torch.cat(got["b"]), want_b, "toy model, request b in portions", **tol)
    # a slot that is given back and taken again starts from zero state
    cache.release("a"); runner.end_request("a")
    again = whole("c", a)
    assert_close(again, want_a, "state slot reused", **tol)


def test_toy_state_model_decodes_through_cuda_graphs(tmp_path):
    """State of fixed size lives at fixed addresses indexed by slot, so the model with the toy mixer is captured
    like any other: the engine with graphs and overlapped scheduling gives the tokens of the engine without, under
    queueing (slots are reused) and with a preemption (state is rebuilt from the first token)."""
    from tensorline_b200 import Engine, SamplingParams
    from tensorline_b200.models import expected_tensors
    from tensorline_b200.weights import write_random_model
    ToyConfig = _define()
    cfg = ToyConfig("ToyStateLM", 120, 32, 0.9)
    folder = write_random_model(tmp_path / "toy", cfg, expected_tensors(cfg), seed=5, std=0.2)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 120, (n,), generator=g).tolist() for n in (9, 2, 14, 5, 11)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    outs = {}
    for graphs in (False, True):
        eng = Engine(str(folder), dtype="float32", block_size=4, num_blocks=12, max_num_seqs=3, max_model_len=48,
                     cuda_graphs=graphs, overlap=graphs)
        assert eng.runner._graphable
        outs[graphs] = [o.token_ids for o in eng.generate(prompts, sp)]
        st = eng.stats()
        assert (st["graph_replays"] > 0) == graphs and (st["overlapped_steps"] > 0) == graphs
        assert st["free_pages"] == st["num_pages"] and st["preemptions"] > 0 and st["max_running_seen"] == 3
    assert outs[True] == outs[False] and all(len(t) == 10 for t in outs[True])
