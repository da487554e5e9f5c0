"""Each part of a layer alone, built through its registry at sizes that no model of the tests has,
against the plain functions; then the run list: a layer named twice, a layer that reads another's cache."""
import pytest
import torch

from tests.gpu_helpers import BF16, F32, assert_close, i32
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DT = [torch.float32, torch.bfloat16]


def tol(dt):
    return F32 if dt == torch.float32 else BF16


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def runtime(dt, page=8):
    from tensorline_b200.parts import Runtime
    return Runtime(torch.device("cuda"), dt, page)


def one_request_ctx(T, page, num_pages, start=0, seed=0):
    """A StepContext for one request that brings tokens [start, start+T); pages scattered."""
    from tensorline_b200.engine.runner import StepContext
    max_pages = 64
    g = torch.Generator().manual_seed(seed)
    table = torch.full((2, max_pages), num_pages, dtype=torch.int32)
    need = -(-(start + T) // page)
    table[0, :need] = torch.randperm(num_pages, generator=g)[:need].to(torch.int32)
    return StepContext(T=T, B=1, ids=i32([0] * T), pos=i32(list(range(start, start + T))), req_slot=i32([0] * T),
                       q_start=i32([0, T]), start_pos=i32([start]), slots=i32([0]), want_rows=i32([T - 1]),
                       tables=[table.cuda()], page_size=page, decode_only=(T == 1), max_q_len=T, max_ctx=start + T,
                       h_q_start=[0, T], h_start_pos=[start], h_slots=[0])


@pytest.mark.parametrize("dt", DT)
def test_rms_norm_part(dt):
    from tensorline_b200.parts import NORMS, PartSpec
    norm = NORMS.build(PartSpec("rms_norm", {"dim": 40, "eps": 1e-4}), runtime(dt))
    assert list(norm.expected_tensors("n")) == ["n.weight"] and norm.expected_tensors("n")["n.weight"].shape == (40,)
    w = (1 + rnd(40, seed=1, scale=0.2)).to(torch.bfloat16)
    norm.bind({"n.weight": w.cuda()}, "n")
    x, r = rnd(6, 40, seed=2), rnd(6, 40, seed=3, dtype=dt)
    xd = x.cuda()
    h = norm.add_norm(xd, r.cuda())
    assert h.dtype == dt
    assert_close(h, plain.rms_norm(x.double() + r.double(), w.double(), 1e-4), "norm part", **tol(dt))


def test_rotary_part_table_is_the_plain_table():
    from tensorline_b200.parts import POSITION_ENCODINGS, PartSpec
    pe = POSITION_ENCODINGS.build(PartSpec("rotary_half", {"theta": 12345.0}), runtime(torch.float32), head_dim=48)
    inv_freq, rot = pe.rotary()
    want = (12345.0 ** (-torch.arange(0, 48, 2, dtype=torch.float64) / 48)).float()
    assert rot == 48 and torch.equal(inv_freq.cpu(), want)
    none = POSITION_ENCODINGS.build(PartSpec("none", {}), runtime(torch.float32), head_dim=48)
    assert none.rotary()[1] == 0


@pytest.mark.parametrize("dt", DT)
def test_gated_mlp_part(dt):
    from tensorline_b200.parts import FEED_FORWARDS, PartSpec
    ff = FEED_FORWARDS.build(PartSpec("gated_mlp", {"hidden": 40, "intermediate": 72}), runtime(dt))
    w = {"f.gate_proj.weight": rnd(72, 40, seed=1, scale=0.2, dtype=torch.bfloat16),
         "f.up_proj.weight": rnd(72, 40, seed=2, scale=0.2, dtype=torch.bfloat16),
         "f.down_proj.weight": rnd(40, 72, seed=3, scale=0.2, dtype=torch.bfloat16)}
    assert {k: v.shape for k, v in ff.expected_tensors("f").items()} == {k: tuple(v.shape) for k, v in w.items()}
    ff.bind({k: v.cuda() for k, v in w.items()}, "f")
    h = rnd(9, 40, seed=4, dtype=dt)
    y = ff.forward(h.cuda(), None)
    want = plain.swiglu(h.double(), *(w[f"f.{n}_proj.weight"].double() for n in ("gate", "up", "down")))
    assert_close(y, want, "mlp part", **tol(dt))


def _attention_weights(hidden, nq, nkv, d, seed):
    w = {}
    for i, (n, rows) in enumerate((("q", nq * d), ("k", nkv * d), ("v", nkv * d))):
        # scores of a few units: sharp enough to tell keys apart, not so sharp that the rounding of
        # q and k to bfloat16 moves the softmax by more than the stated tolerance
        w[f"a.{n}_proj.weight"] = rnd(rows, hidden, seed=seed + i, scale=0.12, dtype=torch.bfloat16)
        w[f"a.{n}_proj.bias"] = rnd(rows, seed=seed + 10 + i, scale=0.1, dtype=torch.bfloat16)
    w["a.o_proj.weight"] = rnd(hidden, nq * d, seed=seed + 20, scale=0.2, dtype=torch.bfloat16)
    return w


def _plain_attention_part(h, w, nq, nkv, d, theta, window):
    T = h.shape[0]
    q = plain.linear(h, w["a.q_proj.weight"].double(), w["a.q_proj.bias"].double()).view(T, nq, d)
    k = plain.linear(h, w["a.k_proj.weight"].double(), w["a.k_proj.bias"].double()).view(T, nkv, d)
    v = plain.linear(h, w["a.v_proj.weight"].double(), w["a.v_proj.bias"].double()).view(T, nkv, d)
    cos, sin = plain.rope_cos_sin(range(T), d, theta)
    o = plain.attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, window)
    return plain.linear(o.reshape(T, nq * d), w["a.o_proj.weight"].double())


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("window", [None, 10])
def test_paged_attention_part_whole_and_resumed(dt, window):
    from tensorline_b200.parts import KVCacheView, MIXERS, PartSpec
    hidden, nq, nkv, d, page, pages, theta = 40, 6, 2, 32, 8, 30, 777.0
    mixer = MIXERS.build(PartSpec("paged_attention", {
        "hidden": hidden, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "qkv_bias": True, "window": window,
        "position": PartSpec("rotary_half", {"theta": theta})}), runtime(dt, page))
    need = mixer.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (nkv, d, window)
    w = _attention_weights(hidden, nq, nkv, d, seed=5)
    assert set(mixer.expected_tensors("a")) == set(w)
    mixer.bind({k: v.cuda() for k, v in w.items()}, "a")
    T = 37
    h = rnd(T, hidden, seed=6, dtype=dt)
    want = _plain_attention_part(h.double(), w, nq, nkv, d, theta, window)
    cache = KVCacheView(torch.zeros(pages + 1, nkv, page, d, dtype=dt, device="cuda"),
                        torch.zeros(pages + 1, nkv, page, d, dtype=dt, device="cuda"), 0)
    y = mixer.forward(h.cuda(), one_request_ctx(T, page, pages, seed=1), cache)
    assert_close(y, want, "attention part, whole", **tol(dt))
    # the same request in two portions through the same pages: 30 tokens, then 7 that read them
    cache.k.zero_(); cache.v.zero_()
    mixer.forward(h[:30].cuda(), one_request_ctx(30, page, pages, seed=2), cache)
    ctx2 = one_request_ctx(7, page, pages, start=30, seed=2)
    y2 = mixer.forward(h[30:].cuda(), ctx2, cache)
    assert_close(y2, want[30:], "attention part, resumed", **tol(dt))


@pytest.mark.parametrize("dt", DT)
def test_embedding_and_head_parts(dt):
    from tensorline_b200.parts import Embedding, LMHead
    rt = runtime(dt)
    table = rnd(50, 24, seed=1, dtype=torch.bfloat16)
    emb = Embedding(rt, 50, 24)
    emb.bind({"e.weight": table.cuda()}, "e")
    x = emb.forward(i32([3, 49, 0]))
    assert x.dtype == torch.float32 and torch.equal(x.cpu(), table[[3, 49, 0]].float())
    tied = LMHead(rt, 50, 24, tied=True)
    tied.bind({}, "lm_head", emb)
    h = rnd(4, 24, seed=2, dtype=dt)
    logits = tied.forward(h.cuda())
    assert logits.dtype == torch.float32
    assert_close(logits, h.double() @ table.double().T, "tied head", **(F32 if dt == torch.float32 else dict(rtol=2e-3, atol=2e-3)))
    untied = LMHead(rt, 50, 24, tied=False)
    assert not untied.expected_tensors("lm_head")["lm_head.weight"].optional
    assert tied.expected_tensors("lm_head")["lm_head.weight"].optional


def _tiny_spec(run):
    from tensorline_b200.models import LayerSpec, ModelSpec, RunEntry
    from tensorline_b200.parts import PartSpec
    norm = PartSpec("rms_norm", {"dim": 48, "eps": 1e-5})
    ff = PartSpec("gated_mlp", {"hidden": 48, "intermediate": 80})
    mixer = PartSpec("paged_attention", {"hidden": 48, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                                         "qkv_bias": True, "position": PartSpec("rotary_half", {"theta": 1e4})})
    block = PartSpec("pre_norm", {"mixer": mixer, "feed_forward": ff, "norm1": norm, "norm2": norm})
    layers = tuple(LayerSpec(block, f"model.layers.{i}") for i in range(2))
    return ModelSpec(vocab_size=90, hidden_size=48, layers=layers, run=tuple(RunEntry(*r) for r in run),
                     final_norm=norm, tie_word_embeddings=True)


def _plain_run(w, ids, run, eps=1e-5, nq=3, nkv=1, d=16, theta=1e4):
    """The run list written out with the plain functions; an entry that reads another's cache uses
    that entry's rotated keys and its values."""
    T = len(ids)
    x = plain.embedding(w["model.embed_tokens.weight"], ids)
    cos, sin = plain.rope_cos_sin(range(T), d, theta)
    kv = {}
    for i, (layer, reads) in enumerate(run):
        p = f"model.layers.{layer}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = plain.apply_rope(plain.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, nq, d), cos, sin)
        if reads is None:
            k = plain.apply_rope(plain.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(T, nkv, d), cos, sin)
            v = plain.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(T, nkv, d)
            kv[i] = (k, v)
        else:
            k, v = kv[reads]
        x = x + plain.linear(plain.attention(q, k, v).reshape(T, nq * d), w[p + "self_attn.o_proj.weight"])
        h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + plain.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("run", [
    [(0, None), (1, None), (0, None)],          # layer 0 runs twice, each run with a cache of its own
    [(0, None), (1, None), (1, 0), (0, 1)],     # entries 2 and 3 read the caches of entries 0 and 1
], ids=["layer_twice", "reads_another_cache"])
def test_run_list_is_data(run):
    from tensorline_b200.cache import CacheManager
    from tensorline_b200.engine.runner import ModelRunner, StepEntry
    from tensorline_b200.models import Model
    from tensorline_b200.weights import random_tensor
    model = Model(_tiny_spec(run), runtime(torch.float32, page=4))
    w = {n: random_tensor(3, n, s.shape, 0.0 if "norm" in n else 0.15, 1.0 if "norm" in n else 0.0).to(torch.bfloat16)
         for n, s in model.expected_tensors().items() if not s.optional}
    model.bind({k: v.cuda() for k, v in w.items()})
    owners = [i for i, r in enumerate(run) if r[1] is None]
    assert sorted(model.cache_needs()) == owners
    cache = CacheManager(model.cache_needs(), page_size=4, num_pages=20, max_num_seqs=2, max_model_len=80)
    runner = ModelRunner(model, cache)
    ids = torch.randint(0, 90, (23,), generator=torch.Generator().manual_seed(1)).tolist()
    want = _plain_run({k: v.double() for k, v in w.items()}, ids, run)
    cache.admit("r"); runner.start_request("r")
    got, s = [], 0
    for n in (9, 1, 2, 11):                      # cut into portions: later ones read what earlier ones cached
        cache.grow("r", s, s + n)
        got.append(runner.step([StepEntry("r", ids[s:s + n], list(range(n)))]))
        s += n
    assert_close(torch.cat(got), want, "run list", rtol=3e-5, atol=3e-5)
