"""The plain implementation itself: against the outputs of tzar-beep/Tensorline's own paged model
(tests/golden/reference_logits.json, made by tests/golden/make_golden.py) and against its own parts."""
import json
from pathlib import Path

import pytest
import torch

from tests.plain import qwen2_plain as plain
from tests.tiny import random_tokens, write_tiny

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_logits.json").read_text())


@pytest.mark.parametrize("name", ["A", "B_FULL"])
def test_plain_matches_the_reference_projects_outputs(name, tmp_path):
    """Against the reference as it really runs (its own loader's model object under its paged model: `as_it_runs/*`)
    and against its paged model over a stand-in written from the formulas (`shim/*`), three schedules each."""
    rec = GOLDEN[name]
    folder = write_tiny(name, tmp_path / "m", seed=0)
    weights = plain.read_safetensors(folder / "model.safetensors")
    checksum = float(sum(v.double().abs().sum() for v in weights.values()))
    assert checksum == pytest.approx(rec["weights_abs_sum"], rel=1e-12), "the seeded weights changed"
    logits = plain.forward(plain.PlainQwen2(folder), rec["ids"])[rec["position"]]
    assert sorted(rec["logits"]) == sorted(f"{how}/{cut}" for how in ("as_it_runs", "shim")
                                           for cut in ("whole", "chunks_of_3", "decode_tail"))
    for how, ref in rec["logits"].items():
        ref = torch.tensor(ref, dtype=torch.float64)
        assert float((logits - ref).abs().max()) < 2e-5, how          # the reference ran in float32


def test_plain_window_model_generates_what_the_reference_engine_generated(tmp_path):
    """Tiny B (layers 1 and 2 see the last 24 keys): greedy tokens of the reference's one-request engine, as stored
    by tests/golden/make_golden.py, for prompts longer than the window; the same weights without the window give
    other tokens, so the comparison pins `sliding_window` and `max_window_layers`."""
    rec = GOLDEN["B"]
    folder = write_tiny("B", tmp_path / "m", seed=0)
    weights = plain.read_safetensors(folder / "model.safetensors")
    assert float(sum(v.double().abs().sum() for v in weights.values())) == pytest.approx(rec["weights_abs_sum"], rel=1e-12)
    m = plain.PlainQwen2(folder)
    full = plain.PlainQwen2(write_tiny("B_FULL", tmp_path / "f", seed=0))
    assert rec["window"] == 24 and len(rec["greedy"]) == 2
    for case in rec["greedy"]:
        assert len(case["prompt"]) > rec["window"]
        assert plain.greedy_generate(m, case["prompt"], len(case["tokens"])) == case["tokens"]
        assert plain.greedy_generate(full, case["prompt"], len(case["tokens"])) != case["tokens"]


def test_window_layer_sees_only_its_window(tmp_path):
    m = plain.PlainQwen2(write_tiny("B", tmp_path / "m"))
    assert m.window == [None, 24, 24]
    T, d = 60, 32
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(T, 3, d, generator=g, dtype=torch.float64),
               torch.randn(T, 1, d, generator=g, dtype=torch.float64),
               torch.randn(T, 1, d, generator=g, dtype=torch.float64))
    full, win = plain.attention(q, k, v), plain.attention(q, k, v, window=24)
    assert torch.allclose(full[:24], win[:24]) and not torch.allclose(full[30:], win[30:])
    v2 = v.clone()
    v2[:10] += 100.0                                                   # keys 0..9 are outside the window of query 40
    assert torch.allclose(plain.attention(q, k, v2, window=24)[34:], win[34:])


def test_rope_is_a_rotation_and_position_zero_is_identity():
    cos, sin = plain.rope_cos_sin([0, 5, 4000], 16, 1e4)
    x = torch.randn(3, 2, 16, dtype=torch.float64)
    y = plain.apply_rope(x, cos, sin)
    assert torch.equal(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))


def test_greedy_generation_appends_argmax(tmp_path):
    m = plain.PlainQwen2(write_tiny("A", tmp_path / "m"))
    prompt = random_tokens(256, 5, 1)
    out = plain.greedy_generate(m, prompt, 3)
    assert out[0] == int(plain.forward(m, prompt)[-1].argmax())
    assert out[1] == int(plain.forward(m, prompt + out[:1])[-1].argmax())


def test_top_p_keeps_the_reference_nucleus():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0])
    p = plain.sampling_distribution(logits, 1.0, 0.7)      # masses .644, .237, ...: first two are kept
    assert (p > 0).tolist() == [True, True, False, False] and float(p.sum()) == pytest.approx(1.0)
    assert plain.inverse_cdf_pick(p, 0.0) == 0 and plain.inverse_cdf_pick(p, 0.99) == 1
