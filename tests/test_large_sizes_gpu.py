"""The engine at the layer sizes of Qwen2.5-7B (two layers of them, random weights N(0, 0.02)): widths
that are no power of two (3584, 18944), 28 query heads in groups of 7, head size 128, vocabulary
152064.  The 32-bit engine and the bfloat16 engine are compared with the plain model: a whole prompt,
then the same prompt in portions with decoded tokens, through the Python entry point's runner."""
import pytest
import torch

from tests.gpu_helpers import BF16_MODEL_REL

pytestmark = pytest.mark.gpu

SIZES = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=3584, num_attention_heads=28,
             num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1e6,
             rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False, max_position_embeddings=32768,
             hidden_act="silu", eos_token_id=151645)


@pytest.fixture(scope="module")
def big():
    from tensorline_b200 import Qwen2Config
    from tensorline_b200.models import expected_tensors
    from tests.plain.qwen2_plain import PlainQwen2, forward
    cfg = Qwen2Config.from_dict(SIZES)
    g = torch.Generator(device="cuda").manual_seed(5)
    weights = {}
    for name, spec in expected_tensors(cfg).items():
        if spec.init == "ones":
            weights[name] = (1 + 0.1 * torch.randn(spec.shape, device="cuda", generator=g)).to(torch.bfloat16)
        else:
            weights[name] = (0.02 * torch.randn(spec.shape, device="cuda", generator=g)).to(torch.bfloat16)
    ids = torch.randint(0, cfg.vocab_size, (83,), generator=torch.Generator().manual_seed(6)).tolist()
    rows = [0, 1, 40, 63, 64, 81, 82]
    plain = PlainQwen2.from_tensors(SIZES, weights, dtype=torch.float32)      # float32 on the CPU: fast enough, and
    want = forward(plain, ids, rows=rows).double()                           # its rounding is far below the tolerances
    return cfg, weights, ids, rows, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_seven_b_layer_sizes_match_the_plain_model(big, dtype):
    from tensorline_b200 import Engine
    from tensorline_b200.engine.runner import StepEntry
    cfg, weights, ids, rows, want = big
    eng = Engine(cfg, dtype=dtype, weights=dict(weights), block_size=16, num_blocks=32, max_num_seqs=4,
                 max_model_len=256, prefix_caching=False)
    runner, cache = eng.runner, eng.cache
    scale = float(want.abs().max())

    def run(cuts, rid):
        cache.admit(rid); runner.start_request(rid)
        got, s = {}, 0
        for n in cuts:
            cache.grow(rid, s, s + n)
            wanted = [r - s for r in rows if s <= r < s + n]
            out = runner.step([StepEntry(rid, ids[s:s + n], wanted)]).double().cpu()
            for i, w in enumerate(wanted):
                got[s + w] = out[i]
            s += n
        cache.release(rid); runner.end_request(rid)
        return torch.stack([got[r] for r in rows])

    whole = run([83], "whole")
    cut = run([40, 23, 2, 16, 1, 1], "cut")
    for what, got in (("whole", whole), ("portions", cut)):
        err = float((got - want).abs().max())
        if dtype == "float32":
            assert err <= 2e-4 * max(1.0, scale), f"{what}: max abs err {err:.3e} (logit scale {scale:.3f})"
        else:
            assert err <= BF16_MODEL_REL * scale, f"{what}: max abs err {err:.3e} (logit scale {scale:.3f})"
    if dtype == "float32":
        assert torch.equal(whole, cut)


def test_long_prompt_takes_the_two_tile_attention_and_agrees_with_the_other_kernels(big):
    """A 1,600-token prompt at these sizes fills the GPU with blocks of two query tiles, so the step runs the
    two-tile tcgen05 attention; the same prompt with that kernel switched off (one-tile kernel), and then with
    the exact-order attention, must give the same logits within bfloat16 rounding.  Then 8 tokens are decoded
    on top (split-K pieces summed by their consumers, activation in the product's epilogue) in one step each
    and together as a portion."""
    from tensorline_b200 import Engine, ops, ops_attention
    from tensorline_b200.engine.runner import StepEntry
    cfg, weights = big[0], big[1]
    n, extra = 1600, 8
    ids = torch.randint(0, cfg.vocab_size, (n + extra,), generator=torch.Generator().manual_seed(9)).tolist()
    eng = Engine(cfg, dtype="bfloat16", weights=dict(weights), block_size=16, num_blocks=240, max_num_seqs=2,
                 max_model_len=2048, prefix_caching=False, cuda_graphs=False)
    runner, cache = eng.runner, eng.cache

    def prompt(rid, exact=False):
        cache.admit(rid); runner.start_request(rid)
        cache.grow(rid, 0, n)
        runner.force_exact_attention = exact
        try:
            return runner.step([StepEntry(rid, ids[:n], [0, 700, n - 1])]).double().cpu()
        finally:
            runner.force_exact_attention = False

    before = ops.launch_count()
    pair = prompt("pair")
    assert ops.launch_count() > before
    g = cfg.num_attention_heads // cfg.num_key_value_heads
    assert -(-n * g // 256) * cfg.num_key_value_heads >= 0.7 * ops_attention.NUM_SMS      # the two-tile kernel did run
    decoded = [runner.step([StepEntry("pair", [ids[n + i]], [0])]).double().cpu()[0] for i in range(extra) if cache.grow("pair", n + i, n + i + 1)]
    cache.release("pair"); runner.end_request("pair")
    ops_attention.TC_PAIR = False
    try:
        single = prompt("single")
        cache.grow("single", n, n + extra)
        portion = runner.step([StepEntry("single", ids[n:n + extra], list(range(extra)))]).double().cpu()
        cache.release("single"); runner.end_request("single")
    finally:
        ops_attention.TC_PAIR = True
    exact = prompt("exact", exact=True)
    cache.release("exact"); runner.end_request("exact")
    scale = float(exact.abs().max())
    for what, got in (("two-tile", pair), ("one-tile", single)):
        err = float((got - exact).abs().max())
        assert err <= BF16_MODEL_REL * scale, f"{what} against exact-order attention: {err:.3e} (scale {scale:.3f})"
    err = float((torch.stack(decoded) - portion).abs().max())
    assert err <= BF16_MODEL_REL * float(portion.abs().max()), f"decoded one by one against a portion: {err:.3e}"
