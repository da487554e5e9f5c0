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

    before = ops.kernel_counts.copy()
    pair = prompt("pair")
    ran = ops.kernel_counts - before
    assert ran["attn_tc2_prefill"] == cfg.num_hidden_layers and not ran["attn_tc_prefill"], ran      # observed, not inferred
    decoded = [runner.step([StepEntry("pair", [ids[n + i]], [0])]).double().cpu()[0] for i in range(extra) if cache.grow("pair", n + i, n + i + 1)]
    cache.release("pair"); runner.end_request("pair")
    ops_attention.TC_PAIR = False
    try:
        before = ops.kernel_counts.copy()
        single = prompt("single")
        ran = ops.kernel_counts - before
        assert ran["attn_tc_prefill"] == cfg.num_hidden_layers and not ran["attn_tc2_prefill"], ran
        cache.grow("single", n, n + extra)
        portion = runner.step([StepEntry("single", ids[n:n + extra], list(range(extra)))]).double().cpu()
        cache.release("single"); runner.end_request("single")
    finally:
        ops_attention.TC_PAIR = True
    exact = prompt("exact", exact=True)
    cache.release("exact"); runner.end_request("exact")
    from tests.plain.qwen2_plain import PlainQwen2, forward
    plain = PlainQwen2.from_tensors(SIZES, weights, dtype=torch.float32)
    want = forward(plain, ids[:n], rows=[0, 700, n - 1]).double()            # the plain model on the same three rows
    for what, got in (("two-tile", pair), ("one-tile", single), ("exact-order", exact)):
        err = float((got - want).abs().max())
        assert err <= BF16_MODEL_REL * float(want.abs().max()), f"{what} against the plain model: {err:.3e}"
    scale = float(exact.abs().max())
    for what, got in (("two-tile", pair), ("one-tile", single)):
        err = float((got - exact).abs().max())
        assert err <= BF16_MODEL_REL * scale, f"{what} against exact-order attention: {err:.3e} (scale {scale:.3f})"
    err = float((torch.stack(decoded) - portion).abs().max())
    assert err <= BF16_MODEL_REL * float(portion.abs().max()), f"decoded one by one against a portion: {err:.3e}"


@pytest.mark.parametrize("batch", [8, 33])
def test_decode_graph_at_these_sizes_agrees_with_the_32_bit_engine_and_the_plain_model(big, batch):
    """The step the benchmark times, asserted: `batch` requests at contexts of 1,000 to 1,500 keys decode through
    the CUDA graph of their bucket (a padding row or more at 33).  Inside it: the tcgen05 product with 16- or
    64-token tiles, its gated epilogue, split-K sums inside clusters or left to their consumers, at batch 8 the norms
    folded into the products around them and the rotary step folded into the TMA decode attention, whose key ranges
    merge inside clusters (observed from the captured graph, not inferred).  The logits are compared with
    the 32-bit engine on the same weights and schedule (every row) and with the plain model (two rows)."""
    from tensorline_b200 import Engine, ops
    from tensorline_b200.engine.runner import StepEntry
    from tests.plain.qwen2_plain import PlainQwen2, forward
    cfg, weights = big[0], big[1]
    g = torch.Generator().manual_seed(40 + batch)
    lens = [1000 + int(x) for x in torch.randint(0, 500, (batch,), generator=g)]
    seqs = [torch.randint(0, cfg.vocab_size, (n + 3,), generator=g).tolist() for n in lens]
    pages = sum(-(-(n + 3) // 16) for n in lens) + 4
    out = {}
    for dtype in ("bfloat16", "float32"):
        eng = Engine(cfg, dtype=dtype, weights=dict(weights), block_size=16, num_blocks=pages, max_num_seqs=64,
                     max_model_len=2048, prefix_caching=False, cuda_graphs=True)
        runner, cache = eng.runner, eng.cache
        for i, (n, toks) in enumerate(zip(lens, seqs)):
            cache.admit(i); runner.start_request(i)
            assert cache.grow(i, 0, n + 3)
            for s in range(0, n, 2048):
                runner.step([StepEntry(i, toks[s:min(n, s + 2048)], [])])
        steps = []
        for k in range(3):                                   # three decode steps through the graph
            entries = [StepEntry(i, [seqs[i][lens[i] + k]], [0]) for i in range(batch)]
            assert runner.can_replay(entries)
            steps.append(runner.step_graph(entries).double().cpu())
        out[dtype] = torch.stack(steps)
        if dtype == "bfloat16":
            kernels = runner.graph_kernels(batch)
            bn = 16 if batch <= 16 else 64
            assert any(k.startswith(f"gemm_tc<{bn}>") for k in kernels), kernels
            assert any("+gated" in k for k in kernels) and any("+cluster" in k or "+pieces" in k for k in kernels), kernels
            assert any(k.startswith("attn_decode_tma") for k in kernels), kernels
            if batch == 8:                                # key ranges merged inside clusters, the rotary step folded in,
                assert "attn_decode_tma+rope+cluster" in kernels and "rope_kv_write" not in kernels, kernels
                assert any(k.endswith("+normed") for k in kernels) and any(k.endswith("+residual") for k in kernels), kernels
                assert kernels["add_rmsnorm"] == 2, kernels     # the first layer's first norm and the last norm: the rest are folded
            assert runner._bucket(batch) > batch or batch == 8
        ops.check_device_status()
        del eng, runner, cache
        torch.cuda.empty_cache()
    scale = float(out["float32"].abs().max())
    err = float((out["bfloat16"] - out["float32"]).abs().max())
    assert err <= BF16_MODEL_REL * scale, f"bfloat16 graph decode against the 32-bit engine: {err:.3e} (scale {scale:.3f})"
    plain = PlainQwen2.from_tensors(SIZES, weights, dtype=torch.float32)
    for i in (0, batch - 1):
        want = forward(plain, seqs[i][:lens[i] + 3], rows=[lens[i], lens[i] + 2]).double()
        got32 = torch.stack([out["float32"][0][i], out["float32"][2][i]])
        got16 = torch.stack([out["bfloat16"][0][i], out["bfloat16"][2][i]])
        assert float((got32 - want).abs().max()) <= 2e-4 * max(1.0, scale)
        assert float((got16 - want).abs().max()) <= BF16_MODEL_REL * scale


def test_two_decode_attention_blocks_share_an_sm_at_the_measured_sizes():
    """The plan of the key ranges counts on two blocks an SM.  A block's shared memory grows with the cluster's number of
    ranges (the receive area) and with its block-table copy, and 64 bytes too many halve the occupancy (it happened:
    32B sizes, attention 26 instead of 16 us).  The launches of the measured configurations stay within the limit."""
    import ctypes
    from tensorline_b200 import ops_attention
    lib = ops_attention.attn_lib(128)
    lib.tl_attn_decode_tma_smem.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.tl_attn_decode_tma_smem.restype = ctypes.c_int
    per_sm = 228 * 1024
    for name, batch, nkv, group, context in (("7B", 8, 4, 7, 4096), ("7B", 1, 4, 7, 4096), ("7B", 4, 4, 7, 4096), ("7B", 16, 4, 7, 4096),
                                             ("14B", 8, 8, 5, 4096), ("32B", 8, 8, 5, 3072), ("32B", 1, 8, 5, 3072), ("7B", 8, 4, 7, 32768)):
        chunk, splits = ops_attention.plan_splits(batch, nkv, group, context, 128, page_size=16)
        ranges = splits if 2 <= splits <= 16 else 0
        smem = lib.tl_attn_decode_tma_smem(ranges, chunk // 16)
        assert 2 * (smem + 1024) <= per_sm, (name, batch, context, chunk, splits, smem)
