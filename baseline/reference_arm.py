"""The reference arm of bench.py: tzar-beep/Tensorline itself, unmodified, from baseline/_ref.

Installed offline with
    pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse --target baseline/_ref <copy of the project>
(`--no-deps` because its `accelerate` dependency is not in the wheelhouse; installed from a copy
because the build writes into the source tree).

The reference loads its model and tokenizer by name through an installed package
(tensorline/engine.py:63-66), so this arm first writes a local model folder that package can open:
config.json with the Qwen2.5-7B layer sizes, random N(0, 0.02) bfloat16 weights in safetensors shards,
and a word-level tokenizer whose words are "t<id>" (so a prompt of given token ids is the text
"t5 t17 ...").  Then it drives the reference's own `BatchEngine.stream()` from one thread per request,
as the reference's tests do (tests/test_batching.py:33-45), and reads its public token counter
(`BatchEngine.metrics.tokens_generated`) to time K decode steps of the whole batch after W warm-up
steps.  None of this repository's models, kernels or engine code is on that path.
"""
from __future__ import annotations

import json
import os
import sys
import threading
import time


def _write_model_folder(folder, raw, torch):
    """config.json, sharded random weights, tokenizer files."""
    os.makedirs(folder, exist_ok=True)
    marker = os.path.join(folder, ".complete")
    if os.path.isfile(marker):
        return
    H, I, V = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    nq, nkv, d, L = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["num_hidden_layers"]
    cfg = dict(raw, model_type="qwen2", torch_dtype="bfloat16", bos_token_id=raw["eos_token_id"])
    cfg.pop("head_dim", None) if H // nq == d else None
    json.dump(cfg, open(os.path.join(folder, "config.json"), "w"))
    # weights: one shard per layer, written with this repository's plain container writer (a file format, not a model)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from tensorline_b200.weights.safetensors_io import write_safetensors
    g = torch.Generator(device="cuda").manual_seed(0)
    index = {}

    def rnd(*shape):                                     # drawn on the GPU (fast), stored from the host
        return (torch.randn(*shape, generator=g, device="cuda") * 0.02).to(torch.bfloat16).cpu()

    def shard(name, tensors):
        write_safetensors(os.path.join(folder, name), tensors)
        for k in tensors:
            index[k] = name

    shard("model-embed.safetensors", {"model.embed_tokens.weight": rnd(V, H), "lm_head.weight": rnd(V, H),
                                      "model.norm.weight": torch.ones(H, dtype=torch.bfloat16)})
    for i in range(L):
        p = f"model.layers.{i}."
        shard(f"model-layer{i:02d}.safetensors", {
            p + "self_attn.q_proj.weight": rnd(nq * d, H), p + "self_attn.q_proj.bias": rnd(nq * d),
            p + "self_attn.k_proj.weight": rnd(nkv * d, H), p + "self_attn.k_proj.bias": rnd(nkv * d),
            p + "self_attn.v_proj.weight": rnd(nkv * d, H), p + "self_attn.v_proj.bias": rnd(nkv * d),
            p + "self_attn.o_proj.weight": rnd(H, nq * d),
            p + "mlp.gate_proj.weight": rnd(I, H), p + "mlp.up_proj.weight": rnd(I, H), p + "mlp.down_proj.weight": rnd(H, I),
            p + "input_layernorm.weight": torch.ones(H, dtype=torch.bfloat16),
            p + "post_attention_layernorm.weight": torch.ones(H, dtype=torch.bfloat16)})
    json.dump({"metadata": {}, "weight_map": index}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    # tokenizer: word level, "t<id>", split on whitespace
    vocab = {f"t{i}": i for i in range(V)}
    tok = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
           "pre_tokenizer": {"type": "WhitespaceSplit"}, "post_processor": None, "decoder": None,
           "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "t0"}}
    json.dump(tok, open(os.path.join(folder, "tokenizer.json"), "w"))
    json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": f"t{raw['eos_token_id']}", "unk_token": "t0",
               "model_max_length": 32768}, open(os.path.join(folder, "tokenizer_config.json"), "w"))
    open(marker, "w").write("ok")


def run(args, model_raw: dict, context: int, prompt: int) -> int:
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "_ref")

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if not os.path.isdir(os.path.join(ref, "tensorline")):
        return unavailable("baseline/_ref is not installed on this box (pip install --no-deps of the reference)")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        raw = dict(model_raw)
        if args.layers:
            raw["num_hidden_layers"] = args.layers
        folder = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"tensorline_ref_model_L{raw['num_hidden_layers']}")
        t0 = time.time()
        _write_model_folder(folder, raw, torch)
        print(f"[reference] model folder ready in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        sys.path.insert(0, ref)
        from tensorline.batch_engine import BatchEngine
        from tensorline.engine import GenStats, SamplingParams
        batch, K, W = args.batch, args.steps, args.warmup
        ctx0 = context - (K + W) - 1 - 3 * batch - 8          # as this repository's end-to-end measurement
        per_block = 2 * raw["num_hidden_layers"] * 16 * raw["num_key_value_heads"] * raw["head_dim"] * 2
        eng = BatchEngine(folder, device="cuda", dtype="bfloat16", block_size=16,
                          num_blocks=batch * (context // 16) + 64, max_num_seqs=64, max_batched_tokens=2048,
                          max_model_len=context, prefix_caching=False, spec_tokens=0)
        gen = torch.Generator().manual_seed(1000 + batch)
        prompts = [" ".join(f"t{t}" for t in torch.randint(0, raw["vocab_size"], (ctx0,), generator=gen).tolist())
                   for _ in range(batch)]
        # Requests that finish their prompt early decode while the others are still in chunked prefill
        # (at most 2*batch steps), so timing starts once batch*(W + 2*batch) tokens exist: by then every
        # request is decoding.
        n_start = batch * (W + 2 * batch)
        n_new = W + 2 * batch + K + 8
        stats = [GenStats() for _ in prompts]
        errors = []

        def go(i):
            try:
                for _ in eng.stream(prompts[i], SamplingParams(n_new, stop_token_ids={-1}), stats[i]):
                    pass
            except Exception as e:          # noqa: BLE001
                errors.append(repr(e))

        threads = [threading.Thread(target=go, args=(i,), daemon=True) for i in range(batch)]
        for t in threads:
            t.start()
        t1 = t2 = None
        deadline = time.time() + 900
        while time.time() < deadline and not errors:
            n = eng.metrics.tokens_generated
            now = time.perf_counter()
            if t1 is None and n >= n_start:
                t1, n1 = now, n
            if t1 is not None and n >= n_start + batch * K:
                t2, n2 = now, n
                break
            time.sleep(0.0005)
        for t in threads:
            t.join(timeout=120)
        if errors:
            return unavailable("the reference failed on this box: " + errors[0][:300])
        if t2 is None:
            return unavailable("the reference did not finish the workload within 15 minutes")
        value = (n2 - n1) / (t2 - t1)
        eng.shutdown()
        print(json.dumps({
            "metric": f"decode tok/s at batch {batch} (Qwen2.5-7B bf16, context 4096)", "value": round(value, 1),
            "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(1000.0 * batch / value, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "reference",
            "config": {"model": "Qwen2.5-7B layer sizes, random weights", "layers": raw["num_hidden_layers"],
                       "layers_full": model_raw["num_hidden_layers"], "global_batch": batch, "seq_len": context,
                       "prompt_tokens": ctx0, "page_size": 16, "parallelism": "single GPU",
                       "timing": "wall clock over batch*K tokens of the reference's own token counter, all requests decoding"},
            "e2e": {"value": round(value, 1), "unit": "tok/s"}, "gpu_launches": None}))
        return 0
    except Exception as e:                  # noqa: BLE001
        return unavailable(f"the reference could not run here: {type(e).__name__}: {str(e)[:300]}")
