"""The `tensorline` command.

tzar-beep/Tensorline's command starts an HTTP server (tensorline/server.py:251-302); servers are
not part of this engine, so the command generates directly and prints one JSON line per prompt.
Options that both have keep the reference's names, meanings and defaults (server.py:257-278):
--model (or $TL_MODEL), --device, --dtype, --max-num-seqs, --max-batched-tokens, --num-blocks,
--no-cuda-graphs, --no-overlap, --graph-warmup-tokens, --no-prefix-caching, --kv-cache-gb.
Its server, quantization, speculation and multi-model options (--host, --port, --engine, --quant,
--spec-tokens, --serve, --gpu-budget-gb) have no counterpart and are refused by name.

    tensorline --model DIR --prompt-ids 1,2,3 --max-tokens 16
    tensorline random-weights --config config.json --out DIR --seed 0
    tensorline replay --model DIR --dtype float32 --out DIR --max-tokens 4096 < trace.jsonl
    tensorline bench [--model 7b|14b|32b] [--workload decode|mix] [--profile] ...
"""
from __future__ import annotations

import argparse
import json
import os
import sys

OUT_OF_SCOPE = ("--host", "--port", "--engine", "--quant", "--spec-tokens", "--serve", "--gpu-budget-gb")


def _generate_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser("tensorline", description="generate with the B200 engine")
    ap.add_argument("--model", default=os.getenv("TL_MODEL"), help="model folder (config.json, model.safetensors)")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default="auto", help="auto (bfloat16), bfloat16 or float32")
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-batched-tokens", type=int, default=2048)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-blocks", type=int, default=None, help="KV pages (default: fit 60%% of free memory)")
    ap.add_argument("--kv-cache-gb", type=float, default=None, help="KV cache size (default: 60%% of free memory)")
    ap.add_argument("--no-cuda-graphs", action="store_true", help="run decode steps eagerly")
    ap.add_argument("--no-overlap", action="store_true", help="read every decode step back before the next one is launched")
    ap.add_argument("--graph-warmup-tokens", type=int, default=512,
                    help="accepted; decode graphs here do not depend on the context length")
    ap.add_argument("--no-prefix-caching", action="store_true", help="never reuse KV pages across requests")
    ap.add_argument("--prompt", action="append", default=[], help="text prompt (needs tokenizer files); repeatable")
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeatable")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    return ap


def _load_tokenizer(folder):
    """A tokenizer, if the folder has one: text is a convenience of the command, token ids are the
    engine's interface."""
    if not any(os.path.isfile(os.path.join(folder, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
        return None
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(folder)


def cmd_generate(argv) -> int:
    for flag in OUT_OF_SCOPE:
        if any(a == flag or a.startswith(flag + "=") for a in argv):
            print(f"tensorline: {flag} belongs to the reference's server, quantization, speculation or "
                  "multi-model serving, which this engine does not have", file=sys.stderr)
            return 2
    a = _generate_parser().parse_args(argv)
    if not a.model:
        print("tensorline: --model (or $TL_MODEL) is required", file=sys.stderr)
        return 2
    from . import Engine, SamplingParams
    tok = _load_tokenizer(a.model) if a.prompt else None
    eng = Engine(a.model, a.device, a.dtype, tokenizer=tok, block_size=a.block_size, num_blocks=a.num_blocks,
                 max_num_seqs=a.max_num_seqs, max_batched_tokens=a.max_batched_tokens, max_model_len=a.max_model_len,
                 cuda_graphs=not a.no_cuda_graphs, prefix_caching=not a.no_prefix_caching, kv_cache_gb=a.kv_cache_gb,
                 graph_warmup_tokens=a.graph_warmup_tokens, overlap=not a.no_overlap, seed=a.seed)
    prompts = list(a.prompt) + [[int(t) for t in s.split(",") if t.strip()] for s in a.prompt_ids]
    if not prompts:
        print("tensorline: give --prompt or --prompt-ids", file=sys.stderr)
        return 2
    params = [SamplingParams(max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p,
                             seed=a.seed + i if a.temperature > 0 else None, ignore_eos=a.ignore_eos)
              for i in range(len(prompts))]
    for out in eng.generate(prompts, params):
        print(json.dumps({"token_ids": out.token_ids, "text": out.text, "finish_reason": out.finish_reason,
                          "prompt_tokens": out.stats.prompt_tokens, "completion_tokens": out.stats.completion_tokens,
                          "cached_tokens": out.stats.cached_tokens, "ttft_s": round(out.stats.ttft_s, 6),
                          "total_s": round(out.stats.total_s, 6)}))
    return 0


def cmd_random_weights(argv) -> int:
    ap = argparse.ArgumentParser("tensorline random-weights")
    ap.add_argument("--config", required=True, help="a config.json of a registered architecture")
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--std", type=float, default=0.02)
    ap.add_argument("--norm-std", type=float, default=0.0, help="norm weights are 1 + N(0, this)")
    ap.add_argument("--store", choices=["bfloat16", "float32"], default="bfloat16")
    a = ap.parse_args(argv)
    import torch
    from .models import architecture, expected_tensors
    from .config import architecture_name
    from .weights import write_random_model
    raw = json.load(open(a.config))
    cfg = architecture(architecture_name(raw)).config_class.from_dict(raw, where=a.config)
    write_random_model(a.out, cfg, expected_tensors(cfg), seed=a.seed, std=a.std, norm_std=a.norm_std,
                       store_dtype=getattr(torch, a.store))
    print(a.out)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "random-weights":
        return cmd_random_weights(argv[1:])
    if argv and argv[0] == "replay":
        from .replay import main as replay_main
        return replay_main(argv[1:])
    if argv and argv[0] == "bench":
        from .benchmark import main as bench_main
        return bench_main(argv[1:])
    if argv and argv[0] == "generate":
        argv = argv[1:]
    return cmd_generate(argv)


if __name__ == "__main__":
    sys.exit(main())
