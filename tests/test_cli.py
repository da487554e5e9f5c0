"""The command line: the reference's option names where both have them, out-of-scope ones refused."""
import json

import pytest

from tensorline_b200 import cli
from tests.tiny import TINY_B


def test_reference_option_names_and_defaults():
    a = cli._generate_parser().parse_args(["--model", "m"])
    assert (a.max_num_seqs, a.max_batched_tokens, a.num_blocks, a.kv_cache_gb) == (64, 2048, None, None)
    assert (a.device, a.dtype, a.graph_warmup_tokens) == ("auto", "auto", 512)
    assert not (a.no_cuda_graphs or a.no_overlap or a.no_prefix_caching)


@pytest.mark.parametrize("flag", ["--quant", "--serve", "--spec-tokens", "--port"])
def test_out_of_scope_options_are_refused_by_name(flag, capsys):
    assert cli.main(["--model", "m", flag, "x"]) == 2
    assert flag in capsys.readouterr().err


def test_random_weights_writes_a_model_folder(tmp_path):
    (tmp_path / "c.json").write_text(json.dumps(TINY_B))
    out = tmp_path / "model"
    assert cli.main(["random-weights", "--config", str(tmp_path / "c.json"), "--out", str(out), "--seed", "3",
                     "--std", "0.05", "--norm-std", "0.1"]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    assert json.loads((out / "config.json").read_text())["num_hidden_layers"] == 3


@pytest.mark.gpu
def test_generate_from_the_command_line(tmp_path, capsys):
    from tests.plain.qwen2_plain import PlainQwen2, greedy_generate
    from tests.tiny import write_tiny
    folder = write_tiny("B_FULL", tmp_path / "m")
    assert cli.main(["--model", str(folder), "--dtype", "float32", "--prompt-ids", "5,9,200,17", "--prompt-ids", "7",
                     "--max-tokens", "5", "--ignore-eos", "--block-size", "8", "--num-blocks", "16",
                     "--max-num-seqs", "4", "--max-model-len", "64"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    plain = PlainQwen2(folder)
    assert [l["token_ids"] for l in lines] == [greedy_generate(plain, [5, 9, 200, 17], 5), greedy_generate(plain, [7], 5)]
    assert all(l["finish_reason"] == "length" for l in lines)
