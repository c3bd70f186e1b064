"""Command-line parsing: the reference's flag names and its errors (no GPU)."""
import json

import pytest

import helpers
from cajeta_llm_b200 import cli


def test_flags_map_onto_options_and_sampling_parameters():
    o, prompts, p = cli.parse_run(["--model", "m", "--prompt", "1 2,3", "--prompt", "7", "-n", "9", "--temp", "0.7", "--top-k", "40",
                                   "--top-p", "0.95", "--seed", "42", "--repeat-penalty", "1.1", "--ctx", "512", "--max-seqs", "2",
                                   "--block-size", "32", "--chunk", "128", "--dtype", "float32", "--verbose"])
    assert (o.model, o.ctx, o.max_seqs, o.block_tokens, o.chunk, o.dtype, o.verbose) == ("m", 512, 2, 32, 128, "float32", True)
    assert prompts == [[1, 2, 3], [7]]
    assert (p.temperature, p.top_k, p.top_p, p.seed, p.repeat_penalty, p.max_new_tokens) == (0.7, 40, 0.95, 42, 1.1, 9)
    o, _, p = cli.parse_run(["--model", "m", "--prompt", "5"])
    assert (o.ctx, o.max_seqs, o.block_tokens, o.chunk, p.temperature, p.max_new_tokens) == (4096, 4, 16, 0, 0.0, 128)   # the reference's defaults


@pytest.mark.parametrize("args,word", [(["--prompt", "1"], "--model is required"), (["--model", "m"], "--prompt is required"),
                                       (["--model", "m", "--bogus"], "unknown flag '--bogus'"),
                                       (["--model"], "--model needs a value"), (["--model", "m", "--prompt", "a b"], "token ids")])
def test_errors(args, word):
    with pytest.raises(cli.CliError, match=word):
        cli.parse_run(args)


def test_unknown_verb_and_chat(capsys):
    assert cli.main(["fly"]) == 2 and "unknown verb" in capsys.readouterr().err
    assert cli.main(["chat", "--model", "m"]) == 2 and "token ids" in capsys.readouterr().err


def test_random_weights_verb_writes_a_model_folder(tmp_path):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(helpers.TINY_B))
    out = tmp_path / "model"
    assert cli.main(["random-weights", "--config", str(cfg), "--seed", "4", "--out", str(out)]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    import plain_qwen2moe as P
    config, weights = P.read_model(str(out))
    assert config["num_experts"] == 6 and weights["model.layers.1.mlp.experts.0.gate_proj.weight"].shape == (48, 96)
