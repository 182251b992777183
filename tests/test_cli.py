"""The command line: make-random, validate, and generate through the parser."""

import json

import pytest

from tiny_configs import TINY_QWEN3

from kairyu_b200.entrypoints import cli


def test_make_random_and_validate(tmp_path, capsys):
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(TINY_QWEN3))
    cli.main(["make-random", str(config_path), str(tmp_path / "model"), "--seed", "3", "--dtype", "float32"])
    assert (tmp_path / "model" / "model.safetensors").exists()
    cli.main(["validate", str(tmp_path / "model")])
    assert "valid: Qwen3ForCausalLM, 3 layers" in capsys.readouterr().out
    (tmp_path / "model" / "model.safetensors").unlink()
    with pytest.raises(SystemExit):
        cli.main(["validate", str(tmp_path / "model")])
    assert "invalid" in capsys.readouterr().out


def test_generate_flags_are_the_sampling_fields():
    parser = cli._build_parser()
    args = parser.parse_args(
        ["generate", "m", "--prompt-token-ids", "1,2,3", "--temperature", "0.8", "--top-p", "0.9", "--top-k", "5",
         "--min-p", "0.1", "--seed", "4", "--max-tokens", "7", "--repetition-penalty", "1.1", "--ignore-eos",
         "--logprobs", "4", "--enable-prefix-caching", "--pipeline-depth", "2"]
    )
    assert args.logprobs == 4 and args.enable_prefix_caching and args.pipeline_depth == 2
    assert (args.temperature, args.top_p, args.top_k, args.min_p, args.seed, args.max_tokens) == (0.8, 0.9, 5, 0.1, 4, 7)
    assert args.ignore_eos and args.repetition_penalty == 1.1
    with pytest.raises(SystemExit):
        parser.parse_args(["serve", "x.yaml"])  # this engine has no server
