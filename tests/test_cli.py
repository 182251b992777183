"""The command line: make-random, validate, and generate, run on the CPU with the
torch statements of the kernels and on the GPU with the kernels, against the plain model."""

import json

import pytest
import torch
from safetensors.torch import load_file

import plain_model
import torch_kernels
from tiny_configs import TINY_LLAMA, TINY_QWEN3

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


def _generate_through_the_cli(tmp_path, capsys, config, device):
    """make-random writes a folder, generate reads it: the greedy tokens are the plain model's."""
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(config))
    folder = tmp_path / "model"
    cli.main(["make-random", str(config_path), str(folder), "--seed", "11", "--dtype", "float32"])
    capsys.readouterr()
    prompts = [[5, 17, 3, 9], [1], list(range(20, 60))]
    cli.main(
        ["generate", str(folder), "--dtype", "float32", "--device", device, "--temperature", "0", "--max-tokens", "9",
         "--num-pages", "24", "--max-num-seqs", "4"] + [arg for p in prompts for arg in ("--prompt-token-ids", ",".join(map(str, p)))]
    )
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert [line["prompt_token_ids"] for line in lines] == prompts
    weights = {name: tensor.float() for name, tensor in load_file(str(folder / "model.safetensors")).items()}
    for prompt, line in zip(prompts, lines):
        tokens = list(prompt)
        for _ in range(9):
            tokens.append(int(plain_model.forward_logits(config, weights, tokens)[-1].argmax()))
        assert line["outputs"][0]["token_ids"] == tokens[len(prompt):]
        assert line["outputs"][0]["finish_reason"] == "length"
    return folder, weights


def test_generate_runs_on_the_cpu_stand_ins(tmp_path, capsys, monkeypatch):
    torch_kernels.install(monkeypatch)
    _generate_through_the_cli(tmp_path, capsys, TINY_LLAMA, "cpu")


def test_llm_over_a_model_folder(tmp_path, capsys, monkeypatch):
    """``LLM(folder)``: the constructor a user calls, with sampling through seeds."""
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    torch_kernels.install(monkeypatch)
    folder, weights = _generate_through_the_cli(tmp_path, capsys, TINY_QWEN3, "cpu")
    llm = LLM(str(folder), dtype="float32", device="cpu", num_pages=24, page_size=8, max_num_seqs=4)
    prompt = [7, 8, 9, 10, 11]
    output = llm.generate(TokensPrompt(tuple(prompt)), SamplingParams(temperature=0.7, top_p=0.9, seed=3, max_tokens=6))[0]
    tokens = list(prompt)
    for position in range(6):
        logits = plain_model.forward_logits(TINY_QWEN3, weights, tokens)[-1]
        tokens.append(plain_model.sample_token(logits, base_seed=3, position=position, temperature=0.7, top_p=0.9))
    assert list(output.outputs[0].token_ids) == tokens[len(prompt):]


@pytest.mark.gpu
def test_generate_runs_on_the_gpu(tmp_path, capsys):
    assert torch.cuda.is_available()
    _generate_through_the_cli(tmp_path, capsys, TINY_LLAMA, "cuda")
