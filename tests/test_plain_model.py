"""The plain implementation against the reference's own model code (through
the committed golden files) and against itself."""

from pathlib import Path

import pytest
import torch

import plain_model
from golden_inputs import golden_prompt, golden_weights
from tiny_configs import TINY

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", sorted(TINY))
def test_plain_matches_reference_model_code(name):
    config, seed, _ = TINY[name]
    golden = torch.load(GOLDEN / f"{name}.pt")
    assert golden["prompt"] == golden_prompt(config, seed)
    weights = golden_weights(config, seed)
    logits = plain_model.forward_logits(config, weights, golden["prompt"])
    assert logits.shape == golden["logits"].shape
    assert (logits - golden["logits"]).abs().max().item() < 1e-5


def test_plain_is_causal():
    config, seed, _ = TINY["qwen3"]
    weights = golden_weights(config, seed)
    prompt = golden_prompt(config, seed, 40)
    full = plain_model.forward_logits(config, weights, prompt)
    prefix = plain_model.forward_logits(config, weights, prompt[:17])
    assert (full[:17] - prefix).abs().max().item() < 1e-5


def test_plain_llama3_scaling_changes_low_frequencies():
    config, _, _ = TINY["llama"]
    cfg = plain_model.plain_config(config)
    scaled_cos, _ = plain_model.rope_cos_sin(cfg, torch.arange(100))
    plain_cfg = dict(cfg, rope_kind=None)
    cos, _ = plain_model.rope_cos_sin(plain_cfg, torch.arange(100))
    # the highest frequency is untouched, the lowest is divided by the factor
    assert torch.equal(scaled_cos[:, 0], cos[:, 0])
    assert not torch.allclose(scaled_cos[:, cfg["head_dim"] // 2 - 1], cos[:, cfg["head_dim"] // 2 - 1])


def test_plain_sampler_is_a_pure_function_of_seed_and_position():
    logits = torch.randn(97, generator=torch.Generator().manual_seed(3))
    a = plain_model.sample_token(logits, temperature=0.8, top_p=0.9, base_seed=7, position=3)
    b = plain_model.sample_token(logits, temperature=0.8, top_p=0.9, base_seed=7, position=3)
    assert a == b
    draws = {plain_model.sample_token(logits, temperature=1.5, base_seed=7, position=p) for p in range(40)}
    assert len(draws) > 5
    assert plain_model.sample_token(logits, temperature=0.0, base_seed=1, position=0) == int(logits.argmax())


def test_plain_filters():
    logits = torch.log(torch.tensor([0.5, 0.2, 0.15, 0.1, 0.05]))
    assert (plain_model.filtered_probs(logits, 1.0, 2, 1.0, 0.0) > 0).tolist() == [True, True, False, False, False]
    assert (plain_model.filtered_probs(logits, 1.0, -1, 0.6, 0.0) > 0).tolist() == [True, True, False, False, False]
    assert (plain_model.filtered_probs(logits, 1.0, -1, 1.0, 0.25) > 0).tolist() == [True, True, True, False, False]
