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


def test_the_engine_tables_are_the_plain_ones_bit_for_bit():
    """The engine's cos/sin tables (default, llama3, yarn) against the plain model's, which the
    golden files anchor on the reference's own code; the yarn one also against its definition:
    pair 0 keeps its frequency, the last pair is slowed ``factor`` times, cos and sin carry
    0.1 ln(factor) + 1."""
    import math

    from kairyu_b200.models.llama import parse_llama as parse_config
    from kairyu_b200.parts.rope import rotary_tables

    for name in sorted(TINY):
        config = TINY[name][0]
        parsed = parse_config(config)
        cfg = plain_model.plain_config(config)
        cos, sin = rotary_tables(parsed.head_dim, parsed.rope_theta, parsed.rope_scaling, parsed.max_position_embeddings)
        plain_cos, plain_sin = plain_model.rope_cos_sin(cfg, torch.arange(parsed.max_position_embeddings))
        half = parsed.head_dim // 2
        assert torch.equal(cos, plain_cos[:, :half]) and torch.equal(sin, plain_sin[:, :half]), name
    config = TINY["yarn"][0]
    parsed = parse_config(config)
    assert parsed.rope_scaling.kind == "yarn" and parsed.rope_theta == 10000.0
    cos, sin = rotary_tables(parsed.head_dim, parsed.rope_theta, parsed.rope_scaling, 256)
    amplitude = 0.1 * math.log(4.0) + 1.0
    assert abs(float(cos[0, 0]) - amplitude) < 1e-6 and float(sin[0].abs().max()) == 0.0
    unscaled, _ = rotary_tables(parsed.head_dim, parsed.rope_theta, None, 256)
    assert torch.allclose(cos[:, 0], unscaled[:, 0] * amplitude, atol=1e-6)  # the fastest pair is kept
    last = parsed.head_dim // 2 - 1
    slow = torch.cos(torch.arange(256, dtype=torch.float32) * (10000.0 ** (-2 * last / parsed.head_dim)) / 4.0) * amplitude
    assert torch.allclose(cos[:, last], slow, atol=1e-5)  # the slowest pair sees positions divided by the factor
    middle = 4  # between the ends, neither kept nor fully slowed
    assert not torch.allclose(cos[:, middle], unscaled[:, middle] * amplitude, atol=1e-3)
