"""SamplingParams validation and the sampler's host side (which edits and seeds
it builds), with the selection kernels replaced by their torch statements."""

import pytest
import torch

import plain_model
import torch_kernels

from kairyu_b200.sampling import Sampler, SamplingParams, SamplingRow, mix_seed, stable_request_seed


@pytest.fixture(autouse=True)
def cpu_kernels(monkeypatch):
    torch_kernels.install(monkeypatch)


def test_defaults_follow_the_reference():
    p = SamplingParams()
    assert (p.n, p.temperature, p.top_p, p.top_k, p.min_p, p.max_tokens, p.min_tokens) == (1, 1.0, 1.0, -1, 0.0, 16, 0)
    assert (p.presence_penalty, p.frequency_penalty, p.repetition_penalty) == (0.0, 0.0, 1.0)
    assert p.stop == () and p.stop_token_ids == () and not p.ignore_eos and p.seed is None
    assert SamplingParams(stop="x").stop == ("x",)
    assert SamplingParams(temperature=0.0).is_greedy_pure and not SamplingParams(temperature=0.0, presence_penalty=0.1).is_greedy_pure


@pytest.mark.parametrize(
    "kwargs",
    [
        dict(temperature=-0.1), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=0), dict(top_k=-2), dict(min_p=1.1),
        dict(repetition_penalty=0.0), dict(presence_penalty=2.5), dict(frequency_penalty=-3.0), dict(n=0),
        dict(max_tokens=0), dict(min_tokens=-1), dict(min_tokens=5, max_tokens=4), dict(seed=1 << 65),
        dict(stop_token_ids=[-1]), dict(top_k=1.5),
    ],
)
def test_invalid_params_are_rejected(kwargs):
    with pytest.raises(ValueError):
        SamplingParams(**kwargs)


def test_seeds():
    assert stable_request_seed("abc") == stable_request_seed("abc") != stable_request_seed("abd")
    assert mix_seed(5, 0) == plain_model.mix_seed(5, 0)
    assert len({mix_seed(5, p) for p in range(100)}) == 100
    assert mix_seed(5, 3) != mix_seed(6, 3)


def test_sampler_applies_masks_penalties_and_seeds():
    vocab = 60
    sampler = Sampler(vocab, "cpu")
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(4, vocab, generator=g) * 2
    prompt = [3, 4, 5, 5]
    outputs = [7, 7, 9]
    rows = [
        SamplingRow("a", SamplingParams(temperature=0.0), 0),
        SamplingRow("b", SamplingParams(temperature=0.0, repetition_penalty=1.5, frequency_penalty=0.5, presence_penalty=0.25), 3, prompt, outputs),
        SamplingRow("c", SamplingParams(temperature=0.9, top_p=0.8, top_k=12, min_p=0.02, seed=11), 5),
        SamplingRow("d", SamplingParams(temperature=0.0, min_tokens=4, stop_token_ids=[int(logits[3].argmax())]), 2, eos_token_ids=(1,)),
    ]
    expected_b = plain_model.apply_penalties(logits[1], prompt, outputs, repetition=1.5, frequency=0.5, presence=0.25)
    expected = [
        int(logits[0].argmax()),
        int(expected_b.argmax()),
        plain_model.sample_token(logits[2], temperature=0.9, top_k=12, top_p=0.8, min_p=0.02, base_seed=11, position=5),
        int(logits[3].clone().index_fill_(0, torch.tensor([int(logits[3].argmax()), 1]), float("-inf")).argmax()),
    ]
    working = logits.clone()
    got = sampler.sample(working, rows).tolist()
    assert got == expected
    assert torch.allclose(working[1], expected_b)
    assert torch.equal(working[0], logits[0])
    # min_tokens reached: the stop token is allowed again
    rows[3] = SamplingRow("d", rows[3].params, 4, eos_token_ids=(1,))
    assert sampler.sample(logits.clone(), rows).tolist()[3] == int(logits[3].argmax())


def test_request_without_a_seed_draws_from_its_id():
    sampler = Sampler(40, "cpu")
    logits = torch.zeros(2, 40)
    params = SamplingParams(temperature=1.0)
    a = sampler.sample(logits.clone(), [SamplingRow("x", params, 0), SamplingRow("y", params, 0)]).tolist()
    b = sampler.sample(logits.clone(), [SamplingRow("y", params, 0), SamplingRow("x", params, 0)]).tolist()
    assert a == b[::-1]  # a draw belongs to (request, position), not to the row it sits in
    assert a[0] == plain_model.sample_token(logits[0], temperature=1.0, base_seed=stable_request_seed("x"), position=0)


def _golden_draws():
    from pathlib import Path

    return torch.load(Path(__file__).resolve().parent / "golden" / "sampler.pt")


def test_plain_sampler_draws_what_the_reference_sampler_drew():
    """tests/golden/sampler.pt holds tokens drawn by the reference's own ``Sampler.sample``
    (script beside it): the plain restatement of its filters, noise and penalties gives the same
    token in every case."""
    cases = _golden_draws()
    assert len(cases) >= 50 and sum(1 for case in cases if case["temperature"] > 0) >= 30
    for index, case in enumerate(cases):
        logits = plain_model.apply_penalties(
            case["logits"], case["prompt"], case["outputs"], repetition=case["repetition_penalty"],
            frequency=case["frequency_penalty"], presence=case["presence_penalty"],
        )
        token = plain_model.sample_token(
            logits, temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"], min_p=case["min_p"],
            base_seed=case["seed"], position=case["position"],
        )
        assert token == case["token"], index


def sampler_rows_of(cases):
    """The golden cases as rows of this package's sampler, grouped by vocabulary size."""
    by_vocab = {}
    for index, case in enumerate(cases):
        params = SamplingParams(
            temperature=case["temperature"], top_k=min(case["top_k"], case["logits"].numel()) if case["top_k"] > 0 else -1,
            top_p=case["top_p"], min_p=case["min_p"], seed=case["seed"], repetition_penalty=case["repetition_penalty"],
            frequency_penalty=case["frequency_penalty"], presence_penalty=case["presence_penalty"],
        )
        row = SamplingRow(f"case-{index}", params, case["position"], list(case["prompt"]), list(case["outputs"]))
        by_vocab.setdefault(case["logits"].numel(), []).append((row, case["logits"], case["token"]))
    return by_vocab


def test_the_sampler_pipeline_draws_what_the_reference_sampler_drew():
    """The same cases through ``sampling.Sampler`` (host side: which logits to edit, which seeds),
    with the torch statements of the kernels."""
    for vocab, entries in sampler_rows_of(_golden_draws()).items():
        sampler = Sampler(vocab, "cpu")
        logits = torch.stack([entry[1] for entry in entries])
        got = sampler.sample(logits.clone(), [entry[0] for entry in entries]).tolist()
        assert got == [entry[2] for entry in entries], vocab
