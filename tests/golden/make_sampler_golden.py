"""Writes ``tests/golden/sampler.pt``: tokens drawn by the reference's own sampler
(``kairyu.engine.core.sampler.Sampler.sample`` on the CPU) for a list of cases that
cross temperature, top-k, top-p, min-p, seeds, positions and the three penalties.

Run from the repository root with the reference importable:

    PYTHONPATH=<path to ytworks/kairyu> python tests/golden/make_sampler_golden.py

Each case keeps its logits row, its parameters and the token the reference drew.
``tests/test_sampling_cpu.py`` checks the plain sampler against the file, and
``tests/test_kernels_gpu.py`` the sampling kernels.
"""

from __future__ import annotations

import random
from pathlib import Path

import torch

from kairyu.engine.core.sampler import Sampler  # the reference
from kairyu.engine.core.sampling_types import EngineSampling


def cases() -> list[dict]:
    rng = random.Random(20)
    out = []
    for index in range(56):
        vocab = rng.choice([97, 203, 256, 331, 500])
        generator = torch.Generator().manual_seed(1000 + index)
        logits = torch.randn(vocab, generator=generator) * rng.choice([0.7, 1.5, 3.0])
        case = dict(
            logits=logits,
            temperature=rng.choice([0.0, 0.3, 0.8, 1.0, 1.7]),
            top_k=rng.choice([-1, -1, 1, 5, 40, vocab + 3]),
            top_p=rng.choice([1.0, 1.0, 0.95, 0.8, 0.3]),
            min_p=rng.choice([0.0, 0.0, 0.02, 0.2]),
            seed=rng.choice([0, 7, 2**40 + 3, 2**63 - 1]),
            position=rng.choice([0, 1, 5, 300]),
            repetition_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0, prompt=(), outputs=(),
        )
        if index % 4 == 3:  # penalties over a prompt and outputs with repeats
            case.update(
                repetition_penalty=rng.choice([1.0, 1.3, 0.8]), frequency_penalty=rng.choice([0.0, 0.5, -0.4]),
                presence_penalty=rng.choice([0.0, 0.7]), prompt=tuple(rng.randrange(vocab) for _ in range(9)),
                outputs=tuple(rng.choice(range(0, vocab, 7)) for _ in range(12)),
            )
        out.append(case)
    return out


def main() -> None:
    drawn = []
    for index, case in enumerate(cases()):
        sampler = Sampler()
        sampling = EngineSampling(
            temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"], min_p=case["min_p"],
            presence_penalty=case["presence_penalty"], frequency_penalty=case["frequency_penalty"],
            repetition_penalty=case["repetition_penalty"], seed=case["seed"],
        )
        token = sampler.sample(
            f"case-{index}", sampling, case["position"], case["logits"].clone(), prompt=case["prompt"], outputs=case["outputs"],
        )
        drawn.append(dict(case, token=int(token.token_id)))
    out = Path(__file__).resolve().parent / "sampler.pt"
    torch.save(drawn, out)
    sampled = sum(1 for case in drawn if case["temperature"] > 0)
    print(f"{len(drawn)} cases ({sampled} with temperature > 0) -> {out.name}")


if __name__ == "__main__":
    main()
