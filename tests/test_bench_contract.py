"""bench.py's decisions that need no GPU: the refusal of more than one GPU, and how many layers of a
shape it runs when the shape does not fit the device beside its cache."""

import importlib
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_more_than_one_gpu_is_refused_with_one_line():
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert done.returncode == 2
    assert len(done.stdout.strip().splitlines()) == 1


@pytest.fixture
def bench(monkeypatch):
    monkeypatch.syspath_prepend(str(ROOT))
    module = importlib.import_module("bench")
    yield module


@pytest.mark.parametrize("free_gib,shape,expected", [(178, None, (32, 32)), (178, "llama31-70b", (38, 46)), (178, "qwen3-32b", (64, 64)), (8, None, (0, 3))])
def test_layers_that_fit(bench, monkeypatch, free_gib, shape, expected):
    """All layers where they fit; fewer (both numbers go into the line's config) where the weights, held
    twice while they are drawn and packed, and the cache of 64 requests do not."""
    if shape is not None:
        chosen = bench.SHAPES[shape]
        monkeypatch.setattr(bench, "MODEL", chosen["model"])
        monkeypatch.setattr(bench, "PROMPT_LEN", chosen["prompt_len"])
        monkeypatch.setattr(bench, "GEN_LEN", chosen["gen_len"])
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda: (free_gib << 30, 180 << 30))
    layers = bench.MODEL["num_hidden_layers"]
    fitting = bench.layers_that_fit(layers, 64)
    assert expected[0] <= fitting <= expected[1]
    assert fitting <= layers
