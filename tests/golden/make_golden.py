"""Writes ``tests/golden/<name>.pt``: logits of the reference's own model code
(``kairyu.models.llama.DenseDecoder`` on the CPU, fp32) for the tiny random
models of ``tests/tiny_configs.py``.

Run from the repository root with the reference importable:

    PYTHONPATH=<path to ytworks/kairyu> python tests/golden/make_golden.py

The weights come from ``kairyu_b200.weights.random_tensors`` (seeded), are
loaded into the reference model by tensor name, and a whole prompt is run the
way the reference's own parity test does (tests/unit/test_model_parity.py:58-75).
``tests/test_plain_model.py`` regenerates the same weights and checks the plain
implementation against these files.
"""

from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from kairyu.engine.core.kv_pool import PagedKVPool  # noqa: E402  (the reference)
from kairyu.models.config import parse_model_config  # noqa: E402
from kairyu.models.llama import DenseDecoder  # noqa: E402

from golden_inputs import golden_prompt, golden_weights  # noqa: E402
from tiny_configs import TINY  # noqa: E402


def main() -> None:
    for name, (config, seed, page_size) in TINY.items():
        weights = golden_weights(config, seed)
        parsed = parse_model_config(config)
        model = DenseDecoder(parsed).eval()
        missing, unexpected = model.load_state_dict(weights, strict=False)
        assert not unexpected, unexpected
        assert all("rotary" in key or "lm_head" in key for key in missing), missing
        prompt = golden_prompt(config, seed)
        pool = PagedKVPool(
            num_layers=parsed.num_hidden_layers,
            num_pages=64,
            page_size=page_size,
            num_kv_heads=parsed.num_key_value_heads,
            head_dim=parsed.head_dim,
        )
        length = len(prompt)
        with torch.no_grad():
            hidden = model.forward_tokens(
                torch.tensor(prompt), torch.arange(length), pool, list(range(-(-length // page_size))), seq_len=length
            )
            logits = model.logits(hidden)
        out = Path(__file__).resolve().parent / f"{name}.pt"
        torch.save({"prompt": prompt, "logits": logits.to(torch.float32).contiguous()}, out)
        print(f"{name}: {tuple(logits.shape)} -> {out.name}")


if __name__ == "__main__":
    main()
