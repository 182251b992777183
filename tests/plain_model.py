"""A plain, slow implementation of the Llama 3 / Qwen3 dense decoder: whole
sequences, no cache, one function per part, plain torch ops in the dtype of its
inputs.  It shares no code with ``kairyu_b200`` and is written from the
reference's formulas; each function cites the file and lines it restates.

It takes a config.json dict and a ``{tensor name: tensor}`` dict with the HF
tensor names.  ``tests/golden/`` holds logits of the reference's own model code
on two tiny random models, which this file is compared with once.
"""

from __future__ import annotations

import math
from typing import Mapping, Optional

import torch


# --------------------------------------------------------------------------- config


def plain_config(config: Mapping) -> dict:
    """The keys the model reads, with the reference's defaults
    (kairyu/models/config.py:508-565, 276-317)."""
    heads = config["num_attention_heads"]
    rope = config.get("rope_parameters") or config.get("rope_scaling") or {}
    return {
        "architecture": config["architectures"][0],
        "hidden": config["hidden_size"],
        "layers": config["num_hidden_layers"],
        "heads": heads,
        "kv_heads": config.get("num_key_value_heads", heads),
        "head_dim": config.get("head_dim") or config["hidden_size"] // heads,
        "intermediate": config["intermediate_size"],
        "vocab": config["vocab_size"],
        "eps": config.get("rms_norm_eps", 1e-6),
        "theta": float(config.get("rope_theta", rope.get("rope_theta", 10000.0))),
        "rope_kind": rope.get("rope_type", rope.get("type")),
        "rope": {"original_max_position_embeddings": config.get("max_position_embeddings", 4096), **rope},
        "max_positions": config.get("max_position_embeddings", 4096),
        "tie": config.get("tie_word_embeddings", False),
        "bias": bool(config.get("attention_bias")),
        # kairyu/models/config.py:190-200: per-head q/k norm goes by architecture name
        "qk_norm": config["architectures"][0] == "Qwen3ForCausalLM",
    }


# --------------------------------------------------------------------------- parts


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """kairyu/models/layers.py:42-46: fp32 statistics, cast back, then the weight."""
    dtype = x.dtype
    xf = x.to(torch.float32)
    variance = xf.pow(2).mean(-1, keepdim=True)
    xf = xf * torch.rsqrt(variance + eps)
    return (weight * xf.to(dtype)).to(dtype)


def llama3_inv_freq(inv_freq: torch.Tensor, rope: Mapping) -> torch.Tensor:
    """kairyu/models/layers.py:93-104."""
    original = rope["original_max_position_embeddings"]
    factor, low, high = rope["factor"], rope["low_freq_factor"], rope["high_freq_factor"]
    low_freq_wavelen = original / low
    high_freq_wavelen = original / high
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_freq_wavelen, inv_freq / factor, inv_freq)
    smooth = (original / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    is_medium = (wavelen >= high_freq_wavelen) & (wavelen <= low_freq_wavelen)
    return torch.where(is_medium, smoothed, scaled)


def rope_cos_sin(cfg: Mapping, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """kairyu/models/layers.py:113-152: fp32 table rows, [T, head_dim] (both halves)."""
    dim = cfg["head_dim"]
    inv_freq = 1.0 / (cfg["theta"] ** (torch.arange(0, dim, 2, dtype=torch.int64).to(torch.float32) / dim))
    amplitude = 1.0
    if cfg["rope_kind"] == "llama3":
        inv_freq = llama3_inv_freq(inv_freq, cfg["rope"])
    elif cfg["rope_kind"] == "yarn":
        inv_freq, amplitude = yarn_inv_freq(dim, cfg["theta"], cfg["rope"])
    elif cfg["rope_kind"] not in (None, "default"):
        raise ValueError(f"plain model: rope type {cfg['rope_kind']!r} is not restated here")
    freqs = positions.cpu().to(torch.float32)[:, None] * inv_freq[None, :]  # the table is made on the CPU, wherever the model runs
    emb = torch.cat((freqs, freqs), dim=-1)
    return (emb.cos() * amplitude).to(positions.device), (emb.sin() * amplitude).to(positions.device)  # kairyu/models/layers.py:143-146


def yarn_inv_freq(dim: int, theta: float, rope: Mapping) -> tuple[torch.Tensor, float]:
    """kairyu/models/layers.py:48-81 and config.py:300-312 (defaults beta_fast 32, beta_slow 1,
    original context = max_position_embeddings), pair by pair in a loop: pair i keeps
    theta^(-2i/dim) up to index ``low``, is divided by ``factor`` from index ``high`` on, and
    blends linearly in i between; cos and sin carry 0.1 ln(factor) + 1."""
    factor = float(rope["factor"])
    context = rope["original_max_position_embeddings"]  # plain_config fills the default in

    def correction(rotations: float) -> float:
        return dim * math.log(context / (rotations * 2 * math.pi)) / (2 * math.log(theta))

    low = max(math.floor(correction(float(rope.get("beta_fast", 32.0)))), 0)
    high = min(math.ceil(correction(float(rope.get("beta_slow", 1.0)))), dim - 1)
    if low == high:
        high = high + 0.001
    out = torch.empty(dim // 2, dtype=torch.float32)
    pos_freqs = theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim)
    for i in range(dim // 2):
        ramp = (torch.tensor(float(i) - low, dtype=torch.float32) / (high - low)).clamp(0, 1)
        out[i] = (1.0 / (factor * pos_freqs[i])) * ramp + (1.0 / pos_freqs[i]) * (1.0 - ramp)

    def mscale(scale: float, m: float = 1.0) -> float:
        return 1.0 if scale <= 1.0 else 0.1 * m * math.log(scale) + 1.0

    if rope.get("mscale") is not None and rope.get("mscale_all_dim") is not None:
        amplitude = mscale(factor, rope["mscale"]) / mscale(factor, rope["mscale_all_dim"])
    else:
        amplitude = mscale(factor)
    return out, amplitude


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """kairyu/models/layers.py:165-167."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """kairyu/models/layers.py:188-190: q,k [T, heads, D]; cos,sin [T, D] cast to q's dtype."""
    cos = cos[:, None, :].to(q.dtype)
    sin = sin[:, None, :].to(q.dtype)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def causal_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, window: Optional[int] = None, scale: Optional[float] = None
) -> torch.Tensor:
    """kairyu/engine/core/attention/torch_backend.py:57-71 for a whole sequence:
    q [T, Hq, D], k, v [T, Hkv, D]; query i sees keys j <= i; query head h uses
    KV head h // (Hq // Hkv); scores / sqrt(D); softmax in fp32; returns [T, Hq*D].
    ``window`` (not in the reference's dense path) keeps keys j > i - window."""
    T, heads, dim = q.shape
    group = heads // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scale = 1.0 / math.sqrt(dim) if scale is None else scale
    scores = torch.einsum("qhd,khd->hqk", q.float(), k.float()) * scale
    i = torch.arange(T, device=q.device)[:, None]
    j = torch.arange(T, device=q.device)[None, :]
    mask = j <= i
    if window is not None:
        mask = mask & (j > i - window)
    scores = scores.masked_fill(~mask[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hqk,khd->qhd", probs, v.float())
    return out.reshape(T, heads * dim).to(q.dtype)


def attention_block(cfg: Mapping, w: Mapping[str, torch.Tensor], prefix: str, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """kairyu/models/attention.py:216-271: q/k/v projections, per-head q/k norm
    (Qwen3), RoPE, attention, o projection."""
    T = x.shape[0]
    heads, kv_heads, dim = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    lin = torch.nn.functional.linear
    q = lin(x, w[f"{prefix}.q_proj.weight"], w.get(f"{prefix}.q_proj.bias")).view(T, heads, dim)
    k = lin(x, w[f"{prefix}.k_proj.weight"], w.get(f"{prefix}.k_proj.bias")).view(T, kv_heads, dim)
    v = lin(x, w[f"{prefix}.v_proj.weight"], w.get(f"{prefix}.v_proj.bias")).view(T, kv_heads, dim)
    if cfg["qk_norm"]:
        q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["eps"])
        k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["eps"])
    cos, sin = rope_cos_sin(cfg, positions)
    q, k = apply_rope(q, k, cos, sin)
    mixed = causal_attention(q, k, v)
    return lin(mixed, w[f"{prefix}.o_proj.weight"], w.get(f"{prefix}.o_proj.bias"))


def swiglu_mlp(w: Mapping[str, torch.Tensor], prefix: str, x: torch.Tensor) -> torch.Tensor:
    """kairyu/models/layers.py:243-244."""
    lin = torch.nn.functional.linear
    gate = lin(x, w[f"{prefix}.gate_proj.weight"])
    up = lin(x, w[f"{prefix}.up_proj.weight"])
    return lin(torch.nn.functional.silu(gate) * up, w[f"{prefix}.down_proj.weight"])


def decoder_layer(cfg: Mapping, w: Mapping[str, torch.Tensor], index: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """kairyu/models/llama.py:88-101: pre-norm residual around attention, then around the MLP."""
    p = f"model.layers.{index}"
    x = x + attention_block(cfg, w, f"{p}.self_attn", rms_norm(x, w[f"{p}.input_layernorm.weight"], cfg["eps"]), positions)
    return x + swiglu_mlp(w, f"{p}.mlp", rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["eps"]))


def forward_logits(config: Mapping, weights: Mapping[str, torch.Tensor], token_ids) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence
    (kairyu/models/llama.py:309-329 and 612-614)."""
    cfg = plain_config(config)
    device = weights["model.embed_tokens.weight"].device  # the CPU in most tests; a GPU for the shapes too large for it
    tokens = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    positions = torch.arange(tokens.numel(), device=device)
    x = weights["model.embed_tokens.weight"][tokens]
    for index in range(cfg["layers"]):
        x = decoder_layer(cfg, weights, index, x, positions)
    x = rms_norm(x, weights["model.norm.weight"], cfg["eps"])
    head = weights["model.embed_tokens.weight"] if cfg["tie"] else weights["lm_head.weight"]
    return torch.nn.functional.linear(x, head)


def greedy_generate(config: Mapping, weights: Mapping[str, torch.Tensor], prompt, steps: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(steps):
        tokens.append(int(forward_logits(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


# --------------------------------------------------------------------------- sampling


_MASK64 = (1 << 64) - 1


def mix_seed(base: int, position: int) -> int:
    """kairyu/engine/core/sampling_types.py:21-31."""
    x = (base ^ ((position + 1) * 0x9E3779B97F4A7C15)) & _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return (x ^ (x >> 31)) & _MASK64


def gumbel_noise(vocab: int, seed: int) -> torch.Tensor:
    """kairyu/kernels/sampling_gpu.py:44-65, 113-127, in Python integers."""
    noise = []
    for i in range(vocab):
        z = (((i + 1) * 0x9E3779B97F4A7C15) & _MASK64) ^ (seed & _MASK64)
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        z = z ^ (z >> 31)
        u = ((z & ((1 << 52) - 1)) + 0.5) / float(1 << 52)
        noise.append(-math.log(-math.log1p(-u)))
    return torch.tensor(noise, dtype=torch.float64)


def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float) -> torch.Tensor:
    """kairyu/engine/core/sampler.py:1237-1378 for one row: softmax(logits/T),
    min-p, top-k (ties kept), top-p on the descending order, renormalise."""
    probs = torch.softmax(logits.float() / temperature, dim=-1)
    if min_p > 0.0:
        probs = torch.where(probs >= min_p * probs.max(), probs, torch.zeros_like(probs))
    vocab = probs.numel()
    if 0 < top_k < vocab:
        threshold = torch.topk(probs, top_k).values[-1]
        probs = torch.where(probs < threshold, torch.zeros_like(probs), probs)
    if top_p < 1.0:
        values, indices = torch.sort(probs, descending=True)
        cumulative = torch.cumsum(values, dim=-1)
        cut = cumulative - values >= top_p * cumulative[-1].clamp(min=1e-12)
        values = values.masked_fill(cut, 0.0)
        probs = torch.zeros_like(probs).scatter(0, indices, values)
    return probs / probs.sum().clamp(min=1e-12)


def sample_token(logits: torch.Tensor, *, temperature: float, top_k: int = -1, top_p: float = 1.0, min_p: float = 0.0, base_seed: int, position: int) -> int:
    """kairyu/engine/core/sampler.py:1379-1389: argmax(log p + Gumbel noise)."""
    if temperature == 0.0:
        return int(logits.argmax())
    probs = filtered_probs(logits, temperature, top_k, top_p, min_p)
    noise = gumbel_noise(probs.numel(), mix_seed(base_seed, position))
    return int(torch.argmax(torch.log(probs).to(torch.float64) + noise))


def apply_penalties(logits: torch.Tensor, prompt, outputs, *, repetition: float, frequency: float, presence: float) -> torch.Tensor:
    """kairyu/engine/core/sampler.py:466-502: repetition over prompt + outputs,
    frequency and presence over outputs."""
    logits = logits.clone().float()
    if repetition != 1.0:
        seen = sorted(set(prompt) | set(outputs))
        values = logits[seen]
        logits[seen] = torch.where(values > 0, values / repetition, values * repetition)
    counts: dict[int, int] = {}
    for token in outputs:
        counts[token] = counts.get(token, 0) + 1
    for token, count in counts.items():
        logits[token] -= frequency * count + presence
    return logits


def logprob_entry(raw_logits: torch.Tensor, token: int, k: int) -> tuple[dict[int, float], float]:
    """kairyu/engine/core/sampler.py:1423-1437 and kairyu/engine/engine_loop.py:219-234: the
    log-softmax of the raw logits; the chosen token's value first, then the k largest that are
    not it already.  Returns the per-token dict and the chosen token's log-probability."""
    logp = torch.log_softmax(raw_logits.to(torch.float32), dim=-1)
    entry = {int(token): float(logp[token])}
    if k > 0:
        values, indices = torch.topk(logp, min(k, logp.numel()))
        for value, index in zip(values.tolist(), indices.tolist()):
            entry.setdefault(int(index), float(value))
    return entry, float(logp[token])
