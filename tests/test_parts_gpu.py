"""Each part alone on the GPU (norm, position encoding, attention mixer,
feed-forward, block, embedding, head) against the plain implementation's
function for that part, in 32-bit and in bfloat16, at the odd sizes."""

import math

import pytest
import torch

import plain_model
from golden_inputs import as_held_in_bf16, golden_weights
from tiny_configs import TINY

from kairyu_b200.engine.workspace import Workspace
from kairyu_b200.models.llama import dense_decoder_spec
from kairyu_b200.config import parse_dense_config
from kairyu_b200.parts import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, CacheView, PartSpec, StepContext
from kairyu_b200.parts.rope import rotary_tables

pytestmark = pytest.mark.gpu
DEV = "cuda"
T = 45
PAGE = 8


def setup(name, dtype):
    config, seed, _ = TINY[name]
    parsed = parse_dense_config(config, config["architectures"][0])
    spec = dense_decoder_spec(parsed, qk_norm=config["architectures"][0] == "Qwen3ForCausalLM")
    weights = golden_weights(config, seed)
    plain_weights = weights if dtype == torch.float32 else as_held_in_bf16(weights)
    cfg = plain_model.plain_config(config)
    return config, parsed, spec, weights, plain_weights, cfg


def load(part, weights, dtype):
    tensors = {}
    for s in part.tensor_specs():
        source = weights[s.name if s.name in weights else s.alias_of]
        keep = s.role == "vector"
        tensors[s.name] = source.to(DEV, torch.float32 if keep else dtype)
    part.load(tensors)
    return part


def context(dtype, tokens, kv_heads, head_dim):
    pages = -(-T // PAGE)
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
    table = ints(list(range(1, pages + 1))).view(1, pages)
    ctx = StepContext(
        num_tokens=T, num_rows=1, dtype=dtype, token_ids=ints(tokens), positions=ints(list(range(T))), row_ids=ints([0] * T),
        qo_indptr=ints([0, T]), seq_lens=ints([T]), write_from=ints([0]), state_slots=ints([0]), block_tables={0: table},
        host_qo_indptr=(0, T), host_seq_lens=(T,), tiles={64: (1, ints([0]), ints([0])), 128: (1, ints([0]), ints([0]))},
        num_decode_rows=0, decode_rows=ints([]), decode_tokens=ints([]), max_seq_len=T, workspace=Workspace(DEV),
        error_flag=torch.zeros(1, dtype=torch.int32, device=DEV),
    )
    cache = CacheView(
        k=torch.zeros(pages + 1, PAGE, kv_heads, head_dim, dtype=dtype, device=DEV),
        v=torch.zeros(pages + 1, PAGE, kv_heads, head_dim, dtype=dtype, device=DEV), page_size=PAGE, group=0, writes=True,
    )
    return ctx, cache


def bound(dtype):
    return dict(atol=3e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def close(got, expected, atol, rtol):
    got, expected = got.float().cpu(), expected.float().cpu()
    diff = (got - expected).abs()
    assert bool((diff <= atol + rtol * expected.abs()).all()), f"max abs diff {diff.max().item():.3e}"


CASES = [(n, d) for n in ("llama", "qwen3", "odd", "wide", "yarn") for d in (torch.float32, torch.bfloat16)]


@pytest.mark.parametrize("name,dtype", CASES)
def test_parts_alone(name, dtype):
    config, parsed, spec, weights, plain_weights, cfg = setup(name, dtype)
    build = dict(dtype=dtype, device=DEV, shared={})
    g = torch.Generator().manual_seed(12)
    tokens = torch.randint(0, parsed.vocab_size, (T,), generator=g).tolist()
    ctx, cache = context(dtype, tokens, parsed.num_key_value_heads, parsed.head_dim)
    x = torch.randn(T, parsed.hidden_size, generator=g)
    x_act = x.to(dtype)
    x_plain = x_act.float()
    layer = spec.layers[1]
    prefix = layer.prefix

    # embedding: rows of the table, as fp32
    embedding = load(EMBEDDINGS.build(spec.embedding, **build), weights, dtype)
    close(embedding.forward(ctx), plain_weights["model.embed_tokens.weight"][torch.tensor(tokens)], 0.0, 0.0)

    # norm, with and without the residual sum
    norm = load(NORMS.build(layer.mixer_norm, **build), weights, dtype)
    residual = x.to(DEV).clone()
    delta = torch.randn(T, parsed.hidden_size, generator=g).to(dtype)
    expected = plain_model.rms_norm(x + delta.float(), plain_weights[f"{prefix}.input_layernorm.weight"], cfg["eps"])
    close(norm.apply(residual, delta.to(DEV), ctx), expected, **bound(dtype))
    close(residual, x + delta.float(), 1e-6, 0.0)

    # position encoding: the table is the plain cos/sin (first half)
    rope = POSITION_ENCODINGS.build(layer.mixer.params["position"], **build)
    cos, sin = rope.rotary_tables()
    plain_cos, plain_sin = plain_model.rope_cos_sin(cfg, torch.arange(parsed.max_position_embeddings))
    half = parsed.head_dim // 2
    assert torch.equal(cos.cpu(), plain_cos[:, :half]) and torch.equal(sin.cpu(), plain_sin[:, :half])

    # attention mixer over a whole sequence
    mixer = load(MIXERS.build(layer.mixer, **build), weights, dtype)
    expected = plain_model.attention_block(cfg, plain_weights, f"{prefix}.self_attn", x_plain, torch.arange(T))
    close(mixer.forward(x_act.to(DEV), ctx, cache), expected, **bound(dtype))
    assert int(ctx.error_flag.item()) == 0
    assert float(cache.k[1 : -(-T // PAGE) + 1].float().abs().sum()) > 0 and float(cache.k[0].float().abs().sum()) == 0

    # feed-forward
    ffn = load(FEED_FORWARDS.build(layer.ffn, **build), weights, dtype)
    close(ffn.forward(x_act.to(DEV), ctx), plain_model.swiglu_mlp(plain_weights, f"{prefix}.mlp", x_plain), **bound(dtype))

    # the block arrangement: residual, pending delta, both sub-layers
    block = load(BLOCKS.build(PartSpec(layer.block), layer=layer, **build), weights, dtype)
    ctx2, cache2 = context(dtype, tokens, parsed.num_key_value_heads, parsed.head_dim)
    residual = x.to(DEV).clone()
    residual_out, pending = block.forward(residual, None, ctx2, cache2)
    expected = plain_model.decoder_layer(cfg, plain_weights, 1, x, torch.arange(T))
    close(residual_out + pending.float(), expected, **(bound(dtype) if dtype == torch.float32 else dict(atol=4e-2, rtol=2e-2)))

    # head: fp32 logits
    head = load(HEADS.build(spec.head, **build), weights, dtype)
    head_weight = plain_weights["model.embed_tokens.weight"] if parsed.tie_word_embeddings else plain_weights["lm_head.weight"]
    close(head.forward(x_act.to(DEV), ctx), x_plain @ head_weight.t(), **bound(dtype))
