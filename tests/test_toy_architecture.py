"""A toy architecture defined here, outside the package: a mixer with per-request
state of its own, registered, built and stepped without a change to the
framework's files.  Its layers differ (attention, the toy mixer, an attention
that reads another layer's keys and values) and its run order names one layer
twice.  The result is compared with a plain whole-sequence computation under
different cuts.  Runs on the CPU with the torch statements of the kernels and
on the GPU with the kernels."""

from typing import Mapping

import numpy as np
import pytest
import torch

import plain_model
import torch_kernels
import traces

from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
from kairyu_b200.engine.engine import build_model
from kairyu_b200.engine.runner import ModelRunner
from kairyu_b200.parts import MIXERS, LayerCall, LayerSpec, Mixer, ModelSpec, PartSpec, StateSpec, TensorSpec
from kairyu_b200.registry import register_architecture, unregister_architecture
from kairyu_b200.weights.random_init import random_tensors

HIDDEN, STATE, VOCAB, HEADS, KV_HEADS, HEAD_DIM, INTER, EPS = 48, 20, 97, 3, 1, 16, 72, 1e-5
DECAY = 0.8


class DecayMixer(Mixer):
    """state <- DECAY * state + (1 - DECAY) * (x W_in^T), y = state W_out^T, token by token.
    The state lives in the request's slot between steps."""

    def __init__(self, *, prefix, hidden_size, state_size, dtype, device, **_):
        self.prefix, self.hidden_size, self.state_size, self.dtype = prefix, hidden_size, state_size, dtype
        self.w_in = self.w_out = None

    def tensor_specs(self):
        return [
            TensorSpec(f"{self.prefix}.in_proj.weight", (self.state_size, self.hidden_size)),
            TensorSpec(f"{self.prefix}.out_proj.weight", (self.hidden_size, self.state_size)),
        ]

    def load(self, tensors):
        self.w_in = tensors[f"{self.prefix}.in_proj.weight"]
        self.w_out = tensors[f"{self.prefix}.out_proj.weight"]

    def cache_specs(self):
        return (StateSpec((self.state_size,), "float32"),)

    def forward(self, x, ctx, cache):
        assert cache.state is not None and cache.k is None
        out = torch.empty(x.shape[0], self.hidden_size, dtype=x.dtype, device=x.device)
        drive = x.float() @ self.w_in.float().t()
        if ctx.num_tokens == ctx.num_rows:
            # One token a row: everything on the device, so that a decode graph can replay it.
            # Padding rows of a graph all name the scratch slot; what lands there is read by nobody.
            slots = ctx.state_slots.long()
            state = cache.state.index_select(0, slots) * DECAY + drive * (1 - DECAY)
            cache.state.index_copy_(0, slots, state)
            return (state @ self.w_out.float().t()).to(x.dtype)
        slots = ctx.state_slots.tolist()
        for row in range(len(ctx.host_qo_indptr) - 1):
            state = cache.state[slots[row]]
            for t in range(ctx.host_qo_indptr[row], ctx.host_qo_indptr[row + 1]):
                state.mul_(DECAY).add_(drive[t], alpha=1 - DECAY)
                out[t] = (state @ self.w_out.float().t()).to(x.dtype)
        return out


def toy_spec(config) -> ModelSpec:
    def norm(name):
        return PartSpec("rmsnorm", name=name, size=HIDDEN, eps=EPS)

    position = PartSpec("rope", rotary_dim=HEAD_DIM, theta=10000.0, scaling=None, max_positions=256)

    def attention(prefix):
        return PartSpec(
            "gqa_attention", prefix=prefix, hidden_size=HIDDEN, num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM,
            qk_norm=False, norm_eps=EPS, qkv_bias=False, o_bias=False, position=position,
        )

    def ffn(prefix):
        return PartSpec("swiglu", prefix=prefix, hidden_size=HIDDEN, intermediate_size=INTER, activation="silu")

    mixers = [attention("layers.0.attn"), PartSpec("toy_decay", prefix="layers.1.decay", hidden_size=HIDDEN, state_size=STATE), attention("layers.2.attn")]
    layers = tuple(
        LayerSpec(f"layers.{i}", "pre_norm", mixers[i], ffn(f"layers.{i}.mlp"), norm(f"layers.{i}.norm1.weight"), norm(f"layers.{i}.norm2.weight"))
        for i in range(3)
    )
    schedule = (
        LayerCall(0, cache_slot=0),
        LayerCall(1, cache_slot=1),
        LayerCall(2, cache_slot=0, writes_cache=False),  # reads layer 0's keys and values
        LayerCall(1, cache_slot=2),  # the stateful layer again, with a second state of its own
    )
    return ModelSpec(
        embedding=PartSpec("token_embedding", name="embed.weight", vocab_size=VOCAB, hidden_size=HIDDEN),
        layers=layers, schedule=schedule, final_norm=norm("final_norm.weight"),
        head=PartSpec("linear_head", name="head.weight", vocab_size=VOCAB, hidden_size=HIDDEN, tied_to=None),
        vocab_size=VOCAB, hidden_size=HIDDEN, max_position_embeddings=256,
    )


@pytest.fixture
def toy():
    MIXERS.register("toy_decay")(DecayMixer)
    register_architecture("ToyDecayForCausalLM", lambda config: dict(config), toy_spec)
    yield {"architectures": ["ToyDecayForCausalLM"]}
    unregister_architecture("ToyDecayForCausalLM")
    MIXERS.unregister("toy_decay")


def plain_toy_logits(w: Mapping[str, torch.Tensor], tokens) -> torch.Tensor:
    """Whole sequence, no cache."""
    cfg = {"head_dim": HEAD_DIM, "theta": 10000.0, "rope_kind": None, "rope": {}}
    lin = torch.nn.functional.linear
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed.weight"][torch.tensor(tokens)]

    def qkv(prefix, h):
        q = lin(h, w[f"{prefix}.q_proj.weight"]).view(T, HEADS, HEAD_DIM)
        k = lin(h, w[f"{prefix}.k_proj.weight"]).view(T, KV_HEADS, HEAD_DIM)
        v = lin(h, w[f"{prefix}.v_proj.weight"]).view(T, KV_HEADS, HEAD_DIM)
        cos, sin = plain_model.rope_cos_sin(cfg, positions)
        q, k = plain_model.apply_rope(q, k, cos, sin)
        return q, k, v

    def decay(prefix, h):
        drive = lin(h, w[f"{prefix}.in_proj.weight"])
        state = torch.zeros(STATE)
        rows = []
        for t in range(T):
            state = DECAY * state + (1 - DECAY) * drive[t]
            rows.append(lin(state, w[f"{prefix}.out_proj.weight"]))
        return torch.stack(rows)

    def ffn(i, x):
        return x + plain_model.swiglu_mlp(w, f"layers.{i}.mlp", plain_model.rms_norm(x, w[f"layers.{i}.norm2.weight"], EPS))

    # call 1: layer 0, attention that writes slot 0
    h = plain_model.rms_norm(x, w["layers.0.norm1.weight"], EPS)
    q0, k0, v0 = qkv("layers.0.attn", h)
    x = ffn(0, x + lin(plain_model.causal_attention(q0, k0, v0), w["layers.0.attn.o_proj.weight"]))
    # call 2: layer 1, decay mixer
    x = ffn(1, x + decay("layers.1.decay", plain_model.rms_norm(x, w["layers.1.norm1.weight"], EPS)))
    # call 3: layer 2, its own queries over layer 0's keys and values
    h = plain_model.rms_norm(x, w["layers.2.norm1.weight"], EPS)
    q2, _, _ = qkv("layers.2.attn", h)
    x = ffn(2, x + lin(plain_model.causal_attention(q2, k0, v0), w["layers.2.attn.o_proj.weight"]))
    # call 4: layer 1 again (same weights, fresh state)
    x = ffn(1, x + decay("layers.1.decay", plain_model.rms_norm(x, w["layers.1.norm1.weight"], EPS)))
    return lin(plain_model.rms_norm(x, w["final_norm.weight"], EPS), w["head.weight"])


def build(toy, device, decode_mode="eager"):
    model, _ = build_model(toy, dtype="float32", device=device)
    weights = random_tensors(model.tensor_specs(), seed=9, device="cpu")
    model.load({name: tensor.to(device) for name, tensor in weights.items()})
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    assert [g.slots for g in layout.groups] == [(0,)] and [b.slot for b in layout.states] == [1, 2]
    cache = CacheManager(layout, num_pages=24, page_size=8, max_requests=4)
    storage = CacheStorage(layout, num_pages=24, page_size=8, max_requests=4, dtype=model.dtype, device=device)
    runner = ModelRunner(model, cache, storage, max_model_len=256, decode_mode=decode_mode, max_graph_batch=4)
    assert not runner.portion_graphs  # the toy mixer loops over rows on the host: its portions are launched one by one
    return runner, weights


def check(toy, device, decode_mode="eager"):
    runner, weights = build(toy, device, decode_mode)
    requests = traces.make_requests(VOCAB, [37, 20, 51, 9, 44, 30], seed=6)
    expected = {name: plain_toy_logits(weights, tokens).numpy() for name, tokens in requests.items()}
    for steps in (traces.trace_whole(requests), traces.trace_chunks(requests), traces.trace_mixed(requests, seed=2)):
        result = traces.run_in_process(runner, steps)  # slots change hands: a stale state would show
        worst = max(float(np.abs(row - expected[n][p]).max()) for (n, p), row in result.items())
        assert worst < 3e-5, worst


def test_toy_architecture_on_cpu(toy, monkeypatch):
    torch_kernels.install(monkeypatch)
    check(toy, "cpu")


@pytest.mark.gpu
def test_toy_architecture_on_gpu(toy):
    check(toy, "cuda")


@pytest.mark.gpu
def test_toy_architecture_in_decode_graphs(toy):
    """Steps of single tokens replay CUDA graphs.  A mixer with state must see every token of a
    request once: the capture runs on padding rows only (they use a state slot no request
    holds), and padding rows of a replay never touch a live request's state."""
    runner, weights = build(toy, "cuda", "cuda_graph")
    requests = traces.make_requests(VOCAB, [37, 20, 51, 9, 44, 30], seed=6)
    expected = {name: plain_toy_logits(weights, tokens).numpy() for name, tokens in requests.items()}
    # decode tails one request at a time (bucket 1), then three at a time in a bucket of four
    # (one padding row), with requests of different lengths ending at different steps
    steps = traces.trace_decode_tail(requests, 12)
    result = traces.run_in_process(runner, steps)
    worst = max(float(np.abs(row - expected[n][p]).max()) for (n, p), row in result.items())
    assert worst < 3e-5, worst
    names = list(requests)[:3]
    head = 6
    together = [{"step": 0, "entries": [{"id": n, "tokens": requests[n][:head], "want": []} for n in names], "end": []}]
    longest = max(len(requests[n]) for n in names)
    for index in range(head, longest):
        live = [n for n in names if index < len(requests[n])]
        together.append({
            "step": len(together),
            "entries": [{"id": n, "tokens": [requests[n][index]], "want": [0]} for n in live],
            "end": [n for n in live if index == len(requests[n]) - 1],
        })
    result = traces.run_in_process(runner, together)
    worst = max(float(np.abs(row - expected[n][p]).max()) for (n, p), row in result.items())
    assert worst < 3e-5, worst
    assert runner.counters["graph_replays"] > 40 and runner.counters["graph_captures"] >= 3


# ------------------------------------------------------------------ a second toy: routing and another position encoding
# A feed-forward that routes every token to one of three experts, and learned absolute positions
# added to the embedding, both defined here and registered from outside the package; attention
# runs without rotary tables.  Compared with a plain whole-sequence computation under all cuts.

from kairyu_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding  # noqa: E402

EXPERTS = 3
R_HIDDEN, R_INTER, R_VOCAB, R_MAXPOS = 40, 24, 61, 160


class LearnedPositions(PositionEncoding):
    """residual[t] += table[position[t]]."""

    def __init__(self, *, name, max_positions, hidden_size, dtype, device, **_):
        self.name, self.max_positions, self.hidden_size = name, max_positions, hidden_size
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.max_positions, self.hidden_size))]

    def load(self, tensors):
        self.table = tensors[self.name]

    def embed_hook(self, residual, ctx):
        residual.add_(self.table[ctx.positions.long()].float())


class TopOneExperts(FeedForward):
    """Router logits in fp32, the best expert per token, y = W2_e relu(W1_e x) scaled by its softmax weight."""

    def __init__(self, *, prefix, hidden_size, intermediate_size, num_experts, dtype, device, **_):
        self.prefix, self.hidden_size, self.inter, self.num_experts = prefix, hidden_size, intermediate_size, num_experts
        self.router = self.w1 = self.w2 = None

    def tensor_specs(self):
        return [
            TensorSpec(f"{self.prefix}.router.weight", (self.num_experts, self.hidden_size)),
            TensorSpec(f"{self.prefix}.w1", (self.num_experts * self.inter, self.hidden_size)),
            TensorSpec(f"{self.prefix}.w2", (self.num_experts * self.hidden_size, self.inter)),
        ]

    def load(self, tensors):
        self.router = tensors[f"{self.prefix}.router.weight"]
        self.w1 = tensors[f"{self.prefix}.w1"].view(self.num_experts, self.inter, self.hidden_size)
        self.w2 = tensors[f"{self.prefix}.w2"].view(self.num_experts, self.hidden_size, self.inter)

    def forward(self, x, ctx):
        return routed_ffn(x.float(), self.router.float(), self.w1.float(), self.w2.float()).to(x.dtype)


def routed_ffn(x, router, w1, w2):
    probs = torch.softmax(x @ router.t(), dim=-1)
    best = probs.argmax(dim=-1)
    out = torch.zeros(x.shape[0], w2.shape[1], dtype=torch.float32, device=x.device)
    for expert in range(router.shape[0]):
        rows = (best == expert).nonzero().flatten()
        if rows.numel():
            h = torch.relu(x[rows] @ w1[expert].t())
            out[rows] = (h @ w2[expert].t()) * probs[rows, expert : expert + 1]
    return out


def routed_spec(config) -> ModelSpec:
    def norm(name):
        return PartSpec("rmsnorm", name=name, size=R_HIDDEN, eps=EPS)

    def layer(i):
        attention = PartSpec(
            "gqa_attention", prefix=f"layers.{i}.attn", hidden_size=R_HIDDEN, num_heads=2, num_kv_heads=2, head_dim=16,
            qk_norm=False, norm_eps=EPS, qkv_bias=False, o_bias=False, position=None,
        )
        ffn = PartSpec("toy_top_one", prefix=f"layers.{i}.moe", hidden_size=R_HIDDEN, intermediate_size=R_INTER, num_experts=EXPERTS)
        return LayerSpec(f"layers.{i}", "pre_norm", attention, ffn, norm(f"layers.{i}.norm1.weight"), norm(f"layers.{i}.norm2.weight"))

    return ModelSpec(
        embedding=PartSpec("token_embedding", name="embed.weight", vocab_size=R_VOCAB, hidden_size=R_HIDDEN),
        layers=(layer(0), layer(1)), schedule=(LayerCall(0, cache_slot=0), LayerCall(1, cache_slot=1)),
        final_norm=norm("final_norm.weight"),
        head=PartSpec("linear_head", name="head.weight", vocab_size=R_VOCAB, hidden_size=R_HIDDEN, tied_to=None),
        vocab_size=R_VOCAB, hidden_size=R_HIDDEN, max_position_embeddings=R_MAXPOS,
        embedding_position=PartSpec("toy_learned_positions", name="positions.weight", max_positions=R_MAXPOS, hidden_size=R_HIDDEN),
    )


@pytest.fixture
def routed():
    FEED_FORWARDS.register("toy_top_one")(TopOneExperts)
    POSITION_ENCODINGS.register("toy_learned_positions")(LearnedPositions)
    register_architecture("ToyRoutedForCausalLM", lambda config: dict(config), routed_spec)
    yield {"architectures": ["ToyRoutedForCausalLM"]}
    unregister_architecture("ToyRoutedForCausalLM")
    FEED_FORWARDS.unregister("toy_top_one")
    POSITION_ENCODINGS.unregister("toy_learned_positions")


def plain_routed_logits(w, tokens):
    lin = torch.nn.functional.linear
    T = len(tokens)
    x = w["embed.weight"][torch.tensor(tokens)] + w["positions.weight"][:T]
    for i in range(2):
        h = plain_model.rms_norm(x, w[f"layers.{i}.norm1.weight"], EPS)
        q = lin(h, w[f"layers.{i}.attn.q_proj.weight"]).view(T, 2, 16)
        k = lin(h, w[f"layers.{i}.attn.k_proj.weight"]).view(T, 2, 16)
        v = lin(h, w[f"layers.{i}.attn.v_proj.weight"]).view(T, 2, 16)
        x = x + lin(plain_model.causal_attention(q, k, v), w[f"layers.{i}.attn.o_proj.weight"])
        h = plain_model.rms_norm(x, w[f"layers.{i}.norm2.weight"], EPS)
        x = x + routed_ffn(
            h, w[f"layers.{i}.moe.router.weight"], w[f"layers.{i}.moe.w1"].view(EXPERTS, R_INTER, R_HIDDEN),
            w[f"layers.{i}.moe.w2"].view(EXPERTS, R_HIDDEN, R_INTER),
        )
    return lin(plain_model.rms_norm(x, w["final_norm.weight"], EPS), w["head.weight"])


def check_routed(config, device):
    model, _ = build_model(config, dtype="float32", device=device)
    weights = random_tensors(model.tensor_specs(), seed=12, device="cpu")
    # Router rows far apart, so that a rounding difference between the two computations does not flip an expert
    for i in range(2):
        weights[f"layers.{i}.moe.router.weight"] = weights[f"layers.{i}.moe.router.weight"] * 40.0
    model.load({name: tensor.to(device) for name, tensor in weights.items()})
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=24, page_size=8, max_requests=4)
    storage = CacheStorage(layout, num_pages=24, page_size=8, max_requests=4, dtype=model.dtype, device=device)
    runner = ModelRunner(model, cache, storage, max_model_len=R_MAXPOS, decode_mode="eager")
    requests = traces.make_requests(R_VOCAB, [37, 20, 51, 9, 44, 30], seed=8)
    expected = {name: plain_routed_logits(weights, tokens).numpy() for name, tokens in requests.items()}
    experts_used = set()
    for tokens in requests.values():
        h = plain_model.rms_norm(weights["embed.weight"][torch.tensor(tokens)] + weights["positions.weight"][: len(tokens)], weights["layers.0.norm1.weight"], EPS)
        experts_used |= set((h @ weights["layers.0.moe.router.weight"].t()).argmax(-1).tolist())
    assert len(experts_used) > 1  # the routing does route
    for steps in (traces.trace_whole(requests), traces.trace_chunks(requests), traces.trace_mixed(requests, seed=4)):
        result = traces.run_in_process(runner, steps)
        worst = max(float(np.abs(row - expected[n][p]).max()) for (n, p), row in result.items())
        assert worst < 3e-5, worst


def test_routed_toy_architecture_on_cpu(routed, monkeypatch):
    torch_kernels.install(monkeypatch)
    check_routed(routed, "cpu")


@pytest.mark.gpu
def test_routed_toy_architecture_on_gpu(routed):
    check_routed(routed, "cuda")


# ------------------------------------------------------------------ a third toy: another norm and another block arrangement
# A LayerNorm with a bias and a block in which the mixer and the feed-forward read the same normed
# rows and their outputs are added together (a parallel residual), both defined here; attention
# and the feed-forward are the package's.

from kairyu_b200.parts import BLOCKS, NORMS, Block, Norm  # noqa: E402

P_HIDDEN, P_INTER, P_VOCAB, P_HEADS, P_KV, P_HEAD = 56, 40, 83, 4, 2, 16
P_EPS = 1e-4


class ToyLayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * weight + bias, statistics in 32-bit; adds the pending delta first."""

    def __init__(self, *, name, size, eps, dtype, device, **_):
        self.name, self.size, self.eps, self.dtype = name, size, eps, dtype
        self.weight = self.bias = None

    def tensor_specs(self):
        return [TensorSpec(f"{self.name}.weight", (self.size,), role="vector", init="norm"), TensorSpec(f"{self.name}.bias", (self.size,), role="vector")]

    def load(self, tensors):
        self.weight, self.bias = tensors[f"{self.name}.weight"], tensors[f"{self.name}.bias"]

    def apply(self, residual, delta, ctx, *, rows=None):
        if rows is None:
            if delta is not None:
                residual.add_(delta.float())
            x = residual
        else:
            x = residual.index_select(0, rows.long())
            if delta is not None:
                x = x + delta.index_select(0, rows.long()).float()
        y = torch.nn.functional.layer_norm(x.float(), (self.size,), self.weight.float(), self.bias.float(), self.eps)
        return y.to(self.dtype)


class ParallelBlock(Block):
    """x += mixer(norm(x)) + ffn(norm(x)): one norm, both branches read it."""

    def __init__(self, *, layer, dtype, device, shared, **_):
        from kairyu_b200.parts import FEED_FORWARDS as feed_forwards

        context = dict(dtype=dtype, device=device, shared=shared)
        self.norm = NORMS.build(layer.mixer_norm, **context)
        self.mixer = MIXERS.build(layer.mixer, **context)
        self.ffn = feed_forwards.build(layer.ffn, **context)
        self._parts = (self.norm, self.mixer, self.ffn)

    def tensor_specs(self):
        return [spec for part in self._parts for spec in part.tensor_specs()]

    def load(self, tensors):
        for part in self._parts:
            part.load(tensors)

    def forward(self, residual, delta, ctx, cache):
        normed = self.norm.apply(residual, delta, ctx)
        return residual, self.mixer.forward(normed, ctx, cache) + self.ffn.forward(normed, ctx)


def parallel_spec(config) -> ModelSpec:
    def norm(name):
        return PartSpec("toy_layer_norm", name=name, size=P_HIDDEN, eps=P_EPS)

    position = PartSpec("rope", rotary_dim=P_HEAD, theta=5000.0, scaling=None, max_positions=192)
    layers = tuple(
        LayerSpec(
            f"layers.{i}", "toy_parallel",
            PartSpec("gqa_attention", prefix=f"layers.{i}.attn", hidden_size=P_HIDDEN, num_heads=P_HEADS, num_kv_heads=P_KV, head_dim=P_HEAD,
                     qk_norm=False, norm_eps=P_EPS, qkv_bias=False, o_bias=False, position=position),
            PartSpec("swiglu", prefix=f"layers.{i}.mlp", hidden_size=P_HIDDEN, intermediate_size=P_INTER, activation="silu"),
            norm(f"layers.{i}.ln"), norm(f"layers.{i}.unused"),
        )
        for i in range(2)
    )
    return ModelSpec(
        embedding=PartSpec("token_embedding", name="embed.weight", vocab_size=P_VOCAB, hidden_size=P_HIDDEN),
        layers=layers, schedule=(LayerCall(0, cache_slot=0), LayerCall(1, cache_slot=1)), final_norm=norm("final_ln"),
        head=PartSpec("linear_head", name="head.weight", vocab_size=P_VOCAB, hidden_size=P_HIDDEN, tied_to=None),
        vocab_size=P_VOCAB, hidden_size=P_HIDDEN, max_position_embeddings=192,
    )


@pytest.fixture
def parallel():
    NORMS.register("toy_layer_norm")(ToyLayerNorm)
    BLOCKS.register("toy_parallel")(ParallelBlock)
    register_architecture("ToyParallelForCausalLM", lambda config: dict(config), parallel_spec)
    yield {"architectures": ["ToyParallelForCausalLM"]}
    unregister_architecture("ToyParallelForCausalLM")
    BLOCKS.unregister("toy_parallel")
    NORMS.unregister("toy_layer_norm")


def plain_parallel_logits(w, tokens):
    lin = torch.nn.functional.linear
    cfg = {"head_dim": P_HEAD, "theta": 5000.0, "rope_kind": None, "rope": {}}
    T = len(tokens)
    cos, sin = plain_model.rope_cos_sin(cfg, torch.arange(T))

    def ln(x, name):
        return torch.nn.functional.layer_norm(x, (P_HIDDEN,), w[f"{name}.weight"], w[f"{name}.bias"], P_EPS)

    x = w["embed.weight"][torch.tensor(tokens)]
    for i in range(2):
        h = ln(x, f"layers.{i}.ln")
        q = lin(h, w[f"layers.{i}.attn.q_proj.weight"]).view(T, P_HEADS, P_HEAD)
        k = lin(h, w[f"layers.{i}.attn.k_proj.weight"]).view(T, P_KV, P_HEAD)
        v = lin(h, w[f"layers.{i}.attn.v_proj.weight"]).view(T, P_KV, P_HEAD)
        q, k = plain_model.apply_rope(q, k, cos, sin)
        x = x + lin(plain_model.causal_attention(q, k, v), w[f"layers.{i}.attn.o_proj.weight"]) + plain_model.swiglu_mlp(w, f"layers.{i}.mlp", h)
    return lin(ln(x, "final_ln"), w["head.weight"])


def check_parallel(config, device):
    model, _ = build_model(config, dtype="float32", device=device)
    weights = random_tensors(model.tensor_specs(), seed=15, device="cpu")
    for name in list(weights):
        if name.endswith(".bias"):  # biases that matter
            weights[name] = torch.randn(weights[name].shape, generator=torch.Generator().manual_seed(len(name))) * 0.3
    model.load({name: tensor.to(device) for name, tensor in weights.items()})
    assert not any("unused" in spec.name for spec in model.tensor_specs())  # the block builds what it uses
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=24, page_size=8, max_requests=4)
    storage = CacheStorage(layout, num_pages=24, page_size=8, max_requests=4, dtype=model.dtype, device=device)
    runner = ModelRunner(model, cache, storage, max_model_len=192, decode_mode="eager")
    requests = traces.make_requests(P_VOCAB, [37, 20, 51, 9, 44, 30], seed=10)
    expected = {name: plain_parallel_logits(weights, tokens).numpy() for name, tokens in requests.items()}
    for steps in (traces.trace_whole(requests), traces.trace_chunks(requests), traces.trace_mixed(requests, seed=5)):
        result = traces.run_in_process(runner, steps)
        worst = max(float(np.abs(row - expected[n][p]).max()) for (n, p), row in result.items())
        assert worst < 3e-5, worst


def test_parallel_toy_architecture_on_cpu(parallel, monkeypatch):
    torch_kernels.install(monkeypatch)
    check_parallel(parallel, "cpu")


@pytest.mark.gpu
def test_parallel_toy_architecture_on_gpu(parallel):
    check_parallel(parallel, "cuda")
