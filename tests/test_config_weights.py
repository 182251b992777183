"""Configuration parsing, the registry, weight loading and its errors, the
random-weights writer.  CPU only."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from tiny_configs import TINY, TINY_LLAMA, TINY_QWEN3

from kairyu_b200.config import ConfigError, EngineConfig, parse_dense_config
from kairyu_b200.engine.engine import load_model
from kairyu_b200.registry import architecture_of, register_architecture, supported_architectures, unregister_architecture
from kairyu_b200.weights import WeightError, write_random_model


def test_both_config_generations_parse_alike():
    old = dict(TINY_LLAMA)
    new = {k: v for k, v in TINY_LLAMA.items() if k not in ("rope_theta", "rope_scaling")}
    new["rope_parameters"] = dict(TINY_LLAMA["rope_scaling"], rope_theta=TINY_LLAMA["rope_theta"])
    new["dtype"] = "bfloat16"
    a = parse_dense_config(old, "LlamaForCausalLM")
    b = parse_dense_config(new, "LlamaForCausalLM")
    assert a.rope_theta == b.rope_theta == 10000.0
    assert a.rope_scaling == b.rope_scaling and a.rope_scaling.kind == "llama3"
    assert a.rope_scaling.original_max_position_embeddings == 64
    assert b.stored_dtype == "bfloat16" and a.stored_dtype == "float32"


def test_defaults_and_derived_sizes():
    config = parse_dense_config(
        {"hidden_size": 64, "num_attention_heads": 4, "num_hidden_layers": 1, "intermediate_size": 8, "vocab_size": 10},
        "LlamaForCausalLM",
    )
    assert config.num_key_value_heads == 4 and config.head_dim == 16
    assert config.rms_norm_eps == 1e-6 and config.rope_theta == 10000.0
    assert config.max_position_embeddings == 4096 and not config.tie_word_embeddings
    assert config.rope_scaling is None and not config.attention_bias
    qwen = parse_dense_config(TINY_QWEN3, "Qwen3ForCausalLM")
    assert qwen.head_dim == 32 and qwen.q_size == 192 and qwen.kv_size == 96


@pytest.mark.parametrize(
    "change,message",
    [
        ({"hidden_size": None}, "hidden_size"),
        ({"num_attention_heads": 0}, "num_attention_heads"),
        ({"num_key_value_heads": 3}, "multiple"),
        ({"vocab_size": "many"}, "vocab_size"),
        ({"rope_scaling": {"rope_type": "dynamic", "factor": 2.0}}, "rope scaling"),
        ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "missing"),
        ({"sliding_window": 128}, "sliding-window"),
        ({"hidden_act": "gelu"}, "hidden_act"),
        ({"quantization_config": {"quant_method": "fp8"}}, "quantized"),
        ({"head_dim": 15}, "even"),
    ],
)
def test_config_errors(change, message):
    config = dict(TINY_LLAMA)
    config.update(change)
    with pytest.raises(ConfigError, match=message):
        parse_dense_config(config, "LlamaForCausalLM")


def test_qwen3_sliding_window_key_with_use_false_is_accepted():
    config = dict(TINY_QWEN3, sliding_window=None, use_sliding_window=False)
    parse_dense_config(config, "Qwen3ForCausalLM")
    parse_dense_config(dict(TINY_QWEN3, sliding_window=4096, use_sliding_window=False), "Qwen3ForCausalLM")


def test_registry_maps_names_to_one_decoder_and_is_open():
    assert {"LlamaForCausalLM", "Qwen3ForCausalLM"} <= set(supported_architectures())
    with pytest.raises(ConfigError, match="unsupported architecture 'GPT2LMHeadModel'.*LlamaForCausalLM"):
        architecture_of({"architectures": ["GPT2LMHeadModel"]})
    with pytest.raises(ConfigError):
        architecture_of({})
    llama = architecture_of(TINY_LLAMA)
    qwen = architecture_of(TINY_QWEN3)
    spec_l = llama.build_spec(llama.parse_config(TINY_LLAMA))
    spec_q = qwen.build_spec(qwen.parse_config(TINY_QWEN3))
    assert spec_l.layers[0].mixer.params["qk_norm"] is False
    assert spec_q.layers[0].mixer.params["qk_norm"] is True
    assert spec_q.head.params["tied_to"] == "model.embed_tokens.weight" and spec_l.head.params["tied_to"] is None
    register_architecture("ToyForCausalLM", llama.parse_config, llama.build_spec)
    try:
        assert architecture_of({"architectures": ["ToyForCausalLM"]}).name == "ToyForCausalLM"
    finally:
        unregister_architecture("ToyForCausalLM")


def test_engine_config_validates_and_rejects_unknown_keys():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    assert EngineConfig(dtype="auto").dtype == "bfloat16"
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(page_size=0)
    with pytest.raises(TypeError, match="unknown engine option"):
        EngineConfig.from_kwargs(num_page=3)


@pytest.mark.parametrize("name", ["llama", "qwen3", "odd", "wide", "yarn"])
def test_random_folder_round_trip(name, tmp_path):
    config, seed, _ = TINY[name]
    folder = write_random_model(config, tmp_path / name, seed=seed, dtype="float32")
    assert json.loads((folder / "config.json").read_text())["architectures"] == config["architectures"]
    stored = load_file(str(folder / "model.safetensors"))
    assert ("lm_head.weight" in stored) == (not config.get("tie_word_embeddings", False))
    model, parsed = load_model(folder, dtype="float32", device="cpu")
    assert parsed.vocab_size == config["vocab_size"]
    mixer = model.blocks[0].mixer
    q = stored["model.layers.0.self_attn.q_proj.weight"]
    assert torch.equal(mixer.w_qkv[: q.shape[0]], q)
    assert torch.equal(model.blocks[-1].ffn.w_down, stored[f"model.layers.{len(model.blocks) - 1}.mlp.down_proj.weight"])
    if config.get("tie_word_embeddings"):
        assert model.head.weight.data_ptr() == model.embedding.weight.data_ptr()
    # a seed fixes every tensor; another seed changes them
    again = write_random_model(config, tmp_path / "again", seed=seed, dtype="float32")
    other = write_random_model(config, tmp_path / "other", seed=seed + 1, dtype="float32")
    a, b = load_file(str(again / "model.safetensors")), load_file(str(other / "model.safetensors"))
    assert all(torch.equal(stored[k], a[k]) for k in stored)
    assert not torch.equal(stored["model.norm.weight"], b["model.norm.weight"])
    # the stated distributions
    assert abs(float(stored["model.embed_tokens.weight"].std()) - 0.02) < 0.002
    assert abs(float(stored["model.norm.weight"].mean()) - 1.0) < 0.05


def test_held_dtypes_in_bfloat16_mode(tmp_path):
    config, seed, _ = TINY["qwen3"]
    folder = write_random_model(config, tmp_path / "m", seed=seed, dtype="float32")
    model, _ = load_model(folder, dtype="bfloat16", device="cpu")
    assert model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    assert model.embedding.weight.dtype == torch.bfloat16
    assert model.blocks[0].mixer_norm.weight.dtype == torch.float32  # stored in 32-bit: stays so
    assert model.blocks[0].mixer.q_norm_weight.dtype == torch.float32
    folder16 = write_random_model(config, tmp_path / "m16", seed=seed, dtype="bfloat16")
    model16, _ = load_model(folder16, dtype="bfloat16", device="cpu")
    assert model16.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    model32, _ = load_model(folder16, dtype="float32", device="cpu")
    assert model32.blocks[0].mixer.w_qkv.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config, seed, _ = TINY["llama"]
    folder = write_random_model(config, tmp_path / "m", seed=seed, dtype="float32")
    path = folder / "model.safetensors"
    tensors = {k: v.clone() for k, v in load_file(str(path)).items()}  # not views of the file about to be rewritten
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(7, 64)
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # ignored, as exporters write it
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    save_file(tensors, str(path))
    with pytest.raises(WeightError) as caught:
        load_model(folder, dtype="float32", device="cpu")
    error = caught.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.0.extra.weight"]
    assert error.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (7, 64), (32, 64))]
    assert error.wrong_dtype and error.wrong_dtype[0][0] == "model.layers.0.input_layernorm.weight"
    text = str(error)
    for part in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [7, 64], expected [32, 64]"):
        assert part in text


def test_missing_files(tmp_path):
    with pytest.raises(ValueError, match="config.json"):
        load_model(tmp_path, dtype="float32", device="cpu")
    (tmp_path / "config.json").write_text(json.dumps(TINY_LLAMA))
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model(tmp_path, dtype="float32", device="cpu")


def test_sharded_checkpoint_with_index(tmp_path):
    config, seed, _ = TINY["llama"]
    folder = write_random_model(config, tmp_path / "m", seed=seed, dtype="float32")
    tensors = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    (folder / "model.safetensors").unlink()
    names = sorted(tensors)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for shard, keys in shards.items():
        save_file({k: tensors[k] for k in keys}, str(folder / shard))
        weight_map.update({k: shard for k in keys})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    model, _ = load_model(folder, dtype="float32", device="cpu")
    assert torch.equal(model.final_norm.weight, tensors["model.norm.weight"])
    weight_map["model.norm.weight"] = "../elsewhere.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(ValueError, match="outside the model folder"):
        load_model(folder, dtype="float32", device="cpu")


def test_tied_head_in_file_is_not_unexpected(tmp_path):
    config, seed, _ = TINY["qwen3"]
    folder = write_random_model(config, tmp_path / "m", seed=seed, dtype="float32")
    path = folder / "model.safetensors"
    tensors = {k: v.clone() for k, v in load_file(str(path)).items()}  # not views of the file about to be rewritten
    tensors["lm_head.weight"] = torch.zeros_like(tensors["model.embed_tokens.weight"])
    save_file(tensors, str(path))
    model, _ = load_model(folder, dtype="float32", device="cpu")
    assert torch.equal(model.head.weight, tensors["model.embed_tokens.weight"])  # the tie wins, as in the reference


def test_tensors_the_model_does_not_ask_for_are_passed_over_unless_strict(tmp_path):
    """kairyu/models/loader.py:250 loads with strict=False: exports carry stray buffers."""
    from kairyu_b200.engine.engine import build_model
    from kairyu_b200.weights.loading import load_into

    config, seed, _ = TINY["llama"]
    folder = write_random_model(config, tmp_path / "m", seed=seed, dtype="float32")
    path = folder / "model.safetensors"
    tensors = {k: v.clone() for k, v in load_file(str(path)).items()}
    tensors["model.layers.0.self_attn.stray_buffer"] = torch.zeros(3)
    save_file(tensors, str(path))
    model, _ = load_model(folder, dtype="float32", device="cpu")
    assert torch.equal(model.embedding.weight, tensors["model.embed_tokens.weight"])
    strict, _ = build_model(config, dtype="float32", device="cpu")
    with pytest.raises(WeightError) as caught:
        load_into(strict, folder, strict_unexpected=True)
    assert caught.value.unexpected == ["model.layers.0.self_attn.stray_buffer"] and not caught.value.missing
