"""Configuration, registry, safetensors reading and weight errors (no GPU)."""

import json

import dataclasses

import pytest
import torch

from matricxon_b200.config import (
    ConfigError,
    Starcoder2Config,
    UnsupportedArchitectureError,
    config_from_dict,
    load_config,
    supported_names,
)
from matricxon_b200.models.decoder import model_weight_specs, plan_cache
from matricxon_b200.parts.spec import ModelSpec, ScheduleEntry
from matricxon_b200.weights.loader import DictSource, WeightLoadError, check_weights, make_fetcher
from matricxon_b200.weights.random_init import random_tensors
from matricxon_b200.weights.safetensors_io import (
    ModelFiles,
    SafetensorsError,
    SafetensorsFile,
    write_safetensors,
)
from plain_reference import plain_read_safetensors
from tiny_configs import TINY, TINY_A, TINY_B, tiny_config, tiny_tensors, write_tiny_model


def test_registry_names_and_fail_closed():
    assert {"starcoder2", "Starcoder2ForCausalLM"} <= set(supported_names())
    assert isinstance(config_from_dict(dict(TINY_A)), Starcoder2Config)
    only_type = {k: v for k, v in TINY_A.items() if k != "architectures"}
    assert isinstance(config_from_dict(only_type), Starcoder2Config)
    with pytest.raises(UnsupportedArchitectureError):
        config_from_dict({**TINY_A, "architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    with pytest.raises(UnsupportedArchitectureError):
        config_from_dict({"hidden_size": 8})


def test_config_reads_every_key():
    a, b = tiny_config("A"), tiny_config("B")
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads,
            a.head_dim, a.intermediate_size, a.vocab_size) == (64, 2, 4, 2, 16, 256, 512)
    assert (a.rope_theta, a.sliding_window, a.norm_epsilon, a.use_bias, a.tie_word_embeddings) == \
        (10000.0, 32, 1e-5, True, True)
    assert (b.hidden_size, b.num_key_value_heads, b.head_dim, b.vocab_size, b.sliding_window,
            b.norm_epsilon, b.use_bias, b.tie_word_embeddings) == (96, 1, 32, 1000, 24, 1e-6, False, False)


def test_config_defaults_follow_the_reference():
    raw = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim",
                                                       "use_bias", "tie_word_embeddings")}
    config = config_from_dict(raw)
    assert config.num_key_value_heads == config.num_attention_heads
    assert config.head_dim == config.hidden_size // config.num_attention_heads
    assert config.use_bias and config.tie_word_embeddings
    assert config_from_dict({**TINY_A, "sliding_window": None}).sliding_window is None


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "vocab_size", "rope_theta", "norm_epsilon",
                                 "max_position_embeddings"])
def test_config_missing_key_is_named(key):
    raw = {k: v for k, v in TINY_A.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        config_from_dict(raw)


def test_config_rejects_bad_values():
    with pytest.raises(ConfigError, match="multiple"):
        config_from_dict({**TINY_A, "num_key_value_heads": 3})
    with pytest.raises(ConfigError, match="hidden_act"):
        config_from_dict({**TINY_A, "hidden_act": "silu"})
    with pytest.raises(ConfigError, match="integer"):
        config_from_dict({**TINY_A, "hidden_size": "64"})
    with pytest.raises(ConfigError, match="true or false"):
        config_from_dict({**TINY_A, "use_bias": 1})


def test_model_spec_carries_config_constants():
    spec = tiny_config("B").model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[0].mixer
    assert (mixer.num_heads, mixer.num_kv_heads, mixer.head_dim, mixer.window, mixer.bias) == (3, 1, 32, 24, False)
    assert mixer.scale == 32 ** -0.5 and mixer.position.theta == 100000.0
    assert spec.final_norm.eps == 1e-6 and not spec.tie_word_embeddings


def test_weight_names_and_shapes():
    names = {s.name: s for s in model_weight_specs(tiny_config("A").model_spec())}
    assert names["model.embed_tokens.weight"].shape == (512, 64)
    assert names["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert names["model.layers.0.mlp.c_fc.bias"].shape == (256,)
    assert names["model.layers.0.input_layernorm.bias"].role == "vector"
    assert "lm_head.weight" not in names
    names_b = {s.name for s in model_weight_specs(tiny_config("B").model_spec())}
    assert "lm_head.weight" in names_b
    assert not any(n.endswith("proj.bias") or n.endswith("c_fc.bias") for n in names_b)
    assert "model.layers.2.input_layernorm.bias" in names_b     # LayerNorm keeps its bias


def test_cache_plan_groups_and_shared_cache():
    spec = tiny_config("A").model_spec()
    plan = plan_cache(spec)
    assert len(plan.groups) == 1 and plan.groups[0].entries == (0, 1)
    assert plan.groups[0].request.window == 32
    shared = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                                 ScheduleEntry(1, cache_of=1)))
    plan = plan_cache(shared)
    assert plan.groups[0].entries == (0, 1, 2)          # layer 0 runs twice: two caches
    assert plan.kv_of_entry == ((0, 0), (0, 1), (0, 2), (0, 1)) and plan.writes[-1] is False
    with pytest.raises(ValueError):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0, cache_of=1), ScheduleEntry(1)))


def test_random_folder_round_trip(tmp_path):
    for name, dtype in (("A", torch.float32), ("B", torch.bfloat16)):
        folder = write_tiny_model(tmp_path / name, name, dtype)
        assert load_config(folder) == tiny_config(name).__class__.from_dict(
            json.loads((folder / "config.json").read_text()))
        files = ModelFiles(folder)
        tensors = tiny_tensors(name, dtype)
        assert set(files.names()) == set(tensors)
        for tensor_name in files.names():
            assert files.dtype(tensor_name) == dtype
            assert torch.equal(files.read(tensor_name), tensors[tensor_name])
        # the plain reader (own code) sees the same values
        plain = plain_read_safetensors(folder / "model.safetensors")
        assert torch.equal(plain["model.norm.weight"], tensors["model.norm.weight"].float())
    assert torch.equal(tiny_tensors("A")["model.embed_tokens.weight"],
                       random_tensors(tiny_config("A"), 0, TINY["A"][1])["model.embed_tokens.weight"])
    other_seed = random_tensors(tiny_config("A"), 5, TINY["A"][1])
    assert not torch.equal(other_seed["model.embed_tokens.weight"],
                           tiny_tensors("A")["model.embed_tokens.weight"])


def test_random_init_statistics():
    tensors = tiny_tensors("A")
    w = tensors["model.layers.0.mlp.c_fc.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    gamma = tensors["model.layers.0.input_layernorm.weight"]
    assert abs(gamma.mean().item() - 1.0) < 0.02 and gamma.std().item() > 0.005
    b = tiny_tensors("B")
    assert torch.all(b["model.norm.weight"] == 1) and torch.all(b["model.norm.bias"] == 0)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    specs = model_weight_specs(tiny_config("A").model_spec())
    tensors = tiny_tensors("A")
    del tensors["model.layers.1.mlp.c_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["lm_head.weight"] = torch.zeros(512, 64)              # tied config: not expected
    tensors["model.layers.7.bogus"] = torch.zeros(1)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    with pytest.raises(WeightLoadError) as caught:
        check_weights(specs, DictSource(tensors))
    error = caught.value
    assert error.missing == ["model.layers.1.mlp.c_proj.bias", "model.norm.weight"]
    assert error.unexpected == ["lm_head.weight", "model.layers.7.bogus"]
    assert error.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 64), (64, 32))]
    text = str(error)
    for fragment in ("missing (2)", "unexpected (2)", "model.norm.weight", "lm_head.weight",
                     "expected [64, 64], found [64, 32]"):
        assert fragment in text


def test_bias_tensors_without_use_bias_are_unexpected():
    specs = model_weight_specs(tiny_config("B").model_spec())
    tensors = tiny_tensors("B")
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(96)
    with pytest.raises(WeightLoadError, match="q_proj.bias"):
        check_weights(specs, DictSource(tensors))


def test_fetcher_holds_matrices_in_compute_dtype_and_vectors_in_float32():
    specs = model_weight_specs(tiny_config("A").model_spec())
    stored = tiny_tensors("A", torch.bfloat16)
    fetch = make_fetcher(specs, DictSource(stored), torch.bfloat16, "cpu")
    assert fetch("model.embed_tokens.weight").dtype == torch.bfloat16
    assert fetch("model.norm.weight").dtype == torch.float32
    assert fetch("model.layers.0.mlp.c_fc.bias").dtype == torch.float32
    fetch32 = make_fetcher(specs, DictSource(tiny_tensors("A")), torch.float32, "cpu")
    assert fetch32("model.embed_tokens.weight").dtype == torch.float32
    # a vector stored in 32-bit keeps every bit in bfloat16 serving
    fetch_mixed = make_fetcher(specs, DictSource(tiny_tensors("A")), torch.bfloat16, "cpu")
    assert torch.equal(fetch_mixed("model.norm.bias"), tiny_tensors("A")["model.norm.bias"])


def test_safetensors_errors(tmp_path):
    path = tmp_path / "model.safetensors"
    path.write_bytes(b"\x00\x01")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(path)
    write_safetensors(path, [("a", torch.arange(6, dtype=torch.float32).reshape(2, 3)),
                             ("b", torch.tensor([1, 2], dtype=torch.int32))])
    handle = SafetensorsFile(path)
    assert handle.entries["a"].shape == (2, 3) and handle.entries["b"].dtype == torch.int32
    data = bytearray(path.read_bytes())
    path.write_bytes(bytes(data[:-4]))                               # truncated payload
    with pytest.raises(SafetensorsError):
        SafetensorsFile(path)
    with pytest.raises(SafetensorsError):
        ModelFiles(tmp_path / "nowhere")
    with pytest.raises(ConfigError):
        load_config(tmp_path)


def test_sharded_folder(tmp_path):
    tensors = tiny_tensors("A")
    names = list(tensors)
    first, second = names[: len(names) // 2], names[len(names) // 2:]
    write_safetensors(tmp_path / "s1.safetensors", [(n, tensors[n]) for n in first])
    write_safetensors(tmp_path / "s2.safetensors", [(n, tensors[n]) for n in second])
    weight_map = {**{n: "s1.safetensors" for n in first}, **{n: "s2.safetensors" for n in second}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    files = ModelFiles(tmp_path)
    assert set(files.names()) == set(names)
    assert torch.equal(files.read(second[0]), tensors[second[0]])


def test_sizes_no_kernel_takes_are_refused_when_the_model_is_described():
    """head sizes in steps of 16 up to 256: anything else is refused by the configuration (and by
    the attention spec itself, for specs built by hand), not by the first kernel launch."""
    from matricxon_b200.config import ConfigError

    for head_dim in (8, 24, 40, 272):
        raw = dict(TINY_A, head_dim=head_dim)
        with pytest.raises(ConfigError, match="multiple of 16"):
            config_from_dict(raw)
    mixer = tiny_config("A").model_spec().layers[0].mixer
    with pytest.raises(ValueError, match="multiple of 16"):
        dataclasses.replace(mixer, head_dim=20)
    with pytest.raises(ValueError, match="kv heads"):
        dataclasses.replace(mixer, num_heads=5)
    with pytest.raises(ValueError, match="projection_names"):
        dataclasses.replace(mixer, projection_names=("q", "kv"))
    for head_dim in (16, 48, 80, 256):
        assert config_from_dict(dict(TINY_A, head_dim=head_dim)).head_dim == head_dim
