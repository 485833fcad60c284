"""Configuration, registry, safetensors container and weight-by-name errors (no GPU)."""
from __future__ import annotations

import copy
import json
import os
import struct

import pytest
import torch

from celeg_b200.config import (ConfigError, Lfm2Config, UnknownArchitectureError, architecture_of,
                               build_lfm2_spec, known_architectures)
from celeg_b200.config.spec import ExecutionEntry
from celeg_b200.weights import (CheckpointFormatError, TensorRepository, WeightsError, load_tensors,
                                write_random_model, write_safetensors)
from tiny_models import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_config():
    a = Lfm2Config.from_dict(TINY_A)
    assert (a.vocab_size, a.hidden_size, a.num_hidden_layers) == (512, 64, 4)
    assert a.head_dim == 16 and a.intermediate_size == 192 and a.conv_L_cache == 3
    assert a.norm_eps == 1e-5 and a.rope_theta == 10000.0 and a.eos_token_ids == (7,)
    b = Lfm2Config.from_dict(TINY_B)
    assert b.head_dim == 32 and b.num_key_value_heads == 1 and b.tie_word_embeddings is False
    assert b.eos_token_ids == (7, 9) and b.layer_types[0] == "full_attention"
    c = Lfm2Config.from_dict(TINY_C)
    assert c.layer_types == ("conv", "full_attention", "conv")


def test_aliases_defaults_and_nested_rope():
    raw = {"model_type": "lfm2", "n_vocab": 50, "d_model": 32, "n_layer": 1, "n_head": 2, "max_seq_len": 64,
           "rms_norm_eps": 2e-5, "rope_parameters": {"rope_theta": 777.0}, "layer_types": ["full_attention"],
           "intermediate_size": 48}
    config = Lfm2Config.from_dict(raw)
    assert config.vocab_size == 50 and config.num_key_value_heads == 2 and config.head_dim == 16
    assert config.norm_eps == 2e-5 and config.rope_theta == 777.0
    del raw["rms_norm_eps"]
    assert Lfm2Config.from_dict(raw).norm_eps == 1e-6


@pytest.mark.parametrize("change,fragment", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"layer_types": ["conv"]}, "layer_types"),
    ({"layer_types": ["conv", "conv", "banana", "conv"]}, "banana"),
    ({"conv_L_cache": None}, "conv_L_cache"),
    ({"rope_theta": None}, "rope_theta"),
    ({"conv_bias": True}, "conv_bias"),
    ({"norm_eps": 0.0}, "norm_eps"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": "big"}, "vocab_size"),
])
def test_config_errors_name_the_key(change, fragment):
    raw = copy.deepcopy(TINY_A)
    for key, value in change.items():
        if value is None:
            raw.pop(key)
        else:
            raw[key] = value
    with pytest.raises(ConfigError) as info:
        Lfm2Config.from_dict(raw)
    assert fragment in str(info.value)


def test_registry_knows_lfm2_and_refuses_others():
    assert "lfm2" in known_architectures()
    assert architecture_of(TINY_A).name == "lfm2"
    with pytest.raises(UnknownArchitectureError) as info:
        architecture_of({"model_type": "llama"})
    assert "lfm2" in str(info.value)
    with pytest.raises(UnknownArchitectureError):
        architecture_of({})


def test_spec_lists_parts_layer_by_layer():
    spec = build_lfm2_spec(Lfm2Config.from_dict(TINY_B).resolved_with({}))
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["attention", "short_conv", "short_conv", "attention", "short_conv", "attention"]
    assert spec.lm_head is not None and spec.lm_head.shape == (1000, 96)
    assert [entry.layer for entry in spec.order] == list(range(6))
    attention = spec.layers[0].mixer
    assert attention.params["num_heads"] == 3 and attention.parts["position"].params["theta"] == 1e6
    assert spec.layers[1].mixer.params["taps"] == 4


def test_run_order_is_validated():
    import dataclasses
    spec = build_lfm2_spec(Lfm2Config.from_dict(TINY_A))
    bad = dataclasses.replace(spec, order=(ExecutionEntry(0), ExecutionEntry(9)))
    with pytest.raises(ConfigError):
        bad.validate()
    bad = dataclasses.replace(spec, order=(ExecutionEntry(2, cache_of=0),))
    with pytest.raises(ConfigError):
        bad.validate()
    twice = dataclasses.replace(spec, order=(ExecutionEntry(2), ExecutionEntry(0), ExecutionEntry(2, cache_of=0)))
    twice.validate()


def test_missing_pieces_are_read_from_tensors(tmp_path):
    raw = copy.deepcopy(TINY_A)
    folder = write_random_model(str(tmp_path / "m"), raw, 0)
    for key in ("layer_types", "block_ff_dim", "tie_word_embeddings"):
        raw.pop(key)
    config = Lfm2Config.from_dict(raw)
    assert config.layer_types is None and config.intermediate_size is None
    with pytest.raises(ConfigError):
        config.require_resolved()
    repository = TensorRepository(folder)
    resolved = config.resolved_with(repository.shapes())
    repository.close()
    assert resolved.layer_types == ("conv", "conv", "full_attention", "conv")
    assert resolved.intermediate_size == 192 and resolved.tie_word_embeddings is True


def test_random_model_round_trip_and_determinism(tmp_path):
    one = write_random_model(str(tmp_path / "one"), TINY_B, 1)
    two = write_random_model(str(tmp_path / "two"), TINY_B, 1)
    other = write_random_model(str(tmp_path / "other"), TINY_B, 2)
    a, b, c = (TensorRepository(p) for p in (one, two, other))
    spec = build_lfm2_spec(Lfm2Config.from_dict(TINY_B))
    ta, tb, tc = load_tensors(a, spec), load_tensors(b, spec), load_tensors(c, spec)
    assert set(ta) == {ref.name for ref in spec.all_tensors()}
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    assert ta["model.layers.1.conv.conv.weight"].shape == (96, 4)        # stored [H,1,L], used [H,L]
    assert ta["model.embed_tokens.weight"].dtype == torch.bfloat16
    norm = ta["model.layers.0.operator_norm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.05
    assert 0.015 < float(ta["lm_head.weight"].float().std()) < 0.025
    assert 0.07 < float(ta["model.layers.1.conv.conv.weight"].float().std()) < 0.13
    # the official reader sees the same bytes
    from safetensors.torch import load_file
    official = load_file(os.path.join(one, "model.safetensors"))
    assert all(torch.equal(official[k].reshape(ta[k].shape), ta[k]) for k in ta)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    repository = TensorRepository(folder)
    tensors = {name: repository.tensor(name) for name in repository.names()}
    repository.close()
    del tensors["model.layers.2.self_attn.k_layernorm.weight"]
    del tensors["model.layers.0.conv.out_proj.weight"]
    tensors["model.layers.0.banana.weight"] = torch.zeros(3)
    tensors["model.layers.1.feed_forward.w2.weight"] = torch.zeros(64, 191, dtype=torch.bfloat16)
    tensors["model.embedding_norm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    repository = TensorRepository(folder)
    spec = build_lfm2_spec(Lfm2Config.from_dict(TINY_A))
    with pytest.raises(WeightsError) as info:
        load_tensors(repository, spec)
    repository.close()
    error = info.value
    assert sorted(error.missing) == ["model.layers.0.conv.out_proj.weight",
                                     "model.layers.2.self_attn.k_layernorm.weight"]
    assert error.unexpected == ["model.layers.0.banana.weight"]
    assert error.wrong_shape == [("model.layers.1.feed_forward.w2.weight", (64, 191), (64, 192))]
    assert error.wrong_dtype == [("model.embedding_norm.weight", "I32")]
    text = str(error)
    for fragment in ("missing", "unexpected", "wrong shapes", "banana", "[64, 191]", "[64, 192]"):
        assert fragment in text


def test_kept_precision(tmp_path):
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {"a": torch.ones(2, dtype=torch.bfloat16), "b": torch.ones(2, dtype=torch.float32),
                             "c": torch.ones(2, dtype=torch.float16), "d": torch.ones(2, dtype=torch.int64)})
    from celeg_b200.weights import kept_precision
    repository = TensorRepository(str(tmp_path))
    got = {name: kept_precision(repository.tensor(name)).dtype for name in "abcd"}
    repository.close()
    assert got == {"a": torch.bfloat16, "b": torch.float32, "c": torch.float32, "d": torch.int32}


def _raw_file(tmp_path, header: dict, data: bytes = b"", raw_header: bytes = None):
    blob = raw_header if raw_header is not None else json.dumps(header).encode()
    path = tmp_path / "model.safetensors"
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + data)
    return str(tmp_path)


@pytest.mark.parametrize("case", ["short", "header_len", "not_json", "dtype", "range", "size", "overlap"])
def test_malformed_containers_are_refused(tmp_path, case):
    if case == "short":
        (tmp_path / "model.safetensors").write_bytes(b"abc")
        folder = str(tmp_path)
    elif case == "header_len":
        (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
        folder = str(tmp_path)
    elif case == "not_json":
        folder = _raw_file(tmp_path, {}, raw_header=b"{nope")
    elif case == "dtype":
        folder = _raw_file(tmp_path, {"t": {"dtype": "F4", "shape": [2], "data_offsets": [0, 2]}}, b"\0" * 2)
    elif case == "range":
        folder = _raw_file(tmp_path, {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4)
    elif case == "size":
        folder = _raw_file(tmp_path, {"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    else:
        folder = _raw_file(tmp_path, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                                      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
    with pytest.raises(CheckpointFormatError):
        TensorRepository(folder)


def test_missing_checkpoint_is_reported(tmp_path):
    with pytest.raises(CheckpointFormatError):
        TensorRepository(str(tmp_path))


def test_generation_config_overrides_stop_ids(tmp_path):
    """celeg lets generation_config.json replace bos/eos (src/checkpoint/catalog.cpp:95-123): a number or a
    list of numbers; other keys and unreadable files change nothing."""
    from celeg_b200.config.registry import read_config_json
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    assert Lfm2Config.from_dict(read_config_json(str(folder))).eos_token_ids == (7,)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 2, 11], "bos_token_id": 5,
                                                               "pad_token_id": 3, "temperature": 0.3}))
    config = Lfm2Config.from_dict(read_config_json(str(folder)))
    assert config.eos_token_ids == (7, 2, 11) and config.bos_token_id == 5 and config.pad_token_id == 0
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": 9}))
    assert Lfm2Config.from_dict(read_config_json(str(folder))).eos_token_ids == (9,)
    (folder / "generation_config.json").write_text("{ not json")
    assert Lfm2Config.from_dict(read_config_json(str(folder))).eos_token_ids == (7,)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": []}))
    assert Lfm2Config.from_dict(read_config_json(str(folder))).eos_token_ids == (7,)


def test_fingerprint_follows_configuration_and_tensor_table(tmp_path):
    """Equal for the same architecture and sizes whatever the weights' values; different as soon as a size, an
    option or a tensor's shape or stored type differs."""
    from celeg_b200.config.fingerprint import model_fingerprint
    from celeg_b200.config.registry import read_config_json
    from celeg_b200.engine.loading import fingerprint_of

    def of(folder):
        raw = read_config_json(folder)
        architecture = architecture_of(raw)
        repository = TensorRepository(folder)
        try:
            config = architecture.resolve_config(architecture.parse_config(raw), repository.shapes())
            return fingerprint_of(config, raw, repository)
        finally:
            repository.close()

    a0 = str(tmp_path / "a0")
    a1 = str(tmp_path / "a1")
    b0 = str(tmp_path / "b0")
    f32 = str(tmp_path / "f32")
    eps = str(tmp_path / "eps")
    write_random_model(a0, copy.deepcopy(TINY_A), 0)
    write_random_model(a1, copy.deepcopy(TINY_A), 1)
    write_random_model(b0, copy.deepcopy(TINY_B), 0)
    write_random_model(f32, copy.deepcopy(TINY_A), 0, torch.float32)
    other = copy.deepcopy(TINY_A)
    other["norm_eps"] = 2e-5
    write_random_model(eps, other, 0)
    prints = {name: of(folder) for name, folder in (("a0", a0), ("a1", a1), ("b0", b0), ("f32", f32), ("eps", eps))}
    assert all(len(value) == 64 and int(value, 16) >= 0 for value in prints.values())
    assert prints["a0"] == prints["a1"]
    assert len({prints["a0"], prints["b0"], prints["f32"], prints["eps"]}) == 4
    shapes = {"w": (2, 3)}
    assert model_fingerprint({"x": 1}, shapes, {"w": "BF16"}) != model_fingerprint({"x": 1}, {"w": (3, 2)}, {"w": "BF16"})


def test_kernel_options_are_typed_and_checked():
    """The switches of the kernel path are fields of one object; the environment is read only on request."""
    from celeg_b200 import KernelOptions
    defaults = KernelOptions()
    assert (defaults.tensor_core_products, defaults.split_norms, defaults.tcgen05_attention) == ("swiglu", True, True)
    read = KernelOptions.from_env({"CELEG_B200_TENSOR_CORE_PRODUCTS": "all", "CELEG_B200_SPLIT_NORMS": "0",
                                   "CELEG_B200_PREFETCH_MB": "4.5", "CELEG_B200_TENSOR_CORE_MIN_ROWS": "512",
                                   "UNRELATED": "1"})
    assert (read.tensor_core_products, read.split_norms, read.prefetch_mb, read.tensor_core_min_rows) == ("all", False, 4.5, 512)
    assert KernelOptions.from_env({}) == defaults
    with pytest.raises(ValueError, match="tensor_core_products"):
        KernelOptions(tensor_core_products="stream").validate()
    with pytest.raises(ValueError):
        KernelOptions.from_env({"CELEG_B200_TENSOR_CORE_VARIANT": "9"})
