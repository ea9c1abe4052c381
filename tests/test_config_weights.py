"""Configuration, registry, safetensors files and the weight loader's single error (CPU only)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from pulse_infer_b200.config import (ConfigError, Qwen3Config, get_architecture, known_architectures, load_config,
                                     register_architecture)
from pulse_infer_b200.engine.builder import build_model
from pulse_infer_b200.parts.model import Runtime
from pulse_infer_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights, normal_tensor,
                                      write_random_model, write_safetensors)
from tiny_configs import CONFIGS, TINY_A, TINY_B, TINY_C

BASE = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256,
        "max_position_embeddings": 128, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": True,
        "torch_dtype": "bfloat16", "eos_token_id": 0}


def _write(tmp_path, obj, name="config.json"):
    with open(tmp_path / name, "w") as fh:
        json.dump(obj, fh)
    return str(tmp_path)


def test_config_reads_every_size_from_json(tmp_path):
    cfg = load_config(_write(tmp_path, BASE))
    assert isinstance(cfg, Qwen3Config) and cfg.architecture == "Qwen3ForCausalLM"
    assert (cfg.hidden_size, cfg.head_dim, cfg.q_size, cfg.kv_size, cfg.group_size) == (64, 16, 64, 32, 2)
    assert cfg.eos_token_ids == (0,) and cfg.layer_types == () and cfg.layer_window(1) is None
    assert load_config(str(tmp_path / "config.json")) == cfg          # a file inside the folder works too
    assert Qwen3Config.from_json_dict(cfg.to_json_dict()) == cfg


def test_config_generation_file_overrides_eos_and_gives_sampling_defaults(tmp_path):
    _write(tmp_path, BASE)
    _write(tmp_path, {"eos_token_id": [5, 6], "temperature": 0.6, "top_k": 20, "top_p": 0.95}, "generation_config.json")
    cfg = load_config(str(tmp_path))
    assert cfg.eos_token_ids == (5, 6) and cfg.temperature == pytest.approx(0.6) and cfg.top_k == 20


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta"])
def test_config_missing_key_is_named(tmp_path, key):
    obj = dict(BASE)
    del obj[key]
    with pytest.raises(ConfigError, match=key):
        load_config(_write(tmp_path, obj))


def test_config_validation(tmp_path):
    for patch, word in (({"num_key_value_heads": 3}, "multiple"), ({"hidden_size": 0}, "positive"),
                        ({"head_dim": 15}, "even"), ({"hidden_size": "64"}, "hidden_size"),
                        ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "not supported"),
                        ({"architectures": ["NoSuchModel"]}, "unknown architecture")):
        with pytest.raises(ConfigError, match=word):
            load_config(_write(tmp_path, {**BASE, **patch}))
    with pytest.raises(ConfigError, match="neither a folder"):
        load_config(str(tmp_path / "nowhere" / "x"))
    os.makedirs(tmp_path / "empty")
    with pytest.raises(ConfigError, match="does not exist"):
        load_config(str(tmp_path / "empty"))


@pytest.mark.parametrize("patch, word", [
    ({"attention_bias": True}, "attention_bias"), ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_dropout": 0.1}, "attention_dropout")])
def test_config_refuses_what_the_parts_cannot_compute(tmp_path, patch, word):
    """A key of the architecture's own config.json that asks for something the parts here do not do is an error that
    names the key - never a model silently computed without it."""
    with pytest.raises(ConfigError, match=word):
        load_config(_write(tmp_path, {**BASE, **patch}))
    # the same keys with the values that the parts do compute are accepted
    ok = {"attention_bias": False, "mlp_bias": False, "hidden_act": "silu", "attention_dropout": 0.0}
    assert load_config(_write(tmp_path, {**BASE, **ok})).hidden_size == 64


def test_config_window_keys(tmp_path):
    cfg = load_config(_write(tmp_path, {**BASE, "num_hidden_layers": 4, "use_sliding_window": True,
                                        "sliding_window": 32, "max_window_layers": 2}))
    assert cfg.layer_types == ("full_attention", "full_attention", "sliding_attention", "sliding_attention")
    assert [cfg.layer_window(i) for i in range(4)] == [None, None, 32, 32]
    cfg = load_config(_write(tmp_path, {**BASE, "sliding_window": 32, "use_sliding_window": False}))
    assert cfg.layer_types == () and cfg.sliding_window is None
    cfg = load_config(_write(tmp_path, {**BASE, "sliding_window": 8,
                                        "layer_types": ["sliding_attention", "full_attention"]}))
    assert [cfg.layer_window(i) for i in range(2)] == [8, None]


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    arch = get_architecture("Qwen3ForCausalLM")
    spec = arch.build_spec(TINY_C)
    assert len(spec.layers) == 4 and [e.cache for e in spec.order] == [0, 1, 2, 3]
    assert spec.layers[1].mixer.params["window"] == 24 and spec.layers[0].mixer.params["window"] is None
    with pytest.raises(ValueError):
        register_architecture("Qwen3ForCausalLM", Qwen3Config, arch.build_spec)


def test_random_weights_are_seeded_and_shaped(tmp_path):
    a = normal_tensor((1000, 64), 3, 5, 0.0, 0.02, torch.float32, "cpu")
    b = normal_tensor((1000, 64), 3, 5, 0.0, 0.02, torch.float32, "cpu")
    c = normal_tensor((1000, 64), 4, 5, 0.0, 0.02, torch.float32, "cpu")
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert abs(float(a.mean())) < 3e-4 and float(a.std()) == pytest.approx(0.02, rel=0.02)
    # a tensor's values do not depend on how it is cut: the first rows of a longer tensor are the same
    assert torch.equal(normal_tensor((10, 64), 3, 5, 0.0, 0.02, torch.float32, "cpu"), a[:10])
    folder = write_random_model(TINY_B, 1, str(tmp_path / "b"))
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    assert f.entries["model.layers.2.self_attn.q_proj.weight"].shape == (256, 96)
    assert f.entries["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert f.entries["lm_head.weight"].dtype == "BF16"
    assert float(f.tensor("model.norm.weight").float().mean()) == pytest.approx(1.0, abs=0.02)
    assert "lm_head.weight" not in SafetensorsFile(os.path.join(
        write_random_model(TINY_A, 0, str(tmp_path / "a")), "model.safetensors")).entries     # tied


def _cpu_model(cfg, mode="float32"):
    return build_model(cfg, Runtime(torch.device("cpu"), mode))


def test_loader_keeps_dtypes_by_policy(tmp_path):
    folder = write_random_model(TINY_A, 0, str(tmp_path / "m"))
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()           # one tensor stored in 32-bit
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    model = _cpu_model(TINY_A, "bfloat16")
    load_weights(model, folder, model.runtime)
    assert model.final_norm.weight.dtype == torch.float32                         # stays 32-bit
    assert model.layers[0].mixer.qkv.dtype == torch.bfloat16                      # stays bfloat16
    assert model.layers[0].mixer.qkv.shape == (64 + 2 * 32, 64)
    assert model.layers[1].feed_forward.gate_up.shape == (256, 64)
    assert model.lm_head.weight.data_ptr() == model.embedding.table.data_ptr()    # tied
    model32 = _cpu_model(TINY_A, "float32")
    load_weights(model32, folder, model32.runtime)
    assert model32.layers[0].mixer.qkv.dtype == torch.float32


def test_loader_reports_everything_in_one_error(tmp_path):
    folder = write_random_model(TINY_B, 1, str(tmp_path / "m"))
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16, dtype=torch.bfloat16)
    tensors["lm_head.weight"] = torch.ones(515, 95, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.ones(3)
    tensors["stray"] = torch.ones(2, dtype=torch.int64)
    write_safetensors(path, tensors)
    model = _cpu_model(TINY_B)
    with pytest.raises(WeightError) as info:
        load_weights(model, folder, model.runtime)
    e = info.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.extra.weight", "stray"]
    assert [w[0] for w in e.wrong_shape] == ["lm_head.weight", "model.layers.0.self_attn.q_norm.weight"]
    text = str(e)
    for word in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (2)", "expected [515, 96], got [515, 95]"):
        assert word in text
    # a second file that repeats a name
    write_safetensors(os.path.join(folder, "extra.safetensors"), {"stray": torch.ones(2)})
    with pytest.raises(WeightError, match="appear in two files"):
        load_weights(model, folder, model.runtime)


def test_safetensors_file_checks(tmp_path):
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
                             "b": torch.tensor([1.5, -2.0], dtype=torch.bfloat16), "i": torch.tensor([7, 8], dtype=torch.int64)})
    f = SafetensorsFile(path)
    assert torch.equal(f.tensor("a"), torch.arange(6.0).reshape(2, 3)) and f.tensor("b").dtype == torch.bfloat16
    assert f.tensor("i").tolist() == [7, 8]
    with pytest.raises(KeyError):
        f.tensor("zzz")

    def raw(header: dict, payload: bytes, declared=None):
        text = json.dumps(header).encode()
        with open(path, "wb") as fh:
            fh.write(struct.pack("<Q", len(text) if declared is None else declared) + text + payload)
    ok = {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}
    for header, payload, declared, word in (
            ({"a": ok}, b"\0" * 8, 10 ** 9, "header length"),
            ({"a": {**ok, "dtype": "F8_E4M3"}}, b"\0" * 8, None, "unsupported dtype"),
            ({"a": {**ok, "data_offsets": [0, 16]}}, b"\0" * 8, None, "outside the payload"),
            ({"a": {**ok, "shape": [3]}}, b"\0" * 8, None, "do not match"),
            ({"a": {**ok, "shape": [0], "data_offsets": [0, 0]}}, b"\0" * 8, None, "no elements"),
            ({"a": ok, "b": {**ok, "data_offsets": [4, 12]}}, b"\0" * 12, None, "overlap")):
        raw(header, payload, declared)
        with pytest.raises(SafetensorsError, match=word):
            SafetensorsFile(path)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", 5) + b"[1,2]")
    with pytest.raises(SafetensorsError, match="JSON object"):
        SafetensorsFile(path)


def test_model_spec_checks_schedule():
    from pulse_infer_b200.models.spec import ScheduleEntry
    from pulse_infer_b200.parts.model import DecoderModel
    import dataclasses
    spec = get_architecture("Qwen3ForCausalLM").build_spec(TINY_A)
    rt = Runtime(torch.device("cpu"), "float32")
    # a layer named twice with caches of its own is fine; two writers of one cache are not
    DecoderModel(dataclasses.replace(spec, order=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2))), rt)
    with pytest.raises(ValueError, match="written by two"):
        DecoderModel(dataclasses.replace(spec, order=(ScheduleEntry(0, 0), ScheduleEntry(1, 0))), rt)
    with pytest.raises(ValueError, match="names layer 5"):
        DecoderModel(dataclasses.replace(spec, order=(ScheduleEntry(5, 0),)), rt)
