"""Configuration and registry (no GPU)."""
import json

import pytest

import ember_cpp_b200 as E
from ember_cpp_b200.config import ConfigError, architectures, config_from_dict, get_architecture, load_config
from ember_cpp_b200.parts import DecoderModel

from conftest import TINY


def test_registry_knows_gpt2():
    assert "GPT2LMHeadModel" in architectures()
    assert get_architecture("GPT2LMHeadModel").config_cls is E.GPT2Config


def test_unknown_architecture_lists_registered():
    with pytest.raises(ConfigError, match="GPT2LMHeadModel"):
        config_from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 8})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"n_embd": 8})


def test_defaults_and_derived():
    cfg = E.GPT2Config.from_dict(dict(vocab_size=10, n_positions=8, n_embd=12, n_layer=1, n_head=3))
    assert cfg.inner == 48 and cfg.head_dim == 4
    assert cfg.activation_function == "gelu_new" and cfg.tie_word_embeddings and cfg.layer_norm_epsilon == 1e-5
    assert cfg.eos_token_id is None and not cfg.scale_attn_by_inverse_layer_idx
    cfg = E.GPT2Config.from_dict(dict(vocab_size=10, n_ctx=8, n_embd=12, n_layer=1, n_head=3, n_inner=None))
    assert cfg.n_positions == 8 and cfg.inner == 48


@pytest.mark.parametrize("patch, word", [
    ({"n_head": 5}, "multiple"), ({"n_layer": 0}, "n_layer"), ({"activation_function": "relu"}, "activation_function"),
    ({"layer_norm_epsilon": 0.0}, "layer_norm_epsilon"), ({"eos_token_id": 9999}, "eos_token_id"),
    ({"n_embd": "wide"}, "n_embd"), ({"n_inner": -3}, "n_inner"), ({"tie_word_embeddings": 1}, "tie_word_embeddings"),
])
def test_validation_names_the_key(patch, word):
    with pytest.raises(ConfigError, match=word):
        E.GPT2Config.from_dict({**TINY["tiny_a"], **patch})


def test_missing_key_is_named():
    d = dict(TINY["tiny_a"])
    del d["n_head"]
    with pytest.raises(ConfigError, match="n_head"):
        E.GPT2Config.from_dict(d)


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps({**TINY["tiny_b"], "architectures": ["GPT2LMHeadModel"],
                                                      "some_unknown_key": 3}))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, E.GPT2Config) and cfg.n_inner == 320 and cfg.scale_attn_by_inverse_layer_idx
    assert E.GPT2Config.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("name", list(TINY))
def test_spec_follows_the_configuration(name):
    cfg = E.GPT2Config.from_dict(TINY[name])
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    assert len(spec.layers) == cfg.n_layer and [a.layer for a in spec.schedule] == list(range(cfg.n_layer))
    assert (spec.head is None) == cfg.tie_word_embeddings
    scales = [layer.mixer.params["scale"] for layer in spec.layers]
    base = cfg.head_dim ** -0.5
    want = [base / (i + 1) if cfg.scale_attn_by_inverse_layer_idx else base for i in range(cfg.n_layer)]
    assert scales == pytest.approx(want)
    model = DecoderModel(spec)
    names = {w.name: w.shape for w in model.weight_specs()}
    assert names["h.0.attn.c_attn.weight"] == (cfg.n_embd, 3 * cfg.n_embd)       # Conv1D: [in, out]
    assert names["h.0.mlp.c_proj.weight"] == (cfg.inner, cfg.n_embd)
    assert names["wpe.weight"] == (cfg.n_positions, cfg.n_embd)
    assert ("lm_head.weight" in names) == (not cfg.tie_word_embeddings)
    n_params = sum(int(__import__("math").prod(s)) for s in names.values())
    assert n_params == {"tiny_a": 141056, "tiny_b": 499872}[name]


def test_spec_check_rejects_bad_schedules():
    from ember_cpp_b200.parts import Application
    import dataclasses
    cfg = E.GPT2Config.from_dict(TINY["tiny_a"])
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    with pytest.raises(ValueError, match="names layer"):
        dataclasses.replace(spec, schedule=(Application(5),)).check()
    with pytest.raises(ValueError, match="earlier"):
        dataclasses.replace(spec, schedule=(Application(0, cache_of=0),)).check()
    dataclasses.replace(spec, schedule=(Application(0), Application(1), Application(0), Application(1, cache_of=1))).check()
