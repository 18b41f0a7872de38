"""The safetensors container, the checked loader and the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

import ember_cpp_b200 as E
from ember_cpp_b200.config import get_architecture
from ember_cpp_b200.parts import DecoderModel
from ember_cpp_b200.weights import (SafetensorsError, UnreadTensor, WeightError, check_tensors, load_checked, random_tensors,
                                    read_file, read_folder, read_header, write_file)

from conftest import TINY


def _model(name="tiny_a"):
    cfg = E.GPT2Config.from_dict(TINY[name])
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    return cfg, spec, DecoderModel(spec)


def test_round_trip_keeps_types(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.randn(2, 2).to(torch.float16),
               "t": torch.arange(6, dtype=torch.int64).reshape(2, 3), "e": torch.empty(0, 4)}
    path = str(tmp_path / "model.safetensors")
    write_file(path, tensors, {"note": "x"})
    back = read_file(path)
    assert back["a"].dtype == torch.bfloat16 and torch.equal(back["a"], tensors["a"])        # kept in bfloat16
    assert back["b"].dtype == torch.float32 and torch.equal(back["b"], tensors["b"])        # 32-bit stays 32-bit
    assert back["c"].dtype == torch.float32 and torch.equal(back["c"], tensors["c"].float())
    assert back["t"].dtype == torch.int32 and back["t"].tolist() == [[0, 1, 2], [3, 4, 5]]   # integer tables: int32
    assert tuple(back["e"].shape) == (0, 4)
    # also readable by the reference reader of the format
    import safetensors.torch
    other = safetensors.torch.load_file(path)
    assert torch.equal(other["a"], tensors["a"]) and torch.equal(other["t"], tensors["t"])


def test_container_errors(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        read_file(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        read_file(str(p))
    p.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(SafetensorsError, match="not JSON"):
        read_file(str(p))
    head = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 8)       # data block too short
    with pytest.raises(SafetensorsError, match="bytes"):
        read_file(str(p))
    head = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="needs 16"):
        read_file(str(p))
    head = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 4)
    got = read_file(str(p))["w"]                  # a type the reader does not know: named, not fetched
    assert isinstance(got, UnreadTensor) and got.dtype_name == "F8_E4M3" and got.shape == (4,)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        read_folder(str(tmp_path / "nowhere"))


def test_sharded_folder(tmp_path):
    write_file(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2)})
    write_file(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    assert sorted(read_folder(str(tmp_path))) == ["a", "b"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    _, spec, model = _model()
    tensors = random_tensors(model.weight_specs(), 0)
    del tensors["h.1.ln_2.bias"], tensors["wpe.weight"]
    tensors["h.0.attn.c_attn.weight"] = tensors["h.0.attn.c_attn.weight"].t().contiguous()   # [out, in]: wrong
    tensors["h.0.mlp.extra"] = torch.zeros(2)
    tensors["transformer.h.9.ln_1.weight"] = torch.zeros(64)
    tensors["h.0.attn.bias"] = torch.ones(1, 1, 8, 8)         # a buffer of GPT-2 checkpoints: ignored
    with pytest.raises(WeightError) as e:
        check_tensors("here", tensors, model.weight_specs(), spec.ignored_tensors, spec.strip_prefixes)
    err = e.value
    assert err.missing == ["h.1.ln_2.bias", "wpe.weight"]
    assert err.unexpected == ["h.0.mlp.extra", "h.9.ln_1.weight"]
    assert err.wrong_shape == [("h.0.attn.c_attn.weight", (64, 192), (192, 64))]
    text = str(err)
    for word in ("missing (2)", "unexpected (2)", "wrong shape", "h.1.ln_2.bias", "h.0.mlp.extra", "[192, 64]",
                 "[64, 192]"):
        assert word in text


def test_prefix_tied_duplicate_and_untied_head():
    _, spec, model = _model("tiny_a")
    tensors = {"transformer." + k: v for k, v in random_tensors(model.weight_specs(), 0).items()}
    tensors["lm_head.weight"] = tensors["transformer.wte.weight"]      # tied checkpoints may repeat it
    got = check_tensors("here", tensors, model.weight_specs(), spec.ignored_tensors, spec.strip_prefixes)
    assert "wte.weight" in got and "lm_head.weight" not in got
    assert spec.strip_prefixes == ("transformer.",)                    # the architecture's own detail, not the loader's
    with pytest.raises(WeightError, match="unexpected"):               # without it the names do not fit
        check_tensors("here", tensors, model.weight_specs(), spec.ignored_tensors)
    _, spec_b, model_b = _model("tiny_b")
    tensors = random_tensors(model_b.weight_specs(), 0)
    del tensors["lm_head.weight"]
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_tensors("here", tensors, model_b.weight_specs(), spec_b.ignored_tensors)


def test_a_buffer_of_a_type_the_reader_does_not_know_is_ignored_unless_wanted(tmp_path):
    """GPT-2 checkpoints of some writers store the causal mask `h.N.attn.bias` as BOOL or U8: the
    folder loads (the spec ignores those names); a wanted tensor of such a type is one clear error."""
    cfg, spec, model = _model("tiny_a")
    folder = str(tmp_path / "m")
    E.write_random_model(folder, cfg, seed=3)
    path = os.path.join(folder, "model.safetensors")
    header, base = read_header(path)
    data = open(path, "rb").read()[base:]
    n = cfg.n_positions
    header["h.0.attn.bias"] = {"dtype": "BOOL", "shape": [1, 1, n, n], "data_offsets": [len(data), len(data) + n * n]}
    raw = json.dumps(header).encode()
    raw += b" " * (-len(raw) % 8)
    open(path, "wb").write(struct.pack("<Q", len(raw)) + raw + data + b"\1" * (n * n))
    t = load_checked(folder, model.weight_specs(), spec.ignored_tensors, spec.strip_prefixes)
    assert "h.0.attn.bias" not in t and "wte.weight" in t
    header["ln_f.bias"]["dtype"] = "U8"          # a wanted tensor in a type that is not read
    raw = json.dumps(header).encode()
    raw += b" " * (-len(raw) % 8)
    open(path, "wb").write(struct.pack("<Q", len(raw)) + raw + data + b"\1" * (n * n))
    with pytest.raises(WeightError, match="ln_f.bias is stored as U8"):
        load_checked(folder, model.weight_specs(), spec.ignored_tensors, spec.strip_prefixes)


def test_integer_where_float_is_wanted():
    _, spec, model = _model()
    tensors = random_tensors(model.weight_specs(), 0)
    tensors["ln_f.bias"] = torch.zeros(64, dtype=torch.int32)
    with pytest.raises(WeightError, match="wrong type: ln_f.bias"):
        check_tensors("here", tensors, model.weight_specs())


def test_random_model_folder(tmp_path):
    cfg, spec, model = _model("tiny_b")
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    E.write_random_model(a, cfg, seed=5)
    E.write_random_model(b, cfg, seed=5)
    assert open(os.path.join(a, "model.safetensors"), "rb").read() == open(os.path.join(b, "model.safetensors"), "rb").read()
    assert E.load_config(a) == cfg
    t = load_checked(a, model.weight_specs(), spec.ignored_tensors)
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    other = random_tensors(model.weight_specs(), 6)
    assert not torch.equal(other["wte.weight"], t["wte.weight"])
    # distributions: matrices N(0, 0.02), output projections 0.02/sqrt(2L), biases N(0, 0.01), gains 1 + N(0, 0.02)
    big = random_tensors(model.weight_specs(), 1, torch.float32)
    assert abs(big["wte.weight"].std().item() - 0.02) < 1e-3
    assert abs(big["h.0.mlp.c_proj.weight"].std().item() - 0.02 / (2 * cfg.n_layer) ** 0.5) < 1e-3
    assert abs(big["h.0.attn.c_attn.bias"].std().item() - 0.01) < 2e-3
    assert abs(big["h.1.ln_1.weight"].mean().item() - 1.0) < 1e-2
    # a tensor's values do not depend on the rest of the model
    cfg2 = E.GPT2Config.from_dict({**TINY["tiny_b"], "n_layer": 1})
    model2 = DecoderModel(get_architecture(cfg2.architecture).build_spec(cfg2))
    small = random_tensors(model2.weight_specs(), 1, torch.float32)
    assert torch.equal(small["h.0.attn.c_attn.weight"], big["h.0.attn.c_attn.weight"])


def test_float32_folder_stays_float32(tmp_path):
    cfg, spec, model = _model("tiny_a")
    E.write_random_model(str(tmp_path), cfg, 0, torch.float32)
    t = load_checked(str(tmp_path), model.weight_specs(), spec.ignored_tensors)
    assert all(v.dtype == torch.float32 for v in t.values())
