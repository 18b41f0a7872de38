"""The runtime's switches in one struct, with the EMBER_* variables as overrides (no GPU)."""
import dataclasses

import pytest

import ember_cpp_b200 as E
from ember_cpp_b200.options import OptionError, RuntimeOptions


def test_defaults_and_variable_names():
    o = RuntimeOptions()
    assert o.dtype == "bfloat16" and o.cuda_graphs and o.gemm == "lt" and o.lt_tune and not o.deterministic
    assert RuntimeOptions.variable("decode_mma") == "EMBER_DECODE_MMA"
    assert {f.name for f in dataclasses.fields(RuntimeOptions)} >= {
        "dtype", "max_tokens", "max_slots", "cuda_graphs", "prompt_graphs", "deterministic", "gemm", "lt_tune", "linear_stream", "attention",
        "decode_mma", "decode_cluster", "decode_bulk", "pdl", "cache_ahead", "warm", "op_timing", "nvtx"}


def test_variables_override_the_given_options():
    base = RuntimeOptions(dtype="float32", max_tokens=512)
    o = RuntimeOptions.from_env(base, {"EMBER_GEMM": "tc", "EMBER_DECODE_MMA": "0", "EMBER_MAX_TOKENS": "2048", "OTHER": "x"})
    assert o.dtype == "float32" and o.gemm == "tc" and not o.decode_mma and o.max_tokens == 2048
    assert RuntimeOptions.from_env(None, {}) == RuntimeOptions()


def test_deterministic_switches_the_timed_choice_off():
    assert not RuntimeOptions(deterministic=True).lt_tune
    assert not RuntimeOptions.from_env(None, {"EMBER_DETERMINISTIC": "1", "EMBER_LT_TUNE": "1"}).lt_tune


@pytest.mark.parametrize("env, word", [({"EMBER_GEMM": "cutlass"}, "gemm"), ({"EMBER_PDL": "maybe"}, "EMBER_PDL"),
                                        ({"EMBER_MAX_TOKENS": "many"}, "EMBER_MAX_TOKENS"), ({"EMBER_DTYPE": "fp8"}, "dtype"),
                                        ({"EMBER_ATTENTION": "flash"}, "attention")])
def test_bad_values_name_the_switch(env, word):
    with pytest.raises(OptionError, match=word):
        RuntimeOptions.from_env(None, env)


def test_arguments_given_in_their_own_right_win():
    o = E.Engine._options(RuntimeOptions(dtype="float32", max_tokens=512), None, 1024, None, False)
    assert o.dtype == "float32" and o.max_tokens == 1024 and o.cuda_graphs is False


def test_a_model_the_bfloat16_kernels_cannot_run_is_refused_by_key():
    cfg = E.GPT2Config.from_dict(dict(vocab_size=10, n_positions=8, n_embd=36, n_layer=1, n_head=3, n_inner=100))
    cfg.check_dtype("float32")                                   # head size 12: the 32-bit path takes it
    with pytest.raises(E.ConfigError, match="n_embd / n_head"):
        cfg.check_dtype("bfloat16")
    cfg = E.GPT2Config.from_dict(dict(vocab_size=10, n_positions=8, n_embd=64, n_layer=1, n_head=4, n_inner=100))
    with pytest.raises(E.ConfigError, match="n_inner"):
        cfg.check_dtype("bfloat16")
    with pytest.raises(E.ConfigError, match="head sizes up to 256"):
        E.GPT2Config.from_dict(dict(vocab_size=10, n_positions=8, n_embd=1024, n_layer=1, n_head=2)).check_dtype("float32")
