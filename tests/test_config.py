"""Configuration and registry (mirrors crates/rllm-model/src/hf_config.rs:128-239)."""
import json
import os

import pytest

from conftest import TINY_A, TINY_B
from rllm_b200.config import (ConfigError, EngineArgs, LlamaConfig, load_model_description,
                              normalize_architecture, resolve_architecture)


def test_defaults_follow_the_reference():
    cfg = LlamaConfig.from_json({"architectures": ["LlamaForCausalLM"]})
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads) == (32000, 4096, 32, 32)
    assert cfg.num_key_value_heads == 32 and cfg.head_dim == 128 and cfg.intermediate_size == 4 * 4096
    assert cfg.max_position_embeddings == 4096 and cfg.rope_theta == 10000.0
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_scaling is None and not cfg.tie_word_embeddings


def test_every_key_is_read():
    a, b = LlamaConfig.from_json(TINY_A), LlamaConfig.from_json(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size) == (2, 64, 4, 2, 16, 176, 256)
    assert a.rms_norm_eps == 1e-5 and a.tie_word_embeddings and a.rope_scaling is None
    assert a.eos_token_ids == (2,) and a.bos_token_id == 1
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim,
            b.intermediate_size, b.vocab_size) == (3, 96, 3, 1, 32, 264, 389)
    assert b.rope_theta == 500000.0 and b.rms_norm_eps == 1e-6 and not b.tie_word_embeddings
    assert b.rope_scaling.factor == 4.0 and b.rope_scaling.original_max_position_embeddings == 32
    assert b.eos_token_ids == (3, 7)


def test_json_round_trip():
    for raw in (TINY_A, TINY_B):
        cfg = LlamaConfig.from_json(raw)
        assert LlamaConfig.from_json(cfg.to_json()) == cfg


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": 0}, "hidden_size"),
    ({"num_attention_heads": 32, "num_key_value_heads": 7, "hidden_size": 4096, "head_dim": 128}, "divisible"),
    ({"num_key_value_heads": 8}, "num_key_value_heads"),
    ({"head_dim": 32}, "head_dim"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "lacks"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"vocab_size": "many"}, "vocab_size"),
])
def test_bad_configs_are_refused(patch, word):
    raw = dict(TINY_A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_json(raw)


def test_architecture_names():
    for name in ("llama", "LlamaModel", "LLaMAForCausalLM", "LlamaForCausalLM"):
        assert normalize_architecture(name) == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="unsupported architecture.*known.*LlamaForCausalLM"):
        resolve_architecture({"architectures": ["GPT2LMHeadModel"]})
    with pytest.raises(ConfigError, match="unknown"):
        resolve_architecture({})


def test_model_description_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    cfg, spec = load_model_description(str(tmp_path))
    assert len(spec.layers) == 3 and [r.layer for r in spec.order] == [0, 1, 2]
    assert spec.layers[0].mixer["num_kv_heads"] == 1 and spec.head["tied_to"] is None
    with pytest.raises(ConfigError, match="no config.json"):
        load_model_description(str(tmp_path / "nothing"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_model_description(str(tmp_path))


def test_engine_args():
    EngineArgs().validate()
    assert EngineArgs().max_num_seqs == 256 and EngineArgs().max_num_batched_tokens == 4096
    assert EngineArgs().gpu_memory_utilization == 0.9
    with pytest.raises(ConfigError, match="0.01"):
        EngineArgs(gpu_memory_utilization=1.5).validate()
    assert EngineArgs().scheduling_policy == "fcfs" and EngineArgs().step_row_multiple == 128
    EngineArgs(scheduling_policy="priority", step_row_multiple=0).validate()
    for bad in (dict(scheduling_policy="lifo"), dict(step_row_multiple=-1), dict(block_size=0), dict(max_num_seqs=0)):
        with pytest.raises(ConfigError):
            EngineArgs(**bad).validate()
    assert EngineArgs(dtype="auto").run_dtype("float32") == "float32"
    assert EngineArgs(dtype="auto").run_dtype("float16") == "bfloat16"
    assert EngineArgs(dtype="bf16").run_dtype("float32") == "bfloat16"
    assert EngineArgs(dtype="fp32").run_dtype("bfloat16") == "float32"
    with pytest.raises(ConfigError):
        EngineArgs(dtype="fp16").run_dtype("float16")
    with pytest.raises(ConfigError):
        EngineArgs(dtype="int8").validate()
