"""Configuration, registry, weight loading errors, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

from conftest import TINY_A, TINY_B
from vapi_b200.config import ConfigError, registered_architectures, resolve_architecture
from vapi_b200.models.lfm2 import Lfm2Config
from vapi_b200.config.runtime import RuntimeConfig, RuntimeConfigError
from vapi_b200.weights import WeightError, load_tensors, write_random_model


def test_tiny_b_feed_forward_rule_and_defaults():
    c = Lfm2Config.from_json(TINY_B)
    # 384 -> 2*384//3 = 256 -> *1.5 = 384 -> rounded up to a multiple of 64 = 384
    assert c.intermediate_size == 384
    assert c.rope_theta == 1e6 and c.conv_L_cache == 4 and c.conv_bias and not c.tie_word_embeddings
    assert c.eos_token_ids == (3, 5) and c.head_dim == 32
    a = Lfm2Config.from_json(TINY_A)
    assert a.intermediate_size == 192 and a.eos_token_ids == (7,) and a.tie_word_embeddings


def test_benchmark_sizes_follow_from_the_rule():
    v = dict(vocab_size=65536, hidden_size=2048, intermediate_size=12288, block_auto_adjust_ff_dim=True,
             block_ffn_dim_multiplier=1.0, block_multiple_of=256, num_hidden_layers=16,
             num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=128000)
    c = Lfm2Config.from_json(v)
    assert c.intermediate_size == 8192 and c.head_dim == 64
    assert c.layer_types == ("conv",) * 16 and c.rope_theta == 1e6 and c.norm_eps == 1e-5 and c.conv_L_cache == 3
    v2 = dict(v, hidden_size=1536, intermediate_size=10240, num_attention_heads=24)
    assert Lfm2Config.from_json(v2).intermediate_size == 6912


def test_config_errors():
    bad = dict(TINY_A)
    del bad["vocab_size"]
    with pytest.raises(ConfigError, match="missing integer `vocab_size`"):
        Lfm2Config.from_json(bad)
    with pytest.raises(ConfigError, match="layer_types does not cover every layer"):
        Lfm2Config.from_json(dict(TINY_A, layer_types=["conv"]))
    with pytest.raises(ConfigError, match="not one of"):
        Lfm2Config.from_json(dict(TINY_A, layer_types=["conv", "sliding", "conv", "conv"]))
    with pytest.raises(ConfigError, match="multiple of"):
        Lfm2Config.from_json(dict(TINY_A, num_key_value_heads=3))


def test_registry_picks_by_architecture_then_model_type():
    assert "Lfm2ForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["Lfm2ForCausalLM"]}).name == "Lfm2ForCausalLM"
    assert resolve_architecture({"model_type": "lfm2"}).name == "Lfm2ForCausalLM"
    with pytest.raises(ConfigError, match="not supported; registered"):
        resolve_architecture({"architectures": ["NopeForCausalLM"], "model_type": "nope"})


def test_config_round_trip():
    c = Lfm2Config.from_json(TINY_B)
    assert Lfm2Config.from_json(c.to_json()) == c


def test_random_model_folder_loads_back(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, seed=3, dtype=torch.bfloat16)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    arch = resolve_architecture(json.load(open(os.path.join(d, "config.json"))))
    plan = arch.plan(arch.parse(TINY_B))
    t = load_tensors(d, plan.tensor_specs(), torch.bfloat16, "cpu")
    assert t["model.layers.2.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert t["model.layers.0.operator_norm.weight"].dtype == torch.float32       # vectors are float32
    assert t["model.layers.0.conv.conv.weight"].shape == (96, 1, 4)
    assert "lm_head.weight" in t
    t32 = load_tensors(d, plan.tensor_specs(), torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    # same seed, same values; another seed, other values
    d2 = write_random_model(str(tmp_path / "m2"), TINY_B, seed=3, dtype=torch.bfloat16)
    t2 = load_tensors(d2, plan.tensor_specs(), torch.bfloat16, "cpu")
    assert all(torch.equal(t[k], t2[k]) for k in t)
    d3 = write_random_model(str(tmp_path / "m3"), TINY_B, seed=4, dtype=torch.bfloat16)
    t3 = load_tensors(d3, plan.tensor_specs(), torch.bfloat16, "cpu")
    assert not torch.equal(t["lm_head.weight"], t3["lm_head.weight"])


def test_float32_stored_matrices_stay_float32(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=1, dtype=torch.float32)
    arch = resolve_architecture(TINY_A)
    plan = arch.plan(arch.parse(TINY_A))
    t = load_tensors(d, plan.tensor_specs(), torch.bfloat16, "cpu")
    assert t["model.embed_tokens.weight"].dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    from safetensors.torch import load_file, save_file
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=1)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.self_attn.k_layernorm.weight"]
    del t["model.layers.0.conv.in_proj.weight"]
    t["model.layers.9.bogus.weight"] = torch.zeros(3)
    t["model.layers.2.feed_forward.w2.weight"] = torch.zeros(64, 191)
    save_file(t, path)
    arch = resolve_architecture(TINY_A)
    plan = arch.plan(arch.parse(TINY_A))
    with pytest.raises(WeightError) as e:
        load_tensors(d, plan.tensor_specs(), torch.float32, "cpu")
    msg = str(e.value)
    assert "model.layers.1.self_attn.k_layernorm.weight" in msg and "model.layers.0.conv.in_proj.weight" in msg
    assert "model.layers.9.bogus.weight" in msg
    assert "model.layers.2.feed_forward.w2.weight: file has [64, 191], model wants [64, 192]" in msg
    assert e.value.missing and e.value.unexpected and e.value.wrong_shape


def test_untied_head_falls_back_to_the_embedding_when_absent(tmp_path, plain_kernels):
    from safetensors.torch import load_file, save_file
    from vapi_b200.engine.runner import ModelRunner
    d = write_random_model(str(tmp_path / "m"), TINY_B, seed=1)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["lm_head.weight"]
    save_file(t, path)
    r = ModelRunner.from_dir(d, dtype="float32", device="cpu", num_pages=4, max_requests=2, page_size=16)
    assert r.plan.head.weight.data_ptr() == r.plan.embedding.table.data_ptr()


def test_no_weights_file(tmp_path):
    os.makedirs(tmp_path / "m")
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_tensors(str(tmp_path / "m"), [], torch.float32, "cpu")


def test_runtime_config_toml(tmp_path):
    p = tmp_path / "vapi.toml"
    p.write_text('[model]\npath = "/x"\ndtype = "f32"\nnum_blocks = 12\n[worker]\nprefill_chunk_tokens = 16\n[cache]\nwatermark = 0.0\n')
    c = RuntimeConfig.load(str(p))
    assert c.model.path == "/x" and c.resolved_dtype() == "float32" and c.model.num_blocks == 12
    assert c.worker.prefill_chunk_tokens == 16 and c.worker.max_concurrent_seqs == 64
    p.write_text("[worker]\nbogus = 1\n")
    with pytest.raises(RuntimeConfigError, match="unknown key `bogus`"):
        RuntimeConfig.load(str(p))
    p.write_text("[gateway]\nbind = 1\n")
    with pytest.raises(RuntimeConfigError, match=r"unknown section \[gateway\]"):
        RuntimeConfig.load(str(p))


def test_cli_rejects_unknown_arguments(capsys):
    from vapi_b200.cli import build_parser
    with pytest.raises(SystemExit):
        build_parser().parse_args(["--bogus"])
    assert "--bogus" in capsys.readouterr().err
