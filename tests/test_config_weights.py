"""Configuration reading, the registry, the strict weight check and the random-weights mode."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers
from qwen_engine_b200.config import ConfigError, EngineConfig, Qwen3Config, preset_config_dict
from qwen_engine_b200.registry import (ARCHITECTURES, build_model, config_from_dict, config_from_folder,
                                       register_architecture)
from qwen_engine_b200.weights import (RandomSource, SafetensorsSource, WeightError, check_against_manifest,
                                      write_model_folder)


def test_every_size_comes_from_config_json(tmp_path):
    raw = dict(helpers.TINY["tiny-b"]["cfg"])
    (tmp_path / "config.json").write_text(json.dumps(raw))
    cfg = config_from_folder(str(tmp_path))
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (3, 80, 4, 1, 32, 224, 389)
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False
    assert cfg.q_width == 128 != cfg.hidden_size
    assert abs(cfg.attention_scale - 32 ** -0.5) < 1e-12


def test_rope_theta_from_rope_parameters_first():
    raw = dict(preset_config_dict("tiny-a"), rope_theta=5.0, rope_parameters={"rope_theta": 777.0})
    assert config_from_dict(raw).rope_theta == 777.0


def test_head_dim_falls_back_to_quotient():
    raw = dict(preset_config_dict("tiny-a"))
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 64 // 4


def test_defaults_are_the_reference_defaults():
    cfg = config_from_dict({"architectures": ["Qwen3ForCausalLM"]})
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.intermediate_size, cfg.vocab_size, cfg.max_position_embeddings) == (28, 1024, 16, 8, 3072, 151936, 40960)
    assert cfg.head_dim == 1024 // 16        # absent: hidden / heads, as the reference's constructor (model.py:320)
    assert cfg.tie_word_embeddings and cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-6


@pytest.mark.parametrize("bad,msg", [
    ({"architectures": ["NoSuchModel"]}, "not registered"),
    ({}, "architectures"),
    ({"architectures": ["Qwen3ForCausalLM"], "num_attention_heads": 6, "num_key_value_heads": 4}, "multiple"),
    ({"architectures": ["Qwen3ForCausalLM"], "head_dim": 15}, "even"),
    ({"architectures": ["Qwen3ForCausalLM"], "attention_bias": True}, "attention_bias"),
    ({"architectures": ["Qwen3ForCausalLM"], "hidden_act": "gelu"}, "hidden_act"),
    ({"architectures": ["Qwen3ForCausalLM"], "rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"architectures": ["Qwen3ForCausalLM"], "use_sliding_window": True}, "sliding_window"),
    ({"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 0}, "num_hidden_layers"),
    ({"architectures": ["Qwen3ForCausalLM"], "vocab_size": "big"}, "vocab_size"),
])
def test_configs_that_are_refused(bad, msg):
    with pytest.raises(ConfigError, match=msg):
        config_from_dict(bad)


def test_missing_config_json(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        config_from_folder(str(tmp_path))


def test_registry_takes_another_architecture():
    from qwen_engine_b200.models.qwen3 import qwen3_layout

    class OtherConfig(Qwen3Config):
        architecture = "OtherForCausalLM"

    register_architecture("OtherForCausalLM", OtherConfig, qwen3_layout)
    try:
        cfg = config_from_dict(dict(preset_config_dict("tiny-a"), architectures=["OtherForCausalLM"]))
        assert type(cfg) is OtherConfig and cfg.to_dict()["architectures"] == ["OtherForCausalLM"]
        assert len(build_model(cfg).blocks) == 2
    finally:
        del ARCHITECTURES["OtherForCausalLM"]


def test_engine_config_checks():
    assert EngineConfig(max_num_seqs=4, max_model_len=256, block_size=16).resolved_num_blocks() == 64
    assert EngineConfig(dtype="fp32").dtype == torch.float32
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(block_size=0)


# ---- weights ------------------------------------------------------------------------------------

def test_manifest_names_are_the_checkpoint_names():
    cfg = config_from_dict(preset_config_dict("tiny-b"))
    names = {s.name for s in build_model(cfg).weight_manifest()}
    per_layer = {"input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                 "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                 "self_attn.q_norm.weight", "self_attn.k_norm.weight", "mlp.gate_proj.weight",
                 "mlp.up_proj.weight", "mlp.down_proj.weight"}
    want = {f"model.layers.{i}.{n}" for i in range(3) for n in per_layer}
    want |= {"model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"}
    assert names == want


def test_random_folder_round_trip(tmp_path, cpu_ops):
    cfg = config_from_dict(preset_config_dict("tiny-b"))
    d = write_model_folder(cfg, str(tmp_path / "m"), seed=1, std=0.05, norm_std=0.2)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert config_from_folder(d) == cfg
    stored = load_file(os.path.join(d, "model.safetensors"))
    assert all(t.dtype == torch.bfloat16 for t in stored.values())
    assert "lm_head.weight" in stored                                   # untied
    # seeded by (seed, name): the same tensor again, whatever else is made
    src = RandomSource(build_model(cfg).weight_manifest(), 1, 0.05, 0.2)
    assert torch.equal(src.get("model.layers.2.mlp.up_proj.weight"), stored["model.layers.2.mlp.up_proj.weight"])
    w = stored["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(w.std()) - 0.05) < 0.005
    nw = stored["model.norm.weight"].float()
    assert abs(float(nw.mean()) - 1.0) < 0.15
    # loading keeps matrices in the compute dtype and norm scales in float32
    model = build_model(cfg)
    model.load_weights(SafetensorsSource(d), torch.bfloat16, "cpu")
    assert model.embed.dtype == torch.bfloat16 and model.head is not model.embed
    assert model.final_norm.weight.dtype == torch.float32
    assert model.blocks[0].mixer.w_qkv.shape == ((4 + 2) * 32, 80)
    # a float32 checkpoint stays float32 in the 32-bit path
    d32 = write_model_folder(cfg, str(tmp_path / "m32"), seed=1, std=0.05, norm_std=0.2, store_dtype=torch.float32)
    model.load_weights(SafetensorsSource(d32), torch.float32, "cpu")
    assert model.embed.dtype == torch.float32


def test_tied_model_has_no_head_tensor_and_shares_storage(tmp_path, cpu_ops):
    cfg = config_from_dict(preset_config_dict("tiny-a"))
    d = write_model_folder(cfg, str(tmp_path / "m"), seed=0)
    assert "lm_head.weight" not in load_file(os.path.join(d, "model.safetensors"))
    model = build_model(cfg)
    model.load_weights(SafetensorsSource(d), torch.float32, "cpu")
    assert model.head is model.embed


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(preset_config_dict("tiny-b"))
    d = write_model_folder(cfg, str(tmp_path / "m"), seed=1)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.down_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(4)
    t["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 80, dtype=torch.bfloat16)
    save_file(t, path)
    model = build_model(cfg)
    with pytest.raises(WeightError) as e:
        model.load_weights(SafetensorsSource(d), torch.float32, "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.down_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "rotary.inv_freq" in msg
    assert "wrong shapes (1)" in msg and "k_proj.weight: stored [64, 80], model needs [32, 80]" in msg
    assert model.embed is None, "nothing is loaded from a checkpoint that does not fit"


def test_no_safetensors_file(tmp_path):
    with pytest.raises(WeightError, match="no .safetensors"):
        SafetensorsSource(str(tmp_path))


def test_tied_checkpoint_may_carry_a_head(tmp_path):
    cfg = config_from_dict(preset_config_dict("tiny-a"))
    d = write_model_folder(cfg, str(tmp_path / "m"), seed=0)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, path)
    check_against_manifest(SafetensorsSource(d), build_model(cfg).weight_manifest())
    # loading it works; the stored head is not used, and the user is told so
    model = build_model(cfg)
    with pytest.warns(UserWarning, match="lm_head.weight"):
        model.load_weights(SafetensorsSource(d), torch.float32, "cpu")
    assert model.head is model.embed


def test_every_end_of_sequence_id_is_kept():
    cfg = config_from_dict(dict(preset_config_dict("tiny-a"), eos_token_id=[7, 9]))
    assert cfg.eos_token_id == 7 and cfg.eos_token_ids == (7, 9)
    assert cfg.to_dict()["eos_token_id"] == [7, 9] and "eos_token_ids" not in cfg.to_dict()
    assert config_from_dict(cfg.to_dict()) == cfg
    one = config_from_dict(dict(preset_config_dict("tiny-a"), eos_token_id=5))
    assert one.eos_token_ids == (5,) and one.to_dict()["eos_token_id"] == 5
    assert config_from_dict(preset_config_dict("tiny-a")).eos_token_ids == ()
