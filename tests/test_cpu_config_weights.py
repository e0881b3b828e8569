"""Configuration, registry, safetensors and weight errors (no device needed)."""
import json
import os
import struct

import pytest
import torch

from tests import configs, helpers

from cpmcu_b200.config import ConfigError, MiniCPMConfig
from cpmcu_b200.models.model import Model
from cpmcu_b200.parts.base import WeightSpec
from cpmcu_b200.registry import architecture, known_architectures, load_config
from cpmcu_b200.weights import SafetensorsError, SafetensorsFile, WeightError, check_and_place, save_file
from cpmcu_b200.weights.loader import load_checkpoint


def test_config_fields_and_derived_scales():
    c = MiniCPMConfig.from_dict(configs.tiny_a())
    assert (c.num_hidden_layers, c.hidden_size, c.head_dim, c.group_size) == (2, 64, 16, 2)
    assert c.residual_scale == pytest.approx(1.4 / 2 ** 0.5)
    assert c.logit_scale == pytest.approx(0.25) and c.scale_emb == 12
    assert c.eos_token_ids == [2] and c.rope_scaling is None and c.sparse_config is None
    b = MiniCPMConfig.from_dict(configs.tiny_b())
    assert b.rope_scaling.rope_type == "longrope" and len(b.rope_scaling.long_factor) == 16
    assert b.sparse_config.block_size == 16 and b.eos_token_ids == [1, 7]
    c3 = MiniCPMConfig.from_dict(configs.tiny_c())          # no scale keys: all scales are 1
    assert c3.residual_scale == 1.0 and c3.logit_scale == 1.0 and c3.scale_emb == 1.0
    assert MiniCPMConfig.from_dict(c.to_dict()) == c and MiniCPMConfig.from_dict(b.to_dict()) == b


def test_config_errors_are_collected():
    bad = configs.tiny_b()
    del bad["vocab_size"]
    bad["num_key_value_heads"] = 3
    bad["rope_scaling"]["long_factor"] = [1.0] * 5
    bad["sparse_config"]["kernel_stride"] = 3
    with pytest.raises(ConfigError) as e:
        MiniCPMConfig.from_dict(bad)
    msg = str(e.value)
    for piece in ("vocab_size", "num_key_value_heads", "long_factor", "kernel_stride"):
        assert piece in msg
    with pytest.raises(ConfigError, match="unknown rope_type"):
        c = configs.tiny_b()
        c["rope_scaling"]["rope_type"] = "yarn"
        MiniCPMConfig.from_dict(c)


def test_registry(tmp_path):
    assert "MiniCPMForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="known:"):
        architecture("LlamaForCausalLM")
    folder = helpers.make_folder(configs.tiny_a(), str(tmp_path / "m"), 0, "float32")
    arch, cfg = load_config(folder)
    assert arch.name == "MiniCPMForCausalLM" and cfg.hidden_size == 64
    spec = arch.model_spec(cfg)
    assert len(spec.layers) == 2 and [e.lane for e in spec.schedule] == [0, 1]
    assert spec.layers[0].mixer.kind == "gqa_attention" and spec.layers[0].mixer.params["position"].kind == "rope"


def test_safetensors_round_trip_and_truncation(tmp_path):
    from safetensors.torch import load_file, save_file as ref_save

    t = {"a.weight": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2)}
    path = str(tmp_path / "x.safetensors")
    save_file(t, path)
    theirs = load_file(path)                                     # our writer, their reader
    for k in t:
        assert torch.equal(theirs[k], t[k])
    ref_save(t, str(tmp_path / "y.safetensors"))                 # their writer, our reader
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))
    for k in t:
        assert torch.equal(f.tensor(k), t[k])
    with open(path, "rb") as fh:
        data = fh.read()
    with open(str(tmp_path / "cut.safetensors"), "wb") as fh:
        fh.write(data[:-9])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(tmp_path / "cut.safetensors"))


def _specs(cfgd):
    arch = architecture("MiniCPMForCausalLM")
    return Model(arch.model_spec(arch.config_class.from_dict(cfgd)), None).weight_specs()


def test_weight_names_and_dtypes(tmp_path):
    specs = _specs(configs.tiny_b())
    assert specs["model.layers.2.self_attn.k_proj.weight"].shape == (32, 128)
    assert specs["model.layers.0.mlp.down_proj.weight"].shape == (128, 320)
    assert specs["lm_head.weight"].shape == (1000, 128) and specs["model.norm.weight"].role == "vector"
    assert "lm_head.weight" not in _specs(configs.tiny_a())      # tied
    folder = helpers.make_folder(configs.tiny_b(), str(tmp_path / "b"), 1, "bfloat16")
    # a norm weight stored in 32-bit stays so; matrices take the compute dtype
    from safetensors.torch import load_file, save_file as ref_save
    w = {k: v.clone() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    w["model.norm.weight"] = w["model.norm.weight"].float()
    ref_save(w, os.path.join(folder, "model.safetensors"))
    out = load_checkpoint(folder, specs, torch.bfloat16, "cpu")
    assert out["model.norm.weight"].dtype == torch.float32
    assert out["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16
    assert out["model.embed_tokens.weight"].dtype == torch.bfloat16
    out32 = load_checkpoint(folder, specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in out32.values())


def test_weight_error_lists_everything(tmp_path):
    from safetensors.torch import load_file, save_file as ref_save

    specs = _specs(configs.tiny_a())
    folder = helpers.make_folder(configs.tiny_a(), str(tmp_path / "a"), 0, "float32")
    path = os.path.join(folder, "model.safetensors")
    w = {k: v.clone() for k, v in load_file(path).items()}
    del w["model.layers.1.mlp.up_proj.weight"]
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)        # tolerated
    w["model.extra.bias"] = torch.zeros(3)
    ref_save(w, path)
    with pytest.raises(WeightError) as e:
        load_checkpoint(folder, specs, torch.float32, "cpu", ignore=architecture("MiniCPMForCausalLM").ignore_tensor)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.extra.bias"]
    assert len(err.wrong_shape) == 1 and "(64, 32)" in err.wrong_shape[0] and "(64, 64)" in err.wrong_shape[0]
    for piece in ("missing tensors", "unexpected tensors", "wrong shapes"):
        assert piece in str(err)


def test_fused_checkpoint_tensors_are_split(tmp_path):
    from safetensors.torch import load_file, save_file as ref_save

    arch = architecture("MiniCPMForCausalLM")
    cfg = arch.config_class.from_dict(configs.tiny_a())
    specs = _specs(configs.tiny_a())
    folder = helpers.make_folder(configs.tiny_a(), str(tmp_path / "a"), 0, "float32")
    path = os.path.join(folder, "model.safetensors")
    w = {k: v.clone() for k, v in load_file(path).items()}
    plain_w = dict(w)
    for i in range(2):
        p = f"model.layers.{i}."
        w[p + "self_attn.qkv_proj.weight"] = torch.cat([w.pop(p + f"self_attn.{n}_proj.weight") for n in "qkv"])
        w[p + "mlp.gate_up_proj.weight"] = torch.cat([w.pop(p + "mlp.gate_proj.weight"), w.pop(p + "mlp.up_proj.weight")])
    ref_save(w, path)
    out = load_checkpoint(folder, specs, torch.float32, "cpu", adapt=lambda n, t: arch.adapt_tensor(cfg, n, t))
    for k, v in plain_w.items():
        assert torch.equal(out[k], v)


def test_random_folder_is_reproducible(tmp_path):
    a = helpers.make_folder(configs.tiny_a(), str(tmp_path / "1"), 3, "bfloat16")
    b = helpers.make_folder(configs.tiny_a(), str(tmp_path / "2"), 3, "bfloat16")
    c = helpers.make_folder(configs.tiny_a(), str(tmp_path / "3"), 4, "bfloat16")
    read = lambda d: open(os.path.join(d, "model.safetensors"), "rb").read()
    assert read(a) == read(b) and read(a) != read(c)
    cfg, w = helpers.read_folder(a)
    assert cfg["architectures"] == ["MiniCPMForCausalLM"] and cfg["torch_dtype"] == "bfloat16"
    assert abs(float(w["model.norm.weight"].float().mean()) - 1.0) < 0.02
    assert abs(float(w["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
