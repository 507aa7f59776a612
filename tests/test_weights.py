"""Safetensors reading, checkpoint errors and the random-weights mode (no GPU)."""
import json

import pytest
import torch

import plain_llama
from conftest import TINY_A, TINY_B
from pytriton_llama_b200.config import LlamaConfig
from pytriton_llama_b200.models.decoder import DecoderModel
from pytriton_llama_b200.models.llama import llama_spec
from pytriton_llama_b200.parts.base import Runtime
from pytriton_llama_b200.weights import (WeightError, check_tensors, read_folder, write_file,
                                         write_random_model)


def _expected(cfg_dict):
    model = DecoderModel(llama_spec(LlamaConfig.from_dict(cfg_dict)), Runtime(torch.device("cpu"), torch.float32, None))
    return model.expected_tensors()


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY_B, seed=5, dtype=torch.bfloat16)
    cfg = json.loads((folder / "config.json").read_text())
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["num_hidden_layers"] == 3
    tensors = read_folder(folder)
    check_tensors(_expected(TINY_B), tensors)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    assert tensors["model.layers.2.mlp.down_proj.weight"].shape == (192, 320)
    assert "lm_head.weight" in tensors                      # untied
    w = tensors["model.layers.0.self_attn.q_proj.weight"].float()
    assert 0.015 < w.std() < 0.025                          # N(0, 0.02)
    # the package's writer and the test oracle's own reader agree byte for byte
    _, again = plain_llama.load_model_folder(folder, dtype=torch.bfloat16)
    assert all(torch.equal(again[k], tensors[k]) for k in tensors)


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a = read_folder(write_random_model(tmp_path / "a", TINY_A, seed=1, dtype=torch.float32, norm_init="ones_jitter"))
    b = read_folder(write_random_model(tmp_path / "b", TINY_A, seed=1, dtype=torch.float32, norm_init="ones_jitter"))
    c = read_folder(write_random_model(tmp_path / "c", TINY_A, seed=2, dtype=torch.float32, norm_init="ones_jitter"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a                        # tied
    assert (a["model.norm.weight"] - 1).abs().max() > 0     # 1 + N(0, 0.01)
    assert (a["model.norm.weight"] - 1).abs().max() < 0.1


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY_A, seed=1, dtype=torch.float32)
    tensors = dict(read_folder(folder))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 64)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    with pytest.raises(WeightError) as e:
        check_tensors(_expected(TINY_A), tensors)
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "rotary_emb.inv_freq" in msg
    assert "k_proj.weight: file has [32, 64], model wants [16, 64]" in msg
    assert e.value.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.value.wrong_type == ["model.layers.0.input_layernorm.weight (torch.int32)"]


def test_stored_element_types_are_kept(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    write_file(tmp_path / "t.safetensors", tensors)
    from pytriton_llama_b200.weights import read_file
    back = read_file(tmp_path / "t.safetensors")
    assert back["a"].dtype == torch.bfloat16 and back["b"].dtype == torch.float32 and back["c"].dtype == torch.int32
    assert all(torch.equal(back[k], tensors[k]) for k in tensors)


def test_norm_weights_stay_32_bit_and_matrices_take_the_compute_type(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY_A, seed=1, dtype=torch.float32, norm_init="ones_jitter")
    model = DecoderModel(llama_spec(LlamaConfig.from_dict(TINY_A)), Runtime(torch.device("cpu"), torch.bfloat16, None))
    tensors = read_folder(folder)
    model.load(tensors)
    blk = model.blocks[0]
    assert blk.norm1.weight.dtype == torch.float32
    assert torch.equal(blk.norm1.weight, tensors["model.layers.0.input_layernorm.weight"])
    assert blk.mixer.w_qkv.dtype == torch.bfloat16 and blk.mixer.w_qkv.shape == ((4 + 2) * 16, 64)
    # fused layout: q rows, then k, then v -- the k|v part is lite_llama's kv_proj_weight
    assert torch.equal(blk.mixer.w_qkv[64:80].float(), tensors["model.layers.0.self_attn.k_proj.weight"].bfloat16().float())
    assert blk.ffn.w_gate_up.shape == (256, 64)
    assert model.lm_head is model.embedding                 # tied: one tensor


def test_missing_file_is_reported(tmp_path):
    with pytest.raises(FileNotFoundError):
        read_folder(tmp_path)
