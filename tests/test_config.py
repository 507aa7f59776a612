"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from pytriton_llama_b200.config import (ConfigError, EngineConfig, LlamaConfig, known_architectures,
                                        register_architecture, resolve_architecture)
from pytriton_llama_b200.models.llama import llama_spec


def test_reads_config_json_keys():
    cfg = LlamaConfig.from_dict(TINY_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 192, 6, 2)
    assert cfg.head_dim == 32 and cfg.intermediate_size == 320 and cfg.vocab_size == 384
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0 and not cfg.tie_word_embeddings
    assert cfg.rope_scaling.rope_type == "llama3" and cfg.rope_scaling.factor == 8.0
    assert cfg.rope_scaling.original_max_position_embeddings == 64
    assert cfg.eos_token_ids == [382, 383]


def test_defaults_follow_the_file_not_the_code():
    d = dict(TINY_A)
    del d["num_key_value_heads"], d["head_dim"]
    cfg = LlamaConfig.from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads == 4   # absent: as many as query heads
    assert cfg.head_dim == 64 // 4
    d["head_dim"] = 32                                                # present: honoured, hidden != heads * head_dim
    assert LlamaConfig.from_dict(d).head_dim == 32


def test_round_trip_through_json():
    cfg = LlamaConfig.from_dict(TINY_B)
    again = LlamaConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg


@pytest.mark.parametrize("change, word", [
    ({"num_key_value_heads": 4}, "multiple"),
    ({"head_dim": 31}, "even"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "lacks"),
    ({"vocab_size": None}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"partial_rotary_factor": 1.5}, "partial_rotary_factor"),
    ({"partial_rotary_factor": 0.3}, "partial_rotary_factor"),       # 32 * 0.3 = 9: an odd rotary width
])
def test_refuses_what_it_cannot_run(change, word):
    d = dict(TINY_B)
    d.update(change)
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert word in str(e.value)


def test_registry_maps_architecture_to_model():
    assert "LlamaForCausalLM" in known_architectures()
    arch = resolve_architecture(TINY_A)
    spec = arch.spec_from_config(arch.config_from_dict(TINY_A))
    assert spec.architecture == "LlamaForCausalLM" and len(spec.layers) == 2
    assert spec.lm_head is None                                   # tied
    assert llama_spec(LlamaConfig.from_dict(TINY_B)).lm_head == "lm_head.weight"
    with pytest.raises(KeyError) as e:
        resolve_architecture({"architectures": ["MambaForCausalLM"]})
    assert "LlamaForCausalLM" in str(e.value)
    with pytest.raises(KeyError):
        resolve_architecture({})


def test_spec_carries_the_configs_constants():
    spec = llama_spec(LlamaConfig.from_dict(TINY_B))
    blk = spec.layers[1]
    assert blk.parts["norm1"].params["eps"] == 1e-6
    assert blk.parts["mixer"].params == {"hidden": 192, "heads": 6, "kv_heads": 2, "head_dim": 32}
    assert blk.parts["mixer"].parts["position"].params["theta"] == 500000.0
    assert blk.parts["mixer"].parts["position"].params["scaling"]["factor"] == 8.0
    assert blk.parts["ffn"].params == {"hidden": 192, "inter": 320}
    assert blk.parts["mixer"].parts["position"].params["rotary_dim"] == 32
    half = llama_spec(LlamaConfig.from_dict(dict(TINY_B, partial_rotary_factor=0.5)))
    assert half.layers[0].parts["mixer"].parts["position"].params["rotary_dim"] == 16
    assert [(e.layer, e.cache, e.write) for e in spec.run_order] == [(0, 0, True), (1, 1, True), (2, 2, True)]


def test_run_order_is_checked():
    from pytriton_llama_b200.models.spec import RunEntry
    spec = llama_spec(LlamaConfig.from_dict(TINY_A))
    spec.run_order = [RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 1, write=False)]   # a layer twice, reading another's cache
    spec.validate()
    spec.run_order = [RunEntry(0, 5, write=False)]
    with pytest.raises(ValueError):
        spec.validate()
    spec.run_order = [RunEntry(7, 0)]
    with pytest.raises(ValueError):
        spec.validate()


def test_engine_config():
    import torch
    assert EngineConfig(dtype="float32").dtype == torch.float32
    assert EngineConfig(dtype="bf16").dtype == torch.bfloat16
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(page_size=0)


def test_new_architecture_can_be_registered():
    register_architecture("ToyForCausalLM", LlamaConfig.from_dict, llama_spec)
    d = dict(TINY_A, architectures=["ToyForCausalLM"])
    assert resolve_architecture(d).name == "ToyForCausalLM"


def test_chat_prompts():
    """The command line's prompt forms: the Llama 3 chat form renders every turn so far and leaves
    the assistant's header open; the plain form passes lines through; the choice follows the tokenizer."""
    from pytriton_llama_b200.utils import Llama3ChatPrompt, PlainPrompt, prompt_for_tokenizer
    chat = Llama3ChatPrompt(system="Be brief.")
    first = chat.render("Hi")
    assert first == ("<|start_header_id|>system<|end_header_id|>\n\nBe brief.<|eot_id|>"
                     "<|start_header_id|>user<|end_header_id|>\n\nHi<|eot_id|>"
                     "<|start_header_id|>assistant<|end_header_id|>\n\n")
    chat.record(" Hello! ")
    second = chat.render("And now?")
    assert second.startswith(first + "Hello!<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nAnd now?<|eot_id|>")
    assert second.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    chat.reset()
    assert chat.render("Hi") == first
    assert Llama3ChatPrompt().render("x") == "<|start_header_id|>user<|end_header_id|>\n\nx<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n"
    plain = PlainPrompt()
    assert plain.render("as it is") == "as it is"
    plain.record("answer")
    assert plain.render("next") == "next"
    with pytest.raises(RuntimeError):
        Llama3ChatPrompt().record("nothing was asked")

    class Knows:
        unk_token_id = 0

        def convert_tokens_to_ids(self, toks):
            return [128006, 128009]

    class KnowsNot(Knows):
        def convert_tokens_to_ids(self, toks):
            return [0, 0]
    assert isinstance(prompt_for_tokenizer(Knows()), Llama3ChatPrompt)
    assert isinstance(prompt_for_tokenizer(KnowsNot()), PlainPrompt)
    assert isinstance(prompt_for_tokenizer(Knows(), raw=True), PlainPrompt)
    assert isinstance(prompt_for_tokenizer(None), PlainPrompt)
