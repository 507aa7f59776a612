"""The dense GQA Llama decoder (architecture name "LlamaForCausalLM") as a ``ModelSpec``.

Tensor names are those of the checkpoint; lite_llama maps the same names onto its own
(lite_llama/executor/weight_convert.py:193-212).  Every layer is the same pre-norm block with
grouped-query attention, rotary positions and a SwiGLU feed-forward
(lite_llama/models/llama.py:122-162); layers run once each, in order, each with its own cache
entry.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.base import PartSpec
from .spec import ModelSpec, RunEntry


def llama_spec(cfg: LlamaConfig, norm_init: str = "ones") -> ModelSpec:
    scaling = None if cfg.rope_scaling is None else cfg.rope_scaling.to_dict()
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling,
                                     "rotary_dim": cfg.rotary_dim})
        mixer = PartSpec(
            "gqa_attention",
            {"hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
             "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim},
            {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
             "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"},
            {"position": position})
        ffn = PartSpec("swiglu", {"hidden": cfg.hidden_size, "inter": cfg.intermediate_size},
                       {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                        "down": p + "mlp.down_proj.weight"})
        norm = {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps, "init": norm_init}
        layers.append(PartSpec("pre_norm", parts={
            "norm1": PartSpec("rmsnorm", dict(norm), {"weight": p + "input_layernorm.weight"}),
            "mixer": mixer,
            "norm2": PartSpec("rmsnorm", dict(norm), {"weight": p + "post_attention_layernorm.weight"}),
            "ffn": ffn}))
    return ModelSpec(
        architecture="LlamaForCausalLM", hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        embedding="model.embed_tokens.weight", layers=layers,
        run_order=[RunEntry(layer=i, cache=i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps, "init": norm_init},
                            {"weight": "model.norm.weight"}),
        lm_head=None if cfg.tie_word_embeddings else "lm_head.weight",
        initializer_range=cfg.initializer_range, eos_token_ids=cfg.eos_token_ids,
        max_position_embeddings=cfg.max_position_embeddings)
