"""Runs lite_llama's OWN model code (lite_llama/models/llama.py with its Triton kernels, executed
on the CPU by Triton's interpreter) on two tiny random models and stores its logits, so that the
plain implementation in tests/plain_llama.py can be compared with the project it restates.

    python tests/golden/make_reference_golden.py /path/to/lite_llama_checkout

writes tests/golden/reference_tiny_{A,B}.pt: the seed of the weights, a checksum of them, the
prompt, lite_llama's float16 logits for the prompt (prefill path) and for one more token
(single-token path).  Weights are drawn by ``golden_weights`` below; the test draws them again
from the same seed.

Three shims make the import work without a GPU (nothing of lite_llama is changed):
TRITON_INTERPRET=1; ``torch.cuda.get_device_name`` answering "cpu" (one kernel file asks at import);
and a bare ``lite_llama`` package object so that its __init__ (which needs ``accelerate`` and CUDA)
is not run.  The attention-info object is filled as lite_llama's executor fills it
(lite_llama/executor/model_executor.py:287-296,306-311).
"""
import os
import sys
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent

CONFIGS = {
    "A": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=1,
              intermediate_size=128, vocab_size=256, rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
              max_position_embeddings=2048, prompt_len=11, seed=101),
    "B": dict(num_hidden_layers=3, hidden_size=192, num_attention_heads=6, num_key_value_heads=2,
              intermediate_size=320, vocab_size=384, rope_theta=500000.0,
              rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 64},
              rms_norm_eps=1e-6, max_position_embeddings=4096, prompt_len=70, seed=202),
}


def golden_weights(cfg, std=0.05):
    """Checkpoint-named float16 tensors of a tiny model, drawn from cfg['seed'] in a fixed order."""
    g = torch.Generator().manual_seed(cfg["seed"])
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = H // nq

    def mat(*shape):
        return (std * torch.randn(*shape, generator=g)).half()

    def norm():
        return (1.0 + 0.05 * torch.randn(H, generator=g)).half()

    w = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": norm(), "lm_head.weight": mat(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = mat(nq * d, H) * 2
        w[p + "self_attn.k_proj.weight"] = mat(nkv * d, H) * 2
        w[p + "self_attn.v_proj.weight"] = mat(nkv * d, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, nq * d)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
        w[p + "input_layernorm.weight"] = norm()
        w[p + "post_attention_layernorm.weight"] = norm()
    return w


def checksum(weights):
    return float(sum(v.double().abs().sum() for v in weights.values()))


def golden_prompt(cfg):
    g = torch.Generator().manual_seed(cfg["seed"] + 1)
    return torch.randint(0, cfg["vocab_size"], (cfg["prompt_len"] + 1,), generator=g)


def import_lite_llama(root):
    torch.cuda.get_device_name = lambda *a, **k: "cpu"
    pkg = types.ModuleType("lite_llama")
    pkg.__path__ = [str(Path(root) / "lite_llama")]
    sys.modules["lite_llama"] = pkg
    import lite_llama.models.llama as llama
    import lite_llama.models.model_config as model_config
    return llama, model_config


def run_reference(root, name):
    llama, model_config = import_lite_llama(root)
    cfg = CONFIGS[name]
    keys = ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "intermediate_size",
            "vocab_size", "rope_theta", "rope_scaling", "rms_norm_eps", "max_position_embeddings")
    lcfg = model_config.LlamaConfig.from_dict({k: cfg[k] for k in keys})
    lcfg.device = "cpu"
    model = llama.LlamaModel(lcfg)
    w = golden_weights(cfg)
    # lite_llama's own renaming and k|v fusing (lite_llama/executor/weight_convert.py:193-246)
    sd = {"embed_tokens.weight": w["model.embed_tokens.weight"], "norm_weight": w["model.norm.weight"],
          "lm_head.weight": w["lm_head.weight"]}
    for i in range(cfg["num_hidden_layers"]):
        p, q = f"model.layers.{i}.", f"layers.{i}."
        sd[q + "self_attn.q_proj.weight"] = w[p + "self_attn.q_proj.weight"]
        sd[q + "self_attn.kv_proj_weight"] = torch.cat([w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"]], 0)
        sd[q + "self_attn.o_proj.weight"] = w[p + "self_attn.o_proj.weight"]
        for m in ("gate_proj", "up_proj", "down_proj"):
            sd[q + f"mlp.{m}.weight"] = w[p + f"mlp.{m}.weight"]
        sd[q + "attention_norm_weight"] = w[p + "input_layernorm.weight"]
        sd[q + "ffn_norm_weight"] = w[p + "post_attention_layernorm.weight"]
    model.load_state_dict(sd, strict=True)
    model = model.half().eval()

    tokens = golden_prompt(cfg)
    P = cfg["prompt_len"]
    nkv, d = cfg["num_key_value_heads"], cfg["hidden_size"] // cfg["num_attention_heads"]
    info = types.SimpleNamespace()
    total = P + 1
    info.kv_buffer = [torch.zeros(total, 2 * nkv, d, dtype=torch.float16) for _ in range(cfg["num_hidden_layers"])]
    info.select_index = torch.arange(total)
    info.start_index = torch.zeros(1, dtype=torch.int32)
    info.cur_select_index = torch.arange(P)
    info.b_seq_len = torch.tensor([P], dtype=torch.long)
    info.max_actual_seq_len = P
    with torch.no_grad():
        prefill = model(tokens[None, :P], 0, info)[0].float()
        info.cur_select_index = info.start_index + info.b_seq_len
        info.b_seq_len = info.b_seq_len + 1
        info.max_actual_seq_len += 1
        decode = model(tokens[None, P:P + 1], P, info)[0].float()
    return {"config": cfg, "checksum": checksum(w), "tokens": tokens, "prefill_logits": prefill.half(),
            "decode_logits": decode.half()}


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_reference_golden.py /path/to/lite_llama_checkout")
    root = sys.argv[1]
    for name in CONFIGS:
        out = run_reference(root, name)
        torch.save(out, HERE / f"reference_tiny_{name}.pt")
        print(name, out["prefill_logits"].shape, out["decode_logits"].shape, "checksum", out["checksum"],
              "max |logit|", float(out["prefill_logits"].abs().max()))
