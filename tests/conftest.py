"""Shared fixtures: the tiny configurations, model folders of random weights made in temporary
folders, and the ``gpu`` marker (tests that need a B200; skipped where no CUDA device exists)."""
import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Three tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 1,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 2048, "eos_token_id": 255,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
    "eos_token_id": [382, 383],
}
# head size 48 (no power of two), as many kv heads as query heads, hidden != heads * head_dim,
# a vocabulary and widths that are no multiples of 64
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 1, "hidden_size": 200, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 264, "vocab_size": 1000, "rope_theta": 25000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 2.0, "high_freq_factor": 8.0,
                     "original_max_position_embeddings": 32},
    "rms_norm_eps": 3e-4, "tie_word_embeddings": True, "max_position_embeddings": 1024,
    "partial_rotary_factor": 0.5,      # only the first 24 elements of a head are rotated
}
# Tolerances, fixed before the kernels were written.  float32 engine against the float64 plain
# implementation: 1e-4 absolute on logits of size up to ~6.  bfloat16 engine (same bfloat16
# weights on both sides, so only activations round): ~30 roundings of relative size 2^-9 on the
# way to a logit give a few times 1e-2 of the largest logit at worst, far less on average.
FP32_TOL = 1e-4
BF16_MAX_REL = 0.04
BF16_MEAN_REL = 0.006

# head sizes 64 and 128: the sizes the tensor-core attention kernels take (groups of 4 and of 3)
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 384, "vocab_size": 512, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 4096,
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 320, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 448, "vocab_size": 640, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}
PAGE_SIZE = {"A": 4, "B": 8, "C": 16, "D": 16, "E": 32}
NORM_INIT = {"A": "ones_jitter", "B": "ones", "C": "ones_jitter", "D": "ones_jitter", "E": "ones"}


def _odd(layers, hidden, nq, nkv, d, inter, vocab, theta=10000.0, scaling=None, eps=1e-5, tied=True, **more):
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers, "hidden_size": hidden,
           "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "intermediate_size": inter, "vocab_size": vocab,
           "rope_theta": theta, "rope_scaling": scaling, "rms_norm_eps": eps, "tie_word_embeddings": tied,
           "max_position_embeddings": 4096}
    cfg.update(more)
    return cfg


# More shapes for the random traces (tests/test_gpu_random_traces.py): head sizes 80, 96, 112 and 256,
# a group of 20 query heads per kv head, as many kv heads as query heads on the tensor-core attention
# (with a quarter of the head rotated), 16 query heads over 2 kv heads of size 128, vocabularies of 50 to 2,049.
TINY.update({
    "F": _odd(2, 288, 3, 1, 96, 200, 1001),
    "G": _odd(1, 256, 2, 1, 256, 136, 300, tied=False),
    "H": _odd(2, 320, 20, 1, 64, 264, 777),
    "I": _odd(2, 72, 3, 3, 80, 104, 131, eps=1e-3),
    "J": _odd(1, 224, 7, 7, 112, 168, 513, theta=500000.0,
              scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                       "original_max_position_embeddings": 64}),
    "K": _odd(3, 128, 16, 2, 128, 96, 2049),
    "L": _odd(2, 512, 8, 8, 64, 1000, 50, partial_rotary_factor=0.25),
})
PAGE_SIZE.update({"F": 16, "G": 8, "H": 16, "I": 4, "J": 32, "K": 64, "L": 16})
NORM_INIT.update({k: "ones_jitter" for k in "FGHIJKL"})


def make_model_folder(folder, name, stored_dtype, seed=11, std=0.08, qk_gain=None):
    """Writes a random-weights folder through the package's random-weights mode, then makes the
    attention scores matter: q and k projections are scaled so that softmax is far from uniform
    (with N(0, 0.02) weights every key would weigh the same and position faults would hide).
    float32 folders get scores of size ~5 (one key in a few dominates).  bfloat16 folders get
    scores of size ~1-2: a score s carries a rounding error of about |s| * 2^-8 from the 8-bit
    q and k, which softmax turns into the same relative error of the weights, so scores of 10-15
    alone would use up the whole bfloat16 tolerance without any fault being present."""
    if qk_gain is None:
        qk_gain = 2.0 if stored_dtype == torch.float32 else 1.0
    from pytriton_llama_b200.weights import read_folder, write_file, write_random_model
    folder = Path(folder)
    write_random_model(folder, TINY[name], seed=seed, dtype=torch.float32, norm_init=NORM_INIT[name], std=std)
    tensors = {k: v.clone() for k, v in read_folder(folder).items()}
    for k in tensors:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            tensors[k] = tensors[k] * qk_gain
    tensors = {k: v.to(stored_dtype) for k, v in tensors.items()}
    write_file(folder / "model.safetensors", tensors)
    return folder


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """(config name, stored element type) -> model folder, made on first use."""
    made = {}

    def get(name, stored_dtype=torch.float32):
        key = (name, stored_dtype)
        if key not in made:
            made[key] = make_model_folder(tmp_path_factory.mktemp(f"model_{name}_{str(stored_dtype)[6:]}"), name, stored_dtype)
        return made[key]
    return get


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
