"""The plain implementation itself (no GPU): against lite_llama's own model code through the
stored outputs under tests/golden/, and against hand-checkable properties."""
import math
from pathlib import Path

import pytest
import torch

import plain_llama
from conftest import TINY_B

GOLDEN = Path(__file__).resolve().parent / "golden"


def _golden_case(name):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_reference_golden", GOLDEN / "make_reference_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    data = torch.load(GOLDEN / f"reference_tiny_{name}.pt")
    cfg = dict(data["config"])
    weights = mod.golden_weights(cfg)
    assert mod.checksum(weights) == pytest.approx(data["checksum"], rel=1e-12), "weights drawn differently than when the outputs were stored"
    cfg["tie_word_embeddings"] = False
    return cfg, {k: v.float() for k, v in weights.items()}, data


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_lite_llama_own_model(name):
    """lite_llama computes in float16 (activations rounded at every kernel), the plain implementation
    in float32 on the same float16 weights: they agree to float16 rounding of logits of size ~1-3."""
    cfg, w, data = _golden_case(name)
    tokens = data["tokens"].tolist()
    P = cfg["prompt_len"]
    logits = plain_llama.forward(cfg, w, tokens)
    ref_prefill = data["prefill_logits"].float()
    ref_decode = data["decode_logits"].float()
    scale = float(ref_prefill.abs().max())
    assert (logits[:P] - ref_prefill).abs().max() < 4e-3 * max(1.0, scale)
    assert (logits[P:P + 1] - ref_decode).abs().max() < 4e-3 * max(1.0, scale)
    assert (logits[:P] - ref_prefill).abs().mean() < 5e-4 * max(1.0, scale)
    # the comparison has teeth: one position off and it fails by far
    assert (logits[1:P] - ref_prefill[:P - 1]).abs().max() > 0.1


def test_llama3_frequencies_follow_the_formula():
    inv = plain_llama.rope_inv_freq(TINY_B)
    d = 32
    base = torch.tensor([500000.0 ** (-2 * j / d) for j in range(d // 2)])
    wavelen = 2 * math.pi / base
    assert torch.allclose(inv[wavelen < 64 / 4], base[wavelen < 64 / 4])          # short waves untouched
    assert torch.allclose(inv[wavelen > 64], base[wavelen > 64] / 8, rtol=1e-6)   # long waves divided by the factor
    mid = (wavelen >= 64 / 4) & (wavelen <= 64)
    assert mid.any() and ((inv[mid] < base[mid]) & (inv[mid] > base[mid] / 8 * 0.999)).all()


def test_rope_is_a_rotation_of_half_pairs():
    x = torch.randn(3, 2, 8)
    inv = torch.tensor([1.0, 0.5, 0.25, 0.125])
    cos, sin = plain_llama.rope_cos_sin(inv, torch.tensor([0, 1, 5]), torch.float32)
    y = plain_llama.apply_rope(x, cos, sin)
    assert torch.allclose(y[0], x[0])                                             # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    a = 5 * 0.5
    assert torch.allclose(y[2, 1, 1], x[2, 1, 1] * math.cos(a) - x[2, 1, 5] * math.sin(a), atol=1e-6)
    assert torch.allclose(y[2, 1, 5], x[2, 1, 5] * math.cos(a) + x[2, 1, 1] * math.sin(a), atol=1e-6)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = plain_llama.causal_gqa_attention(q, k, v)
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6)                          # first token sees itself only; head 3 -> kv head 1
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 7.0, -3.0
    assert torch.allclose(plain_llama.causal_gqa_attention(q, k2, v2)[:4], out[:4])   # later keys never matter
    w = plain_llama.causal_gqa_attention(q, k, v, window=2)
    s = (q[5, 0] @ k[4:6, 0].T) / math.sqrt(8)
    assert torch.allclose(w[5, 0], torch.softmax(s, 0) @ v[4:6, 0], atol=1e-6)


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(plain_llama.rms_norm(x, torch.tensor([1.0, 2.0]), 0.5),
                          torch.tensor([[3.0, 8.0]]) / math.sqrt(12.5 + 0.5))
    wg, wu, wd = torch.tensor([[1.0, 0.0]]), torch.tensor([[0.0, 1.0]]), torch.tensor([[2.0], [1.0]])
    y = plain_llama.swiglu_ffn(x, wg, wu, wd)
    h = 3.0 / (1 + math.exp(-3.0)) * 4.0
    assert torch.allclose(y, torch.tensor([[2 * h, h]]))


def test_top_p_keeps_tokens_whose_preceding_mass_is_within_p():
    probs = torch.tensor([0.05, 0.5, 0.15, 0.3])
    assert plain_llama.top_p_keep_mask(probs, 0.7).tolist() == [False, True, False, True]   # 0.5, then 0.3 (mass before: 0.5)
    assert plain_llama.top_p_keep_mask(probs, 0.81).tolist() == [False, True, True, True]   # 0.15 has 0.8 before it: kept
    assert plain_llama.top_p_keep_mask(probs, 0.01).tolist() == [False, True, False, False]  # the most likely always stays
    logits = torch.log(probs)
    assert plain_llama.sample_token(logits, 0.0, 0.9, 0.3) == 1
    # kept {1, 3} with mass 0.8: u below 0.5/0.8 gives token 1, above gives token 3
    assert plain_llama.sample_token(logits, 1.0, 0.7, 0.6) == 1
    assert plain_llama.sample_token(logits, 1.0, 0.7, 0.65) == 3
    assert plain_llama.sample_token(logits, 1.0, 0.7, 0.999999) == 3
