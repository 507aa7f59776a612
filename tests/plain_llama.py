"""Plain, slow restatement of the dense GQA Llama decoder, used only as the tests' oracle.

It works on whole sequences without any cache, has one function per part and
shares no code with the package under test (it even reads safetensors files with
its own few lines).  Every function names the place in lite_llama whose formula
it restates (paths are relative to the lite_llama project root).

Differences from lite_llama that are deliberate: all arithmetic happens in one
dtype (float32 by default, float64 on request) instead of float16 with float32
islands, the causal mask is -inf instead of an additive -1e8, and
``tie_word_embeddings`` is honoured when the file carries no ``lm_head.weight``.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
}


def read_safetensors(path):
    """name -> tensor, copied out of a .safetensors file (8-byte length, JSON header, raw data)."""
    blob = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(blob[base + lo:base + hi]), dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def load_model_folder(folder, dtype=torch.float32):
    """(config dict, weights dict in ``dtype``) of a folder with config.json and model.safetensors."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {k: v.to(dtype) for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, weights


def head_dim_of(cfg):
    # lite_llama/models/llama.py:17 (config.head_dim if given, else hidden_size // num_heads)
    hd = cfg.get("head_dim")
    return hd if hd is not None else cfg["hidden_size"] // cfg["num_attention_heads"]


def rotary_dim_of(cfg):
    # lite_llama/models/RotaryEmbedding.py:43-44: dim = int(head_dim * partial_rotary_factor), factor 1.0 when absent
    return int(head_dim_of(cfg) * cfg.get("partial_rotary_factor", 1.0))


def rope_inv_freq(cfg):
    """Inverse frequencies, float32.  lite_llama/models/RotaryEmbedding.py:51 (default) and
    :80-98 (llama3 scaling: long wavelengths divided by ``factor``, a smooth blend in the
    medium band, short wavelengths untouched)."""
    d = rotary_dim_of(cfg)
    base = cfg.get("rope_theta", 10000.0)
    inv_freq = 1.0 / (base ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    sc = cfg.get("rope_scaling")
    if sc is None:
        return inv_freq
    kind = sc.get("rope_type", sc.get("type"))
    if kind == "default":
        return inv_freq
    assert kind == "llama3", kind
    factor = sc["factor"]
    low = sc["low_freq_factor"]
    high = sc["high_freq_factor"]
    old_len = sc["original_max_position_embeddings"]
    low_wavelen = old_len / low
    high_wavelen = old_len / high
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old_len / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) * ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled)


def rope_cos_sin(inv_freq, positions, dtype):
    """cos/sin tables [S, d].  RotaryEmbedding.py:200-217: angle = position * inv_freq in
    float32, the half table repeated twice along the last axis."""
    freqs = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32).to(positions.device)[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    if dtype == torch.float64:  # the angle stays the float32 product; only cos/sin get more digits
        emb = emb.double()
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x, cos, sin):
    """x [S, heads, d] rotated by halves.  lite_llama/kernels/rope_emb.py:94-103:
    out1 = x1*cos - x2*sin ; out2 = x2*cos + x1*sin with x1 = x[..., :d/2], x2 = x[..., d/2:]."""
    d = x.shape[-1]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    c, s = cos[:, None, : d // 2], sin[:, None, : d // 2]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def rms_norm(x, w, eps):
    """lite_llama/kernels/skip_rmsnorm.py:113-119: y = x / sqrt(mean(x^2) + eps) * w
    (eps inside the root, plain weight, no 1+w)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(var + eps)) * w


def causal_gqa_attention(q, k, v, window=None):
    """q [S, nq, d], k/v [S, nkv, d] -> [S, nq, d].  lite_llama/kernels/flashattentionv2.py:108
    (kv head = q head // group), :32-59 (scaled scores, causal mask, softmax, P@V) and
    lite_llama/models/llama.py:173 (scale 1/sqrt(d)).  ``window`` (not in lite_llama) keeps only
    the last ``window`` keys of each query, itself included."""
    S, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(d)
    pos = torch.arange(S, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    out = torch.empty_like(q)
    for h in range(nq):
        kh = h // group
        scores = (q[:, h] @ k[:, kh].T) * scale
        scores = scores.masked_fill(~allowed, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h] = probs @ v[:, kh]
    return out


def swiglu_ffn(x, w_gate, w_up, w_down):
    """lite_llama/models/llama.py:120 with lite_llama/kernels/swiglu.py:44-46,64-66:
    down( silu(gate(x)) * up(x) ), silu(a) = a * sigmoid(a), no biases."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (g * torch.sigmoid(g) * u) @ w_down.T


def attention_block(x, positions, cfg, w, prefix, window=None):
    """lite_llama/models/llama.py:37-61: q/k/v projections without bias, head-major split,
    RoPE on q and k, attention, output projection."""
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nq
    d = head_dim_of(cfg)
    S = x.shape[0]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).view(S, nq, d)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).view(S, nkv, d)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).view(S, nkv, d)
    cos, sin = rope_cos_sin(rope_inv_freq(cfg), positions, x.dtype)
    rot = rotary_dim_of(cfg)      # the leading `rot` elements of a head are rotated, the rest pass through
    q = torch.cat((apply_rope(q[..., :rot], cos, sin), q[..., rot:]), dim=-1)
    k = torch.cat((apply_rope(k[..., :rot], cos, sin), k[..., rot:]), dim=-1)
    o = causal_gqa_attention(q, k, v, window)
    return o.reshape(S, nq * d) @ w[prefix + "self_attn.o_proj.weight"].T


def decoder_layer(h, positions, cfg, w, i):
    """lite_llama/models/llama.py:149-162: pre-norm block.  lite_llama carries (hidden, residual)
    and adds inside the next norm (skip_rmsnorm.py:145-149); written here as the plain sums."""
    p = f"model.layers.{i}."
    eps = cfg.get("rms_norm_eps", 1e-5)
    h = h + attention_block(rms_norm(h, w[p + "input_layernorm.weight"], eps), positions, cfg, w, p)
    h = h + swiglu_ffn(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps),
                       w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])
    return h


def forward(cfg, w, tokens):
    """Logits [S, vocab] of one whole sequence.  lite_llama/models/llama.py:189-223: embedding,
    positions 0..S-1, the layers in order, final norm, LM head over every position."""
    device = w["model.embed_tokens.weight"].device      # the weights may have been moved to an accelerator by the caller
    tokens = torch.as_tensor(tokens, dtype=torch.long, device=device)
    positions = torch.arange(tokens.shape[0], device=device)
    h = w["model.embed_tokens.weight"][tokens]
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, positions, cfg, w, i)
    h = rms_norm(h, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = w.get("lm_head.weight")
    if head is None:
        assert cfg.get("tie_word_embeddings", True), "untied model without lm_head.weight"
        head = w["model.embed_tokens.weight"]
    return h @ head.T


def top_p_keep_mask(probs, top_p):
    """Which tokens survive nucleus filtering.  lite_llama/generate.py:30-35: sort descending,
    cumulative sum, drop a token when the mass *before* it exceeds p (the first always stays)."""
    sorted_p, idx = torch.sort(probs, dim=-1, descending=True)
    before = torch.cumsum(sorted_p, dim=-1) - sorted_p
    keep_sorted = ~(before > top_p)
    keep = torch.zeros_like(keep_sorted)
    keep.scatter_(-1, idx, keep_sorted)
    return keep


def sample_token(logits, temperature, top_p, u):
    """One token from one row of logits.  lite_llama/generate_stream.py:143-150: argmax when
    temperature is 0, else softmax(logits / temperature), top-p filter and renormalisation
    (lite_llama/generate.py:30-38).  Where lite_llama draws with torch.multinomial, this takes the
    uniform number ``u`` in [0,1) and walks the kept tokens in vocabulary order."""
    logits = logits.double()
    if temperature <= 0:
        return int(torch.argmax(logits))
    probs = torch.softmax(logits / temperature, dim=-1)
    keep = top_p_keep_mask(probs, top_p)
    kept = torch.where(keep, probs, torch.zeros_like(probs))
    cdf = torch.cumsum(kept, dim=-1)
    target = u * float(cdf[-1])
    tok = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype), right=True))
    last_kept = int(torch.nonzero(keep)[-1])
    return min(tok, last_kept)


def greedy_generate(cfg, w, prompt, max_new_tokens, stop_ids=()):
    """Greedy continuation by recomputing the whole sequence for every new token."""
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        nxt = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(nxt)
        seq.append(nxt)
        if nxt in stop_ids:
            break
    return out
