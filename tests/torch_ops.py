"""Plain PyTorch statements of the engine's operators, one loop-level function each.

Two uses, both in tests only: (1) the reference each CUDA kernel is compared with, and (2) an
operator set that lets the engine's host logic (step function, cache, scheduler) be exercised on
a machine without a GPU.  The package never imports this file.  Everything is computed in
float32 (float64 where noted) whatever the element type of the inputs, and rounded once.
"""
from __future__ import annotations

import math

import torch


class TorchOps:
    name = "torch-reference"

    def __init__(self, device="cpu"):
        self.device = torch.device(device)

    def empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def embed(self, ids, table):
        return table[ids.long()].clone()

    def add_rmsnorm(self, x, residual, weight, eps, rows=None, dtype=None):
        dtype = dtype or x.dtype
        s = None
        if residual is not None:
            s = residual.float()
        if x is not None:
            s = x.float() if s is None else s + x.float()
        if rows is not None:
            s = s[rows.long()]
        y = s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * weight.float()
        if rows is not None:
            return y.to(dtype), None
        if residual is not None:
            residual.copy_(s)
            return y.to(dtype), residual
        return y.to(dtype), s

    def linear(self, x, w, out_dtype=None):
        return (x.float() @ w.float().T).to(out_dtype or x.dtype)

    linear_simt = linear

    def linear_add(self, x, w, residual):
        return self.linear(x, w)          # never fused: the caller's norm adds it

    def fused_ffn_layout(self, dtype, hidden, inter):
        return False

    def silu_mul(self, gu):
        inter = gu.shape[1] // 2
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
        return (g * torch.sigmoid(g) * u).to(gu.dtype)

    def rope_kv_write(self, qkv, positions, inv_freq, rot, slots, cache, nq, nkv, d, page_size):
        T = qkv.shape[0]
        heads = qkv.view(T, nq + 2 * nkv, d)
        if inv_freq is not None and rot > 0:
            half = rot // 2
            ang = positions.float()[:, None] * inv_freq.float()[None, :half]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            qk = heads[:, : nq + nkv].float()
            x1, x2 = qk[..., :half].clone(), qk[..., half:rot].clone()
            qk[..., :half] = x1 * cos - x2 * sin
            qk[..., half:rot] = x2 * cos + x1 * sin
            heads[:, : nq + nkv] = qk.to(qkv.dtype)
        if cache is not None:
            for t in range(T):
                s = int(slots[t])
                if s < 0:
                    continue
                page, off = divmod(s, page_size)
                cache[page, 0, :, off, :] = heads[t, nq:nq + nkv]
                cache[page, 1, :, off, :] = heads[t, nq + nkv:]

    def paged_attention(self, q, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                        window=0, splits=1, hints=None):
        T = q.shape[0]
        out = torch.zeros((T, nq * d), dtype=torch.float32, device=q.device)
        group = nq // nkv
        for t in range(T):
            r, p = int(tok_req[t]), int(positions[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            keys = torch.arange(lo, p + 1)
            pages = block_table[r][(keys // page_size).long()].long()
            assert (pages >= 0).all(), "attention reads a page that was given back"
            offs = (keys % page_size).long()
            k = cache[pages, 0, :, offs, :].float()   # [n, nkv, d]
            v = cache[pages, 1, :, offs, :].float()
            qt = q[t, : nq * d].view(nq, d).float()
            for h in range(nq):
                s = (k[:, h // group] @ qt[h]) * scale
                out[t, h * d:(h + 1) * d] = torch.softmax(s, dim=0) @ v[:, h // group]
        return out.to(q.dtype)

    def sample(self, logits, temperature, top_p, u, out=None):
        rows = logits.shape[0]
        given, out = out, torch.empty(rows, dtype=torch.int32)
        for i in range(rows):
            t = 0.0 if temperature is None else float(temperature[i])
            x = logits[i].double()
            if t <= 0:
                out[i] = int(torch.argmax(x))
                continue
            p = torch.softmax(x / t, dim=-1)
            sp, idx = torch.sort(p, descending=True)
            keep_sorted = ~((torch.cumsum(sp, 0) - sp) > float(top_p[i]))
            keep = torch.zeros_like(keep_sorted)
            keep[idx] = keep_sorted
            kept = torch.where(keep, p, torch.zeros_like(p))
            cdf = torch.cumsum(kept, 0)
            tok = int(torch.searchsorted(cdf, torch.tensor(float(u[i]) * float(cdf[-1]), dtype=cdf.dtype), right=True))
            out[i] = min(tok, int(torch.nonzero(keep)[-1]))
        if given is not None:
            given.copy_(out)
            return given
        return out.to(logits.device)

    def take_tokens(self, tokens, src, sampled):
        pick = src >= 0
        tokens[pick] = sampled[src[pick].long()]

    def token_logprobs(self, logits, tokens):
        lp = torch.log_softmax(logits.double(), dim=-1)
        return lp.gather(1, tokens.long().view(-1, 1)).view(-1).float()

    def bad_token_seen(self):
        return False
