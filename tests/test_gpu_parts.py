"""Each part of a layer alone against the plain implementation's function for it, the block that
arranges them, run orders that name a layer twice or share a cache entry, and a toy mixer with
state of its own that is registered here, built and stepped without touching the package (GPU)."""
import math

import pytest
import torch

import plain_llama
from conftest import TINY, TINY_B, random_tokens
from gpu_common import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from pytriton_llama_b200.ops.cuda import CudaOps
    from pytriton_llama_b200.parts import Runtime
    dev = torch.device("cuda:0")
    return {d: Runtime(dev, d, CudaOps(dev)) for d in (torch.float32, torch.bfloat16)}


def _ctx(q_lens, starts, page_size, tables, slots, window=0):
    from pytriton_llama_b200.engine.context import GroupStepView, StepContext
    R = len(q_lens)
    dev = "cuda:0"
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    width = max(len(t) for t in tables)
    bt = torch.full((R, width), -1, dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
    group = GroupStepView(page_size, bt.to(dev), i32(slots), window)
    pos = [p for s, n in zip(starts, q_lens) for p in range(s, s + n)]
    tok_req = [r for r, n in enumerate(q_lens) for _ in range(n)]
    return StepContext(num_tokens=sum(q_lens), num_requests=R, positions=i32(pos), tok_req=i32(tok_req),
                       q_start=i32([0] + list(torch.tensor(q_lens).cumsum(0))), ctx_len=i32([s + n for s, n in zip(starts, q_lens)]),
                       state_slot=i32(list(range(R))), fresh=i32([int(s == 0) for s in starts]), groups={0: group},
                       q_lens=q_lens, ctx_lens=[s + n for s, n in zip(starts, q_lens)], max_q_len=max(q_lens),
                       max_ctx_len=max(s + n for s, n in zip(starts, q_lens))), group


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(rt, dtype):
    from pytriton_llama_b200.parts import PartSpec, build_part
    part = build_part("norm", PartSpec("rmsnorm", {"width": 200, "eps": 3e-4}, {"weight": "w"}), rt[dtype])
    assert part.tensor_specs()["weight"].shape == (200,)
    w = 1 + 0.1 * torch.randn(200)
    part.load({"weight": w.to(torch.bfloat16)})            # stored in 16 bits: read exactly, kept as float32
    assert part.weight.dtype == torch.float32
    x = torch.randn(6, 200).to(dtype)
    res = torch.randn(6, 200)
    y, r = part.forward(x.cuda(), res.clone().cuda())
    s = res.double() + x.double()
    want = plain_llama.rms_norm(s, w.to(torch.bfloat16).double(), 3e-4)
    assert (r.double().cpu() - s).abs().max() < 1e-6
    assert (y.double().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)


def test_rope_part_builds_the_reference_frequencies(rt):
    from pytriton_llama_b200.parts import PartSpec, build_part
    for cfg in TINY.values():
        hd = cfg["head_dim"]
        want_rot = plain_llama.rotary_dim_of(cfg)
        part = build_part("position", PartSpec("rope", {"head_dim": hd, "theta": cfg["rope_theta"], "scaling": cfg["rope_scaling"],
                                                        "rotary_dim": want_rot}), rt[torch.float32])
        inv, rot = part.rotary_table()
        assert rot == want_rot and inv.dtype == torch.float32
        assert torch.equal(inv.cpu(), plain_llama.rope_inv_freq(cfg))      # bit for bit, llama3 scaling included


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 13])
def test_attention_part_over_two_steps(rt, dtype, window):
    """The mixer alone with a cache of its own: a 29-token portion, then 11 more tokens, equals the
    plain attention block over all 40 (projections, rotation, cache write, attention, output)."""
    from pytriton_llama_b200.engine.context import LayerCacheView
    from pytriton_llama_b200.parts import PartSpec, build_part
    cfg = dict(TINY_B)
    H, nq, nkv, d = 192, 6, 2, 32
    spec = PartSpec("gqa_attention", {"hidden": H, "heads": nq, "kv_heads": nkv, "head_dim": d, "window": window},
                    {"q": "q", "k": "k", "v": "v", "o": "o"},
                    {"position": PartSpec("rope", {"head_dim": d, "theta": cfg["rope_theta"], "scaling": cfg["rope_scaling"]})})
    part = build_part("mixer", spec, rt[dtype])
    need = part.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim, need.window) == ("window" if window else "full", nkv, d, window)
    g = torch.Generator().manual_seed(1)
    w = {n: (0.12 * torch.randn(s.shape, generator=g)).to(dtype) for n, s in part.tensor_specs().items()}
    part.load(w)
    x = torch.randn(40, H, generator=g).to(dtype)
    names = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight"}
    want = plain_llama.attention_block(x.double(), torch.arange(40), cfg, {names[n]: t.double() for n, t in w.items()}, "",
                                       window=window or None)
    page, pages = 8, 7
    table = [5, 2, 6, 0, 3]
    kv = torch.zeros(pages, 2, nkv, page, d, dtype=dtype, device="cuda")
    slot = lambda p: table[p // page] * page + p % page
    ctx, group = _ctx([29], [0], page, [table[:4]], [slot(p) for p in range(29)], window)
    out1 = part.forward(x[:29].cuda(), ctx, LayerCacheView(group, kv, None, True))
    ctx, group = _ctx([11], [29], page, [table], [slot(p) for p in range(29, 40)], window)
    out2 = part.forward(x[29:].cuda(), ctx, LayerCacheView(group, kv, None, True))
    got = torch.cat([out1, out2]).double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 0.03 * float(want.abs().max())
    assert (got - want).abs().max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(rt, dtype):
    from pytriton_llama_b200.parts import PartSpec, build_part
    part = build_part("ffn", PartSpec("swiglu", {"hidden": 200, "inter": 264}, {"gate": "g", "up": "u", "down": "d"}), rt[dtype])
    g = torch.Generator().manual_seed(2)
    w = {n: (0.1 * torch.randn(s.shape, generator=g)).to(dtype) for n, s in part.tensor_specs().items()}
    part.load(w)
    x = torch.randn(9, 200, generator=g).to(dtype)
    want = plain_llama.swiglu_ffn(x.double(), w["gate"].double(), w["up"].double(), w["down"].double())
    got = part.forward(x.cuda()).double().cpu()
    assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.03 * float(want.abs().max()))


# ---------------------------------------------------------------------------------------------
# A toy mixer with state of its own, defined here: y_t = x_t * gain + decay * s_{t-1},  s_t = y_t,
# one state vector per request that survives between steps.  It uses no attention cache at all.

def _register_toy():
    from pytriton_llama_b200.parts import CacheNeed, Part, TensorSpec, register_part

    @register_part("mixer", "toy_running_state")
    class ToyRunningState(Part):
        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.hidden = spec.params["hidden"]
            self.decay = spec.params["decay"]

        def tensor_specs(self):
            return {"gain": TensorSpec((self.hidden,), init="ones_jitter")}

        def load(self, tensors):
            self.gain = self._to_f32(tensors["gain"])

        def cache_need(self):
            return CacheNeed(kind="none", state_shape=(self.hidden,), state_dtype=torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            starts = [0]
            for n in ctx.q_lens:
                starts.append(starts[-1] + n)
            slots = ctx.state_slot.tolist()
            fresh = ctx.fresh.tolist()
            for r, n in enumerate(ctx.q_lens):
                s = cache.state[slots[r]]
                if fresh[r]:
                    s.zero_()
                for t in range(starts[r], starts[r] + n):
                    y = x[t].float() * self.gain + self.decay * s
                    s.copy_(y)
                    out[t] = y.to(x.dtype)
            return out
    return ToyRunningState


def _toy_spec(cfg, toy_layers, run_order=None):
    from pytriton_llama_b200.config import LlamaConfig
    from pytriton_llama_b200.models.llama import llama_spec
    from pytriton_llama_b200.parts import PartSpec
    spec = llama_spec(LlamaConfig.from_dict(cfg), norm_init="ones_jitter")
    for i in toy_layers:
        spec.layers[i].parts["mixer"] = PartSpec("toy_running_state", {"hidden": cfg["hidden_size"], "decay": 0.5},
                                                 {"gain": f"model.layers.{i}.toy.gain"})
    if run_order is not None:
        spec.run_order = run_order
    return spec


def _plain_toy_forward(cfg, w, tokens, toy_layers, run_order):
    """The plain implementation's pieces with the toy mixer in some layers (float64, whole sequence)."""
    tokens = torch.as_tensor(tokens)
    pos = torch.arange(len(tokens))
    h = w["model.embed_tokens.weight"][tokens]
    eps = cfg["rms_norm_eps"]
    for layer in run_order:
        p = f"model.layers.{layer}."
        x = plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        if layer in toy_layers:
            s = torch.zeros_like(x[0])
            rows = []
            for t in range(len(tokens)):
                s = x[t] * w[p + "toy.gain"] + 0.5 * s
                rows.append(s)
            a = torch.stack(rows)
        else:
            a = plain_llama.attention_block(x, pos, cfg, w, p)
        h = h + a
        h = h + plain_llama.swiglu_ffn(plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps),
                                       w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    h = plain_llama.rms_norm(h, w["model.norm.weight"], eps)
    return h @ w["model.embed_tokens.weight"].T


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """One layer keeps attention, one gets the toy mixer: different mixers in different layers of
    one model, fixed-size state in the manager's slots, no change to the package's files."""
    import traces
    from pytriton_llama_b200.config import EngineConfig, register_architecture, LlamaConfig
    from pytriton_llama_b200.engine.engine import Engine
    from pytriton_llama_b200.weights import read_folder, write_random_model
    _register_toy()
    cfg = dict(TINY["A"], architectures=["ToyStateForCausalLM"])
    register_architecture("ToyStateForCausalLM", LlamaConfig.from_dict,
                          lambda c, norm_init="ones": _toy_spec(cfg, toy_layers=[1]))
    folder = write_random_model(tmp_path / "toy", cfg, seed=4, dtype=torch.float32, std=0.08)
    tensors = read_folder(folder)
    assert "model.layers.1.toy.gain" in tensors and "model.layers.1.self_attn.q_proj.weight" not in tensors
    eng = Engine(folder, EngineConfig(dtype="float32", page_size=4, max_gpu_num_blocks=40, max_seq_len=128, max_num_seqs=3))
    assert len(eng.cache.groups) == 2 and eng.cache.groups[1].state[1].shape == (3, 64)
    seqs = {f"t{i}": random_tokens(n, 256, 50 + i) for i, n in enumerate([21, 9, 33, 14])}
    w = {k: v.double() for k, v in tensors.items()}
    ref = {r: _plain_toy_forward(cfg, w, s, [1], [0, 1]) for r, s in seqs.items()}
    got = traces.replay(eng, traces.mixed(seqs, live=3))       # slots are reused: the state must restart at zero
    for r in seqs:
        assert_close(got[r], ref[r], "float32", r)


def test_run_order_may_repeat_a_layer_and_share_a_cache_entry(tmp_path):
    """Run order [0, 1, 0']: layer 0 runs twice; its second run has a cache entry of its own.  And
    [0, 1(reads entry 0)]: layer 1 stores nothing and attends over the keys and values layer 0 wrote."""
    import traces
    from pytriton_llama_b200.config import EngineConfig, LlamaConfig, register_architecture
    from pytriton_llama_b200.engine.engine import Engine
    from pytriton_llama_b200.models.spec import RunEntry
    from pytriton_llama_b200.weights import read_folder, write_random_model
    base = dict(TINY["A"])
    # (a) a layer twice
    cfg = dict(base, architectures=["TwiceForCausalLM"])
    register_architecture("TwiceForCausalLM", LlamaConfig.from_dict,
                          lambda c, norm_init="ones": _toy_spec(cfg, [], [RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2)]))
    folder = write_random_model(tmp_path / "twice", cfg, seed=5, dtype=torch.float32, std=0.08)
    w = {k: v.double() for k, v in read_folder(folder).items()}
    seqs = {f"s{i}": random_tokens(n, 256, 70 + i) for i, n in enumerate([19, 30, 8])}
    eng = Engine(folder, EngineConfig(dtype="float32", page_size=4, max_gpu_num_blocks=30, max_seq_len=64, max_num_seqs=3))
    assert sorted(eng.cache.groups[0].entries) == [0, 1, 2]
    got = traces.replay(eng, traces.mixed(seqs, live=3))
    for r, s in seqs.items():
        assert_close(got[r], _plain_toy_forward(cfg, w, s, [], [0, 1, 0]), "float32", r)
    # (b) a layer that reads another layer's cache entry
    cfg2 = dict(base, architectures=["SharedForCausalLM"])
    register_architecture("SharedForCausalLM", LlamaConfig.from_dict,
                          lambda c, norm_init="ones": _toy_spec(cfg2, [], [RunEntry(0, 0), RunEntry(1, 0, write=False)]))
    folder2 = write_random_model(tmp_path / "shared", cfg2, seed=6, dtype=torch.float32, std=0.08)
    w2 = {k: v.double() for k, v in read_folder(folder2).items()}
    eng2 = Engine(folder2, EngineConfig(dtype="float32", page_size=4, max_gpu_num_blocks=30, max_seq_len=64, max_num_seqs=3))
    assert eng2.cache.groups[0].entries == [0]                       # one entry: a third of the cache memory
    got2 = traces.replay(eng2, traces.portions(seqs))

    def shared_forward(tokens):
        tokens = torch.as_tensor(tokens)
        pos = torch.arange(len(tokens))
        S = len(tokens)
        h = w2["model.embed_tokens.weight"][tokens]
        eps = base["rms_norm_eps"]
        nq, nkv, d = 4, 1, 16
        cos, sin = plain_llama.rope_cos_sin(plain_llama.rope_inv_freq(base), pos, torch.float64)
        kv0 = None
        for layer in (0, 1):
            p = f"model.layers.{layer}."
            x = plain_llama.rms_norm(h, w2[p + "input_layernorm.weight"], eps)
            q = plain_llama.apply_rope((x @ w2[p + "self_attn.q_proj.weight"].T).view(S, nq, d), cos, sin)
            if layer == 0:
                k = plain_llama.apply_rope((x @ w2[p + "self_attn.k_proj.weight"].T).view(S, nkv, d), cos, sin)
                v = (x @ w2[p + "self_attn.v_proj.weight"].T).view(S, nkv, d)
                kv0 = (k, v)
            a = plain_llama.causal_gqa_attention(q, *kv0).reshape(S, nq * d) @ w2[p + "self_attn.o_proj.weight"].T
            h = h + a
            h = h + plain_llama.swiglu_ffn(plain_llama.rms_norm(h, w2[p + "post_attention_layernorm.weight"], eps),
                                           w2[p + "mlp.gate_proj.weight"], w2[p + "mlp.up_proj.weight"], w2[p + "mlp.down_proj.weight"])
        return plain_llama.rms_norm(h, w2["model.norm.weight"], eps) @ w2["model.embed_tokens.weight"].T
    for r, s in seqs.items():
        assert_close(got2[r], shared_forward(s), "float32", r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_get_pages_of_their_own(tmp_path, dtype):
    """A toy architecture whose second layer attends over a window of 24 keys while the first sees
    everything: two cache groups with their own pools and block tables; the windowed group gives
    pages back as decoding moves on, and the logits still equal the plain implementation's."""
    import traces
    from conftest import make_model_folder
    from pytriton_llama_b200.config import EngineConfig, LlamaConfig, register_architecture
    from pytriton_llama_b200.engine.engine import Engine, StepEntry
    from pytriton_llama_b200.models.llama import llama_spec
    from pytriton_llama_b200.weights import read_folder, write_file, write_random_model
    from conftest import TINY_D
    window = 24
    cfg = dict(TINY_D, architectures=["WindowedForCausalLM"])

    def spec(c, norm_init="ones"):
        sp = llama_spec(c, norm_init=norm_init)
        sp.layers[1].parts["mixer"].params["window"] = window
        return sp
    register_architecture("WindowedForCausalLM", LlamaConfig.from_dict, spec)
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_random_model(tmp_path / "windowed", cfg, seed=9, dtype=torch.float32, std=0.08, norm_init="ones_jitter")
    tensors = {k: v.clone() for k, v in read_folder(folder).items()}
    gain = 2.0 if dtype == "float32" else 1.0
    for k in tensors:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            tensors[k] = tensors[k] * gain
    tensors = {k: v.to(stored) for k, v in tensors.items()}
    write_file(folder / "model.safetensors", tensors)
    w = {k: v.double() for k, v in tensors.items()}

    def plain(tokens):
        tokens = torch.as_tensor(tokens)
        pos = torch.arange(len(tokens))
        h = w["model.embed_tokens.weight"][tokens]
        eps = cfg["rms_norm_eps"]
        for layer in (0, 1):
            pre = f"model.layers.{layer}."
            x = plain_llama.rms_norm(h, w[pre + "input_layernorm.weight"], eps)
            h = h + plain_llama.attention_block(x, pos, cfg, w, pre, window=window if layer == 1 else None)
            h = h + plain_llama.swiglu_ffn(plain_llama.rms_norm(h, w[pre + "post_attention_layernorm.weight"], eps),
                                           w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"], w[pre + "mlp.down_proj.weight"])
        return plain_llama.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T

    eng = Engine(folder, EngineConfig(dtype=dtype, page_size=16, max_gpu_num_blocks=40, max_seq_len=320, max_num_seqs=3))
    assert len(eng.cache.groups) == 2
    kinds = sorted((g.need.kind, g.need.window) for g in eng.cache.groups)
    assert kinds == [("full", 0), ("window", window)]
    seqs = {f"w{i}": random_tokens(n, 512, 90 + i) for i, n in enumerate([150, 70, 300, 40])}
    got = traces.replay(eng, traces.mixed(seqs, live=3, sizes=(40, 7, 130, 2, 19), decode_tail=40))
    for r, s_ in seqs.items():
        assert_close(got[r], plain(s_), dtype, r)
    # the windowed group really gives pages back: a long request holds few of its pages
    win_group = [i for i, g in enumerate(eng.cache.groups) if g.need.kind == "window"][0]
    full_group = 1 - win_group
    eng.step([StepEntry("long", random_tokens(200, 512, 1), [])])
    for i in range(60):
        eng.step([StepEntry("long", [i % 512], [])])
    held_window = sum(1 for p_ in eng.cache.block_table("long", win_group) if p_ >= 0)
    held_full = sum(1 for p_ in eng.cache.block_table("long", full_group) if p_ >= 0)
    assert held_full == -(-260 // 16) and held_window <= -(-window // 16) + 1
    eng.cache.check_invariants()


# ---------------------------------------------------------------------------------------------
# A toy feed-forward with routing and a toy position encoding, both defined here and registered
# from outside the package: layer 0 keeps the dense feed-forward, layer 1 routes every token to
# one of three small experts; attention rotates only half of every head, with frequencies of its own.

def _register_toy_routed_ffn_and_position():
    from pytriton_llama_b200.parts import Part, TensorSpec, register_part

    @register_part("ffn", "toy_top1_experts")
    class ToyTop1Experts(Part):
        """y = p_e * W2_e relu(W1_e x) for the expert e with the largest router logit, p = softmax(logits)."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.hidden, self.inter, self.experts = spec.params["hidden"], spec.params["inter"], spec.params["experts"]

        def tensor_specs(self):
            return {"router": TensorSpec((self.experts, self.hidden)),
                    "w1": TensorSpec((self.experts * self.inter, self.hidden)),
                    "w2": TensorSpec((self.experts * self.hidden, self.inter))}

        def load(self, tensors):
            self.router = self._to_f32(tensors["router"])
            self.w1 = self._to_f32(tensors["w1"]).view(self.experts, self.inter, self.hidden)
            self.w2 = self._to_f32(tensors["w2"]).view(self.experts, self.hidden, self.inter)

        def forward(self, x):
            xf = x.float()
            logits = xf @ self.router.T                       # router logits in float32
            probs = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(xf[rows] @ self.w1[e].T) @ self.w2[e].T
                    out[rows] = probs[rows, e:e + 1] * h
            return out.to(x.dtype)

    @register_part("position", "toy_half_rotary")
    class ToyHalfRotary(Part):
        """Rotates the first half of every head only, with frequencies 0.3 / (j + 1)."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.rot = spec.params["head_dim"] // 2
            self.inv_freq = (0.3 / (torch.arange(self.rot // 2, dtype=torch.float32) + 1.0)).to(runtime.device)

        def rotary_table(self):
            return self.inv_freq, self.rot

        def apply(self, qk, positions, heads, head_dim):
            raise NotImplementedError


def _plain_routed_forward(cfg, w, tokens, experts, inter):
    """Float64, whole sequence, from the plain implementation's pieces."""
    tokens = torch.as_tensor(tokens)
    S = len(tokens)
    pos = torch.arange(S)
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = plain_llama.head_dim_of(cfg)
    rot = d // 2
    inv_freq = 0.3 / (torch.arange(rot // 2, dtype=torch.float32) + 1.0)
    cos, sin = plain_llama.rope_cos_sin(inv_freq, pos, torch.float64)      # [S, rot]

    def half_rotary(x):                                                    # x [S, heads, d]
        return torch.cat((plain_llama.apply_rope(x[..., :rot], cos, sin), x[..., rot:]), dim=-1)

    h = w["model.embed_tokens.weight"][tokens]
    eps = cfg["rms_norm_eps"]
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        x = plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        q = half_rotary((x @ w[p + "self_attn.q_proj.weight"].T).view(S, nq, d))
        k = half_rotary((x @ w[p + "self_attn.k_proj.weight"].T).view(S, nkv, d))
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(S, nkv, d)
        h = h + plain_llama.causal_gqa_attention(q, k, v).reshape(S, nq * d) @ w[p + "self_attn.o_proj.weight"].T
        x = plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        if layer == 1:
            logits = x @ w[p + "moe.router"].T
            probs = torch.softmax(logits, -1)
            choice = logits.argmax(-1)
            w1 = w[p + "moe.w1"].view(experts, inter, -1)
            w2 = w[p + "moe.w2"].view(experts, -1, inter)
            y = torch.stack([probs[t, choice[t]] * (w2[choice[t]] @ torch.relu(w1[choice[t]] @ x[t])) for t in range(S)])
        else:
            y = plain_llama.swiglu_ffn(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        h = h + y
    h = plain_llama.rms_norm(h, w["model.norm.weight"], eps)
    return h @ w.get("lm_head.weight", w["model.embed_tokens.weight"]).T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path, dtype):
    """Different feed-forwards in different layers, one of them with routing, and a position
    encoding the package does not have: registered here, built by the model's spec, stepped
    through the engine in mixed batches, compared with a plain float64 statement."""
    import traces
    from pytriton_llama_b200.config import EngineConfig, LlamaConfig, register_architecture
    from pytriton_llama_b200.engine.engine import Engine
    from pytriton_llama_b200.models.llama import llama_spec
    from pytriton_llama_b200.parts import PartSpec
    from pytriton_llama_b200.weights import read_folder, write_random_model
    _register_toy_routed_ffn_and_position()
    cfg = dict(TINY["B"], architectures=["ToyRoutedForCausalLM"], num_hidden_layers=2)
    experts, inter = 3, 48

    def spec(c, norm_init="ones"):
        sp = llama_spec(LlamaConfig.from_dict(cfg), norm_init="ones_jitter")
        for i, layer in enumerate(sp.layers):
            layer.parts["mixer"].parts["position"] = PartSpec("toy_half_rotary", {"head_dim": LlamaConfig.from_dict(cfg).head_dim})
            if i == 1:
                p = f"model.layers.{i}.moe."
                layer.parts["ffn"] = PartSpec("toy_top1_experts", {"hidden": cfg["hidden_size"], "inter": inter, "experts": experts},
                                              {"router": p + "router", "w1": p + "w1", "w2": p + "w2"})
        return sp

    register_architecture("ToyRoutedForCausalLM", LlamaConfig.from_dict, spec)
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_random_model(tmp_path / "routed", cfg, seed=9, dtype=stored, std=0.08)
    tensors = read_folder(folder)
    assert "model.layers.1.moe.router" in tensors and "model.layers.1.mlp.gate_proj.weight" not in tensors
    vocab = cfg["vocab_size"]
    eng = Engine(folder, EngineConfig(dtype=dtype, page_size=8, max_gpu_num_blocks=40, max_seq_len=160, max_num_seqs=3))
    seqs = {f"m{i}": random_tokens(n, vocab, 70 + i) for i, n in enumerate([37, 9, 70, 18])}
    w = {k: v.double() for k, v in tensors.items()}
    ref = {r: _plain_routed_forward(cfg, w, s, experts, inter) for r, s in seqs.items()}
    got = traces.replay(eng, traces.mixed(seqs, live=3))
    for r in seqs:
        assert_close(got[r], ref[r], dtype, r)


# ---------------------------------------------------------------------------------------------
# A position encoding that is no rotation of (j, j + rot/2) pairs: neighbouring elements
# (2j, 2j+1) are turned together.  The kernels cannot apply it from a table of frequencies, so the
# part says so (``rotary_table()`` is None) and the mixer calls its ``apply`` on q and k before the
# kernels store and attend.

def _register_toy_interleaved_rotary():
    from pytriton_llama_b200.parts import Part, register_part

    @register_part("position", "toy_interleaved_rotary")
    class ToyInterleavedRotary(Part):
        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            d = spec.params["head_dim"]
            self.inv_freq = (1.0 / (100.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(runtime.device)

        def rotary_table(self):
            return None

        def apply(self, qk, positions, heads, head_dim):
            ang = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            x = qk.unflatten(1, (heads, head_dim))             # a view of the projection's columns
            even, odd = x[..., 0::2].float(), x[..., 1::2].float()       # (views of x when it is float32: both results first)
            new_even, new_odd = (even * cos - odd * sin).to(qk.dtype), (odd * cos + even * sin).to(qk.dtype)
            x[..., 0::2] = new_even
            x[..., 1::2] = new_odd


def _plain_interleaved_forward(cfg, w, tokens):
    tokens = torch.as_tensor(tokens)
    S = len(tokens)
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = plain_llama.head_dim_of(cfg)
    inv_freq = 1.0 / (100.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = (torch.arange(S).float()[:, None] * inv_freq[None, :]).double()
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def turn(x):                                               # x [S, heads, d]
        out = torch.empty_like(x)
        out[..., 0::2] = x[..., 0::2] * cos - x[..., 1::2] * sin
        out[..., 1::2] = x[..., 1::2] * cos + x[..., 0::2] * sin
        return out

    h = w["model.embed_tokens.weight"][tokens]
    eps = cfg["rms_norm_eps"]
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        x = plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        q = turn((x @ w[p + "self_attn.q_proj.weight"].T).view(S, nq, d))
        k = turn((x @ w[p + "self_attn.k_proj.weight"].T).view(S, nkv, d))
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(S, nkv, d)
        h = h + plain_llama.causal_gqa_attention(q, k, v).reshape(S, nq * d) @ w[p + "self_attn.o_proj.weight"].T
        x = plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + plain_llama.swiglu_ffn(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    h = plain_llama.rms_norm(h, w["model.norm.weight"], eps)
    return h @ w.get("lm_head.weight", w["model.embed_tokens.weight"]).T


@pytest.mark.parametrize("dtype, name", [("float32", "B"), ("bfloat16", "D")])
def test_toy_position_encoding_that_the_kernels_cannot_apply(tmp_path, dtype, name):
    """Interleaved-pair rotary registered from here: the mixer hands q and k to the part's ``apply``
    and the kernels only store and attend -- prompts in portions, single tokens (in bfloat16 with
    head size 64 through the decode kernel that otherwise rotates itself) and captured graphs."""
    import traces
    from pytriton_llama_b200.config import EngineConfig, LlamaConfig, register_architecture
    from pytriton_llama_b200.engine.engine import Engine
    from pytriton_llama_b200.models.llama import llama_spec
    from pytriton_llama_b200.parts import PartSpec
    from pytriton_llama_b200.weights import read_folder, write_random_model
    _register_toy_interleaved_rotary()
    cfg = dict(TINY[name], architectures=["ToyInterleavedForCausalLM"])

    def spec(c, norm_init="ones"):
        sp = llama_spec(LlamaConfig.from_dict(cfg), norm_init="ones_jitter")
        for layer in sp.layers:
            layer.parts["mixer"].parts["position"] = PartSpec("toy_interleaved_rotary", {"head_dim": LlamaConfig.from_dict(cfg).head_dim})
        return sp

    register_architecture("ToyInterleavedForCausalLM", LlamaConfig.from_dict, spec)
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_random_model(tmp_path / "interleaved", cfg, seed=13, dtype=stored, std=0.08)
    w = {k: v.double() for k, v in read_folder(folder).items()}
    vocab = cfg["vocab_size"]
    seqs = {f"p{i}": random_tokens(n, vocab, 170 + i) for i, n in enumerate([37, 9, 150, 18])}
    ref = {r: _plain_interleaved_forward(cfg, w, s) for r, s in seqs.items()}
    for graphs in (False, True):
        eng = Engine(folder, EngineConfig(dtype=dtype, page_size=16, max_gpu_num_blocks=24, max_seq_len=256, max_num_seqs=3,
                                          compiled_model=graphs))
        got = traces.replay(eng, traces.mixed(seqs, live=3, decode_tail=12))
        for r in seqs:
            assert_close(got[r], ref[r], dtype, f"{r} graphs={graphs}")
        eng.check_device_status()
