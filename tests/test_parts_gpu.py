"""Each part alone, the run order as data, and parts that the framework has never seen:
a mixer with a state of its own, a routed feed-forward and an additive position encoding,
all defined here, registered, built and stepped without touching the package."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------- a minimal harness
class Harness:
    """A cache and a step context for a model made of arbitrary parts."""

    def __init__(self, model, dtype, max_tokens=256, page_size=8, max_requests=4):
        from ferrum_b200.cache import CacheStorage
        from ferrum_b200.engine import ModelRunner
        self.cache = CacheStorage(model, dtype, "cuda", page_size=page_size, max_tokens=max_tokens,
                                  max_requests=max_requests, max_model_len=max_tokens)
        self.runner = ModelRunner(model, self.cache, max_batch_tokens=max_tokens, max_batch_requests=max_requests)

    def run(self, cuts):
        """cuts: list of steps; a step is a list of (request key, tokens).  Returns
        {key: logits [n, V]} over everything fed."""
        from ferrum_b200.engine import StepEntry
        slots, rows = {}, {}
        for step in cuts:
            entries = []
            for key, toks in step:
                if key not in slots:
                    slots[key] = self.cache.open()
                entries.append(StepEntry(slots[key], self.cache.manager.seq_len(slots[key]), toks, range(len(toks))))
            out = self.runner.step(entries).float().cpu().numpy()
            k = 0
            for key, toks in step:
                rows.setdefault(key, []).append(out[k:k + len(toks)])
                k += len(toks)
        for s in slots.values():
            self.cache.close(s)
        return {k: np.concatenate(v) for k, v in rows.items()}


def cut(tokens, sizes):
    out, i, k = [], 0, 0
    while i < len(tokens):
        n = min(sizes[k % len(sizes)], len(tokens) - i)
        out.append(tokens[i:i + n])
        i += n
        k += 1
    return out


def build_llama_like(cfg_dict, dtype, **kw):
    from ferrum_b200.config import LlamaConfig
    from ferrum_b200.models.llama import build_llama
    from ferrum_b200.weights import init_random
    cfg = LlamaConfig.from_dict(cfg_dict)
    model = build_llama(cfg, dtype, "cuda", max_positions=256)
    return cfg, model


# ---------------------------------------------------------------- parts alone
def test_rotary_table_matches_plain(cuda):
    from conftest import TINY_B
    from ferrum_b200.config import LlamaConfig
    from ferrum_b200.parts import RotaryEmbedding
    c = LlamaConfig.from_dict(TINY_B)
    rot = RotaryEmbedding(c.head_dim, c.rope_dim, c.rope_freq_base, c.rope_scaling, "half", 200, "cuda")
    ang = np.arange(200)[:, None] * P.rope_inv_freq(TINY_B)[None, :]
    table = rot.cos_sin.cpu().numpy()
    assert table.shape == (200, 16, 2)
    assert np.abs(table[..., 0] - np.cos(ang)).max() < 1e-7 and np.abs(table[..., 1] - np.sin(ang)).max() < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_feed_forward_parts(cuda, dtype):
    """RMSNorm and SwiGLU as parts, with sizes no model here uses (width 136, hidden 344)."""
    from ferrum_b200.engine.batch import StepContext, StepEntry
    from ferrum_b200.parts import RMSNorm, SwiGLU
    g = torch.Generator(device="cuda").manual_seed(0)
    E, F, T = 136, 344, 19
    norm, ffn = RMSNorm(E, 3e-5, dtype), SwiGLU(E, F, dtype)
    norm.assign("weight", 1 + 0.1 * torch.randn(E, device="cuda", generator=g))
    for n, shape in (("gate.weight", (F, E)), ("up.weight", (F, E)), ("down.weight", (E, F))):
        ffn.assign(n, (torch.randn(shape, device="cuda", generator=g) * 0.1).to(dtype))
    ffn.finalize()
    ctx = StepContext("cuda", 64, 2, [])
    ctx.fill([StepEntry(0, 0, list(range(T)))], [])
    h = torch.randn(T, E, device="cuda", generator=g)
    x = norm.forward(h, ctx)
    ref_x = P.rms_norm(h.double().cpu().numpy(), norm.w_weight.double().cpu().numpy(), 3e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(x[:T].double().cpu().numpy() - ref_x).max() <= tol
    res = h.clone()
    ffn.forward(x, ctx, res)
    ctx.flush_residual()           # the residual sum may be left for the next norm; ask for it now
    wgu = ffn.w_gate_up.double().cpu().numpy()
    xin = x[:T].double().cpu().numpy()
    ref = h.double().cpu().numpy() + P.swiglu_ffn(xin, wgu[:F], wgu[F:], ffn.w_down_weight.double().cpu().numpy())
    assert np.abs(res.double().cpu().numpy() - ref).max() <= (1e-4 if dtype == torch.float32 else 3e-2)
    assert ctx.err.item() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,head_dim", [(0, 64), (24, 64), (24, 16)])
def test_attention_part_with_and_without_window(cuda, dtype, window, head_dim):
    """The attention mixer alone inside a one-block model whose other parts are identities is
    hard to isolate; instead a whole tiny model with a windowed mixer is compared with the
    plain implementation given the same window."""
    from conftest import TINY_D
    from ferrum_b200.weights import init_random
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    cfg_d = dict(TINY_D, head_dim=head_dim, num_hidden_layers=1)
    cfg, model = build_llama_like(cfg_d, td)
    for b in model.blocks:
        b.mixer.window = window
    init_random(model, 7)
    toks = np.random.default_rng(3).integers(0, cfg.n_vocab, 90).tolist()
    got = Harness(model, td).run([[("a", part)] for part in cut(toks, [40, 1, 1, 7, 1, 30, 2])])["a"]
    w = export_hf(model, cfg)
    ref = plain_forward_window(cfg_d, w, toks, window)
    tol = 2e-4 if dtype == "float32" else 0.06
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


def export_hf(model, cfg):
    """The model's weights under checkpoint names, as float64 (rounded as the model holds them)."""
    from ferrum_b200.models.llama import hf_names
    back = {v: k for k, v in hf_names(cfg).items()}
    out = {}
    Hq, Hkv, D, F = cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.n_ff
    for i, b in enumerate(model.blocks):
        qkv = b.mixer.w_qkv.double().cpu().numpy()
        gu = b.ffn.w_gate_up.double().cpu().numpy()
        p = f"model.layers.{i}."
        out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"] = qkv[:Hq * D], qkv[Hq * D:(Hq + Hkv) * D]
        out[p + "self_attn.v_proj.weight"] = qkv[(Hq + Hkv) * D:]
        out[p + "self_attn.o_proj.weight"] = b.mixer.w_output_weight.double().cpu().numpy()
        out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = gu[:F], gu[F:]
        out[p + "mlp.down_proj.weight"] = b.ffn.w_down_weight.double().cpu().numpy()
        out[p + "input_layernorm.weight"] = b.norm1.w_weight.double().cpu().numpy()
        out[p + "post_attention_layernorm.weight"] = b.norm2.w_weight.double().cpu().numpy()
    out["model.embed_tokens.weight"] = model.embedding.w_weight.double().cpu().numpy()
    out["model.norm.weight"] = model.final_norm.w_weight.double().cpu().numpy()
    if model.head.w_weight is not model.embedding.w_weight:
        out["lm_head.weight"] = model.head.w_weight.double().cpu().numpy()
    return out


def plain_forward_window(cfg, w, tokens, window, schedule=None):
    """plain_llama.forward with a window in every attention and an optional run order
    [(layer, cache_of)], written out here from the plain parts."""
    tokens = np.asarray(tokens)
    eps, inv = float(cfg["rms_norm_eps"]), P.rope_inv_freq(cfg)
    pos = np.arange(len(tokens))
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg["head_dim"]
    T = len(tokens)
    h = w["model.embed_tokens.weight"][tokens]
    schedule = schedule or [(i, None) for i in range(cfg["num_hidden_layers"])]
    kv = {}
    for k_run, (i, cache_of) in enumerate(schedule):
        p = f"model.layers.{i}."
        n = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        q = P.rope((n @ w[p + "self_attn.q_proj.weight"].T).reshape(T, hq, hd), pos, inv, "half")
        if cache_of is None:
            k = P.rope((n @ w[p + "self_attn.k_proj.weight"].T).reshape(T, hkv, hd), pos, inv, "half")
            v = (n @ w[p + "self_attn.v_proj.weight"].T).reshape(T, hkv, hd)
            kv[k_run] = (k, v)
        else:
            k, v = kv[cache_of]
        h = h + P.attention(q, k, v, window).reshape(T, hq * hd) @ w[p + "self_attn.o_proj.weight"].T
        n = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + P.swiglu_ffn(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    out = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return P.rms_norm(h, w["model.norm.weight"], eps) @ out.T


# ---------------------------------------------------------------- the run order is data
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_names_a_layer_twice_and_shares_a_cache(cuda, dtype):
    """Run order [0, 1, 0 again (own cache), 1 reading the cache of its first run]."""
    from conftest import TINY_D
    from ferrum_b200.models import Run
    from ferrum_b200.weights import init_random
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    cfg, model = build_llama_like(TINY_D, td)
    model.schedule = [Run(0), Run(1), Run(0), Run(1, cache_of=1)]
    init_random(model, 9)
    toks = np.random.default_rng(4).integers(0, cfg.n_vocab, 70).tolist()
    h = Harness(model, td)
    assert h.cache.layout.group_planes == [3] and h.cache.layout.run_plane == [0, 1, 2, 1]
    got = h.run([[("a", part)] for part in cut(toks, [33, 1, 1, 5, 2, 1])])["a"]
    ref = plain_forward_window(TINY_D, export_hf(model, cfg), toks, 0, [(0, None), (1, None), (0, None), (1, 1)])
    tol = 2e-4 if dtype == "float32" else 0.06
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


def test_layers_with_different_mixers_get_cache_groups_of_their_own(cuda):
    """A windowed layer beside a full one: two groups, two block tables, and the windowed
    group hands pages back while the request still runs."""
    from conftest import TINY_D
    from ferrum_b200.weights import init_random
    cfg, model = build_llama_like(TINY_D, torch.float32)
    model.blocks[1].mixer.window = 16
    init_random(model, 11)
    toks = np.random.default_rng(5).integers(0, cfg.n_vocab, 120).tolist()
    h = Harness(model, torch.float32, max_tokens=128, page_size=8)
    assert len(h.cache.pools) == 2 and h.cache.layout.run_group == [0, 1]
    from ferrum_b200.engine import StepEntry
    slot = h.cache.open()
    outs, fed = [], 0
    for part in cut(toks, [50, 1, 1, 20, 3, 1]):
        outs.append(h.runner.step([StepEntry(slot, fed, part, range(len(part)))]).float().cpu().numpy())
        fed += len(part)
        assert h.cache.manager.pages_held(1, slot) <= 16 // 8 + 1 + 1       # the window's pages only
        assert h.cache.manager.pages_held(0, slot) == (fed + 7) // 8
    got = np.concatenate(outs)
    w = export_hf(model, cfg)
    # plain: layer 0 full, layer 1 windowed
    ref = plain_two_windows(TINY_D, w, toks, [0, 16])
    assert np.abs(got - ref).max() <= 2e-4 * max(1.0, np.abs(ref).max())


def plain_two_windows(cfg, w, tokens, windows):
    tokens = np.asarray(tokens)
    eps, inv, pos, T = float(cfg["rms_norm_eps"]), P.rope_inv_freq(cfg), np.arange(len(tokens)), len(tokens)
    hq, hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    h = w["model.embed_tokens.weight"][tokens]
    for i, win in enumerate(windows):
        p = f"model.layers.{i}."
        n = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        q = P.rope((n @ w[p + "self_attn.q_proj.weight"].T).reshape(T, hq, hd), pos, inv, "half")
        k = P.rope((n @ w[p + "self_attn.k_proj.weight"].T).reshape(T, hkv, hd), pos, inv, "half")
        v = (n @ w[p + "self_attn.v_proj.weight"].T).reshape(T, hkv, hd)
        h = h + P.attention(q, k, v, win).reshape(T, hq * hd) @ w[p + "self_attn.o_proj.weight"].T
        n = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + P.swiglu_ffn(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.rms_norm(h, w["model.norm.weight"], eps) @ w.get("lm_head.weight", w["model.embed_tokens.weight"]).T


# ---------------------------------------------------------------- parts the framework has never seen
def make_toy_architecture():
    """Registers "ToyForCausalLM": blocks of (RMSNorm, EMA mixer with a per-request state,
    RMSNorm, top-1 routed feed-forward), learned absolute positions added to the embedding.
    Everything toy is written with torch ops on the tensors the interfaces hand over."""
    from ferrum_b200.config import registry
    from ferrum_b200.models import DecoderModel
    from ferrum_b200.parts import (CacheNeed, FeedForward, Mixer, OutputHead, ParamSpec, PositionEncoding,
                                   PreNormBlock, RMSNorm, StateNeed, TokenEmbedding)

    class EmaMixer(Mixer):
        """s_t = a * s_{t-1} + (1 - a) * (W x_t); output s_t.  The state s lives in the
        request's slot of a [max_requests, width] array."""

        def __init__(self, width, decay):
            self.width, self.decay = width, decay

        def param_specs(self):
            return {"in.weight": ParamSpec((self.width, self.width))}

        def cache_need(self):
            return CacheNeed(state=StateNeed((self.width,), torch.float32))

        def forward(self, x, ctx, cache, residual):
            W = self.w_in_weight.float()
            for r in range(ctx.n_reqs):
                t0, n, slot = ctx.h_q_start[r], ctx.h_q_len[r], ctx.h_slots[r]
                u = x[t0:t0 + n].float() @ W.T
                s = cache.state[slot]
                for i in range(n):
                    s = self.decay * s + (1 - self.decay) * u[i]
                    residual[t0 + i] += s
                cache.state[slot] = s

    class RoutedFFN(FeedForward):
        """Two experts, the token goes to argmax(router x)."""

        def __init__(self, width, hidden):
            self.width, self.hidden = width, hidden

        def param_specs(self):
            return {"router.weight": ParamSpec((2, self.width), kind="vector"),
                    "up.weight": ParamSpec((2 * self.hidden, self.width)),
                    "down.weight": ParamSpec((2 * self.width, self.hidden))}

        def forward(self, x, ctx, residual):
            T = ctx.n_tokens
            xf = x[:T].float()
            choice = (xf @ self.w_router_weight.T).argmax(-1)
            up = self.w_up_weight.float().view(2, self.hidden, self.width)
            down = self.w_down_weight.float().view(2, self.width, self.hidden)
            for e in range(2):
                m = choice == e
                if m.any():
                    residual[:T][m] += torch.relu(xf[m] @ up[e].T) @ down[e].T

    class LearnedPositions(PositionEncoding):
        def __init__(self, n_pos, width):
            self.n_pos, self.width = n_pos, width

        def param_specs(self):
            return {"weight": ParamSpec((self.n_pos, self.width), kind="vector")}

        def on_embedding(self, h, ctx):
            h[:ctx.n_tokens] += self.w_weight[ctx.positions.long()]

    class ToyConfig:
        def __init__(self, d):
            self.n_vocab, self.n_embd, self.n_layer = d["vocab_size"], d["hidden_size"], d["num_hidden_layers"]
            self.hidden, self.decay, self.eps, self.n_pos = d["expert_hidden"], d["decay"], d["eps"], d["positions"]
            self.eos_token_id = None
            # layers named here mix by the framework's own paged attention instead: (heads, kv heads, head size)
            self.attention_layers = {int(k): tuple(v) for k, v in d.get("attention_layers", {}).items()}

    def build(cfg, dtype, device, max_positions=None):
        from ferrum_b200.parts import PagedAttention, RotaryEmbedding
        blocks = []
        for i in range(cfg.n_layer):
            if i in cfg.attention_layers:      # the mixer is chosen layer by layer
                hq, hkv, hd = cfg.attention_layers[i]
                rope = RotaryEmbedding(hd, hd, 10000.0, None, "adjacent", cfg.n_pos, device)
                mixer, name = PagedAttention(cfg.n_embd, hq, hkv, hd, rope, dtype), "attn_"
            else:
                mixer, name = EmaMixer(cfg.n_embd, cfg.decay), "ema_"
            blocks.append(PreNormBlock(RMSNorm(cfg.n_embd, cfg.eps, dtype), mixer, RMSNorm(cfg.n_embd, cfg.eps, dtype),
                                       RoutedFFN(cfg.n_embd, cfg.hidden), names=("norm_a.", name, "norm_b.", "moe_")))
        emb = TokenEmbedding(cfg.n_vocab, cfg.n_embd)
        return DecoderModel(cfg, dtype, emb, LearnedPositions(cfg.n_pos, cfg.n_embd), blocks,
                            RMSNorm(cfg.n_embd, cfg.eps, dtype), OutputHead(cfg.n_vocab, cfg.n_embd, emb, tied=True))

    registry.register(registry.Architecture("ToyForCausalLM", ToyConfig, build))
    return registry


def toy_reference(model, cfg, tokens):
    """Whole-sequence float64 computation of the toy model."""
    f = lambda t: t.double().cpu().numpy()
    tokens = np.asarray(tokens)
    h = f(model.embedding.w_weight)[tokens] + f(model.position.w_weight)[np.arange(len(tokens))]
    for b in model.blocks:
        x = P.rms_norm(h, f(b.norm1.w_weight), cfg.eps)
        if model.dtype == torch.bfloat16:
            x = P.round_bf16(x)
        u = x @ f(b.mixer.w_in_weight).T
        s = np.zeros(cfg.n_embd)
        for t in range(len(tokens)):
            s = np.float32(cfg.decay) * s + (1 - np.float32(cfg.decay)) * u[t]
            h[t] = h[t] + s
        x = P.rms_norm(h, f(b.norm2.w_weight), cfg.eps)
        if model.dtype == torch.bfloat16:
            x = P.round_bf16(x)
        choice = (x @ f(b.ffn.w_router_weight).T).argmax(-1)
        up = f(b.ffn.w_up_weight).reshape(2, cfg.hidden, cfg.n_embd)
        down = f(b.ffn.w_down_weight).reshape(2, cfg.n_embd, cfg.hidden)
        for t in range(len(tokens)):
            e = choice[t]
            h[t] = h[t] + np.maximum(x[t] @ up[e].T, 0) @ down[e].T
    return P.rms_norm(h, f(model.final_norm.w_weight), cfg.eps) @ f(model.embedding.w_weight).T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_architecture_is_registered_built_and_stepped(cuda, dtype, tmp_path):
    import json
    from ferrum_b200.weights import init_random
    registry = make_toy_architecture()
    try:
        d = {"architectures": ["ToyForCausalLM"], "vocab_size": 97, "hidden_size": 40, "num_hidden_layers": 2,
             "expert_hidden": 56, "decay": 0.75, "eps": 1e-5, "positions": 128}
        (tmp_path / "config.json").write_text(json.dumps(d))
        arch, cfg = registry.read_config(str(tmp_path))
        model = arch.build(cfg, dtype, "cuda")
        assert "blk.1.ema_in.weight" in model.weight_specs() and "position.weight" in model.weight_specs()
        init_random(model, 13)
        rng = np.random.default_rng(6)
        ta, tb = rng.integers(0, 97, 50).tolist(), rng.integers(0, 97, 31).tolist()
        h = Harness(model, dtype)
        assert h.cache.pools == [] and len(h.cache.states) == 2 and h.cache.states[0].shape == (4, 40)
        # two requests interleaved, cut anywhere: the state must follow each request
        pa, pb = cut(ta, [7, 1, 1, 20, 2]), cut(tb, [1, 13, 1, 1])
        steps = []
        for i in range(max(len(pa), len(pb))):
            steps.append([(k, p[i]) for k, p in (("a", pa), ("b", pb)) if i < len(p)])
        got = h.run(steps)
        tol = 1e-4 if dtype == torch.float32 else 0.05
        for key, toks in (("a", ta), ("b", tb)):
            ref = toy_reference(model, cfg, toks)
            assert np.abs(got[key] - ref).max() <= tol * max(1.0, np.abs(ref).max()), key
        # a slot that is used again starts from a zero state
        again = h.run([[("c", ta)]])["c"]
        assert np.abs(again - got["a"]).max() <= tol
    finally:
        registry.unregister("ToyForCausalLM")


def test_engine_over_state_and_pages_with_preemption(cuda):
    """The Python entry point over a model the framework has never seen: layer 0 mixes by the toy
    EMA recurrence (a state per request), layer 1 by the framework's paged attention (pages), the
    feed-forwards are routed.  With so few pages that two decoding requests cannot both stay, one
    is preempted: its pages AND its state are dropped, it is recomputed from its first token, and
    both requests still generate exactly what they generate alone."""
    from ferrum_b200 import Engine
    from ferrum_b200.weights import init_random
    registry = make_toy_architecture()
    try:
        d = {"architectures": ["ToyForCausalLM"], "vocab_size": 97, "hidden_size": 48, "num_hidden_layers": 2,
             "expert_hidden": 56, "decay": 0.75, "eps": 1e-5, "positions": 128, "attention_layers": {"1": [3, 1, 16]}}
        arch = registry.lookup("ToyForCausalLM")
        cfg = arch.read_config(d)
        model = arch.build(cfg, torch.float32, "cuda")
        assert "blk.0.ema_in.weight" in model.weight_specs() and "blk.1.attn_q.weight" in model.weight_specs()
        init_random(model, 17)
        rng = np.random.default_rng(8)
        prompts = [rng.integers(0, 97, 20).tolist(), rng.integers(0, 97, 20).tolist()]

        def engine(**kw):
            args = dict(model=model, page_size=16, num_pages=64, max_batch_tokens=64, max_batch_seqs=4, max_model_len=64)
            args.update(kw)
            return Engine(**args)

        roomy = engine()
        assert len(roomy.cache.states) == 1 and roomy.cache.n_groups == 1
        alone = [roomy.generate([p], max_new_tokens=40)[0] for p in prompts]
        assert all(len(a) == 40 for a in alone) and alone[0] != alone[1]
        tight = engine(num_pages=6)                       # 96 positions of cache, 120 needed
        assert tight.generate(prompts, max_new_tokens=40) == alone
        st = tight.stats()
        assert st["preemptions"] >= 1 and st["pages_used"] == [0] and st["active"] == 0
        # in portions of 8 tokens with a budget of 12 a step, prompts and decoded tokens share steps
        chunked = engine(chunk_size=8, max_batch_tokens=12)
        assert chunked.generate(prompts, max_new_tokens=40) == alone
    finally:
        registry.unregister("ToyForCausalLM")
