"""Plain, slow Llama: whole sequences, no cache, one function per part, float64.

This file is the oracle of the test-suite.  It shares no code with the product
package: it has its own safetensors reader, its own config reader and its own
math.  It rests on the formulas of the reference (JustinA988/ferrum), cited by
the file's path within that project; the reference itself cannot be compiled
here (no Rust toolchain), so nothing in this file was checked against its
binaries.  Where the reference has no formula (llama3 rope scaling, temperature
sampling, the half-split pairing of HF checkpoints) the docstring says so.

All arithmetic is float64 on values that were rounded to the storage dtype, so
the result is "what exact arithmetic gives on these weights".
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# --------------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> float64 array.  Format: u64 header length, JSON header, raw bytes."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[lo:hi]
        dt = info["dtype"]
        if dt == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif dt == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = a.reshape(info["shape"])
    return out


def read_gguf(path):
    """(metadata dict, name -> float64 array) of a GGUF v2/v3 file with F32, F16 or BF16 tensors.

    The layout is the one the reference parses (crates/gguf/src/parse.rs:99-248): magic, version,
    tensor count, key/value count; key/values (string key, u32 type, value); tensor infos (name,
    n_dims, dims with the contiguous one first, ggml type, offset); padding to the alignment
    (`general.alignment`, default 32); data.  Own code: nothing of the product is used."""
    with open(path, "rb") as f:
        data = f.read()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, data, pos)
        pos += struct.calcsize(fmt)
        return v[0] if len(v) == 1 else v

    def string():
        nonlocal pos
        n = take("<Q")
        v = data[pos:pos + n].decode("utf-8")
        pos += n
        return v

    scalar = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}

    def value(t):
        if t == 8:
            return string()
        if t == 9:
            et, n = take("<I"), take("<Q")
            return [value(et) for _ in range(n)]
        v = take(scalar[t])
        return bool(v) if t == 7 else v

    assert data[:4] == b"GGUF"
    pos = 4
    version, n_tensors, n_kv = take("<I"), take("<Q"), take("<Q")
    assert version in (2, 3)
    meta = {}
    for _ in range(n_kv):
        k = string()
        meta[k] = value(take("<I"))
    infos = []
    for _ in range(n_tensors):
        name = string()
        nd = take("<I")
        dims = [take("<Q") for _ in range(nd)]
        infos.append((name, dims, take("<I"), take("<Q")))
    align = int(meta.get("general.alignment", 32))
    base = (pos + align - 1) // align * align
    out = {}
    for name, dims, typ, off in infos:
        n = int(np.prod(dims)) if dims else 1
        lo = base + off
        if typ == 0:
            a = np.frombuffer(data, dtype="<f4", count=n, offset=lo).astype(np.float64)
        elif typ == 1:
            a = np.frombuffer(data, dtype="<f2", count=n, offset=lo).astype(np.float64)
        elif typ == 30:
            u = np.frombuffer(data, dtype="<u2", count=n, offset=lo).astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        else:
            raise ValueError(f"plain reader: ggml type {typ} of {name}")
        out[name] = a.reshape(dims[::-1])          # the first dimension of the file is the contiguous one
    return meta, out


_GGUF_LAYER = {"attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
               "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "ffn_norm": "post_attention_layernorm",
               "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}


def read_gguf_model(path, weights_as="stored"):
    """(config dict with this file's own keys, weights under the names `forward` uses) of a GGUF
    Llama file: metadata keys of crates/core-types/src/model.rs:64-128, tensor names of :35-41.
    Rows of such a file are in the adjacent-pair order: call forward(..., pairing="adjacent")."""
    m, t = read_gguf(path)
    cfg = {"hidden_size": m["llama.embedding_length"], "num_hidden_layers": m["llama.block_count"],
           "num_attention_heads": m["llama.attention.head_count"],
           "num_key_value_heads": m.get("llama.attention.head_count_kv", m["llama.attention.head_count"]),
           "intermediate_size": m["llama.feed_forward_length"], "rms_norm_eps": m["llama.attention.layer_norm_rms_epsilon"],
           "rope_theta": m.get("llama.rope.freq_base", 10000.0)}
    if "llama.attention.key_length" in m:
        cfg["head_dim"] = m["llama.attention.key_length"]
    if m.get("llama.rope.scaling.type") == "llama3":
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": m["llama.rope.scaling.factor"],
                               "low_freq_factor": m["llama.rope.scaling.low_freq_factor"],
                               "high_freq_factor": m["llama.rope.scaling.high_freq_factor"],
                               "original_max_position_embeddings": m["llama.rope.scaling.original_context_length"]}
    w = {}
    for name, a in t.items():
        if name == "token_embd.weight":
            new = "model.embed_tokens.weight"
        elif name == "output_norm.weight":
            new = "model.norm.weight"
        elif name == "output.weight":
            new = "lm_head.weight"
        else:
            _, i, rest = name.split(".", 2)
            part, tail = rest.rsplit(".", 1)
            new = f"model.layers.{i}.{_GGUF_LAYER[part]}.{tail}"
        w[new] = round_as(a, weights_as) if (weights_as != "stored" and a.ndim == 2) else a
    return cfg, w


def round_bf16(a):
    """Round float64/float32 values to the nearest bfloat16 (ties to even)."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).astype(np.float64).reshape(f.shape)


def round_f16(a):
    """Round to the nearest IEEE half (ties to even), as crates/core-types/src/dtype.rs:135-154 reads them back."""
    return np.asarray(a, dtype=np.float64).astype(np.float16).astype(np.float64)


def round_as(a, kind):
    return {"bfloat16": round_bf16, "float16": round_f16}[kind](a)


def read_model(folder, weights_as="stored"):
    """(config dict, name -> float64 array) of a folder with config.json + model.safetensors.

    weights_as="bfloat16" (or "float16") rounds matrices (2-D tensors) to that type first,
    which is what an engine that computes in it holds; 1-D norm weights stay as stored.
    """
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    if weights_as != "stored":
        w = {k: (round_as(v, weights_as) if v.ndim == 2 else v) for k, v in w.items()}
    return cfg, w


# --------------------------------------------------------------------------- parts
def rms_norm(x, weight, eps):
    """out_i = x_i * (1/sqrt(mean(x^2)+eps)) * w_i  -- crates/kernels/src/scalar.rs:143-156."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x * (1.0 / np.sqrt(ms + eps)) * weight


def rope_inv_freq(cfg):
    """Per pair i in [0, R/2): theta^(-2i/R)  -- crates/kernels/src/math.rs:31-34
    (the reference divides pos by theta^(2i/R)).

    llama3 scaling is not in the reference (it rejects every scaling,
    crates/core-types/src/model.rs:82-88); the rule here is the published one for
    rope_type "llama3": wavelengths shorter than orig/high keep their frequency,
    longer than orig/low are divided by factor, and between them the two are blended.
    """
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    theta = float(cfg.get("rope_theta", 10000.0))
    i = np.arange(hd // 2, dtype=np.float64)
    f = theta ** (-2.0 * i / hd)
    rs = cfg.get("rope_scaling")
    if rs:
        kind = rs.get("rope_type", rs.get("type"))
        if kind != "llama3":
            raise ValueError(f"plain: rope scaling {kind}")
        factor = float(rs["factor"])
        low = float(rs["low_freq_factor"])
        high = float(rs["high_freq_factor"])
        orig = float(rs["original_max_position_embeddings"])
        out = np.empty_like(f)
        for k, fk in enumerate(f):
            wavelen = 2.0 * math.pi / fk
            if wavelen < orig / high:
                out[k] = fk
            elif wavelen > orig / low:
                out[k] = fk / factor
            else:
                s = (orig / wavelen - low) / (high - low)
                out[k] = (1.0 - s) * fk / factor + s * fk
        f = out
    return f


def rope(x, positions, inv_freq, pairing):
    """Rotate pairs of x [T, H, D] by angle pos*inv_freq[i].

    pairing "adjacent": pair i = (2i, 2i+1) -- crates/kernels/src/scalar.rs:167-189.
    pairing "half": pair i = (i, i + D/2): the order in which HF-named Llama
    checkpoints store q_proj/k_proj rows (the reference reads GGUF files only, whose
    rows were permuted to the adjacent order when they were converted).
    a' = a cos - b sin ; b' = a sin + b cos.
    """
    T, H, D = x.shape
    ang = positions.astype(np.float64)[:, None] * inv_freq[None, :]  # [T, D/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    if pairing == "adjacent":
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = a * s + b * c
    elif pairing == "half":
        a, b = x[..., : D // 2], x[..., D // 2:]
        out[..., : D // 2] = a * c - b * s
        out[..., D // 2:] = a * s + b * c
    else:
        raise ValueError(pairing)
    return out


def softmax(s):
    """exp(s - max) / sum  -- crates/kernels/src/scalar.rs:125-141."""
    m = np.max(s, axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def attention(q, k, v, window=0):
    """Causal grouped-query attention over a whole sequence.

    q [T, Hq, D], k, v [T, Hkv, D].  Query head h reads KV head h // (Hq/Hkv); score
    = q.k / sqrt(D) over positions 0..=pos -- crates/model/src/llama.rs:168-169,220-247.
    window > 0 keeps only the last `window` keys (pos-window, pos]; the reference has
    no window, the parameter exists for the part tests.
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    out = np.zeros_like(q)
    scale = 1.0 / math.sqrt(D)
    for h in range(Hq):
        kh = k[:, h // g, :]
        vh = v[:, h // g, :]
        s = (q[:, h, :] @ kh.T) * scale
        i = np.arange(T)
        mask = i[None, :] > i[:, None]
        if window > 0:
            mask |= i[None, :] <= i[:, None] - window
        s = np.where(mask, -np.inf, s)
        out[:, h, :] = softmax(s) @ vh
    return out


def silu(x):
    """x / (1 + exp(-x))  -- crates/kernels/src/math.rs:8-10."""
    return x / (1.0 + np.exp(-x))


def swiglu_ffn(x, w_gate, w_up, w_down):
    """down(silu(gate(x)) * up(x))  -- crates/model/src/llama.rs:261-283."""
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def attention_block(x, positions, w, prefix, cfg, inv_freq, pairing):
    """q,k,v projections, rope on q and k, attention, output projection
    -- crates/model/src/llama.rs:185-255."""
    T = x.shape[0]
    hq = cfg["num_attention_heads"]
    hkv = cfg.get("num_key_value_heads") or hq
    hd = cfg.get("head_dim") or cfg["hidden_size"] // hq
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).reshape(T, hq, hd)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).reshape(T, hkv, hd)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).reshape(T, hkv, hd)
    q = rope(q, positions, inv_freq, pairing)
    k = rope(k, positions, inv_freq, pairing)
    o = attention(q, k, v).reshape(T, hq * hd)
    return o @ w[prefix + "self_attn.o_proj.weight"].T


def forward(cfg, w, tokens, pairing="half"):
    """Logits [T, V] of a whole sequence -- crates/model/src/llama.rs:150-293.

    h = x + Attn(norm(x)); y = h + FFN(norm(h)); logits = W_out . norm(y).  The
    output matrix is lm_head.weight, or the embedding when the file has none
    (crates/model/src/llama.rs:103-111).
    """
    tokens = np.asarray(tokens, dtype=np.int64)
    eps = float(cfg["rms_norm_eps"])
    inv_freq = rope_inv_freq(cfg)
    positions = np.arange(len(tokens))
    h = w["model.embed_tokens.weight"][tokens]            # crates/model/src/weights.rs:29-51
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        n = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        h = h + attention_block(n, positions, w, p, cfg, inv_freq, pairing)
        n = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu_ffn(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
    n = rms_norm(h, w["model.norm.weight"], eps)
    out = w.get("lm_head.weight")
    if out is None:
        out = w["model.embed_tokens.weight"]
    return n @ out.T


# --------------------------------------------------------------------------- sampling
def argmax(row):
    """Lowest index wins ties, NaN skipped -- crates/core-types/src/model.rs:44-62."""
    best, best_i = -math.inf, None
    for i, v in enumerate(row):
        if v != v:
            continue
        if best_i is None or v > best:
            best, best_i = v, i
    if best_i is None:
        raise ValueError("logits are empty or all NaN")
    return best_i


def _mix32(x):
    """A 32-bit finaliser (two multiply-xorshift rounds); all arithmetic mod 2^32."""
    x = np.asarray(x, dtype=np.uint64) & 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x ^= x >> 15
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def gumbel_uniform(seed, counter, n):
    """u_i in (0,1) for i < n, a pure function of (seed, counter, i).

    Not in the reference (it samples greedily only).  key = mix(seed_lo ^ mix(seed_hi
    ^ mix(counter))); u_i = ((mix(key ^ mix(i)) >> 9) + 0.5) / 2^23, exact in float32 and never 0 or 1.
    """
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    key = _mix32((seed & 0xFFFFFFFF) ^ int(_mix32((seed >> 32) ^ int(_mix32(counter)))))
    i = np.arange(n, dtype=np.uint64)
    bits = _mix32(np.uint64(int(key)) ^ _mix32(i)) >> 9
    return (bits.astype(np.float64) + 0.5) / 8388608.0


def sample(row, temperature, seed, counter):
    """temperature 0: argmax.  Else the Gumbel-max draw from softmax(row / temperature):
    argmax_i(row_i / temperature - log(-log(u_i))), computed in float32 like the engine.
    `counter` is the number of tokens the request has generated before this one."""
    if temperature == 0.0:
        return argmax(row)
    row = np.asarray(row, dtype=np.float32)
    u = gumbel_uniform(seed, counter, len(row)).astype(np.float32)
    g = -np.log(-np.log(u))
    z = row * np.float32(1.0 / temperature) + g.astype(np.float32)
    return argmax(z.astype(np.float32))


def generate(cfg, w, prompt, max_new_tokens, temperature=0.0, seed=0, pairing="half",
             stop=(), eos=None):
    """Whole-sequence recompute per token; returns the generated ids.  The stopping
    token is emitted before generation ends -- crates/scheduler/src/batcher.rs:257-288."""
    toks = list(prompt)
    out = []
    for n in range(max_new_tokens):
        logits = forward(cfg, w, toks, pairing)[-1]
        t = sample(logits, temperature, seed, n)
        out.append(t)
        toks.append(t)
        if t in stop or (eos is not None and t == eos):
            break
    return out
