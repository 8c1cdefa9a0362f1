"""The Llama dense decoder, built from parts, and its entry in the registry.

Pre-norm RMSNorm, grouped-query attention with rotary encoding, SwiGLU feed-forward, tied or
untied output (crates/model/src/llama.rs).  Canonical tensor names are the reference's
(crates/core-types/src/model.rs:35-41; docs/ARCHITECTURE.md tensor table):
token_embd.weight, blk.{i}.attn_{norm,q,k,v,output}.weight, blk.{i}.ffn_{norm,gate,up,down}.weight,
output_norm.weight, output.weight.  `hf_names` maps the names of a config.json/safetensors
checkpoint onto them.
"""
from __future__ import annotations

import dataclasses

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register
from ..parts import OutputHead, PagedAttention, PreNormBlock, RMSNorm, RotaryEmbedding, SwiGLU, TokenEmbedding
from .decoder import DecoderModel


def build_llama(config: LlamaConfig, dtype, device, max_positions=None):
    c = config
    max_positions = int(max_positions or c.n_ctx_train)
    rope = RotaryEmbedding(c.head_dim, c.rope_dim, c.rope_freq_base, c.rope_scaling, c.rope_pairing,
                           max_positions, device)
    blocks = []
    for _ in range(c.n_layer):
        blocks.append(PreNormBlock(
            RMSNorm(c.n_embd, c.rms_norm_eps, dtype),
            PagedAttention(c.n_embd, c.n_head, c.n_head_kv, c.head_dim, rope, dtype),
            RMSNorm(c.n_embd, c.rms_norm_eps, dtype),
            SwiGLU(c.n_embd, c.n_ff, dtype)))
    emb = TokenEmbedding(c.n_vocab, c.n_embd)
    head = OutputHead(c.n_vocab, c.n_embd, tied_to=emb, tied=True if c.tie_word_embeddings else "auto")
    return DecoderModel(c, dtype, emb, None, blocks, RMSNorm(c.n_embd, c.rms_norm_eps, dtype), head)


_HF_LAYER = {
    "input_layernorm.weight": "attn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight",
    "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight",
    "self_attn.o_proj.weight": "attn_output.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight",
    "mlp.up_proj.weight": "ffn_up.weight",
    "mlp.down_proj.weight": "ffn_down.weight",
}


def hf_names(config: LlamaConfig):
    """{name in a HF-style safetensors file: canonical name}."""
    out = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
           "lm_head.weight": "output.weight"}
    for i in range(config.n_layer):
        for hf, ours in _HF_LAYER.items():
            out[f"model.layers.{i}.{hf}"] = f"blk.{i}.{ours}"
    return out


def read_gguf(gguf):
    """Typed config of an opened GGUF file.  A file without a tokenizer (random weights) gives
    its vocabulary through `llama.vocab_size` or the embedding's row count; the dtype recorded is
    the one the embedding is stored in."""
    emb = "token_embd.weight"
    have = emb in gguf.entries
    cfg = LlamaConfig.from_gguf_metadata(gguf.metadata, gguf.shape(emb)[0] if have else None)
    if have:
        stored = str(gguf.dtype(emb)).replace("torch.", "")
        cfg = dataclasses.replace(cfg, stored_dtype=stored)
    return cfg


register(Architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama, hf_names, read_gguf), "llama")
