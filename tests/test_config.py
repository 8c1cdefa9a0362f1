"""Typed configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from ferrum_b200.config import LlamaConfig, registry
from ferrum_b200.errors import ConfigError


def test_reads_every_key_of_config_json():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.n_embd, c.n_layer, c.n_head, c.n_head_kv, c.head_dim, c.n_ff, c.n_vocab) == (96, 3, 3, 1, 32, 256, 512)
    assert c.rms_norm_eps == 1e-6 and c.rope_freq_base == 500000.0 and c.tie_word_embeddings
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.factor == 8.0
    assert c.rope_scaling.original_max_position_embeddings == 64 and c.rope_dim == 32
    assert c.q_width == 96 and c.kv_width == 32


def test_defaults_follow_the_reference():
    """head_dim = n_embd / n_head, kv heads = heads, theta 10000
    (crates/core-types/src/model.rs:94-114)."""
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "num_key_value_heads", "rope_theta")}
    c = LlamaConfig.from_dict(d)
    assert c.head_dim == 16 and c.n_head_kv == 4 and c.rope_freq_base == 10000.0 and c.rope_dim == 16


def test_round_trip_through_config_json(tmp_path):
    c = LlamaConfig.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    arch, c2 = registry.read_config(str(tmp_path))
    assert c2 == c and arch.name == "LlamaForCausalLM"


def test_a_list_of_end_tokens_is_kept_whole(tmp_path):
    """Llama-3 instruct files list several ids that end a sequence; every one of them is kept."""
    c = LlamaConfig.from_dict({**TINY_A, "eos_token_id": [200, 208, 209]})
    assert c.eos_token_ids == (200, 208, 209) and c.eos_token_id == 200
    assert LlamaConfig.from_dict(c.to_dict()) == c
    assert LlamaConfig.from_dict({**TINY_A, "eos_token_id": 7}).eos_token_ids == (7,)
    assert LlamaConfig.from_dict(TINY_A).eos_token_ids == ()
    with pytest.raises(ConfigError, match="vocab"):
        LlamaConfig.from_dict({**TINY_A, "eos_token_id": [3, 999]})
    with pytest.raises(ConfigError, match="eos_token_id"):
        LlamaConfig.from_dict({**TINY_A, "eos_token_id": ["x"]})


@pytest.mark.parametrize("change,msg", [
    ({"rms_norm_eps": 0.0}, "epsilon"), ({"rms_norm_eps": 1.5}, "epsilon"), ({"num_key_value_heads": 3}, "divisible"),
    ({"head_dim": 15}, "rope"), ({"rope_theta": -1.0}, "frequency"), ({"num_hidden_layers": 0}, "positive"),
    ({"attention_bias": True}, "bias"), ({"mlp_bias": True}, "bias"), ({"eos_token_id": 999}, "vocab"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0, "original_max_position_embeddings": 64}}, "rope scaling"),
    ({"rope_scaling": {"rope_type": "llama3"}}, "factor"),
])
def test_rejects_what_it_cannot_build(change, msg):
    with pytest.raises(ConfigError, match=msg):
        LlamaConfig.from_dict({**TINY_A, **change})


@pytest.mark.parametrize("missing", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                     "vocab_size", "max_position_embeddings", "rms_norm_eps"])
def test_required_keys(missing):
    d = {k: v for k, v in TINY_A.items() if k != missing}
    with pytest.raises(ConfigError, match=missing):
        LlamaConfig.from_dict(d)


def test_registry_names_and_unknown_architecture(tmp_path):
    assert "LlamaForCausalLM" in registry.names() and "llama" in registry.names()
    (tmp_path / "config.json").write_text(json.dumps({**TINY_A, "architectures": ["MambaForCausalLM"]}))
    with pytest.raises(ConfigError, match="unsupported architecture MambaForCausalLM"):
        registry.read_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        registry.read_config(str(tmp_path))


def test_gguf_metadata_reader_uses_the_reference_keys():
    """crates/core-types/src/model.rs:209-310 (its own unit test of defaults)."""
    meta = {"general.architecture": "llama", "llama.context_length": 32, "llama.embedding_length": 8,
            "llama.block_count": 2, "llama.attention.head_count": 2, "llama.feed_forward_length": 16,
            "llama.attention.layer_norm_rms_epsilon": 1e-5, "tokenizer.ggml.tokens": ["a", "b", "c"]}
    c = LlamaConfig.from_gguf_metadata(meta)
    assert (c.head_dim, c.rope_dim, c.rope_freq_base, c.n_head_kv, c.n_vocab) == (4, 4, 10000.0, 2, 3)
    assert c.rope_pairing == "adjacent"
    with pytest.raises(ConfigError, match="unsupported architecture"):
        LlamaConfig.from_gguf_metadata({**meta, "general.architecture": "gpt2"})
    with pytest.raises(ConfigError, match="mixture"):
        LlamaConfig.from_gguf_metadata({**meta, "llama.expert_count": 8})
    with pytest.raises(ConfigError, match="parallel residual"):
        LlamaConfig.from_gguf_metadata({**meta, "llama.use_parallel_residual": True})
    with pytest.raises(ConfigError, match="rope scaling"):
        LlamaConfig.from_gguf_metadata({**meta, "llama.rope.scaling.type": "linear"})


def test_another_rope_scaling_rule_is_one_registration():
    """The rotary part looks its scaling rule up by name; a rule it has never seen is registered
    from outside, and the part also takes ready-made frequencies."""
    from types import SimpleNamespace
    from ferrum_b200.parts import rope
    rope.register_scaling("halve_all", lambda f, block: [x / block.factor for x in f])
    try:
        block = SimpleNamespace(rope_type="halve_all", factor=2.0)
        base = rope.inverse_frequencies(8, 100.0)
        assert rope.inverse_frequencies(8, 100.0, block) == [x / 2.0 for x in base]
        rot = rope.RotaryEmbedding(8, 8, 100.0, block, "adjacent", 4, "cpu")
        given = rope.RotaryEmbedding(8, 8, 0.0, None, "adjacent", 4, "cpu", frequencies=[x / 2.0 for x in base])
        assert (rot.cos_sin == given.cos_sin).all()
    finally:
        rope.SCALINGS.pop("halve_all")
    with pytest.raises(ValueError, match="unsupported rope scaling halve_all"):
        rope.inverse_frequencies(8, 100.0, SimpleNamespace(rope_type="halve_all", factor=2.0))
