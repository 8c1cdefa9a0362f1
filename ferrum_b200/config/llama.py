"""Typed configuration of the Llama dense decoder.

The fields are the reference's `LlamaConfig` (crates/core-types/src/model.rs:17-33)
plus what the reference rejects but this engine builds: llama3 rope scaling and a
tied-output flag.  Two readers fill the same struct: `from_config_json` (the
architecture's own config.json keys) and `from_gguf_metadata` (the keys and defaults
of crates/core-types/src/model.rs:64-185).  No size or constant that the file gives
is repeated anywhere else in the package.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Optional, Tuple

from ..errors import ConfigError


@dataclass(frozen=True)
class RopeScaling:
    """rope_type "llama3": frequencies of long wavelengths are divided by `factor`,
    with a linear blend between original/high_freq_factor and original/low_freq_factor."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    n_vocab: int
    n_embd: int
    n_layer: int
    n_head: int
    n_head_kv: int
    head_dim: int
    n_ff: int
    n_ctx_train: int
    rms_norm_eps: float
    rope_freq_base: float = 10000.0
    rope_dim: int = 0                      # 0 -> head_dim
    rope_scaling: Optional[RopeScaling] = None
    rope_pairing: str = "half"             # "half": (i, i+R/2) HF order; "adjacent": (2i, 2i+1) GGUF order
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None     # the first of eos_token_ids
    eos_token_ids: Tuple[int, ...] = ()    # every id that ends a sequence (config.json may list several)
    stored_dtype: str = "float32"
    name: str = ""
    extra: dict = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ checks
    def __post_init__(self):
        if self.rope_dim == 0:
            object.__setattr__(self, "rope_dim", self.head_dim)
        ids = tuple(int(t) for t in self.eos_token_ids)
        if not ids and self.eos_token_id is not None:
            ids = (int(self.eos_token_id),)
        object.__setattr__(self, "eos_token_ids", ids)
        object.__setattr__(self, "eos_token_id", ids[0] if ids else None)
        self.validate()

    def validate(self):
        """The cross-checks of crates/core-types/src/model.rs:130-166, minus the rule
        n_embd == n_head*head_dim: the query width n_head*head_dim is its own size here."""
        counts = dict(n_vocab=self.n_vocab, n_embd=self.n_embd, n_layer=self.n_layer,
                      n_head=self.n_head, n_head_kv=self.n_head_kv, n_ff=self.n_ff,
                      n_ctx_train=self.n_ctx_train, head_dim=self.head_dim, rope_dim=self.rope_dim)
        for k, v in counts.items():
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"llama hyperparameter {k} must be a positive integer, found {v!r}")
        if self.n_head % self.n_head_kv:
            raise ConfigError("head count is not divisible by kv head count")
        if self.head_dim % 2 or self.rope_dim % 2 or self.rope_dim > self.head_dim:
            raise ConfigError("invalid rope dimension")
        if not (math.isfinite(self.rms_norm_eps) and 0.0 < self.rms_norm_eps < 1.0):
            raise ConfigError("invalid rms norm epsilon")
        if not (math.isfinite(self.rope_freq_base) and self.rope_freq_base > 0.0):
            raise ConfigError("invalid rope frequency base")
        if self.rope_pairing not in ("half", "adjacent"):
            raise ConfigError(f"unknown rope pairing {self.rope_pairing!r}")
        for v in (self.bos_token_id,) + self.eos_token_ids:
            if v is not None and not (0 <= v < self.n_vocab):
                raise ConfigError("special token id is outside the vocab")
        rs = self.rope_scaling
        if rs is not None:
            if rs.rope_type != "llama3":
                raise ConfigError(f"unsupported rope scaling {rs.rope_type}")
            if not (rs.factor >= 1.0 and rs.high_freq_factor > rs.low_freq_factor > 0.0
                    and rs.original_max_position_embeddings > 0):
                raise ConfigError("invalid llama3 rope scaling parameters")

    # ------------------------------------------------------------------ readers
    @staticmethod
    def from_dict(d: dict) -> "LlamaConfig":
        """Read the keys of a Llama config.json."""
        archs = d.get("architectures") or []
        if not archs:
            raise ConfigError("config.json has no 'architectures'")

        def need(key):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: missing required key {key!r}")
            return d[key]

        if d.get("attention_bias") or d.get("mlp_bias"):
            # the reference refuses every bias tensor: crates/model/src/weights.rs:165-167
            raise ConfigError("bias terms are not supported")
        n_embd = int(need("hidden_size"))
        n_head = int(need("num_attention_heads"))
        n_head_kv = d.get("num_key_value_heads")
        n_head_kv = n_head if n_head_kv is None else int(n_head_kv)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if n_head <= 0 or n_embd % n_head:
                raise ConfigError("embedding length is not divisible by head count")
            head_dim = n_embd // n_head
        rs = d.get("rope_scaling")
        scaling = None
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            if kind not in (None, "default", "none"):
                try:
                    scaling = RopeScaling(
                        rope_type=str(kind), factor=float(rs["factor"]),
                        low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                        high_freq_factor=float(rs.get("high_freq_factor", 4.0)),
                        original_max_position_embeddings=int(rs["original_max_position_embeddings"]))
                except KeyError as e:
                    raise ConfigError(f"rope_scaling: missing key {e.args[0]!r}") from None
        known = {"architectures", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                 "num_hidden_layers", "intermediate_size", "vocab_size", "max_position_embeddings",
                 "rms_norm_eps", "rope_theta", "rope_scaling", "tie_word_embeddings", "bos_token_id",
                 "eos_token_id", "torch_dtype", "dtype", "attention_bias", "mlp_bias", "rope_pairing",
                 "partial_rotary_dim", "model_type", "_name_or_path"}
        eos = d.get("eos_token_id")
        try:
            eos_ids = tuple(int(t) for t in eos) if isinstance(eos, (list, tuple)) else (() if eos is None else (int(eos),))
        except (TypeError, ValueError):
            raise ConfigError(f"config.json: eos_token_id must be an integer or a list of integers, found {eos!r}") from None
        return LlamaConfig(
            architecture=str(archs[0]),
            n_vocab=int(need("vocab_size")), n_embd=n_embd, n_layer=int(need("num_hidden_layers")),
            n_head=n_head, n_head_kv=n_head_kv, head_dim=int(head_dim),
            n_ff=int(need("intermediate_size")),
            n_ctx_train=int(need("max_position_embeddings")),
            rms_norm_eps=float(need("rms_norm_eps")),
            rope_freq_base=float(d.get("rope_theta", 10000.0)),
            rope_dim=int(d.get("partial_rotary_dim") or 0),
            rope_scaling=scaling,
            rope_pairing=str(d.get("rope_pairing", "half")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            bos_token_id=d.get("bos_token_id"), eos_token_ids=eos_ids,
            stored_dtype=str(d.get("torch_dtype") or d.get("dtype") or "float32"),
            name=str(d.get("_name_or_path", "")),
            extra={k: v for k, v in d.items() if k not in known})

    @staticmethod
    def from_config_json(path: str) -> "LlamaConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        try:
            with open(path) as f:
                d = json.load(f)
        except (OSError, ValueError) as e:
            raise ConfigError(f"cannot read {path}: {e}") from None
        if not isinstance(d, dict):
            raise ConfigError(f"{path}: not a JSON object")
        return LlamaConfig.from_dict(d)

    @staticmethod
    def from_gguf_metadata(meta: dict, n_vocab_from_tensor: Optional[int] = None, stored_dtype: str = "float32") -> "LlamaConfig":
        """GGUF keys and defaults of crates/core-types/src/model.rs:64-185.  Differences:
        a `llama3` scaling block is read instead of refused, and the vocabulary size
        may come from `llama.vocab_size` or the embedding tensor when the file carries
        no tokenizer (requests arrive as token ids here)."""
        arch = meta.get("general.architecture")
        if arch != "llama":
            raise ConfigError(f"unsupported architecture {arch}")
        if meta.get("llama.use_parallel_residual") is True:
            raise ConfigError("parallel residual is not supported")
        if meta.get("llama.expert_count", 0) not in (0, None):
            raise ConfigError("mixture-of-experts is not supported")

        def need(key):
            if key not in meta:
                raise ConfigError(f"missing metadata key {key}")
            return meta[key]

        n_embd = int(need("llama.embedding_length"))
        n_head = int(need("llama.attention.head_count"))
        head_dim = meta.get("llama.attention.key_length")
        if head_dim is None:
            if n_head <= 0 or n_embd % n_head:
                raise ConfigError("embedding length is not divisible by head count")
            head_dim = n_embd // n_head
        vlen = meta.get("llama.attention.value_length")
        if vlen is not None and int(vlen) != int(head_dim):
            raise ConfigError("separate value head length is not supported")
        scaling = None
        kind = meta.get("llama.rope.scaling.type")
        if kind not in (None, "none"):
            if kind != "llama3":
                raise ConfigError(f"unsupported rope scaling {kind}")
            scaling = RopeScaling(
                rope_type="llama3", factor=float(need("llama.rope.scaling.factor")),
                low_freq_factor=float(meta.get("llama.rope.scaling.low_freq_factor", 1.0)),
                high_freq_factor=float(meta.get("llama.rope.scaling.high_freq_factor", 4.0)),
                original_max_position_embeddings=int(need("llama.rope.scaling.original_context_length")))
        if "tokenizer.ggml.tokens" in meta:
            n_vocab = len(meta["tokenizer.ggml.tokens"])
        elif "llama.vocab_size" in meta:
            n_vocab = int(meta["llama.vocab_size"])
        elif n_vocab_from_tensor is not None:
            n_vocab = int(n_vocab_from_tensor)
        else:
            raise ConfigError("missing metadata key tokenizer.ggml.tokens")
        return LlamaConfig(
            architecture="llama", n_vocab=n_vocab, n_embd=n_embd,
            n_layer=int(need("llama.block_count")), n_head=n_head,
            n_head_kv=int(meta.get("llama.attention.head_count_kv", n_head)),
            head_dim=int(head_dim), n_ff=int(need("llama.feed_forward_length")),
            n_ctx_train=int(need("llama.context_length")),
            rms_norm_eps=float(need("llama.attention.layer_norm_rms_epsilon")),
            rope_freq_base=float(meta.get("llama.rope.freq_base", 10000.0)),
            rope_dim=int(meta.get("llama.rope.dimension_count", 0)),
            rope_scaling=scaling, rope_pairing="adjacent",
            tie_word_embeddings=False,     # decided by the tensor list: output.weight absent -> tied
            bos_token_id=meta.get("tokenizer.ggml.bos_token_id"),
            eos_token_id=meta.get("tokenizer.ggml.eos_token_id"),
            stored_dtype=stored_dtype, name=str(meta.get("general.name", "")))

    # ------------------------------------------------------------------ writers
    def to_dict(self) -> dict:
        """config.json keys, the inverse of `from_dict`."""
        d = {
            "architectures": [self.architecture if self.architecture != "llama" else "LlamaForCausalLM"],
            "model_type": "llama",
            "hidden_size": self.n_embd, "num_hidden_layers": self.n_layer,
            "num_attention_heads": self.n_head, "num_key_value_heads": self.n_head_kv,
            "head_dim": self.head_dim, "intermediate_size": self.n_ff, "vocab_size": self.n_vocab,
            "max_position_embeddings": self.n_ctx_train, "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_freq_base, "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings, "torch_dtype": self.stored_dtype,
            "attention_bias": False, "mlp_bias": False,
        }
        if self.rope_dim != self.head_dim:
            d["partial_rotary_dim"] = self.rope_dim
        if self.rope_pairing != "half":
            d["rope_pairing"] = self.rope_pairing
        if self.rope_scaling is not None:
            d["rope_scaling"] = asdict(self.rope_scaling)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_id if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d

    def to_gguf_metadata(self) -> dict:
        """GGUF keys, the inverse of `from_gguf_metadata` (crates/core-types/src/model.rs:64-128)."""
        m = {"general.architecture": "llama", "general.name": self.name or "ferrum_b200",
             "llama.context_length": self.n_ctx_train, "llama.embedding_length": self.n_embd,
             "llama.block_count": self.n_layer, "llama.attention.head_count": self.n_head,
             "llama.attention.head_count_kv": self.n_head_kv, "llama.feed_forward_length": self.n_ff,
             "llama.attention.layer_norm_rms_epsilon": float(self.rms_norm_eps),
             "llama.rope.freq_base": float(self.rope_freq_base), "llama.attention.key_length": self.head_dim,
             "llama.attention.value_length": self.head_dim, "llama.rope.dimension_count": self.rope_dim,
             "llama.vocab_size": self.n_vocab}
        if self.rope_scaling is not None:
            rs = self.rope_scaling
            m.update({"llama.rope.scaling.type": rs.rope_type, "llama.rope.scaling.factor": float(rs.factor),
                      "llama.rope.scaling.low_freq_factor": float(rs.low_freq_factor),
                      "llama.rope.scaling.high_freq_factor": float(rs.high_freq_factor),
                      "llama.rope.scaling.original_context_length": rs.original_max_position_embeddings})
        if self.bos_token_id is not None:
            m["tokenizer.ggml.bos_token_id"] = self.bos_token_id
        if self.eos_token_id is not None:
            m["tokenizer.ggml.eos_token_id"] = self.eos_token_id
        return m

    @property
    def q_width(self) -> int:
        return self.n_head * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.n_head_kv * self.head_dim
