"""Rotary position encoding: a table of (cos, sin) per position and pair.

The reference rotates adjacent pairs (2i, 2i+1) by pos / theta^(2i/R)
(crates/kernels/src/math.rs:31-34, scalar.rs:167-189) and refuses every scaling
(crates/core-types/src/model.rs:82-88).  Here the pairing is a parameter ("adjacent" for
GGUF-ordered rows, "half" = (i, i+R/2) for HF-ordered rows).  A scaling rule is a function from
the unscaled frequencies to the scaled ones, looked up by the `rope_type` of the scaling block:
`llama3` is registered here, another rule is one `register_scaling` call (or the part is given
its frequencies directly).  Frequencies and angles are computed once in float64 and stored as
float32, so a rotation is as exact at position 100000 as at position 1.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding

PAIRING = {"adjacent": 0, "half": 1}


SCALINGS = {}        # rope_type -> function(frequencies, scaling block) -> frequencies


def register_scaling(rope_type, fn):
    """fn(list of R/2 frequencies, the configuration's scaling block) -> list of scaled frequencies."""
    SCALINGS[rope_type] = fn


def inverse_frequencies(rope_dim, theta, scaling=None):
    f = [theta ** (-2.0 * i / rope_dim) for i in range(rope_dim // 2)]
    if scaling is None:
        return f
    try:
        rule = SCALINGS[scaling.rope_type]
    except KeyError:
        raise ValueError(f"unsupported rope scaling {scaling.rope_type}") from None
    return rule(f, scaling)


def llama3_scaling(f, scaling):
    """Wavelengths shorter than original/high_freq_factor keep their frequency, longer than
    original/low_freq_factor are divided by `factor`, and between them the two are blended."""
    orig = float(scaling.original_max_position_embeddings)
    lo_wave, hi_wave = orig / scaling.high_freq_factor, orig / scaling.low_freq_factor
    out = []
    for fk in f:
        wave = 2.0 * math.pi / fk
        if wave < lo_wave:
            out.append(fk)
        elif wave > hi_wave:
            out.append(fk / scaling.factor)
        else:
            s = (orig / wave - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)
            out.append((1.0 - s) * fk / scaling.factor + s * fk)
    return out


register_scaling("llama3", llama3_scaling)


class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim, rope_dim, theta, scaling, pairing, max_positions, device, frequencies=None):
        """frequencies: the R/2 rotation frequencies themselves, for a rule that is no function of
        (theta, scaling block); theta and scaling are not looked at then."""
        if rope_dim % 2 or rope_dim > head_dim:
            raise ValueError("invalid rope dimension")
        self.head_dim, self.rope_dim = head_dim, rope_dim
        self.pairing = PAIRING[pairing]
        self.max_positions = int(max_positions)
        if frequencies is None:
            frequencies = inverse_frequencies(rope_dim, float(theta), scaling)
        if len(frequencies) != rope_dim // 2:
            raise ValueError("a rotation of R dimensions needs R/2 frequencies")
        inv = torch.tensor(list(frequencies), dtype=torch.float64)
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32)
        self.cos_sin = table.contiguous().to(device)      # [positions, rope_dim/2, 2]

    def rotary(self):
        return self
