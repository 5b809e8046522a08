"""Rotary position encoding: the table of angles, built once on the host in float64."""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope")
class RotaryEncoding(PositionEncoding):
    """Pair j of a head is turned by the angle pos / theta^(2j/rotary_dim)
    (crates/mach-model/src/kernels.rs:609-659 of gqf2008/machserve; the reference calls
    powf, cosf and sinf per element in float32).  Here cos and sin are computed in float64
    for every position up to the runtime's limit and rounded to float32 once; the attention
    kernel reads them by absolute position.

    params: head_dim, rotary_dim (<= head_dim, even), theta,
    pairing: "half" pairs coordinate j with j + rotary_dim/2, "interleaved" pairs 2j with 2j+1,
    scaling (optional): {factor, original, fast, slow}, the stretching of the slow waves for contexts longer than the
    `original` one (YaRN).  With n(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), the pair index whose wave makes
    t turns over `original` positions, lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), rotary_dim - 1) and
    r_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1), pair j turns by pos * (f_j / factor * r_j + f_j * (1 - r_j)), and cos
    and sin are both multiplied by 0.1 ln(factor) + 1.
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.theta = float(spec["theta"])
        pairing = spec.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rope: pairing '{pairing}' is neither 'half' nor 'interleaved'")
        self.interleaved = pairing == "interleaved"
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        scaling = spec.get("scaling")
        self.scaling = None
        if scaling is not None:
            self.scaling = tuple(float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
            if self.scaling[0] <= 0 or self.scaling[1] <= 0 or self.scaling[2] <= 0 or self.scaling[3] <= 0 or self.theta <= 1.0:
                raise ValueError(f"rope: scaling {dict(scaling)} needs positive numbers and theta above 1")
        self._table = None

    def frequencies(self):
        """(f [rotary_dim/2] float64, the multiplier of cos and sin)."""
        j = np.arange(self.rotary_dim // 2, dtype=np.float64)
        freq = 1.0 / (self.theta ** (2.0 * j / self.rotary_dim))
        if self.scaling is None:
            return freq, 1.0
        factor, original, fast, slow = self.scaling

        def pair_of(turns):
            return self.rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), self.rotary_dim - 1)
        ramp = np.clip((j - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def rotary_table(self, rt):
        if self._table is None or self._table.shape[0] < rt.max_positions:
            key = ("rope", self.rotary_dim, self.theta, self.scaling, rt.max_positions)
            shared = rt.__dict__.setdefault("shared_tables", {})
            if key not in shared:
                freq, mult = self.frequencies()
                ang = np.arange(rt.max_positions, dtype=np.float64)[:, None] * freq[None, :]
                table = (np.stack([np.cos(ang), np.sin(ang)], axis=-1) * mult).astype(np.float32)
                shared[key] = torch.from_numpy(table).to(rt.device).contiguous()
            self._table = shared[key]
        return self._table
