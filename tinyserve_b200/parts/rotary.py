"""Rotary position encoding.  Tables as tinyserve builds them (serve.py:1225-1228):
inv_freq and angles in float64, cos and sin stored in float32, one row per absolute
position up to the engine's max_model_len (serve.py:1621).  ``pairing`` "half"
rotates (i, i + rotary_dim/2) as serve.py:811-814 does; "interleaved" rotates
(2i, 2i+1).  ``rotary_dim`` may be smaller than the head size (partial rotary); the
other dimensions pass through.  ``scaling`` = {factor, low, high, original} stretches the long
waves: with wavelength l = 2 pi / f, f stays where l < original / high, becomes f / factor where
l > original / low, and in between is (1 - s) f / factor + s f with
s = (original / l - low) / (high - low).

``scaling`` = {factor, original, fast, slow} is the other rule, a ramp over the pair index i: a
wave that fits the original context ``t`` times has the (fractional) index
d(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta); with lo = max(floor(d(fast)), 0),
hi = min(ceil(d(slow)), rotary_dim - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the
frequency is r_i f_i / factor + (1 - r_i) f_i, and cos and sin are both multiplied by
0.1 ln(factor) + 1."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding

class Rotary(PositionEncoding):
    capturable = True

    def __init__(self, rotary_dim: int, theta: float, pairing: str = "half", scaling: dict | None = None):
        super().__init__()
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.interleaved = pairing == "interleaved"
        self.scaling = None
        if scaling and "fast" in scaling:
            self.scaling = ("ramp",) + tuple(float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
            if not all(v > 0 for v in self.scaling[1:]):
                raise ValueError(f"rotary scaling {scaling!r}: factor, original, fast and slow are positive")
        elif scaling:
            self.scaling = tuple(float(scaling[k]) for k in ("factor", "low", "high", "original"))
            factor, low, high, original = self.scaling
            if not (factor > 0 and high > low and original > 0 and low > 0):
                raise ValueError(f"rotary scaling {scaling!r}: factor, low and original positive, high above low")
        self.cos = self.sin = None

    @staticmethod
    def scaled(inv_freq, scaling):
        factor, low, high, original = scaling
        wave = 2.0 * math.pi / inv_freq
        s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
        mixed = (1.0 - s) * inv_freq / factor + s * inv_freq
        out = torch.where(wave > original / low, inv_freq / factor, mixed)
        return torch.where(wave < original / high, inv_freq, out)

    @staticmethod
    def ramped(inv_freq, rotary_dim, theta, scaling):
        """(frequencies, factor on cos and sin) of the ramp rule."""
        _, factor, original, fast, slow = scaling

        def index_of(turns):
            return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

        lo = max(math.floor(index_of(fast)), 0)
        hi = min(math.ceil(index_of(slow)), rotary_dim - 1)
        i = torch.arange(rotary_dim // 2, dtype=torch.float64)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return inv_freq / factor * ramp + inv_freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    @staticmethod
    def tables(rotary_dim, theta, num_positions, scaling=None):
        inv_freq = 1.0 / theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)
        magnitude = 1.0
        if scaling and scaling[0] == "ramp":
            inv_freq, magnitude = Rotary.ramped(inv_freq, rotary_dim, theta, scaling)
        elif scaling:
            inv_freq = Rotary.scaled(inv_freq, scaling)
        freqs = torch.outer(torch.arange(num_positions, dtype=torch.float64), inv_freq)
        return (freqs.cos() * magnitude).float(), (freqs.sin() * magnitude).float()

    def prepare(self, runtime):
        # one table per (sizes, base) and engine: the layers of a model share it
        key = ("rotary", self.rotary_dim, self.theta, self.scaling)
        if key not in runtime.shared:
            cos, sin = self.tables(self.rotary_dim, self.theta, runtime.max_positions, self.scaling)
            runtime.shared[key] = (cos.to(runtime.device).contiguous(), sin.to(runtime.device).contiguous())
        self.cos, self.sin = runtime.shared[key]


register_position_encoding("rotary", Rotary)
