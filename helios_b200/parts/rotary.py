"""Rotary position encoding (python/helios/exec/model.py:117-153) with the ``llama3``
and ``yarn`` frequency scalings (not in the reference).  The encoding only makes the
cos/sin tables; how a mixer pairs dimensions (halves, or 2i with 2i + 1) is the mixer's.

Frequencies are computed once on the host in float64.  Each step the part turns
the batch's positions into a cos/sin table [T, rot/2] (float32, angles taken in
float64), kept for the step under the encoding's own identity: a mixer that was
handed an encoding reads that encoding's table, so layers may rotate by different
bases.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..csrc import ops
from .base import PositionEncoding, register_part


def rotary_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """inv_freq[j] = theta^(-2j/rotary_dim) in float64; with ``scaling`` (an object with
    factor, low_freq_factor, high_freq_factor, original_max_position_embeddings):
    wavelengths below P/high stay, above P/low are divided by factor, between are
    interpolated linearly in (P/wavelength - low) / (high - low)."""
    j = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (j / rotary_dim))
    if scaling is None:
        return inv
    f, lo, hi = float(scaling.factor), float(scaling.low_freq_factor), float(scaling.high_freq_factor)
    P = float(scaling.original_max_position_embeddings)
    if hi <= lo:
        raise ValueError("rope_scaling: high_freq_factor must exceed low_freq_factor")
    wavelen = 2.0 * math.pi / inv
    smooth = (P / wavelen - lo) / (hi - lo)
    mid = (1.0 - smooth) * inv / f + smooth * inv
    out = torch.where(wavelen > P / lo, inv / f, mid)
    out = torch.where(wavelen < P / hi, inv, out)
    return out


def yarn_frequencies(rotary_dim: int, theta: float, factor: float, original: float,
                     fast: float, slow: float) -> torch.Tensor:
    """f_i = theta^(-2i/rotary_dim) blended with f_i / factor by a ramp over the pair index
    i: with d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(d(fast)),
    0), hi = min(ceil(d(slow)), rotary_dim - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001),
    0, 1), the frequency is f_i / factor * ramp_i + f_i * (1 - ramp_i): pairs that turn often
    within the original length keep their frequency, slow ones are stretched.  float64."""
    i = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
    inv = float(theta) ** (-2.0 * i / rotary_dim)

    def pair_of(turns: float) -> float:
        return rotary_dim * math.log(float(original) / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), rotary_dim - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return inv / float(factor) * ramp + inv * (1.0 - ramp)


def yarn_attention_factor(factor: float) -> float:
    """What cos and sin are multiplied by under ``yarn`` scaling: 0.1 ln(factor) + 1."""
    return 0.1 * math.log(float(factor)) + 1.0


class RotaryEncoding(PositionEncoding):
    def __init__(self, rotary_dim: int, theta: float, scaling=None, inv_freq=None,
                 attention_factor: float = 1.0) -> None:
        """``scaling``: a ``llama3`` scaling object (see ``rotary_frequencies``).  ``inv_freq``
        (float64 [rotary_dim / 2]) gives the frequencies outright, ``attention_factor`` a
        factor on cos and sin (``yarn_frequencies`` / ``yarn_attention_factor``)."""
        if rotary_dim % 2:
            raise ValueError(f"rotary dimension {rotary_dim} must be even")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.scaling = scaling
        self.attention_factor = float(attention_factor)
        if inv_freq is not None:
            self.inv_freq64 = torch.as_tensor(inv_freq, dtype=torch.float64)
            if self.inv_freq64.numel() != rotary_dim // 2:
                raise ValueError(f"{self.inv_freq64.numel()} frequencies for {rotary_dim // 2} pairs")
        else:
            self.inv_freq64 = rotary_frequencies(rotary_dim, theta, scaling)
        self._dev: Optional[torch.Tensor] = None

    def tables(self, ctx):
        """(cos, sin) [T, rot/2] for the step's positions, computed once per step."""
        hit = ctx.step_tables.get(id(self))
        if hit is None:
            if self._dev is None or self._dev.device != ctx.positions.device:
                self._dev = self.inv_freq64.to(ctx.positions.device)
            hit = ctx.step_tables[id(self)] = ops.rotary_table(ctx.positions, self._dev,
                                                               self.attention_factor)
        return hit

    def prepare(self, ctx) -> None:
        # the plan's own encoding also serves the mixers that were given none
        ctx.rotary_cos, ctx.rotary_sin = self.tables(ctx)


register_part("position_encoding", "rotary", RotaryEncoding)
