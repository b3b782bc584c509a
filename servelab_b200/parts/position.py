"""Position encodings.

``rotary``: rotate-half rotary embedding; inv_freq_i = theta^(-2i/rotary_dim) in
float32, as the reference builds it (servelab/parallel/tp_model.py:94-95; the
buffer is never cast to the model dtype here, unlike tp_model.py:96-97).  The
rotation itself is fused into the mixer's q/k kernel, which asks this part for
its table.  ``none``: no position information.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_position


def stretch_long_wavelengths(f: torch.Tensor, factor: float, low: float, high: float,
                             original: float) -> torch.Tensor:
    """Frequencies ``f`` (float64) with the long wavelengths stretched: with l = 2 pi / f, a frequency
    with l > original / low becomes f / factor, one with l < original / high stays, and between the
    two s = (original / l - low) / (high - low) blends them, (1 - s) f / factor + s f."""
    wavelength = 2.0 * math.pi / f
    s = ((original / wavelength - low) / (high - low)).clamp(0.0, 1.0)
    blended = (1.0 - s) * f / factor + s * f
    return torch.where(wavelength < original / high, f,
                       torch.where(wavelength > original / low, f / factor, blended))


@register_position("rotary")
class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        rd = spec.rotary_dim or spec.head_dim
        if rd % 2 or rd > spec.head_dim:
            raise ValueError(f"rotary_dim {rd} must be even and <= head_dim {spec.head_dim}")
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        if spec.precise or spec.stretch_factor is not None:
            f = float(spec.theta) ** (-2.0 * torch.arange(rd // 2, dtype=torch.float64) / rd)
            if spec.stretch_factor is not None:
                if not (spec.stretch_factor > 0 and spec.stretch_high > spec.stretch_low >= 0
                        and spec.stretch_original > 0):
                    raise ValueError("rotary: a stretch needs factor > 0, high > low >= 0 and original > 0")
                f = stretch_long_wavelengths(f, float(spec.stretch_factor), float(spec.stretch_low),
                                             float(spec.stretch_high), float(spec.stretch_original))
            inv_freq = f.to(torch.float32)
        self.rotary_dim = rd
        self.inv_freq = inv_freq.to(env.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim


@register_position("rotary_pairs")
class PairRotary(PositionEncoding):
    """Rotation of neighbouring pairs (2i, 2i + 1), optionally with YaRN-scaled frequencies.
    ``pair_table()`` -> (frequencies float32 [dims / 2], dims, factor on cos and sin); the
    rotation itself runs in the mixer's head kernel (``ops.kernels.head_prep``).  The
    frequencies are formed in float64 on the host and rounded once."""
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        d = spec.dims
        if d <= 0 or d % 2:
            raise ValueError(f"rotary_pairs: dims must be positive and even, got {d}")
        i = torch.arange(d // 2, dtype=torch.float64)
        f = float(spec.theta) ** (-2.0 * i / d)
        self.magnitude = 1.0
        if spec.yarn_factor is not None:
            factor = float(spec.yarn_factor)

            def pair_that_turns(times: float) -> float:
                return d * math.log(spec.yarn_original / (2.0 * math.pi * times)) / (2.0 * math.log(spec.theta))
            lo = max(math.floor(pair_that_turns(spec.yarn_fast)), 0)
            hi = min(math.ceil(pair_that_turns(spec.yarn_slow)), d - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        if spec.stretch_factor is not None:
            f = stretch_long_wavelengths(f, float(spec.stretch_factor), float(spec.stretch_low),
                                         float(spec.stretch_high), float(spec.stretch_original))
        self.dims = d
        self.freq = f.to(torch.float32).to(env.device)

    def pair_table(self):
        return self.freq, self.dims, self.magnitude


@register_position("none")
class NoPosition(PositionEncoding):
    graph_safe = True
