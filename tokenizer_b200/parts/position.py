"""Rotary position encoding, half-split form: lane i of a head pairs with lane
i + rotary_dim/2.  inv_freq_i = 1 / theta^(2i / rotary_dim) is computed in
float64 and stored in float32; the angle float32(position) * inv_freq_i and its
cosine and sine are float32 tables of `max_positions` rows
(reference: qwen-infer/src/model.rs:138-172)."""
from __future__ import annotations

import math

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from .base import register_part


class RotaryHalfSplit:
    @staticmethod
    def tensors(spec):
        return []

    def __init__(self, spec, store, runtime):
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ConfigError(f"rotary width {self.rotary_dim} must be even and positive")
        inv_freq = [1.0 / (self.theta ** (i / self.rotary_dim)) for i in range(0, self.rotary_dim, 2)]
        self.inv_freq = torch.tensor(inv_freq, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.cos, self.sin = ops.rope_table(self.inv_freq, self.max_positions)

    def key(self):
        return (self.theta, self.rotary_dim, self.max_positions)


def scaled_frequencies(freq, scaling):
    """The frequencies of a rotation after `scaling` (None: as they are), in float64.
    {"kind": "linear", factor}: every frequency divided by the factor (positions stretched).
    {"kind": "bands", factor, low, high, original}: by wavelength l = 2 pi / f: kept where l <
    original / high, divided by the factor where l > original / low, and in between blended with
    s = (original / l - low) / (high - low) as (1 - s) f / factor + s f."""
    if scaling is None:
        return list(freq)
    kind, factor = scaling.get("kind"), float(scaling["factor"])
    if factor <= 0:
        raise ConfigError("a rotation's scaling factor is positive")
    if kind == "linear":
        return [f / factor for f in freq]
    if kind != "bands":
        raise ConfigError(f"a rotation's frequencies are scaled linearly or by bands, found {kind!r}")
    low, high, original = float(scaling["low"]), float(scaling["high"]), float(scaling["original"])
    if high == low:
        raise ConfigError("the bands of a rotation's scaling need low and high apart")
    out = []
    for f in freq:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


class RotaryInterleaved:
    """Rotary position encoding with computed angles.  Interleaved form (`layout` "interleaved"): lane
    2i of the rotated lanes pairs with lane 2i + 1, i < dims / 2; half form (`layout` "half", kind
    `rope_half`): lane i pairs with lane i + dims / 2.  The pair (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = float32(p) * f_i, f_i = base^(-2i / dims), rescaled
    where the part has a `scaling` (`scaled_frequencies`), computed in float64 and stored in float32.
    There are no tables and no longest position: the kernels that rotate take the frequencies and
    compute sine and cosine of the 32-bit angle themselves."""

    layout = "interleaved"

    @staticmethod
    def tensors(spec):
        return []

    def __init__(self, spec, store, runtime):
        self.base = float(spec.params["base"])
        self.dims = int(spec.params["dims"])
        if self.dims % 2 or self.dims <= 0 or self.base <= 0:
            raise ConfigError(f"rotary width {self.dims} must be even and positive, the base positive")
        freq = scaled_frequencies([self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)],
                                  spec.params.get("scaling"))
        self.inv_freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(runtime.device)
        # the same in 64-bit, for kernels that take the angle in 64-bit (an angle of thousands of radians
        # carries the 32-bit product's rounding, 6e-8 of itself, straight into its sine)
        self.inv_freq64 = torch.tensor(freq, dtype=torch.float64).to(runtime.device)


class RotaryHalfComputed(RotaryInterleaved):
    layout = "half"


register_part("position", "rope_half_split", RotaryHalfSplit)
register_part("position", "rope_interleaved", RotaryInterleaved)
register_part("position", "rope_half", RotaryHalfComputed)
