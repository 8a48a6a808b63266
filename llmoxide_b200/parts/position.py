"""Position encodings.  ``rope_neox`` rotates pairs (i, i + n_rot/2) of the
first n_rot dims of a head by angle pos * base^(-2i/n_rot).  The angle is a
float64 recurrence theta_{i+1} = theta_i * base^(-2/n_rot) starting at pos,
and only sin/cos are rounded to float32, as the reference computes it
(crates/model/src/ops.rs:142-159, base held as float32).  With
``angles="float32"`` the angle itself is a float32 product of the position and
the float32 frequency base^(-2i/n_rot), for designs that compute positions and
angles in 32-bit.  With ``scaling`` (factor, original, fast, slow,
amplitude_slope) the frequencies are stretched for contexts beyond the
``original`` length: pair i has ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
with lo = max(floor(t(fast)), 0), hi = min(ceil(t(slow)), n_rot - 1) and
t(turns) = n_rot ln(original / (2 pi turns)) / (2 ln base); its frequency becomes
f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by
amplitude_slope * ln(factor) + 1.  That is the rule "ramp"; with ``scaling["rule"] = "wavelength"`` (factor, low, high,
original) a pair keeps its frequency f while its wavelength 2 pi / f is shorter than original / high, turns at
f / factor when it is longer than original / low, and in between at (1 - s) f / factor + s f with
s = (original / wavelength - low) / (high - low); cos and sin are not scaled.

``pairing="neighbours"`` says that the design rotates the pairs (2i, 2i+1).  A scalar product of a rotated query and
a rotated key does not depend on the order of a head's dimensions as long as both have the same, so a mixer brings
the rows of its query and key projections into the order (0, 2, 4, .., 1, 3, 5, ..) once, when the model is built
(``halves_order``), and every kernel rotates the pairs (i, i + n_rot/2) as for any other model.  ``none`` rotates
nothing."""

from __future__ import annotations

import math

import numpy as np
import torch

from .registry import register_position


@register_position("rope_neox")
class RotaryNeox:
    def __init__(self, spec, weights: dict, rt):
        self.n_rot, self.base, self.rt = int(spec["n_rot"]), float(spec["base"]), rt
        self.factors = spec.get("factors")  # optional per-pair divisors of the angle
        self.angles = spec.get("angles", "float64")
        self.scaling = spec.get("scaling")
        self.pairing = spec.get("pairing", "halves")
        if self.pairing not in ("halves", "neighbours"):
            raise ValueError(f"pairing {self.pairing!r}: 'halves' or 'neighbours'")
        if self.n_rot % 2:
            raise ValueError(f"n_rot {self.n_rot} must be even")
        self._tables = None
        self.rotary_tables()        # made when the model is built (tens of milliseconds), not in its first step

    def rotary_tables(self):
        if self._tables is None:
            half, n = self.n_rot // 2, self.rt.max_positions
            theta_scale = float(np.float32(self.base)) ** (-2.0 / self.n_rot)
            theta = np.arange(n, dtype=np.float64)
            cos = np.empty((n, half), dtype=np.float32)
            sin = np.empty((n, half), dtype=np.float32)
            freqs, amplitude = self._scaling()
            for i in range(half):
                if self.angles == "float32":
                    freq = np.float32(freqs[i])
                    angle = (np.arange(n, dtype=np.float32) * freq).astype(np.float64)
                    cos[:, i] = (np.cos(angle) * amplitude).astype(np.float32)
                    sin[:, i] = (np.sin(angle) * amplitude).astype(np.float32)
                    continue
                angle = theta if self.factors is None else theta / float(np.float32(self.factors[i]))
                cos[:, i] = np.cos(angle).astype(np.float32)
                sin[:, i] = np.sin(angle).astype(np.float32)
                theta = theta * theta_scale
            dev = self.rt.device
            self._tables = (torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev), self.n_rot)
        return self._tables


    def _scaling(self):
        """Per pair its frequency, and the factor on cos and sin (1 without ``scaling``)."""
        half = self.n_rot // 2
        sc = self.scaling
        plain = [self.base ** (-2.0 * i / self.n_rot) for i in range(half)]
        if not sc:
            return plain, 1.0
        if self.angles != "float32" or self.factors is not None:
            raise ValueError("scaled frequencies are built for angles='float32' without per-pair factors")
        factor, original = float(sc["factor"]), float(sc["original"])
        if sc.get("rule", "ramp") == "wavelength":
            low, high = float(sc["low"]), float(sc["high"])
            freqs = []
            for f in plain:
                wave = 2.0 * math.pi / f
                if wave < original / high:
                    freqs.append(f)
                elif wave > original / low:
                    freqs.append(f / factor)
                else:
                    s = (original / wave - low) / (high - low)
                    freqs.append((1.0 - s) * f / factor + s * f)
            return freqs, 1.0
        if sc.get("rule", "ramp") != "ramp":
            raise ValueError(f"scaling rule {sc['rule']!r}: 'ramp' or 'wavelength'")
        turn = lambda turns: self.n_rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
        lo = max(math.floor(turn(float(sc["fast"]))), 0)
        hi = min(math.ceil(turn(float(sc["slow"]))), self.n_rot - 1)
        freqs = []
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freqs.append(plain[i] / factor * ramp + plain[i] * (1.0 - ramp))
        return freqs, float(sc.get("amplitude_slope", 0.1)) * math.log(factor) + 1.0


def halves_order(position, weight, n_heads: int, head_dim: int, first: int = 0):
    """The rows of a projection [n_heads * head_dim, in] in the order the rotation kernels pair them: unchanged
    unless ``position`` pairs neighbours; then, in every head, the rotated dims first .. first + n_rot - 1 become
    (even ones, then odd ones).  Queries and keys must both go through this."""
    if position is None or getattr(position, "pairing", "halves") != "neighbours":
        return weight
    n_rot = position.n_rot
    order = list(range(head_dim))
    order[first : first + n_rot] = [first + i for i in range(0, n_rot, 2)] + [first + i for i in range(1, n_rot, 2)]
    index = torch.tensor([h * head_dim + i for h in range(n_heads) for i in order], device=weight.device)
    return weight.index_select(0, index).contiguous()


@register_position("none")
class NoPosition:
    def __init__(self, spec, weights: dict, rt):
        pass

    def rotary_tables(self):
        return None
