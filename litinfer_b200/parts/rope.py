"""Rotary position encoding, rotate-half pairing (src/ops/rope/op.cpp:13-20, 33-39).

For pair j of the first ``rotary_dim`` elements of a head:
``phi = float(pos) / theta^(2j / rotary_dim)``, ``(a, b) = (x[j], x[j + rotary_dim/2])``,
``x'[j] = a cos(phi) - b sin(phi)``, ``x'[j + rotary_dim/2] = b cos(phi) + a sin(phi)``.
The part owns the table of denominators ``theta^(2j/rotary_dim)`` (float32);
the kernel divides the position by it and takes sine and cosine in float32.
Another frequency rule (scaled, partial) is another table or ``rotary_dim``.

``scaling`` (a mapping with ``factor``, ``low``, ``high``, ``original``) slows the long waves down, by wavelength
``l = 2 pi * denominator``: below ``original / high`` the frequency stays, beyond ``original / low`` it is divided by
``factor``, and between the two it is ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``.
The table of denominators is made once, in float64, and rounded to float32.

``scaling`` with ``kind`` "yarn" (``factor``, ``original``, ``fast``, ``slow``) blends by the index of the pair instead: with
``index(t) = dims ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(index(fast)), 0)``, ``hi = min(ceil(index(slow)),
dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency of pair i is ``f_i / factor * ramp_i +
f_i (1 - ramp_i)``, and cosines and sines carry the magnitude ``0.1 ln(factor) + 1`` (:attr:`Rotary.magnitude`).

``pairing`` "interleaved": element 2j turns with element 2j + 1.  Only mixers whose kernels take that pairing accept it
(:attr:`Rotary.interleaved`); the paged attention part rotates halves.
"""

from __future__ import annotations

import torch

from .base import POSITIONS, Position, Rotary


def scaled_denominators(theta: float, rotary_dim: int, scaling) -> list:
    """1 / frequency of every pair after the scaling by wavelength (see the module's text), as Python floats."""
    import math

    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    if factor <= 0 or high <= low or original <= 0:
        raise ValueError(f"rope scaling needs factor > 0, high > low and original > 0, got {dict(scaling)}")
    out = []
    for j in range(rotary_dim // 2):
        f = float(theta) ** (-2.0 * j / rotary_dim)
        wave = 2.0 * math.pi / f
        if wave > original / low:
            f = f / factor
        elif wave >= original / high:
            s = (original / wave - low) / (high - low)
            f = (1.0 - s) * f / factor + s * f
        out.append(1.0 / f)
    return out


def yarn_denominators(theta: float, rotary_dim: int, scaling) -> list:
    """1 / frequency of every pair after the blend by the pair's index (see the module's text), as Python floats."""
    import math

    factor, original, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
    if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0:
        raise ValueError(f"yarn scaling needs factor, original, fast and slow > 0, got {dict(scaling)}")

    def index_of(turns):
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), rotary_dim - 1)
    out = []
    for i in range(rotary_dim // 2):
        f = float(theta) ** (-2.0 * i / rotary_dim)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(1.0 / (f / factor * ramp + f * (1.0 - ramp)))
    return out


def yarn_magnitude(scaling) -> float:
    import math

    return 0.1 * math.log(float(scaling["factor"])) + 1.0


@POSITIONS.register("rope")
class RotaryEmbedding(Position):
    def __init__(self, spec, prefix, dtype, device, head_dim=None):
        super().__init__(spec, prefix, dtype, device)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec.get("rotary_dim") or head_dim)
        pairing = spec.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing '{pairing}' is not supported (half, interleaved)")
        self.interleaved = pairing == "interleaved"
        self.magnitude = 1.0
        if self.rotary_dim % 2 or (head_dim is not None and self.rotary_dim > head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        scaling = spec.get("scaling")
        if not scaling:
            j = torch.arange(self.rotary_dim // 2, dtype=torch.float32)
            denom = torch.pow(torch.tensor(self.theta, dtype=torch.float32), (2.0 * j) / float(self.rotary_dim))
        elif scaling.get("kind") == "yarn":
            denom = torch.tensor(yarn_denominators(self.theta, self.rotary_dim, scaling), dtype=torch.float64).to(torch.float32)
            self.magnitude = yarn_magnitude(scaling)
        else:
            denom = torch.tensor(scaled_denominators(self.theta, self.rotary_dim, scaling), dtype=torch.float64).to(torch.float32)
        self.scaling = dict(scaling) if scaling else None
        self.denominators = denom.to(self.device)

    # Steps of more tokens than this get a table of cosines and sines, made once and shared by the layers (products that
    # rotate in their epilogue read it); shorter steps compute the angles where they rotate.
    TABLE_FROM_TOKENS = 65

    def fused_decode(self):
        plain = type(self) is RotaryEmbedding and not self.interleaved and self.magnitude == 1.0
        return {"denominators": self.denominators, "rotary_dim": self.rotary_dim} if plain else None

    def rotary(self, ctx) -> Rotary:
        if self.interleaved or self.magnitude != 1.0:
            # (no kernel that rotates in a product's epilogue takes these: no table)
            return Rotary(self.denominators, self.rotary_dim, None, self.magnitude, self.interleaved)
        return Rotary(self.denominators, self.rotary_dim, self.table(ctx))

    def table(self, ctx):
        """``[tokens, rotary_dim / 2, 2]`` float32 cos and sin of this step's positions, or None for a short step."""
        if ctx.num_tokens < self.TABLE_FROM_TOKENS or self.dtype != torch.bfloat16:
            return None
        key = ("rope_table", self.theta, self.rotary_dim, tuple(sorted(self.scaling.items())) if self.scaling else None)
        t = ctx.scratch.get(key)
        if t is None:
            from .. import kernels as K

            t = torch.empty((ctx.num_tokens, self.rotary_dim // 2, 2), dtype=torch.float32, device=ctx.positions.device)
            K.rope_table(ctx.positions, self.denominators, t)
            ctx.scratch[key] = t
        return t
