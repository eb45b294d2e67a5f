"""Rotate-half ("neox") rotary position encoding.

For pair i of a head, f_i = 1 / theta^(2i/hd); the angle p·f_i is a float32 product of the
integer position and the float32 frequency; (x_i, x_{i+hd/2}) ← (x_i·c − x_{i+hd/2}·s,
x_i·s + x_{i+hd/2}·c) (src/ops.cpp:125-141).  The frequencies are computed on the host the
way the reference computes them; cos and sin are tabulated once per context on the device
and every kernel reads the table.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part


def neox_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """f_i as float32: the exponent 2i/hd is a float32 quotient, the power is rounded to
    float32, then 1/x in float32 (src/ops.cpp:132)."""
    i2 = np.arange(0, head_dim, 2, dtype=np.float32)
    expo = i2 / np.float32(head_dim)
    power = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
    return torch.from_numpy((np.float32(1.0) / power).astype(np.float32))


# One table per (head size, theta, positions, device), shared by every layer and every model that asks for it: the
# attention layers of a model all rotate alike, and a decode step that pulled a private copy per layer through the
# cache hierarchy would read the same numbers two dozen times.
_TABLES: Dict[Tuple[int, float, int, str], torch.Tensor] = {}


def shared_table(inv_freq: torch.Tensor, head_dim: int, theta: float, max_positions: int) -> torch.Tensor:
    key = (head_dim, float(theta), max_positions, str(inv_freq.device))
    table = _TABLES.get(key)
    if table is None:
        table = _TABLES[key] = kernels.rope_table(inv_freq, max_positions)
    return table


@register_part("position", "rope_neox")
class RopeNeox(Part):
    graph_safe = True

    # How the attention part applies a position encoding.  `fusable = True`: the encoding is a rotation of the pairs
    # (i, i + head_dim/2) by angles that depend on the position alone; it offers `table`, [positions][head_dim/2][2]
    # float32 cos and sin (or None for "no rotation"), and the Q/K/V kernel's epilogue applies it.  `fusable = False`:
    # anything else; the attention part then calls `rotate(x, positions)` on the float32 queries and keys itself.
    fusable = True

    def __init__(self, name: str, head_dim: int, theta: float, max_positions: int):
        super().__init__(name, head_dim=head_dim, theta=theta, max_positions=max_positions)
        if head_dim <= 0 or head_dim % 2:
            raise ValueError(f"rope: head_dim must be positive and even, got {head_dim}")      # src/ops.cpp:164-168
        if not math.isfinite(theta) or theta <= 0:
            raise ValueError("rope: theta must be finite and positive")                        # src/ops.cpp:151-153
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)
        self.table: Optional[torch.Tensor] = None

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.inv_freq = neox_inv_freq(self.head_dim, self.theta).to(runtime.device)

    def prepare(self, n_positions: int) -> None:
        """Make sure the table exists.  It is built once, for every position the model allows,
        and never replaced: captured graphs keep reading the same memory."""
        if self.table is None:
            self.table = shared_table(self.inv_freq, self.head_dim, self.theta, self.max_positions)

    def rotate(self, x: torch.Tensor, positions: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Rotate float32 x [n, heads, head_dim] by int32 positions [n]; on its own, outside attention."""
        n, heads, hd = x.shape
        assert hd == self.head_dim
        self.prepare(int(positions.max().item()) + 1)
        out = self.runtime.empty(n, heads, hd, dtype=out_dtype or self.runtime.dtype)
        zeros = torch.zeros(n, dtype=torch.int32, device=x.device)
        kernels.qkv_post(x.reshape(n, heads * hd).contiguous(), None, positions, zeros, self.table, heads, 0, hd, out, None)
        return out


@register_part("position", "none")
class NoPosition(Part):
    graph_safe = True

    fusable = True

    def __init__(self, name: str, **_):
        super().__init__(name)
        self.table = None

    def prepare(self, n_positions: int) -> None:
        pass


def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[np.ndarray, float]:
    """Frequencies of a rotation over `dims` entries, pair i with i + dims/2, f_i = base^(-2i/dims), optionally
    stretched for contexts longer than the trained one ("YaRN"; Peng et al., "YaRN: Efficient Context Window Extension
    of Large Language Models"): with scaling = {factor, original, fast, slow},

        turn(t) = dims · ln(original / (2π t)) / (2 ln base)        the pair that makes t turns over `original` positions
        lo = max(floor(turn(fast)), 0),  hi = min(ceil(turn(slow)), dims - 1)
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f'_i = f_i / factor · ramp_i + f_i · (1 - ramp_i)

    so that fast pairs keep their frequency and slow ones are divided by `factor`; cos and sin are both multiplied by
    0.1 · ln(factor) + 1.  With scaling = {factor} alone the stretching is linear: every frequency is divided by the
    factor (positions count `factor` times slower) and the multiplier is one.  Returns (float32 frequencies [dims/2], that
    multiplier).  Computed in float64, rounded once."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = np.power(float(base), -2.0 * i / dims)
    if not scaling:
        return f.astype(np.float32), 1.0
    if "original" not in scaling:
        # linear stretching: positions are divided by the factor, that is, every frequency is
        factor = float(scaling["factor"])
        if factor <= 0:
            raise ValueError("rope scaling: factor must be positive")
        return (f / factor).astype(np.float32), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if factor <= 0 or original <= 0 or float(scaling["fast"]) <= 0 or float(scaling["slow"]) <= 0:
        raise ValueError("rope scaling: factor, original, fast and slow must be positive")

    def turn(t: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(float(base)))
    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f.astype(np.float32), 0.1 * math.log(factor) + 1.0


@register_part("position", "rope_partial")
class RopePartial(Part):
    """Rotation of the first `dims` entries of each head (the rest pass unchanged), with optional stretching of the
    frequencies (`stretched_frequencies`).  `pairing` says which entries form a pair: "half" pairs entry i with i + dims/2
    (rotate-half), "interleaved" pairs entry 2i with 2i + 1; the pair (u, v) becomes (u cos a - v sin a, v cos a + u sin a)
    with a = position · f_i either way, so the table is the same and only the mixer's kernel reads `interleaved`.  The model gives no largest position, so the table
    [positions][dims/2] of (cos, sin) grows: it is rebuilt, twice as long, when a step reaches beyond it.  Tables
    once handed out stay alive and valid for the positions they hold, so a captured graph that reads one keeps
    reading the same memory; a step is captured for a bound on its positions and asks for its table with that bound."""
    graph_safe = True
    fusable = False

    MIN_POSITIONS = 4096

    PAIRINGS = ("half", "interleaved")

    def __init__(self, name: str, dims: int, base: float, scaling: Optional[dict] = None, pairing: str = "half"):
        super().__init__(name, dims=dims, base=base, scaling=scaling, pairing=pairing)
        if pairing not in self.PAIRINGS:
            raise ValueError(f"rope: pairing must be one of {', '.join(self.PAIRINGS)}; got {pairing!r}")
        self.interleaved = pairing == "interleaved"
        if dims < 0 or dims % 2:
            raise ValueError(f"rope: the rotated size must be even and not negative, got {dims}")
        if not math.isfinite(base) or base <= 0:
            raise ValueError("rope: base must be finite and positive")
        self.dims, self.base = int(dims), float(base)
        self.scaling = dict(scaling) if scaling else None
        self.table: Optional[torch.Tensor] = None
        self._old = []                     # tables handed out before the latest one

    def bind(self, get, runtime):
        super().bind(get, runtime)
        if self.dims:
            f, self.factor = stretched_frequencies(self.dims, self.base, self.scaling)
            self.inv_freq = torch.from_numpy(f).to(runtime.device)

    def prepare(self, n_positions: int) -> None:
        if self.dims == 0 or (self.table is not None and self.table.shape[0] >= n_positions):
            return
        size = self.MIN_POSITIONS
        while size < n_positions:
            size *= 2
        if self.table is not None:
            self._old.append(self.table)
        self.table = kernels.rope_table(self.inv_freq, size, self.factor)

    def table_for(self, n_positions: int) -> Optional[torch.Tensor]:
        """The table, holding at least `n_positions` positions (None: nothing is rotated)."""
        self.prepare(n_positions)
        return self.table
