"""Position encodings.

``rope``: rotate-half rotary encoding.  inv_freq[i] = 1 / theta^(2i/rotary_dim)
with theta and the power in float32, angle = float32(position) * inv_freq[i] as
a float32 product (thanhauco/rust-inference src/ops/rope.rs:19-47; theta is read
as float32, src/models/config.rs:33-34).  The table holds cos and sin of that
float32 angle, evaluated in float64 and rounded once, times ``scaling``.
The attention kernel applies the table itself (``fused_table``).  Parts with
the same rotary size, base, scaling and device share one table (a model's layers
usually do), so it is held once, not once per layer.

``rope_pairs``: neighbouring elements (2i, 2i+1) are turned, not the two halves, optionally with YaRN's
blended frequencies and its factor on cos and sin, or with frequencies slowed by wavelength
(:class:`~..config.specs.RopePairsSpec` has both rules).  The
frequencies are evaluated in float64 and rounded to float32, the angle is the float32 product with the float32
position, cos and sin of it are evaluated in float64 and rounded once.  The table has the same layout
[positions, rot/2, 2]; the kernels of the mixers that name this kind pair the elements accordingly.

``none``: nothing.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding
from .registry import register_position


_shared_tables = {}        # (device, rot, float32 theta, scaling) -> table [positions, rot/2, 2]


@register_position("rope")
class Rope(PositionEncoding):
    graph_safe = True
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rot % 2 or spec.rot > spec.head_dim or spec.rot <= 0:
            raise ValueError(f"rotary_dim {spec.rot} must be even and within head_dim {spec.head_dim}")
        self._table = None

    def inv_freq(self) -> np.ndarray:
        rot = self.spec.rot
        if getattr(self.spec, "freq64", False):
            i = np.arange(rot // 2, dtype=np.float64)
            return (float(self.spec.theta) ** (-2.0 * i / rot)).astype(np.float32)
        theta = np.float32(self.spec.theta)
        exps = np.arange(0, rot, 2, dtype=np.float32) / np.float32(rot)
        return (np.float32(1.0) / np.power(theta, exps, dtype=np.float32)).astype(np.float32)

    def prepare(self, max_positions: int) -> None:
        if self._table is not None and self._table.shape[0] >= max_positions:
            return
        key = (str(self.env.device), int(self.spec.rot), float(np.float32(self.spec.theta)), float(self.spec.scaling),
               bool(getattr(self.spec, "freq64", False)), float(self.spec.theta))
        shared = _shared_tables.get(key)
        if shared is not None and shared.shape[0] >= max_positions:
            self._table = shared
            return
        pos = np.arange(max_positions, dtype=np.float32)
        ang = (pos[:, None] * self.inv_freq()[None, :]).astype(np.float32).astype(np.float64)
        scale = float(self.spec.scaling)
        table = np.stack([np.cos(ang) * scale, np.sin(ang) * scale], axis=-1).astype(np.float32)
        self._table = _shared_tables[key] = torch.from_numpy(table).to(self.env.device).contiguous()

    def fused_table(self):
        return self._table


@register_position("rope_pairs")
class RopePairs(PositionEncoding):
    graph_safe = True
    pairs = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be positive and even")
        if spec.yarn is not None and getattr(spec, "by_wavelength", None) is not None:
            raise ValueError("a rotation has YaRN's blend of frequencies or the rule by wavelength, not both")
        self._table = None

    def frequencies(self):
        """(float32 frequencies [rot/2], factor on cos and sin)."""
        rot, theta = self.spec.rotary_dim, float(self.spec.theta)
        i = np.arange(rot // 2, dtype=np.float64)
        f = theta ** (-2.0 * i / rot)
        mult = 1.0
        if self.spec.yarn is not None:
            factor, original, fast, slow = (float(v) for v in self.spec.yarn)

            def where(turns):
                return rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

            lo = max(math.floor(where(fast)), 0)
            hi = min(math.ceil(where(slow)), rot - 1)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            mult = 0.1 * math.log(factor) + 1.0
        rule = getattr(self.spec, "by_wavelength", None)
        if rule is not None:
            factor, low, high, original = (float(v) for v in rule)
            wave = 2.0 * math.pi / f
            s = (original / wave - low) / (high - low) if high != low else np.ones_like(f)
            f = np.where(wave < original / high, f, np.where(wave > original / low, f / factor,
                                                              (1.0 - s) * f / factor + s * f))
        return f.astype(np.float32), mult

    def prepare(self, max_positions: int) -> None:
        if self._table is not None and self._table.shape[0] >= max_positions:
            return
        key = (str(self.env.device), "pairs", int(self.spec.rotary_dim), float(self.spec.theta), self.spec.yarn,
               getattr(self.spec, "by_wavelength", None))
        shared = _shared_tables.get(key)
        if shared is not None and shared.shape[0] >= max_positions:
            self._table = shared
            return
        f, mult = self.frequencies()
        pos = np.arange(max_positions, dtype=np.float32)
        ang = (pos[:, None] * f[None, :]).astype(np.float32).astype(np.float64)
        table = np.stack([np.cos(ang) * mult, np.sin(ang) * mult], axis=-1).astype(np.float32)
        self._table = _shared_tables[key] = torch.from_numpy(table).to(self.env.device).contiguous()

    def fused_table(self):
        return self._table


@register_position("none")
class NoPosition(PositionEncoding):
    graph_safe = True
