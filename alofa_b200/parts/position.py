"""Position encodings.

``rotary_neox`` is the half-split rotary encoding: for position p and pair
index i < rot/2, ``inv_i = f32(1) / f32(theta^(2i/rot))`` with the power in
f64, ``angle = f32(p) * inv_i`` as an fp32 product, and cos/sin taken in f64
and rounded once to fp32 (src/alofa/model/arch/qwen.mojo:830-880).  The
rotation itself, ``y[d] = a cos - b sin``, ``y[d + rot/2] = b cos + a sin``
(src/alofa/kernels/cpu/scalar.mojo:283-344), runs inside the mixer's
rotate-and-store kernel, which reads the table built here."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..errors import AlofaError
from .base import Part, register_part


class RotaryNeox(Part):
    family = "position"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.head_dim = int(self.param("head_dim"))
        self.rotary_dim = int(self.param("rotary_dim", self.head_dim))
        self.theta = float(self.param("theta"))
        self.max_position = int(self.param("max_position"))
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise AlofaError("unsupported", "rotary_dim must be even, positive and at most head_dim", f"rotary_dim={self.rotary_dim} head_dim={self.head_dim}")
        self._table = None

    def key(self):
        return ("rotary_neox", self.rotary_dim, self.theta, self.max_position)

    def build_table(self, n_positions: int) -> torch.Tensor:
        """[n_positions, rot/2, 2] fp32 (cos, sin) on the device."""
        half = self.rotary_dim // 2
        i = np.arange(half, dtype=np.float64)
        inv = np.float32(1.0) / np.power(np.float64(self.theta), 2.0 * i / self.rotary_dim).astype(np.float32)
        pos = np.arange(n_positions, dtype=np.float32)
        angle = (pos[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)
        table = np.stack([np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)], axis=-1)
        return torch.from_numpy(np.ascontiguousarray(table)).to(self.rt.device)

    def load(self, state):
        # one table per distinct (rot, theta, length) is shared through the state dict
        tables = state.setdefault("__rotary_tables__", {})
        if self.key() not in tables:
            tables[self.key()] = self.build_table(self.max_position)
        self._table = tables[self.key()]

    def rotary_table(self):
        """(table, rotary_dim) for the fused rotate-and-store kernel."""
        return self._table, self.rotary_dim


class RotaryInterleaved(Part):
    """Rotary encoding on neighbouring pairs: dimension 2i goes with 2i + 1, i
    < dims / 2; at position p the pair (u, v) becomes (u cos a - v sin a, v cos
    a + u sin a) with a = p * f_i, f_i = base^(-2i / dims).  f_i is rounded to
    fp32 once (from the power in f64); position, angle, cosine and sine are
    fp32 in the kernels that turn, so no table and no longest position.

    ``layout`` "halves" pairs dimension i with i + dims / 2 instead (kernels
    that take a ``halves`` flag; :meth:`apply` does neighbouring pairs only).
    ``scaling`` = ``{factor, original, fast, slow}`` stretches the slow
    frequencies (YaRN): with ``turns(t) = dims * ln(original / (2 pi t)) / (2 ln
    base)``, ``lo = max(floor(turns(fast)), 0)``, ``hi = min(ceil(turns(slow)),
    dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the
    frequency is ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and cosine and
    sine are multiplied by ``magnitude = 0.1 * ln(factor) + 1``."""

    family = "position"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.dims = int(self.param("dims"))
        self.base = float(self.param("base"))
        self.layout = str(self.params.get("layout", "pairs"))
        self.scaling = self.params.get("scaling")
        if self.dims < 0 or self.dims % 2 or self.base <= 0 or self.layout not in ("pairs", "halves"):
            raise AlofaError("unsupported", "rotary dims must be even, the base positive, the layout 'pairs' or 'halves'", f"dims={self.dims} base={self.base} layout={self.layout}")
        self.magnitude = 1.0
        if self.scaling:
            sc = {k: float(self.scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if min(sc.values()) <= 0 or self.base == 1.0:
                raise AlofaError("invalid_argument", "rotary scaling wants positive numbers and a base other than 1", f"scaling={self.scaling}")
            self.scaling = sc
            self.magnitude = 0.1 * math.log(sc["factor"]) + 1.0
        self._freq = None

    @property
    def halves(self) -> bool:
        return self.layout == "halves"

    def key(self):
        return ("rotary_interleaved", self.dims, self.base, tuple(sorted(self.scaling.items())) if self.scaling else None)

    def make_frequencies(self) -> np.ndarray:
        """f_i, i < dims / 2, in float64 (rounded to fp32 once, by the caller)."""
        i = np.arange(max(self.dims // 2, 1), dtype=np.float64)
        freq = np.power(np.float64(self.base), -2.0 * i / max(self.dims, 1))
        if self.scaling:
            sc = self.scaling

            def turns(t):
                return self.dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(self.base))

            lo = max(math.floor(turns(sc["fast"])), 0)
            hi = min(math.ceil(turns(sc["slow"])), self.dims - 1)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            freq = freq / sc["factor"] * ramp + freq * (1.0 - ramp)
        return freq

    def load(self, state):
        tables = state.setdefault("__rotary_tables__", {})
        if self.key() not in tables:
            tables[self.key()] = torch.from_numpy(self.make_frequencies().astype(np.float32)).to(self.rt.device)
        self._freq = tables[self.key()]

    def frequencies(self) -> torch.Tensor:
        """f_i as fp32 [dims / 2] on the device."""
        return self._freq

    def rotary_table(self):
        return None, 0  # no table: mixers that hold whole heads call apply()

    def apply(self, ctx, q, k):
        """Turn q [T, heads, hd] and k [T, kv_heads, hd] (views) in place."""
        from ..csrc import ops

        if self.halves or self.magnitude != 1.0:
            raise AlofaError("unsupported", "apply() turns neighbouring pairs without a magnitude only", f"layout={self.layout} magnitude={self.magnitude}")

        ops.rotary_interleaved(q, self._freq, ctx.positions, q.shape[1], q.shape[2], self.dims)
        if k.shape[1]:
            ops.rotary_interleaved(k, self._freq, ctx.positions, k.shape[1], k.shape[2], self.dims)


class NoPosition(Part):
    """No position encoding: queries and keys are used as projected."""

    family = "position"
    graph_safe = True

    def rotary_table(self):
        return None, 0


register_part("position", "rotary_neox", RotaryNeox)
register_part("position", "rotary_interleaved", RotaryInterleaved)
register_part("position", "none", NoPosition)
