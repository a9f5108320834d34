"""Rotary position encoding (rotate-half) as a part.

``inv_freq[i] = 1 / theta**(2i/d)`` is formed in float32 on the host exactly as the
reference does (src/mini_engine/model.py:75 of YuvGev00/mini-engine); the angle
``position * inv_freq`` and its cosine and sine are evaluated in 32-bit inside the
attention mixer's fused kernel (:79-90).  Unlike the reference, whose frequency buffer is
cast to bfloat16 together with the module (src/mini_engine/engine.py:63), the table stays
float32 in every mode.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import PositionEncoding, register


@register("position_encoding", "rope")
class RotaryEncoding(PositionEncoding):
    capturable = True

    def __init__(
        self, prefix: str, hidden_size: int, *, head_dim: int, theta: float, rotary_dim: int | None = None,
        wavelength_scaling: Mapping[str, float] | None = None, frequency_divisor: float = 1.0,
    ):  # fmt: skip
        """``rotary_dim`` (default: all of ``head_dim``) is how many leading elements of a head are
        rotated, in two halves of ``rotary_dim / 2``; the rest of the head passes through.  The
        reference rotates the whole head (src/mini_engine/model.py:88-90).

        ``wavelength_scaling`` (``factor``, ``low``, ``high``, ``original``) stretches the slow frequencies for
        contexts longer than the ``original`` one: with wavelength ``l = 2 pi / f``, ``f`` stays where ``l <
        original / high``, becomes ``f / factor`` where ``l > original / low``, and in between is ``(1 - s) f /
        factor + s f`` with ``s = (original / l - low) / (high - low)``.  ``frequency_divisor`` divides every
        frequency (linear position scaling: positions count ``1 / divisor`` as fast)."""
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if head_dim % 2 or rotary_dim % 2 or not 2 <= rotary_dim <= head_dim:
            raise ValueError(f"rotate-half RoPE needs an even rotary_dim <= head_dim, got {rotary_dim} of {head_dim}")
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.divisor = float(frequency_divisor)
        if not self.divisor > 0:
            raise ValueError(f"the frequency divisor must be positive, got {frequency_divisor}")
        self.scaling = None
        if wavelength_scaling is not None:
            self.scaling = tuple(float(wavelength_scaling[key]) for key in ("factor", "low", "high", "original"))
            factor, low, high, original = self.scaling
            if not (factor > 0 and original > 0 and 0 < low < high):
                raise ValueError(f"wavelength scaling needs factor, original > 0 and 0 < low < high, got {self.scaling}")
        self._table: torch.Tensor | None = None

    def inv_freq(self) -> torch.Tensor:
        if self.scaling is None and self.divisor == 1.0:
            exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            return 1.0 / (self.theta**exponents)
        if self.scaling is None:  # in double precision on the host, rounded once
            values = [self.theta ** (-2.0 * i / self.rotary_dim) / self.divisor for i in range(self.rotary_dim // 2)]
            return torch.tensor(values, dtype=torch.float64).to(torch.float32)
        factor, low, high, original = self.scaling
        values = []
        for i in range(self.rotary_dim // 2):  # in double precision on the host, rounded once
            f = self.theta ** (-2.0 * i / self.rotary_dim)
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
            values.append(f / self.divisor)
        return torch.tensor(values, dtype=torch.float64).to(torch.float32)

    def fused_rotary_table(self) -> torch.Tensor:
        if self._table is None:
            self._table = self.inv_freq().to("cuda")
        return self._table

    def step_angles(self, ctx) -> torch.Tensor:
        key = ("rope", self.rotary_dim, self.theta, self.scaling, self.divisor)
        held = ctx.memo.get(key)
        if held is None:
            name = f"rope.angles.{self.rotary_dim}.{self.theta}" + ("" if self.scaling is None else "." + ".".join(map(str, self.scaling))) + ("" if self.divisor == 1.0 else f"./{self.divisor}")
            held = ctx.buffer(name, (ctx.num_tokens, self.rotary_dim // 2, 2), torch.float32)
            ops.rope_table(self.fused_rotary_table(), ctx.positions, held)
            ctx.memo[key] = held
        return held


@register("position_encoding", "none")
class NoEncoding(PositionEncoding):
    """Queries and keys are used as projected (and normalised)."""

    capturable = True

    def __init__(self, prefix: str, hidden_size: int):
        pass

    def apply(self, q, k, positions) -> None:
        return None
