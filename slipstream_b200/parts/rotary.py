"""Rotary position encoding.  Pairing: half-split (element d with d + D/2, the default) or interleaved
(element 2i with 2i + 1).  ``YarnRotaryEncoding`` stretches the slow frequencies of a longer context.

Inverse frequencies ``1 / theta**(2i/D)`` are formed in float32 on the host
exactly as the reference does (slipstream/models/layers/rope.py:39-42); angles,
cosines and sines are float32 inside the kernel (:93-106), which also writes the
rotated keys and the values to their cache pages.
"""

from __future__ import annotations

import math

import torch

from .base import POSITION_ENCODINGS, PositionEncoding, Runtime


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    cuda_graph_safe = True

    mscale = 1.0  # factor on every cosine and sine

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None, interleaved: bool = False,
                 exact_table: bool = False, stretch: float = 1.0) -> None:
        """``stretch``: every frequency is divided by it (positions stretched linearly; with ``exact_table``).
        ``exact_table``: form the frequencies in double precision and round them once, instead of in float32.
        ``interleaved``: neighbouring elements (2i, 2i+1) form a pair instead of (i, i + rotary_dim/2).  The
        fused rotary kernels of the plain attention path take the half-split pairing only; an attention part
        asks ``plain`` before it uses them."""
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        self.interleaved = bool(interleaved)
        self.exact_table = bool(exact_table)
        self.stretch = float(stretch)
        if not self.stretch > 0.0 or (self.stretch != 1.0 and not exact_table):
            raise ValueError("stretch must be positive, and comes with exact_table")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim must be even and in (0, {head_dim}], got {self.rotary_dim}")
        self.inv_freq: torch.Tensor | None = None

    @property
    def plain(self) -> bool:
        """Half-split pairs with unscaled cosines and sines: what every rotary kernel of the package computes."""
        return not self.interleaved and self.mscale == 1.0

    def inverse_frequencies(self) -> torch.Tensor:
        if self.exact_table:
            dims = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
            return (self.theta ** (-dims / self.rotary_dim) / self.stretch).to(torch.float32)
        dims = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        return 1.0 / (self.theta ** (dims / self.rotary_dim))

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.inv_freq = self.inverse_frequencies().to(runtime.device)

    def rotary_table(self) -> tuple[torch.Tensor | None, int]:
        return self.inv_freq, self.rotary_dim


@POSITION_ENCODINGS.register("yarn_rotary")
class YarnRotaryEncoding(RotaryEncoding):
    """Rotary frequencies blended between the trained ones and those of a context ``factor`` times longer.

    With f_i = theta^(-2i/d) over the d rotated elements, and dim(t) = d ln(original / (2 pi t)) / (2 ln theta) the
    (fractional) pair index whose wave turns t times within ``original`` positions:
    lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), d - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    frequency_i = f_i / factor * ramp_i + f_i * (1 - ramp_i): pairs that turn often within the trained context
    keep their frequency, pairs that turn rarely are slowed by ``factor``.  Every cosine and sine is multiplied by
    0.1 ln(factor) + 1.  The table is formed in double precision on the host and rounded to float32 once."""

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None, interleaved: bool = False, *,
                 factor: float, original: float, fast: float, slow: float) -> None:
        super().__init__(head_dim, theta, rotary_dim, interleaved)
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)
        if self.factor <= 0.0 or self.original <= 0.0 or self.fast <= 0.0 or self.slow <= 0.0:
            raise ValueError("factor, original, fast and slow must be positive")
        self.mscale = 0.1 * math.log(self.factor) + 1.0

    def _turn_dim(self, turns: float) -> float:
        return self.rotary_dim * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

    def inverse_frequencies(self) -> torch.Tensor:
        d = self.rotary_dim
        i = torch.arange(d // 2, dtype=torch.float64)
        f = self.theta ** (-2.0 * i / d)
        lo = max(math.floor(self._turn_dim(self.fast)), 0)
        hi = min(math.ceil(self._turn_dim(self.slow)), d - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return (f / self.factor * ramp + f * (1.0 - ramp)).to(torch.float32)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """Queries and keys are used as projected."""

    cuda_graph_safe = True
