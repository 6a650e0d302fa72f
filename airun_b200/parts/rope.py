"""Rotary position encoding with the NeoX pairing.

Pair i couples dimensions i and i + r/2 of a head; the angle is
pos * inv_freq[i] with inv_freq[i] = theta^(-2i/r); dimensions >= r are left
alone (crates/airun-cuda/kernels/ops.cu:158-184,
crates/airun-cuda/kernels/airun.cuh:147-163).  inv_freq is computed once in
double precision and rounded to float32; the position is multiplied in float32
on the device, where the accurate sincosf is used.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..kernels import ops
from .base import PositionEncoding, register_part


class RotaryNeox(PositionEncoding):
    kind = ops.ROPE_NEOX

    def __init__(self, prefix: str = "", rotary_dim: int = 0, theta: float = 10000.0,
                 dtype=None, device=None):
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be a positive even number, found {rotary_dim}")
        self.rotary_dim, self.theta = int(rotary_dim), float(theta)
        i = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / rotary_dim)
        self.inv_freq = inv.to(torch.float32).to(device)

    def fused(self) -> Optional[Tuple[int, int, Optional[torch.Tensor]]]:
        return self.kind, self.rotary_dim, self.inv_freq


class RotaryInterleaved(RotaryNeox):
    """The same angles with the older pairing of neighbouring dimensions (2i, 2i + 1), which the reference
    keeps as a kernel parameter beside the NeoX pairing (crates/airun-cuda/kernels/ops.cu:154-157, :176-179).
    The dense Qwen3 decoder does not use it."""
    kind = ops.ROPE_INTERLEAVED


class NoPosition(PositionEncoding):
    def __init__(self, prefix: str = "", dtype=None, device=None):
        pass

    def fused(self):
        return ops.ROPE_NONE, 0, None


register_part("position", "rotary_neox", RotaryNeox)
register_part("position", "rotary_interleaved", RotaryInterleaved)
register_part("position", "none", NoPosition)


class RotaryScaledInterleaved(RotaryInterleaved):
    """Neighbouring dimensions (2i, 2i + 1) with frequencies stretched for longer contexts than the model was
    trained on: with ``scaling`` = {factor, original, fast, slow}, a pair that turns more than ``fast`` times over
    ``original`` positions keeps its frequency, one that turns fewer than ``slow`` times has it divided by
    ``factor``, and the pairs between are blended linearly by their index,

        at(t) = dims * ln(original / (2 pi t)) / (2 ln theta),  lo = max(floor(at(fast)), 0),
        hi = min(ceil(at(slow)), dims - 1),  ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
        f_i' = f_i / factor * ramp_i + f_i * (1 - ramp_i);

    cos and sin are both multiplied by ``mult`` = 0.1 ln(factor) + 1.  Without ``scaling`` it is RotaryInterleaved
    with mult 1.  Everything is computed once in double precision and rounded to float32."""

    def __init__(self, prefix: str = "", rotary_dim: int = 0, theta: float = 10000.0, scaling: Optional[dict] = None,
                 dtype=None, device=None):
        import math
        super().__init__(prefix, rotary_dim, theta, dtype, device)
        self.mult = 1.0
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])
            fast, slow = float(scaling["fast"]), float(scaling["slow"])
            if not (factor > 0 and original > 0 and fast > 0 and slow > 0):
                raise ValueError("factor, original, fast and slow of a rotary scaling must be positive")

            def at(turns: float) -> float:
                return rotary_dim * math.log(original / (2 * math.pi * turns)) / (2 * math.log(self.theta))

            lo = max(math.floor(at(fast)), 0)
            hi = min(math.ceil(at(slow)), rotary_dim - 1)
            i = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
            f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / rotary_dim)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            self.inv_freq = (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32).to(device)
            self.mult = 0.1 * math.log(factor) + 1.0


register_part("position", "rotary_scaled_interleaved", RotaryScaledInterleaved)
