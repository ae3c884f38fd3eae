"""Rotary position encoding tables (reference model/model_architecture.cpp:67-75): inv_freq_i = theta^(-2i/rot),
angle = position * inv_freq in float64, cos and sin stored as float32 [max_positions, rot/2].  The rotation
itself happens inside the mixer's fused projection epilogue, which reads these tables; ``pairing`` says which
elements form a pair: "half" pairs (i, i + rot/2) as the reference does (fused_ops.cu:157-166), "interleaved"
pairs (2i, 2i+1).

``rotary_blended`` stretches the slow pairs for contexts longer than the one trained on: with pair_of(turns) =
rot * ln(original / (2 pi turns)) / (2 ln theta), lo = max(floor(pair_of(fast)), 0), hi = min(ceil(pair_of(slow)), rot - 1)
and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at inv_freq_i * ((1 - ramp_i) + ramp_i / factor), and
cos and sin are multiplied by 0.1 ln(factor) + 1.  A model that names no position limit gets tables as long as the engine's
longest sequence (``Runtime.max_positions``)."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_part


@register_part("position", "rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, runtime, prefix="", names=None, *, rotary_dim: int, theta: float, max_positions: int = 0,
                 pairing: str = "half"):
        super().__init__(runtime, prefix, names)
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing must be 'half' or 'interleaved', got {pairing!r}")
        self.rotary_dim, self.theta, self.pairing = int(rotary_dim), float(theta), pairing
        self.max_positions = int(max_positions) or int(runtime.max_positions)      # no limit named: the engine's longest sequence
        idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), idx / self.rotary_dim).reciprocal()
        angle = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), inv_freq)
        self.cos = angle.cos().to(torch.float32).contiguous().to(runtime.device)
        self.sin = angle.sin().to(torch.float32).contiguous().to(runtime.device)

    @property
    def interleaved(self) -> bool:
        return self.pairing == "interleaved"


@register_part("position", "rotary_blended")
class BlendedRotaryEmbedding(PositionEncoding):
    def __init__(self, runtime, prefix="", names=None, *, rotary_dim: int, theta: float, max_positions: int = 0,
                 factor: float = 1.0, original: float = 0.0, fast: float = 0.0, slow: float = 0.0, pairing: str = "interleaved"):
        super().__init__(runtime, prefix, names)
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing must be 'half' or 'interleaved', got {pairing!r}")
        self.rotary_dim, self.theta, self.pairing = int(rotary_dim), float(theta), pairing
        self.max_positions = int(max_positions) or int(runtime.max_positions)
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)
        idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), idx / self.rotary_dim).reciprocal()
        magnitude = 1.0
        if self.original > 0 and self.factor > 0:
            def pair_of(turns: float) -> float:
                return self.rotary_dim * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(pair_of(self.fast)), 0)
            hi = min(math.ceil(pair_of(self.slow)), self.rotary_dim - 1)
            ramp = ((torch.arange(self.rotary_dim // 2, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            inv_freq = inv_freq / self.factor * ramp + inv_freq * (1.0 - ramp)
            magnitude = 0.1 * math.log(self.factor) + 1.0
        angle = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), inv_freq)
        self.cos = (angle.cos() * magnitude).to(torch.float32).contiguous().to(runtime.device)
        self.sin = (angle.sin() * magnitude).to(torch.float32).contiguous().to(runtime.device)

    @property
    def interleaved(self) -> bool:
        return self.pairing == "interleaved"
