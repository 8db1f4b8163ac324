"""Rotate-half rotary position encoding: the 32-bit angle tables.

``inv_freq_i = 1 / theta^(2i / D)`` computed as ``1.0 / (theta ** (arange(0, D, 2).float() / D))``,
``angle = position.float() * inv_freq`` and 32-bit cos / sin, exactly as the reference builds its
tables (src/infer/model/layers.py:47-52). The reference's table repeats each half ([P, D]); only the
distinct half [P, D/2] is kept here. The rotation itself runs inside the mixer's fused kernel.
"""

from __future__ import annotations

import torch

from ..registry import register_position_encoding

_TABLES: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


class RotaryEmbedding:
    def __init__(self, *, head_dim: int, theta: float, max_positions: int, precise: bool = False,
                 scaling: dict | None = None):
        if head_dim % 2:
            raise ValueError(f"rotary position encoding needs an even head_dim, got {head_dim}")
        self.head_dim = head_dim
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        # precise: frequencies and angles in 64-bit, rounded once to the 32-bit tables (for designs that define the
        # angle as position * theta^(-2i/D) without naming an order of 32-bit operations)
        self.precise = bool(precise)
        # scaling {factor, low, high, original}: frequencies rescaled by wavelength (the Llama 3.1 rule). With wavelength
        # l = 2 pi / f: f is kept where l < original / high, divided by factor where l > original / low, and in between
        # blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low). Computed in 64-bit.
        self.scaling = None
        if scaling is not None:
            missing = [k for k in ("factor", "low", "high", "original") if k not in scaling]
            if missing:
                raise ValueError(f"rotary frequency scaling lacks {missing}")
            self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
            if self.scaling["high"] == self.scaling["low"] or self.scaling["factor"] <= 0:
                raise ValueError("rotary frequency scaling needs high != low and a positive factor")
            self.precise = True

    def limit_positions(self, n: int) -> None:
        """No position >= n will be asked for: the tables are built that short
        (src/infer/model/qwen2.py:34: min(max_positions, max_position_embeddings))."""
        self.max_positions = max(1, min(self.max_positions, int(n)))

    def scaled(self, inv_freq: torch.Tensor) -> torch.Tensor:
        """The frequencies after the wavelength rule (64-bit in, 64-bit out)."""
        import math
        sc = self.scaling
        wave = 2.0 * math.pi / inv_freq
        s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
        blend = (1.0 - s) * inv_freq / sc["factor"] + s * inv_freq
        out = torch.where(wave > sc["original"] / sc["low"], inv_freq / sc["factor"], blend)
        return torch.where(wave < sc["original"] / sc["high"], inv_freq, out)

    def tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
        """(cos, sin), each [max_positions, head_dim / 2] float32 on ``device``; shared between layers."""
        key = (self.head_dim, self.theta, self.max_positions, str(device), self.precise,
               tuple(sorted(self.scaling.items())) if self.scaling else None)
        if key not in _TABLES and self.precise:
            inv_freq = self.theta ** (-torch.arange(0, self.head_dim, 2, dtype=torch.float64) / self.head_dim)
            if self.scaling is not None:
                inv_freq = self.scaled(inv_freq)
            freqs = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), inv_freq)
            _TABLES[key] = (freqs.cos().float().to(device).contiguous(), freqs.sin().float().to(device).contiguous())
        if key not in _TABLES:
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.int64).float()
                                             / self.head_dim))
            freqs = torch.outer(torch.arange(self.max_positions).float(), inv_freq)
            _TABLES[key] = (freqs.cos().to(device).contiguous(), freqs.sin().to(device).contiguous())
        return _TABLES[key]


register_position_encoding("rope", RotaryEmbedding)
