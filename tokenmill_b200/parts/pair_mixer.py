"""Two mixers side by side: both read the same input, and the result is half the sum of their outputs, each first
RMS-normed over the model width with a plain weight of its own (``<left>.out`` / ``<right>.out``).

The two may be any registered mixers; their tensors live under the sub-prefixes ``left`` and ``right``. At most one of
them keeps pages and at most one keeps per-request state: the pair hands its ``LayerCache`` to both. Mixers that can
take their columns of a shared product (``projection_weight`` / ``forward_projected``) are fed from ONE matrix product
over the concatenated weights, which keeps its 32-bit accumulator.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import get_part, register_mixer
from .base import LayerCache, StepInputs, part_activation_bytes
from .spec import PartSpec, WeightSpec


class PairMixer:
    def __init__(self, *, hidden_size: int, eps: float, left: PartSpec, right: PartSpec, names: dict[str, str] | None = None,
                 dtype: torch.dtype, device: torch.device):
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.dtype, self.device = dtype, device
        self.names = {"left": "left", "right": "right", "left_out": "left.out", "right_out": "right.out", **(names or {})}
        self.sides = [get_part("mixer", s.kind)(dtype=dtype, device=device, **s.params) for s in (left, right)]
        if sum(m.cache_need() is not None for m in self.sides) > 1 or sum(m.state_need() is not None for m in self.sides) > 1:
            raise ValueError("of two mixers side by side at most one keeps pages and at most one keeps state")
        self.shared = all(callable(getattr(m, "forward_projected", None)) for m in self.sides)
        self.w_out: list = [None, None]
        self.w_in = None

    def sub_parts(self) -> list:
        return list(self.sides)

    def weight_specs(self) -> list[WeightSpec]:
        out = []
        for key, m in zip(("left", "right"), self.sides):
            out += [WeightSpec(f"{self.names[key]}.{w.name}", w.shape, w.dtype, w.init) for w in m.weight_specs()]
        out += [WeightSpec(self.names[k], (self.hidden_size,), dtype="float32", init=("ones_plus_normal", 0.1))
                for k in ("left_out", "right_out")]
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for key, m in zip(("left", "right"), self.sides):
            m.bind({w.name: tensors[f"{self.names[key]}.{w.name}"] for w in m.weight_specs()})
        self.w_out = [tensors[self.names["left_out"]], tensors[self.names["right_out"]]]
        if self.shared:
            self.w_in = torch.cat([m.projection_weight() for m in self.sides], dim=0).contiguous()

    def cache_need(self):
        return next((n for n in (m.cache_need() for m in self.sides) if n is not None), None)

    def state_need(self):
        return next((n for n in (m.state_need() for m in self.sides) if n is not None), None)

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return sum(part_activation_bytes(m, n_tokens, self.hidden_size) for m in self.sides) + 3 * n_tokens * self.hidden_size * elt

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        if self.shared:
            proj = ops.linear32(x, self.w_in)
            split = self.sides[0].proj_width
            a = self.sides[0].forward_projected(proj[:, :split], step, cache)
            b = self.sides[1].forward_projected(proj[:, split:], step, cache)
        else:
            a, b = (m.forward(x, step, cache) for m in self.sides)
        return ops.norm_pair_mean(a, b, self.w_out[0], self.w_out[1], self.eps, torch.empty_like(a))


register_mixer("pair", PairMixer)
