"""Matrix-memory mixer (the mLSTM of xLSTM): per head a d x dv memory with exponential input and forget gates and a
running maximum that keeps the exponentials in range.

From the mixer's input h: ``q = W_q h * d^(-1/2)``, ``k = W_k h`` (heads x d), ``v = W_v h`` (heads x dv), and per head
the log gates ``i = cap tanh((W_i h + b_i) / cap)``, ``f = logsigmoid(cap tanh((W_f h + b_f) / cap))``. Then, from
S = 0, n = 0, m = 0:
    m_t = max(f + m_(t-1), i)      S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T      n_t likewise with k
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
each head's o divided by its root mean square, the heads side by side times a weight, times sigmoid(W_g h), then W_o.
Gates, exponentials, state and the head norm are 32-bit in both run dtypes; the projections' product keeps its 32-bit
accumulator. Per request the mixer keeps S, n and m in ONE state slot of 32-bit floats (laid out for its kernel,
``ops.matrix_memory_state_floats``), zero for a new request; prompt portions and single decoded tokens run the same
kernel, which walks a request's tokens in order whatever the cut.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import register_mixer
from .base import LayerCache, StepInputs
from .spec import StateNeed, WeightSpec


SLICED_FROM = 256       # a step whose longest portion has this many tokens runs the recurrence over time slices
SLICE_LEN = 128


class MatrixMemoryMixer:
    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, gate_cap: float = 0.0,
                 eps: float = 1e-6, names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if head_dim > 1024:
            raise ValueError("memories of up to 1024 rows per head are built")
        self.hidden_size, self.nh, self.d, self.dv = hidden_size, num_heads, head_dim, value_dim
        self.cap, self.eps = float(gate_cap or 0.0), float(eps)
        self.dtype, self.device = dtype, device
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b",
                      "norm": "norm", "o": "o", **(names or {})}
        self.qk, self.inner = num_heads * head_dim, num_heads * value_dim
        # columns of the projection: [q | k | v | g | i | f]
        self.col = {"q": 0, "k": self.qk, "v": 2 * self.qk, "g": 2 * self.qk + self.inner, "i": 2 * self.qk + 2 * self.inner,
                    "f": 2 * self.qk + 2 * self.inner + num_heads}
        self.proj_width = 2 * self.qk + 2 * self.inner + 2 * num_heads
        self.state_floats = ops.matrix_memory_state_floats(num_heads, head_dim, value_dim)
        self.w_in = self.w_o = self.b_i = self.b_f = self.g = None

    def weight_specs(self) -> list[WeightSpec]:
        n, W = self.names, self.hidden_size
        f32 = dict(dtype="float32")
        return [WeightSpec(n["q"], (self.qk, W), init=("normal", 0.05)), WeightSpec(n["k"], (self.qk, W), init=("normal", 0.05)),
                WeightSpec(n["v"], (self.inner, W), init=("normal", 0.05)),
                WeightSpec(n["g"], (self.inner, W), init=("normal", 0.05)),
                WeightSpec(n["o"], (W, self.inner), init=("normal", 0.05)),
                WeightSpec(n["norm"], (self.inner,), init=("ones_plus_normal", 0.1), **f32),
                WeightSpec(n["i"], (self.nh, W), init=("normal", 0.1)),
                WeightSpec(n["i_bias"], (self.nh,), init=("normal", 1.0), **f32),
                WeightSpec(n["f"], (self.nh, W), init=("normal", 0.1)),
                WeightSpec(n["f_bias"], (self.nh,), init=("normal", 1.0, 3.0), **f32)]

    def cache_need(self):
        return None

    def state_need(self) -> StateNeed:
        return StateNeed((self.state_floats,), "float32")

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((self.proj_width + self.inner) * 4 + (self.inner + self.hidden_size) * elt)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        self.w_o, self.g = tensors[n["o"]], tensors[n["norm"]]
        self.b_i, self.b_f = tensors[n["i_bias"]], tensors[n["f_bias"]]

    def projection_weight(self) -> torch.Tensor:
        """[proj_width, hidden] rows [q; k; v; g; i; f]: what a shared product multiplies for this mixer."""
        return self.w_in

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        return self.forward_projected(ops.linear32(x, self.w_in), step, cache)

    def forward_projected(self, proj: torch.Tensor, step: StepInputs, cache: LayerCache, state_off: int = 0) -> torch.Tensor:
        """``proj`` [T, proj_width] float32 (a view of a wider product is fine); the request's memory starts
        ``state_off`` floats into its slot."""
        T, dev, c = proj.shape[0], proj.device, self.col
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        den = torch.empty((T, self.nh), dtype=torch.float32, device=dev)
        # Long portions: three passes over time slices instead of one walk over the whole portion (kernels/ops.py).
        sliced = {}
        if step.max_q_len >= SLICED_FROM and step.workspace is not None:
            records = ops.matrix_memory_slice_records(T, step.n_seqs, SLICE_LEN)
            sliced = dict(slice_len=SLICE_LEN,
                          slices=step.workspace.get("matrix_memory_slices", records * self.state_floats, torch.float32))
        ops.matrix_memory(proj, q_col=c["q"], k_col=c["k"], v_col=c["v"], i_col=c["i"], f_col=c["f"], i_bias=self.b_i,
                          f_bias=self.b_f, cap=self.cap, q_scale=self.d ** -0.5, state=cache.state, state_off=state_off,
                          cu_q=step.cu_q, state_slots=step.state_slots, y=y, den=den, n_seqs=step.n_seqs, heads=self.nh, dim=self.d,
                          vdim=self.dv, **sliced)
        gated = torch.empty((T, self.inner), dtype=self.dtype, device=dev)
        ops.head_norm_gate(y, proj[:, c["g"]:c["g"] + self.inner], self.g, self.eps, self.nh, gated, den=den)
        return ops.linear(gated, self.w_o)


register_mixer("matrix_memory", MatrixMemoryMixer)
