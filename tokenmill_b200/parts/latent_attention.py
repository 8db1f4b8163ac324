"""Attention through low-rank latents, with a sliding window.

Per token, from the mixer's input h (width d):
    c_q = rmsnorm(W_dq h) * g_q                      q = W_uq c_q        -> per head [nope (dim) | rot (rot_dim)]
    [c_raw | k_rot_raw] = W_dkv h                    c = rmsnorm(c_raw) * g_kv         k_rot = rope(k_rot_raw)
    k_nope[head] = W_uk[head] c                      v[head] = W_uv[head] c
    score = (q_nope . k_nope + rope(q_rot) . k_rot) * scale over the last ``window`` positions, softmax, W_o.
The rotation is rotate-half over the first ``rot_dims`` of the rotated part (the rest pass unchanged).

Only [c | k_rot] is cached: one row per token for all heads (a paged cache of one plane, one "head" of width
kv_rank + rot_dim). Keys and values are never expanded. Since q_nope . (W_uk c) = (W_uk^T q_nope) . c and
sum_j p_j W_uv c_j = W_uv sum_j p_j c_j, the two per-head maps are applied to the query and to the attention result
(two small batched products), and the attention kernel works on the cached rows directly. The mapped query keeps
its 32-bit accumulator; scores, softmax and the weighted sum are 32-bit.

Every size and constant is a constructor parameter. The two down-projections are held as one matrix.
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..registry import get_part, register_mixer
from .base import LayerCache, StepInputs, StepMetadata, StepShape, part_limit_positions, part_max_positions
from .spec import PagedKVNeed, PartSpec, StateNeed, WeightSpec


SPLIT_BLOCKS = 296      # blocks the tensor-core kernel should have in flight before its keys stop being dealt out


class LatentAttention:
    def __init__(self, *, hidden_size: int, num_heads: int, nope_dim: int, rot_dim: int, value_dim: int, q_rank: int,
                 kv_rank: int, window: int | None, scale: float, eps: float, position: PartSpec, rot_dims: int | None = None,
                 names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        self.hidden_size, self.nh = hidden_size, num_heads
        self.dn, self.dr, self.dv = nope_dim, rot_dim, value_dim
        self.q_rank, self.rank = q_rank, kv_rank
        self.window = int(window) if window else 0
        self.scale, self.eps = float(scale), float(eps)
        self.rot_dims = rot_dim if rot_dims is None else int(rot_dims)
        if self.rot_dims % 2 or self.rot_dims > rot_dim:
            raise ValueError(f"rot_dims ({self.rot_dims}) must be even and at most rot_dim ({rot_dim})")
        if kv_rank > 512:
            raise ValueError(f"kv_rank up to 512 is built, got {kv_rank}")
        self.dtype, self.device = dtype, device
        self.position = get_part("position", position.kind)(**position.params)
        # checkpoint names of the tensors, relative to the mixer's prefix
        self.names = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                      "uv": "uv", "o": "o", **(names or {})}
        # bfloat16 with both parts of a cache row multiples of 16 wide: tensor cores; anything else (and the 32-bit
        # path): the shape-generic kernel on CUDA cores
        self.tensor_cores = ops.latent_attention_tc_ok(dtype, kv_rank, rot_dim)
        self.tile_rows = ops.LATENT_TC_TILE_ROWS if self.tensor_cores else ops.LATENT_TILE_ROWS
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None
        self.g_q = self.g_kv = self.cos = self.sin = None

    def weight_specs(self) -> list[WeightSpec]:
        n, H, nh = self.names, self.hidden_size, self.nh
        return [WeightSpec(n["dq"], (self.q_rank, H)),
                WeightSpec(n["dq_norm"], (self.q_rank,), dtype="float32", init=("ones_plus_normal", 0.1)),
                WeightSpec(n["uq"], (nh * (self.dn + self.dr), self.q_rank), init=("normal", 0.1)),
                WeightSpec(n["dkv"], (self.rank + self.dr, H)),
                WeightSpec(n["dkv_norm"], (self.rank,), dtype="float32", init=("ones_plus_normal", 0.1)),
                WeightSpec(n["uk"], (nh * self.dn, self.rank), init=("normal", 0.1)),
                WeightSpec(n["uv"], (nh * self.dv, self.rank), init=("normal", 0.1)),
                WeightSpec(n["o"], (H, nh * self.dv), init=("normal", 0.05))]

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(1, self.rank + self.dr, self.window or None, planes=1)

    def state_need(self) -> StateNeed | None:
        return None

    def max_positions(self) -> int | None:
        return part_max_positions(self.position)

    def limit_positions(self, n: int) -> None:
        part_limit_positions(self.position, n)

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        per = (self.q_rank + self.rank + self.dr) * 2 + self.nh * (self.dn + self.dr + self.rank + self.dv) + self.hidden_size
        return n_tokens * (per * elt + self.nh * self.rank * 4)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n, nh = self.names, self.nh
        self.w_down = torch.cat([tensors[n["dq"]], tensors[n["dkv"]]], dim=0).contiguous()
        self.g_q, self.g_kv = tensors[n["dq_norm"]], tensors[n["dkv_norm"]]
        self.w_uq = tensors[n["uq"]]
        # [heads, rank, dim]: the key map transposed, so that it maps a query head into the latent space
        self.w_uk_t = tensors[n["uk"]].view(nh, self.dn, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(nh, self.dv, self.rank).contiguous()
        self.w_o = tensors[n["o"]]
        self.cos, self.sin = self.position.tables(self.device)

    # --- per-step work list -----------------------------------------------------------------------------------

    def metadata_key(self):
        return ("latent_attention", self.nh, self.tile_rows)

    def step_metadata(self, shape: StepShape) -> StepMetadata:
        """Row tiles of the attention kernel: ``tile_rows`` consecutive (token, head) rows of one request each."""
        per_seq = (shape.q_lens.astype(np.int64) * self.nh + self.tile_rows - 1) // self.tile_rows
        tile_seq = np.repeat(np.arange(len(per_seq), dtype=np.int32), per_seq)
        first = np.cumsum(per_seq) - per_seq
        tile_row0 = ((np.arange(tile_seq.size) - np.repeat(first, per_seq)) * self.tile_rows).astype(np.int32)
        # Few row tiles (decoding): deal each tile's keys out over enough blocks to put two on every multiprocessor.
        # (A captured graph serves every context: it takes the split for the longest.)
        n_tiles, splits = int(tile_seq.size), 1
        if self.tensor_cores and n_tiles:
            chunks = ops.latent_attention_tc_chunks(self.rank)
            if shape.for_graph:
                longest = shape.max_kv_len
            else:
                longest = int((shape.starts.astype(np.int64) + shape.q_lens).max())
            keys = min(longest, self.window + self.tile_rows // self.nh + 1) if self.window else longest
            key_tiles = keys // 32 + 2
            splits = max(1, min(key_tiles // 2, SPLIT_BLOCKS // (n_tiles * chunks), 32))
        return StepMetadata({"tile_seq": tile_seq, "tile_row0": tile_row0}, {"n_tiles": n_tiles, "n_splits": splits},
                            constant_in_graph=True)

    # --- run --------------------------------------------------------------------------------------------------

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        T, nh, dev = x.shape[0], self.nh, x.device
        down = ops.linear(x, self.w_down)                                   # [T, q_rank + rank + rot]
        cq = torch.empty((T, self.q_rank), dtype=self.dtype, device=dev)
        slot_map = step.slot_maps[cache.group] if cache.writes else torch.full((T,), -1, dtype=torch.int32, device=dev)
        ops.latent_prepare(down, self.q_rank, self.rank, self.dr, self.rot_dims, self.g_q, self.g_kv, self.eps,
                           step.positions, self.cos, self.sin, slot_map, cq, cache.k)
        q = ops.linear(cq, self.w_uq).view(T, nh, self.dn + self.dr)
        if self.dtype == torch.float32:
            q_lat = ops.bmm_nt(q[:, :, :self.dn].transpose(0, 1), self.w_uk_t,
                               torch.empty((nh, T, self.rank), dtype=torch.float32, device=dev))
        else:       # the library's batched product keeps its 32-bit accumulator as the result
            q_lat = torch.bmm(q[:, :, :self.dn].transpose(0, 1), self.w_uk_t.transpose(1, 2), out_dtype=torch.float32)
        meta = step.meta[self.metadata_key()]
        o_lat = torch.empty((nh, T, self.rank), dtype=self.dtype, device=dev)
        splits, part = meta.host["n_splits"], None
        if splits > 1:
            part = step.workspace.get("latent_attention_part", meta.host["n_tiles"] * splits * self.tile_rows * (self.rank + 2),
                                      torch.float32)
        ops.latent_attention(q_lat.transpose(0, 1), q[:, :, self.dn:], self.cos, self.sin, self.rot_dims, cache.k,
                             step.block_tables[cache.group], step.cu_q, step.kv_before, meta.arrays["tile_seq"],
                             meta.arrays["tile_row0"], meta.host["n_tiles"], o_lat.transpose(0, 1), scale=self.scale,
                             window=self.window, tensor_cores=self.tensor_cores, n_splits=splits, part=part)
        heads = torch.empty((T, nh, self.dv), dtype=self.dtype, device=dev)
        ops.bmm_nt(o_lat, self.w_uv, heads.transpose(0, 1))
        return ops.linear(heads.view(T, nh * self.dv), self.w_o)


register_mixer("latent_attention", LatentAttention)
