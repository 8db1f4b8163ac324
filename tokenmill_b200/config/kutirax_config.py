"""Typed configuration of the Kutirax decoder, read from the keys of its config.json.

    architecture    "Kutirax"
    vocab, width    vocabulary and residual width
    norm.eps        eps of every RMS norm
    residual_mult   multiplier of a layer's summed branches
    layers          one entry per layer: type ("latent_attention" | "mamba2"), mixer (its sizes), mlp (null, or
                    kind "dense" with ff, or kind "moe" with expert.ff, router.experts, router.top)
    latent_attention mixer: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask.size, rot.base, rot.dims
    mamba2 mixer:           heads, vdim, state, groups, conv, norm_groups

Every size and constant comes from the file; a key the design does not have is refused rather than ignored.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .model_config import ConfigError

MAX_POSITIONS = 1 << 20        # the design names no limit; position tables are sized for the engine's own


def _need(d: dict, keys: tuple[str, ...], where: str) -> None:
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks key(s) {missing}")


def _only(d: dict, keys: tuple[str, ...], where: str) -> None:
    extra = sorted(set(d) - set(keys))
    if extra:
        raise ConfigError(f"config.json: {where} has key(s) this design does not know: {extra}")


def _pos_int(v: Any, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


@dataclass
class KutiraxLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass
class KutiraxConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: list[KutiraxLayer] = field(default_factory=list)
    max_positions: int = MAX_POSITIONS
    eos_token_ids: list[int] = field(default_factory=list)
    architecture: str = "Kutirax"

    @classmethod
    def from_dict(cls, raw: dict[str, Any], generation: dict[str, Any] | None = None) -> "KutiraxConfig":
        _need(raw, ("vocab", "width", "layers", "norm", "residual_mult"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        layers = []
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(entry, ("type", "mixer"), where)
            m = entry["mixer"]
            if entry["type"] == "latent_attention":
                keys = ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "mask", "rot")
                _need(m, keys, where + ".mixer")
                _only(m, keys, where + ".mixer")
                _need(m["mask"], ("size",), where + ".mixer.mask")
                _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                    _pos_int(m[k], f"{where}.mixer.{k}")
                _pos_int(m["mask"]["size"], f"{where}.mixer.mask.size")
                if m["rot"]["dims"] % 2 or not 0 < m["rot"]["dims"] <= m["rot_dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most rot_dim")
            elif entry["type"] == "mamba2":
                keys = ("heads", "vdim", "state", "groups", "conv", "norm_groups")
                _need(m, keys, where + ".mixer")
                _only(m, keys, where + ".mixer")
                for k in keys:
                    _pos_int(m[k], f"{where}.mixer.{k}")
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"config.json: {where}.mixer: heads must divide by groups, heads * vdim by norm_groups")
            else:
                raise ConfigError(f"config.json: {where}.type {entry['type']!r} is not a mixer of this design")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ("ff",), where + ".mlp")
                    _pos_int(mlp["ff"], f"{where}.mlp.ff")
                elif mlp["kind"] == "moe":
                    _need(mlp, ("expert", "router"), where + ".mlp")
                    _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                    _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                    _pos_int(mlp["expert"]["ff"], f"{where}.mlp.expert.ff")
                    if not 1 <= _pos_int(mlp["router"]["top"], f"{where}.mlp.router.top") <= \
                            _pos_int(mlp["router"]["experts"], f"{where}.mlp.router.experts"):
                        raise ConfigError(f"config.json: {where}.mlp.router.top exceeds the number of experts")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
            layers.append(KutiraxLayer(entry["type"], dict(m), dict(mlp) if mlp is not None else None))
        eos = []
        for src in (generation or {}, raw):
            v = src.get("eos_token_id")
            if v is not None:
                eos += v if isinstance(v, list) else [v]
        eps = float(raw["norm"]["eps"])
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        return cls(vocab=_pos_int(raw["vocab"], "vocab"), width=_pos_int(raw["width"], "width"), eps=eps,
                   residual_mult=float(raw["residual_mult"]), layers=layers,
                   max_positions=int(raw.get("max_positions", MAX_POSITIONS)), eos_token_ids=sorted(set(eos)))
