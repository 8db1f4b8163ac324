"""Typed configuration of the Bobunex decoder, read from the keys of its config.json.

    architecture      "Bobunex"
    vocab, width      vocabulary and residual width
    norm.eps          eps of every RMS norm
    embedding.scale   multiplier of the embedding rows
    canon.taps        taps of the causal convolution in front of every sublayer
    layers            one entry per layer: type ("parallel"), mixer (its sizes), mlp (null, or kind "dense" with ff)
    parallel mixer    left  (attention): heads, kv_heads, dim, vdim, scale, softcap, mask.size, mask.keep_first,
                                         rot.base, rot.dims, rot.scaling {factor, low, high, original} (optional)
                      right (matrix memory): heads, dim, vdim, gate_cap

Every size and constant comes from the file; a layer type or feed-forward kind the design does not have is refused.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .kutirax_config import MAX_POSITIONS, _need, _pos_int
from .model_config import ConfigError


@dataclass
class BobunexLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass
class BobunexConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    taps: int
    layers: list[BobunexLayer] = field(default_factory=list)
    max_positions: int = MAX_POSITIONS
    eos_token_ids: list[int] = field(default_factory=list)
    architecture: str = "Bobunex"

    @classmethod
    def from_dict(cls, raw: dict[str, Any], generation: dict[str, Any] | None = None) -> "BobunexConfig":
        _need(raw, ("vocab", "width", "layers", "norm", "embedding", "canon"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        _need(raw["embedding"], ("scale",), "embedding")
        _need(raw["canon"], ("taps",), "canon")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(entry, ("type", "mixer"), where)
            if entry["type"] != "parallel":
                raise ConfigError(f"config.json: {where}.type {entry['type']!r} is not a mixer of this design")
            m = entry["mixer"]
            _need(m, ("left", "right"), where + ".mixer")
            left, right = m["left"], m["right"]
            _need(left, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"), where + ".mixer.left")
            _need(left["mask"], ("size",), where + ".mixer.left.mask")
            _need(left["rot"], ("base", "dims"), where + ".mixer.left.rot")
            for k in ("heads", "kv_heads", "dim", "vdim"):
                _pos_int(left[k], f"{where}.mixer.left.{k}")
            _pos_int(left["mask"]["size"], f"{where}.mixer.left.mask.size")
            keep = left["mask"].get("keep_first", 0) or 0
            if not isinstance(keep, int) or keep < 0:
                raise ConfigError(f"config.json: {where}.mixer.left.mask.keep_first must be a non-negative integer")
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"config.json: {where}.mixer.left: heads must be a multiple of kv_heads")
            dims = left["rot"]["dims"]
            if not isinstance(dims, int) or dims % 2 or not 0 <= dims <= left["dim"]:
                raise ConfigError(f"config.json: {where}.mixer.left.rot.dims must be even and at most dim")
            scaling = left["rot"].get("scaling")
            if scaling is not None:
                _need(scaling, ("factor", "low", "high", "original"), where + ".mixer.left.rot.scaling")
            _need(right, ("heads", "dim", "vdim"), where + ".mixer.right")
            for k in ("heads", "dim", "vdim"):
                _pos_int(right[k], f"{where}.mixer.right.{k}")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
                _need(mlp, ("ff",), where + ".mlp")
                _pos_int(mlp["ff"], f"{where}.mlp.ff")
            layers.append(BobunexLayer(entry["type"], {"left": dict(left), "right": dict(right)},
                                       dict(mlp) if mlp is not None else None))
        eos = []
        for src in (generation or {}, raw):
            v = src.get("eos_token_id")
            if v is not None:
                eos += v if isinstance(v, list) else [v]
        eps = float(raw["norm"]["eps"])
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        return cls(vocab=_pos_int(raw["vocab"], "vocab"), width=_pos_int(raw["width"], "width"), eps=eps,
                   embedding_scale=float(raw["embedding"]["scale"]), taps=_pos_int(raw["canon"]["taps"], "canon.taps"),
                   layers=layers, max_positions=int(raw.get("max_positions", MAX_POSITIONS)), eos_token_ids=sorted(set(eos)))
