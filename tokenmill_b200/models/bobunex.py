"""Bobunex as data: config.json -> ``ModelSpec``.

A pre-norm decoder whose sublayers read their normed input through a short causal convolution and enter the stream
through a learned gate (block ``conv_gated``). The mixer of a layer is a pair side by side: windowed grouped-query
attention (norm over the whole q and k projections, partial rotation with wavelength-scaled frequencies, capped
scores, kept first tokens, a sink in the softmax, a gate per head) and a matrix memory; their outputs are RMS-normed
and averaged. The feed-forward is a gated dense layer with the tanh form of gelu, or absent. Embedding rows are
multiplied by a constant; the output matrix is a tensor of its own. Tensor names: ``embed``, ``final.norm``, ``head``,
and per layer ``l<i>.{norm1, norm2, canon1, canon2, rg1, rg1.b, rg2, rg2.b, mix.left.*, mix.right.*, mlp.*}``.
"""

from __future__ import annotations

from ..config.bobunex_config import BobunexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture


def bobunex_spec(cfg: BobunexConfig) -> ModelSpec:
    d = cfg.width
    norm = PartSpec("rmsnorm_gated", {"hidden_size": d, "eps": cfg.eps, "weight_name": ""})
    layers, unused = [], []
    for i, layer in enumerate(cfg.layers):
        a, r = layer.mixer["left"], layer.mixer["right"]
        rope = None
        if a["rot"]["dims"] > 0:
            rope = PartSpec("rope", {"head_dim": a["rot"]["dims"], "theta": float(a["rot"]["base"]),
                                     "max_positions": cfg.max_positions, "precise": True,
                                     "scaling": a["rot"].get("scaling")})
        left = PartSpec("sink_window_attention", {
            "hidden_size": d, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"],
            "value_dim": a["vdim"], "scale": float(a["scale"]), "position": rope, "rot_dims": a["rot"]["dims"],
            "window": a["mask"]["size"], "keep_first": a["mask"].get("keep_first", 0) or 0,
            "softcap": float(a.get("softcap") or 0.0), "sink": True, "qk_norm": True, "head_gate": True, "eps": cfg.eps})
        right = PartSpec("matrix_memory", {"hidden_size": d, "num_heads": r["heads"], "head_dim": r["dim"],
                                           "value_dim": r["vdim"], "gate_cap": float(r.get("gate_cap") or 0.0),
                                           "eps": cfg.eps})
        mixer = PartSpec("pair", {"hidden_size": d, "eps": cfg.eps, "left": left, "right": right})
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("glu", {"hidden_size": d, "intermediate_size": layer.mlp["ff"], "activation": "gelu_tanh"})
        if ffn is None:     # a file may still carry the absent sublayer's norm, convolution and gate: they are not loaded
            unused += [f"l{i}.norm2", f"l{i}.canon2", f"l{i}.rg2", f"l{i}.mlp."]
        layers.append(LayerSpec(prefix=f"l{i}", block="conv_gated", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm if ffn is not None else None, mixer_name="mix",
                                feed_forward_name="mlp", mixer_norm_name="norm1", feed_forward_norm_name="norm2",
                                block_params={"hidden_size": d, "taps": cfg.taps}))
    return ModelSpec(architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=layers, run_order=[RunEntry(i) for i in range(len(layers))], final_norm=norm,
                     final_norm_prefix="final.norm", lm_head_name="head", max_positions=cfg.max_positions,
                     eos_token_ids=list(cfg.eos_token_ids), embedding_scale=cfg.embedding_scale,
                     ignored_name_patterns=tuple(unused))


register_architecture("Bobunex", BobunexConfig.from_dict, bobunex_spec)
