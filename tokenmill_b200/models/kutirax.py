"""Kutirax as data: config.json -> ``ModelSpec``.

A decoder whose layers are parallel blocks: ``x <- x + m * (mixer(shift(norm1(x))) + ff(norm2(x)))`` with a token
shift in front of the mixer, RMS norms whose weights are stored around zero, and, layer by layer as the file
lists them, a latent-attention mixer with a sliding window or a state-space mixer, and a dense squared-relu
feed-forward, a mixture of experts, or none. The output matrix is the embedding. Tensor names: ``embed``,
``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.kutirax_config import KutiraxConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture


def kutirax_spec(cfg: KutiraxConfig) -> ModelSpec:
    d = cfg.width
    norm = PartSpec("rmsnorm32", {"hidden_size": d, "eps": cfg.eps, "offset": 1.0, "weight_name": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "latent_attention":
            rope = PartSpec("rope", {"head_dim": m["rot"]["dims"], "theta": float(m["rot"]["base"]),
                                     "max_positions": cfg.max_positions, "precise": True})
            mixer = PartSpec("latent_attention", {
                "hidden_size": d, "num_heads": m["heads"], "nope_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "window": m["mask"]["size"],
                "scale": float(m["scale"]), "eps": cfg.eps, "position": rope, "rot_dims": m["rot"]["dims"]})
        else:
            mixer = PartSpec("state_space", {
                "hidden_size": d, "num_heads": m["heads"], "value_dim": m["vdim"], "state_size": m["state"],
                "groups": m["groups"], "conv_taps": m["conv"], "norm_groups": m["norm_groups"], "eps": cfg.eps})
        ffn = None
        if layer.mlp is not None and layer.mlp["kind"] == "dense":
            ffn = PartSpec("relu2", {"hidden_size": d, "intermediate_size": layer.mlp["ff"]})
        elif layer.mlp is not None:
            ffn = PartSpec("routed_experts", {"hidden_size": d, "expert_size": layer.mlp["expert"]["ff"],
                                              "num_experts": layer.mlp["router"]["experts"],
                                              "top": layer.mlp["router"]["top"]})
        layers.append(LayerSpec(prefix=f"l{i}", block="parallel_shift", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm if ffn is not None else None, mixer_name="mix",
                                feed_forward_name="mlp", mixer_norm_name="norm1", feed_forward_norm_name="norm2",
                                block_params={"hidden_size": d, "residual_mult": cfg.residual_mult}))
    return ModelSpec(architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=layers, run_order=[RunEntry(i) for i in range(len(layers))], final_norm=norm,
                     final_norm_prefix="final.norm", lm_head_name=None, max_positions=cfg.max_positions,
                     eos_token_ids=list(cfg.eos_token_ids))


register_architecture("Kutirax", KutiraxConfig.from_dict, kutirax_spec)
