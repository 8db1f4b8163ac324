"""Kutirax without a GPU: configuration, the model as data, tensor names, cache and state needs, the random-weights
writer, and properties of the plain restatement that the GPU tests lean on."""

from __future__ import annotations

import copy
import json

import pytest
import torch

import plain_kutirax as pk
from tokenmill_b200.config import ConfigError, KutiraxConfig
from tokenmill_b200.parts.model import DecoderModel
from tokenmill_b200.weights import named_config, read_spec, write_random_model


def _weights(folder):
    from safetensors import safe_open
    out = {}
    with safe_open(str(folder / "model.safetensors"), "pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).float()
    return out


def test_config_reads_every_size_and_refuses_what_it_does_not_know():
    raw = named_config("kutirax-tiny-a")
    cfg = KutiraxConfig.from_dict(raw)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.residual_mult, len(cfg.layers)) == (211, 48, 1e-6, 0.7, 4)
    assert cfg.layers[2].mlp is None and cfg.layers[0].mixer["mask"]["size"] == 9
    for path, value in ((("layers", 0, "type"), "conv_mixer"), (("layers", 1, "mlp", "kind"), "glu"),
                        (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 3, "mlp", "router", "top"), 4),
                        (("layers", 1, "mixer", "groups"), 4)):
        bad = copy.deepcopy(raw)
        d = bad
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        with pytest.raises(ConfigError):
            KutiraxConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][0]["mixer"]["sink"] = 4
    with pytest.raises(ConfigError):
        KutiraxConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    del bad["layers"][1]["mixer"]["conv"]
    with pytest.raises(ConfigError):
        KutiraxConfig.from_dict(bad)


def test_spec_names_tensors_and_cache_needs(tmp_path):
    folder = write_random_model(tmp_path / "m", named_config("kutirax-tiny-a"), seed=3)
    spec, cfg = read_spec(folder)
    assert spec.architecture == "Kutirax" and spec.lm_head_name is None
    model = DecoderModel(spec, torch.float32, torch.device("cpu"))
    names = {w.name: tuple(w.shape) for w in model.weight_specs()}
    stored = _weights(folder)
    assert set(names) == set(stored) and all(tuple(stored[k].shape) == v for k, v in names.items())
    assert names["l0.norm1"] == (48,) and names["l0.shift"] == (48,) and names["final.norm"] == (48,)
    assert names["l0.mix.dkv"] == (40 + 8, 48) and names["l0.mix.uq"] == (3 * 24, 24) and names["l0.mlp.e4.down"] == (48, 24)
    assert names["l1.mix.in"] == (2 * 60 + 2 * 3 * 12 + 6, 48) and names["l1.mix.conv"] == (60 + 72, 3)
    assert "l2.norm2" not in names and not any(k.startswith("l2.mlp") for k in names)
    layout = model.cache_layout()
    # two windows: two groups of one-plane pages; every layer keeps the shift's state, state-space layers their own
    assert [(g.need.window, g.need.head_dim, g.need.planes, g.entries) for g in layout.groups] == \
        [(9, 48, 1, [0]), (20, 36, 1, [2])]
    assert sorted(layout.block_state) == [0, 1, 2, 3] and sorted(layout.entry_state) == [1, 3]
    assert layout.entry_state[1].shape == (2 * 132 + 6 * 10 * 12,) and layout.has_state
    assert layout.bytes_per_token(2) == (48 + 36) * 2


def test_same_sized_windows_share_a_group():
    spec, _ = None, None
    from tokenmill_b200.models.kutirax import kutirax_spec
    spec = kutirax_spec(KutiraxConfig.from_dict(named_config("kutirax-tiny-b")))
    layout = DecoderModel(spec, torch.float32, torch.device("cpu")).cache_layout()
    assert len(layout.groups) == 1 and layout.groups[0].entries == [1, 2] and layout.windows == [33]


def test_plain_window_and_shift_mean_what_they_say():
    """A key `window` positions back is not seen, one `window - 1` back is; the shift reads exactly one token back."""
    torch.manual_seed(0)
    n, d = 30, 16
    p = dict(heads=2, dim=4, rot_dim=4, vdim=6, kv_rank=8, q_rank=8, window=5, scale=0.4, rot_base=100.0, rot_dims=4)
    w = {"dq": torch.randn(8, d, dtype=pk.F), "dq.norm": torch.ones(8, dtype=pk.F), "uq": torch.randn(16, 8, dtype=pk.F),
         "dkv": torch.randn(12, d, dtype=pk.F), "dkv.norm": torch.ones(8, dtype=pk.F), "uk": torch.randn(8, 8, dtype=pk.F),
         "uv": torch.randn(12, 8, dtype=pk.F), "o": torch.randn(d, 12, dtype=pk.F)}
    h = torch.randn(n, d, dtype=pk.F)
    base = pk.latent_attention(h, w, p, 1e-5)
    for back, seen in ((4, True), (5, False)):
        h2 = h.clone()
        h2[20 - back] += 1.0
        moved = (pk.latent_attention(h2, w, p, 1e-5)[20] - base[20]).abs().max() > 1e-9
        assert bool(moved) == seen
    mu = torch.rand(d, dtype=pk.F)
    s = pk.token_shift(h, mu)
    assert torch.allclose(s[0], h[0] * (1 - mu)) and torch.allclose(s[7], h[7] + (h[6] - h[7]) * mu)


def test_plain_state_space_is_a_recurrence():
    """Outputs up to t do not depend on later tokens, and the convolution's last tap weighs the current token."""
    torch.manual_seed(1)
    p = dict(heads=2, vdim=3, state=4, groups=1, conv=3, norm_groups=1)
    d, inner, ch = 8, 6, 6 + 8
    w = {"in": torch.randn(2 * inner + 8 + 2, d, dtype=pk.F) * 0.3, "conv": torch.randn(ch, 3, dtype=pk.F),
         "conv.b": torch.randn(ch, dtype=pk.F), "dt_bias": torch.randn(2, dtype=pk.F), "A_log": torch.randn(2, dtype=pk.F),
         "D": torch.randn(2, dtype=pk.F), "norm": torch.ones(inner, dtype=pk.F), "o": torch.randn(d, inner, dtype=pk.F)}
    h = torch.randn(12, d, dtype=pk.F)
    full = pk.mamba2(h, w, p, 1e-5)
    assert torch.allclose(pk.mamba2(h[:7], w, p, 1e-5), full[:7])
    w2 = dict(w)
    w2["conv"] = w["conv"].clone()
    w2["conv"][:, :2] = 0                     # only the current token's tap is left
    one = pk.mamba2(h[:1], w2, p, 1e-5)
    assert torch.allclose(pk.mamba2(h, w2, p, 1e-5)[:1], one)


def test_plain_router_uses_only_the_chosen_logits():
    torch.manual_seed(2)
    d, E, F = 6, 4, 5
    w = {"router": torch.randn(E, d, dtype=pk.F), "router.b": torch.randn(E, dtype=pk.F)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (torch.randn(F, d, dtype=pk.F), torch.randn(F, d, dtype=pk.F),
                                                           torch.randn(d, F, dtype=pk.F))
    h = torch.randn(3, d, dtype=pk.F)
    out = pk.routed_feed_forward(h, w, dict(experts=E, top=1))
    logits = h @ w["router"].T + w["router.b"]
    for t in range(3):
        e = int(logits[t].argmax())
        a = pk.silu(h[t] @ w[f"e{e}.gate"].T) * (h[t] @ w[f"e{e}.up"].T)
        assert torch.allclose(out[t], a @ w[f"e{e}.down"].T)          # weight 1 whatever the other logits are


def test_random_writer_round_trip(tmp_path):
    a = write_random_model(tmp_path / "a", named_config("kutirax-tiny-b"), seed=5)
    b = write_random_model(tmp_path / "b", named_config("kutirax-tiny-b"), seed=5)
    wa, wb = _weights(a), _weights(b)
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert json.loads((a / "config.json").read_text())["architecture"] == "Kutirax"
    assert float(wa["l0.shift"].mean()) > 0.2 and float(wa["l1.norm1"].abs().max()) < 1.0     # around 0.5, around 0
