"""Bobunex without a GPU: config.json -> typed configuration -> model as data, the tensors it declares, the cache
layout (pages with kept first positions, state slots), what the cache manager gives back behind a window with kept
tokens, and the plain restatement's own invariances (a sequence's prefix does not depend on what follows)."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_bobunex as pb
from tokenmill_b200.cache.manager import CacheManager
from tokenmill_b200.config.bobunex_config import BobunexConfig
from tokenmill_b200.config.model_config import ConfigError
from tokenmill_b200.models.bobunex import bobunex_spec
from tokenmill_b200.parts.model import DecoderModel
from tokenmill_b200.weights import named_config
from tokenmill_b200.weights.random_init import random_tensors


def _model(name):
    cfg = BobunexConfig.from_dict(named_config(name))
    return cfg, DecoderModel(bobunex_spec(cfg), torch.float32, torch.device("cpu"))


def test_config_reads_every_size_and_refuses_what_the_design_lacks():
    raw = named_config("bobunex-tiny-a")
    cfg = BobunexConfig.from_dict(raw)
    assert (cfg.vocab, cfg.width, cfg.taps, cfg.embedding_scale, cfg.eps) == (173, 48, 3, 5.0, 1e-6)
    assert cfg.layers[0].mixer["left"]["mask"] == {"size": 11, "keep_first": 3} and cfg.layers[1].mlp is None
    for path, value in ((("layers", 0, "type"), "serial"), (("layers", 0, "mlp", "kind"), "moe"),
                        (("layers", 0, "mixer", "left", "heads"), 5), (("layers", 0, "mixer", "left", "rot", "dims"), 7),
                        (("canon", "taps"), 0), (("norm", "eps"), 0.0)):
        bad = copy.deepcopy(raw)
        d = bad
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        with pytest.raises(ConfigError):
            BobunexConfig.from_dict(bad)
    for path in (("embedding",), ("layers", 0, "mixer", "right"), ("layers", 1, "mixer", "left", "mask", "size")):
        bad = copy.deepcopy(raw)
        d = bad
        for k in path[:-1]:
            d = d[k]
        del d[path[-1]]
        with pytest.raises(ConfigError):
            BobunexConfig.from_dict(bad)


def test_spec_declares_the_tensors_by_name():
    _, model = _model("bobunex-tiny-a")
    names = {w.name: tuple(w.shape) for w in model.weight_specs()}
    assert names["embed"] == (173, 48) and names["head"] == (173, 48) and names["final.norm"] == (48,)
    assert names["l0.mix.left.q"] == (72, 48) and names["l0.mix.left.k"] == (36, 48) and names["l0.mix.left.v"] == (60, 48)
    assert names["l0.mix.left.q.norm"] == (72,) and names["l0.mix.left.g"] == (6, 48) and names["l0.mix.left.o"] == (48, 120)
    assert names["l0.mix.right.q"] == (30, 48) and names["l0.mix.right.v"] == (42, 48) and names["l0.mix.right.i.b"] == (3,)
    assert names["l0.mix.right.norm"] == (42,) and names["l0.mix.left.out"] == (48,) and names["l0.mix.right.out"] == (48,)
    assert names["l0.canon1"] == (48, 3) and names["l0.rg2"] == (48, 48) and names["l0.rg2.b"] == (48,)
    assert names["l0.mlp.gate"] == (56, 48) and names["l0.mlp.down"] == (48, 56)
    assert "l1.norm2" not in names and "l1.canon2" not in names and "l1.rg2" not in names and "l1.mlp.up" not in names
    assert model.spec.embedding_scale == 5.0


def test_cache_layout_pages_state_and_kept_positions():
    _, model = _model("bobunex-tiny-a")
    layout = model.cache_layout()
    assert [(g.need.head_dim, g.need.window, g.need.keep_first, g.need.planes) for g in layout.groups] == \
        [(3 * (12 + 20), 11, 3, 1), (16 + 8, 37, 18, 1)]
    assert layout.keep_first == [3, 18] and layout.has_state
    assert layout.block_state[0].shape == (2 * 2 * 48,) and set(layout.entry_state) == {0, 1}
    parts = model.parts()
    assert sum(type(p).__name__ == "SinkWindowAttention" for p in parts) == 2      # the pair's mixers are asked too
    _, one_tap = _model("bobunex-tiny-b")
    assert one_tap.cache_layout().block_state[0].shape == (2 * 80,)


def test_pages_behind_a_window_go_back_except_the_kept_ones():
    m = CacheManager([12, 12], page_size=4, windows=[None, 6], watermark=0.0, keep_first=[0, 5])
    h = m.new_handle()
    m.allocate(h, list(range(30)))
    assert m.release_behind_window(h, 30) == 4                 # pages 2..5 of group 1; 0 and 1 hold positions < 5
    assert h.tables[1][:2] != [-1, -1] and h.tables[1][2:6] == [-1] * 4 and h.tables[1][6] >= 0
    assert all(p >= 0 for p in h.tables[0])
    m.slot(h, 1, 4)
    with pytest.raises(RuntimeError):
        m.slot(h, 1, 9)
    m.free(h)
    assert m.all_free
    with pytest.raises(ValueError):
        CacheManager([4, 4], 4, windows=[None, 6], keep_first=[0])


def test_plain_prefixes_do_not_depend_on_what_follows():
    cfg, model = _model("bobunex-tiny-c")
    raw = named_config("bobunex-tiny-c")
    w = {k: v.float() for k, v in random_tensors(model, 5, torch.bfloat16).items()}
    toks = [(7 * i + 3) % cfg.vocab for i in range(60)]
    full, streams = pb.forward(raw, w, toks)
    part, _ = pb.forward(raw, w, toks[:33])
    assert streams.shape == (2, 60, cfg.width)
    assert (full[:33] - part).abs().max() < 1e-9
