"""Kutirax on the GPU against the plain restatement (tests/plain_kutirax.py, float64 on the CPU).

Small configurations of its own (three, differing in every size, with values that coincide nowhere: vdim != dim,
partial rotation, heads that are no power of two, top == experts, top == 1, layers without feed-forward, two windows
in one model) and random weights. Mechanisms alone (kernels against the plain functions), then the whole model through
the trace replay under every cut (whole, tail decoded one by one, portions down to two tokens, mixed batches over a
pool with no spare page and as many state slots as live requests), windows and carried state made visible by
sharpened weights, long decoding, and greedy generation through the engine's own entry point.
"""

from __future__ import annotations

import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_kutirax as pk
from replay_util import (check_against_plain, make_requests, mixed_steps, portion_steps, run_trace, tail_decode_steps,
                         whole_steps)

pytestmark = pytest.mark.gpu

SIZES = ["kutirax-tiny-a", "kutirax-tiny-b", "kutirax-tiny-c"]
LENGTHS = [70, 133, 45, 200, 96, 61]


def _read(folder):
    from safetensors import safe_open
    w = {}
    with safe_open(str(Path(folder) / "model.safetensors"), "pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).float()
    return json.loads((Path(folder) / "config.json").read_text()), w


def _write(folder, config, tensors):
    from safetensors.torch import save_file
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


@pytest.fixture(scope="session")
def kutirax_dirs(tmp_path_factory):
    from tokenmill_b200.weights import named_config, write_random_model
    return {n: write_random_model(tmp_path_factory.mktemp(n.replace("-", "_")), named_config(n), seed=3 + i)
            for i, n in enumerate(SIZES)}


def _plain(folder, reqs, memo):
    cfg, w = None, None
    out = {}
    for rid, toks in reqs.items():
        key = (str(folder), tuple(toks))
        if key not in memo:
            if cfg is None:
                cfg, w = _read(folder)
            memo[key] = pk.forward(cfg, w, toks).float()
        out[rid] = memo[key]
    return out


def _check(steps, outputs, reqs, plain, dtype):
    """float32: every row within tolerance. bfloat16: a router logit computed from rounded inputs may choose another
    expert where two logits nearly tie, which moves that token's logits (and, faintly, later ones) by more than
    rounding; so a few rows in a hundred may lie outside, and everything else is held to the tolerance."""
    if dtype == "float32":
        return check_against_plain(steps, outputs, reqs, plain, dtype)
    fed = {rid: 0 for rid in reqs}
    over = total = 0
    for s in steps:
        row = 0
        for e in s["entries"]:
            for wpos in e["want"]:
                ref = plain[e["id"]][fed[e["id"]] + wpos]
                diff = float((torch.from_numpy(outputs[s["step"]][row]) - ref).abs().max())
                over += diff > 3e-2 * float(ref.abs().max())
                total += 1
                row += 1
            fed[e["id"]] += len(e["tokens"])
    assert over <= 0.04 * total, f"{over} of {total} rows differ by more than bfloat16 rounding"
    return over / max(total, 1)


def _steps(mode, reqs):
    if mode == "whole":
        return whole_steps(reqs)
    if mode == "tail":
        return tail_decode_steps(reqs)
    if mode == "portions":
        return portion_steps(reqs, seed=5)
    return mixed_steps(reqs, seed=7)


# --- mechanisms alone -------------------------------------------------------------------------------------------

DEV = "cuda:0"


def _step_arrays(q_lens, slots):
    cu = np.zeros(len(q_lens) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    seq = np.repeat(np.arange(len(q_lens), dtype=np.int32), q_lens)
    t = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=DEV)      # noqa: E731
    return t(cu), t(seq), t(slots)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_norm_and_token_shift_kernels(dtype):
    """One pass: stream += m (a + b), two norms with weights stored around zero; then the shift with its carried
    row, two requests side by side in two steps, slots 2 and 0 of 3."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(0)
    H, m, eps = 50, 0.6, 1e-5
    x0 = torch.randn(9, H)
    a, b = torch.randn(9, H).to(dtype), torch.randn(9, H).to(dtype)
    w1, w2, mu = torch.randn(H) * 0.2, torch.randn(H) * 0.2, torch.rand(H)
    x = x0 + m * (a.float() + b.float())
    ref_h = pk.offset_rms_norm(x.double(), w1.double(), eps)
    ref_g = pk.offset_rms_norm(x.double(), w2.double(), eps)
    resid = x0.to(DEV)
    h = torch.empty(9, H, dtype=torch.float32, device=DEV)
    g = torch.empty(9, H, dtype=dtype, device=DEV)
    ops.add_norm_pair(resid, (1 + w1).to(DEV), eps, h, dtype=dtype, w2=(1 + w2).to(DEV), out2=g, a=a.to(DEV), b=b.to(DEV), scale=m)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (resid.cpu() - x).abs().max() < 1e-6
    assert (h.cpu().double() - ref_h).abs().max() < 1e-5 and (g.cpu().double() - ref_g).abs().max() < tol
    # request A: rows 0..3 then 4..5; request B: rows 6..6 then 7..8 (a single token first)
    seqs = {"A": ref_h[:6], "B": ref_h[6:]}
    want = {k: pk.token_shift(v, mu.double()) for k, v in seqs.items()}
    state = torch.zeros(3, H + 5, device=DEV)
    got = {}
    for rows_a, rows_b in (((0, 4), (6, 7)), ((4, 6), (7, 9))):
        hh = torch.cat([h[rows_a[0]:rows_a[1]], h[rows_b[0]:rows_b[1]]]).contiguous()
        cu, seq, slots = _step_arrays([rows_a[1] - rows_a[0], rows_b[1] - rows_b[0]], [2, 0])
        out = torch.empty(hh.shape, dtype=dtype, device=DEV)
        ops.token_shift(hh, mu.to(DEV), state, cu, seq, slots, out)
        na = rows_a[1] - rows_a[0]
        got.setdefault("A", []).append(out[:na].cpu())
        got.setdefault("B", []).append(out[na:].cpu())
    for k in want:
        assert (torch.cat(got[k]).double() - want[k]).abs().max() < tol, k
    assert float(state[1].abs().max()) == 0.0          # nobody's slot stays untouched


@pytest.mark.parametrize("nh,rank,rot,rot_dims,window,page", [(5, 48, 16, 16, 33, 16), (16, 64, 32, 16, 7, 8), (3, 160, 16, 16, 400, 16),
                                                             (7, 72, 6, 4, 20, 16), (4, 272, 32, 32, 1, 32), (40, 32, 16, 16, 50, 16)])
def test_latent_attention_kernels(nh, rank, rot, rot_dims, window, page):
    """The attention kernels alone over a hand-made paged cache of latents: three requests (a prompt portion that
    continues 150 cached tokens, a single decoded token at position 400, a fresh prompt) against a plain 64-bit
    computation from the same cache rows; the tensor-core kernel where it takes the shapes, the generic one always."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(nh)
    D = rank + rot
    starts, lens = [150, 400, 0], [37, 1, 70]
    n_pages = sum(-(-(a + b) // page) for a, b in zip(starts, lens)) + 3
    cache = (torch.randn(n_pages, page, 1, D) * 0.5).to(torch.bfloat16)
    order = torch.randperm(n_pages).tolist()
    width = max(-(-(a + b) // page) for a, b in zip(starts, lens))
    table = np.zeros((3, width), dtype=np.int32)
    for s in range(3):
        for i in range(-(-(starts[s] + lens[s]) // page)):
            table[s, i] = order.pop()
    T = sum(lens)
    q_lat = torch.randn(T, nh, rank)
    q_rot = torch.randn(T, nh, rot).to(torch.bfloat16)
    pos = np.concatenate([np.arange(a, a + b) for a, b in zip(starts, lens)])
    half = rot_dims // 2
    freq = 10000.0 ** (-2.0 * torch.arange(half, dtype=torch.float64) / rot_dims)
    ang = torch.arange(512, dtype=torch.float64)[:, None] * freq
    cos, sin = ang.cos().float(), ang.sin().float()
    scale = 0.3
    ref = torch.zeros(T, nh, rank, dtype=torch.float64)
    t = 0
    for s in range(3):
        rows = torch.stack([cache[table[s, j // page], j % page, 0] for j in range(starts[s] + lens[s])]).double()
        for i in range(lens[s]):
            p = starts[s] + i
            qr = pk.rotate_half(q_rot[t:t + 1].double(), torch.tensor([p]), 10000.0, rot_dims)[0]
            q = torch.cat([q_lat[t].double(), qr], dim=-1)                      # [nh, D]
            lo = max(0, p - window + 1)
            sc = (q @ rows[lo:p + 1].T) * scale
            ref[t] = torch.softmax(sc, -1) @ rows[lo:p + 1, :rank]
            t += 1
    t32 = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=DEV)      # noqa: E731
    cu = np.zeros(4, dtype=np.int32)
    cu[1:] = np.cumsum(lens)
    kinds = [(False, 32, 1, False)] + ([(True, 64, 1, False), (True, 64, 3, False), (True, 64, 32, False), (True, 64, 1, True),
                                        (True, 64, 5, True)] if ops.latent_attention_tc_ok(torch.bfloat16, rank, rot) else [])
    assert len(kinds) == 6 or rank % 16 or rot % 16
    for tc, tile, splits, paired in kinds:
        per = [-(-n * nh // tile) for n in lens]
        tile_seq = np.repeat(np.arange(3), per)
        tile_row0 = np.concatenate([np.arange(k) * tile for k in per])
        out = torch.zeros(nh, T, rank, dtype=torch.bfloat16, device=DEV)
        part = torch.full((len(tile_seq) * splits * 64 * (rank + 2),), float("nan"), device=DEV) if splits > 1 else None
        ops.latent_attention(q_lat.to(DEV), q_rot.to(DEV), cos.to(DEV), sin.to(DEV), rot_dims, cache.to(DEV), t32(table),
                             t32(cu), t32(starts), t32(tile_seq), t32(tile_row0), len(tile_seq), out.transpose(0, 1),
                             scale=scale, window=window, tensor_cores=tc, n_splits=splits, part=part, paired=paired)
        got = out.transpose(0, 1).float().cpu().double()
        err = float((got - ref).abs().max())
        assert err < 2e-2, (tc, splits, paired, err)
        if part is not None:
            part.zero_()             # (the allocator hands this memory to later tests)


@pytest.mark.parametrize("top,E", [(1, 5), (3, 12), (4, 4), (2, 37)])
def test_router_kernel(top, E):
    from tokenmill_b200.kernels import ops
    torch.manual_seed(top)
    T, H = 19, 44
    x, w, b = torch.randn(T, H), torch.randn(E, H), torch.randn(E)
    idx, tw, dense = ops.moe_route(x.to(DEV), w.to(DEV), b.to(DEV), top)
    logits = x.double() @ w.double().T + b.double()
    tv, ti = torch.topk(logits, top, dim=-1)
    assert torch.equal(idx.cpu().long(), ti)
    assert (tw.cpu().double() - torch.softmax(tv, -1)).abs().max() < 1e-6
    ref = torch.zeros(T, E, dtype=torch.float64).scatter_(1, ti, torch.softmax(tv, -1))
    assert (dense.cpu().double() - ref).abs().max() < 1e-6 and int((dense != 0).sum()) == T * top


@pytest.mark.parametrize("sizes", [dict(heads=6, vdim=7, state=11, groups=2, conv=5, norm_groups=3),
                                   dict(heads=8, vdim=8, state=16, groups=2, conv=4, norm_groups=2),
                                   dict(heads=2, vdim=70, state=1, groups=1, conv=1, norm_groups=1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_space_mixer_alone_under_cuts(dtype, sizes):
    """The mixer part with slots of its own: a sequence whole, and the same sequence cut 1 + 2 + 5 + 1 + rest beside
    another request, equal the plain recurrence; sizes that are multiples of nothing, and sizes whose rows the
    convolution kernel takes 16 bytes at a time."""
    from tokenmill_b200.parts.base import LayerCache, StepInputs
    from tokenmill_b200.parts.state_space import StateSpaceMixer
    torch.manual_seed(4)
    H = 40
    p = sizes
    mix = StateSpaceMixer(hidden_size=H, num_heads=p["heads"], value_dim=p["vdim"], state_size=p["state"], groups=p["groups"],
                          conv_taps=p["conv"], norm_groups=p["norm_groups"], eps=1e-5, dtype=dtype, device=torch.device(DEV))
    tensors, plain_w = {}, {}
    for s in mix.weight_specs():
        t = torch.randn(s.shape) * (0.3 if len(s.shape) > 1 else 0.5)
        if s.name in ("norm", "D"):
            t = t + 1.0
        t = t.to(torch.bfloat16).float()
        plain_w[s.name] = t.double()
        tensors[s.name] = t.to(DEV, dtype if s.dtype == "compute" else torch.float32)
    mix.bind(tensors)
    seqs = [torch.randn(23, H).to(torch.bfloat16).float(), torch.randn(9, H).to(torch.bfloat16).float()]
    want = [pk.mamba2(s.double(), plain_w, p, 1e-5) for s in seqs]
    state = torch.zeros(4, mix.state_need().shape[0], device=DEV)
    cache = LayerCache(state=state)
    cuts = [[1, 2, 5, 1, 14], [3, 0, 2, 4, 0]]
    got, at = [[], []], [0, 0]
    for k in range(5):
        parts, lens, slots, who = [], [], [], []
        for r in (0, 1):
            n = cuts[r][k]
            if n:
                parts.append(seqs[r][at[r]:at[r] + n])
                lens.append(n); slots.append(3 if r == 0 else 1); who.append(r)
                at[r] += n
        cu, seq, sl = _step_arrays(lens, slots)
        step = StepInputs(n_tokens=sum(lens), n_seqs=len(lens), token_ids=None, positions=None, seq_of_token=seq, cu_q=cu,
                          kv_before=None, state_slots=sl, block_tables=[], slot_maps=[], want_rows=None, n_want=0,
                          max_q_len=max(lens), max_kv_len=0)
        out = mix.forward(torch.cat(parts).to(DEV, dtype).contiguous(), step, cache).float().cpu()
        o = 0
        for r, n in zip(who, lens):
            got[r].append(out[o:o + n]); o += n
    tol = 2e-4 if dtype == torch.float32 else 4e-2
    for r in (0, 1):
        ref = want[r]
        assert (torch.cat(got[r]).double() - ref).abs().max() < tol * float(ref.abs().max()), r
    assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


# --- the model under every cut ----------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("size", SIZES)
def test_replay_matches_plain(kutirax_dirs, size, dtype, mode, tmp_path, plain_cache):
    folder = kutirax_dirs[size]
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    reqs = make_requests(vocab, LENGTHS, seed=11)
    steps, max_tokens = _steps(mode, reqs)
    if mode == "mixed":
        assert max(len(s["entries"]) for s in steps) >= 3
    outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / "out")
    frac = _check(steps, outputs, reqs, _plain(folder, reqs, plain_cache), dtype)
    print(f"{size} {dtype} {mode}: {frac}")


@pytest.mark.parametrize("order", ["state_space_only", "attention_only", "three_windows", "one_layer"])
def test_other_layer_orders(order, tmp_path):
    """Models without any paged cache (state-space layers only), without any mixer state (attention only; the shift's
    state remains), with three windows (three cache groups, one of them longer than any request), and of one layer."""
    from tokenmill_b200.weights import write_random_model
    from tokenmill_b200.weights.random_init import kutirax_config, kutirax_latent, kutirax_mamba
    L, M = "latent_attention", "mamba2"
    lat = lambda w, **kw: kutirax_latent(heads=4, dim=8, rot_dim=8, vdim=6, q_rank=12, kv_rank=16, window=w, **kw)     # noqa: E731
    layers = {
        "state_space_only": [(M, kutirax_mamba(heads=4, vdim=8, state=8, groups=2, conv=3, norm_groups=2), ("dense", 48)),
                             (M, kutirax_mamba(heads=2, vdim=12, state=6, groups=2, conv=2), None)],
        "attention_only": [(L, lat(11), ("moe", 6, 2, 16)), (L, lat(11), None), (L, lat(11), ("dense", 40))],
        "three_windows": [(L, lat(5), None), (L, lat(1000), ("dense", 32)), (L, lat(64), None)],
        "one_layer": [(L, lat(17, rot_dims=4), ("moe", 2, 1, 8))],
    }[order]
    cfg = kutirax_config(vocab=97, width=40, eps=1e-5, residual_mult=0.8, layers=layers)
    folder = write_random_model(tmp_path / "m", cfg, seed=8)
    reqs = make_requests(97, [70, 133, 45, 96], seed=15)
    _, w = _read(folder)
    plain = {r: pk.forward(cfg, w, t).float() for r, t in reqs.items()}
    for mode in ("whole", "mixed"):
        steps, max_tokens = _steps(mode, reqs)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")
    steps, max_tokens = _steps("mixed", reqs)
    _check(steps, run_trace(folder, "bfloat16", steps, max_tokens, tmp_path / "bf16"), reqs, plain, "bfloat16")


@pytest.mark.parametrize("page", [8, 32])
def test_replay_at_other_page_sizes(kutirax_dirs, page, tmp_path, plain_cache):
    folder = kutirax_dirs["kutirax-tiny-a"]
    reqs = make_requests(211, LENGTHS, seed=13)
    steps, max_tokens = mixed_steps(reqs, seed=9)
    outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / "out", page_size=page)
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_cache), "float32")


def test_cuts_do_not_move_the_logits_in_float32(kutirax_dirs, tmp_path):
    """Whole prompts against mixed batches of portions and single tokens: beyond rounding nothing may differ, and in
    32-bit that means a few units in the last place."""
    folder = kutirax_dirs["kutirax-tiny-b"]
    reqs = make_requests(300, LENGTHS, seed=21)
    rows = {}
    for mode in ("whole", "mixed", "portions"):
        steps, max_tokens = _steps(mode, reqs)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        fed = {r: 0 for r in reqs}
        for s in steps:
            row = 0
            for e in s["entries"]:
                for wpos in e["want"]:
                    rows.setdefault(mode, {})[(e["id"], fed[e["id"]] + wpos)] = outputs[s["step"]][row]
                    row += 1
                fed[e["id"]] += len(e["tokens"])
    for mode in ("mixed", "portions"):
        worst = max(float(np.abs(rows[mode][k] - rows["whole"][k]).max()) for k in rows["whole"])
        assert worst <= 2e-6, (mode, worst)


# --- faults that random weights would hide ----------------------------------------------------------------------

def _sharpen(src, dst, *, attention=8.0, decay=None):
    """A copy of a model whose attention is sharp (queries scaled up: the softmax picks single keys, so a window that
    is one token off picks another) and, optionally, whose state-space layers forget slowly (a lost state shows
    hundreds of tokens later)."""
    cfg, w = _read(src)
    for k in list(w):
        if k.endswith(".mix.uq"):
            w[k] = w[k] * attention
        if decay is not None and k.endswith(".mix.A_log"):
            w[k] = torch.full_like(w[k], decay)
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}          # what the file will hold
    return _write(dst, cfg, w), cfg, w


def _with_windows(cfg, delta):
    import copy
    c = copy.deepcopy(cfg)
    for layer in c["layers"]:
        if layer["type"] == "latent_attention":
            layer["mixer"]["mask"]["size"] += delta
    return c


@pytest.mark.parametrize("size", ["kutirax-tiny-a", "kutirax-tiny-b"])
def test_window_edges_in_prompts_and_in_decoding(kutirax_dirs, size, tmp_path):
    """Sharp attention: the plain model with every window one longer or one shorter differs from the true one by far
    more than the tolerance at most positions beyond the windows, so an engine that agrees with the true one has its
    windows right: inside prompts, in decoded tokens, across page borders (windows of 9, 20 and 33 over pages of 16)."""
    folder, cfg, w = _sharpen(kutirax_dirs[size], tmp_path / "sharp")
    reqs = make_requests(cfg["vocab"], [150, 97], seed=31)
    plain = {r: pk.forward(cfg, w, t).float() for r, t in reqs.items()}
    for delta in (-1, 1):
        other = pk.forward(_with_windows(cfg, delta), w, reqs["r0"]).float()
        tol = 2e-4 * float(plain["r0"].abs().max())
        differs = ((other - plain["r0"]).abs().amax(dim=1) > 20 * tol).float()[40:].mean()
        assert differs > 0.5, (delta, float(differs))
    for mode in ("whole", "tail", "portions", "mixed"):
        steps, max_tokens = _steps(mode, reqs) if mode != "tail" else tail_decode_steps(reqs, tail=60)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")


def test_a_far_key_and_an_old_state_show(kutirax_dirs, tmp_path):
    """A window of 300 keys with sharp attention, and a state that decays by a thousandth a token: the first tokens
    of a 420-token request still move the last logits (checked on the plain model), so keys 299 back, the first pages
    once they are given back, and state carried over many steps are all looked at. Decoding runs 120 tokens."""
    folder, cfg, w = _sharpen(kutirax_dirs["kutirax-tiny-c"], tmp_path / "far", attention=6.0, decay=-7.0)
    reqs = make_requests(cfg["vocab"], [420, 310], seed=41)
    plain = {r: pk.forward(cfg, w, t).float() for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    changed = list(reqs["r0"])
    changed[3] = (changed[3] + 1) % cfg["vocab"]
    assert (pk.forward(cfg, w, changed).float()[-1] - plain["r0"][-1]).abs().max() > 20 * tol      # the state remembers
    for mode in ("whole", "tail", "mixed"):       # (portions of 256 tokens and more run the recurrence over time slices)
        steps, max_tokens = tail_decode_steps(reqs, tail=120) if mode == "tail" else _steps(mode, reqs) if mode == "whole" \
            else mixed_steps(reqs, seed=3)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_time_sliced_recurrence_under_every_cut(kutirax_dirs, dtype, tmp_path, plain_cache, monkeypatch):
    """The three-pass recurrence over time slices, switched on for portions from 12 tokens with slices of 8: whole
    prompts, portions and mixed batches (requests of one token beside requests of many slices, last slices that
    are not full) against the plain recurrence."""
    from tokenmill_b200.parts import state_space
    monkeypatch.setattr(state_space, "SLICED_FROM", 12)
    monkeypatch.setattr(state_space, "SLICE_LEN", 8)
    for size in ("kutirax-tiny-a", "kutirax-tiny-c"):
        folder = kutirax_dirs[size]
        vocab = json.loads((folder / "config.json").read_text())["vocab"]
        reqs = make_requests(vocab, LENGTHS, seed=11)
        for mode in ("whole", "portions", "mixed"):
            steps, max_tokens = _steps(mode, reqs)
            outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / f"{size}_{mode}")
            _check(steps, outputs, reqs, _plain(folder, reqs, plain_cache), dtype)


def test_slots_and_pages_used_again_start_clean(kutirax_dirs, tmp_path, plain_cache):
    """Nine requests through a pool for two live ones with two state slots: every slot and page is used several times,
    and a request that follows a long one on its slot gets the same logits as alone."""
    folder = kutirax_dirs["kutirax-tiny-a"]
    reqs = make_requests(211, [90, 30, 64, 12, 100, 5, 77, 48, 33], seed=51)
    steps, max_tokens = mixed_steps(reqs, seed=2, max_live=2)
    from tokenmill_b200.engine.trace import run
    import io
    out_dir = tmp_path / "out"
    stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    assert run(str(folder), "float32", str(out_dir), max_tokens, stdin=stdin, stdout=io.StringIO(), state_slots=2) == 0
    outputs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, 211) for s in steps}
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_cache), "float32")


# --- through the engine's own entry point -----------------------------------------------------------------------

@pytest.mark.parametrize("graphs,chunked,dtype", [(False, False, "float32"), (True, True, "float32"), (False, True, "bfloat16")])
def test_greedy_generation_through_the_engine(kutirax_dirs, graphs, chunked, dtype):
    """LLMEngine with its scheduler: admission (state slots, two page groups), chunked prompts beside decodes, decode
    graphs with padded rows, a pool so small that requests are evicted and recomputed. The logits behind every
    generated token equal the plain model's on the request's own history, and the token is their arg-max."""
    from tokenmill_b200 import EngineConfig
    from tokenmill_b200.engine import LLMEngine
    from tokenmill_b200.sampling import SamplingParams

    folder = kutirax_dirs["kutirax-tiny-a"]
    cfg, w = _read(folder)
    rng = random.Random(5)
    prompts = [[rng.randrange(211) for _ in range(n)] for n in (9, 30, 17, 44, 5, 26, 12)]
    per_token = (48 + 36) * (4 if dtype == "float32" else 2)
    eng = LLMEngine(EngineConfig(model=str(folder), dtype=dtype, block_size=8, max_model_len=128, max_num_seqs=4,
                                 kv_cache_mb=(14 * 8 + (8 if graphs else 0) + 1) * per_token / 2 ** 20, watermark=0.0, cuda_graphs=graphs,
                                 cuda_graph_max_batch=4, enable_chunked_prefill=chunked,
                                 max_num_batched_tokens=24 if chunked else 256))
    assert eng.cache.state_slots.num_slots == 4 and len(eng.cache.num_pages) == 2
    rows: dict[str, list] = {}

    def tap(where, logits):
        cpu = logits.float().cpu()
        for (rid, pos), row in zip(where, cpu):
            rows.setdefault(rid, []).append((pos, row.clone()))

    eng.on_logits = tap
    reqs = [eng.add_request(f"t{i}", p, SamplingParams(max_tokens=24, ignore_eos=True)) for i, p in enumerate(prompts)]
    while eng.has_unfinished():
        eng.step()
    eng.drain()
    assert eng.cache.all_free
    if graphs:
        assert eng.runner.stats["graph_steps"] > 0
    compared = over = 0
    for i, (p, r) in enumerate(zip(prompts, reqs)):
        assert len(r.output_ids) == 24
        plain = pk.forward(cfg, w, p + r.output_ids).float()
        for pos, row in rows[f"t{i}"]:
            ref = plain[pos]
            if dtype == "float32":
                assert (row - ref).abs().max() <= 2e-4 * float(ref.abs().max()), (i, pos)
                assert int(row.argmax()) == r.output_ids[pos - len(p) + 1]
            else:
                over += float((row - ref).abs().max()) > 3e-2 * float(ref.abs().max())     # (see _check)
            compared += 1
    assert compared >= 7 * 24 and over <= 0.04 * compared


def test_generate_command_line_and_trace_runner(kutirax_dirs, tmp_path):
    """The two programs a user starts: ``python -m tokenmill_b200.generate`` on a Kutirax folder, and bin/trace_run."""
    root = Path(__file__).resolve().parents[1]
    folder = kutirax_dirs["kutirax-tiny-b"]
    res = subprocess.run([sys.executable, "-m", "tokenmill_b200.generate", "--model", str(folder), "--prompt-ids", "5,17,3,250",
                          "--max-tokens", "6", "--dtype", "float32", "--max-model-len", "64", "--kv-cache-mb", "1"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    cfg, w = _read(folder)
    toks = [5, 17, 3, 250]
    for _ in range(6):
        toks.append(int(pk.forward(cfg, w, toks)[-1].argmax()))
    assert out["output_ids"] == toks[4:]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:7], "want": [0, 6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[8:10], "want": [1]}], "end": ["a"]}]
    res = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "bfloat16", "--out",
                          str(tmp_path / "o"), "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps),
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (tmp_path / "o" / "1.f32").exists()
    plain = pk.forward(cfg, w, toks).float()
    got = np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(2, 300)
    last = np.fromfile(tmp_path / "o" / "2.f32", dtype="<f4").reshape(1, 300)
    for row, pos in ((got[0], 0), (got[1], 6), (last[0], 9)):
        assert np.abs(row - plain[pos].numpy()).max() <= 3e-2 * float(plain[pos].abs().max())
