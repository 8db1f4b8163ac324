"""Bobunex on the GPU against the plain restatement (tests/plain_bobunex.py, float64 on the CPU).

Small configurations of its own (three, differing in every size: vdim != dim, partial / full / no rotation, with and
without frequency scaling, 2 / 3 / 5 taps, one key head / one per query head, kept first tokens inside and across
pages, two cache groups in one model, a layer without feed-forward) and random weights. Mechanisms alone (kernels
against the plain functions), then the whole model through the trace replay under every cut (whole, tail decoded one
by one, portions down to two tokens, mixed batches over a pool with no spare page and as many state slots as live
requests), window edges, kept tokens and carried state made visible by sharpened weights, long decoding, and greedy
generation through the engine's own entry point.
"""

from __future__ import annotations

import copy
import io
import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_bobunex as pb
from replay_util import (check_against_plain, make_requests, mixed_steps, portion_steps, run_trace, tail_decode_steps,
                         whole_steps)

pytestmark = pytest.mark.gpu

SIZES = ["bobunex-tiny-a", "bobunex-tiny-b", "bobunex-tiny-c", "bobunex-tiny-d"]
LENGTHS = [70, 133, 45, 200, 96, 61]
DEV = "cuda:0"


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


def _logits(cfg, w, toks):
    return pb.forward(cfg, w, toks)[0].float()


@pytest.fixture(scope="session")
def bobunex_dirs(tmp_path_factory):
    from tokenmill_b200.weights import named_config, write_random_model
    return {n: write_random_model(tmp_path_factory.mktemp(n.replace("-", "_")), named_config(n), seed=3 + i)
            for i, n in enumerate(SIZES)}


@pytest.fixture(scope="session")
def plain_memo():
    return {}


def _plain(folder, reqs, memo):
    cfg, w = None, None
    out = {}
    for rid, toks in reqs.items():
        key = (str(folder), tuple(toks))
        if key not in memo:
            if cfg is None:
                cfg, w = _read(folder)
            memo[key] = _logits(cfg, w, toks)
        out[rid] = memo[key]
    return out


def _check(steps, outputs, reqs, plain, dtype):
    """float32: every row within 2e-4 of the largest logit. bfloat16: rounding passes through several norms of small
    vectors (a head's output, a mixer's output) and is not evenly spread over the rows: measured against the 64-bit
    restatement, the median row is 0.8 % of the largest logit off, the 99th percentile 2.2 %, the worst 4.5 % (first
    positions). So every row is held to 6 % and all but 2 in 100 to 3 %."""
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
                assert diff <= 6e-2 * float(ref.abs().max()), (s["step"], e["id"], fed[e["id"]] + wpos, diff)
                over += diff > 3e-2 * float(ref.abs().max())
                total += 1
                row += 1
            fed[e["id"]] += len(e["tokens"])
    assert over <= 0.02 * total, f"{over} of {total} rows differ by more than 3 % of the largest logit"


def _steps(mode, reqs):
    if mode == "whole":
        return whole_steps(reqs)
    if mode == "tail":
        return tail_decode_steps(reqs)
    if mode == "portions":
        return portion_steps(reqs, seed=5)
    return mixed_steps(reqs, seed=7)


def _t(a, dtype=np.int32):
    return torch.as_tensor(np.asarray(a, dtype=dtype), device=DEV)


def _step_arrays(q_lens, slots):
    cu = np.zeros(len(q_lens) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    return _t(cu), _t(np.repeat(np.arange(len(q_lens)), q_lens)), _t(slots)


# --- mechanisms alone -------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_add_norm_kernel(dtype):
    """stream += sigmoid(gate + bias) * branch, then the norm; the start from embedding rows times a constant; rows."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(0)
    H, eps = 50, 1e-5
    x0, y = torch.randn(9, H), torch.randn(9, H).to(dtype)
    wide = torch.randn(9, H + 7)                        # the gate's rows are strided
    bias, w = torch.randn(H), 1 + 0.1 * torch.randn(H)
    x = x0.double() + torch.sigmoid(wide[:, 3:3 + H].double() + bias.double()) * y.double()
    resid = x0.to(DEV)
    out = torch.empty(9, H, dtype=dtype, device=DEV)
    ops.gated_add_rmsnorm(resid, w.to(DEV), eps, out, branch=y.to(DEV), gate=wide.to(DEV)[:, 3:3 + H], gate_bias=bias.to(DEV))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (resid.cpu().double() - x).abs().max() < 1e-5
    assert (out.cpu().double() - pb.rms_norm(x, w.double(), eps)).abs().max() < tol
    rows = _t([7, 2])
    picked = torch.empty(2, H, dtype=dtype, device=DEV)
    ops.gated_add_rmsnorm(resid, w.to(DEV), eps, picked, rows=rows)
    assert (picked.cpu().double() - pb.rms_norm(resid.cpu().double()[[7, 2]], w.double(), eps)).abs().max() < tol
    table, ids = torch.randn(11, H).to(dtype), _t([4, 0, 10])
    start = torch.zeros(3, H, device=DEV)
    ops.gated_add_rmsnorm(start, w.to(DEV), eps, picked.new_empty(3, H), ids=ids, table=table.to(DEV), table_scale=3.0)
    assert (start.cpu().double() - table.double()[[4, 0, 10]] * 3.0).abs().max() < 1e-6


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_input_convolution_carries_its_last_inputs(taps, dtype):
    """Two requests in slots 2 and 0 of 3, cut into steps of 1, 2, 1, 7 and 4, 1, 1, 5 tokens (portions shorter than the
    carried inputs included) against the convolution over the whole sequences."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(1)
    C = 21
    w = torch.randn(C, taps) * 0.5
    seqs = [torch.randn(11, C).to(dtype), torch.randn(11, C).to(dtype)]
    want = [s.double() + pb.causal_taps(s.double(), w.double()) for s in seqs]
    state = torch.zeros(3, (taps - 1) * C + 3, device=DEV)[:, :max((taps - 1) * C, 0)]
    fed = [0, 0]
    for na, nb in ((1, 4), (2, 1), (1, 1), (7, 5)):
        h = torch.cat([seqs[0][fed[0]:fed[0] + na], seqs[1][fed[1]:fed[1] + nb]]).to(DEV)
        cu, seq, slots = _step_arrays([na, nb], [2, 0])
        out = ops.canon_conv(h, w.to(DEV), state, cu, seq, slots, torch.empty_like(h)).cpu().double()
        ref = torch.cat([want[0][fed[0]:fed[0] + na], want[1][fed[1]:fed[1] + nb]])
        assert (out - ref).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2)
        fed = [fed[0] + na, fed[1] + nb]
    if taps > 1:
        assert float(state[1].abs().max()) == 0.0          # nobody's slot


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_glu_pair_mean_and_head_norm_kernels(dtype):
    from tokenmill_b200.kernels import ops
    torch.manual_seed(2)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    gu = (torch.randn(5, 2 * 37) * 2).to(dtype)
    out = ops.glu(gu.to(DEV), torch.empty(5, 37, dtype=dtype, device=DEV), "gelu_tanh").cpu().double()
    assert (out - pb.gelu_tanh(gu.double()[:, :37]) * gu.double()[:, 37:]).abs().max() < tol
    out = ops.glu(gu.to(DEV), torch.empty(5, 37, dtype=dtype, device=DEV), "silu").cpu().double()
    assert (out - torch.nn.functional.silu(gu.double()[:, :37]) * gu.double()[:, 37:]).abs().max() < tol
    a, b = torch.randn(6, 44).to(dtype), (3 * torch.randn(6, 44)).to(dtype)
    wa, wb = torch.randn(44), torch.randn(44)
    out = ops.norm_pair_mean(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-6, torch.empty_like(a, device=DEV)).cpu().double()
    ref = 0.5 * (pb.rms_norm(a.double(), wa.double(), 1e-6) + pb.rms_norm(b.double(), wb.double(), 1e-6))
    assert (out - ref).abs().max() < tol
    heads, dv = 3, 14
    y, wide, w = torch.randn(7, heads * dv) * 5, torch.randn(7, heads * dv + 9), torch.randn(heads * dv)
    out = ops.head_norm_gate(y.to(DEV), wide.to(DEV)[:, 9:], w.to(DEV), 1e-5, heads,
                             torch.empty(7, heads * dv, dtype=dtype, device=DEV)).cpu().double()
    ref = pb.rms_norm(y.double().view(7, heads, dv), None, 1e-5).reshape(7, -1) * w.double() * torch.sigmoid(wide.double()[:, 9:])
    assert (out - ref).abs().max() < tol


def test_rotary_frequencies_with_wavelength_scaling():
    """All three branches of the rule (kept, divided, blended) against the plain frequencies, through the tables."""
    from tokenmill_b200.parts.rope import RotaryEmbedding
    scaling = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    f = pb.rotary_frequencies(16, 300.0, scaling)
    plainf = pb.rotary_frequencies(16, 300.0, None)
    ratio = (f / plainf).tolist()
    assert any(r == 1.0 for r in ratio) and any(abs(r - 1 / 8) < 1e-12 for r in ratio) and any(1 / 8 + 1e-6 < r < 1 - 1e-6 for r in ratio)
    cos, sin = RotaryEmbedding(head_dim=16, theta=300.0, max_positions=50, scaling=scaling).tables(torch.device("cpu"))
    ang = torch.arange(50, dtype=torch.float64)[:, None] * f[None, :]
    assert (cos.double() - ang.cos()).abs().max() < 1e-7 and (sin.double() - ang.sin()).abs().max() < 1e-7


def _attend(dtype, H, G, d, dv, rot_dims, window, keep_first, softcap, sink, q_lens, starts, page=8, sharpen=None, tc=False, hot=None, splits=1):
    """Kernel pair (norm + rotation + cache write, attention) over a paged cache filled step by step, against the plain
    attention over whole sequences. Returns (engine output, plain output) for the LAST step's rows."""
    from tokenmill_b200.kernels import ops
    from tokenmill_b200.parts.rope import RotaryEmbedding
    torch.manual_seed(3)
    n_seq = len(q_lens)
    total = [s + q for s, q in zip(starts, q_lens)]
    P = H * d + G * d + G * dv + H
    proj = [torch.randn(t, P) for t in total]
    wq, wk = 1 + 0.1 * torch.randn(H * d), 1 + 0.1 * torch.randn(G * d)
    if sharpen is not None:             # (the norm undoes a scaling of q itself: scale its weight)
        wq = wq * sharpen
    if hot is not None:                 # all scores equal; a few keys carry large values, so that seeing one shows
        for p in proj:
            p[:, :H * d] = 0.0
            for j in hot:
                if j < p.shape[0]:
                    p[j, H * d + G * d:H * d + G * d + G * dv] *= 60.0
    rope = RotaryEmbedding(head_dim=max(rot_dims, 2), theta=100.0, max_positions=max(total) + 1, precise=True)
    cos, sin = rope.tables(torch.device(DEV))
    if rot_dims == 0:
        cos = sin = torch.zeros((1, 0), device=DEV)
    pages = sum(-(-t // page) for t in total)
    order = list(range(pages))
    random.Random(0).shuffle(order)                     # pages lie anywhere
    tables, at = [], 0
    for t in total:
        n = -(-t // page)
        tables.append(order[at:at + n])
        at += n
    width = max(len(t) for t in tables)
    bt = _t([t + [0] * (width - len(t)) for t in tables])
    cache = torch.zeros(pages, page, 1, G * (d + dv), dtype=dtype, device=DEV)
    outs = None
    for phase in (0, 1):                                # first the cached part, then the step under test
        lens = starts if phase == 0 else q_lens
        befores = [0] * n_seq if phase == 0 else starts
        if sum(lens) == 0:
            continue
        rows = torch.cat([proj[s][befores[s]:befores[s] + lens[s]] for s in range(n_seq)]).to(DEV)
        positions = _t(np.concatenate([np.arange(befores[s], befores[s] + lens[s]) for s in range(n_seq)]))
        slots = _t(np.concatenate([[tables[s][p // page] * page + p % page for p in range(befores[s], befores[s] + lens[s])]
                                   for s in range(n_seq)]))
        T = rows.shape[0]
        q = torch.empty(T, H * d, dtype=dtype, device=DEV)
        gate = torch.empty(T, H, device=DEV)
        ops.qk_norm_rope_write(rows, heads=H, kv_heads=G, dim=d, vdim=dv, rot_dims=rot_dims, wq=wq.to(DEV), wk=wk.to(DEV),
                               eps=1e-6, positions=positions, cos=cos, sin=sin, slot_map=slots, q_out=q,
                               cache=cache.view(-1, G * (d + dv)), gate_out=gate)
        if phase == 1:
            Gq = H // G
            tile = 64 if tc else 32
            per = [-(-n * Gq // tile) for n in lens]
            tile_seq = np.repeat(np.arange(n_seq), per)
            tile_row0 = np.concatenate([np.arange(n) * tile for n in per])
            cu = np.zeros(n_seq + 1, dtype=np.int32)
            cu[1:] = np.cumsum(lens)
            outs = ops.sink_attention(q, cache, bt, _t(cu), _t(befores), _t(tile_seq), _t(tile_row0), int(tile_seq.size), gate,
                                      torch.empty(T, H * dv, dtype=dtype, device=DEV), heads=H, kv_heads=G, dim=d, vdim=dv,
                                      scale=0.3, softcap=softcap, window=window, keep_first=keep_first, sink=sink,
                                      tensor_cores=tc, n_splits=splits,
                                      part=torch.full((int(tile_seq.size) * G * splits * 64 * (dv + 2),), float("nan"), device=DEV)
                                      if splits > 1 else None)
    ref = []
    freqs = pb.rotary_frequencies(rot_dims, 100.0, None) if rot_dims else None
    for s in range(n_seq):
        p = proj[s].double()
        t = total[s]
        qq = pb.rms_norm(p[:, :H * d], wq.double(), 1e-6).view(t, H, d)
        kk = pb.rms_norm(p[:, H * d:H * d + G * d], wk.double(), 1e-6).view(t, G, d)
        vv = p[:, H * d + G * d:H * d + G * d + G * dv].reshape(t, G, dv)
        if rot_dims:
            qq, kk = pb.rotate_half(qq, torch.arange(t), freqs, rot_dims), pb.rotate_half(kk, torch.arange(t), freqs, rot_dims)
        if dtype == torch.bfloat16:
            qq, kk, vv = (x.to(torch.bfloat16).double() for x in (qq, kk, vv))
        o = pb.sink_window_attention(qq, kk, vv, scale=0.3, softcap=softcap, window=window or 10 ** 9, keep_first=keep_first)
        if not sink:        # the plain function always has the sink: take it out of the denominator again
            o = _without_sink(qq, kk, vv, 0.3, softcap, window or 10 ** 9, keep_first)
        o = o * torch.sigmoid(p[:, -H:])[:, :, None]
        ref.append(o[starts[s]:].reshape(q_lens[s], H * dv))
    return outs.cpu().double(), torch.cat(ref)


def _without_sink(q, k, v, scale, softcap, window, keep_first):
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if (i - j < window or j < keep_first)]
            s = (k[js, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            out[i, h] = torch.softmax(s, 0) @ v[js, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(H=6, G=3, d=12, dv=20, rot_dims=8, window=11, keep_first=3, softcap=4.0, sink=True),
    dict(H=4, G=1, d=16, dv=8, rot_dims=16, window=37, keep_first=18, softcap=0.0, sink=True),
    dict(H=5, G=5, d=10, dv=40, rot_dims=0, window=0, keep_first=0, softcap=2.0, sink=False),
    dict(H=2, G=2, d=34, dv=10, rot_dims=2, window=5, keep_first=70, softcap=50.0, sink=True),
])
def test_attention_kernels_prompt_portion_and_decoding(dtype, case):
    """Three requests in one step: a prompt from position 0, a portion that continues 61 cached tokens (its window and
    its kept tokens lie in other pages than its queries), and single decoded tokens behind 40 and 95."""
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    got, ref = _attend(dtype, q_lens=[50, 23, 1, 1], starts=[0, 61, 40, 95], **case)
    assert (got - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("case", [
    dict(H=4, G=2, d=32, dv=64, rot_dims=8, window=70, keep_first=20, softcap=4.0, sink=True),
    dict(H=6, G=1, d=64, dv=32, rot_dims=64, window=13, keep_first=130, softcap=0.0, sink=True),
    dict(H=2, G=2, d=128, dv=128, rot_dims=0, window=0, keep_first=0, softcap=30.0, sink=False),
    dict(H=8, G=2, d=64, dv=128, rot_dims=16, window=100, keep_first=1, softcap=50.0, sink=True),
])
def test_tensor_core_attention_kernel(case):
    """The mma.sync kernel on the same mixed step (a 200-token prompt so that kept blocks, skipped blocks and window
    blocks all occur; a portion behind 150 cached tokens; single tokens), against the plain attention on the rounded
    q, k, v; and against the CUDA-core kernel."""
    q_lens, starts = [200, 23, 1, 1], [0, 150, 40, 333]
    got, ref = _attend(torch.bfloat16, q_lens=q_lens, starts=starts, tc=True, **case)
    assert (got - ref).abs().max() < 3e-2 * max(1.0, float(ref.abs().max()))
    slow, _ = _attend(torch.bfloat16, q_lens=q_lens, starts=starts, tc=False, **case)
    assert (got - slow).abs().max() < 3e-2 * max(1.0, float(ref.abs().max()))
    for splits in (2, 3, 8):            # key blocks dealt out over several blocks and merged (more splits than blocks too)
        cut, _ = _attend(torch.bfloat16, q_lens=q_lens, starts=starts, tc=True, splits=splits, **case)
        assert (cut - ref).abs().max() < 3e-2 * max(1.0, float(ref.abs().max())), splits


@pytest.mark.parametrize("tc", [False, True])
def test_attention_window_edges_with_hot_keys(tc):
    """All scores equal and a few keys with values sixty times the others': a row that sees such a key one position
    too early or too late is off by far more than rounding. Hot keys sit where rows of the step have their window's
    first key, the key before it, the last kept token and the one behind it, and at the borders of the kernels' key
    blocks (31, 32, 63, 64, 128), in a prompt and in decoded tokens."""
    case = dict(H=4, G=2, d=64, dv=32, rot_dims=8, softcap=30.0, sink=True)
    hot = [5, 6, 31, 32, 63, 64, 100, 128, 129, 140]
    kw = dict(q_lens=[230, 1, 1, 1], starts=[0, 133, 134, 209], hot=hot, tc=tc, splits=3 if tc else 1, **case)
    got, ref = _attend(torch.bfloat16, window=70, keep_first=6, **kw)
    assert (got - ref).abs().max() < 3e-2 * float(ref.abs().max())
    for dw, dk in ((1, 0), (-1, 0), (0, 1), (0, -1)):
        _, other = _attend(torch.bfloat16, window=70 + dw, keep_first=6 + dk, **kw)
        rows = (other - ref).abs().amax(dim=1) > 6e-2 * float(ref.abs().max())
        assert int(rows[:230].sum()) >= 5 and (dk != 0 or bool(rows[230:].any())), (dw, dk)


def test_window_and_kept_edges_with_sharp_queries():
    """Queries scaled up so that single keys carry the softmax: the plain result with the window or the kept count one
    off differs visibly; the kernel agrees with the true one, in a prompt and in decoded tokens."""
    case = dict(H=4, G=2, d=16, dv=12, rot_dims=8, softcap=30.0, sink=True)
    got, ref = _attend(torch.float32, q_lens=[90, 1, 1], starts=[0, 33, 77], window=13, keep_first=6, sharpen=6.0, **case)
    assert (got - ref).abs().max() < 2e-5 * max(1.0, float(ref.abs().max()))
    for dw, dk in ((1, 0), (-1, 0), (0, 1), (0, -1)):
        _, other = _attend(torch.float32, q_lens=[90, 1, 1], starts=[0, 33, 77], window=13 + dw, keep_first=6 + dk, sharpen=6.0, **case)
        assert ((other - ref).abs().amax(dim=1) > 1e-3).float()[20:].mean() > 0.3, (dw, dk)


@pytest.mark.parametrize("heads,d,dv", [(3, 10, 14), (1, 40, 72), (2, 64, 300), (2, 260, 24)])
def test_matrix_memory_kernel_under_cuts(heads, d, dv):
    """Two requests (slots 1 and 3 of 4) fed in steps of unequal sizes, single tokens among them, against the plain
    recurrence over the whole sequences; the projection's rows are strided and carry the gates' raw values."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(4)
    cap, n = 6.0, 40
    P = 2 * heads * d + heads * dv + 2 * heads
    col = {"q": 0, "k": heads * d, "v": 2 * heads * d, "i": 2 * heads * d + heads * dv, "f": 2 * heads * d + heads * dv + heads}
    seqs = [torch.randn(n, P + 5), torch.randn(n, P + 5)]
    bi, bf = torch.randn(heads), torch.randn(heads) + 2
    want = []
    for s in seqs:
        p = s.double()[:, 5:]
        q = p[:, :heads * d].view(n, heads, d) * d ** -0.5
        k = p[:, col["k"]:col["v"]].view(n, heads, d)
        v = p[:, col["v"]:col["i"]].reshape(n, heads, dv)
        li = cap * torch.tanh((p[:, col["i"]:col["f"]] + bi.double()) / cap)
        lf = torch.nn.functional.logsigmoid(cap * torch.tanh((p[:, col["f"]:] + bf.double()) / cap))
        want.append(pb.matrix_memory(q, k, v, li, lf)[0].reshape(n, heads * dv))
    floats = ops.matrix_memory_state_floats(heads, d, dv)
    state = torch.zeros(4, 8 + floats, device=DEV)
    fed = [0, 0]
    for na, nb in ((1, 17), (20, 1), (2, 1), (17, 21)):
        rows = torch.cat([seqs[0][fed[0]:fed[0] + na], seqs[1][fed[1]:fed[1] + nb]]).to(DEV)
        cu, _, slots = _step_arrays([na, nb], [1, 3])
        y, den = torch.empty(na + nb, heads * dv, device=DEV), torch.empty(na + nb, heads, device=DEV)
        ops.matrix_memory(rows[:, 5:], q_col=col["q"], k_col=col["k"], v_col=col["v"], i_col=col["i"], f_col=col["f"],
                          i_bias=bi.to(DEV), f_bias=bf.to(DEV), cap=cap, q_scale=d ** -0.5, state=state, state_off=8, cu_q=cu,
                          state_slots=slots, y=y, den=den, n_seqs=2, heads=heads, dim=d, vdim=dv)
        y = (y.view(-1, heads, dv) / den[:, :, None]).view(-1, heads * dv)
        ref = torch.cat([want[0][fed[0]:fed[0] + na], want[1][fed[1]:fed[1] + nb]])
        assert (y.cpu().double() - ref).abs().max() < 2e-5 * max(1.0, float(ref.abs().max()))
        fed = [fed[0] + na, fed[1] + nb]
    assert float(state[0].abs().max()) == 0.0 and float(state[:, :8].abs().max()) == 0.0


@pytest.mark.parametrize("heads,d,dv,slice_len", [(3, 10, 14, 8), (2, 64, 40, 16), (1, 260, 24, 5)])
def test_matrix_memory_over_time_slices(heads, d, dv, slice_len):
    """Three passes over time slices against the walk in one piece, from a state that an earlier step left: three
    requests of 61, 1 and 16 tokens (last slices that are not full, a request of one slice, one that fills its slices
    exactly); outputs and the states left behind agree to rounding."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(5)
    P = 2 * heads * d + heads * dv + 2 * heads
    col = dict(q_col=0, k_col=heads * d, v_col=2 * heads * d, i_col=2 * heads * d + heads * dv,
               f_col=2 * heads * d + heads * dv + heads)
    floats = ops.matrix_memory_state_floats(heads, d, dv)
    bi, bf = torch.randn(heads, device=DEV), torch.randn(heads, device=DEV) + 2
    kw = dict(i_bias=bi, f_bias=bf, cap=6.0, q_scale=d ** -0.5, state_off=0, n_seqs=3, heads=heads, dim=d, vdim=dv, **col)
    warm, rows = torch.randn(9, P, device=DEV), torch.randn(78, P, device=DEV)
    results = []
    for sliced in (False, True):
        state = torch.zeros(5, floats, device=DEV)
        cu, _, slots = _step_arrays([3, 3, 3], [4, 0, 2])
        ops.matrix_memory(warm, state=state, cu_q=cu, state_slots=slots, y=torch.empty(9, heads * dv, device=DEV),
                          den=torch.empty(9, heads, device=DEV), **kw)
        cu, _, slots = _step_arrays([61, 1, 16], [4, 0, 2])
        y, den = torch.empty(78, heads * dv, device=DEV), torch.empty(78, heads, device=DEV)
        extra = {}
        if sliced:
            n = ops.matrix_memory_slice_records(78, 3, slice_len)
            extra = dict(slice_len=slice_len, slices=torch.full((n * floats,), float("nan"), device=DEV))
        ops.matrix_memory(rows, state=state, cu_q=cu, state_slots=slots, y=y, den=den, **kw, **extra)
        results.append(((y.view(-1, heads, dv) / den[:, :, None]).view(-1, heads * dv).cpu(), state.cpu()))
    (y0, s0), (y1, s1) = results
    assert (y0 - y1).abs().max() < 2e-5 * max(1.0, float(y0.abs().max()))
    assert (s0 - s1).abs().max() < 2e-5 * max(1.0, float(s0.abs().max()))
    assert float(s1[1].abs().max()) == 0.0 and float(s1[3].abs().max()) == 0.0


# --- the whole model under every cut ----------------------------------------------------------------------------

@pytest.mark.parametrize("size", SIZES)
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_against_plain(bobunex_dirs, plain_memo, size, mode, dtype, tmp_path):
    folder = bobunex_dirs[size]
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    reqs = make_requests(vocab, LENGTHS, seed=11)
    steps, max_tokens = _steps(mode, reqs)
    outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / "out")
    _check(steps, outputs, reqs, _plain(folder, reqs, plain_memo), dtype)


@pytest.mark.parametrize("page", [8, 32])
def test_replay_at_other_page_sizes(bobunex_dirs, plain_memo, page, tmp_path):
    folder = bobunex_dirs["bobunex-tiny-a"]
    reqs = make_requests(173, LENGTHS, seed=13)
    steps, max_tokens = mixed_steps(reqs, seed=9)
    outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / "out", page_size=page)
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_memo), "float32")


def test_cuts_do_not_move_the_logits_in_float32(bobunex_dirs, tmp_path):
    """Whole prompts against mixed batches of portions and single tokens: every sum walks keys and tokens in the same
    order whatever the cut, so in 32-bit the rows agree to a few units in the last place."""
    folder = bobunex_dirs["bobunex-tiny-a"]
    reqs = make_requests(173, LENGTHS, seed=21)
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
    scale = max(float(np.abs(v).max()) for v in rows["whole"].values())
    for mode in ("mixed", "portions"):
        worst = max(float(np.abs(rows[mode][k] - rows["whole"][k]).max()) for k in rows["whole"])
        assert worst <= 4e-6 * scale, (mode, worst)


# --- faults that random weights would hide ----------------------------------------------------------------------

def _sharpen(src, dst, *, attention=8.0, forget_bias=None):
    """A copy of a model whose attention is sharp (query weights scaled up: after the norm single keys carry the
    softmax, so a window or a kept count that is one off picks other keys) and, optionally, whose memory forgets
    slowly (a lost or stale state shows hundreds of tokens later)."""
    cfg, w = _read(src)
    for k in list(w):
        if k.endswith(".left.q.norm"):
            w[k] = w[k] * attention
        if forget_bias is not None and k.endswith(".right.f.b"):
            w[k] = torch.full_like(w[k], forget_bias)
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}          # what the file will hold
    return _write(dst, cfg, w), cfg, w


def _with_masks(cfg, d_window, d_keep):
    c = copy.deepcopy(cfg)
    for layer in c["layers"]:
        layer["mixer"]["left"]["mask"]["size"] += d_window
        layer["mixer"]["left"]["mask"]["keep_first"] = max(0, layer["mixer"]["left"]["mask"]["keep_first"] + d_keep)
    return c


def test_window_and_kept_tokens_in_prompts_and_in_decoding(bobunex_dirs, tmp_path):
    """Sharp attention: the plain model with every window, or every kept count, one larger or smaller differs from the
    true one by far more than the tolerance at many positions, so an engine that agrees with the true one has both
    right: inside prompts, in decoded tokens, across page borders (windows of 11 and 37, 3 and 18 kept, pages of 16)."""
    folder, cfg, w = _sharpen(bobunex_dirs["bobunex-tiny-a"], tmp_path / "sharp")
    for layer in cfg["layers"]:
        layer["mixer"]["left"]["softcap"] = 40.0
    _write(folder, cfg, w)
    reqs = make_requests(cfg["vocab"], [150, 97], seed=31)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    for dw, dk in ((-1, 0), (1, 0), (0, -1), (0, 1)):
        other = _logits(_with_masks(cfg, dw, dk), w, reqs["r0"])
        differs = ((other - plain["r0"]).abs().amax(dim=1) > 10 * tol).float()[40:].mean()
        assert differs > 0.3, (dw, dk, float(differs))
    for mode in ("whole", "tail", "portions", "mixed"):
        steps, max_tokens = _steps(mode, reqs) if mode != "tail" else tail_decode_steps(reqs, tail=60)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")


def test_a_far_key_and_an_old_state_show(bobunex_dirs, tmp_path):
    """A window of 300 keys with 40 kept and a memory that forgets slowly: changing one of the first tokens of a
    420-token request still moves its last logits (checked on the plain model), so keys 299 back, kept tokens whose
    pages outlive the window, and state carried over many steps are all looked at. Decoding runs 120 tokens."""
    folder, cfg, w = _sharpen(bobunex_dirs["bobunex-tiny-c"], tmp_path / "far", attention=6.0, forget_bias=8.0)
    reqs = make_requests(cfg["vocab"], [420, 310], seed=41)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    changed = list(reqs["r0"])
    changed[3] = (changed[3] + 1) % cfg["vocab"]
    assert (_logits(cfg, w, changed)[-1] - plain["r0"][-1]).abs().max() > 20 * tol
    for mode in ("whole", "tail", "mixed"):
        steps, max_tokens = tail_decode_steps(reqs, tail=120) if mode == "tail" else _steps(mode, reqs) if mode == "whole" \
            else mixed_steps(reqs, seed=3)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_time_sliced_memory_under_every_cut(bobunex_dirs, plain_memo, dtype, tmp_path, monkeypatch):
    """The three-pass recurrence switched on for portions from 12 tokens with slices of 8: whole prompts, portions and
    mixed batches (requests of one token beside requests of many slices) against the plain recurrence."""
    from tokenmill_b200.parts import matrix_memory
    monkeypatch.setattr(matrix_memory, "SLICED_FROM", 12)
    monkeypatch.setattr(matrix_memory, "SLICE_LEN", 8)
    for size in ("bobunex-tiny-a", "bobunex-tiny-c"):
        folder = bobunex_dirs[size]
        vocab = json.loads((folder / "config.json").read_text())["vocab"]
        reqs = make_requests(vocab, LENGTHS, seed=11)
        for mode in ("whole", "portions", "mixed"):
            steps, max_tokens = _steps(mode, reqs)
            outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / f"{size}_{mode}")
            _check(steps, outputs, reqs, _plain(folder, reqs, plain_memo), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_unlike_sizes_and_portions_beyond_the_slice_threshold(dtype, tmp_path):
    """Three layers that share no size (three cache groups; one layer's heads take the tensor-core kernel in bfloat16,
    the others do not; a memory of 96 rows), prompts of 300 and 270 tokens whole (the memory runs over time slices of
    its real length, pages behind the windows go back while kept pages stay) and in mixed batches, then decoded."""
    from tokenmill_b200.weights import write_random_model
    from tokenmill_b200.weights.random_init import bobunex_attention as A, bobunex_config, bobunex_memory as M
    cfg = bobunex_config(vocab=157, width=72, eps=1e-5, embedding_scale=0.7, taps=4, layers=[
        (A(heads=10, kv_heads=5, dim=12, vdim=20, window=100, keep_first=33, scale=0.25, rot_dims=6, scaling=(8.0, 1.0, 4.0, 256)),
         M(heads=3, dim=96, vdim=16, gate_cap=12.0), 88),
        (A(heads=4, kv_heads=2, dim=64, vdim=64, window=40, keep_first=2, softcap=20.0, rot_dims=32), M(heads=2, dim=20, vdim=40), None),
        (A(heads=3, kv_heads=3, dim=16, vdim=8, window=1000, keep_first=0, softcap=0.0, rot_dims=16), M(heads=6, dim=8, vdim=12, gate_cap=4.0), 40)])
    folder = write_random_model(tmp_path / "m", cfg, seed=12)
    _, w = _read(folder)
    reqs = make_requests(157, [300, 270], seed=71)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    for mode in ("whole", "tail", "mixed"):
        steps, max_tokens = _steps(mode, reqs)
        _check(steps, run_trace(folder, dtype, steps, max_tokens, tmp_path / mode), reqs, plain, dtype)


def test_slots_and_pages_used_again_start_clean(bobunex_dirs, plain_memo, tmp_path):
    """Nine requests through a pool for two live ones with two state slots: every slot and page is used several times,
    and a request that follows a long one on its slot gets the same logits as alone."""
    folder = bobunex_dirs["bobunex-tiny-a"]
    reqs = make_requests(173, [90, 30, 64, 12, 100, 5, 77, 48, 33], seed=51)
    steps, max_tokens = mixed_steps(reqs, seed=2, max_live=2)
    from tokenmill_b200.engine.trace import run
    out_dir = tmp_path / "out"
    stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    assert run(str(folder), "float32", str(out_dir), max_tokens, stdin=stdin, stdout=io.StringIO(), state_slots=2) == 0
    outputs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, 173) for s in steps}
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_memo), "float32")


def test_first_tokens_and_single_token_requests(bobunex_dirs, plain_memo, tmp_path):
    """Requests of one, two and three tokens (shorter than the convolution's carried inputs), fed whole and token by
    token, beside each other."""
    folder = bobunex_dirs["bobunex-tiny-c"]       # five taps
    reqs = make_requests(130, [1, 2, 3, 4, 6], seed=61)
    plain = _plain(folder, reqs, plain_memo)
    whole = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in list(reqs.items())[:4]],
              "end": list(reqs)[:4]}]
    check_against_plain(whole, run_trace(folder, "float32", whole, 256, tmp_path / "w"), reqs, plain, "float32")
    reqs4 = {r: t for r, t in reqs.items() if r != "r0"}
    steps = [{"step": p, "entries": [{"id": r, "tokens": [t[p]], "want": [0]} for r, t in reqs4.items() if p < len(t)],
              "end": [r for r, t in reqs4.items() if p == len(t) - 1]} for p in range(6)]
    check_against_plain(steps, run_trace(folder, "float32", steps, 256, tmp_path / "t"), reqs4, plain, "float32")


# --- through the engine's own entry point -----------------------------------------------------------------------

@pytest.mark.parametrize("size,graphs,chunked,dtype", [
    ("bobunex-tiny-a", False, False, "float32"), ("bobunex-tiny-a", True, True, "float32"),
    ("bobunex-tiny-a", False, True, "bfloat16"), ("bobunex-tiny-d", True, True, "bfloat16")])
def test_greedy_generation_through_the_engine(bobunex_dirs, size, graphs, chunked, dtype):
    """LLMEngine with its scheduler: admission (state slots, two page groups with kept first pages), chunked prompts
    beside decodes, decode graphs with padded rows, a pool so small that requests are evicted and recomputed. The
    logits behind every generated token equal the plain model's on the request's own history, and the token is their
    arg-max."""
    from tokenmill_b200 import EngineConfig
    from tokenmill_b200.engine import LLMEngine
    from tokenmill_b200.sampling import SamplingParams

    folder = bobunex_dirs[size]
    cfg, w = _read(folder)
    rng = random.Random(5)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (9, 30, 17, 44, 5, 26, 12)]
    lefts = [layer["mixer"]["left"] for layer in cfg["layers"]]
    per_token = sum(a["kv_heads"] * (a["dim"] + a["vdim"]) for a in lefts) * (4 if dtype == "float32" else 2)
    eng = LLMEngine(EngineConfig(model=str(folder), dtype=dtype, block_size=8, max_model_len=128, max_num_seqs=4,
                                 kv_cache_mb=(16 * 8 + (8 if graphs else 0) + 1) * per_token / 2 ** 20, watermark=0.0,
                                 cuda_graphs=graphs, cuda_graph_max_batch=4, enable_chunked_prefill=chunked,
                                 max_num_batched_tokens=24 if chunked else 256))
    assert eng.cache.state_slots.num_slots == 4 and len(eng.cache.num_pages) == 2
    assert eng.cache.keep_first == [a["mask"]["keep_first"] for a in lefts]
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
    compared = 0
    for i, (p, r) in enumerate(zip(prompts, reqs)):
        assert len(r.output_ids) == 24
        plain = _logits(cfg, w, p + r.output_ids)
        for pos, row in rows[f"t{i}"]:
            ref = plain[pos]
            assert (row - ref).abs().max() <= (2e-4 if dtype == "float32" else 6e-2) * float(ref.abs().max()), (i, pos)
            if dtype == "float32":
                assert int(row.argmax()) == r.output_ids[pos - len(p) + 1]
            compared += 1
    assert compared >= 7 * 24


def test_generate_command_line_and_trace_runner(bobunex_dirs, tmp_path):
    """The two programs a user starts: ``python -m tokenmill_b200.generate`` on a Bobunex folder, and bin/trace_run."""
    root = Path(__file__).resolve().parents[1]
    folder = bobunex_dirs["bobunex-tiny-b"]
    res = subprocess.run([sys.executable, "-m", "tokenmill_b200.generate", "--model", str(folder), "--prompt-ids", "5,17,3,250",
                          "--max-tokens", "6", "--dtype", "float32", "--max-model-len", "64", "--kv-cache-mb", "1"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    cfg, w = _read(folder)
    toks = [5, 17, 3, 250]
    for _ in range(6):
        toks.append(int(_logits(cfg, w, toks)[-1].argmax()))
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
    plain = _logits(cfg, w, toks)
    got = np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(2, 300)
    last = np.fromfile(tmp_path / "o" / "2.f32", dtype="<f4").reshape(1, 300)
    for row, pos in ((got[0], 0), (got[1], 6), (last[0], 9)):
        assert np.abs(row - plain[pos].numpy()).max() <= 6e-2 * float(plain[pos].abs().max())
