"""A plain, slow statement of the Kutirax decoder, one function per mechanism, in float64 on the CPU.

Nothing here is shared with the engine: the tests build a tiny configuration and random weights, run
the engine on a GPU, and compare against these functions. Every function takes a whole sequence
[tokens, ...] and recomputes everything from position 0 (no cache, no state): that is what makes it an
independent answer to every question about caches, windows and carried state.

Notation: n tokens, width d. Weights are [out, in] and applied as ``x @ W.T``.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def offset_rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the weight is stored around zero."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + w)


def plain_rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu, with h_{-1} = 0 and h_{t-1} taken before the replacement."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mu


def rotate_half(v, positions, base, dims):
    """v [n, ..., D]: the first ``dims`` dimensions rotate, dimension i paired with i + dims/2, by the
    angle position * base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(F)[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = ang.cos().view(shape), ang.sin().view(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], dim=-1)


def latent_attention(h, w, p, eps):
    """Queries through a normed latent; keys and values expanded from a normed latent c, plus one rotated
    key part shared by the heads; softmax over the last ``window`` positions. p: heads, dim, rot_dim, vdim,
    kv_rank, q_rank, window, scale, rot_base, rot_dims."""
    n = h.shape[0]
    H, dn, dr, dv, rk = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    pos = torch.arange(n)
    cq = plain_rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(n, H, dn + dr)
    q_n, q_r = q[..., :dn], rotate_half(q[..., dn:], pos, p["rot_base"], p["rot_dims"])
    ckv = h @ w["dkv"].T
    c = plain_rms_norm(ckv[:, :rk], w["dkv.norm"], eps)
    k_r = rotate_half(ckv[:, rk:], pos, p["rot_base"], p["rot_dims"])           # [n, dr], one for all heads
    k_n = (c @ w["uk"].T).view(n, H, dn)
    v = (c @ w["uv"].T).view(n, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_n, k_n) + torch.einsum("ihd,jd->hij", q_r, k_r)) * p["scale"]
    i, j = pos[:, None], pos[None, :]
    visible = (i - j >= 0) & (i - j < p["window"])
    s = s.masked_fill(~visible[None], -math.inf)
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(n, H * dv)
    return o @ w["o"].T


def silu(z):
    return z * torch.sigmoid(z)


def mamba2(h, w, p, eps):
    """State-space mixer, token by token. p: heads, vdim, state, groups, conv, norm_groups."""
    n = h.shape[0]
    Hh, P, N, G, taps = p["heads"], p["vdim"], p["state"], p["groups"], p["conv"]
    inner = Hh * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    ch = xbc.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, ch, dtype=h.dtype), xbc], dim=0)
    conv = torch.zeros_like(xbc)
    for k in range(taps):                     # the last column weighs the current token
        conv = conv + padded[k:k + n] * w["conv"][:, k]
    xbc = silu(conv + w["conv.b"])
    x = xbc[:, :inner].view(n, Hh, P)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = torch.nn.functional.softplus(dt + w["dt_bias"], threshold=1e9)
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)                  # [n, heads]
    S = torch.zeros(Hh, N, P, dtype=h.dtype)
    y = torch.zeros(n, Hh, P, dtype=h.dtype)
    per = Hh // G
    for t in range(n):
        for hd in range(Hh):
            g = hd // per
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w["D"][hd] * x[t, hd]
    y = y.reshape(n, inner) * silu(z)
    parts = y.view(n, p["norm_groups"], inner // p["norm_groups"])
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    y = parts.reshape(n, inner) * w["norm"]
    return y @ w["o"].T


def relu2_feed_forward(h, w):
    return (torch.relu(h @ w["up"].T) ** 2) @ w["down"].T


def routed_feed_forward(h, w, p):
    """p: experts, top. The chosen experts' weights are a softmax over their logits alone."""
    logits = h @ w["router"].T + w["router.b"]
    top_v, top_i = torch.topk(logits, p["top"], dim=-1)
    gate = torch.softmax(top_v, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(p["top"]):
            e = int(top_i[t, k])
            a = silu(h[t] @ w[f"e{e}.gate"].T) * (h[t] @ w[f"e{e}.up"].T)
            out[t] = out[t] + gate[t, k] * (a @ w[f"e{e}.down"].T)
    return out


def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer_params(entry):
    m = entry["mixer"]
    if entry["type"] == "latent_attention":
        return dict(heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"],
                    q_rank=m["q_rank"], window=m["mask"]["size"], scale=m["scale"], rot_base=m["rot"]["base"],
                    rot_dims=m["rot"]["dims"])
    return dict(heads=m["heads"], vdim=m["vdim"], state=m["state"], groups=m["groups"], conv=m["conv"],
                norm_groups=m["norm_groups"])


def forward(config, weights, tokens, collect=None):
    """Logits [n, vocab] of a whole sequence. weights: name -> tensor. ``collect``, a list, receives the
    residual stream after every layer."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps, m = config["norm"]["eps"], config["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens)]
    for i, entry in enumerate(config["layers"]):
        pre = f"l{i}."
        h = token_shift(offset_rms_norm(x, w[pre + "norm1"], eps), w[pre + "shift"])
        mw, p = _sub(w, pre + "mix."), mixer_params(entry)
        mixed = latent_attention(h, mw, p, eps) if entry["type"] == "latent_attention" else mamba2(h, mw, p, eps)
        branch = mixed
        if entry["mlp"] is not None:
            g = offset_rms_norm(x, w[pre + "norm2"], eps)
            fw = _sub(w, pre + "mlp.")
            if entry["mlp"]["kind"] == "dense":
                branch = branch + relu2_feed_forward(g, fw)
            else:
                r = entry["mlp"]["router"]
                branch = branch + routed_feed_forward(g, fw, dict(experts=r["experts"], top=r["top"]))
        x = x + m * branch
        if collect is not None:
            collect.append(x.clone())
    x = offset_rms_norm(x, w["final.norm"], eps)
    return x @ w["embed"].T
