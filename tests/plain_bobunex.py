"""A plain, slow restatement of the Bobunex decoder: one function per mechanism, whole sequences at once, on
the CPU in 64-bit unless told otherwise. It shares no code with the engine: the tests hold the engine's kernels,
cache, state slots and batching against it.

``cfg`` is the parsed config.json; ``w`` maps tensor names to torch tensors.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_taps(h: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """conv(h)_t = sum_j weight[:, j] * h_(t - taps + 1 + j), zeros before the start. h [T, C], weight [C, taps]."""
    T, taps = h.shape[0], weight.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += weight[:, j] * h[s]
    return out


def rotary_frequencies(dims: int, base: float, scaling: dict | None) -> torch.Tensor:
    """f_i = base^(-2i/dims), then the wavelength-dependent scaling: short waves kept, long waves divided by
    ``factor``, a linear blend in between."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            wave = 2.0 * math.pi / f
            orig, lo, hi, factor = scaling["original"], scaling["low"], scaling["high"], scaling["factor"]
            if wave < orig / hi:
                pass
            elif wave > orig / lo:
                f = f / factor
            else:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate_half(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, heads, dim]: dimension i pairs with i + dims/2 for i < dims/2; the rest pass."""
    half = dims // 2
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]           # [T, half]
    c, s = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float, softcap: float,
                          window: int, keep_first: int) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]. Position i sees j <= i with i - j < window or
    j < keep_first; the softmax has one more term of score 0 and no value."""
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
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            out[i, h] = p @ v[js, g]
    return out


def matrix_memory(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_i: torch.Tensor, log_f: torch.Tensor,
                  state=None):
    """One head group of the matrix memory, token by token. q, k [T, H, d]; v [T, H, dv]; log_i, log_f [T, H].
    State (S [H, d, dv], n [H, d], m [H]) starts at zero. Returns (o [T, H, dv], state)."""
    T, H, d = q.shape
    dv = v.shape[-1]
    if state is None:
        state = (torch.zeros((H, d, dv), dtype=q.dtype), torch.zeros((H, d), dtype=q.dtype), torch.zeros((H,), dtype=q.dtype))
    S, n, m = (t.clone() for t in state)
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(log_f[t] + m, log_i[t])
        a = torch.exp(log_f[t] + m - m_new)
        b = torch.exp(log_i[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out, (S, n, m)


def left_mixer(h: torch.Tensor, positions: torch.Tensor, w: dict, p: str, c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = rms_norm(h @ w[p + ".q"].T, w[p + ".q.norm"], eps).view(T, H, d)
    k = rms_norm(h @ w[p + ".k"].T, w[p + ".k.norm"], eps).view(T, G, d)
    v = (h @ w[p + ".v"].T).view(T, G, dv)
    freqs = rotary_frequencies(c["rot"]["dims"], c["rot"]["base"], c["rot"].get("scaling"))
    q = rotate_half(q, positions, freqs, c["rot"]["dims"])
    k = rotate_half(k, positions, freqs, c["rot"]["dims"])
    o = sink_window_attention(q, k, v, scale=c["scale"], softcap=c["softcap"], window=c["mask"]["size"],
                              keep_first=c["mask"]["keep_first"])
    gate = torch.sigmoid(h @ w[p + ".g"].T)                                # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * dv) @ w[p + ".o"].T


def right_mixer(h: torch.Tensor, w: dict, p: str, c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv, cap = c["heads"], c["dim"], c["vdim"], c["gate_cap"]
    q = (h @ w[p + ".q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + ".k"].T).view(T, H, d)
    v = (h @ w[p + ".v"].T).view(T, H, dv)
    log_i = cap * torch.tanh((h @ w[p + ".i"].T + w[p + ".i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + ".f"].T + w[p + ".f.b"]) / cap))
    o, _ = matrix_memory(q, k, v, log_i, log_f)
    o = rms_norm(o, None, eps).reshape(T, H * dv) * w[p + ".norm"]
    return (o * torch.sigmoid(h @ w[p + ".g"].T)) @ w[p + ".o"].T


def pair_mixer(h, positions, w, p, c, eps):
    left = rms_norm(left_mixer(h, positions, w, p + ".left", c["left"], eps), w[p + ".left.out"], eps)
    right = rms_norm(right_mixer(h, w, p + ".right", c["right"], eps), w[p + ".right.out"], eps)
    return 0.5 * (left + right)


def feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


def forward(cfg: dict, w: dict, tokens: list[int], dtype=torch.float64):
    """(logits [T, vocab], residual stream after every layer [L, T, width])."""
    w = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in w.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = rms_norm(x, w[p + ".norm1"], eps)
        gate = torch.sigmoid(h @ w[p + ".rg1"].T + w[p + ".rg1.b"])
        x = x + gate * pair_mixer(h + causal_taps(h, w[p + ".canon1"]), positions, w, p + ".mix", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[p + ".norm2"], eps)
            gate = torch.sigmoid(h @ w[p + ".rg2"].T + w[p + ".rg2.b"])
            x = x + gate * feed_forward(h + causal_taps(h, w[p + ".canon2"]), w, p + ".mlp")
        streams.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(streams)
