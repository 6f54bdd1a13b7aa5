"""Plain float64 restatement of the Goponex decoder (test oracle only; the product path never imports it).

One function per mechanism, whole sequences at a time, no cache and no batching: every token's output is
computed from the full prefix the slow way. `weights` maps tensor names to float arrays, `cfg` is the
parsed config.json dictionary.

Notation: h [T, W] is a sublayer's input, positions count from 0, linear maps are stored [out, in].
"""
from __future__ import annotations

import math

import numpy as np

F = np.float64


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def rotary_tables(rot, positions):
    """cos, sin [T, dims/2] of the scaled rotary embedding (frequency blend between interpolated and original,
    magnitude correction on both tables)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = np.arange(half, dtype=F)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = np.asarray(positions, dtype=F)[:, None] * f[None, :]
    return np.cos(ang) * mag, np.sin(ang) * mag


def rotate_interleaved(x, cos, sin, dims):
    """x [T, heads, d]: pairs (2i, 2i+1) of the first `dims` entries are rotated, the rest pass through."""
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def window_attention(h, w, pre, m, eps):
    """Grouped-query attention whose values are the un-normalised, un-rotated keys; sliding window plus a kept prefix."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[pre + "q"].T).reshape(T, H, d)
    k = (h @ w[pre + "k"].T).reshape(T, G, d)
    v = k.copy()
    q = unit_rms(q, eps) * w[pre + "q.norm"]
    k = unit_rms(k, eps) * w[pre + "k.norm"]
    pos = np.arange(T)
    cos, sin = rotary_tables(m["rot"], pos)
    rd = int(m["rot"]["dims"])
    q = rotate_interleaved(q, cos, sin, rd)
    k = rotate_interleaved(k, cos, sin, rd)
    size, keep = int(m["mask"]["size"]), int(m["mask"]["keep_first"])
    ii, jj = pos[:, None], pos[None, :]
    visible = (jj <= ii) & ((ii - jj < size) | (jj < keep))
    out = np.zeros((T, H, d), dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh, :] @ k[:, g, :].T) * float(m["scale"])
        s = np.where(visible, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(-1, keepdims=True)
        out[:, hh, :] = p @ v[:, g, :]
    return out.reshape(T, H * d) @ w[pre + "o"].T


def selective_scan(h, w, pre, m):
    """Mamba block: gated causal depthwise convolution, input-dependent step size, diagonal state recurrence."""
    T = h.shape[0]
    inner, N, R, taps = int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m["conv"])
    xz = h @ w[pre + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    cw, cb = w[pre + "conv"], w[pre + "conv.b"]
    xp = np.concatenate([np.zeros((taps - 1, inner), dtype=F), x], 0)
    xc = np.zeros_like(x)
    for j in range(taps):
        xc += xp[j:j + T, :] * cw[:, j][None, :]
    xc = silu(xc + cb)
    proj = xc @ w[pre + "x"].T
    dt_in, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = softplus(dt_in @ w[pre + "dt"].T + w[pre + "dt.b"])
    A = -np.exp(w[pre + "A_log"])
    S = np.zeros((inner, N), dtype=F)
    y = np.zeros((T, inner), dtype=F)
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * xc[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[pre + "D"] * xc[t]
    y = y * silu(z)
    return y @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    a = window_attention(h, w, pre + "left.", m["left"], eps)
    b = selective_scan(h, w, pre + "right.", m["right"])
    return 0.5 * (unit_rms(a, eps) * w[pre + "left.out"] + unit_rms(b, eps) * w[pre + "right.out"])


def matrix_memory(h, w, pre, m, eps):
    """mLSTM: per-head matrix memory with exponential input gate, stabilised by a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ w[pre + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).reshape(T, H, d)
    v = (h @ w[pre + "v"].T).reshape(T, H, dv)
    ig = cap * np.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)
    fg = log_sigmoid(cap * np.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    S = np.zeros((H, d, dv), dtype=F)
    n = np.zeros((H, d), dtype=F)
    mx = np.zeros(H, dtype=F)
    o = np.zeros((T, H, dv), dtype=F)
    for t in range(T):
        m_new = np.maximum(fg[t] + mx, ig[t])
        a = np.exp(fg[t] + mx - m_new)
        b = np.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = np.einsum("hdv,hd->hv", S, q[t])
        den = np.maximum(np.abs((n * q[t]).sum(-1)), np.exp(-mx)) + 1e-6
        o[t] = num / den[:, None]
    o = unit_rms(o, eps).reshape(T, H * dv) * w[pre + "norm"]
    o = o * sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def feed_forward(h, w, pre):
    u = h @ w[pre + "up"].T + w[pre + "up.b"]
    u = np.maximum(u, 0.0) ** 2
    return u @ w[pre + "down"].T + w[pre + "down.b"]


def forward(cfg, weights, tokens, return_layers=False):
    """logits [T, vocab] (and the residual stream after every layer [L, T, W])."""
    w = {k: np.asarray(v, dtype=F) for k, v in weights.items()}
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    x = w["embed"][np.asarray(tokens, dtype=np.int64)]
    trace = []
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        if L["type"] == "parallel":
            y = parallel_mixer(x, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "mlstm":
            y = matrix_memory(x, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {L['type']!r}")
        x = layer_norm(alpha * x + y, w[p + "norm1"], eps)
        if L.get("mlp"):
            x = layer_norm(alpha * x + feed_forward(x, w, p + "mlp."), w[p + "norm2"], eps)
        trace.append(x.copy())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(trace)) if return_layers else logits
