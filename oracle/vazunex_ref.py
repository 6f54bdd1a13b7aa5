"""Plain float64 restatement of the Vazunex decoder (test oracle only; the product path never imports it).

Vazunex is a pre-norm hybrid: every layer is  x <- x + m * mixer(norm1(x)),  x <- x + m * moe(norm2(x))  with one of three
token mixers -- windowed latent attention with a softmax sink, a gated delta rule with per-channel decay, or a Mamba-2
state-space layer -- and a routed mixture of small gated feed-forward experts (some of them identities).

One function per mechanism, whole sequences at a time, no cache and no batching: every token's output is computed from
the full prefix the slow way. `weights` maps tensor names to float arrays, `cfg` is the parsed config.json dictionary.

Notation: h [T, W] is a sublayer's input, positions count from 0, linear maps are stored [out, in].
"""
from __future__ import annotations

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def zero_centred_norm(x, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return unit_rms(x, eps) * (1.0 + w)


def causal_conv(x, taps_w, bias=None):
    """x [T, C], taps_w [C, taps] with the last column on the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    xp = np.concatenate([np.zeros((taps - 1, C), dtype=F), x], 0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += xp[j:j + T, :] * taps_w[:, j][None, :]
    return y if bias is None else y + bias


def rotate_half(x, positions, base, dims):
    """x [T, ..., d]: entry i of the first `dims` is paired with entry i + dims/2; the rest pass through."""
    half = dims // 2
    f = float(base) ** (-2.0 * np.arange(half, dtype=F) / dims)
    ang = np.asarray(positions, dtype=F)[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def latent_attention(h, w, pre, m, eps):
    """Keys and values are expanded per head from one normed low-rank latent per token; one rotated key part is shared
    by all heads; sliding window; the softmax denominator carries one extra learned term per head (the sink)."""
    T = h.shape[0]
    H, d, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m["rot"]
    q = (h @ w[pre + "q"].T).reshape(T, H, d + dr)
    q_c, q_r = q[..., :d], q[..., d:]
    dkv = h @ w[pre + "dkv"].T
    c = unit_rms(dkv[:, :rank], eps) * w[pre + "dkv.norm"]
    k_r = dkv[:, rank:rank + dr]
    pos = np.arange(T)
    q_r = rotate_half(q_r, pos, rot["base"], int(rot["dims"]))
    k_r = rotate_half(k_r, pos, rot["base"], int(rot["dims"]))
    k_c = (c @ w[pre + "uk"].T).reshape(T, H, d)
    v = (c @ w[pre + "uv"].T).reshape(T, H, dv)
    window = int(m["mask"]["size"]) if m.get("mask") else T
    ii, jj = pos[:, None], pos[None, :]
    visible = (jj <= ii) & (ii - jj < window)
    out = np.zeros((T, H, dv), dtype=F)
    for hh in range(H):
        s = (q_c[:, hh, :] @ k_c[:, hh, :].T + q_r[:, hh, :] @ k_r.T) * float(m["scale"])
        s = np.where(visible, s, -np.inf)
        sink = float(w[pre + "sink"][hh])
        mx = np.maximum(s.max(-1, keepdims=True), sink)
        p = np.exp(s - mx)
        den = p.sum(-1, keepdims=True) + np.exp(sink - mx)
        out[:, hh, :] = (p / den) @ v[:, hh, :]
    gate = sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[pre + "o"].T


def channel_delta(h, w, pre, m, eps):
    """Gated delta rule: per head a [dim, vdim] memory whose rows decay each with its own input-dependent rate; the write
    is the error between the value and what the memory already returns for the key."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[pre + "b"].T)
    rate = np.exp(w[pre + "A_log"])
    a = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]
    decay = np.exp(-rate[None, :, None] * softplus(a).reshape(T, H, d))
    S = np.zeros((H, d, dv), dtype=F)
    o = np.zeros((T, H, dv), dtype=F)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = decay[t, hh][:, None] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, g])
            S[hh] = S[hh] + np.outer(k[t, g], u)
            o[t, hh] = S[hh].T @ q[t, g]
    o = unit_rms(o, eps) * w[pre + "norm"]
    gate = sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T)
    return (o.reshape(T, H * dv) * gate) @ w[pre + "o"].T


def mamba2(h, w, pre, m, eps):
    """State-space layer with one scalar decay per head and input/output maps shared by the heads of a group."""
    T = h.shape[0]
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    parts = int(m.get("norm_groups", 1))
    inner = H * P
    zx = h @ w[pre + "in"].T
    z = zx[:, :inner]
    xbc = silu(causal_conv(zx[:, inner:2 * inner + 2 * G * N], w[pre + "conv"], w[pre + "conv.b"]))
    dt = softplus(zx[:, 2 * inner + 2 * G * N:] + w[pre + "dt_bias"])
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    rate = np.exp(w[pre + "A_log"])
    S = np.zeros((H, N, P), dtype=F)
    y = np.zeros((T, H, P), dtype=F)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = np.exp(-rate[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + w[pre + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def route(h, w, pre, r):
    """Chosen slots [T, top] and their weights. Slots >= experts are identities."""
    n_slots = int(r["experts"]) + int(r.get("identity", 0))
    top = int(r["top"])
    z = h @ w[pre + "router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(-1, keepdims=True)
    choice = s + w[pre + "correction"]
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = n_slots // count
        best = choice.reshape(-1, count, per).max(-1)
        kept = np.argsort(-best, axis=-1, kind="stable")[:, :keep]
        allowed = np.zeros((h.shape[0], count), dtype=bool)
        np.put_along_axis(allowed, kept, True, axis=-1)
        choice = np.where(np.repeat(allowed, per, axis=-1), choice, -np.inf)
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    weight = np.take_along_axis(s, chosen, axis=-1) * float(r["scale"])
    return chosen, weight


def mixture(h, w, pre, mlp):
    r = mlp["router"]
    E = int(r["experts"])
    chosen, weight = route(h, w, pre, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], weight[t]):
            if e >= E:
                out[t] += a * h[t]
            else:
                p = f"{pre}e{e}."
                out[t] += a * (w[p + "down"] @ (silu(w[p + "gate"] @ h[t]) * (w[p + "up"] @ h[t])))
    return out


MIXERS = {"latent_attention": latent_attention, "channel_delta": channel_delta, "mamba2": mamba2}


def forward(cfg, weights, tokens, return_layers=False):
    """logits [T, vocab] (and the residual stream after every layer [L, T, W])."""
    w = {k: np.asarray(v, dtype=F) for k, v in weights.items()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = zero_centred_norm(w["embed"][np.asarray(tokens, dtype=np.int64)], w["embed.norm"], eps)
    trace = []
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        x = x + mult * MIXERS[L["type"]](zero_centred_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            x = x + mult * mixture(zero_centred_norm(x, w[p + "norm2"], eps), w, p + "mlp.", L["mlp"])
        trace.append(x.copy())
    logits = zero_centred_norm(x, w["final.norm"], eps) @ w["head"].T * float(cfg["logit_scale"])
    return (logits, np.stack(trace)) if return_layers else logits
