"""Vazunex: a pre-norm hybrid decoder served by the layer-list graph of the native engine.

A model folder holds `config.json` and `model.safetensors`. Every layer is
    x <- x + m * mixer(norm1(x)),   x <- x + m * moe(norm2(x))        (m = `residual_mult`; `mlp` may be null)
with RMS norms whose stored weight is the deviation from one, and one of three token mixers:
  "latent_attention": sliding-window attention whose keys and values are per-head linear maps of one cached, normed
                      low-rank latent per token, plus one rotated key part shared by all heads (rotate-half pairing);
                      each head's softmax denominator carries a learned sink term; sigmoid output gate
  "channel_delta":    gated delta rule -- a [dim, vdim] memory per head whose rows decay at their own input-dependent rate;
                      short causal convolutions + SiLU on q, k, v; unit-length q and k; gated per-head output norm
  "mamba2":           state-space recurrence with one scalar decay per head, grouped B / C, gate before the grouped norm
The feed-forward block is a routed mixture of small gated (SiLU) experts: softmax scores, an additive correction that
only steers the choice, group-limited top-k, and identity slots that return their input.

This module turns the config into the C ABI's `b2_layer_desc` list (every size and constant comes from the file; the
inner sizes of the two-step decay / gate projections are read off the tensors) and checks the tensor set; the arithmetic
is in csrc/layered.cu, latent_attn.cu, state_mixers.cu, moe.cu and dense.cu.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from . import _cabi
from .goponex import LayeredDims, _need
from .models import Family, register

MIXERS = ("latent_attention", "channel_delta", "mamba2")


def layer_desc(i: int, layer: dict, ranks: Optional[Tuple[int, int]] = None) -> _cabi.B2LayerDesc:
    """`ranks`: inner sizes of the decay and gate projections of a channel_delta layer (rows of `a1` and `g1`)."""
    where = f"layers[{i}]"
    kind = _need(layer, "type", where)
    mix = _need(layer, "mixer", where)
    d = _cabi.B2LayerDesc()
    mlp = layer.get("mlp")
    if mlp:
        if mlp.get("kind", "moe") != "moe":
            raise ValueError(f"config.json: {where}: feed-forward kind {mlp.get('kind')!r} is not supported")
        r = _need(mlp, "router", where + ".mlp")
        d.ff_kind = _cabi.B2_FF_MOE
        d.n_ff = int(_need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert"))
        d.moe_experts, d.moe_identity, d.moe_top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
        groups = r.get("groups") or {}
        d.moe_groups = int(groups.get("count", 1))
        d.moe_keep = int(groups.get("keep", d.moe_groups))
        d.moe_scale = float(r.get("scale", 1.0))
    if kind == "latent_attention":
        d.mixer = _cabi.B2_MIX_LATENT_ATTN
        d.n_head, d.head_dim, d.la_rot_dim = int(mix["heads"]), int(mix["dim"]), int(mix["rot_dim"])
        d.la_vdim, d.la_rank = int(mix["vdim"]), int(mix["kv_rank"])
        rot = mix.get("rot") or {}
        d.rot_dims = int(rot.get("dims", d.la_rot_dim))
        d.rope_base = float(rot.get("base", 10000.0))
        d.rope_factor = 0.0
        mask = mix.get("mask")
        d.window = int(mask["size"]) if mask else 0
        d.attn_scale = float(_need(mix, "scale", where + ".mixer"))
    elif kind == "channel_delta":
        d.mixer = _cabi.B2_MIX_DELTA_RULE
        d.mm_heads, d.mm_dim, d.mm_vdim = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
        d.key_heads = int(mix.get("kv_heads", d.mm_heads))
        d.conv_taps = int(mix["conv"])
        if ranks is None:
            raise ValueError(f"config.json: {where}: the decay and gate projections' inner sizes come from the tensors")
        d.rank_a, d.rank_g = int(ranks[0]), int(ranks[1])
    elif kind == "mamba2":
        d.mixer = _cabi.B2_MIX_SSD
        d.mm_heads, d.mm_vdim, d.d_state = int(mix["heads"]), int(mix["vdim"]), int(mix["state"])
        d.key_heads = int(mix.get("groups", 1))
        d.norm_groups = int(mix.get("norm_groups", 1))
        d.conv_taps = int(mix["conv"])
    else:
        raise ValueError(f"config.json: {where}: unknown layer type {kind!r}")
    return d


def _ranks(i: int, shapes: Dict[str, Tuple[int, ...]]) -> Optional[Tuple[int, int]]:
    a, g = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
    return (int(a[0]), int(g[0])) if a and g else None


def read_dims(cfg: dict, shapes: Dict[str, Tuple[int, ...]]) -> LayeredDims:
    """`shapes`: name -> shape of the tensors at hand (the file's, or a synthetic set's)."""
    layers = _need(cfg, "layers", "the config")
    descs = [layer_desc(i, L, _ranks(i, shapes)) for i, L in enumerate(layers)]
    return LayeredDims(n_layer=len(descs), n_embd=int(_need(cfg, "width", "the config")), n_vocab=int(_need(cfg, "vocab", "the config")),
                       norm_eps=float(_need(_need(cfg, "norm", "the config"), "eps", "norm")),
                       residual_scale=float(cfg.get("residual_mult", 1.0)), layers=descs,
                       block_style=_cabi.B2_BLOCK_PRENORM_RMS, logit_scale=float(cfg.get("logit_scale", 1.0)))


def tensor_shapes(cfg: dict, ranks: Optional[Dict[int, Tuple[int, int]]] = None) -> Dict[str, Tuple[int, ...]]:
    """Every tensor the design needs, with its shape ([out, in] for linear maps). `ranks[i]` gives the inner sizes of layer
    i's decay and gate projections."""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (W,)
        if L["type"] == "latent_attention":
            H, d, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
            out.update({p + "mix.q": (H * (d + dr), W), p + "mix.dkv": (rank + dr, W), p + "mix.dkv.norm": (rank,),
                        p + "mix.uk": (H * d, rank), p + "mix.uv": (H * dv, rank), p + "mix.sink": (H,), p + "mix.g": (H * dv, W),
                        p + "mix.o": (W, H * dv)})
        elif L["type"] == "channel_delta":
            H, G, d, dv, taps = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"]), int(m["conv"])
            ra, rg = (ranks or {}).get(i, (0, 0))
            out.update({p + "mix.q": (G * d, W), p + "mix.q.conv": (G * d, taps), p + "mix.k": (G * d, W), p + "mix.k.conv": (G * d, taps),
                        p + "mix.v": (H * dv, W), p + "mix.v.conv": (H * dv, taps), p + "mix.b": (H, W), p + "mix.A_log": (H,),
                        p + "mix.norm": (dv,), p + "mix.a1": (ra, W), p + "mix.a2": (H * d, ra), p + "mix.dt_bias": (H * d,),
                        p + "mix.g1": (rg, W), p + "mix.g2": (H * dv, rg), p + "mix.o": (W, H * dv)})
        elif L["type"] == "mamba2":
            H, P, N, G, taps = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m.get("groups", 1)), int(m["conv"])
            inner, C = H * P, H * P + 2 * G * N
            out.update({p + "mix.in": (2 * inner + 2 * G * N + H, W), p + "mix.conv": (C, taps), p + "mix.conv.b": (C,),
                        p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        else:
            raise ValueError(f"config.json: layers[{i}]: unknown layer type {L['type']!r}")
        if L.get("mlp"):
            r, F = L["mlp"]["router"], int(L["mlp"]["expert"]["ff"])
            slots = int(r["experts"]) + int(r.get("identity", 0))
            out.update({p + "norm2": (W,), p + "mlp.router": (slots, W), p + "mlp.correction": (slots,)})
            for e in range(int(r["experts"])):
                out.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    return out


def synthetic(width: int, heads: int, ff: int, vocab: int, pattern: str = "ldsd", experts: int = 16, top: int = 4,
              window: int = 1024, seed: int = 0):
    """A random-weight model of realistic layer sizes, in memory (timing only). `pattern` lists the layers: "l" latent
    attention, "d" delta rule, "s" state-space; every layer has a mixture of `experts` experts of width `ff` (+ 2 identity
    slots). Returns (config dict, {name: tensor})."""
    import numpy as np
    from .safetensors_file import STensor
    moe = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "identity": 2, "top": top, "scale": 1.5, "groups": {"count": 3 if (experts + 2) % 3 == 0 else 1, "keep": 2 if (experts + 2) % 3 == 0 else 1}}}
    la = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "mask": {"size": window},
          "rot": {"base": 1e6, "dims": 64}, "scale": 192 ** -0.5}
    dl = {"heads": heads, "kv_heads": heads, "dim": 128, "vdim": 128, "conv": 4}
    ss = {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}
    kinds = {"l": ("latent_attention", la), "d": ("channel_delta", dl), "s": ("mamba2", ss)}
    cfg = {"architecture": "Vazunex", "layers": [{"type": kinds[ch][0], "mixer": kinds[ch][1], "mlp": moe} for ch in pattern],
           "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_scale": 1.0, "vocab": vocab, "width": width}
    rank = max(16, width // 64)
    ranks = {i: (rank, rank) for i, ch in enumerate(pattern) if ch == "d"}
    rng = np.random.default_rng(seed)
    tensors = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        n = int(np.prod(shape))
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "A_log":
            a = np.log(rng.uniform(0.5, 4.0, size=n)).astype(np.float32)
        elif leaf == "dt_bias":
            a = np.log(np.expm1(rng.uniform(0.01, 0.2, size=n))).astype(np.float32)
        elif leaf == "conv":
            a = rng.standard_normal(n, dtype=np.float32) * 0.4
        elif len(shape) == 2:
            a = rng.standard_normal(n, dtype=np.float32) / np.sqrt(shape[1])
        elif leaf == "D" or name.endswith("mix.norm"):
            a = np.ones(n, dtype=np.float32)
        else:                       # zero-centred norm weights, sinks, corrections, convolution biases
            a = rng.standard_normal(n, dtype=np.float32) * 0.05
        bits = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)       # truncation is fine for random weights
        tensors[name] = STensor(name, "BF16", tuple(shape), bits.reshape(shape))
    return cfg, tensors


def open_synthetic(cfg, tensors, **kw):
    from .engine import LayeredEngine
    return LayeredEngine(read_dims(cfg, {n: tuple(t.shape) for n, t in tensors.items()}), tensors, **kw)


def _open(src, **kw):
    from .engine import LayeredEngine
    have = src.weights.tensors
    shapes = {n: tuple(t.shape) for n, t in have.items()}
    dims = read_dims(src.config, shapes)
    ranks = {i: r for i in range(dims.n_layer) if (r := _ranks(i, shapes))}
    want = tensor_shapes(src.config, ranks)
    for name, shape in want.items():
        if name not in have:
            raise ValueError(f"{src.path}: tensor {name} is missing")
        if tuple(have[name].shape) != tuple(shape):
            raise ValueError(f"{src.path}: tensor {name} has shape {tuple(have[name].shape)}, the config asks for {tuple(shape)}")
    return LayeredEngine(dims, {n: have[n] for n in want}, **kw)


VAZUNEX = register(Family(name="Vazunex", source="folder", open_engine=_open))
