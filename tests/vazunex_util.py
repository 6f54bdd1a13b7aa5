"""Small random Vazunex models for the tests: a config, bf16-rounded random weights, the folder the product loads."""
import json
import os

import numpy as np

from goponex_util import bf16_round, rel_err  # noqa: F401  (shared helpers)
from llama_cpp.safetensors_file import write_safetensors


def moe(experts=5, identity=1, top=2, ff=24, groups=(3, 2), scale=1.3):
    r = {"experts": experts, "identity": identity, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def latent(mlp=None, heads=3, dim=20, rot_dim=8, vdim=12, rank=28, window=16, base=5000.0, scale=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}, "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def delta(mlp=None, heads=4, kv_heads=2, dim=20, vdim=12, conv=3):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def ssd(mlp=None, heads=4, groups=2, vdim=12, state=20, norm_groups=2, conv=3):
    return {"type": "mamba2", "mixer": {"heads": heads, "groups": groups, "vdim": vdim, "state": state, "norm_groups": norm_groups, "conv": conv},
            "mlp": mlp}


def config(layers, width=72, vocab=131, mult=0.6, eps=1e-6, logit_scale=1.7):
    return {"architecture": "Vazunex", "layers": layers, "norm": {"eps": eps}, "residual_mult": mult, "logit_scale": logit_scale,
            "vocab": vocab, "width": width}


def random_weights(cfg, seed=0, ranks=(5, 7)):
    """Weights at a scale that keeps every mechanism alive (decays neither 0 nor 1, gates unsaturated, routing corrections
    large enough to change choices and to make choice scores negative), rounded to bf16 so the file and the oracle hold the
    same numbers. `ranks`: inner sizes of the delta rule's decay and gate projections."""
    from llama_cpp.vazunex import tensor_shapes
    rng = np.random.default_rng(seed)
    rk = {i: ranks for i, L in enumerate(cfg["layers"]) if L["type"] == "channel_delta"}
    w = {}
    for name, shape in tensor_shapes(cfg, rk).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "A_log":
            a = np.log(rng.uniform(0.3, 3.0, size=shape))
        elif leaf == "dt_bias":
            a = np.log(np.expm1(rng.uniform(0.02, 0.4, size=shape)))
        elif leaf == "conv":
            a = rng.standard_normal(shape) * 0.5
        elif leaf == "correction":
            a = rng.uniform(-0.6, 0.3, size=shape)
        elif leaf == "sink":
            a = rng.uniform(-1.0, 2.0, size=shape)
        elif leaf == "D":
            a = rng.uniform(0.5, 1.5, size=shape)
        elif leaf == "router":
            a = rng.standard_normal(shape) * 3.0 / np.sqrt(shape[1])
        elif len(shape) == 2:
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif name.endswith(("mix.norm", "dkv.norm")):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "b":                       # convolution bias
            a = rng.standard_normal(shape) * 0.2
        else:                                   # zero-centred norm weights
            a = 0.2 * rng.standard_normal(shape)
        w[name] = bf16_round(a)
    w["embed"] = bf16_round(rng.standard_normal(w["embed"].shape))
    return w


def write_model(folder, cfg, weights):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights, bf16=True)
    return folder
