"""Small random Goponex models for the tests: a config, bf16-rounded random weights, the folder the product loads."""
import json
import os

import numpy as np

from llama_cpp.safetensors_file import float32_to_bf16_bits, write_safetensors


def attn(heads=4, kv_heads=2, dim=24, rot=8, window=16, keep=3, scale=None, scaling=True, base=5000.0):
    r = {"base": base, "dims": rot}
    if scaling:
        r["scaling"] = {"factor": 4.0, "fast": 16.0, "original": 64, "slow": 2.0}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "rot": r,
            "mask": {"size": window, "keep_first": keep}, "scale": float(scale if scale is not None else dim ** -0.5)}


def scan(inner=40, state=12, dt_rank=5, conv=3):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def parallel(mlp=None, left=None, right=None):
    return {"type": "parallel", "mixer": {"left": left or attn(), "right": right or scan()},
            "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def mlstm(mlp=None, heads=3, dim=20, vdim=28, cap=12.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def config(layers, width=72, vocab=131, alpha=1.5, eps=1e-6):
    return {"architecture": "Goponex", "layers": layers, "norm": {"eps": eps}, "postln_alpha": alpha, "vocab": vocab, "width": width}


def bf16_round(a):
    return (float32_to_bf16_bits(np.asarray(a, dtype=np.float32)).astype(np.uint32) << 16).view(np.float32)


def random_weights(cfg, seed=0):
    """Weights at a scale that keeps every mechanism alive (decays neither 0 nor 1, gates unsaturated), rounded to bf16 so
    the file and the oracle hold the same numbers."""
    from llama_cpp.goponex import tensor_shapes
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if len(shape) == 2 and not leaf.endswith(("conv", "A_log")):
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
            if leaf in ("mix.i", "mix.f"):
                a *= 2.0
        elif leaf.endswith("A_log"):
            a = np.log(rng.uniform(0.5, 8.0, size=shape))
        elif leaf.endswith("conv"):
            a = rng.standard_normal(shape) * 0.5
        elif leaf.endswith("dt.b"):
            a = np.log(np.expm1(rng.uniform(0.01, 0.3, size=shape)))
        elif leaf.endswith("f.b"):
            a = rng.uniform(1.0, 4.0, size=shape)
        elif leaf.endswith(".b"):
            a = rng.standard_normal(shape) * 0.2
        elif leaf.endswith("D"):
            a = rng.uniform(0.5, 1.5, size=shape)
        else:                                   # norm weights
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        w[name] = bf16_round(a)
    w["embed"] = bf16_round(rng.standard_normal(w["embed"].shape))
    return w


def write_model(folder, cfg, weights):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights, bf16=True)
    return folder


def rel_err(got, want):
    """Root mean square of the difference over the root mean square of the reference, rows centred like logits."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    ref = want - want.mean(-1, keepdims=True)
    return float(np.sqrt((d ** 2).mean(-1)).max() / max(np.sqrt((ref ** 2).mean()), 1e-12))
