"""Host-side pieces of the Vazunex family (no GPU): config -> layer descriptors, the tensor set, the registry, and sanity
properties of the float64 oracle's mechanisms."""
import numpy as np
import pytest

import vazunex_util as vu
from oracle import vazunex_ref as ref


def test_config_to_descriptors():
    from llama_cpp import _cabi, vazunex
    cfg = vu.config([vu.latent(mlp=vu.moe(experts=7, identity=2, top=3, ff=16, groups=(3, 2), scale=2.5), window=21),
                     vu.delta(heads=6, kv_heads=2, dim=10, vdim=14, conv=5), vu.ssd(heads=4, groups=2, vdim=6, state=9, norm_groups=4, conv=2)],
                    mult=0.25, logit_scale=3.0)
    shapes = vazunex.tensor_shapes(cfg, {1: (11, 13)})
    d = vazunex.read_dims(cfg, shapes)
    assert d.block_style == _cabi.B2_BLOCK_PRENORM_RMS and d.logit_scale == 3.0 and d.residual_scale == 0.25
    a, b, c = d.layers
    assert (a.mixer, a.n_head, a.head_dim, a.la_rot_dim, a.la_vdim, a.la_rank, a.window, a.rot_dims) == (_cabi.B2_MIX_LATENT_ATTN, 3, 20, 8, 12, 28, 21, 8)
    assert (a.ff_kind, a.n_ff, a.moe_experts, a.moe_identity, a.moe_top, a.moe_groups, a.moe_keep, a.moe_scale) == (_cabi.B2_FF_MOE, 16, 7, 2, 3, 3, 2, 2.5)
    assert (b.mixer, b.mm_heads, b.key_heads, b.mm_dim, b.mm_vdim, b.conv_taps, b.rank_a, b.rank_g, b.n_ff) == (_cabi.B2_MIX_DELTA_RULE, 6, 2, 10, 14, 5, 11, 13, 0)
    assert (c.mixer, c.mm_heads, c.key_heads, c.mm_vdim, c.d_state, c.norm_groups, c.conv_taps) == (_cabi.B2_MIX_SSD, 4, 2, 6, 9, 4, 2)
    assert shapes["l0.mlp.router"] == (9, 72) and shapes["l1.mix.a2"] == (60, 11) and shapes["l2.mix.in"] == (2 * 24 + 2 * 18 + 4, 72)


def test_registry_and_folder(tmp_path):
    from llama_cpp import models
    cfg = vu.config([vu.delta(mlp=vu.moe())])
    path = vu.write_model(str(tmp_path / "m"), cfg, vu.random_weights(cfg))
    src = models.open_model(path)
    assert src.family.name == "Vazunex" and "Vazunex" in models.architectures() and "Goponex" in models.architectures()
    with pytest.raises(ValueError):
        from llama_cpp import vazunex
        vazunex.layer_desc(0, {"type": "nope", "mixer": {}})


def test_delta_rule_stores_and_returns_a_value():
    """With no decay and full write strength the memory returns exactly the value just written for its key."""
    rng = np.random.default_rng(0)
    k = rng.standard_normal(6)
    k /= np.linalg.norm(k)
    S = rng.standard_normal((6, 4))
    v = rng.standard_normal(4)
    S2 = S + np.outer(k, 1.0 * (v - S.T @ k))
    assert np.allclose(S2.T @ k, v)


def test_sink_only_takes_weight():
    cfg = vu.config([vu.latent(window=8)])
    w = vu.random_weights(cfg, seed=1)
    h = np.random.default_rng(2).standard_normal((12, cfg["width"]))
    wd = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    a = ref.latent_attention(h, wd, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6)
    wd["l0.mix.sink"] = wd["l0.mix.sink"] + 50.0
    b = ref.latent_attention(h, wd, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6)
    assert np.abs(b).max() < 1e-12 < np.abs(a).max()


def test_dropped_groups_count_as_minus_infinity():
    """All choice scores negative: a slot of a dropped group must not win against a kept group's negative score."""
    r = {"experts": 4, "identity": 0, "top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}}
    w = {"p.router": np.zeros((4, 3)), "p.correction": np.array([-0.9, -0.8, -0.3, -0.95])}
    chosen, weight = ref.route(np.ones((1, 3)), w, "p.", r)
    assert sorted(chosen[0]) == [2, 3] and np.allclose(weight, 0.25)


def test_oracle_streams_are_causal():
    cfg = vu.config([vu.latent(mlp=vu.moe()), vu.delta(), vu.ssd()])
    w = vu.random_weights(cfg, seed=4)
    toks = [int(t) for t in np.random.default_rng(5).integers(0, cfg["vocab"], size=30)]
    full = ref.forward(cfg, w, toks)
    assert np.allclose(ref.forward(cfg, w, toks[:17]), full[:17], atol=1e-10)
