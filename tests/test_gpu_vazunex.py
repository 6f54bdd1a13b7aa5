"""Vazunex through the native engine against the float64 oracle (oracle/vazunex_ref.py), on small random models the tests
make themselves: each mixer and the expert mixture alone, prompt against token-by-token decoding, portions down to two
tokens, unequal batches against each request alone, slots and pages used again, keys just inside and just outside the
window and at page borders, the softmax sink, far tokens through the recurrent state, the first tokens, long decoding,
degenerate and odd sizes, and greedy generation through `Llama` and the scheduler."""
import copy
import threading

import numpy as np
import pytest

import vazunex_util as vu
from oracle import vazunex_ref as ref

pytestmark = pytest.mark.gpu

TOL = {"float32": 3e-4, "bfloat16": 6e-2}


def open_engine(path, dtype="float32", n_ctx=512, max_seqs=4, kv_tokens=None, max_step_tokens=None, flags=0):
    from llama_cpp import models
    return models.open_engine(models.open_model(path), n_ctx=n_ctx, max_seqs=max_seqs, dtype=dtype, kv_tokens=kv_tokens,
                              max_step_tokens=max_step_tokens, flags=flags)


def run_cut(eng, seqs, key, tokens, cuts):
    """All logits of `tokens`, fed in portions of the given sizes (cycled)."""
    rows, pos, k = [], 0, 0
    seqs.open(key)
    while pos < len(tokens):
        n = min(cuts[k % len(cuts)], len(tokens) - pos)
        k += 1
        slot = seqs.extend(key, n)
        lg, _ = eng.step([(slot, tokens[pos:pos + n])], want=[list(range(n))])
        rows.append(lg)
        pos += n
    seqs.close(key)
    return np.concatenate(rows)


def close(got, want, dtype):
    """float32: every row within the tolerance. bfloat16: the rounded activations can tip a near-tie of the router the other
    way than the oracle's, which moves that row (and, slightly, later ones) by a whole expert; so the typical row must be
    well inside the tolerance and at most one row in twenty may leave it."""
    if dtype == "float32":
        return vu.rel_err(got, want) < TOL[dtype]
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    ref_rms = np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())
    rows = np.sqrt((d ** 2).mean(-1)) / ref_rms
    return np.median(rows) < TOL[dtype] / 4 and (rows > TOL[dtype]).mean() <= 0.05


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


@pytest.fixture(scope="module")
def hybrid(native_lib, tmp_path_factory):
    cfg = vu.config([vu.latent(mlp=vu.moe()), vu.delta(mlp=vu.moe(experts=7, identity=2, top=3, ff=16)), vu.ssd(mlp=None),
                     vu.delta(mlp=vu.moe(groups=None), heads=3, kv_heads=3, dim=16, vdim=24, conv=4),
                     vu.latent(mlp=vu.moe(experts=4, identity=0, top=2, groups=(2, 1)), heads=2, dim=16, rot_dim=16, vdim=16, rank=48, window=70)])
    w = vu.random_weights(cfg, seed=3)
    path = vu.write_model(str(tmp_path_factory.mktemp("vazunex_hybrid")), cfg, w)
    return cfg, w, path


LAYERS = {
    "latent": lambda: vu.latent(),
    "latent_moe": lambda: vu.latent(mlp=vu.moe(), heads=2, dim=32, rot_dim=4, vdim=40, rank=64, window=33),
    "delta": lambda: vu.delta(),
    "delta_moe": lambda: vu.delta(mlp=vu.moe(experts=10, identity=2, top=4, ff=20, groups=(4, 3)), heads=2, kv_heads=1, dim=40, vdim=36, conv=2),
    "ssd": lambda: vu.ssd(),
    "ssd_moe": lambda: vu.ssd(mlp=vu.moe(experts=3, identity=3, top=2, groups=(2, 2)), heads=6, groups=3, vdim=8, state=36, norm_groups=1, conv=4),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", sorted(LAYERS))
def test_each_mixer_alone(native_lib, tmp_path, layer, dtype):
    from llama_cpp.kv_pages import SequenceSlots
    cfg = vu.config([LAYERS[layer]()])
    w = vu.random_weights(cfg, seed=11)
    eng = open_engine(vu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 90, 1)
    want_logits, want_layers = ref.forward(cfg, w, toks, return_layers=True)
    seqs = SequenceSlots(eng)
    eng.trace_layers(True)
    seqs.open("a")
    slot = seqs.extend("a", len(toks))
    got, _ = eng.step([(slot, toks)], want=[list(range(len(toks)))])
    layers = eng.layer_outputs(len(toks))
    eng.close()
    assert close(layers[0], want_layers[0], dtype)
    assert close(got, want_logits, dtype)


def test_routing_is_not_trivial(hybrid):
    """The test weights make the routing mechanisms matter: identity slots are chosen, a dropped group holds a slot that would
    have been chosen, the correction changes choices, and some choice scores are negative."""
    cfg, w, _ = hybrid
    wd = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    h = np.random.default_rng(0).standard_normal((200, cfg["width"]))
    r = cfg["layers"][1]["mlp"]["router"]
    chosen, weight = ref.route(h, wd, "l1.mlp.", r)
    assert (chosen >= r["experts"]).any() and (chosen < r["experts"]).any()
    free = copy.deepcopy(r)
    del free["groups"]
    assert (np.sort(ref.route(h, wd, "l1.mlp.", free)[0]) != np.sort(chosen)).any()
    flat = dict(wd)
    flat["l1.mlp.correction"] = np.zeros_like(wd["l1.mlp.correction"])
    assert (np.sort(ref.route(h, flat, "l1.mlp.", r)[0]) != np.sort(chosen)).any()
    z = h @ wd["l1.mlp.router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    assert ((s / s.sum(-1, keepdims=True) + wd["l1.mlp.correction"]) < 0).any()
    assert abs(weight.sum(-1) - float(r["scale"])).max() > 0.05          # not renormalised


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_against_token_by_token(hybrid, dtype):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    seqs = SequenceSlots(eng)
    toks = tokens_for(cfg, 150, 2)
    want = ref.forward(cfg, w, toks)
    whole = run_cut(eng, seqs, "w", toks, [len(toks)])
    single = run_cut(eng, seqs, "s", toks, [1])
    eng.close()
    assert close(whole, want, dtype)
    assert close(single, want, dtype)
    assert close(single, whole, dtype)


@pytest.mark.parametrize("cuts", [[2], [3, 2, 5, 1], [17, 64, 2, 9], [63, 1, 1, 70]])
def test_portions(hybrid, cuts):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32")
    toks = tokens_for(cfg, 140, 4)
    got = run_cut(eng, SequenceSlots(eng), "p", toks, cuts)
    eng.close()
    assert vu.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(hybrid, dtype):
    """Three requests of different lengths advance together, portions of some beside single tokens of others."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    seqs = SequenceSlots(eng)
    reqs = {"a": tokens_for(cfg, 131, 5), "b": tokens_for(cfg, 40, 6), "c": tokens_for(cfg, 77, 7)}
    alone = {k: run_cut(eng, seqs, k + "_alone", t, [len(t)]) for k, t in reqs.items()}
    plan = {"a": [50, 1, 1, 30, 2, 1], "b": [1, 1, 9, 1], "c": [2, 40, 1, 1, 20]}
    at = {k: 0 for k in reqs}
    turn = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for k in reqs:
        seqs.open(k)
    while any(at[k] < len(reqs[k]) for k in reqs):
        entries, want, who = [], [], []
        for k, t in reqs.items():
            if at[k] >= len(t):
                continue
            n = min(plan[k][turn[k] % len(plan[k])], len(t) - at[k])
            turn[k] += 1
            entries.append((seqs.extend(k, n), t[at[k]:at[k] + n]))
            want.append(list(range(n)))
            who.append((k, n))
            at[k] += n
        lg, _ = eng.step(entries, want=want)
        r = 0
        for k, n in who:
            got[k].append(lg[r:r + n])
            r += n
    eng.close()
    for k, t in reqs.items():
        mixed = np.concatenate(got[k])
        assert vu.rel_err(mixed, alone[k]) < 2e-5 if dtype == "float32" else close(mixed, alone[k], dtype)
        assert close(mixed, ref.forward(cfg, w, t), dtype)


def test_slots_and_pages_used_again(hybrid):
    """One slot, a pool of three pages: every sequence runs in the pages and the state slot the previous one left."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32", n_ctx=192, max_seqs=1, kv_tokens=192)
    seqs = SequenceSlots(eng)
    for i, n in enumerate([150, 70, 192, 3]):
        toks = tokens_for(cfg, n, 20 + i)
        got = run_cut(eng, seqs, f"s{i}", toks, [40, 1, 23])
        assert seqs.free_slots == 1 and eng.pages.free_pages == 3
        assert vu.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"], i
    eng.close()


def _peaky_latent_model(tmp_path, window):
    """One latent-attention layer in which a token attends to earlier copies of itself whenever the mask lets it: the key map
    of every head is the identity on the latent and the unrotated query rows repeat the latent's projection, so a copy's key
    is parallel to the query and scores as high as the token's own key, far above the random rest; the rotated part is small.
    The score scale is low enough that the token's own key, the copy, the sink and the rest all hold a visible share."""
    H, d = 2, 32
    cfg = vu.config([vu.latent(heads=H, dim=d, rot_dim=16, vdim=24, rank=d, window=window, scale=0.08)], width=64)
    w = vu.random_weights(cfg, seed=5)
    q = w["l0.mix.q"].reshape(H, d + 16, -1).copy()
    q[:, :d, :] = w["l0.mix.dkv"][:d] * 1.5
    q[:, d:, :] *= 0.1
    w["l0.mix.q"] = vu.bf16_round(q.reshape(H * (d + 16), -1))
    w["l0.mix.uk"] = vu.bf16_round(np.tile(np.eye(d), (H, 1)))
    w["l0.mix.dkv.norm"] = vu.bf16_round(np.ones(d))
    w["l0.mix.sink"] = vu.bf16_round(np.array([3.0, 4.0]))
    return cfg, w, vu.write_model(str(tmp_path / "peaky"), cfg, w)


def _with_window(cfg, size):
    c = copy.deepcopy(cfg)
    c["layers"][0]["mixer"]["mask"]["size"] = size
    return c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_window_edges_and_sink(native_lib, tmp_path, decode, dtype):
    """The marked token sits exactly one step inside / outside the window of the probing position, or at a page border; an
    off-by-one mask, or a missing sink, changes the logits by far more than the tolerance."""
    from llama_cpp.kv_pages import SequenceSlots
    window, n = 70, 200
    cfg, w, path = _peaky_latent_model(tmp_path, window)
    eng = open_engine(path, dtype)
    tol = TOL["float32"] if dtype == "float32" else 0.012        # one layer: bf16 rounding stays well under the edge's effect
    seqs = SequenceSlots(eng)
    mark = 7
    base = [int(t) for t in np.random.default_rng(9).integers(8, cfg["vocab"], size=n)]
    probe = n - 1
    cases = {"last_in_window": probe - window + 1, "first_outside_window": probe - window, "at_page_border": 191, "after_page_border": 192}
    for name, at in cases.items():
        toks = list(base)
        toks[at] = mark
        toks[probe] = mark
        true = ref.forward(cfg, w, toks)[probe]
        other = None
        if name in ("last_in_window", "first_outside_window"):
            other = ref.forward(_with_window(cfg, window + (1 if "outside" in name else -1)), w, toks)[probe]
        seqs.open(name)
        if decode:
            slot = seqs.extend(name, probe - 20)
            eng.step([(slot, toks[:probe - 20])])
            for t in range(probe - 20, probe):
                eng.step([(seqs.extend(name, 1), [toks[t]])])
            got, _ = eng.step([(seqs.extend(name, 1), [toks[probe]])], want=[[0]])
        else:
            slot = seqs.extend(name, n)
            got, _ = eng.step([(slot, toks)], want=[[probe]])
        seqs.close(name)
        err = vu.rel_err(got[0], true)
        assert err < tol, (name, err)
        if other is not None:
            assert vu.rel_err(other, true) > 0.02, f"{name}: the test model does not show the edge"
    no_sink = dict(w)
    no_sink["l0.mix.sink"] = np.full(2, -40.0)
    assert vu.rel_err(ref.forward(cfg, no_sink, base)[probe], ref.forward(cfg, w, base)[probe]) > 0.02, "the test model does not show the sink"
    eng.close()


@pytest.mark.parametrize("kind", ["delta", "ssd"])
def test_far_token_through_the_recurrent_state(native_lib, tmp_path, kind):
    """A token 600 positions back reaches the last logits only through the matrix state (slow decays). Delta rule: later
    writes erase what the memory holds along THEIR keys, so the filler draws from three token ids (with a one-tap key
    convolution: three key directions) and the far token's write survives beside them. State-space layer: the step size
    answers to the far token's direction, so its write is far stronger than the others'. The prompt is cut at odd places."""
    from llama_cpp.kv_pages import SequenceSlots
    layer = vu.delta(heads=2, kv_heads=1, dim=24, vdim=16) if kind == "delta" else vu.ssd(heads=2, groups=1, vdim=16, state=24, norm_groups=1)
    cfg = vu.config([layer], width=48)
    w = vu.random_weights(cfg, seed=6)
    w["l0.mix.A_log"] = vu.bf16_round(np.log(np.full_like(w["l0.mix.A_log"], 0.004)))
    n, mark = 600, 5
    rng = np.random.default_rng(12)
    if kind == "delta":
        taps = np.zeros((24, 3))
        taps[:, -1] = 1.0
        w["l0.mix.k.conv"] = vu.bf16_round(taps)
        toks = [int(t) for t in rng.integers(8, 11, size=n)]
    else:
        wd = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
        h = ref.zero_centred_norm(ref.zero_centred_norm(wd["embed"][mark], wd["embed.norm"], 1e-6), wd["l0.norm1"], 1e-6)
        win = w["l0.mix.in"].copy()
        win[-2:] = 8.0 * h / (h @ h)
        w["l0.mix.in"] = vu.bf16_round(win)
        w["l0.mix.dt_bias"] = vu.bf16_round(np.full(2, -5.0))
        toks = [int(t) for t in rng.integers(8, cfg["vocab"], size=n)]
    path = vu.write_model(str(tmp_path / "far"), cfg, w)
    toks[1] = mark
    changed = list(toks)
    changed[1] = mark + 1
    true = ref.forward(cfg, w, toks)[n - 1]
    assert vu.rel_err(ref.forward(cfg, w, changed)[n - 1], true) > 0.02, "the test model forgets the far token"
    eng = open_engine(path, "float32", n_ctx=640)
    got = run_cut(eng, SequenceSlots(eng), "far", toks, [257, 64, 1, 2])
    eng.close()
    assert vu.rel_err(got[n - 1], true) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [16, 64, 100, 1000])
def test_prompt_tiles(native_lib, tmp_path, window, dtype):
    """Sizes the tensor-core prompt kernels take: latents wider than 128 and than one 256-column output chunk, windows narrower and wider
    than the 64-query tile, enough (token, expert) pairs for 128-row expert tiles; a 300-token prompt at once and in portions
    that straddle the tiles."""
    from llama_cpp.kv_pages import SequenceSlots
    mlp = vu.moe(experts=6, identity=0, top=4, ff=16, groups=(2, 2))
    cfg = vu.config([vu.latent(mlp=mlp, heads=4, dim=16, rot_dim=16, vdim=32, rank=144, window=window),
                     vu.latent(mlp=None, heads=2, dim=48, rot_dim=32, vdim=16, rank=272, window=window), vu.delta(mlp=mlp, dim=16, vdim=16)], width=64)
    w = vu.random_weights(cfg, seed=13, ranks=(8, 16))
    eng = open_engine(vu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 300, 14)
    want = ref.forward(cfg, w, toks)
    seqs = SequenceSlots(eng)
    whole = run_cut(eng, seqs, "w", toks, [300])
    parts = run_cut(eng, seqs, "p", toks, [100, 7, 64, 129])
    eng.close()
    assert close(whole, want, dtype)
    assert close(parts, want, dtype)


def test_steps_larger_than_the_engine_takes_at_once(hybrid):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32", max_step_tokens=16)
    seqs = SequenceSlots(eng)
    reqs = {"a": tokens_for(cfg, 50, 70), "b": tokens_for(cfg, 3, 71), "c": tokens_for(cfg, 37, 72)}
    for k in reqs:
        seqs.open(k)
    entries = [(seqs.extend(k, len(t)), t) for k, t in reqs.items()]
    want = [[0, 17, 49], [2], list(range(37))]
    got, _ = eng.step(entries, want=want)
    eng.close()
    expect = np.concatenate([ref.forward(cfg, w, t)[wi] for t, wi in zip(reqs.values(), want)])
    assert got.shape == expect.shape and vu.rel_err(got, expect) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_equal_direct_launches(hybrid, dtype):
    """Repeating small steps are replayed as CUDA graphs; the logits are bit-identical to launching the kernels directly."""
    from llama_cpp import _cabi
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    toks = {"a": tokens_for(cfg, 40, 80), "b": tokens_for(cfg, 30, 81)}
    outs = []
    for flags in (0, _cabi.B2_FLAG_NO_GRAPH):
        eng = open_engine(path, dtype, n_ctx=256, max_seqs=2, flags=flags)
        seqs = SequenceSlots(eng)
        rows = []
        for k, t in toks.items():
            seqs.open(k)
            eng.step([(seqs.extend(k, 5), t[:5])])
        for i in range(5, 30):
            lg, _ = eng.step([(seqs.extend(k, 1), [t[i]]) for k, t in toks.items()], want=[[0], [0]])
            rows.append(lg)
        eng.close()
        outs.append(np.concatenate(rows))
    assert np.array_equal(outs[0], outs[1])
    want = np.concatenate([np.stack([ref.forward(cfg, w, t)[i] for t in toks.values()]) for i in range(5, 30)])
    assert close(outs[0], want, dtype)


def test_first_tokens(hybrid):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32")
    seqs = SequenceSlots(eng)
    for n in (1, 2, 3, 5):
        toks = tokens_for(cfg, n, 30 + n)
        want = ref.forward(cfg, w, toks)
        assert vu.rel_err(run_cut(eng, seqs, f"w{n}", toks, [n]), want) < TOL["float32"]
        assert vu.rel_err(run_cut(eng, seqs, f"s{n}", toks, [1]), want) < TOL["float32"]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(hybrid, dtype):
    """A short prompt and 300 single-token steps: the windows slide over decoded tokens and over page borders."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    toks = tokens_for(cfg, 310, 40)
    got = run_cut(eng, SequenceSlots(eng), "d", toks, [10] + [1] * 300)
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_one_odd_or_large(native_lib, tmp_path, dtype):
    """One head, one expert, one choice, one group, one tap, one state, a window of one token, no identity slot, no
    feed-forward, residual and logit scale 1, rotation over part of the rotated entries; odd sizes that no vector path
    takes; keys wider than 160 and 320 entries, memories with more than 128 rows, more row groups than a warp has lanes."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = vu.config([
        vu.latent(mlp=vu.moe(experts=1, identity=0, top=1, ff=8, groups=None), heads=1, dim=8, rot_dim=2, vdim=8, rank=8, window=1),
        vu.delta(mlp=None, heads=1, kv_heads=1, dim=1, vdim=1, conv=1),
        vu.ssd(mlp=vu.moe(experts=2, identity=1, top=3, ff=9, groups=(1, 1)), heads=1, groups=1, vdim=1, state=1, norm_groups=1, conv=1),
        vu.latent(mlp=None, heads=5, dim=13, rot_dim=10, vdim=7, rank=171, window=500, rot_dims=6),
        vu.latent(mlp=None, heads=2, dim=24, rot_dim=16, vdim=24, rank=330, window=37),
        vu.delta(mlp=vu.moe(experts=33, identity=3, top=5, ff=11, groups=(4, 2)), heads=6, kv_heads=2, dim=37, vdim=45, conv=5),
        vu.delta(mlp=None, heads=2, kv_heads=2, dim=150, vdim=20, conv=2),
        vu.ssd(mlp=None, heads=3, groups=1, vdim=33, state=131, norm_groups=3, conv=2),
    ], width=40, vocab=50, mult=1.0, eps=1e-5, logit_scale=1.0)
    w = vu.random_weights(cfg, seed=8, ranks=(1, 3))
    eng = open_engine(vu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 100, 3)
    got = run_cut(eng, SequenceSlots(eng), "x", toks, [5, 1, 2, 30])
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [45, 50])
def test_widths_no_vector_path_takes(native_lib, tmp_path, width, dtype):
    """A model width that is odd, or even but no multiple of four: every product over the width takes its scalar path, in
    prompts (tiles) and in few-token steps (rows); no mask entry (full causal attention); full attention over page borders."""
    from llama_cpp.kv_pages import SequenceSlots
    la = vu.latent(mlp=vu.moe(experts=4, identity=1, top=2, ff=10, groups=None), heads=2, dim=12, rot_dim=4, vdim=10, rank=18)
    del la["mixer"]["mask"]
    cfg = vu.config([la, vu.delta(mlp=vu.moe(ff=7)), vu.ssd(mlp=vu.moe(experts=2, identity=0, top=1, groups=None, ff=12))], width=width, vocab=77)
    w = vu.random_weights(cfg, seed=21, ranks=(3, 9))
    eng = open_engine(vu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 150, 22)
    got = run_cut(eng, SequenceSlots(eng), "x", toks, [70, 1, 3, 20, 1])
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


def random_config(seed):
    """A random model: layer count and order, every size and constant drawn anew (sizes of the scale small real models have)."""
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(0, len(xs)))]

    def mixture():
        if rng.random() < 0.15:
            return None
        count = pick(1, 2, 3, 4)
        per = pick(2, 3, 4, 6)
        identity = pick(0, 0, 1, 2, 3)
        identity = min(identity, count * per - 1)
        keep = int(rng.integers(1, count + 1))
        top = int(rng.integers(1, min(keep * per, 6) + 1))
        return vu.moe(experts=count * per - identity, identity=identity, top=top, ff=pick(8, 24, 40, 64, 72),
                      groups=None if count == 1 and rng.random() < 0.5 else (count, keep), scale=float(rng.uniform(0.5, 2.5)))

    layers = []
    for _ in range(int(rng.integers(2, 6))):
        kind = pick("latent", "delta", "ssd")
        if kind == "latent":
            rot_dim = pick(4, 8, 16, 32)
            layers.append(vu.latent(mlp=mixture(), heads=pick(1, 2, 4, 5, 8), dim=pick(16, 32, 48, 64, 96), rot_dim=rot_dim, vdim=pick(16, 32, 48, 80),
                                    rank=pick(32, 64, 96, 160, 192, 272), window=pick(1, 7, 24, 40, 64, 65, 100, 129, 300),
                                    base=pick(1e4, 5e5, 1e6), rot_dims=pick(rot_dim, rot_dim, rot_dim // 2)))
        elif kind == "delta":
            g = pick(1, 2, 3, 4)
            layers.append(vu.delta(mlp=mixture(), heads=g * pick(1, 1, 2), kv_heads=g, dim=pick(16, 32, 48, 64, 96, 128), vdim=pick(16, 32, 48, 64, 100),
                                   conv=pick(2, 3, 4, 5)))
        else:
            g = pick(1, 1, 2)
            heads = g * pick(1, 2, 4, 5)
            vdim = pick(16, 32, 48, 64)
            parts = pick(1, 1, 2, heads)
            layers.append(vu.ssd(mlp=mixture(), heads=heads, groups=g, vdim=vdim, state=pick(16, 32, 48, 64, 128), norm_groups=parts, conv=pick(2, 3, 4)))
    cfg = vu.config(layers, width=pick(64, 96, 128, 192, 200, 320), vocab=pick(97, 256, 500), mult=float(rng.uniform(0.2, 1.0)),
                    eps=pick(1e-5, 1e-6), logit_scale=float(rng.uniform(0.5, 3.0)))
    return cfg, (pick(4, 8, 24, 32), pick(4, 8, 24, 32))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(native_lib, tmp_path, seed):
    """Eight models nobody chose: each runs a 330-token prompt at once and in uneven portions with decoded tokens at the end,
    in both modes, from a pool that forces page reuse."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, ranks = random_config(100 + seed)
    w = vu.random_weights(cfg, seed=seed, ranks=ranks)
    path = vu.write_model(str(tmp_path / "m"), cfg, w)
    toks = tokens_for(cfg, 330, seed)
    want = ref.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        eng = open_engine(path, dtype, n_ctx=384, max_seqs=2, kv_tokens=384 + 128)
        seqs = SequenceSlots(eng)
        whole = run_cut(eng, seqs, "w", toks, [330])
        parts = run_cut(eng, seqs, "p", toks, [61, 3, 128, 2, 70, 37] + [1] * 29)
        eng.close()
        assert close(whole, want, dtype), (seed, dtype, "whole")
        assert close(parts, want, dtype), (seed, dtype, "parts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(hybrid, tmp_path, dtype):
    """`bin/trace_run` as a user starts it: six requests, at most four live, portions of some beside single tokens of others, a
    request that sits out steps, a pool of --max-tokens sized for the live ones only, so pages and slots are used again; every
    written row against the oracle."""
    import json
    import os
    import subprocess
    import sys
    cfg, w, path = hybrid
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    reqs = {f"r{i}": tokens_for(cfg, n, 90 + i) for i, n in enumerate([130, 7, 64, 201, 33, 90])}
    plans = {"r0": [64, 2, 1, 1, 40, 1], "r1": [1, 1], "r2": [3, 61], "r3": [100, 1, 1, 64, 2], "r4": [33], "r5": [2, 1, 50, 1]}
    order, live, at, turn, steps, wanted = list(reqs), [], {k: 0 for k in reqs}, {k: 0 for k in reqs}, [], []
    most = 0
    while order or live:
        while order and len(live) < 4:
            live.append(order.pop(0))
        entries, end = [], []
        for k in list(live):
            if k == "r3" and len(steps) % 3 == 1:          # sits this step out
                continue
            n = min(plans[k][turn[k] % len(plans[k])], len(reqs[k]) - at[k])
            turn[k] += 1
            want = sorted({0, n - 1})
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": want})
            wanted.append((len(steps), k, [at[k] + x for x in want]))
            at[k] += n
        most = max(most, sum((at[k] + 63) // 64 * 64 for k in live))
        for k in list(live):
            if at[k] == len(reqs[k]):
                end.append(k)
                live.remove(k)
        steps.append({"step": len(steps), "entries": entries, "end": end})
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(most)], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.split("\n") if ln.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    refs = {k: ref.forward(cfg, w, t) for k, t in reqs.items()}
    for i in range(len(steps)):
        rows = [(k, pos) for st, k, ps in wanted if st == i for pos in ps]
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"])
        expect = np.stack([refs[k][pos] for k, pos in rows])
        assert close(got, expect, dtype) if len(rows) >= 20 else vu.rel_err(got, expect) < (TOL[dtype] if dtype == "float32" else 0.2), i


def test_greedy_generation_through_llama_and_the_scheduler(hybrid):
    """`Llama(model_path=<folder>)`: three callers at once, prompts of different lengths, greedy. Every generated token is
    the oracle's argmax for the sequence so far wherever the oracle's top-two margin is clear."""
    from llama_cpp import Llama
    cfg, w, path = hybrid
    llm = Llama(model_path=path, n_gpu_layers=-1, n_ctx=256, n_seq_max=3, verbose=False, dtype="float32")
    prompts = [tokens_for(cfg, n, 50 + n) for n in (9, 70, 33)]
    outs = [None] * len(prompts)

    def call(i):
        outs[i] = llm.create_completion(prompts[i], max_tokens=12, temperature=0.0, repeat_penalty=1.0)

    threads = [threading.Thread(target=call, args=(i,)) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    stats = llm._scheduler.stats
    llm.close()
    assert stats["max_batch"] >= 2
    for p, o in zip(prompts, outs):
        assert o["usage"]["completion_tokens"] == 12
        gen = [int(x[1:-1]) for x in o["choices"][0]["text"].replace("><", "> <").split()]
        logits = ref.forward(cfg, w, p + gen)
        for i, g in enumerate(gen):
            row = logits[len(p) + i - 1]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > 1e-3:
                assert int(np.argmax(row)) == g


def test_direct_eval_and_scores(hybrid):
    from llama_cpp import Llama
    cfg, w, path = hybrid
    llm = Llama(model_path=path, n_gpu_layers=-1, n_ctx=128, verbose=False, dtype="float32")
    toks = tokens_for(cfg, 40, 60)
    llm.eval(toks[:30])
    for t in toks[30:]:
        llm.eval([t])
    got = llm.scores[0]
    llm.close()
    assert vu.rel_err(got, ref.forward(cfg, w, toks)[-1]) < TOL["float32"]
