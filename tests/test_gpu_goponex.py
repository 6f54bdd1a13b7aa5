"""Goponex through the native engine against the float64 oracle (oracle/goponex_ref.py), on small random models the
tests make themselves: each mixer alone, prompt against token-by-token decoding, portions down to two tokens, unequal
batches against each request alone, slots and pages used again, keys just inside and just outside the window and the
kept prefix, the first tokens, long decoding, degenerate sizes, and greedy generation through `Llama` and the scheduler."""
import threading

import numpy as np
import pytest

import goponex_util as gu
from oracle import goponex_ref as ref

pytestmark = pytest.mark.gpu

TOL = {"float32": 3e-4, "bfloat16": 6e-2}


def open_engine(path, dtype="float32", n_ctx=512, max_seqs=4, kv_tokens=None, max_step_tokens=None):
    from llama_cpp import models
    return models.open_engine(models.open_model(path), n_ctx=n_ctx, max_seqs=max_seqs, dtype=dtype, kv_tokens=kv_tokens,
                              max_step_tokens=max_step_tokens)


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


@pytest.fixture(scope="module")
def hybrid(native_lib, tmp_path_factory):
    cfg = gu.config([gu.parallel(mlp=None), gu.mlstm(mlp=96), gu.parallel(mlp=80, right=gu.scan(inner=36, state=24, dt_rank=4, conv=4)),
                     gu.mlstm(mlp=None)])
    w = gu.random_weights(cfg, seed=3)
    path = gu.write_model(str(tmp_path_factory.mktemp("goponex_hybrid")), cfg, w)
    return cfg, w, path


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", ["parallel", "parallel_mlp", "mlstm", "mlstm_mlp"])
def test_each_mixer_alone(native_lib, tmp_path, layer, dtype):
    from llama_cpp.kv_pages import SequenceSlots
    L = {"parallel": gu.parallel(), "parallel_mlp": gu.parallel(mlp=100, right=gu.scan(inner=24, state=40, dt_rank=3, conv=2)), "mlstm": gu.mlstm(), "mlstm_mlp": gu.mlstm(mlp=64)}[layer]
    cfg = gu.config([L])
    w = gu.random_weights(cfg, seed=11)
    eng = open_engine(gu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 90, 1)
    want_logits, want_layers = ref.forward(cfg, w, toks, return_layers=True)
    seqs = SequenceSlots(eng)
    eng.trace_layers(True)
    seqs.open("a")
    slot = seqs.extend("a", len(toks))
    got, _ = eng.step([(slot, toks)], want=[list(range(len(toks)))])
    layers = eng.layer_outputs(len(toks))
    eng.close()
    assert np.abs(layers[0] - want_layers[0]).max() < (2e-4 if dtype == "float32" else 8e-2)
    assert gu.rel_err(got, want_logits) < TOL[dtype]


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
    assert gu.rel_err(whole, want) < TOL[dtype]
    assert gu.rel_err(single, want) < TOL[dtype]
    assert gu.rel_err(single, whole) < TOL[dtype]


@pytest.mark.parametrize("cuts", [[2], [3, 2, 5, 1], [17, 64, 2, 9], [63, 1, 1, 70]])
def test_portions(hybrid, cuts):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32")
    toks = tokens_for(cfg, 140, 4)
    got = run_cut(eng, SequenceSlots(eng), "p", toks, cuts)
    eng.close()
    assert gu.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"]


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
        assert gu.rel_err(mixed, alone[k]) < (2e-5 if dtype == "float32" else TOL[dtype])
        assert gu.rel_err(mixed, ref.forward(cfg, w, t)) < TOL[dtype]


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
        assert gu.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"], i
    eng.close()


def _peaky_attention_model(tmp_path, window, keep):
    """One attention+scan layer in which a token attends to earlier copies of itself whenever the mask lets it: the query
    and key maps are the same matrix (a copy scores as high as the token itself, far above the random rest), only two
    dimensions rotate, and the score scale is low enough that the token's own key does not take all the weight."""
    cfg = gu.config([gu.parallel(left=gu.attn(heads=2, kv_heads=2, dim=32, rot=2, window=window, keep=keep, scale=0.15))], width=64)
    w = gu.random_weights(cfg, seed=5)
    w["l0.mix.left.k"] = w["l0.mix.left.q"].copy()
    w["l0.mix.left.k.norm"] = w["l0.mix.left.q.norm"].copy()
    return cfg, w, gu.write_model(str(tmp_path / "peaky"), cfg, w)


def _variant(cfg, size=None, keep=None):
    import copy
    c = copy.deepcopy(cfg)
    m = c["layers"][0]["mixer"]["left"]["mask"]
    if size is not None:
        m["size"] = size
    if keep is not None:
        m["keep_first"] = keep
    return c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_window_and_kept_prefix_edges(native_lib, tmp_path, decode, dtype):
    """The marked token sits exactly one step inside / outside the window, and inside / just after the kept prefix, of the
    probing position; an off-by-one mask changes the logits by far more than the tolerance."""
    from llama_cpp.kv_pages import SequenceSlots
    window, keep, n = 70, 4, 200
    cfg, w, path = _peaky_attention_model(tmp_path, window, keep)
    eng = open_engine(path, dtype)
    tol = TOL["float32"] if dtype == "float32" else 0.012        # one layer: bf16 rounding stays well under the edge's effect
    seqs = SequenceSlots(eng)
    mark = 7
    base = [int(t) for t in np.random.default_rng(9).integers(8, cfg["vocab"], size=n)]
    probe = n - 1
    cases = {"last_in_window": probe - window + 1, "first_outside_window": probe - window,
             "last_kept": keep - 1, "first_not_kept": keep, "at_page_border": 127, "after_page_border": 128}
    for name, at in cases.items():
        toks = list(base)
        toks[at] = mark
        toks[probe] = mark
        true = ref.forward(cfg, w, toks)[probe]
        if name in ("last_in_window", "first_outside_window"):
            other = ref.forward(_variant(cfg, size=window + (1 if "outside" in name else -1)), w, toks)[probe]
        elif name in ("last_kept", "first_not_kept"):
            other = ref.forward(_variant(cfg, keep=keep + (1 if "not" in name else -1)), w, toks)[probe]
        else:
            other = None
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
        err = gu.rel_err(got[0], true)
        assert err < tol, (name, err)
        if other is not None:
            assert gu.rel_err(other, true) > 0.02, f"{name}: the test model does not show the edge"
    eng.close()


def test_far_token_reaches_through_the_kept_prefix_and_the_state(native_lib, tmp_path):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = _peaky_attention_model(tmp_path, 32, 3)
    eng = open_engine(path, "float32", n_ctx=640)
    n, mark = 600, 5
    toks = [int(t) for t in np.random.default_rng(12).integers(8, cfg["vocab"], size=n)]
    toks[1] = mark
    toks[n - 1] = mark
    true = ref.forward(cfg, w, toks)[n - 1]
    assert gu.rel_err(ref.forward(_variant(cfg, keep=1), w, toks)[n - 1], true) > 0.005
    seqs = SequenceSlots(eng)
    got = run_cut(eng, seqs, "far", toks, [257, 64, 1])
    eng.close()
    assert gu.rel_err(got[n - 1], true) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep", [(16, 3), (64, 0), (20, 70), (100, 64), (1000, 5), (65, 129)])
def test_prompt_attention_tiles(native_lib, tmp_path, window, keep, dtype):
    """Grouped heads with a head size the tensor-core prompt kernel takes: windows narrower and wider than its 64-query tile,
    kept prefixes of no, one and several key blocks, a 300-token prompt at once and in portions that straddle the tiles."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = gu.config([gu.parallel(mlp=48, left=gu.attn(heads=4, kv_heads=2, dim=32, rot=16, window=window, keep=keep)),
                     gu.parallel(left=gu.attn(heads=6, kv_heads=2, dim=48, rot=48, window=window, keep=keep, scaling=False))], width=64)
    w = gu.random_weights(cfg, seed=13)
    eng = open_engine(gu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 300, 14)
    want = ref.forward(cfg, w, toks)
    seqs = SequenceSlots(eng)
    whole = run_cut(eng, seqs, "w", toks, [300])
    parts = run_cut(eng, seqs, "p", toks, [100, 7, 64, 129])
    eng.close()
    assert gu.rel_err(whole, want) < TOL[dtype]
    assert gu.rel_err(parts, want) < TOL[dtype]


def test_steps_larger_than_the_engine_takes_at_once(hybrid):
    """A batch above `max_step_tokens` runs as several native steps that cut the entries where needed."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32", max_step_tokens=16)
    seqs = SequenceSlots(eng)
    reqs = {"a": tokens_for(cfg, 50, 70), "b": tokens_for(cfg, 3, 71), "c": tokens_for(cfg, 37, 72)}
    for k in reqs:
        seqs.open(k)
    entries = [(seqs.extend(k, len(t)), t) for k, t in reqs.items()]
    want = [[0, 17, 49], [2], list(range(37))]
    got, sampled = eng.step(entries, want=want, sample=[True, False, True])
    eng.close()
    refs = [ref.forward(cfg, w, t) for t in reqs.values()]
    expect = np.concatenate([r[wi] for r, wi in zip(refs, want)])
    assert got.shape == expect.shape and gu.rel_err(got, expect) < TOL["float32"]
    assert sampled[1] is None
    for s, r in ((sampled[0], refs[0]), (sampled[2], refs[2])):
        top = np.sort(r[-1])[-2:]
        assert top[1] - top[0] < 1e-3 or s == int(np.argmax(r[-1]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_equal_direct_launches(hybrid, dtype):
    """Repeating small steps are replayed as CUDA graphs; the logits are bit-identical to launching the kernels directly."""
    from llama_cpp import _cabi, models
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    toks = {"a": tokens_for(cfg, 60, 80), "b": tokens_for(cfg, 45, 81)}
    outs = []
    for flags in (0, _cabi.B2_FLAG_NO_GRAPH):
        eng = models.open_engine(models.open_model(path), n_ctx=256, max_seqs=2, dtype=dtype, flags=flags)
        assert eng.mode()["graph"] == (flags == 0)
        seqs = SequenceSlots(eng)
        rows = []
        for k, t in toks.items():
            seqs.open(k)
            eng.step([(seqs.extend(k, 5), t[:5])])
        for i in range(5, 45):
            lg, _ = eng.step([(seqs.extend(k, 1), [t[i]]) for k, t in toks.items()], want=[[0], [0]])
            rows.append(lg)
        for i in range(45, 60):          # one sequence has ended: another shape
            lg, _ = eng.step([(seqs.extend("a", 1), [toks["a"][i]])], want=[[0]])
            rows.append(lg)
        eng.close()
        outs.append(np.concatenate(rows))
    assert np.array_equal(outs[0], outs[1])
    want = np.concatenate([np.stack([ref.forward(cfg, w, t)[i] for t in toks.values()]) for i in range(5, 45)] +
                          [ref.forward(cfg, w, toks["a"])[45:60]])
    assert gu.rel_err(outs[0], want) < TOL[dtype]


def test_first_tokens(hybrid):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32")
    seqs = SequenceSlots(eng)
    for n in (1, 2, 3, 5):
        toks = tokens_for(cfg, n, 30 + n)
        want = ref.forward(cfg, w, toks)
        assert gu.rel_err(run_cut(eng, seqs, f"w{n}", toks, [n]), want) < TOL["float32"]
        assert gu.rel_err(run_cut(eng, seqs, f"s{n}", toks, [1]), want) < TOL["float32"]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(hybrid, dtype):
    """A short prompt and 300 single-token steps: the window slides over decoded tokens and over three page borders."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    toks = tokens_for(cfg, 310, 40)
    got = run_cut(eng, SequenceSlots(eng), "d", toks, [10] + [1] * 300)
    eng.close()
    assert gu.rel_err(got, ref.forward(cfg, w, toks)) < TOL[dtype]


def test_sizes_that_are_one_or_equal(native_lib, tmp_path):
    """One head, one state, one convolution tap, a window of one token, no kept prefix, full-width rotary without frequency
    scaling, head sizes that are equal where the other tests have them differ, an odd head size, a state wider than a
    warp, residual scale 1."""
    from llama_cpp.kv_pages import SequenceSlots
    left = gu.attn(heads=1, kv_heads=1, dim=16, rot=16, window=1, keep=0, scaling=False)
    cfg = gu.config([gu.mlstm(mlp=32, heads=1, dim=16, vdim=16, cap=30.0),
                     gu.parallel(mlp=32, left=left, right=gu.scan(inner=8, state=1, dt_rank=1, conv=1)),
                     gu.parallel(mlp=None, left=gu.attn(heads=6, kv_heads=1, dim=41, rot=2, window=500, keep=600),
                                 right=gu.scan(inner=33, state=70, dt_rank=7, conv=6))],
                    width=48, vocab=50, alpha=1.0, eps=1e-5)
    w = gu.random_weights(cfg, seed=8)
    eng = open_engine(gu.write_model(str(tmp_path / "m"), cfg, w), "float32")
    toks = tokens_for(cfg, 100, 3)
    got = run_cut(eng, SequenceSlots(eng), "x", toks, [5, 1, 2, 30])
    eng.close()
    assert gu.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"]


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
    assert gu.rel_err(got, ref.forward(cfg, w, toks)[-1]) < TOL["float32"]
