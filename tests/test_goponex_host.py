"""Host side of the Goponex family (no GPU): safetensors round trip, config.json -> layer descriptors, the registry,
sequence slots over a stand-in engine, and sanity of the float64 oracle's own mechanisms."""
import json
import os

import numpy as np
import pytest

import goponex_util as gu
from oracle import goponex_ref as ref


def test_safetensors_round_trip(tmp_path):
    from llama_cpp.safetensors_file import SafetensorsFile, write_safetensors
    rng = np.random.default_rng(0)
    a = gu.bf16_round(rng.standard_normal((5, 7)))
    b = rng.integers(0, 100, size=(9,)).astype(np.int32)
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": a, "b": b})
    f = SafetensorsFile(p)
    assert f.tensors["a"].dtype == "BF16" and f.tensors["a"].shape == (5, 7)
    assert np.array_equal(f.tensors["a"].to_float32(), a)
    assert f.tensors["b"].dtype == "I32" and np.array_equal(f.tensors["b"].data, b)
    f.close()
    with open(p, "r+b") as fh:
        fh.write(b"\xff" * 8)
    with pytest.raises(ValueError):
        SafetensorsFile(p)


def test_bf16_rounding_is_to_nearest_even():
    from llama_cpp.safetensors_file import float32_to_bf16_bits
    x = np.array([1.0, 1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8, -2.5], dtype=np.float32)
    assert list(float32_to_bf16_bits(x)) == [0x3F80, 0x3F80, 0x3F82, 0xC020]


def test_config_to_layer_descriptors():
    from llama_cpp import _cabi, goponex
    cfg = gu.config([gu.parallel(mlp=80), gu.mlstm()], width=72, vocab=131, alpha=1.5, eps=1e-6)
    d = goponex.read_dims(cfg)
    assert (d.n_layer, d.n_embd, d.n_vocab, d.residual_scale) == (2, 72, 131, 1.5)
    a, m = d.layers
    assert a.mixer == _cabi.B2_MIX_WINDOW_SCAN and a.n_ff == 80
    assert (a.n_head, a.n_head_kv, a.head_dim, a.rot_dims, a.window, a.keep_first) == (4, 2, 24, 8, 16, 3)
    assert (a.rope_factor, a.rope_orig_ctx, a.rope_fast, a.rope_slow, a.rope_base) == (4.0, 64, 16.0, 2.0, 5000.0)
    assert (a.conv_taps, a.dt_rank, a.d_inner, a.d_state) == (3, 5, 40, 12)
    assert m.mixer == _cabi.B2_MIX_MATRIX_MEMORY and m.n_ff == 0
    assert (m.mm_heads, m.mm_dim, m.mm_vdim, m.gate_cap) == (3, 20, 28, 12.0)
    shapes = goponex.tensor_shapes(cfg)
    assert shapes["l0.mix.left.k"] == (48, 72) and shapes["l0.mix.right.x"] == (5 + 24, 40) and shapes["l1.mix.i"] == (3, 72)
    assert "l1.norm2" not in shapes and shapes["l0.mlp.down"] == (72, 80)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError, match="unknown layer type"):
        goponex.read_dims(bad)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["mixer"]["left"]["vdim"] = 8
    with pytest.raises(ValueError, match="vdim"):
        goponex.read_dims(bad)


def test_registry_picks_the_family(tmp_path):
    from llama_cpp import models
    cfg = gu.config([gu.mlstm()])
    path = gu.write_model(str(tmp_path / "m"), cfg, gu.random_weights(cfg))
    src = models.open_model(path)
    assert src.family.name == "Goponex" and src.family.source == "folder" and "embed" in src.weights.tensors
    assert {"Goponex", "llama"} <= set(models.architectures())
    cfg["architecture"] = "Nothing"
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    with pytest.raises(ValueError, match="unsupported architecture"):
        models.open_model(path)


class _StubEngine:
    max_seqs = 2

    def __init__(self):
        from llama_cpp.kv_pages import PageAllocator
        self.pages = PageAllocator(4, 64)
        self.begun = []

    def seq_begin(self, slot, n_past, hist, sampling, uniforms=None):
        self.begun.append((slot, n_past))

    def ensure_pages(self, slot, n):
        self.pages.ensure(slot, n)

    def release(self, slot):
        self.pages.release(slot)


def test_sequence_slots_hand_out_and_take_back():
    from llama_cpp.kv_pages import OutOfPages, SequenceSlots
    eng = _StubEngine()
    s = SequenceSlots(eng)
    a = s.open("a")
    b = s.open("b")
    assert {a, b} == {0, 1} and s.free_slots == 0
    with pytest.raises(RuntimeError):
        s.open("c")
    s.extend("a", 65)
    assert eng.pages.free_pages == 2 and s.length("a") == 65
    s.extend("b", 128)
    with pytest.raises(OutOfPages):
        s.extend("a", 64)
    s.close("b")
    assert eng.pages.free_pages == 2 and s.free_slots == 1
    c = s.open("c")
    assert c == b and eng.begun[-1] == (b, 0)          # the slot is used again, from position 0
    s.close("a")
    s.close("c")
    assert eng.pages.free_pages == 4


def test_oracle_mask_and_rotary():
    # window 3, keep 1: position 5 sees 0 (kept) and 3, 4, 5
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "rot": {"base": 100.0, "dims": 4}, "mask": {"size": 3, "keep_first": 1}, "scale": 1.0}
    rng = np.random.default_rng(0)
    w = {"q": rng.standard_normal((4, 6)), "k": rng.standard_normal((4, 6)), "q.norm": np.ones(4), "k.norm": np.ones(4), "o": np.eye(4)}
    h = rng.standard_normal((6, 6))
    full = ref.window_attention(h, w, "", m, 1e-6)
    h2 = h.copy()
    h2[1] += 5.0            # invisible to position 5
    h2[2] -= 3.0
    assert np.allclose(ref.window_attention(h2, w, "", m, 1e-6)[5], full[5])
    h3 = h.copy()
    h3[0] += 1.0            # kept: visible
    assert not np.allclose(ref.window_attention(h3, w, "", m, 1e-6)[5], full[5])
    cos, sin = ref.rotary_tables({"base": 100.0, "dims": 4}, [0, 1, 2])
    assert np.allclose(cos[1], [np.cos(1.0), np.cos(0.1)]) and np.allclose(sin[2], [np.sin(2.0), np.sin(0.2)])
    x = np.arange(8, dtype=float).reshape(1, 1, 8)
    r = ref.rotate_interleaved(np.repeat(x, 3, 0), cos, sin, 4)
    assert np.allclose(r[0], x[0]) and np.allclose(r[1, 0, 4:], x[0, 0, 4:])
    assert np.isclose(r[1, 0, 0], 0 * np.cos(1.0) - 1 * np.sin(1.0)) and np.isclose(r[1, 0, 1], 1 * np.cos(1.0) + 0 * np.sin(1.0))


def test_oracle_recurrences_do_not_look_ahead():
    cfg = gu.config([gu.parallel(mlp=40), gu.mlstm(mlp=None)])
    w = gu.random_weights(cfg, seed=2)
    toks = [int(t) for t in np.random.default_rng(1).integers(0, cfg["vocab"], size=30)]
    a = ref.forward(cfg, w, toks)
    b = ref.forward(cfg, w, toks[:20])
    assert np.allclose(a[:20], b, atol=1e-9)
