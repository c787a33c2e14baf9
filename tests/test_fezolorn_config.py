"""The Fezolorn configuration, its tensor list, what its parts ask of the cache (a branch that itself
asks for two things: tuples inside a tuple), the frequency table with stretched bands, and the plain
implementation's mechanisms against closed forms (no device needed)."""
import copy
import math

import numpy as np
import pytest
import torch

import torchless_rs_b200 as tl
from fezolorn_tiny import CONFIGS, random_config, tensor_shapes
from plain import fezolorn_plain as plain
from torchless_rs_b200.cache import Cache, PAGE, PagedKVRequest, StateRequest
from torchless_rs_b200.cache.requests import PagedLatentRequest
from torchless_rs_b200.config import ConfigError
from torchless_rs_b200.engine.model import expected_tensors
from torchless_rs_b200.parts.position import RotaryHalfSplit

ALL = {**CONFIGS, **{f"seed{s}": random_config(s) for s in range(1, 9)}}


@pytest.mark.parametrize("name", sorted(ALL))
def test_keys_are_read_and_written_back(name):
    raw = ALL[name]
    cfg = tl.config_from_dict(raw)
    assert type(cfg).__name__ == "FezolornConfig"
    assert tl.config_from_dict(cfg.to_dict()) == cfg
    assert (cfg.width, cfg.vocab, cfg.eps) == (raw["width"], raw["vocab"], raw["norm"]["eps"])
    for layer, entry in zip(cfg.layers, raw["layers"]):
        m, got = entry["mixer"], layer.mixer
        assert got.type == entry["type"]
        if entry["type"] == "parallel":
            a, b = m["left"], m["right"]
            l, r = got.left, got.right
            assert (l.heads, l.kv_heads, l.dim, l.vdim, l.scale) == (a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"])
            assert l.window == (a.get("mask") or {}).get("size")
            assert (l.rot.dims if l.rot else 0) == (a.get("rot") or {}).get("dims", 0)
            if l.rot and a["rot"].get("scaling"):
                assert l.rot.scaling == tuple(a["rot"]["scaling"][k] for k in ("factor", "low", "high", "original"))
            assert (r.heads, r.kv_heads, r.dim, r.vdim, r.conv) == (b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"])
            assert (got.left_scale, got.right_scale) == (m["left_scale"], m["right_scale"])
        elif entry["type"] == "lightning":
            assert (got.heads, got.dim, got.vdim, list(got.decay)) == (m["heads"], m["dim"], m["vdim"], m["decay"])
        else:
            assert (got.heads, got.dim, got.rot_dim, got.vdim, got.q_rank, got.kv_rank, got.scale) == \
                (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"], m["scale"])
        assert (layer.mlp is None) == (entry["mlp"] is None)
        if layer.mlp is not None:
            assert layer.mlp.ff == entry["mlp"]["ff"]


def test_errors_name_the_key():
    base = CONFIGS["P"]
    for change, word in ((lambda c: c["layers"][0].__setitem__("type", "serial"), "type"),
                         (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
                         (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
                         (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
                         (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("vdim", 8), "vdim"),
                         (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "dims"),
                         (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 18), "dims"),
                         (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("factor"), "factor"),
                         (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
                         (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("conv", 0), "conv"),
                         (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("kv_heads", 3), "kv_heads"),
                         (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.5]), "decay"),
                         (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
                         (lambda c: c.pop("width"), "width")):
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError) as e:
            tl.config_from_dict(c)
        assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(ALL))
def test_the_model_asks_for_the_designs_tensors(name):
    exp = expected_tensors(tl.config_from_dict(ALL[name]).model_spec())
    want = tensor_shapes(ALL[name])
    got = {n: tuple(s.shape) for n, s in exp.items() if not s.optional}
    assert got == want
    # a layer without a feed-forward accepts the second norm it does not use
    optional = {n for n, s in exp.items() if s.optional}
    assert optional == {f"l{i}.norm2" for i, l in enumerate(ALL[name]["layers"]) if l["mlp"] is None}


def test_parts_and_what_they_ask_of_the_cache():
    spec = tl.config_from_dict(CONFIGS["P"]).model_spec()
    assert spec.tie_head_to_embedding and spec.final_norm.kind == "rmsnorm" and spec.streams is None
    kinds = [(l.block.kind, l.mixer.kind, l.feed_forward.kind) for l in spec.layers]
    assert kinds == [("prenorm", "parallel", "swiglu"), ("prenorm", "lightning_attention", "swiglu"),
                     ("prenorm_mixer_only", "latent_attention", "none"), ("prenorm_mixer_only", "parallel", "none")]
    par = spec.layers[0].mixer
    assert par.params["combine"] == "weighted_sum" and par.params["scales"] == (0.7, 1.3)
    assert [(n, ps.kind) for n, ps in par.params["branches"]] == [("left", "sink_rotary_attention"), ("right", "gated_delta_rule")]
    lp = dict(par.params["branches"])["left"].params
    assert lp["values_are_keys"] and lp["sink"] and lp["bias"] and lp["unit_norm"] and lp["window"] == 20 and lp["rot_dims"] == 8
    assert spec.layers[0].position.kind == "rope_interleaved" and spec.layers[0].position.params["scaling"]["factor"] == 4.0
    assert spec.layers[1].position is None
    lat = spec.layers[2].mixer.params
    assert lat["sink"] and not lat["gate"] and lat["window"] is None and spec.layers[2].position.kind == "rope_interleaved"


def test_a_branch_that_asks_for_two_things_inside_a_mixer_that_asks_for_two():
    """The parallel mixer's request is (pages of the attention, (matrix state, kept convolution inputs)): a
    tuple inside a tuple, whose views come back in the same shape; equal requests of two layers share a group
    and not their storage."""
    kv = PagedKVRequest(2, 16, 20, v_head_dim=16)
    delta = (StateRequest((4, 16, 8)), StateRequest((3, 96)))
    other = (StateRequest((2, 40, 12)), StateRequest((1, 104)))
    reqs = [(kv, delta), StateRequest((3, 16, 24)), PagedLatentRequest(52, None), (PagedKVRequest(1, 24, 70, v_head_dim=24), other),
            (kv, delta), None]
    c = Cache(reqs, max_tokens=4 * PAGE, max_slots=3, dtype=torch.float32, device="cpu")
    pages, (state, kept) = c.view(0)
    assert tuple(pages.k_pages.shape) == (4, 2, PAGE, 16) and pages.window == 20
    assert tuple(state.shape) == (3, 4, 16, 8) and tuple(kept.shape) == (3, 3, 96)
    pages2, (state2, kept2) = c.view(4)
    assert state2.shape == state.shape and state2.data_ptr() != state.data_ptr() and kept2.data_ptr() != kept.data_ptr()
    assert pages2.group is pages.group
    assert tuple(c.view(1).shape) == (3, 3, 16, 24) and tuple(c.view(2).pages.shape) == (4, PAGE, 52)
    assert tuple(c.view(3)[1][1].shape) == (3, 1, 104) and c.view(5) is None
    s = c.acquire(2)
    kept[s[1]].fill_(5.0)
    state2[s[1]].fill_(6.0)
    c.release(s)
    again = c.acquire(3)
    assert s[1] in again and float(kept.abs().sum()) == 0.0 and float(state2.abs().sum()) == 0.0
    c.check()


def test_frequencies_stretched_band_by_band():
    """The three bands: short waves keep their frequency, long ones are slowed by the factor, between them the two
    are blended with a weight that runs from 0 to 1; the package's table and the plain one agree."""
    rot = {"base": 10000.0, "dims": 64, "scaling": {"factor": 6.0, "low": 1.0, "high": 4.0, "original": 1024}}
    f0 = plain.frequencies({"base": 10000.0, "dims": 64})
    f = plain.frequencies(rot)
    wave = 2 * math.pi / f0
    assert np.allclose(f0, 10000.0 ** (-np.arange(32) / 32.0))
    short, long_ = wave < 1024 / 4.0, wave > 1024 / 1.0
    assert short.any() and long_.any() and (~short & ~long_).any()
    assert np.array_equal(f[short], f0[short]) and np.allclose(f[long_], f0[long_] / 6.0)
    mid = ~short & ~long_
    assert np.all(f[mid] < f0[mid]) and np.all(f[mid] > f0[mid] / 6.0)
    s = (1024 / wave[mid] - 1.0) / 3.0
    assert np.allclose(f[mid], (1 - s) * f0[mid] / 6.0 + s * f0[mid])
    table = RotaryHalfSplit.frequencies(64, 10000.0, rot["scaling"]).numpy()
    assert np.allclose(table, f, rtol=1e-14)
    assert np.allclose(RotaryHalfSplit.frequencies(64, 10000.0).numpy(), f0, rtol=1e-14)


def test_plain_rotation_is_a_complex_multiplication_and_leaves_the_rest():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 3, 10))
    f = np.array([1.0, 0.3, 0.01])
    pos = np.array([0.0, 1.0, 2.0, 50.0, 700.0])
    y = plain.rotate_pairs(x, pos, f)
    z = (x[..., 0:6:2] + 1j * x[..., 1:6:2]) * np.exp(1j * pos[:, None, None] * f)
    assert np.allclose(y[..., 0:6:2], z.real) and np.allclose(y[..., 1:6:2], z.imag)
    assert np.array_equal(y[..., 6:], x[..., 6:]) and np.array_equal(y[0], x[0])
    # scores depend on the distance only
    q, k = rng.normal(size=(1, 1, 6)), rng.normal(size=(1, 1, 6))
    a = plain.rotate_pairs(q, np.array([40.0]), f) @ plain.rotate_pairs(k, np.array([33.0]), f).reshape(6)
    b = plain.rotate_pairs(q, np.array([7.0]), f) @ k.reshape(6)
    assert np.allclose(a, b)


def test_plain_visibility_and_sink():
    v = plain.visible(6, 3)
    assert v[5].tolist() == [False, False, False, True, True, True] and v[1].tolist() == [True, True] + [False] * 4
    assert plain.visible(4, None)[3].all() and plain.visible(4, 1).sum() == 4
    s = np.log(np.array([[1.0, 2.0, 5.0]]))
    p = plain.sink_softmax(s, np.array([[True, True, False]]), math.log(3.0))
    assert np.allclose(p, [[1 / 6, 2 / 6, 0.0]])            # the sink takes 3 of 6 and has no value


def test_plain_short_convolution():
    x = np.arange(1.0, 6.0)[:, None] * np.array([[1.0, 10.0]])
    w = np.array([[0.5, 0.0, 1.0], [0.0, 2.0, 0.0]])        # [channels, taps], the last column is the current token's
    y = plain.short_convolution(x, w)
    assert np.allclose(y[:, 0], [1.0, 2.0, 3.5, 5.0, 6.5])  # x_t + 0.5 x_(t-2), zeros before the start
    assert np.allclose(y[:, 1], [0.0, 20.0, 40.0, 60.0, 80.0])


def test_plain_delta_rule_against_its_unrolled_form():
    """Without decay and with beta = 1, writing v under a unit key k replaces what k held; with decay g and
    orthogonal keys the read-out of a key written m tokens ago is g^m times its value."""
    dim, vdim = 4, 3
    S = np.zeros((dim, vdim))
    keys = np.eye(dim)
    vals = np.arange(12.0).reshape(4, 3) + 1
    g, beta = 0.5, 1.0
    for t in range(4):
        S = g * S
        S = S + np.outer(keys[t], beta * (vals[t] - S.T @ keys[t]))
    for t in range(4):
        assert np.allclose(S.T @ keys[t], g ** (3 - t) * vals[t])
    S2 = S + np.outer(keys[1], 1.0 * (np.ones(3) - S.T @ keys[1]))
    assert np.allclose(S2.T @ keys[1], np.ones(3)) and np.allclose(S2.T @ keys[0], S.T @ keys[0])


def test_plain_lightning_attention_is_its_unrolled_sum():
    rng = np.random.default_rng(1)
    n, W = 9, 12
    p = {"heads": 2, "dim": 3, "vdim": 4, "decay": [0.5, 0.9]}
    w = {"q": rng.normal(size=(6, W)), "k": rng.normal(size=(6, W)), "v": rng.normal(size=(8, W)),
         "g": rng.normal(size=(8, W)), "o": np.eye(8), "norm": np.ones(8)}
    h = rng.normal(size=(n, W))
    out = plain.lightning_attention(h, w, p, 1e-6)
    q, k, v = (plain.silu(h @ w[x].T) for x in "qkv")
    o = np.zeros((n, 8))
    for head in range(2):
        for t in range(n):
            for j in range(t + 1):
                o[t, 4 * head:4 * head + 4] += p["decay"][head] ** (t - j) * \
                    (q[t, 3 * head:3 * head + 3] @ k[j, 3 * head:3 * head + 3]) * v[j, 4 * head:4 * head + 4]
    ref = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-6) * plain.sigmoid(h @ w["g"].T)
    assert np.allclose(out, ref)
