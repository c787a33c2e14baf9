"""The Rupasun configuration, its tensor list, what its mixers ask of the cache, and the plain
implementation's mechanisms against closed forms (no device needed)."""
import copy

import numpy as np
import pytest

import torchless_rs_b200 as tl
from plain import rupasun_plain as plain
from rupasun_tiny import CONFIGS, tensor_shapes
from torchless_rs_b200.config import ConfigError
from torchless_rs_b200.engine.model import expected_tensors


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_keys_are_read_and_written_back(name):
    raw = CONFIGS[name]
    cfg = tl.config_from_dict(raw)
    assert type(cfg).__name__ == "RupasunConfig"
    assert tl.config_from_dict(cfg.to_dict()) == cfg
    assert (cfg.width, cfg.vocab, cfg.eps) == (raw["width"], raw["vocab"], raw["norm"]["eps"])
    for layer, entry in zip(cfg.layers, raw["layers"]):
        m, a = layer.mixer, entry["mixer"]
        assert m.type == entry["type"]
        assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale) == (a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"])
        assert (m.rot.dims, m.rot.base) == (a["rot"]["dims"], a["rot"]["base"]) if "rot" in a else m.rot is None
        if entry["type"] == "attention":
            assert m.diff == a["diff"]
        else:
            assert m.window == (a.get("mask") or {}).get("size") and m.softcap == a.get("softcap")
        mlp = entry["mlp"]
        if mlp is None:
            assert layer.mlp is None
        elif mlp["kind"] == "dense":
            assert layer.mlp.ff == mlp["ff"]
        else:
            r, g = mlp["router"], mlp["router"].get("groups") or {"count": 1, "keep": 1}
            assert (layer.mlp.ff, layer.mlp.limit) == (mlp["expert"]["ff"], mlp["expert"]["limit"])
            assert (layer.mlp.experts, layer.mlp.top, layer.mlp.route_scale) == (r["experts"], r["top"], r["scale"])
            assert (layer.mlp.groups, layer.mlp.keep) == (g["count"], g["keep"])
            sh = mlp.get("shared")
            assert (layer.mlp.shared_ff, layer.mlp.shared_limit) == ((sh["ff"], sh["limit"]) if sh else (None, None))


def test_errors_name_the_key():
    base = CONFIGS["P"]
    for change, word in ((lambda c: c["layers"][0].__setitem__("type", "attention_9"), "type"),
                         (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
                         (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
                         (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
                         (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 2), "kv_heads"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "dims"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
                         (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "top"),
                         (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
                         (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("keep", 4), "keep"),
                         (lambda c: c["layers"][1]["mlp"]["shared"].pop("limit"), "limit"),
                         (lambda c: c.pop("width"), "width")):
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError) as e:
            tl.config_from_dict(c)
        assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_model_asks_for_the_designs_tensors(name):
    exp = expected_tensors(tl.config_from_dict(CONFIGS[name]).model_spec())
    want = tensor_shapes(CONFIGS[name])
    got = {n: tuple(s.shape) for n, s in exp.items() if not s.optional}
    assert got == want
    # a layer without a feed-forward accepts the norms it does not use
    without = [i for i, l in enumerate(CONFIGS[name]["layers"]) if l["mlp"] is None]
    assert {n for n, s in exp.items() if s.optional} == {f"l{i}.{n}" for i in without for n in ("norm2", "norm2b")}


def test_parts_and_what_they_ask_of_the_cache():
    from torchless_rs_b200.parts import lookup
    spec = tl.config_from_dict(CONFIGS["P"]).model_spec()
    kinds = [(l.block.kind, l.mixer.kind, l.feed_forward.kind, l.position.kind if l.position else None)
             for l in spec.layers]
    assert kinds == [("sandwich", "differential_attention", "relu_squared", "rope_half_split"),
                     ("sandwich", "gated_window_attention", "moe_grouped_sigmoid", "rope_interleaved"),
                     ("sandwich_mixer_only", "gated_window_attention", "none", "rope_interleaved"),
                     ("sandwich", "differential_attention", "moe_grouped_sigmoid", None)]
    for l in spec.layers:
        assert set(lookup("block", l.block.kind).norm_roles) == set(l.norms)
    # the two maps' keys of a key/value head share a row of the cache; the window is the cache's too
    assert spec.layers[0].mixer.get("dim") == 16 and spec.layers[0].position.get("head_dim") == 8
    assert spec.layers[1].mixer.get("window") == 20 and spec.layers[3].mixer.get("rot_dims") == 0


# ---- the plain mechanisms against closed forms ---------------------------------------------------
def test_plain_rotation():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 2, 10))
    pos = np.array([0.0, 1.0, 2.0, 7.0, 300.0])
    for inter in (False, True):
        y = plain.rotate(x, pos, 6, 100.0, inter)
        assert np.array_equal(y[0], x[0]) and np.array_equal(y[..., 6:], x[..., 6:])      # position 0; the rest
        assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
        # pair 1 of position 7 turns by 7 * 100^(-2/6)
        a = 7.0 * 100.0 ** (-2.0 / 6.0)
        i, j = (2, 3) if inter else (1, 4)
        u, v = x[3, 0, i], x[3, 0, j]
        assert np.allclose([y[3, 0, i], y[3, 0, j]], [u * np.cos(a) - v * np.sin(a), v * np.cos(a) + u * np.sin(a)])
    # the dot product of a rotated query and key depends on the distance only
    q, k = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    d1 = (plain.rotate(q, np.array([9.0]), 8, 50.0, True) * plain.rotate(k, np.array([4.0]), 8, 50.0, True)).sum()
    d2 = (plain.rotate(q, np.array([105.0]), 8, 50.0, True) * plain.rotate(k, np.array([100.0]), 8, 50.0, True)).sum()
    assert np.allclose(d1, d2)


def test_plain_visibility():
    pos = np.arange(6, dtype=np.float64)
    v = plain.visible(pos, 3)
    assert [list(np.flatnonzero(r)) for r in v] == [[0], [0, 1], [0, 1, 2], [1, 2, 3], [2, 3, 4], [3, 4, 5]]
    assert plain.visible(pos, None).sum() == 21 and np.array_equal(plain.visible(pos, 1), np.eye(6, dtype=bool))


def test_plain_differential_attention():
    """With equal maps the two outputs are equal and o = (1 - lambda) a; the per-head norm then leaves
    sign(1 - lambda) a / rms(a) times (1 - diff), whatever lambda is."""
    rng = np.random.default_rng(1)
    W, H, G, d, v, n = 20, 2, 1, 4, 6, 9
    p = {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "diff": 0.25, "scale": 0.5, "rot": {"dims": 4, "base": 10.0}}
    q1, k1 = rng.normal(size=(H, d, W)), rng.normal(size=(G, d, W))
    w = {"q": np.stack([q1, q1], 1).reshape(H * 2 * d, W), "k": np.stack([k1, k1], 1).reshape(G * 2 * d, W),
         "v": rng.normal(size=(G * v, W)), "o": np.eye(H * v),
         "lq1": rng.normal(size=d), "lk1": rng.normal(size=d), "lq2": rng.normal(size=d), "lk2": rng.normal(size=d)}
    lam = plain.difference_factor(w, 0.25)
    assert np.isclose(lam, np.exp(w["lq1"] @ w["lk1"]) - np.exp(w["lq2"] @ w["lk2"]) + 0.25)
    h = rng.normal(size=(n, W))
    out = plain.differential_attention(h, w, p, 0.0).reshape(n, H, v)
    # one map alone, by hand
    pos = np.arange(n, dtype=np.float64)
    q = plain.rotate((h @ q1.reshape(H * d, W).T).reshape(n, H, d), pos, 4, 10.0, False)
    k = plain.rotate((h @ k1.reshape(G * d, W).T).reshape(n, G, d), pos, 4, 10.0, False)
    vv = (h @ w["v"].T).reshape(n, G, v)
    for head in range(H):
        a = plain.softmax_rows((q[:, head] @ k[:, 0].T) * 0.5, plain.visible(pos, None)) @ vv[:, 0]
        assert np.allclose(out[:, head], np.sign(1 - lam) * plain.rms_normalise(a, 0.0) * 0.75)
    assert np.allclose(out[0, 0], np.sign(1 - lam) * plain.rms_normalise(vv[0, 0], 0.0) * 0.75)     # one key: its value


def test_plain_window_attention_gate_and_cap():
    rng = np.random.default_rng(2)
    W, n = 12, 7
    p = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 2.0, "softcap": 1.5, "mask": {"size": 1},
         "rot": {"dims": 2, "base": 3.0}}
    w = {"q": rng.normal(size=(4, W)), "k": rng.normal(size=(4, W)), "v": rng.normal(size=(3, W)),
         "g": rng.normal(size=(3, W)), "o": np.eye(3)}
    h = rng.normal(size=(n, W))
    # a window of one key: every position returns its own value times its gate
    assert np.allclose(plain.window_attention(h, w, p, 1e-6), (h @ w["v"].T) * plain.sigmoid(h @ w["g"].T))
    # unit-normed q and k: |score| <= scale * dim before the cap, and below the cap after it
    p2 = {**p, "mask": None, "scale": 100.0}
    out = plain.window_attention(h[:2], w, p2, 1e-6)
    q = plain.rms_normalise(plain.rotate((h[:2] @ w["q"].T).reshape(2, 1, 4), np.arange(2.0), 2, 3.0, True), 1e-6)
    k = plain.rms_normalise(plain.rotate((h[:2] @ w["k"].T).reshape(2, 1, 4), np.arange(2.0), 2, 3.0, True), 1e-6)
    s = 1.5 * np.tanh((q[1, 0] @ k[:, 0].T) * 100.0 / 1.5)
    pr = np.exp(s) / np.exp(s).sum()
    assert np.allclose(out[1], (pr @ (h[:2] @ w["v"].T)) * plain.sigmoid(h[1] @ w["g"].T))


def test_plain_router_and_experts():
    s = np.array([0.9, 0.1, 0.5, 0.6, 0.8, 0.0, 0.7, 0.75])
    # groups of two: sums 1.0, 1.1, 0.8, 1.45 -> groups 3 and 1 are kept; the best two there: 7 and 6
    chosen, allowed = plain.route(s, 2, 4, 2)
    assert list(chosen) == [7, 6] and list(np.flatnonzero(allowed)) == [2, 3, 6, 7]
    # groups of four: only the two largest of a group count: 0.9 + 0.6 against 0.8 + 0.75
    chosen, allowed = plain.route(s, 3, 2, 1)
    assert list(chosen) == [4, 7, 6] and list(np.flatnonzero(allowed)) == [4, 5, 6, 7]
    # groups of one; all groups kept; a tie goes to the lower index
    assert list(plain.route(s, 2, 8, 8)[0]) == [0, 4] and list(plain.route(np.array([0.5, 0.5, 0.5]), 2, 1, 1)[0]) == [0, 1]
    rng = np.random.default_rng(3)
    W, f, E = 10, 6, 4
    w = {"router": rng.normal(size=(E, W))}
    for e in list(range(E)) + ["s"]:
        name = "shared" if e == "s" else f"e{e}"
        w.update({f"{name}.gate": rng.normal(size=(f, W)), f"{name}.up": rng.normal(size=(f, W)),
                  f"{name}.down": rng.normal(size=(W, f))})
    h = rng.normal(size=(1, W))
    p = {"kind": "moe", "expert": {"ff": f, "limit": 0.4}, "router": {"experts": E, "top": 2, "scale": 3.0},
         "shared": {"ff": f, "limit": 9.0}}
    sc = plain.sigmoid(h[0] @ w["router"].T)
    a, b = np.argsort(-sc)[:2]
    one = lambda e, lim: plain.expert(h, w[f"{e}.gate"], w[f"{e}.up"], w[f"{e}.down"], lim)[0]
    ref = 3.0 * (sc[a] * one(f"e{a}", 0.4) + sc[b] * one(f"e{b}", 0.4)) / (sc[a] + sc[b]) + one("shared", 9.0)
    assert np.allclose(plain.expert_ff(h, w, p)[0], ref)
    # the expert's clamps: the gate from above only, the other factor on both sides
    g = np.array([[-3.0, 0.2, 5.0]])
    y = plain.expert(g, np.eye(3), -np.eye(3), np.eye(3), 1.0)[0]
    gg, uu = np.array([-3.0, 0.2, 1.0]), np.array([1.0, -0.2, -1.0])
    assert np.allclose(y, gg * plain.sigmoid(1.702 * gg) * (uu + 1.0))
    assert np.allclose(plain.dense_ff(g, {"up": np.eye(3), "down": np.eye(3)}), [[0.0, 0.04, 25.0]])


def test_plain_layer_norms_both_sides():
    """With a mixer and feed-forward whose outputs are huge or tiny, the output norms bring both to the
    size of their weights: x grows by sqrt(width) * |w| per sublayer at most."""
    cfg = CONFIGS["Q"]
    from rupasun_tiny import make_weights
    import torch
    w = {k: v.double().numpy() for k, v in make_weights(cfg, 1, torch.float32).items()}
    big = {k: (v * 1e3 if k.endswith((".o", ".down")) else v) for k, v in w.items()}
    a = plain.forward(cfg, w, [3, 5, 8])
    b = plain.forward(cfg, big, [3, 5, 8])
    assert np.allclose(a, b, rtol=0, atol=2e-3 * np.abs(a).max())      # up to what eps does to small outputs
