"""Small Rupasun configurations with weights made here (numpy, not the package's generator), a model
folder written with the `safetensors` package, and a loader through the package's entry point.
Matrices are N(0, 1/in) so that activations are of order one and attention scores spread over a few
units: a key that is wrongly seen or missed, a wrong rotation or a wrong expert changes the result by
far more than rounding.

The configurations differ from one another, layer by layer, in every size: heads and key/value heads
(also equal, also one), query and value sizes that differ and are no multiples of 4, rotated entries
fewer than the query's (and none), windows of one key, inside a page, across pages and absent, caps
present and absent, layers without a feed-forward, experts in groups of one, two and three, all groups
kept, a choice of one and of all that can be chosen, with and without a shared expert."""
from __future__ import annotations

import json
import os
import shutil
import tempfile

import numpy as np
import torch

from plain import rupasun_plain as plain


def diff_mixer(heads, kv_heads, dim, vdim, diff, rot=None, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": scale if scale is not None else 1.0 / float(np.sqrt(dim))}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return {"type": "attention", "mixer": m}


def window_mixer(heads, kv_heads, dim, vdim, window, rot=None, base=10000.0, scale=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else 1.5}      # unit-normed q and k: q . k is at most dim
    if softcap:
        m["softcap"] = softcap
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return {"type": "attention_2", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups=None, keep=None, limit=1.0, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(mixer, mlp):
    return {**mixer, "mlp": mlp}


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Rupasun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # rotation of a part of the query; a window inside a page with a cap; a window across pages without a
    # feed-forward; no rotation at all; groups of two with a shared expert; no groups, a choice of one
    "P": config(96, 211, [
        layer(diff_mixer(3, 1, 16, 24, diff=0.3, rot=8), dense(160)),
        layer(window_mixer(4, 2, 32, 12, window=20, rot=32, base=500.0, softcap=6.0),
              moe(24, experts=6, top=2, groups=3, keep=2, limit=0.8, scale=1.5, shared=(40, 1.5))),
        layer(window_mixer(2, 2, 24, 10, window=70, rot=12), None),
        layer(diff_mixer(2, 2, 8, 8, diff=0.8), moe(16, experts=3, top=1, limit=2.5)),
    ], eps=1e-6),
    # a window of one key; one head; groups of one member; all groups kept; a choice of all that can be chosen
    "Q": config(80, 130, [
        layer(window_mixer(1, 1, 24, 36, window=1, rot=24, scale=0.7), moe(40, experts=4, top=2, groups=4, keep=2)),
        layer(diff_mixer(4, 1, 12, 6, diff=0.1, rot=12, base=77.0, scale=0.4),
              moe(16, experts=6, top=4, groups=3, keep=2, limit=0.5, scale=2.5, shared=(8, 3.0))),
        layer(window_mixer(4, 4, 8, 6, window=5, softcap=3.0), moe(12, experts=4, top=3, groups=2, keep=2)),
    ], eps=3e-5),
    # sizes that the tensor-core kernels take (multiples of 16), windows across pages and absent
    "R": config(192, 520, [
        layer(diff_mixer(4, 2, 32, 64, diff=0.5, rot=32), dense(448)),
        layer(window_mixer(8, 2, 64, 64, window=130, rot=64, softcap=30.0),
              moe(64, experts=8, top=2, groups=4, keep=3, scale=2.0, shared=(64, 2.0))),
        layer(window_mixer(2, 2, 128, 128, window=None, rot=64, softcap=10.0), dense(256)),
        layer(diff_mixer(2, 1, 64, 32, diff=0.7, rot=16, base=300.0), None),
    ]),
    # two maps together as wide as the values (64 and 128), a window without a cap: what the plain attention
    # kernels take in bfloat16
    "S": config(128, 300, [
        layer(diff_mixer(2, 1, 64, 128, diff=0.4, rot=64), dense(192)),
        layer(window_mixer(4, 2, 64, 64, window=70, rot=32), None),
        layer(diff_mixer(4, 2, 32, 64, diff=0.6, rot=16, base=900.0), moe(32, experts=4, top=2, groups=2, keep=1, scale=1.5)),
    ]),
}


def random_config(seed: int) -> dict:
    """A configuration drawn from `seed`: two to five layers, each with its own mixer (either kind; one to
    eight heads over any divisor of key/value heads; query sizes 8 to 128 with value sizes that are and are
    not twice the query's; rotation of all, of a part, of nothing; windows of 1 to 150 and none; caps
    present and absent) and feed-forward (none, dense, or 4 to 32 experts in 1 to 8 groups with any number
    kept and chosen, with and without a shared expert).  Scores stay within a few units, as a trained
    model's do, so that bfloat16 rounding stays within the models' bound."""
    r = np.random.default_rng(seed)

    def pick(xs):
        return xs[int(r.integers(0, len(xs)))]
    width, vocab = pick([64, 128, 192, 320]), pick([97, 300, 1000])
    layers = []
    for _ in range(int(r.integers(2, 6))):
        H = pick([1, 2, 4, 6, 8])
        G = pick([g for g in (1, 2, 3, 4, 6, 8) if H % g == 0])
        if r.random() < 0.5:
            dim = pick([8, 24, 32, 40, 64])
            vdim = pick([2 * dim, 2 * dim, 24, 40, 64, 128])
            rot = pick([None, dim, 2 * int(r.integers(1, dim // 2 + 1))])
            mixer = diff_mixer(H, G, dim, vdim, diff=float(r.uniform(0.1, 0.9)), rot=rot,
                               base=float(pick([100.0, 10000.0, 5e5])))
        else:
            dim = pick([24, 32, 64, 128])
            vdim = pick([dim, dim, 24, 40, 64])
            rot = pick([None, dim, 2 * int(r.integers(1, dim // 2 + 1))])
            mixer = window_mixer(H, G, dim, vdim, window=pick([None, 1, 7, 33, 64, 100, 150]), rot=rot,
                                 base=float(pick([100.0, 10000.0, 5e5])), scale=float(r.uniform(0.7, 1.5)) * 8.0 / dim,
                                 softcap=pick([None, 5.0, 20.0, 50.0]))
        k = r.random()
        if k < 0.2:
            mlp = None
        elif k < 0.55:
            mlp = dense(pick([64, 200, 384]))
        else:
            E = pick([4, 6, 8, 12, 16, 32])
            count = pick([c for c in (1, 2, 3, 4, 8) if E % c == 0])
            keep = int(r.integers(1, count + 1))
            top = int(r.integers(1, min(8, keep * (E // count)) + 1))
            mlp = moe(pick([16, 32, 64]), E, top, groups=count if r.random() < 0.85 else None, keep=keep,
                      limit=pick([0.5, 1.0, 7.0]), scale=float(r.uniform(0.5, 3.0)),
                      shared=(pick([16, 48]), pick([0.7, 3.0])) if r.random() < 0.6 else None)
        layers.append(layer(mixer, mlp))
    return config(width, vocab, layers, eps=pick([1e-6, 1e-5]))


def tensor_shapes(cfg: dict) -> dict:
    """Tensor names and shapes, as the design lays them out."""
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    for i, l in enumerate(cfg["layers"]):
        m, p = l["mixer"], f"l{i}."
        H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (W,), p + "norm1b": (W,)})
        if l["type"] == "attention":
            out.update({p + "mix.q": (H * 2 * d, W), p + "mix.k": (G * 2 * d, W), p + "mix.v": (G * v, W),
                        p + "mix.lq1": (d,), p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,),
                        p + "mix.o": (W, H * v)})
        else:
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * v, W),
                        p + "mix.g": (H * v, W), p + "mix.o": (W, H * v)})
        mlp = l.get("mlp")
        if mlp:
            out.update({p + "norm2": (W,), p + "norm2b": (W,)})
            if mlp["kind"] == "dense":
                out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                E, f = mlp["router"]["experts"], mlp["expert"]["ff"]
                out[p + "mlp.router"] = (E, W)
                for e in range(E):
                    out.update({p + f"mlp.e{e}.gate": (f, W), p + f"mlp.e{e}.up": (f, W), p + f"mlp.e{e}.down": (W, f)})
                if mlp.get("shared"):
                    sf = mlp["shared"]["ff"]
                    out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W),
                                p + "mlp.shared.down": (W, sf)})
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def make_weights(cfg: dict, seed: int, store: torch.dtype) -> dict:
    """name -> torch tensor in `store`."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("lq1", "lk1", "lq2", "lk2"):
            v = rng.normal(0, 0.5 / np.sqrt(shape[0]) ** 0.5, shape)      # exp(lq . lk) of order one
        elif leaf == "router":
            v = rng.normal(0, 2.0 / np.sqrt(shape[1]), shape)
        elif len(shape) == 1:
            v = 1.0 + rng.normal(0, 0.2, shape)
        elif name == "embed":
            v = rng.normal(0, 1.0, shape)
        else:
            v = rng.normal(0, 1.0 / np.sqrt(shape[1]), shape)
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(store)
    return out


def write_folder(cfg: dict, weights: dict, where: str | None = None) -> str:
    from safetensors.torch import save_file
    d = where or tempfile.mkdtemp(prefix="tl_rupasun_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


class TModel:
    """A configuration loaded through the package's entry point, with the plain implementation (in
    float64, on the stored values) beside it."""

    def __init__(self, cfg, dtype: str, seed: int = 0, max_tokens: int = 1024, max_batch=None, weights=None):
        import torchless_rs_b200 as tl
        self.cfg = CONFIGS[cfg] if isinstance(cfg, str) else cfg
        self.dtype = dtype
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        self.stored = weights if weights is not None else make_weights(self.cfg, seed, store)
        self.weights = {k: v.to(torch.float64).numpy() for k, v in self.stored.items()}
        d = write_folder(self.cfg, self.stored)
        try:
            self.model = tl.load(d, dtype=dtype, max_tokens=max_tokens, max_batch=max_batch)
        finally:
            shutil.rmtree(d, ignore_errors=True)
        self.engine = self.model.engine
        self._ref = {}

    def reference(self, tokens) -> np.ndarray:
        key = tuple(tokens)
        if key not in self._ref:
            self._ref[key] = plain.forward(self.cfg, self.weights, list(tokens))
        return self._ref[key]

    def step_np(self, slots, tokens, want) -> np.ndarray:
        return self.engine.step(slots, tokens, want).float().cpu().numpy().copy()


def tokens_of(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def sure_tokens(tm: "TModel", rng, n: int, margin: float | None = None):
    """`n` random tokens none of which leaves a router within `margin` of another choice (by default what
    the rounding of the router's input to the model's activation type can move: a token that does would
    run through other experts than in the plain implementation, and every later token would see it).
    A position's routers depend on the tokens up to it only, so the first close position gets another
    token until none is left."""
    if margin is None:
        margin = 1e-4 if tm.dtype == "float32" else 2e-2
    V = tm.cfg["vocab"]
    toks = tokens_of(rng, n, V)
    for _ in range(20 * n):
        m: list = []
        plain.forward(tm.cfg, tm.weights, toks, margins=m)
        close = np.nonzero(np.min(np.stack(m), axis=0) < margin)[0] if m else []
        if len(close) == 0:
            return toks
        toks[int(close[0])] = int(rng.integers(0, V))
    raise AssertionError("no sequence without a close call was found")
