"""Small Fezolorn configurations with weights made here (numpy, not the package's generator), a model
folder written with the `safetensors` package, and a loader through the package's entry point.
Matrices are N(0, 1/in) so that activations are of order one and attention scores spread over a few
units: a key that is wrongly seen or missed, a sink that is left out or a lost state changes the
result by far more than rounding.

The configurations differ from one another, layer by layer, in every size and in the order of the
layers: heads and key/value heads (equal, one, several per group), key and value sizes that differ
and are no multiples of 4, rotations of a part of a head, of all of it and of nothing, with and without
stretched frequencies, windows of one key, inside a page, across pages and absent, convolutions of one
to five taps, states that are not square, decays from strong to nearly none, latents whose sizes the
tensor-core kernels take and latents they do not, layers without a feed-forward."""
from __future__ import annotations

import json
import os
import shutil
import tempfile

import numpy as np
import torch

from plain import fezolorn_plain as plain


def rot(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def left(heads, kv_heads, dim, window, rotation=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
         "scale": scale if scale is not None else 2.0 / float(np.sqrt(dim))}
    if window:
        m["mask"] = {"size": window}
    if rotation:
        m["rot"] = rotation
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(l, r, mlp, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def lightning(heads, dim, vdim, decay, mlp):
    assert len(decay) == heads
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, mlp, base=10000.0, scale=None, scaling=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale if scale is not None else 2.0 / float(np.sqrt(dim + rot_dim)),
                      "rot": rot(rot_dim, base, scaling)},
            "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, eps=1e-6):
    return {"architecture": "Fezolorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # a window inside a page, part of each head rotated with stretched frequencies; a latent the tensor-core
    # kernels do not take; a layer without feed-forward
    "P": config(96, 211, [
        parallel(left(4, 2, 16, 20, rot(8, 500.0, (4.0, 1.0, 4.0, 64))), right(4, 2, 16, 8, 4), dense(160), 0.7, 1.3),
        lightning(3, 16, 24, (0.5, 0.9, 0.995), dense(120)),
        latent(3, 24, 8, 20, 40, 44, None),
        parallel(left(3, 1, 24, 70, rot(24, 10000.0)), right(2, 1, 40, 12, 2), None, 1.5, 0.5),
    ]),
    # the latent first; as many key/value heads as heads; a window of one key; no window and no rotation; a
    # convolution of one tap; one head; odd sizes
    "Q": config(80, 130, [
        latent(2, 10, 6, 7, 12, 36, dense(96), base=100.0, scaling=(2.0, 1.0, 2.0, 16)),
        parallel(left(3, 3, 24, 1, rot(4, 50.0)), right(2, 2, 33, 5, 1), dense(64), 1.0, 1.0),
        lightning(1, 40, 12, (0.97,), None),
        parallel(left(1, 1, 20, None, None), right(3, 1, 8, 36, 5), dense(48), 0.4, 2.0),
        lightning(4, 5, 9, (0.2, 0.6, 0.9, 1.0), dense(40)),
    ], eps=3e-5),
    # sizes that the tensor-core kernels take (multiples of 16 and more), windows across pages
    "R": config(256, 520, [
        lightning(4, 64, 32, (0.8, 0.95, 0.99, 0.999), dense(448)),
        parallel(left(8, 2, 64, 130, rot(32, 1e6, (8.0, 1.0, 4.0, 256))), right(4, 2, 64, 64, 4), dense(448), 1.2, 0.9),
        latent(4, 32, 16, 32, 64, 64, dense(256), base=1e6),
        parallel(left(4, 4, 32, 64, rot(32, 1e4)), right(8, 2, 32, 16, 3), dense(256), 0.8, 1.1),
        latent(6, 64, 32, 48, 96, 128, dense(256)),
    ]),
}


def random_config(seed: int) -> dict:
    """Another configuration for every seed: two to five layers of any kind in any order, any sizes."""
    rng = np.random.default_rng(seed)
    width = int(rng.choice([64, 72, 96, 128]))
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        mlp = dense(int(rng.choice([48, 100, 128]))) if rng.random() < 0.8 else None
        kind = pick("parallel", "lightning", "latent")
        if kind == "parallel":
            G = pick(1, 2, 3)
            H = G * pick(1, 2, 4)
            dim = pick(8, 16, 24, 32, 64)
            rd = pick(0, 2, dim // 2, dim)
            rd -= rd % 2
            sc = pick(None, (float(rng.uniform(2, 8)), 1.0, float(rng.uniform(2, 4)), int(rng.choice([32, 128]))))
            rG = pick(1, 2)
            layers.append(parallel(
                left(H, G, dim, pick(None, 1, 3, 30, 64, 65, 100), rot(rd, float(rng.choice([100.0, 1e4])), sc) if rd else None,
                     scale=float(rng.uniform(0.1, 0.5))),
                right(rG * pick(1, 2, 3), rG, pick(8, 16, 20, 32), pick(4, 16, 24, 32), pick(1, 2, 3, 4)),
                mlp, float(rng.uniform(0.5, 1.5)), float(rng.uniform(0.5, 1.5))))
        elif kind == "lightning":
            H = pick(1, 2, 4)
            layers.append(lightning(H, pick(8, 16, 32), pick(8, 12, 32), [float(rng.uniform(0.3, 1.0)) for _ in range(H)], mlp))
        else:
            rd = pick(2, 8, 16)
            layers.append(latent(pick(1, 2, 5), pick(8, 16, 24), rd, pick(8, 16, 20), pick(16, 24, 32), pick(16, 32, 40),
                                 mlp, base=float(rng.choice([100.0, 1e4])), scale=float(rng.uniform(0.1, 0.4))))
    return config(width, int(rng.choice([97, 150, 256])), layers, eps=float(rng.choice([1e-6, 1e-5])))


def tensor_shapes(cfg: dict) -> dict:
    """Tensor names and shapes, as the design lays them out."""
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        out[p + "norm1"] = (W,)
        if l["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, d = a["heads"], a["kv_heads"], a["dim"]
            out.update({p + "mix.left.q": (H * d, W), p + "mix.left.q.b": (H * d,), p + "mix.left.k": (G * d, W),
                        p + "mix.left.k.b": (G * d,), p + "mix.left.sink": (H,), p + "mix.left.o": (W, H * d),
                        p + "mix.left.o.b": (W,)})
            H, G, d, v, t = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            out.update({p + "mix.right.q": (G * d, W), p + "mix.right.q.conv": (G * d, t), p + "mix.right.k": (G * d, W),
                        p + "mix.right.k.conv": (G * d, t), p + "mix.right.v": (H * v, W),
                        p + "mix.right.v.conv": (H * v, t), p + "mix.right.b": (H, W), p + "mix.right.a": (H, W),
                        p + "mix.right.A_log": (H,), p + "mix.right.dt_bias": (H,), p + "mix.right.g": (H * v, W),
                        p + "mix.right.norm": (v,), p + "mix.right.o": (W, H * v)})
        elif l["type"] == "lightning":
            H, d, v = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * v, W), p + "mix.g": (H * v, W),
                        p + "mix.o": (W, H * v), p + "mix.norm": (H * v,)})
        else:
            H, d, r, v, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + r), qr),
                        p + "mix.dkv": (kr + r, W), p + "mix.dkv.norm": (kr,), p + "mix.uk": (H * d, kr),
                        p + "mix.uv": (H * v, kr), p + "mix.sink": (H,), p + "mix.o": (W, H * v)})
        mlp = l.get("mlp")
        if mlp:
            out.update({p + "norm2": (W,), p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W),
                        p + "mlp.down": (W, mlp["ff"])})
    out["final.norm"] = (W,)
    return out


def make_weights(cfg: dict, seed: int, store: torch.dtype) -> dict:
    """name -> torch tensor in `store`."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".sink"):
            v = rng.normal(0.5, 1.0, shape)
        elif name.endswith(".conv"):
            v = rng.normal(0, 1.0 / np.sqrt(shape[1]), shape) + (np.arange(shape[1]) == shape[1] - 1)
        elif name.endswith(".A_log"):
            v = rng.normal(-1.0, 0.7, shape)
        elif name.endswith(".dt_bias"):
            v = rng.normal(0.0, 1.0, shape)
        elif name.endswith(".b") and len(shape) == 1:
            v = rng.normal(0, 0.5, shape)
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
    d = where or tempfile.mkdtemp(prefix="tl_fezolorn_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


class FModel:
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
