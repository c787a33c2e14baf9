"""Plain, slow restatement of the Fezolorn decoder, for tests only: numpy, whole sequences, no cache,
one function per mechanism, token-by-token loops where the design is a recurrence.  It shares no code
with the package under test.

The design in short.  Pre-norm residual layers, x <- x + mixer(N(x)); x <- x + ff(N(x)), N an RMS norm
with a weight.  A layer's mixer is one of three:
  * `parallel`: two branches on the same input, summed with one factor each.  Left: softmax attention
    with grouped key/value heads whose values are the projected keys themselves (taken before rotation
    and norm), biased projections, a rotation of the first entries of every head by position
    (neighbouring pairs, frequencies stretched band by band), a unit RMS norm of rotated queries and
    keys, a sliding window and a sink logit per head in the denominator.  Right: the gated delta rule,
    a matrix state per head that decays by one number per token and head and is corrected towards the
    token's value, fed through short causal convolutions.
  * `lightning`: linear attention with a fixed decay per head, S_t = d S_(t-1) + k_t v_t^T.
  * `latent_attention`: causal softmax attention whose keys and values are rebuilt from a low-rank
    latent, with one rotated key part shared by all heads and a sink.
The feed-forward is SwiGLU or absent; the head is the embedding table.  Arrays are float64 by default,
so this is also the oracle for error budgets."""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def rms_normalise(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return rms_normalise(x, eps) * w


# ---- positions ---------------------------------------------------------------------------------------

def frequencies(rot: dict) -> np.ndarray:
    """One frequency per rotated pair: base^(-2i / dims), then, if `scaling` is given, stretched by
    wavelength: short waves stay, long waves are slowed by `factor`, and in between the two are blended."""
    dims = int(rot["dims"])
    f = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            out[i] = fi
        elif wave > original / low:
            out[i] = fi / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_pairs(x: np.ndarray, positions: np.ndarray, freq: np.ndarray) -> np.ndarray:
    """x: [n, ..., d]; entries 2i and 2i + 1 (i < len(freq)) turn by positions * freq[i]; the rest stay."""
    out = x.copy()
    shape = (len(positions),) + (1,) * (x.ndim - 2)
    for i, fi in enumerate(freq):
        a = (positions * fi).reshape(shape)
        c, s = np.cos(a), np.sin(a)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ---- softmax attention ---------------------------------------------------------------------------------

def visible(n: int, size) -> np.ndarray:
    """[n, n] booleans: query i sees key j iff 0 <= i - j (< size, if a size is given)."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    ok = j <= i
    if size:
        ok &= (i - j) < size
    return ok


def sink_softmax(scores: np.ndarray, mask: np.ndarray, sink: float) -> np.ndarray:
    """Softmax over the visible keys of each row whose denominator also holds exp(sink)."""
    s = np.where(mask, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def keys_as_values_attention(h: np.ndarray, w: dict, p: dict, eps: float) -> np.ndarray:
    """The left branch.  h: [n, width]; w: the branch's tensors by short name; p: its sizes and constants."""
    n = h.shape[0]
    H, G, dim = p["heads"], p["kv_heads"], p["dim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(n, H, dim)
    k = (h @ w["k"].T + w["k.b"]).reshape(n, G, dim)
    v = k.copy()                                        # the values: the keys as they were projected
    rot = p.get("rot")
    if rot and rot.get("dims"):
        f = frequencies(rot)
        pos = np.arange(n, dtype=np.float64)
        q, k = rotate_pairs(q, pos, f), rotate_pairs(k, pos, f)
    q, k = rms_normalise(q, eps), rms_normalise(k, eps)
    mask = visible(n, (p.get("mask") or {}).get("size"))
    out = np.zeros((n, H, dim))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * p["scale"]
        out[:, head] = sink_softmax(s, mask, float(w["sink"][head])) @ v[:, g]
    return out.reshape(n, H * dim) @ w["o"].T + w["o.b"]


def latent_attention(h: np.ndarray, w: dict, p: dict, eps: float) -> np.ndarray:
    n = h.shape[0]
    H, dim, rd, vdim, rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(n, H, dim + rd)
    dkv = h @ w["dkv"].T
    c = rms_norm(dkv[:, :rank], w["dkv.norm"], eps)
    f = frequencies(p["rot"])
    pos = np.arange(n, dtype=np.float64)
    kr = rotate_pairs(dkv[:, rank:], pos, f)                              # [n, rd], shared by the heads
    qr = rotate_pairs(q[:, :, dim:], pos, f)
    kp = (c @ w["uk"].T).reshape(n, H, dim)
    v = (c @ w["uv"].T).reshape(n, H, vdim)
    mask = visible(n, None)
    out = np.zeros((n, H, vdim))
    for head in range(H):
        s = (q[:, head, :dim] @ kp[:, head].T + qr[:, head] @ kr.T) * p["scale"]
        out[:, head] = sink_softmax(s, mask, float(w["sink"][head])) @ v[:, head]
    return out.reshape(n, H * vdim) @ w["o"].T


# ---- recurrences ---------------------------------------------------------------------------------------

def short_convolution(x: np.ndarray, taps: np.ndarray) -> np.ndarray:
    """x: [n, channels]; taps: [channels, m], the last column weighing the current token, the one before
    it the previous token and so on; what lies before the sequence's start is zero."""
    n, m = x.shape[0], taps.shape[1]
    y = np.zeros_like(x)
    for t in range(n):
        for j in range(m):
            src = t - (m - 1 - j)
            if src >= 0:
                y[t] += taps[:, j] * x[src]
    return y


def gated_delta_rule(h: np.ndarray, w: dict, p: dict, eps: float) -> np.ndarray:
    """The right branch, token by token."""
    n = h.shape[0]
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = silu(short_convolution(h @ w["q"].T, w["q.conv"])).reshape(n, G, dim)
    k = silu(short_convolution(h @ w["k"].T, w["k.conv"])).reshape(n, G, dim)
    v = silu(short_convolution(h @ w["v"].T, w["v.conv"])).reshape(n, H, vdim)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)                                           # [n, H]
    decay = np.exp(-np.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))   # [n, H]
    gate = silu(h @ w["g"].T).reshape(n, H, vdim)
    o = np.zeros((n, H, vdim))
    for head in range(H):
        g = head // (H // G)
        S = np.zeros((dim, vdim))
        for t in range(n):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, head] = S.T @ q[t, g]
    o = rms_normalise(o, eps) * w["norm"] * gate
    return o.reshape(n, H * vdim) @ w["o"].T


def lightning_attention(h: np.ndarray, w: dict, p: dict, eps: float) -> np.ndarray:
    n = h.shape[0]
    H, dim, vdim = p["heads"], p["dim"], p["vdim"]
    q = silu(h @ w["q"].T).reshape(n, H, dim)
    k = silu(h @ w["k"].T).reshape(n, H, dim)
    v = silu(h @ w["v"].T).reshape(n, H, vdim)
    o = np.zeros((n, H, vdim))
    for head in range(H):
        d = float(p["decay"][head])
        S = np.zeros((dim, vdim))
        for t in range(n):
            S = d * S + np.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_norm(o.reshape(n, H * vdim), w["norm"], eps) * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ---- layers and the model ------------------------------------------------------------------------------

def sub(w: dict, prefix: str) -> dict:
    return {k[len(prefix) + 1:]: v for k, v in w.items() if k.startswith(prefix + ".")}


def parallel_mixer(h, w, p, eps):
    return (p["left_scale"] * keys_as_values_attention(h, sub(w, "left"), p["left"], eps)
            + p["right_scale"] * gated_delta_rule(h, sub(w, "right"), p["right"], eps))


MIXERS = {"parallel": parallel_mixer, "lightning": lightning_attention, "latent_attention": latent_attention}


def swiglu(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def forward(config: dict, weights: dict, tokens, dtype=np.float64, streams_out=None) -> np.ndarray:
    """Logits [n, vocab] of one sequence.  `weights`: name -> array.  `streams_out`, a list, receives the
    residual stream after every layer."""
    w = {k: np.asarray(v, dtype=dtype) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)]
    for i, layer in enumerate(config["layers"]):
        lw = sub(w, f"l{i}")
        x = x + MIXERS[layer["type"]](rms_norm(x, lw["norm1"], eps), sub(lw, "mix"), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + swiglu(rms_norm(x, lw["norm2"], eps), sub(lw, "mlp"))
        if streams_out is not None:
            streams_out.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
