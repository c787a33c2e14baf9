"""Plain, slow restatement of the Rupasun decoder, for tests only: numpy, whole sequences, no
cache, one function per mechanism.  It shares no code with the package under test.

The design in short.  A layer wraps each sublayer in two norms:
    x <- x + N_1b(mixer(N_1(x)));   x <- x + N_2b(ff(N_2(x)))          N: RMS norm with a weight
A layer's mixer is one of two kinds of softmax attention with grouped key/value heads:
  * differential attention: every head has two query/key maps over the same values, rotated
    (half-split pairs) on their first `rot.dims` entries; the second map's output, times one number
    per layer, is subtracted from the first's, and the difference is RMS-normed per head (no weight)
    and multiplied by 1 - diff;
  * windowed attention: rotation of interleaved pairs, queries and keys divided by their root mean
    square after the rotation, tanh-capped scores, a sliding window, and a sigmoid gate per output
    entry computed from the mixer's input.
The feed-forward is dense with a squared relu, or a mixture of clamped, gated experts chosen by
sigmoid scores among the experts of the best groups, plus a shared expert; or absent.
Arrays are float64 by default, so this is also the oracle for error budgets."""
from __future__ import annotations

import numpy as np

GATE_ALPHA = 1.702


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_normalise(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return rms_normalise(x, eps) * w


def rotate(x: np.ndarray, positions: np.ndarray, dims: int, base: float, interleaved: bool) -> np.ndarray:
    """x: [n, heads, size].  The first `dims` entries of every head are turned by the angle
    position * base^(-2i/dims) in pairs (i, i + dims/2), or (2i, 2i + 1) if `interleaved`; the rest pass."""
    out = x.copy()
    if not dims:
        return out
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    a = positions[:, None, None] * freq[None, None, :]
    c, s = np.cos(a), np.sin(a)
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def visible(positions: np.ndarray, size) -> np.ndarray:
    """[n, n] booleans: query i sees key j iff 0 <= i - j (< size, if there is a window)."""
    d = positions[:, None] - positions[None, :]
    return (d >= 0) & ((d < size) if size else True)


def softmax_rows(scores: np.ndarray, mask: np.ndarray) -> np.ndarray:
    s = np.where(mask, scores, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def difference_factor(w: dict, diff: float) -> float:
    """The number by which the second map's output is multiplied before it is subtracted."""
    return float(np.exp(np.sum(w["lq1"] * w["lk1"])) - np.exp(np.sum(w["lq2"] * w["lk2"])) + diff)


def differential_attention(h: np.ndarray, w: dict, p: dict, eps: float, positions=None) -> np.ndarray:
    """h: [n, width]; w: the mixer's tensors by short name; p: its sizes and constants."""
    n = h.shape[0]
    positions = np.arange(n, dtype=np.float64) if positions is None else positions
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    rot = p.get("rot") or {"dims": 0, "base": 1.0}
    # rows head by head, within a head map 1 then map 2: [n, heads * 2, dim]
    q = rotate((h @ w["q"].T).reshape(n, H * 2, dim), positions, rot["dims"], rot["base"], False).reshape(n, H, 2, dim)
    k = rotate((h @ w["k"].T).reshape(n, G * 2, dim), positions, rot["dims"], rot["base"], False).reshape(n, G, 2, dim)
    v = (h @ w["v"].T).reshape(n, G, vdim)
    mask = visible(positions, None)
    lam = difference_factor(w, p["diff"])
    out = np.zeros((n, H, vdim))
    for head in range(H):
        g = head // (H // G)
        a = [softmax_rows((q[:, head, m] @ k[:, g, m].T) * p["scale"], mask) @ v[:, g] for m in (0, 1)]
        out[:, head] = rms_normalise(a[0] - lam * a[1], eps) * (1.0 - p["diff"])
    return out.reshape(n, H * vdim) @ w["o"].T


def window_attention(h: np.ndarray, w: dict, p: dict, eps: float, positions=None) -> np.ndarray:
    n = h.shape[0]
    positions = np.arange(n, dtype=np.float64) if positions is None else positions
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    rot = p.get("rot") or {"dims": 0, "base": 1.0}
    q = rms_normalise(rotate((h @ w["q"].T).reshape(n, H, dim), positions, rot["dims"], rot["base"], True), eps)
    k = rms_normalise(rotate((h @ w["k"].T).reshape(n, G, dim), positions, rot["dims"], rot["base"], True), eps)
    v = (h @ w["v"].T).reshape(n, G, vdim)
    mask = visible(positions, (p.get("mask") or {}).get("size"))
    cap = p.get("softcap")
    out = np.zeros((n, H, vdim))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * p["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        out[:, head] = softmax_rows(s, mask) @ v[:, g]
    return (out.reshape(n, H * vdim) * sigmoid(h @ w["g"].T)) @ w["o"].T


def dense_ff(h: np.ndarray, w: dict) -> np.ndarray:
    return (np.maximum(h @ w["up"].T, 0.0) ** 2) @ w["down"].T


def expert(h: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray, limit: float) -> np.ndarray:
    """A clamped, gated expert: g is bounded above, u on both sides, and u enters as u + 1."""
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(GATE_ALPHA * g) * (u + 1.0)) @ down.T


def route(scores: np.ndarray, top: int, groups: int, keep: int):
    """scores: [experts] of one token.  Returns (chosen indices, by falling score; allowed experts)."""
    E = scores.shape[0]
    size = E // groups
    per_group = scores.reshape(groups, size)
    group_score = np.sort(per_group, axis=1)[:, ::-1][:, :2].sum(axis=1)
    best = np.argsort(-group_score, kind="stable")[:keep]
    allowed = np.zeros(E, bool)
    for g in best:
        allowed[g * size:(g + 1) * size] = True
    masked = np.where(allowed, scores, -np.inf)
    return np.argsort(-masked, kind="stable")[:top], allowed


def route_margin(scores: np.ndarray, top: int, groups: int, keep: int) -> float:
    """How far the scores of one token are from another choice: the smaller of the gap between the last
    kept and the first dropped group's score (halved: it is a sum of two scores) and the gap between the
    last chosen and the first not chosen score among the allowed experts."""
    E = scores.shape[0]
    _, allowed = route(scores, top, groups, keep)
    margin = np.inf
    if keep < groups:
        g = np.sort(np.sort(scores.reshape(groups, E // groups), axis=1)[:, ::-1][:, :2].sum(axis=1))[::-1]
        margin = min(margin, (g[keep - 1] - g[keep]) / 2.0)
    if top < allowed.sum():
        a = np.sort(scores[allowed])[::-1]
        margin = min(margin, a[top - 1] - a[top])
    return float(margin)


def expert_ff(h: np.ndarray, w: dict, p: dict, margins: list | None = None) -> np.ndarray:
    """`margins`, if given, receives one array [n] of `route_margin` per call."""
    r, e = p["router"], p["expert"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = sigmoid(h @ w["router"].T)
    if margins is not None:
        margins.append(np.array([route_margin(s[t], r["top"], groups["count"], groups["keep"]) for t in range(h.shape[0])]))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, _ = route(s[t], r["top"], groups["count"], groups["keep"])
        weights = s[t, chosen] / (s[t, chosen].sum() + 1e-20) * r.get("scale", 1.0)
        for c, wt in zip(chosen, weights):
            out[t] += wt * expert(h[t:t + 1], w[f"e{c}.gate"], w[f"e{c}.up"], w[f"e{c}.down"], e["limit"])[0]
    sh = p.get("shared")
    if sh:
        out += expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], sh["limit"])
    return out


def feed_forward(h: np.ndarray, w: dict, p: dict, margins: list | None = None) -> np.ndarray:
    return dense_ff(h, w) if p["kind"] == "dense" else expert_ff(h, w, p, margins)


MIXERS = {"attention": differential_attention, "attention_2": window_attention}


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, return_layers: bool = False, dtype=np.float64, margins: list | None = None):
    """Logits [n, vocab] of one sequence from its first token (and the stream after every layer).
    `margins` receives every expert layer's `route_margin` per position."""
    W = {k: np.asarray(v, dtype=dtype) if np.asarray(v).dtype.kind == "f" else np.asarray(v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    streams = []
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[l["type"]](norm(x, W[p + "norm1"], eps), sub(W, p + "mix."), l["mixer"], eps)
        x = x + norm(y, W[p + "norm1b"], eps)
        if l.get("mlp"):
            y = feed_forward(norm(x, W[p + "norm2"], eps), sub(W, p + "mlp."), l["mlp"], margins)
            x = x + norm(y, W[p + "norm2b"], eps)
        streams.append(x.copy())
    logits = norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
