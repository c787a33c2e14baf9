"""Softmax attentions with grouped key/value heads whose queries and keys are rotated by position
on their first `rot_dims` entries (the pairing and the frequencies come from the layer's position
part), over the paged cache.

`differential_attention`: every head has two query/key maps over the same values,
    a_m = softmax_j(scale q_m,i . k_m,j) V      (m = 1, 2; causal)
    o = a_1 - lambda a_2,   out = o / sqrt(mean(o^2) + eps) * (1 - diff)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff      (one number for the layer)
The rows of W_q and W_k are laid out head by head as [map 1, map 2].  A key/value head's two key
vectors lie side by side in one row of the cache, and each map's query is a row of that width that is
zero in the other map's half, so the attention kernels see 2 H query heads over G key heads of
twice the size and read every key and every value once per group.

`gated_window_attention`: queries and keys are divided by their root mean square after the rotation,
    score = cap tanh(scale (q_i . k_j) / cap),   j visible iff 0 <= i - j < window
    out = sigmoid(W_g h) * concatenated heads     (entry by entry, h the mixer's input)

`sink_rotary_attention`: optionally biased projections, optionally no value projection at all (a
head's values are its keys as projected, bias included, before rotation and norm), queries and keys
divided by their root mean square after the rotation if asked,
    score = scale (q_i . k_j),   j visible iff 0 <= i - j < window,
    p(i, j) = exp(score(i, j)) / (sum over visible j' of exp(score(i, j')) + exp(sink_head))
    out = W_o (concatenated heads) + b_o

All: one stacked product for the projections of the input (32-bit), one kernel that rotates, norms
and writes q and the token's k and v into the pages, attention from pages only (so a position's
result does not depend on the step that computes it), a closing kernel, W_o.  Attention runs on the
kernels of the plain rotary attention where these take it (bfloat16, a key row as wide as a value row,
32, 64 or 128; with a cap only prompt steps and rows of 64 or 128), else on those of the windowed
attention with a cap."""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.requests import PagedKVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_mixer
from .runtime import Runtime
from .sink_attention import run_attention


class _RotaryAttention:
    graph_safe = True
    can_overwrite = True
    slots = 1            # query/key maps per head
    unit_norm = False    # q and k divided by their root mean square after the rotation
    plain_scores = True  # nothing but the keys enters the softmax (False: a sink does; the plain kernels are not built)
    proj_bias = None     # 32-bit, one number per column of the stacked projections (None: no bias)
    values_are_keys = False   # no value projection: a head's values are its keys as projected

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.rot = int(p.get("rot_dims") or 0)
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads cannot share {self.nkv} key/value heads")
        if self.rot % 2 or self.rot > self.dim:
            raise ValueError(f"{self.rot} rotated entries do not fit a query of {self.dim}")
        if self.rot and position is None:
            raise ValueError("rotated queries and keys need the layer's position part")
        if self.rot and position.inv_freq.numel() != self.rot // 2:
            raise ValueError("the position part's frequencies do not match the rotated entries")
        self.position = position
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)
        self.cache = None
        # scores without a cap over keys and values of one size are what the framework's plain
        # attention kernels compute (tensor-memory kernels for prompts, split keys for decode steps)
        self.fast = None
        if not rt.is_f32 and self.width == self.vdim and self.plain_scores:
            from ..csrc import attention_bf16
            if self.width in attention_bf16.FAST_HEAD_DIMS:
                self.fast = attention_bf16.AttentionBf16.get(self.width)

    @property
    def width(self) -> int:
        """Of a key row in the cache and of a query row."""
        return self.slots * self.dim

    def cache_request(self):
        return PagedKVRequest(self.nkv, self.width, self.window, v_head_dim=self.vdim)

    def bind_cache(self, view) -> None:
        self.cache = view

    def _project_and_write(self, xn, batch, cols: int):
        """z = the stacked projections (32-bit); q rotated (normed) in the activation type; k and v in the
        pages.  Returns (z, q)."""
        rt, ws, c = self.rt, self.rt.workspace, self.cache
        T = xn.shape[0]
        S, H, G = self.slots, self.nh, self.nkv
        z = ws.get("rot_attn_in", (T, cols), torch.float32)
        self.matmul(xn, self.w_in, z, ops.MODE_STORE_F32)
        q = ws.get("rot_attn_q", (T, H * S * self.width), rt.act_dtype)
        pos = self.position
        rt.ops.rotary_cache_write(z, pos.inv_freq if self.rot else None, self.rot, pos.style if self.rot else 0,
                                  self.unit_norm, self.eps, q, c.k_pages, c.v_pages, batch.token_pos,
                                  batch.token_seq, batch.seq_slot, c.page_table, H * S, G * S, G, self.dim,
                                  self.vdim, S, bias=self.proj_bias, values_are_keys=self.values_are_keys)
        return z, q

    def _attend(self, q, out, batch, softcap, sink=None):
        c = self.cache
        if self.fast is not None and sink is None:
            H = self.nh * self.slots
            if softcap is None:
                if self.fast.run(q, c, out, batch, H, self.nkv, self.window, self.scale, self.rt.workspace):
                    return
            elif self.fast.run_capped(q, c, out, batch, H, self.nkv, self.window, self.scale, softcap):
                return
        run_attention(self.rt.ops, q, c.k_pages, c.v_pages, None, sink, out, batch.token_pos, batch.token_seq,
                      batch.seq_slot, c.page_table, self.nh * self.slots, self.nkv, self.width, self.vdim,
                      self.window, 0, self.scale, softcap, batch, self.rt.workspace)


@register_mixer("differential_attention")
class DifferentialAttention(_RotaryAttention):
    """Parameters: `hidden_size`, `heads`, `kv_heads`, `dim` (of one map's query), `vdim`, `rot_dims`,
    `scale`, `diff`, `eps` (of the per-head norm).  Tensors under the prefix: q [heads * 2 * dim, hidden],
    k [kv_heads * 2 * dim, hidden], v, lq1, lk1, lq2, lk2 [dim], o."""
    slots = 2
    window = None

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        super().__init__(spec, prefix, rt, position)
        self.diff = float(spec.params["diff"])
        self.lam = 0.0

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, G, dim, vdim = (int(p[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        std = hidden ** -0.5
        out = {f"{prefix}.q": TensorSpec((H * 2 * dim, hidden), init=(std, 0.0)),
               f"{prefix}.k": TensorSpec((G * 2 * dim, hidden), init=(std, 0.0)),
               f"{prefix}.v": TensorSpec((G * vdim, hidden), init=(std, 0.0)),
               f"{prefix}.o": TensorSpec((hidden, H * vdim), init=((H * vdim) ** -0.5, 0.0))}
        for n in ("lq1", "lk1", "lq2", "lk2"):
            out[f"{prefix}.{n}"] = TensorSpec((dim,), init=(dim ** -0.5, 0.0))
        return out

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        self.w_in = rt.stack([weights[f"{p}.q"], weights[f"{p}.k"], weights[f"{p}.v"]])
        self.w_o = rt.matrix(weights[f"{p}.o"])
        # lambda depends on the weights only: 32-bit, once
        l = {n: weights[f"{p}.{n}"].to(torch.float32).cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
        one = torch.exp(torch.sum(l["lq1"] * l["lk1"])) - torch.exp(torch.sum(l["lq2"] * l["lk2"]))
        self.lam = float(one + torch.tensor(self.diff, dtype=torch.float32))

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        H, G, dim, vdim = self.nh, self.nkv, self.dim, self.vdim
        _, q = self._project_and_write(xn, batch, (H + G) * 2 * dim + G * vdim)
        maps = ws.get("rot_attn_maps", (T, H * 2 * vdim), rt.act_dtype)
        self._attend(q, maps, batch, None)
        out = ws.get("rot_attn_out", (T, H * vdim), rt.act_dtype)
        rt.ops.diff_heads(maps, self.lam, self.eps, 1.0 - self.diff, out, H, vdim)
        self.matmul(out, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)


@register_mixer("gated_window_attention")
class GatedWindowAttention(_RotaryAttention):
    """Parameters: `hidden_size`, `heads`, `kv_heads`, `dim`, `vdim`, `rot_dims`, `scale`, `softcap` (None: no
    cap), `window` (None: all keys), `eps` (of the query and key norms).  Tensors under the prefix: q, k, v,
    g [heads * vdim, hidden], o."""
    unit_norm = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        super().__init__(spec, prefix, rt, position)
        p = spec.params
        self.window = int(p["window"]) if p.get("window") else None
        self.softcap = float(p["softcap"]) if p.get("softcap") else None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, G, dim, vdim = (int(p[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        std = hidden ** -0.5
        return {f"{prefix}.q": TensorSpec((H * dim, hidden), init=(std, 0.0)),
                f"{prefix}.k": TensorSpec((G * dim, hidden), init=(std, 0.0)),
                f"{prefix}.v": TensorSpec((G * vdim, hidden), init=(std, 0.0)),
                f"{prefix}.g": TensorSpec((H * vdim, hidden), init=(std, 0.0)),
                f"{prefix}.o": TensorSpec((hidden, H * vdim), init=((H * vdim) ** -0.5, 0.0))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        self.w_in = rt.stack([weights[f"{p}.q"], weights[f"{p}.k"], weights[f"{p}.v"], weights[f"{p}.g"]])
        self.w_o = rt.matrix(weights[f"{p}.o"])

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        H, G, dim, vdim = self.nh, self.nkv, self.dim, self.vdim
        g_off = (H + G) * dim + G * vdim
        z, q = self._project_and_write(xn, batch, g_off + H * vdim)
        out = ws.get("rot_attn_out", (T, H * vdim), rt.act_dtype)
        self._attend(q, out, batch, self.softcap)
        rt.ops.sigmoid_gate(out, z[:, g_off:])
        self.matmul(out, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)


@register_mixer("sink_rotary_attention")
class SinkRotaryAttention(_RotaryAttention):
    """Parameters: `hidden_size`, `heads`, `kv_heads`, `dim`, `vdim`, `rot_dims`, `scale`, `window` (None: all
    keys), `eps` (of the query and key norms), `unit_norm` (queries and keys divided by their root mean square
    after the rotation), `sink` (a learned logit per head in the denominator), `bias` (q, k, v and o have
    biases, stored under the tensor's name with `.b`), `values_are_keys` (no v: `vdim` must equal `dim`).
    Tensors under the prefix: q, k, [v], o, [q.b, k.b, v.b, o.b], [sink].

    `output_bias` is the output projection's bias (or None); `forward(..., defer_bias=True)` leaves it out, for
    a caller that adds it where it sums this mixer's output with others'."""

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.unit_norm = bool(p.get("unit_norm", False))
        self.values_are_keys = bool(p.get("values_are_keys", False))
        self.plain_scores = not bool(p.get("sink", False))
        super().__init__(spec, prefix, rt, position)
        self.window = int(p["window"]) if p.get("window") else None
        self.has_sink = bool(p.get("sink", False))
        self.has_bias = bool(p.get("bias", False))
        if self.values_are_keys and self.vdim != self.dim:
            raise ValueError(f"values that are the keys have the keys' size {self.dim}, not {self.vdim}")
        self.sink = None
        self.output_bias = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, G, dim, vdim = (int(p[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        std = hidden ** -0.5
        out = {f"{prefix}.q": TensorSpec((H * dim, hidden), init=(std, 0.0)),
               f"{prefix}.k": TensorSpec((G * dim, hidden), init=(std, 0.0)),
               f"{prefix}.o": TensorSpec((hidden, H * vdim), init=((H * vdim) ** -0.5, 0.0))}
        if not p.get("values_are_keys"):
            out[f"{prefix}.v"] = TensorSpec((G * vdim, hidden), init=(std, 0.0))
        if p.get("bias"):
            out[f"{prefix}.q.b"] = TensorSpec((H * dim,), init=(0.1, 0.0))
            out[f"{prefix}.k.b"] = TensorSpec((G * dim,), init=(0.1, 0.0))
            out[f"{prefix}.o.b"] = TensorSpec((hidden,), init=(0.1, 0.0))
            if not p.get("values_are_keys"):
                out[f"{prefix}.v.b"] = TensorSpec((G * vdim,), init=(0.1, 0.0))
        if p.get("sink"):
            out[f"{prefix}.sink"] = TensorSpec((H,), init=(1.0, 0.0))
        return out

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        names = ["q", "k"] + ([] if self.values_are_keys else ["v"])
        self.w_in = rt.stack([weights[f"{p}.{n}"] for n in names])
        self.w_o = rt.matrix(weights[f"{p}.o"])
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        if self.has_bias:
            self.proj_bias = torch.cat([f32(weights[f"{p}.{n}.b"]) for n in names])
            self.output_bias = f32(weights[f"{p}.o.b"])
        if self.has_sink:
            self.sink = f32(weights[f"{p}.sink"])

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False,
                defer_bias: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        H, G, dim, vdim = self.nh, self.nkv, self.dim, self.vdim
        cols = (H + G) * dim + (0 if self.values_are_keys else G * vdim)
        _, q = self._project_and_write(xn, batch, cols)
        out = ws.get("rot_attn_out", (T, H * vdim), rt.act_dtype)
        self._attend(q, out, batch, None, sink=self.sink)
        if self.output_bias is None or defer_bias:
            self.matmul(out, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)
            return
        y = residual if overwrite else ws.get("rot_attn_proj", (T, self.hidden), torch.float32)
        self.matmul(out, self.w_o, y, ops.MODE_STORE_F32)
        rt.ops.weighted_sum([y], [self.output_bias], [1.0], residual, accumulate=not overwrite)
