"""Linear attention with a matrix state per head: gated linear attention, whose state decays per key
channel by a gate computed from the input, and lightning attention, whose decay is a constant of the
head.

Gated linear attention.

With h the mixer's input, per token and head (q, k, alpha of `dim` channels; v of `vdim`):
    q = W_q h * dim^(-1/2),  k = W_k h,  v = W_v h
    alpha = sigmoid(W_a2 (W_a1 h) + b_a2)^(1 / tau)          a low-rank map to one decay per key channel
    S <- diag(alpha) S + k v^T,   o = S^T q
each head's o is RMS-normed over its `vdim` entries with one weight vector shared by the heads, the
heads are concatenated, multiplied by silu(W_g h) and projected by W_o.  S starts at zero, is 32-bit
and is carried from token to token in the cache's per-sequence state (`StateRequest`), so a prompt
may come in any number of pieces.  q, k, v and the gate are one stacked product; the decay, its
logarithm and the state are computed in 32-bit by the scan kernel.

Lightning attention.  Per token and head, with d_head the head's constant decay:
    q = silu(W_q h),  k = silu(W_k h),  v = silu(W_v h)
    S <- d_head S + k v^T,   o = S^T q
the concatenated heads are RMS-normed together with one weight over the whole width, multiplied by
sigmoid(W_g h) and projected by W_o.  The same scan kernels run it: they are given the decays
themselves, one row [heads * dim] that serves every token."""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.requests import StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_mixer
from .runtime import Runtime


@register_mixer("gated_linear_attention")
class GatedLinearAttention:
    """Parameters: `hidden_size`, `heads`, `dim`, `vdim`, `tau`, `eps` (of the output norm), `rank`
    (the inner size of the decay's low-rank map; None: whatever the stored tensors have).
    Tensors under the prefix: q, k, v, g, o, norm, a1, a2, a2.b."""
    graph_safe = True
    can_overwrite = True
    state_attributes = ("state",)

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.tau = float(p["tau"])
        self.eps = float(p["eps"])
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)
        self.state = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, dim, vdim = int(p["hidden_size"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        rank = int(p["rank"]) if p.get("rank") else -1      # -1: any size, read from the stored tensor
        std = hidden ** -0.5
        return {
            f"{prefix}.q": TensorSpec((H * dim, hidden), init=(std, 0.0)),
            f"{prefix}.k": TensorSpec((H * dim, hidden), init=(std, 0.0)),
            f"{prefix}.v": TensorSpec((H * vdim, hidden), init=(std, 0.0)),
            f"{prefix}.g": TensorSpec((H * vdim, hidden), init=(std, 0.0)),
            f"{prefix}.o": TensorSpec((hidden, H * vdim), init=((H * vdim) ** -0.5, 0.0)),
            f"{prefix}.norm": TensorSpec((vdim,)),
            f"{prefix}.a1": TensorSpec((rank, hidden), init=(std, 0.0)),
            f"{prefix}.a2": TensorSpec((H * dim, rank), init=(0.5, 0.0)),
            f"{prefix}.a2.b": TensorSpec((H * dim,), init=(1.0, 2.0)),
        }

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        a1, a2 = weights[f"{p}.a1"], weights[f"{p}.a2"]
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{p}: a1 has {a1.shape[0]} rows but a2 has {a2.shape[1]} columns")
        self.rank = int(a1.shape[0])
        self.w_in = rt.stack([weights[f"{p}.q"], weights[f"{p}.k"], weights[f"{p}.v"], weights[f"{p}.g"]])
        self.w_a1 = rt.matrix(a1)
        self.w_a2 = rt.matrix(a2)
        self.w_o = rt.matrix(weights[f"{p}.o"])
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        self.a_bias = f32(weights[f"{p}.a2.b"])
        self.norm_w = f32(weights[f"{p}.norm"])

    def cache_request(self):
        return StateRequest((self.heads, self.dim, self.vdim), torch.float32)

    def bind_cache(self, view) -> None:
        self.state = view        # [slots, heads, dim, vdim]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        H, dim, vdim = self.heads, self.dim, self.vdim
        hd, hv = H * dim, H * vdim
        z = ws.get("gla_in", (T, 2 * hd + 2 * hv), torch.float32)
        self.matmul(xn, self.w_in, z, ops.MODE_STORE_F32)
        low = ws.get("gla_low", (T, self.rank), rt.act_dtype)
        self.matmul(xn, self.w_a1, low, ops.MODE_STORE_ACT)
        za = ws.get("gla_decay", (T, hd), torch.float32)
        self.matmul(low, self.w_a2, za, ops.MODE_STORE_F32)
        o = ws.get("gla_out", (T, hv), torch.float32)
        rt.ops.gla_scan(z[:, :hd], z[:, hd:2 * hd], z[:, 2 * hd:2 * hd + hv], za, self.a_bias, self.tau,
                        dim ** -0.5, self.state, o, batch.seq_start, batch.seq_slot, H, dim, vdim, workspace=ws)
        gated = ws.get("gla_gated", (T, hv), rt.act_dtype)
        rt.ops.headnorm_silu_gate(o, self.norm_w, self.eps, z[:, 2 * hd + hv:], gated, H, vdim)
        self.matmul(gated, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)


@register_mixer("lightning_attention")
class LightningAttention:
    """Parameters: `hidden_size`, `heads`, `dim`, `vdim`, `decay` (one number per head), `eps` (of the output
    norm).  Tensors under the prefix: q, k, v, g, o, norm [heads * vdim]."""
    graph_safe = True
    can_overwrite = True
    state_attributes = ("state",)

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.eps = float(p["eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays were given for {self.heads} heads")
        # one row of decays for every token: head h's number for each of its key channels
        self.decays = torch.tensor(decay, dtype=torch.float64).to(torch.float32).repeat_interleave(self.dim) \
            .reshape(1, self.heads * self.dim).contiguous().to(rt.device)
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)
        self.state = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, dim, vdim = int(p["hidden_size"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        std = hidden ** -0.5
        return {
            f"{prefix}.q": TensorSpec((H * dim, hidden), init=(std, 0.0)),
            f"{prefix}.k": TensorSpec((H * dim, hidden), init=(std, 0.0)),
            f"{prefix}.v": TensorSpec((H * vdim, hidden), init=(std, 0.0)),
            f"{prefix}.g": TensorSpec((H * vdim, hidden), init=(std, 0.0)),
            f"{prefix}.o": TensorSpec((hidden, H * vdim), init=((H * vdim) ** -0.5, 0.0)),
            f"{prefix}.norm": TensorSpec((H * vdim,)),
        }

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        self.w_in = rt.stack([weights[f"{p}.q"], weights[f"{p}.k"], weights[f"{p}.v"], weights[f"{p}.g"]])
        self.w_o = rt.matrix(weights[f"{p}.o"])
        self.norm_w = weights[f"{p}.norm"].to(device=rt.device, dtype=torch.float32).contiguous()

    def cache_request(self):
        return StateRequest((self.heads, self.dim, self.vdim), torch.float32)

    def bind_cache(self, view) -> None:
        self.state = view        # [slots, heads, dim, vdim]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        H, dim, vdim = self.heads, self.dim, self.vdim
        hd, hv = H * dim, H * vdim
        z = ws.get("lightning_in", (T, 2 * hd + 2 * hv), torch.float32)
        self.matmul(xn, self.w_in, z, ops.MODE_STORE_F32)
        rt.ops.silu_rows(z[:, :2 * hd + hv])
        o = ws.get("lightning_out", (T, hv), torch.float32)
        rt.ops.gla_scan(z[:, :hd], z[:, hd:2 * hd], z[:, 2 * hd:2 * hd + hv], self.decays, None, 1.0, 1.0,
                        self.state, o, batch.seq_start, batch.seq_slot, H, dim, vdim, workspace=ws, given=True)
        gated = ws.get("lightning_gated", (T, hv), rt.act_dtype)
        # one "head" of the whole width: the concatenated heads are normed together
        rt.ops.headnorm_silu_gate(o, self.norm_w, self.eps, z[:, 2 * hd + hv:], gated, 1, hv, sigmoid=True)
        self.matmul(gated, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)
