"""The gated delta rule: a matrix state per head that decays by one number per token and head and is
corrected towards the token's value, fed through short causal convolutions.

With h the mixer's input, per token (q, k of `kv_heads` x `dim`; v of `heads` x `vdim`; value head n
reads the query/key head n // (heads / kv_heads)):
    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     conv: over the last `conv` tokens
                                                                           of each channel, zeros before
                                                                           the sequence's start
    q <- q / sqrt(sum q^2 + unit_eps) / sqrt(dim),   k <- k / sqrt(sum k^2 + unit_eps)    (per head)
    beta = sigmoid(W_b h),   g = exp(-exp(A_log) softplus(W_a h + dt_bias))                (per value head)
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
each head's o is RMS-normed over its `vdim` entries with one weight vector shared by the heads,
multiplied by silu(W_g h), the heads are concatenated and projected by W_o.  S starts at zero, is
32-bit and is carried from token to token in the cache's per-sequence state together with the
convolutions' last `conv` - 1 inputs (two `StateRequest`s), so a prompt may come in any number of
pieces.  All six projections of h are one stacked product; convolution, activations, unit norms, gates,
decay and the walk over the tokens are 32-bit."""
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


@register_mixer("gated_delta_rule")
class GatedDeltaRule:
    """Parameters: `hidden_size`, `heads`, `kv_heads`, `dim`, `vdim`, `conv` (taps), `eps` (of the output
    norm), `unit_eps` (inside the root of the unit norms of q and k).
    Tensors under the prefix: q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, g, norm, o."""
    graph_safe = True
    can_overwrite = True
    state_attributes = ("state", "kept")

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.taps = int(p["conv"])
        self.eps = float(p["eps"])
        self.unit_eps = float(p["unit_eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} value heads cannot share {self.kv_heads} query/key heads")
        if self.taps < 1:
            raise ValueError("a convolution needs at least one tap")
        self.channels = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)
        self.state = None
        self.kept = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, G, dim, vdim, taps = (int(p[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim", "conv"))
        std = hidden ** -0.5
        return {
            f"{prefix}.q": TensorSpec((G * dim, hidden), init=(std, 0.0)),
            f"{prefix}.q.conv": TensorSpec((G * dim, taps), init=(0.5, 0.0)),
            f"{prefix}.k": TensorSpec((G * dim, hidden), init=(std, 0.0)),
            f"{prefix}.k.conv": TensorSpec((G * dim, taps), init=(0.5, 0.0)),
            f"{prefix}.v": TensorSpec((H * vdim, hidden), init=(std, 0.0)),
            f"{prefix}.v.conv": TensorSpec((H * vdim, taps), init=(0.5, 0.0)),
            f"{prefix}.b": TensorSpec((H, hidden), init=(std, 0.0)),
            f"{prefix}.a": TensorSpec((H, hidden), init=(std, 0.0)),
            f"{prefix}.A_log": TensorSpec((H,), init=(0.5, -1.0)),
            f"{prefix}.dt_bias": TensorSpec((H,), init=(0.5, 0.0)),
            f"{prefix}.g": TensorSpec((H * vdim, hidden), init=(std, 0.0)),
            f"{prefix}.norm": TensorSpec((vdim,)),
            f"{prefix}.o": TensorSpec((hidden, H * vdim), init=((H * vdim) ** -0.5, 0.0)),
        }

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        self.w_in = rt.stack([weights[f"{p}.{n}"] for n in ("q", "k", "v", "g", "b", "a")])
        self.w_o = rt.matrix(weights[f"{p}.o"])
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        self.taps_w = torch.cat([f32(weights[f"{p}.{n}.conv"]) for n in ("q", "k", "v")]).contiguous()
        self.neg_a = -torch.exp(f32(weights[f"{p}.A_log"]))       # the decay's rate, 32-bit, once
        self.dt_bias = f32(weights[f"{p}.dt_bias"])
        self.norm_w = f32(weights[f"{p}.norm"])

    def cache_request(self):
        return (StateRequest((self.heads, self.dim, self.vdim), torch.float32),
                StateRequest((max(self.taps - 1, 1), self.channels), torch.float32))

    def bind_cache(self, views) -> None:
        self.state, self.kept = views       # [slots, heads, dim, vdim], [slots, taps - 1, channels]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        H, G, dim, vdim, C = self.heads, self.kv_heads, self.dim, self.vdim, self.channels
        hv = H * vdim
        z = ws.get("delta_in", (T, C + hv + 2 * H), torch.float32)
        self.matmul(xn, self.w_in, z, ops.MODE_STORE_F32)
        y = ws.get("delta_qkv", (T, C), torch.float32)
        gates = ws.get("delta_gates", (T, 2 * H + G), torch.float32)
        kept = self.kept[:, :self.taps - 1]
        rt.ops.delta_prep(z, self.taps_w, kept, y, gates, self.neg_a, self.dt_bias, C + hv, C + hv + H,
                          batch.token_seq, batch.seq_start, batch.seq_slot, G, H, dim, vdim, self.unit_eps,
                          dim ** -0.5)
        if self.taps > 1:
            rt.ops.conv_state_update(z, kept, batch.seq_start, batch.seq_slot, C)
        o = ws.get("delta_out", (T, hv), torch.float32)
        rt.ops.delta_scan(y, gates, self.state, o, batch.seq_start, batch.seq_slot, G, H, dim, vdim)
        gated = ws.get("delta_gated", (T, hv), rt.act_dtype)
        rt.ops.headnorm_silu_gate(o, self.norm_w, self.eps, z[:, C:C + hv], gated, H, vdim)
        self.matmul(gated, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)
