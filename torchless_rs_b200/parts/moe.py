"""Mixture of experts with clamped, gated experts and router outputs that hand the input through.

    z = W_router h (32-bit),  s = softmax(z) over all `experts + identity` outputs
    chosen: the `top` outputs with the largest s + correction;  their weights: s (not renormalised)
    expert e < experts:  g = min(W_gate,e h, limit),  u = clamp(W_up,e h, -limit, limit),
                         y_e = W_down,e ( g * sigmoid(gate_alpha * g) * (u + 1) )
    expert e >= experts: y_e = h
    output = sum over the chosen of weight * y_e
The (token, expert) pairs are grouped by expert on the device; the experts' products run over the
groups (no host value is read, so decode steps replay from CUDA graphs)."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_feed_forward
from .runtime import Runtime


@register_feed_forward("moe_clamped")
class ClampedMoE:
    """Parameters: `hidden_size`, `ff` (an expert's inner size), `experts`, `identity`, `top`, `limit`,
    `gate_alpha` (default 1.702).  Tensors under the prefix: e<i>.gate, e<i>.up, e<i>.down for
    i < experts; router [experts + identity, hidden]; correction [experts + identity]."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        p = spec.params
        self.hidden, self.ff = int(p["hidden_size"]), int(p["ff"])
        self.experts, self.identity, self.top = int(p["experts"]), int(p.get("identity") or 0), int(p["top"])
        self.limit = float(p["limit"])
        self.gate_alpha = float(p.get("gate_alpha", 1.702))
        if not 1 <= self.top <= self.experts + self.identity:
            raise ValueError("a token cannot choose more experts than there are")
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        h, f, E, I = int(p["hidden_size"]), int(p["ff"]), int(p["experts"]), int(p.get("identity") or 0)
        out = {f"{prefix}.router": TensorSpec((E + I, h), init=(h ** -0.5, 0.0)),
               f"{prefix}.correction": TensorSpec((E + I,), init=(0.02, 0.0))}
        for e in range(E):
            out[f"{prefix}.e{e}.gate"] = TensorSpec((f, h), init=(h ** -0.5, 0.0))
            out[f"{prefix}.e{e}.up"] = TensorSpec((f, h), init=(h ** -0.5, 0.0))
            out[f"{prefix}.e{e}.down"] = TensorSpec((h, f), init=(f ** -0.5, 0.0))
        return out

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt, E = self.prefix, self.rt, self.experts
        # per expert the gate rows, then the up rows: [experts, 2 ff, hidden]
        self.w_up = rt.stack([weights[f"{p}.e{e}.{n}"] for e in range(E) for n in ("gate", "up")]) \
            .view(E, 2 * self.ff, self.hidden) if E else None
        self.w_down = rt.stack([weights[f"{p}.e{e}.down"] for e in range(E)]).view(E, self.hidden, self.ff) \
            if E else None
        self.w_router = rt.matrix(weights[f"{p}.router"])
        self.correction = weights[f"{p}.correction"].to(device=rt.device, dtype=torch.float32).contiguous()

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T, E, top = residual.shape[0], self.experts, self.top
        z = ws.get("moe_logits", (T, E + self.identity), torch.float32)
        self.matmul(xn, self.w_router, z, ops.MODE_STORE_F32)
        idx = ws.get("moe_idx", (T, top), torch.int32)
        wt = ws.get("moe_wt", (T, top), torch.float32)
        rt.ops.moe_route(z, self.correction, top, idx, wt)
        offsets = ws.get("moe_offsets", (E + 1,), torch.int32)
        row_token = ws.get("moe_row_token", (T * top,), torch.int32)
        row_of = ws.get("moe_row_of", (T, top), torch.int32)
        rt.ops.moe_plan(idx, E, offsets, row_token, row_of)
        yk = ws.get("moe_expert_out", (T * top, self.hidden), torch.float32)
        if E:
            act = ws.get("moe_act", (T * top, self.ff), rt.act_dtype)
            rt.ops.moe_gemm(xn, row_token, self.w_up, act, offsets, up=True, limit=self.limit,
                            alpha=self.gate_alpha)
            rt.ops.moe_gemm(act, None, self.w_down, yk, offsets, up=False)
        rt.ops.moe_combine(yk, row_of, wt, xn, residual, accumulate=not overwrite)


@register_feed_forward("moe_grouped_sigmoid")
class GroupedSigmoidMoE:
    """Clamped, gated experts (the form above) chosen by sigmoid scores among the experts of the best
    groups, plus an optional shared expert that every token uses.

        s = sigmoid(W_router h) (32-bit).  The experts form `groups` equal groups of neighbours; a group's
        score is the sum of its two largest s; only experts of the `keep` best groups can be chosen; the
        `top` largest s among them are chosen, with weights s / (sum of the chosen s + 1e-20) * route_scale.
        output = sum over the chosen of weight * expert(h)  +  shared(h)

    Parameters: `hidden_size`, `ff`, `experts`, `top`, `limit`, `groups`, `keep`, `route_scale`,
    `gate_alpha` (default 1.702), `shared_ff` (None: no shared expert), `shared_limit`.  Tensors under the
    prefix: e<i>.gate, e<i>.up, e<i>.down, router [experts, hidden], shared.gate, shared.up, shared.down.
    The chosen experts' products run over (token, expert) pairs grouped by expert on the device, the
    shared expert's through the plain product kernels."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        p = spec.params
        self.hidden, self.ff = int(p["hidden_size"]), int(p["ff"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        self.limit = float(p["limit"])
        self.groups, self.keep = int(p.get("groups") or 1), int(p.get("keep") or 1)
        self.route_scale = float(p.get("route_scale", 1.0))
        self.gate_alpha = float(p.get("gate_alpha", 1.702))
        self.shared_ff = int(p["shared_ff"]) if p.get("shared_ff") else None
        self.shared_limit = float(p.get("shared_limit") or 0.0)
        if self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.experts} experts do not form {self.groups} equal groups of which "
                             f"{self.keep} are kept")
        if not 1 <= self.top <= self.keep * (self.experts // self.groups):
            raise ValueError("a token cannot choose more experts than the kept groups hold")
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        h, f, E = int(p["hidden_size"]), int(p["ff"]), int(p["experts"])
        out = {f"{prefix}.router": TensorSpec((E, h), init=(h ** -0.5, 0.0))}
        for e in range(E):
            out[f"{prefix}.e{e}.gate"] = TensorSpec((f, h), init=(h ** -0.5, 0.0))
            out[f"{prefix}.e{e}.up"] = TensorSpec((f, h), init=(h ** -0.5, 0.0))
            out[f"{prefix}.e{e}.down"] = TensorSpec((h, f), init=(f ** -0.5, 0.0))
        if p.get("shared_ff"):
            sf = int(p["shared_ff"])
            out[f"{prefix}.shared.gate"] = TensorSpec((sf, h), init=(h ** -0.5, 0.0))
            out[f"{prefix}.shared.up"] = TensorSpec((sf, h), init=(h ** -0.5, 0.0))
            out[f"{prefix}.shared.down"] = TensorSpec((h, sf), init=(sf ** -0.5, 0.0))
        return out

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt, E = self.prefix, self.rt, self.experts
        self.w_up = rt.stack([weights[f"{p}.e{e}.{n}"] for e in range(E) for n in ("gate", "up")]) \
            .view(E, 2 * self.ff, self.hidden)
        self.w_down = rt.stack([weights[f"{p}.e{e}.down"] for e in range(E)]).view(E, self.hidden, self.ff)
        self.w_router = rt.matrix(weights[f"{p}.router"])
        if self.shared_ff:
            self.w_shared_up = rt.stack([weights[f"{p}.shared.gate"], weights[f"{p}.shared.up"]])
            self.w_shared_down = rt.matrix(weights[f"{p}.shared.down"])

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T, E, top = residual.shape[0], self.experts, self.top
        z = ws.get("moe_logits", (T, E), torch.float32)
        self.matmul(xn, self.w_router, z, ops.MODE_STORE_F32)
        idx = ws.get("moe_idx", (T, top), torch.int32)
        wt = ws.get("moe_wt", (T, top), torch.float32)
        rt.ops.moe_route_grouped(z, self.groups, self.keep, top, self.route_scale, idx, wt)
        offsets = ws.get("moe_offsets", (E + 1,), torch.int32)
        row_token = ws.get("moe_row_token", (T * top,), torch.int32)
        row_of = ws.get("moe_row_of", (T, top), torch.int32)
        rt.ops.moe_plan(idx, E, offsets, row_token, row_of)
        yk = ws.get("moe_expert_out", (T * top, self.hidden), torch.float32)
        act = ws.get("moe_act", (T * top, self.ff), rt.act_dtype)
        rt.ops.moe_gemm(xn, row_token, self.w_up, act, offsets, up=True, limit=self.limit, alpha=self.gate_alpha)
        rt.ops.moe_gemm(act, None, self.w_down, yk, offsets, up=False)
        rt.ops.moe_combine(yk, row_of, wt, xn, residual, accumulate=not overwrite)
        if self.shared_ff:
            sact = ws.get("moe_shared_act", (T, self.shared_ff), rt.act_dtype)
            if not self.matmul.activated(xn, self.w_shared_up, sact, ops.MODE_SWIGLU,
                                         (ops.ACT_CLAMPED_GLU, self.shared_limit, self.gate_alpha)):
                zs = ws.get("moe_shared_pre", (T, 2 * self.shared_ff), torch.float32)
                self.matmul(xn, self.w_shared_up, zs, ops.MODE_STORE_F32)
                rt.ops.clamped_glu(zs, self.shared_limit, self.gate_alpha, sact)
            self.matmul(sact, self.w_shared_down, residual, ops.MODE_ACCUM_F32)
