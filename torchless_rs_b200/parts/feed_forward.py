"""Dense SwiGLU feed-forward: down( silu(gate x) * (up x) )
(reference: src/model/modules/mlp.rs:23-45).  Gate and up rows are stacked into one
matrix at load time so that one product yields both and the SiLU-gate happens where
the product is written."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_feed_forward
from .runtime import Runtime


@register_feed_forward("swiglu")
class SwiGLU:
    """Parameters: `hidden_size`, `intermediate_size`; optionally `tensor_names`, the names of the
    gate, up and down matrices under the prefix (default: gate_proj.weight, up_proj.weight,
    down_proj.weight).  Interface of every
    feed-forward: `expected_tensors(spec, prefix)` (a class method), `load(weights)`, and `forward(xn, residual, batch)`,
    which adds its output to the 32-bit `residual` in place (or stores it there with `overwrite=True`,
    if the part says `can_overwrite`)."""
    graph_safe = True   # forward launches kernels whose arguments do not depend on host values
    can_overwrite = True
    DEFAULT_NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.prefix = prefix
        self.names = tuple(spec.params.get("tensor_names") or self.DEFAULT_NAMES)
        self.rt = rt
        self.matmul = Matmul(rt)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        gate, up, down = tuple(spec.params.get("tensor_names") or cls.DEFAULT_NAMES)
        return {
            f"{prefix}.{gate}": TensorSpec((i, h)),
            f"{prefix}.{up}": TensorSpec((i, h)),
            f"{prefix}.{down}": TensorSpec((h, i)),
        }

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up, down = self.names
        self.w_gate_up = self.rt.stack([weights[f"{p}.{gate}"], weights[f"{p}.{up}"]])
        self.w_down = self.rt.matrix(weights[f"{p}.{down}"])

    accepts_carry = True   # `xn` may be a NormCarry; `emit` may ask for the next norm's input

    def forward(self, xn, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        T = residual.shape[0]
        act = self.rt.workspace.get("ffn_act", (T, self.inter), self.rt.act_dtype)
        self.matmul(xn, self.w_gate_up, act, ops.MODE_SWIGLU)
        if overwrite:
            self.matmul(act, self.w_down, residual, ops.MODE_STORE_F32)
        else:
            self.matmul(act, self.w_down, residual, ops.MODE_ACCUM_F32, emit=emit)


@register_feed_forward("polynorm")
class PolyNormFeedForward:
    """down( act(up x) ) with act(z) = a N(z) + b N(z^2) + c N(z^3) + e: powers element by element,
    N the division of a token's vector by its root mean square (32-bit), and four learned numbers.
    Parameters: `hidden_size`, `intermediate_size`, `eps`.  Tensors under the prefix: up, down, act."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.eps = float(spec.params["eps"])
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return {f"{prefix}.up": TensorSpec((i, h)), f"{prefix}.down": TensorSpec((h, i)),
                f"{prefix}.act": TensorSpec((4,), init=(0.5, 0.3))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_up = self.rt.matrix(weights[f"{p}.up"])
        self.w_down = self.rt.matrix(weights[f"{p}.down"])
        self.coeff = weights[f"{p}.act"].to(device=self.rt.device, dtype=torch.float32).contiguous()

    def forward(self, xn, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        z = ws.get("ffn_pre", (T, self.inter), torch.float32)
        self.matmul(xn, self.w_up, z, ops.MODE_STORE_F32)
        act = ws.get("ffn_act", (T, self.inter), rt.act_dtype)
        rt.ops.poly_norm(z, self.coeff, self.eps, act)
        self.matmul(act, self.w_down, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)


@register_feed_forward("none")
class NoFeedForward:
    """A layer without a feed-forward: no tensors, and nothing is added."""
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        pass

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        return {}

    def load(self, weights) -> None:
        pass

    def forward(self, xn, residual, batch, emit=None) -> None:
        pass


@register_feed_forward("relu_squared")
class ReluSquaredFeedForward:
    """down( max(up x, 0)^2 ).  Parameters: `hidden_size`, `intermediate_size`.  Tensors under the prefix:
    up, down."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return {f"{prefix}.up": TensorSpec((i, h)), f"{prefix}.down": TensorSpec((h, i))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_up = self.rt.matrix(weights[f"{p}.up"])
        self.w_down = self.rt.matrix(weights[f"{p}.down"])

    def forward(self, xn, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        act = ws.get("ffn_act", (T, self.inter), rt.act_dtype)
        # the square of the relu in the product's epilogue, on the 32-bit sums, where the kernel has one
        if not self.matmul.activated(xn, self.w_up, act, ops.MODE_STORE_ACT, (ops.ACT_RELU_SQUARED,)):
            z = ws.get("ffn_pre", (T, self.inter), torch.float32)
            self.matmul(xn, self.w_up, z, ops.MODE_STORE_F32)
            rt.ops.relu_squared(z, act)
        self.matmul(act, self.w_down, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)
