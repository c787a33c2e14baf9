"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, computed in 32-bit
(reference: src/kernels/mod.rs:558-568, src/model/modules/rmsnorm.rs:6-25)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .registry import register_norm
from .runtime import Runtime


@register_norm("rmsnorm")
class RMSNorm:
    """Parameters: `size`, `eps`; optionally `bare_name` (the weight is stored under the norm's own name,
    without `.weight`).  Interface of every norm: `expected_tensors(spec, prefix)` (a class method),
    `load(weights)`, and `__call__(x, out, rows=None)` from the 32-bit stream to an
    activation tensor; `rows` (int32, on the device) picks input rows."""

    foldable = True   # x / rms * w with a plain weight: the products around it can take it over

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = prefix if spec.params.get("bare_name") else f"{prefix}.weight"
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        name = prefix if spec.params.get("bare_name") else f"{prefix}.weight"
        return {name: TensorSpec((int(spec.params["size"]),))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        self.weight = self.rt.vector(weights[self.name])

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out


@register_norm("rmsnorm_scalar")
class ScalarRMSNorm:
    """y = x / sqrt(mean(x^2) + eps) * g with one number g for all coordinates.  Parameters: `size`,
    `eps`.  Its tensor is a single number stored under the norm's own name (no `.weight`).

    Besides the interface of every norm it offers `gain` (g as a 32-bit tensor of one element on
    the device), which a block that normalises a branch's output reads."""

    foldable = False

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = prefix
        self.rt = rt
        self.gain: Optional[torch.Tensor] = None
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        return {prefix: TensorSpec((), init=(0.1, 1.0))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        self.gain = weights[self.name].reshape(1).to(device=self.rt.device, dtype=torch.float32)
        self.weight = self.gain.expand(self.size).contiguous()   # what the row kernel reads

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out


@register_norm("rmsnorm_one_plus")
class OnePlusRMSNorm:
    """y = x / sqrt(mean(x^2) + eps) * (1 + w): the stored weight lies around zero.  Parameters:
    `size`, `eps`.  Its tensor is stored under the norm's own name (no `.weight`).  `weight` is
    the 32-bit factor 1 + w, which is what the row kernel and the stream kernels multiply by."""

    foldable = False

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = prefix
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        return {prefix: TensorSpec((int(spec.params["size"]),), init=(0.1, 0.0))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        w = weights[self.name].to(device=self.rt.device, dtype=torch.float32)
        self.weight = (w + 1.0).contiguous()

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out
