"""A mixer made of several mixers side by side: every branch reads the same input.  Two ways of
joining them (`combine`):
  "norm_mean" (the default): each branch's output is RMS-normed over the model width with a weight
    vector of its own, and the result is the mean of the normed outputs,
    y = (1 / n) sum_b  norm_b(branch_b(h)),   norm_b(z) = z / sqrt(mean(z^2) + eps) * w_b
  "weighted_sum": y = sum_b scale_b branch_b(h), one constant factor per branch and no tensors of the
    mixer's own.
The branches are registered mixers of any kind; each keeps its own cache or state, so the mixer asks
the cache for a tuple of requests and is bound to a tuple of views."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .registry import lookup, register_mixer
from .runtime import Runtime


@register_mixer("parallel")
class ParallelMixer:
    """Parameters: `hidden_size`, `eps`, `branches` = ((name, PartSpec), ...), at most four; `combine`
    and, for "weighted_sum", `scales` (one number per branch).  Tensors: those of branch b under
    `<prefix>.<name_b>`, and, for "norm_mean", its output norm's weight `<prefix>.<name_b>.out` [hidden]."""
    can_overwrite = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        self.hidden = int(spec.params["hidden_size"])
        self.eps = float(spec.params.get("eps", 0.0))
        self.combine = spec.params.get("combine", "norm_mean")
        if self.combine not in ("norm_mean", "weighted_sum"):
            raise ValueError(f"a parallel mixer joins its branches by 'norm_mean' or 'weighted_sum', not '{self.combine}'")
        self.scales = [float(x) for x in spec.params.get("scales", ())]
        self.prefix = prefix
        self.rt = rt
        self.names = [n for n, _ in spec.params["branches"]]
        if not 1 <= len(self.names) <= 4:
            raise ValueError("a parallel mixer takes one to four branches")
        if self.combine == "weighted_sum" and len(self.scales) != len(self.names):
            raise ValueError("a weighted sum of branches needs one factor per branch")
        self.branches = [lookup("mixer", ps.kind)(ps, f"{prefix}.{n}", rt, position=position)
                         for n, ps in spec.params["branches"]]
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        self.out_weights = []

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for n, ps in spec.params["branches"]:
            out.update(lookup("mixer", ps.kind).expected_tensors(ps, f"{prefix}.{n}"))
            if spec.params.get("combine", "norm_mean") == "norm_mean":
                out[f"{prefix}.{n}.out"] = TensorSpec((int(spec.params["hidden_size"]),))
        return out

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        for b in self.branches:
            b.load(weights)
        if self.combine != "norm_mean":
            return
        self.out_weights = [weights[f"{self.prefix}.{n}.out"].to(device=self.rt.device, dtype=torch.float32)
                            .contiguous() for n in self.names]

    def cache_request(self):
        return tuple(b.cache_request() for b in self.branches)

    def bind_cache(self, views) -> None:
        for b, v in zip(self.branches, views):
            b.bind_cache(v)

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        ys, biases = [], []
        for j, b in enumerate(self.branches):
            y = ws.get(f"parallel_out_{j}", (T, self.hidden), torch.float32)
            # a branch whose output projection has a bias lets the sum below add it
            bias = getattr(b, "output_bias", None) if self.combine == "weighted_sum" else None
            extra = {"defer_bias": True} if bias is not None else {}
            if getattr(b, "can_overwrite", False):
                b.forward(xn, y, batch, overwrite=True, **extra)
            else:
                y.zero_()
                b.forward(xn, y, batch, **extra)
            ys.append(y)
            biases.append(bias)
        if self.combine == "weighted_sum":
            rt.ops.weighted_sum(ys, biases, self.scales, residual, accumulate=not overwrite)
        else:
            rt.ops.branch_norm_mean(ys, self.out_weights, self.eps, residual, accumulate=not overwrite)
