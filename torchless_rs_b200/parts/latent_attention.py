"""Attention whose keys and values are reconstructed from a low-rank latent, with a rotated key
part shared by all heads; optionally a sliding window, a sigmoid output gate and a sink logit per
head in the softmax's denominator.

With h the mixer's input, per token:
    c_q = norm(W_dq h) * w_q,        q = W_uq c_q        (per head: `dim` plain + `rot_dim` rotated)
    [c' | r'] = W_dkv h,             c = norm(c') * w_c,  r = rotate(r')
    k_h = [W_uk,h c | r],  v_h = W_uv,h c,  score = (q_h . k_h) * scale over the window
    p(i, j) = exp(score(i, j)) / (sum over visible j' of exp(score(i, j')) [+ exp(sink_h)])
    out = W_o ((heads' weighted values, concatenated) [* sigmoid(W_g h)])
Only [c | r] is cached, one vector per position (`PagedLatentRequest`).  Keys and values are
never formed: q's plain part is carried into the latent space (W_uk,h^T q_h), the weighted sum
is taken over the c's, and W_uv,h is applied to the sum, so prefill and decode run the same
kernels on the same pages and a position's result does not depend on the step that computes it.
The projections of h (W_dq, W_dkv and, with a gate, W_g) are one stacked product.

The rotated parts of a query and of the shared key only ever meet in their dot product, which does
not change when both are permuted alike.  A model whose rotation pairs entries (2i, 2i + 1) (the
position part's style) is therefore run by the kernels for pairs (i, i + n/2): the rows of
W_uq's rotated part and of W_dkv's last rows are reordered once, when the weights come in."""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..cache.requests import PagedLatentRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_mixer
from .runtime import Runtime


@register_mixer("latent_attention")
class LatentAttention:
    """Parameters: `hidden_size`, `heads`, `dim` (plain query/key size per head), `rot_dim` (rotated
    size), `vdim`, `q_rank`, `kv_rank`, `window` (None = all keys), `scale` (default
    1/sqrt(dim + rot_dim)), `eps` (of the two latent norms), `rot_dims` (how many of the rot_dim
    entries turn; default all), `gate` (default True: the sigmoid output gate and its tensor g), `sink`
    (default False: a learned logit per head, tensor sink).  The position part gives the frequencies of
    `rot_dims` entries and the pairing.
    Tensors under the prefix: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, [g], [sink], o."""
    graph_safe = True
    can_overwrite = True
    FEW_TOKENS = 16     # up to here a step keeps W_uq and W_uk apart

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.rot = int(p["rot_dim"])
        self.vdim = int(p["vdim"])
        self.q_rank = int(p["q_rank"])
        self.rank = int(p["kv_rank"])
        self.window = int(p["window"]) if p.get("window") else None
        self.eps = float(p["eps"])
        self.rot_dims = int(p.get("rot_dims", self.rot)) if position is not None else 0
        self.has_gate = bool(p.get("gate", True))
        self.has_sink = bool(p.get("sink", False))
        # the layer's position part names the pairing, as for the other rotated mixers
        self.pairing = "interleaved" if getattr(position, "style", 0) == 1 else "half_split"
        self.sink = None
        self.scale = float(p["scale"]) if p.get("scale") else 1.0 / math.sqrt(self.dim + self.rot)
        if self.rot_dims > self.rot or self.rot_dims % 2:
            raise ValueError(f"{self.rot_dims} rotated entries do not fit a rotated part of {self.rot}")
        if position is not None and self.rot_dims and position.inv_freq.numel() != self.rot_dims // 2:
            raise ValueError("the position part's frequencies do not fit the rotated entries")
        self.prefix = prefix
        self.rt = rt
        self.position = position
        self.matmul = Matmul(rt)
        self.cache = None

    @staticmethod
    def _shapes(p):
        H, dim, rot, vdim = int(p["heads"]), int(p["dim"]), int(p["rot_dim"]), int(p["vdim"])
        return int(p["hidden_size"]), H, dim, rot, vdim, int(p["q_rank"]), int(p["kv_rank"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        hidden, H, dim, rot, vdim, q_rank, rank = cls._shapes(spec.params)
        out = {
            f"{prefix}.dq": TensorSpec((q_rank, hidden)),
            f"{prefix}.dq.norm": TensorSpec((q_rank,)),
            f"{prefix}.uq": TensorSpec((H * (dim + rot), q_rank)),
            f"{prefix}.dkv": TensorSpec((rank + rot, hidden)),
            f"{prefix}.dkv.norm": TensorSpec((rank,)),
            f"{prefix}.uk": TensorSpec((H * dim, rank)),
            f"{prefix}.uv": TensorSpec((H * vdim, rank)),
            f"{prefix}.o": TensorSpec((hidden, H * vdim)),
        }
        if spec.params.get("gate", True):
            out[f"{prefix}.g"] = TensorSpec((H * vdim, hidden))
        if spec.params.get("sink", False):
            out[f"{prefix}.sink"] = TensorSpec((H,), init=(1.0, 0.0))
        return out

    def _reordered(self, t: torch.Tensor, first: int) -> torch.Tensor:
        """Rows first .. first + rot_dims of `t` so that the pair (2i, 2i + 1) becomes (i, i + rot_dims/2)."""
        n = self.rot_dims
        if self.pairing != "interleaved" or n == 0:
            return t
        order = list(range(0, n, 2)) + list(range(1, n, 2))
        t = t.clone()
        t[first:first + n] = t[first:first + n][order]
        return t

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        w_dkv = self._reordered(weights[f"{p}.dkv"], self.rank)
        w_uq = weights[f"{p}.uq"].reshape(self.heads, self.dim + self.rot, self.q_rank)
        w_uq = torch.stack([self._reordered(w_uq[h], self.dim) for h in range(self.heads)]) \
            .reshape(self.heads * (self.dim + self.rot), self.q_rank)
        self.w_in = rt.stack([weights[f"{p}.dq"], w_dkv] + ([weights[f"{p}.g"]] if self.has_gate else []))
        self.w_uq = rt.matrix(w_uq)
        # per head, transposed: the query's plain part is multiplied by W_uk,h^T
        uk = weights[f"{p}.uk"].reshape(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uk_t = rt.matrix(uk)                                          # [heads, rank, dim]
        self.w_uv = rt.matrix(weights[f"{p}.uv"].reshape(self.heads, self.vdim, self.rank))
        self.w_o = rt.matrix(weights[f"{p}.o"])
        # For steps of many tokens W_uk,h^T is folded into W_uq: one product gives every head's
        # [latent-space query | part to rotate].  (Folded in 64-bit, once, when the weights come in.)
        uq64 = w_uq.to(device=rt.device, dtype=torch.float64).reshape(
            self.heads, self.dim + self.rot, self.q_rank)
        uk64 = weights[f"{p}.uk"].to(device=rt.device, dtype=torch.float64).reshape(self.heads, self.dim, self.rank)
        folded = torch.cat([torch.bmm(uk64.transpose(1, 2), uq64[:, :self.dim]), uq64[:, self.dim:]], dim=1)
        self.w_q_latent = rt.matrix(folded.reshape(self.heads * (self.rank + self.rot), self.q_rank)
                                    .to(torch.float32 if rt.is_f32 else torch.bfloat16))
        del uq64, uk64, folded
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        self.norm_q = f32(weights[f"{p}.dq.norm"])
        self.norm_c = f32(weights[f"{p}.dkv.norm"])
        if self.has_sink:
            self.sink = f32(weights[f"{p}.sink"])

    def cache_request(self):
        return PagedLatentRequest(self.rank + self.rot, self.window)

    def bind_cache(self, view) -> None:
        self.cache = view

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws, o = self.rt, self.rt.workspace, self.rt.ops
        T = residual.shape[0]
        H, dim, rot, rank, vdim, q_rank = self.heads, self.dim, self.rot, self.rank, self.vdim, self.q_rank
        c = self.cache
        inv_freq = self.position.inv_freq if self.rot_dims else None
        n_in = q_rank + rank + rot + (H * vdim if self.has_gate else 0)
        s = ws.get("latent_in", (T, n_in), torch.float32)
        self.matmul(xn, self.w_in, s, ops.MODE_STORE_F32)
        cq = ws.get("latent_cq", (T, q_rank), rt.act_dtype)
        o.latent_prep(s[:, :q_rank], s[:, q_rank:q_rank + rank + rot], self.norm_q, self.norm_c, self.eps, cq,
                      c.pages, batch.token_pos, batch.token_seq, batch.seq_slot, c.page_table, inv_freq,
                      rank, rot, self.rot_dims)
        mix = ws.get("latent_mix", (T, H, rank), torch.float32)
        if T <= self.FEW_TOKENS:
            # few tokens: the two small matrices are fewer bytes to stream than the folded one
            q = ws.get("latent_q", (T, H * (dim + rot)), torch.float32)
            self.matmul(cq, self.w_uq, q, ops.MODE_STORE_F32)
            qa = ws.get("latent_qa", (T, H * rank), torch.float32)
            o.headwise_gemm(q, dim + rot, self.w_uk_t, qa, rank)
            o.latent_attn(qa, rank, q, dim + rot, dim, c.pages, mix, batch.token_pos, batch.token_seq,
                          batch.seq_slot, c.page_table, inv_freq, H, rank, rot, self.rot_dims, self.window, self.scale,
                          max_keys=batch.len_bucket, workspace=ws, sink=self.sink)
        else:
            q = ws.get("latent_ql", (T, H * (rank + rot)), torch.float32)
            self.matmul(cq, self.w_q_latent, q, ops.MODE_STORE_F32)
            o.latent_attn(q, rank + rot, q, rank + rot, rank, c.pages, mix, batch.token_pos, batch.token_seq,
                          batch.seq_slot, c.page_table, inv_freq, H, rank, rot, self.rot_dims, self.window, self.scale,
                          max_keys=batch.len_bucket, workspace=ws, sink=self.sink)
        gated = ws.get("latent_gated", (T, H * vdim), rt.act_dtype)
        o.headwise_gemm(mix.view(T, H * rank), rank, self.w_uv, gated, vdim,
                        gate=s[:, q_rank + rank + rot:] if self.has_gate else None, act_out=True)
        self.matmul(gated, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)
