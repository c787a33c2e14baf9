"""Typed configuration of the Rupasun decoder, read from its config.json.

The design: every sublayer stands between two RMS norms with weights (x <- x + N_b(sub(N(x)))); a
layer's mixer is differential attention (`attention`: two rotated query/key maps per head over the
same values, the second subtracted from the first, then a per-head norm) or windowed attention
(`attention_2`: interleaved rotation, unit-normed queries and keys, capped scores, a sliding window,
a sigmoid gate per output entry); its feed-forward is dense with a squared relu, a mixture of clamped
experts chosen by sigmoid scores among the best groups with a shared expert, or absent.  config.json
lists the layers one by one with all their sizes and constants (`layers[i].type`, `.mixer`, `.mlp`),
so layers of one model may differ in all of them.  Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm1b`,
`l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .errors import ConfigError
from .reader import KeyReader
from .spec import LayerSpec, ModelSpec, PartSpec

LAYER_TENSOR_NAMES = {"mixer_norm": "norm1", "mixer_out_norm": "norm1b", "mixer": "mix",
                      "feed_forward_norm": "norm2", "feed_forward_out_norm": "norm2b", "feed_forward": "mlp"}
EXPERT_GATE_ALPHA = 1.702      # the experts' activation is g * sigmoid(1.702 g): fixed by the design


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float

    @classmethod
    def read(cls, r: KeyReader, dim: int) -> Optional["Rotation"]:
        rot = r.data.get("rot")
        if rot is None:
            return None
        rr = KeyReader(rot, f"{r.where}.rot")
        dims = rr.integer("dims", dim, minimum=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{rr.where}: 'dims' {dims} must be even and at most 'dim' {dim}")
        return cls(dims=dims, base=rr.number("base")) if dims else None

    def to_dict(self) -> dict:
        return {"dims": self.dims, "base": self.base}


def _heads(r: KeyReader) -> Tuple[int, int, int, int]:
    heads, kv = r.integer("heads"), r.integer("kv_heads")
    if heads % kv:
        raise ConfigError(f"{r.where}: 'heads' {heads} is no multiple of 'kv_heads' {kv}")
    dim = r.integer("dim")
    return heads, kv, dim, r.integer("vdim", dim)


@dataclass(frozen=True)
class DifferentialAttentionLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    rot: Optional[Rotation]

    type = "attention"
    rotation_kind = "rope_half_split"

    @classmethod
    def read(cls, r: KeyReader) -> "DifferentialAttentionLayer":
        heads, kv, dim, vdim = _heads(r)
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=r.number("scale"),
                   diff=r.number("diff", positive=False), rot=Rotation.read(r, dim))

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale, "diff": self.diff}
        if self.rot:
            d["rot"] = self.rot.to_dict()
        return d

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("differential_attention", {
            "hidden_size": hidden, "heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
            "vdim": self.vdim, "rot_dims": self.rot.dims if self.rot else 0, "scale": self.scale,
            "diff": self.diff, "eps": eps})


@dataclass(frozen=True)
class WindowAttentionLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    rot: Optional[Rotation]

    type = "attention_2"
    rotation_kind = "rope_interleaved"

    @classmethod
    def read(cls, r: KeyReader) -> "WindowAttentionLayer":
        heads, kv, dim, vdim = _heads(r)
        mask = r.data.get("mask")
        window = KeyReader(mask, f"{r.where}.mask").integer("size", None) if mask is not None else None
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=r.number("scale"),
                   softcap=r.number("softcap", None), window=window, rot=Rotation.read(r, dim))

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot:
            d["rot"] = self.rot.to_dict()
        return d

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("gated_window_attention", {
            "hidden_size": hidden, "heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
            "vdim": self.vdim, "rot_dims": self.rot.dims if self.rot else 0, "scale": self.scale,
            "softcap": self.softcap, "window": self.window, "eps": eps})


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int

    kind = "dense"

    @classmethod
    def read(cls, r: KeyReader) -> "DenseFeedForward":
        return cls(ff=r.integer("ff"))

    def to_dict(self) -> dict:
        return {"kind": self.kind, "ff": self.ff}

    def part(self, hidden: int) -> PartSpec:
        return PartSpec("relu_squared", {"hidden_size": hidden, "intermediate_size": self.ff})


@dataclass(frozen=True)
class ExpertFeedForward:
    ff: int
    limit: float
    experts: int
    top: int
    groups: int
    keep: int
    route_scale: float
    shared_ff: Optional[int]
    shared_limit: Optional[float]

    kind = "moe"

    @classmethod
    def read(cls, r: KeyReader) -> "ExpertFeedForward":
        for key in ("expert", "router"):
            if not isinstance(r.data.get(key), dict):
                raise ConfigError(f"{r.where}: required key '{key}' is missing")
        er = KeyReader(r.data["expert"], f"{r.where}.expert")
        rr = KeyReader(r.data["router"], f"{r.where}.router")
        experts, top = rr.integer("experts"), rr.integer("top")
        groups, keep = 1, 1
        if rr.data.get("groups") is not None:
            gr = KeyReader(rr.data["groups"], f"{rr.where}.groups")
            groups = gr.integer("count", 1)
            keep = gr.integer("keep", groups)
        if experts % groups:
            raise ConfigError(f"{rr.where}: {experts} experts do not form {groups} equal groups")
        if keep > groups:
            raise ConfigError(f"{rr.where}: groups.keep {keep} exceeds groups.count {groups}")
        if top > keep * (experts // groups):
            raise ConfigError(f"{rr.where}: top {top} exceeds the {keep * (experts // groups)} experts of the "
                              f"kept groups")
        shared_ff = shared_limit = None
        if r.data.get("shared") is not None:
            sr = KeyReader(r.data["shared"], f"{r.where}.shared")
            shared_ff, shared_limit = sr.integer("ff"), sr.number("limit")
        return cls(ff=er.integer("ff"), limit=er.number("limit"), experts=experts, top=top, groups=groups,
                   keep=keep, route_scale=rr.number("scale", 1.0), shared_ff=shared_ff, shared_limit=shared_limit)

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"kind": self.kind, "expert": {"ff": self.ff, "limit": self.limit},
                             "router": {"experts": self.experts, "top": self.top, "scale": self.route_scale,
                                        "groups": {"count": self.groups, "keep": self.keep}}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d

    def part(self, hidden: int) -> PartSpec:
        return PartSpec("moe_grouped_sigmoid", {
            "hidden_size": hidden, "ff": self.ff, "experts": self.experts, "top": self.top, "limit": self.limit,
            "groups": self.groups, "keep": self.keep, "route_scale": self.route_scale,
            "gate_alpha": EXPERT_GATE_ALPHA, "shared_ff": self.shared_ff, "shared_limit": self.shared_limit})


MIXERS = {c.type: c for c in (DifferentialAttentionLayer, WindowAttentionLayer)}
FEED_FORWARDS = {c.kind: c for c in (DenseFeedForward, ExpertFeedForward)}


@dataclass(frozen=True)
class RupasunLayer:
    mixer: Any                     # one of the classes in MIXERS
    mlp: Any                       # one of the classes in FEED_FORWARDS, or None: the layer has none


@dataclass(frozen=True)
class RupasunConfig:
    width: int
    vocab: int
    layers: Tuple[RupasunLayer, ...]
    eps: float
    max_position_embeddings: int = 4096         # the default size of the cache, no bound of the design
    architecture: str = "Rupasun"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "RupasunConfig":
        r = KeyReader(data, where)
        norm = KeyReader(data.get("norm") or {}, f"{where}: norm")
        layers = []
        for i, entry in enumerate(r.list_of("layers")):
            lr = KeyReader(entry, f"{where}: layers[{i}]")
            kind = lr.string("type")
            if kind not in MIXERS:
                raise ConfigError(f"{where}: layers[{i}].type '{kind}' is not known; known: {', '.join(sorted(MIXERS))}")
            mixer = MIXERS[kind].read(KeyReader(entry.get("mixer"), f"{where}: layers[{i}].mixer"))
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                mr = KeyReader(mlp, f"{where}: layers[{i}].mlp")
                ff_kind = mr.string("kind", "dense")
                if ff_kind not in FEED_FORWARDS:
                    raise ConfigError(f"{where}: layers[{i}].mlp.kind '{ff_kind}' is not known; known: "
                                      f"{', '.join(sorted(FEED_FORWARDS))}")
                ff = FEED_FORWARDS[ff_kind].read(mr)
            layers.append(RupasunLayer(mixer, ff))
        if not layers:
            raise ConfigError(f"{where}: 'layers' is empty")
        return cls(width=r.integer("width"), vocab=r.integer("vocab"), layers=tuple(layers),
                   eps=norm.number("eps", 1e-6),
                   max_position_embeddings=r.integer("max_position_embeddings", 4096),
                   architecture=r.string("architecture", "Rupasun"))

    def to_dict(self) -> dict:
        """The config.json dictionary that reads back to this configuration."""
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                "norm": {"eps": self.eps},
                "layers": [{"type": l.mixer.type, "mixer": l.mixer.to_dict(),
                            "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "bare_name": True})
        layers = []
        for i, l in enumerate(self.layers):
            prefix = f"l{i}"
            mixer = l.mixer.part(self.width, self.eps)
            rot = l.mixer.rot
            position = PartSpec(l.mixer.rotation_kind, {"head_dim": rot.dims, "theta": rot.base}) if rot else None
            if l.mlp is None:
                block, ff = PartSpec("sandwich_mixer_only"), PartSpec("none")
                norms = {"mixer_norm": norm, "mixer_out_norm": norm}
                # without a feed-forward its norms are not used; a folder that stores them all the same is accepted
                unused = {LAYER_TENSOR_NAMES["feed_forward_norm"]: (self.width,),
                          LAYER_TENSOR_NAMES["feed_forward_out_norm"]: (self.width,)}
            else:
                block, ff = PartSpec("sandwich"), l.mlp.part(self.width)
                norms = {"mixer_norm": norm, "mixer_out_norm": norm, "feed_forward_norm": norm,
                         "feed_forward_out_norm": norm}
                unused = {}
            layers.append(LayerSpec(prefix=prefix, block=block, mixer=mixer, feed_forward=ff, norms=norms,
                                    names=LAYER_TENSOR_NAMES, position=position, unused_tensors=unused))
        spec = ModelSpec(hidden_size=self.width, vocab_size=self.vocab, embedding_name="embed", head_name="head",
                         tie_head_to_embedding=False, final_norm=norm, final_norm_prefix="final.norm",
                         layers=tuple(layers), order=tuple(range(len(layers))), stop_token_ids=())
        spec.validate()
        return spec
