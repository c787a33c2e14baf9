"""Typed configuration of the Fezolorn decoder, read from its config.json.

The design: pre-norm residual layers (x <- x + mixer(N(x)); x <- x + ff(N(x)), N an RMS norm with a
weight), each with one of three mixers:
  * `parallel`: two mixers on the same input, summed with one factor each (`left_scale`, `right_scale`).
    `left` is softmax attention with grouped key/value heads whose values are the projected keys
    themselves, biased projections, a rotation of the first `rot.dims` entries of every head
    (neighbouring pairs; frequencies optionally stretched band by band, `rot.scaling`), a unit RMS norm
    of rotated queries and keys, a sliding window (`mask.size`) and a sink logit per head.  `right` is
    the gated delta rule behind short causal convolutions of `conv` taps.
  * `lightning`: linear attention with a constant decay per head (`decay`).
  * `latent_attention`: causal softmax attention through low-rank latents with a rotated key part
    shared by the heads and a sink logit per head.
The feed-forward is SwiGLU (`mlp.kind` = "dense") or absent (`mlp` null); the head is the embedding
table.  config.json lists the layers one by one with all their sizes and constants (`layers[i].type`,
`.mixer`, `.mlp`), so layers of one model may differ in all of them.  Tensor names: `embed`,
`l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*` (`l<i>.mix.left.*` and `l<i>.mix.right.*` for a parallel
mixer), `l<i>.mlp.*`, `final.norm`."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .errors import ConfigError
from .reader import KeyReader
from .spec import LayerSpec, ModelSpec, PartSpec

LAYER_TENSOR_NAMES = {"mixer_norm": "norm1", "mixer": "mix", "feed_forward_norm": "norm2", "feed_forward": "mlp"}
SWIGLU_NAMES = ("gate", "up", "down")
UNIT_NORM_EPS = 1e-6      # inside the root of the delta rule's unit norms of q and k: fixed by the design


@dataclass(frozen=True)
class Rotation:
    """Rotary positions of the first `dims` entries, pairs (2i, 2i + 1), frequency base^(-2i / dims);
    `scaling` = (factor, low, high, original) stretches them band by band, None leaves them."""
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None

    @classmethod
    def read(cls, data, where: str, limit: int) -> Optional["Rotation"]:
        if data is None:
            return None
        r = KeyReader(data, where)
        dims = r.integer("dims", minimum=0)
        if dims % 2 or dims > limit:
            raise ConfigError(f"{where}: 'dims' {dims} must be even and at most {limit}")
        scaling = None
        if data.get("scaling") is not None:
            sr = KeyReader(data["scaling"], f"{where}.scaling")
            scaling = (sr.number("factor"), sr.number("low"), sr.number("high"), sr.number("original"))
            if scaling[2] == scaling[1]:
                raise ConfigError(f"{where}.scaling: 'high' and 'low' must differ")
        return cls(base=r.number("base"), dims=dims, scaling=scaling) if dims else None

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return d

    def part(self) -> PartSpec:
        params: Dict[str, Any] = {"head_dim": self.dims, "theta": self.base}
        if self.scaling is not None:
            params["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return PartSpec("rope_interleaved", params)


@dataclass(frozen=True)
class KeyValueAttentionBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot: Optional[Rotation]

    @classmethod
    def read(cls, r: KeyReader) -> "KeyValueAttentionBranch":
        heads, kv = r.integer("heads"), r.integer("kv_heads")
        if heads % kv:
            raise ConfigError(f"{r.where}: 'heads' {heads} is no multiple of 'kv_heads' {kv}")
        dim = r.integer("dim")
        vdim = r.integer("vdim", dim)
        if vdim != dim:
            raise ConfigError(f"{r.where}: the values are the keys, so 'vdim' {vdim} must equal 'dim' {dim}")
        mask = r.data.get("mask")
        window = KeyReader(mask, f"{r.where}.mask").integer("size", None) if mask is not None else None
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=r.number("scale"), window=window or None,
                   rot=Rotation.read(r.data.get("rot"), f"{r.where}.rot", dim))

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("sink_rotary_attention", {
            "hidden_size": hidden, "heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
            "vdim": self.vdim, "rot_dims": self.rot.dims if self.rot else 0, "scale": self.scale,
            "window": self.window, "eps": eps, "unit_norm": True, "sink": True, "bias": True,
            "values_are_keys": True})


@dataclass(frozen=True)
class DeltaRuleBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def read(cls, r: KeyReader) -> "DeltaRuleBranch":
        heads, kv = r.integer("heads"), r.integer("kv_heads")
        if heads % kv:
            raise ConfigError(f"{r.where}: 'heads' {heads} is no multiple of 'kv_heads' {kv}")
        dim = r.integer("dim")
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=r.integer("vdim", dim), conv=r.integer("conv", minimum=1))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "conv": self.conv}

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("gated_delta_rule", {
            "hidden_size": hidden, "heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
            "vdim": self.vdim, "conv": self.conv, "eps": eps, "unit_eps": UNIT_NORM_EPS})


@dataclass(frozen=True)
class ParallelMixerLayer:
    left: KeyValueAttentionBranch
    right: DeltaRuleBranch
    left_scale: float
    right_scale: float

    type = "parallel"

    @classmethod
    def read(cls, r: KeyReader) -> "ParallelMixerLayer":
        for side in ("left", "right"):
            if not isinstance(r.data.get(side), dict):
                raise ConfigError(f"{r.where}: required key '{side}' is missing")
        return cls(KeyValueAttentionBranch.read(KeyReader(r.data["left"], f"{r.where}.left")),
                   DeltaRuleBranch.read(KeyReader(r.data["right"], f"{r.where}.right")),
                   left_scale=r.number("left_scale", 1.0, positive=False),
                   right_scale=r.number("right_scale", 1.0, positive=False))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}

    def position(self) -> Optional[PartSpec]:
        return self.left.rot.part() if self.left.rot else None

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("parallel", {"hidden_size": hidden, "combine": "weighted_sum",
                                     "scales": (self.left_scale, self.right_scale),
                                     "branches": (("left", self.left.part(hidden, eps)),
                                                  ("right", self.right.part(hidden, eps)))})


@dataclass(frozen=True)
class LightningLayer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    type = "lightning"

    @classmethod
    def read(cls, r: KeyReader) -> "LightningLayer":
        heads, dim = r.integer("heads"), r.integer("dim")
        decay = r.data.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or \
                not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            raise ConfigError(f"{r.where}: 'decay' must list one number for each of the {heads} heads")
        return cls(heads=heads, dim=dim, vdim=r.integer("vdim", dim), decay=tuple(float(d) for d in decay))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}

    def position(self) -> Optional[PartSpec]:
        return None

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("lightning_attention", {"hidden_size": hidden, "heads": self.heads, "dim": self.dim,
                                                "vdim": self.vdim, "decay": self.decay, "eps": eps})


@dataclass(frozen=True)
class LatentAttentionLayer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Optional[Rotation]

    type = "latent_attention"

    @classmethod
    def read(cls, r: KeyReader) -> "LatentAttentionLayer":
        rot_dim = r.integer("rot_dim", 0, minimum=0)
        dim = r.integer("dim")
        rot = Rotation.read(r.data.get("rot"), f"{r.where}.rot", rot_dim) if rot_dim else None
        return cls(heads=r.integer("heads"), dim=dim, rot_dim=rot_dim, vdim=r.integer("vdim", dim),
                   q_rank=r.integer("q_rank"), kv_rank=r.integer("kv_rank"), scale=r.number("scale"), rot=rot)

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                             "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d

    def position(self) -> Optional[PartSpec]:
        return self.rot.part() if self.rot else None

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("latent_attention", {
            "hidden_size": hidden, "heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim,
            "vdim": self.vdim, "q_rank": self.q_rank, "kv_rank": self.kv_rank, "window": None,
            "scale": self.scale, "eps": eps, "rot_dims": self.rot.dims if self.rot else 0, "gate": False,
            "sink": True})


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
        return PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": self.ff,
                                   "tensor_names": SWIGLU_NAMES})


MIXERS = {c.type: c for c in (ParallelMixerLayer, LightningLayer, LatentAttentionLayer)}
FEED_FORWARDS = {c.kind: c for c in (DenseFeedForward,)}


@dataclass(frozen=True)
class FezolornLayer:
    mixer: Any                     # one of the classes in MIXERS
    mlp: Any                       # one of the classes in FEED_FORWARDS, or None: the layer has none


@dataclass(frozen=True)
class FezolornConfig:
    width: int
    vocab: int
    layers: Tuple[FezolornLayer, ...]
    eps: float
    max_position_embeddings: int = 4096         # the default size of the cache, no bound of the design
    architecture: str = "Fezolorn"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "FezolornConfig":
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
            layers.append(FezolornLayer(mixer, ff))
        if not layers:
            raise ConfigError(f"{where}: 'layers' is empty")
        return cls(width=r.integer("width"), vocab=r.integer("vocab"), layers=tuple(layers),
                   eps=norm.number("eps", 1e-6),
                   max_position_embeddings=r.integer("max_position_embeddings", 4096),
                   architecture=r.string("architecture", "Fezolorn"))

    def to_dict(self) -> dict:
        """The config.json dictionary that reads back to this configuration."""
        return {
            "architecture": self.architecture, "width": self.width, "vocab": self.vocab,
            "norm": {"eps": self.eps},
            "layers": [{"type": l.mixer.type, "mixer": l.mixer.to_dict(),
                        "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers],
        }

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "bare_name": True})
        layers = []
        for i, l in enumerate(self.layers):
            prefix = f"l{i}"
            mixer = l.mixer.part(self.width, self.eps)
            if l.mlp is None:
                block, ff = PartSpec("prenorm_mixer_only"), PartSpec("none")
                norms = {"mixer_norm": norm}
                # a folder may store the second norm of a layer without feed-forward all the same
                unused = {LAYER_TENSOR_NAMES["feed_forward_norm"]: (self.width,)}
            else:
                block, ff = PartSpec("prenorm"), l.mlp.part(self.width)
                norms = {"mixer_norm": norm, "feed_forward_norm": norm}
                unused = {}
            layers.append(LayerSpec(prefix=prefix, block=block, mixer=mixer, feed_forward=ff, norms=norms,
                                    names=LAYER_TENSOR_NAMES, position=l.mixer.position(), unused_tensors=unused))
        spec = ModelSpec(hidden_size=self.width, vocab_size=self.vocab, embedding_name="embed", head_name="head",
                         tie_head_to_embedding=True, final_norm=norm, final_norm_prefix="final.norm",
                         layers=tuple(layers), order=tuple(range(len(layers))), stop_token_ids=())
        spec.validate()
        return spec
