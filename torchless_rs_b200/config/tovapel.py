"""Typed configuration of the Tovapel decoder, read from its config.json.

The design: the embedded token is kept in `streams` residual streams (hyper-connections: every
sublayer reads a weighted sum of the streams through a norm, and writes its output into all of them
while they are mixed); a layer's mixer runs two branches on the same input, softmax attention with
a sink, capped scores and a window that keeps the first keys (`left`), and gated linear attention
(`right`), and averages their normed outputs; the feed-forward is SwiGLU, a mixture of clamped
experts some of whose router outputs hand the input through, or absent; a norm whose stored weight
lies around zero, a head, and a soft cap on the logits.  config.json lists the layers one by one with
all their sizes and constants (`layers[i].type`, `.mixer`, `.mlp`), so layers of one model may differ
in all of them.  Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.hc1.*`, `l<i>.hc2.*`,
`l<i>.mix.left.*`, `l<i>.mix.right.*`, `l<i>.mlp.*`, `final.norm`, `head`."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .errors import ConfigError
from .reader import KeyReader
from .spec import LayerSpec, ModelSpec, PartSpec

LAYER_TENSOR_NAMES = {"mixer_norm": "norm1", "mixer": "mix", "feed_forward_norm": "norm2", "feed_forward": "mlp"}
CONNECTION_NAMES = ("hc1", "hc2")
SWIGLU_NAMES = ("gate", "up", "down")
EXPERT_GATE_ALPHA = 1.702      # the experts' activation is g * sigmoid(1.702 g): fixed by the design


@dataclass(frozen=True)
class WindowAttentionBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    keep_first: int

    @classmethod
    def read(cls, r: KeyReader) -> "WindowAttentionBranch":
        mask = r.data.get("mask")
        window, keep = None, 0
        if mask is not None:
            mr = KeyReader(mask, f"{r.where}.mask")
            window = mr.integer("size", None)
            keep = mr.integer("keep_first", 0, minimum=0)
        heads, kv = r.integer("heads"), r.integer("kv_heads")
        if heads % kv:
            raise ConfigError(f"{r.where}: 'heads' {heads} is no multiple of 'kv_heads' {kv}")
        dim = r.integer("dim")
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=r.integer("vdim", dim), scale=r.number("scale"),
                   softcap=r.number("softcap", None), window=window, keep_first=keep if window else 0)

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.window:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return d

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("sink_window_attention", {
            "hidden_size": hidden, "heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
            "vdim": self.vdim, "window": self.window, "keep_first": self.keep_first, "scale": self.scale,
            "softcap": self.softcap, "eps": eps})


@dataclass(frozen=True)
class LinearAttentionBranch:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None     # inner size of the decay's low-rank map; None: as the stored tensors have it

    @classmethod
    def read(cls, r: KeyReader) -> "LinearAttentionBranch":
        dim = r.integer("dim")
        return cls(heads=r.integer("heads"), dim=dim, vdim=r.integer("vdim", dim), tau=r.number("tau"),
                   rank=r.integer("rank", None))

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank is not None:
            d["rank"] = self.rank
        return d

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("gated_linear_attention", {
            "hidden_size": hidden, "heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau,
            "eps": eps, "rank": self.rank})


@dataclass(frozen=True)
class ParallelMixerLayer:
    left: WindowAttentionBranch
    right: LinearAttentionBranch

    type = "parallel"

    @classmethod
    def read(cls, r: KeyReader) -> "ParallelMixerLayer":
        for side in ("left", "right"):
            if not isinstance(r.data.get(side), dict):
                raise ConfigError(f"{r.where}: required key '{side}' is missing")
        return cls(WindowAttentionBranch.read(KeyReader(r.data["left"], f"{r.where}.left")),
                   LinearAttentionBranch.read(KeyReader(r.data["right"], f"{r.where}.right")))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}

    def part(self, hidden: int, eps: float) -> PartSpec:
        return PartSpec("parallel", {"hidden_size": hidden, "eps": eps,
                                     "branches": (("left", self.left.part(hidden, eps)),
                                                  ("right", self.right.part(hidden, eps)))})


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


@dataclass(frozen=True)
class ExpertFeedForward:
    ff: int
    limit: float
    experts: int
    identity: int
    top: int

    kind = "moe"

    @classmethod
    def read(cls, r: KeyReader) -> "ExpertFeedForward":
        for key in ("expert", "router"):
            if not isinstance(r.data.get(key), dict):
                raise ConfigError(f"{r.where}: required key '{key}' is missing")
        er = KeyReader(r.data["expert"], f"{r.where}.expert")
        rr = KeyReader(r.data["router"], f"{r.where}.router")
        experts, identity = rr.integer("experts", minimum=0), rr.integer("identity", 0, minimum=0)
        top = rr.integer("top")
        if top > experts + identity:
            raise ConfigError(f"{r.where}.router: top {top} exceeds the {experts + identity} router outputs")
        return cls(ff=er.integer("ff"), limit=er.number("limit"), experts=experts, identity=identity, top=top)

    def to_dict(self) -> dict:
        return {"kind": self.kind, "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}

    def part(self, hidden: int) -> PartSpec:
        return PartSpec("moe_clamped", {"hidden_size": hidden, "ff": self.ff, "experts": self.experts,
                                        "identity": self.identity, "top": self.top, "limit": self.limit,
                                        "gate_alpha": EXPERT_GATE_ALPHA})


MIXERS = {c.type: c for c in (ParallelMixerLayer,)}
FEED_FORWARDS = {c.kind: c for c in (DenseFeedForward, ExpertFeedForward)}


@dataclass(frozen=True)
class TovapelLayer:
    mixer: Any                     # one of the classes in MIXERS
    mlp: Any                       # one of the classes in FEED_FORWARDS, or None: the layer has none


@dataclass(frozen=True)
class TovapelConfig:
    width: int
    vocab: int
    streams: int
    layers: Tuple[TovapelLayer, ...]
    eps: float
    logit_softcap: Optional[float]
    max_position_embeddings: int = 4096         # the default size of the cache, no bound of the design
    architecture: str = "Tovapel"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "TovapelConfig":
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
            layers.append(TovapelLayer(mixer, ff))
        if not layers:
            raise ConfigError(f"{where}: 'layers' is empty")
        streams = r.integer("streams", 1)
        if streams > 8:
            raise ConfigError(f"{where}: key 'streams' must be <= 8, got {streams}")
        return cls(width=r.integer("width"), vocab=r.integer("vocab"), streams=streams, layers=tuple(layers),
                   eps=norm.number("eps", 1e-5), logit_softcap=r.number("logit_softcap", None),
                   max_position_embeddings=r.integer("max_position_embeddings", 4096),
                   architecture=r.string("architecture", "Tovapel"))

    def to_dict(self) -> dict:
        """The config.json dictionary that reads back to this configuration."""
        d: Dict[str, Any] = {
            "architecture": self.architecture, "width": self.width, "vocab": self.vocab, "streams": self.streams,
            "norm": {"eps": self.eps},
            "layers": [{"type": l.mixer.type, "mixer": l.mixer.to_dict(),
                        "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers],
        }
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm_one_plus", {"size": self.width, "eps": self.eps})
        layers = []
        for i, l in enumerate(self.layers):
            prefix = f"l{i}"
            mixer = l.mixer.part(self.width, self.eps)
            params = {"streams": self.streams, "prefix": prefix, "names": CONNECTION_NAMES}
            if l.mlp is None:
                block, ff = PartSpec("hyper_connections_mixer_only", params), PartSpec("none")
                norms = {"mixer_norm": norm}
                # without a feed-forward neither its norm nor its connections are used; a folder that
                # stores them all the same is accepted
                S = self.streams
                unused = {LAYER_TENSOR_NAMES["feed_forward_norm"]: (self.width,),
                          f"{CONNECTION_NAMES[1]}.in": (S,), f"{CONNECTION_NAMES[1]}.out": (S,),
                          f"{CONNECTION_NAMES[1]}.mix": (S, S)}
            else:
                block, ff = PartSpec("hyper_connections", params), l.mlp.part(self.width)
                norms = {"mixer_norm": norm, "feed_forward_norm": norm}
                unused = {}
            layers.append(LayerSpec(prefix=prefix, block=block, mixer=mixer, feed_forward=ff, norms=norms,
                                    names=LAYER_TENSOR_NAMES, unused_tensors=unused))
        spec = ModelSpec(hidden_size=self.width, vocab_size=self.vocab, embedding_name="embed", head_name="head",
                         tie_head_to_embedding=False, final_norm=norm, final_norm_prefix="final.norm",
                         layers=tuple(layers), order=tuple(range(len(layers))), stop_token_ids=(),
                         logit_softcap=self.logit_softcap, streams=self.streams)
        spec.validate()
        return spec
