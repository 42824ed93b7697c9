"""Typed configuration of the Kikopel decoder, read from its config.json.

The design: embedded tokens (times `embedding.scale`) plus a table row chosen by a hash of the
previous and the current token; layers x <- x + m * norm(mixer(x)), x <- x + m * norm(ff(x)) with
single-gain RMS norms on the branches' outputs and m = `residual_mult`; per layer one of two
mixers, attention through low-rank latents with a sliding window (`latent_attention`) or a gated
linear recurrence with a matrix state (`hgrn2`); a feed-forward with a polynomial activation of
normalised powers, or none; a single-gain RMS norm and a head.  config.json gives every size and
every constant per layer (`layers[i].type`, `.mixer`, `.mlp`), so layers of one model may differ in
all of them.  Tensor names: `embed`, `bigram`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`,
`l<i>.mlp.*`, `final.norm`, `head`."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .errors import ConfigError
from .reader import KeyReader
from .spec import LayerSpec, ModelSpec, PartSpec

LAYER_TENSOR_NAMES = {"mixer_out_norm": "norm1", "mixer": "mix", "feed_forward_out_norm": "norm2",
                      "feed_forward": "mlp"}


@dataclass(frozen=True)
class LatentAttentionLayer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    window: Optional[int]
    scale: float
    rot_base: float
    rot_dims: int

    type = "latent_attention"

    @classmethod
    def read(cls, r: KeyReader) -> "LatentAttentionLayer":
        dim, rot_dim = r.integer("dim"), r.integer("rot_dim", 0, minimum=0)
        mask = r.data.get("mask")
        window = KeyReader(mask, f"{r.where}.mask").integer("size", None) if isinstance(mask, dict) else None
        rot = r.data.get("rot")
        if rot_dim and not isinstance(rot, dict):
            raise ConfigError(f"{r.where}: a rotated part of {rot_dim} needs the key 'rot'")
        rr = KeyReader(rot, f"{r.where}.rot") if isinstance(rot, dict) else None
        rot_dims = rr.integer("dims", rot_dim, minimum=0) if rr else 0
        if rot_dims > rot_dim or rot_dims % 2:
            raise ConfigError(f"{r.where}: rot.dims {rot_dims} must be even and at most rot_dim {rot_dim}")
        return cls(heads=r.integer("heads"), dim=dim, rot_dim=rot_dim, vdim=r.integer("vdim"),
                   q_rank=r.integer("q_rank"), kv_rank=r.integer("kv_rank"), window=window,
                   scale=r.number("scale", 1.0 / math.sqrt(dim + rot_dim)),
                   rot_base=rr.number("base", 10000.0) if rr else 10000.0, rot_dims=rot_dims)

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                             "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dim:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d

    def parts(self, hidden: int, eps: float) -> Tuple[PartSpec, Optional[PartSpec]]:
        mixer = PartSpec("latent_attention", {
            "hidden_size": hidden, "heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim,
            "vdim": self.vdim, "q_rank": self.q_rank, "kv_rank": self.kv_rank, "window": self.window,
            "scale": self.scale, "eps": eps, "rot_dims": self.rot_dims})
        position = (PartSpec("rope_half_split", {"head_dim": self.rot_dims, "theta": self.rot_base})
                    if self.rot_dims else None)
        return mixer, position


@dataclass(frozen=True)
class RecurrenceLayer:
    heads: int
    dim: int
    vdim: int

    type = "hgrn2"

    @classmethod
    def read(cls, r: KeyReader) -> "RecurrenceLayer":
        return cls(heads=r.integer("heads"), dim=r.integer("dim"), vdim=r.integer("vdim"))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}

    def parts(self, hidden: int, eps: float) -> Tuple[PartSpec, Optional[PartSpec]]:
        return PartSpec("hgrn2", {"hidden_size": hidden, "heads": self.heads, "dim": self.dim,
                                  "vdim": self.vdim, "eps": eps}), None


MIXERS = {c.type: c for c in (LatentAttentionLayer, RecurrenceLayer)}
FEED_FORWARD_KINDS = ("dense",)


@dataclass(frozen=True)
class KikopelLayer:
    mixer: Any                     # one of the classes in MIXERS
    ff: Optional[int]              # the feed-forward's inner size; None: the layer has none
    ff_kind: str = "dense"


@dataclass(frozen=True)
class KikopelConfig:
    width: int
    vocab: int
    layers: Tuple[KikopelLayer, ...]
    eps: float
    residual_mult: float
    embedding_scale: float
    bigram: Optional[Tuple[int, int, int]]      # (buckets, mul_prev, mul_cur), or no second table
    max_position_embeddings: int = 4096         # the default size of the cache, no bound of the design
    architecture: str = "Kikopel"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "KikopelConfig":
        r = KeyReader(data, where)
        norm = KeyReader(data.get("norm") or {}, f"{where}: norm")
        emb = KeyReader(data.get("embedding") or {}, f"{where}: embedding")
        big = emb.data.get("bigram")
        bigram = None
        if big is not None:
            b = KeyReader(big, f"{where}: embedding.bigram")
            bigram = (b.integer("buckets"), b.integer("mul_prev", minimum=0), b.integer("mul_cur", minimum=0))
        layers = []
        for i, entry in enumerate(r.list_of("layers")):
            lr = KeyReader(entry, f"{where}: layers[{i}]")
            kind = lr.string("type")
            if kind not in MIXERS:
                raise ConfigError(f"{where}: layers[{i}].type '{kind}' is not known; known: {', '.join(sorted(MIXERS))}")
            mixer = MIXERS[kind].read(KeyReader(entry.get("mixer"), f"{where}: layers[{i}].mixer"))
            mlp = entry.get("mlp")
            ff, ff_kind = None, "dense"
            if mlp is not None:
                mr = KeyReader(mlp, f"{where}: layers[{i}].mlp")
                ff_kind = mr.string("kind", "dense")
                if ff_kind not in FEED_FORWARD_KINDS:
                    raise ConfigError(f"{where}: layers[{i}].mlp.kind '{ff_kind}' is not known; known: "
                                      f"{', '.join(FEED_FORWARD_KINDS)}")
                ff = mr.integer("ff")
            layers.append(KikopelLayer(mixer, ff, ff_kind))
        if not layers:
            raise ConfigError(f"{where}: 'layers' is empty")
        return cls(width=r.integer("width"), vocab=r.integer("vocab"), layers=tuple(layers),
                   eps=norm.number("eps", 1e-5), residual_mult=r.number("residual_mult", 1.0),
                   embedding_scale=emb.number("scale", 1.0), bigram=bigram,
                   max_position_embeddings=r.integer("max_position_embeddings", 4096),
                   architecture=r.string("architecture", "Kikopel"))

    def to_dict(self) -> dict:
        """The config.json dictionary that reads back to this configuration."""
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        return {
            "architecture": self.architecture, "width": self.width, "vocab": self.vocab,
            "embedding": emb, "norm": {"eps": self.eps}, "residual_mult": self.residual_mult,
            "layers": [{"type": l.mixer.type, "mixer": l.mixer.to_dict(),
                        "mlp": None if l.ff is None else {"kind": l.ff_kind, "ff": l.ff}} for l in self.layers],
        }

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm_scalar", {"size": self.width, "eps": self.eps})
        layers = []
        for i, l in enumerate(self.layers):
            mixer, position = l.mixer.parts(self.width, self.eps)
            if l.ff is None:
                block, ff = "branchnorm_mixer_only", PartSpec("none")
                norms = {"mixer_out_norm": norm}
            else:
                block = "branchnorm"
                ff = PartSpec("polynorm", {"hidden_size": self.width, "intermediate_size": l.ff, "eps": self.eps})
                norms = {"mixer_out_norm": norm, "feed_forward_out_norm": norm}
            # a layer without a feed-forward needs no second norm; a folder that stores its gain all the
            # same is accepted
            unused = {} if l.ff is not None else {LAYER_TENSOR_NAMES["feed_forward_out_norm"]: ()}
            layers.append(LayerSpec(prefix=f"l{i}", block=PartSpec(block, {"residual_mult": self.residual_mult}),
                                    mixer=mixer, feed_forward=ff, norms=norms, names=LAYER_TENSOR_NAMES,
                                    position=position, unused_tensors=unused))
        addend = None
        if self.bigram is not None:
            addend = PartSpec("pair_hash", {"name": "bigram", "hidden_size": self.width, "vocab_size": self.vocab,
                                            "buckets": self.bigram[0], "mul_prev": self.bigram[1],
                                            "mul_cur": self.bigram[2]})
        spec = ModelSpec(hidden_size=self.width, vocab_size=self.vocab, embedding_name="embed", head_name="head",
                         tie_head_to_embedding=False, final_norm=norm, final_norm_prefix="final.norm",
                         layers=tuple(layers), order=tuple(range(len(layers))), stop_token_ids=(),
                         embedding_scale=self.embedding_scale, embedding_addend=addend)
        spec.validate()
        return spec
