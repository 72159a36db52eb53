"""Sigalorn's configuration: the keys of its config.json, typed.

config.json names the architecture under `architecture` and nests its values:

    vocab, width, logit_softcap, embedding.scale, norm.eps,
    layers: [ {type: "attention" | "gla", mixer: {...}, mlp: {kind: "dense", ff} | null}, ... ]

An attention mixer gives heads, kv_heads, dim (queries and keys), vdim (values), scale, rot.base, rot.dims,
mask.size (keys are seen inside blocks of that many positions) and optionally kv_from (the layer whose keys and
values it reads; it then has no projections of its own for them).  A gla mixer gives heads, dim, vdim and tau; the
rank of its decay projection is read from the tensor's shape when the folder is opened, or from `rank` when a
model is built from a configuration alone.  Every size and constant of a model comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    block: int                     # 0: every earlier key is seen
    kv_from: int | None = None

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.block:
            d["mask"] = {"size": self.block}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class GlaSpec:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int | None = None        # None: taken from the stored tensor

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank is not None:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class DenseSpec:
    ff: int
    kind: str = "dense"

    def to_dict(self) -> dict:
        return {"kind": self.kind, "ff": self.ff}


@dataclass(frozen=True)
class LayerSpec:
    type: str                      # "attention" | "gla"
    mixer: Any
    mlp: DenseSpec | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


def _sub(r: ConfigReader, key: str, required: bool = True) -> ConfigReader | None:
    v = r.raw.get(key)
    r.seen.add(key)
    if v is None:
        if required:
            raise ConfigError(f"{r.where}: required key {key!r} is missing")
        return None
    if not isinstance(v, Mapping):
        raise ConfigError(f"{r.where}: {key!r} must be an object, found {v!r}")
    return ConfigReader(v, f"{r.where}: {key}")


def _attention(r: ConfigReader, index: int, before: list) -> AttentionSpec:
    heads = r.integer("heads", minimum=1)
    kv = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: heads ({heads}) not divisible by kv_heads ({kv})")
    dim = r.integer("dim", minimum=1)
    vdim = r.integer("vdim", default=dim, minimum=1)
    if vdim % 2:
        raise ConfigError(f"{r.where}: vdim must be even (values are rotated in pairs), found {vdim}")
    rot = _sub(r, "rot")
    rot_dims = rot.integer("dims", default=dim, minimum=0)
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{r.where}: rot.dims must be even and at most dim ({dim}), found {rot_dims}")
    mask = _sub(r, "mask", required=False)
    block = mask.integer("size", default=0, minimum=0) if mask is not None else 0
    src = r.integer("kv_from", minimum=0) if r.has("kv_from") else None
    spec = AttentionSpec(heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                         scale=r.number("scale", default=dim ** -0.5, minimum=0.0, exclusive=True),
                         rot_base=rot.number("base", default=10000.0, minimum=0.0, exclusive=True), rot_dims=rot_dims,
                         block=block, kv_from=src)
    if src is not None:
        if src >= index or before[src].type != "attention" or before[src].mixer.kv_from is not None:
            raise ConfigError(f"{r.where}: kv_from {src} must name an earlier attention layer with keys and values of its own")
        w = before[src].mixer
        if (w.kv_heads, w.dim, w.vdim, w.rot_base, w.rot_dims) != (kv, dim, vdim, spec.rot_base, rot_dims):
            raise ConfigError(f"{r.where}: layer {src}'s keys and values do not fit this layer's heads and rotation")
    return spec


def _gla(r: ConfigReader) -> GlaSpec:
    return GlaSpec(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1),
                   vdim=r.integer("vdim", minimum=1), tau=r.number("tau", default=1.0, minimum=0.0, exclusive=True),
                   rank=r.integer("rank", minimum=1) if r.has("rank") else None)


@dataclass(frozen=True)
class SigalornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: float           # 0 = no cap
    layers: tuple[LayerSpec, ...]
    architecture: str = "Sigalorn"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "SigalornConfig":
        r = ConfigReader(raw, where)
        emb = _sub(r, "embedding", required=False)
        norm = _sub(r, "norm", required=False)
        listed = r.raw.get("layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers: list[LayerSpec] = []
        for i, entry in enumerate(listed):
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where}: layers[{i}] must be an object")
            lr = ConfigReader(entry, f"{where}: layers[{i}]")
            kind = lr.string("type")
            mr = _sub(lr, "mixer")
            mr.where = f"{where}: layers[{i}].mixer"
            if kind == "attention":
                mixer = _attention(mr, i, layers)
            elif kind == "gla":
                mixer = _gla(mr)
            else:
                raise ConfigError(f"{where}: layers[{i}]: unknown layer type {kind!r} (known: attention, gla)")
            fr = _sub(lr, "mlp", required=False)
            mlp = None
            if fr is not None:
                fk = fr.string("kind", default="dense")
                if fk != "dense":
                    raise ConfigError(f"{where}: layers[{i}].mlp: unknown kind {fk!r} (known: dense)")
                mlp = DenseSpec(ff=fr.integer("ff", minimum=1), kind=fk)
            layers.append(LayerSpec(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   embedding_scale=emb.number("scale", default=1.0) if emb is not None else 1.0,
                   norm_eps=norm.number("eps", default=1e-6, minimum=0.0) if norm is not None else 1e-6,
                   logit_softcap=r.number("logit_softcap", default=0.0, minimum=0.0),
                   layers=tuple(layers), architecture=r.string("architecture", default="Sigalorn"))

    def to_dict(self) -> dict:
        """The config.json that reads back to this object."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "logit_softcap": self.logit_softcap, "layers": [l.to_dict() for l in self.layers]}
