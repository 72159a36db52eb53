"""Nosolix's configuration: the keys of its config.json, typed.

config.json names the architecture under `architecture` and nests its values:

    vocab, width, embedding.scale, norm.eps,
    layers: [ {type: "mamba1" | "parallel", mixer: {...}, mlp: {...} | null}, ... ]

A "mamba1" mixer gives inner, state, dt_rank and conv (the taps of its short convolution).  A "parallel" mixer
gives two mixers that read the same input: `left`, attention over a sliding window (heads, kv_heads, dim, vdim,
scale, mask.size, rot.base, rot.dims and optionally rot.scaling with factor, low, high, original), and `right`, a
state-space-duality mixer (heads, vdim, state, groups, norm_groups, conv).  A feed-forward is dense
({kind: "dense", ff}) or a mixture of experts ({kind: "moe", expert: {ff, limit}, router: {experts, top, scale,
groups: {count, keep}}, shared: {ff, limit} | null}).  Every size and constant of a model comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ConfigReader
from .sigalorn import DenseSpec, _sub


@dataclass(frozen=True)
class SelectiveScanSpec:
    inner: int
    state: int
    dt_rank: int
    conv: int

    def to_dict(self) -> dict:
        return {"inner": self.inner, "state": self.state, "dt_rank": self.dt_rank, "conv": self.conv}


@dataclass(frozen=True)
class FrequencyScaling:
    factor: float
    low: float
    high: float
    original: float

    def to_dict(self) -> dict:
        return {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}


@dataclass(frozen=True)
class WindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                    # 0: every earlier key is seen
    rot_base: float
    rot_dims: int
    rot_scaling: FrequencyScaling | None = None

    def to_dict(self) -> dict:
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = self.rot_scaling.to_dict()
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": rot}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class DualitySpec:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "norm_groups": self.norm_groups, "conv": self.conv}


@dataclass(frozen=True)
class ParallelSpec:
    left: WindowAttentionSpec
    right: DualitySpec

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class ExpertSpec:
    ff: int
    limit: float

    def to_dict(self) -> dict:
        return {"ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class MoeSpec:
    experts: int
    top: int
    scale: float
    group_count: int
    group_keep: int
    expert: ExpertSpec
    shared: ExpertSpec | None
    kind: str = "moe"

    def to_dict(self) -> dict:
        return {"kind": self.kind, "expert": self.expert.to_dict(),
                "router": {"experts": self.experts, "top": self.top, "scale": self.scale,
                           "groups": {"count": self.group_count, "keep": self.group_keep}},
                "shared": self.shared.to_dict() if self.shared is not None else None}


@dataclass(frozen=True)
class LayerSpec:
    type: str                      # "mamba1" | "parallel"
    mixer: Any
    mlp: Any                       # DenseSpec | MoeSpec | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


def _selective(r: ConfigReader) -> SelectiveScanSpec:
    return SelectiveScanSpec(inner=r.integer("inner", minimum=1), state=r.integer("state", minimum=1),
                             dt_rank=r.integer("dt_rank", minimum=1), conv=r.integer("conv", minimum=1))


def _window_attention(r: ConfigReader) -> WindowAttentionSpec:
    heads = r.integer("heads", minimum=1)
    kv = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: heads ({heads}) not divisible by kv_heads ({kv})")
    dim = r.integer("dim", minimum=1)
    vdim = r.integer("vdim", default=dim, minimum=1)
    rot = _sub(r, "rot", required=False)
    rot_dims, rot_base, scaling = 0, 10000.0, None
    if rot is not None:
        rot_dims = rot.integer("dims", default=dim, minimum=0)
        rot_base = rot.number("base", default=10000.0, minimum=0.0, exclusive=True)
        sc = _sub(rot, "scaling", required=False)
        if sc is not None:
            scaling = FrequencyScaling(factor=sc.number("factor", minimum=0.0, exclusive=True), low=sc.number("low"),
                                       high=sc.number("high"), original=sc.number("original", minimum=0.0, exclusive=True))
            if not scaling.high > scaling.low > 0:
                raise ConfigError(f"{r.where}: rot.scaling needs 0 < low < high, found {scaling.low}, {scaling.high}")
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{r.where}: rot.dims must be even and at most dim ({dim}), found {rot_dims}")
    mask = _sub(r, "mask", required=False)
    window = mask.integer("size", default=0, minimum=0) if mask is not None else 0
    return WindowAttentionSpec(heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                               scale=r.number("scale", default=dim ** -0.5, minimum=0.0, exclusive=True), window=window,
                               rot_base=rot_base, rot_dims=rot_dims, rot_scaling=scaling)


def _duality(r: ConfigReader) -> DualitySpec:
    heads = r.integer("heads", minimum=1)
    groups = r.integer("groups", default=1, minimum=1)
    if heads % groups:
        raise ConfigError(f"{r.where}: heads ({heads}) not divisible by groups ({groups})")
    vdim = r.integer("vdim", minimum=1)
    parts = r.integer("norm_groups", default=1, minimum=1)
    if (heads * vdim) % parts:
        raise ConfigError(f"{r.where}: heads x vdim ({heads * vdim}) not divisible by norm_groups ({parts})")
    return DualitySpec(heads=heads, vdim=vdim, state=r.integer("state", minimum=1), groups=groups, norm_groups=parts,
                       conv=r.integer("conv", minimum=1))


def _expert(r: ConfigReader) -> ExpertSpec:
    return ExpertSpec(ff=r.integer("ff", minimum=1), limit=r.number("limit", minimum=0.0, exclusive=True))


def _mlp(fr: ConfigReader):
    kind = fr.string("kind", default="dense")
    if kind == "dense":
        return DenseSpec(ff=fr.integer("ff", minimum=1), kind=kind)
    if kind != "moe":
        raise ConfigError(f"{fr.where}: unknown kind {kind!r} (known: dense, moe)")
    rr = _sub(fr, "router")
    experts = rr.integer("experts", minimum=1)
    top = rr.integer("top", minimum=1)
    gr = _sub(rr, "groups", required=False)
    count = gr.integer("count", default=1, minimum=1) if gr is not None else 1
    keep = gr.integer("keep", default=count, minimum=1) if gr is not None else 1
    if experts % count or keep > count:
        raise ConfigError(f"{fr.where}: {experts} experts in {count} groups of which {keep} are kept")
    if top > keep * (experts // count):
        raise ConfigError(f"{fr.where}: top ({top}) exceeds the experts of the kept groups ({keep * (experts // count)})")
    sh = _sub(fr, "shared", required=False)
    return MoeSpec(experts=experts, top=top, scale=rr.number("scale", default=1.0), group_count=count, group_keep=keep,
                   expert=_expert(_sub(fr, "expert")), shared=_expert(sh) if sh is not None else None)


@dataclass(frozen=True)
class NosolixConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple[LayerSpec, ...]
    architecture: str = "Nosolix"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "NosolixConfig":
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
            if kind == "mamba1":
                mixer = _selective(mr)
            elif kind == "parallel":
                left, right = _sub(mr, "left"), _sub(mr, "right")
                left.where, right.where = f"{mr.where}.left", f"{mr.where}.right"
                mixer = ParallelSpec(_window_attention(left), _duality(right))
            else:
                raise ConfigError(f"{where}: layers[{i}]: unknown layer type {kind!r} (known: mamba1, parallel)")
            fr = _sub(lr, "mlp", required=False)
            if fr is not None:
                fr.where = f"{where}: layers[{i}].mlp"
            layers.append(LayerSpec(kind, mixer, _mlp(fr) if fr is not None else None))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   embedding_scale=emb.number("scale", default=1.0) if emb is not None else 1.0,
                   norm_eps=norm.number("eps", default=1e-6, minimum=0.0) if norm is not None else 1e-6,
                   layers=tuple(layers), architecture=r.string("architecture", default="Nosolix"))

    def to_dict(self) -> dict:
        """The config.json that reads back to this object."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [l.to_dict() for l in self.layers]}
