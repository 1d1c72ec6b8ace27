"""The Vifanex configuration: a list of layers over several residual streams, each layer a
windowed grouped-query attention or a gated delta rule, each with a dense or a
mixture-of-experts feed-forward of the clamped gated form, or none.

config.json of this design is nested:

    {"architecture": "Vifanex", "vocab": V, "width": W, "streams": S, "norm": {"eps": e},
     "embedding": {"scale": c}, "logit_softcap": c,
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s,
                           "mask": {"size": w}, "v_mix": true,
                           "rot": {"base": b, "dims": r,
                                   "scaling": {"factor": f, "low": l, "high": h, "original": n}}},
                 "mlp": {"kind": "dense", "ff": F, "limit": L}},
                {"type": "channel_delta",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps},
                 "mlp": {"kind": "moe", "expert": {"ff": F, "limit": L},
                         "router": {"experts": E, "top": k, "scale": c,
                                    "groups": {"count": g, "keep": m}},
                         "shared": {"ff": F, "limit": L}}}]}

Every size and constant is read from the file; a key that is absent means the thing does not
exist (no streams: one residual; no mask: every earlier key is seen; no rot: no rotation; no
scaling: plain frequencies; no v_mix: values stay; no groups: every expert can be chosen; no
shared: no shared expert; mlp null: the layer is its mixer alone; no embedding scale, no
logit_softcap: left out).  Two sizes are in no key: the ranks of the delta rule's decay and
gate products.  They are the shapes of the tensors `l<i>.mix.a1` and `l<i>.mix.g1`
(`with_tensor_shapes`); a configuration made here may name them as `decay_rank` and
`gate_rank` in the mixer.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from ..errors import ConfigError
from .base import Reader

ATTENTION = "attention"
DELTA = "channel_delta"


@dataclass(frozen=True)
class VifanexGlu:
    ff: int
    limit: float


@dataclass(frozen=True)
class VifanexMlp:
    kind: str                          # "dense" or "moe"
    ff: int
    limit: float
    experts: int = 0
    top: int = 0
    route_scale: Optional[float] = None
    groups: int = 1
    keep: int = 1
    grouped: bool = False              # whether config.json had a "groups" object
    shared: Optional[VifanexGlu] = None


@dataclass(frozen=True)
class VifanexLayer:
    type: str
    mlp: Optional[VifanexMlp]
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    # attention
    scale: float = 0.0
    window: Optional[int] = None
    rot_dims: int = 0
    rot_base: float = 0.0
    rot_scaling: Optional[Tuple[float, float, float, int]] = None   # factor, low, high, original
    v_mix: bool = False
    # channel_delta
    taps: int = 0
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None


def _glu(entry, at) -> VifanexGlu:
    r = Reader(entry, at)
    limit = r.float("limit")
    if not limit > 0:
        raise ConfigError(f"{at}: key 'limit' must be positive, got {limit}")
    return VifanexGlu(r.int("ff", minimum=1), limit)


def _mlp(entry, at) -> VifanexMlp:
    kind = Reader(entry, at).str("kind")
    if kind == "dense":
        g = _glu(entry, at)
        return VifanexMlp("dense", g.ff, g.limit)
    if kind != "moe":
        raise ConfigError(f"{at}: unknown kind {kind!r} (known: 'dense', 'moe')")
    if not isinstance(entry.get("expert"), dict) or not isinstance(entry.get("router"), dict):
        raise ConfigError(f"{at}: a mixture needs the objects 'expert' and 'router'")
    g = _glu(entry["expert"], at + ".expert")
    rr = Reader(entry["router"], at + ".router")
    experts, top = rr.int("experts", minimum=1), rr.int("top", minimum=1)
    groups, keep, grouped = 1, 1, False
    if entry["router"].get("groups") is not None:
        gr = Reader(entry["router"]["groups"], at + ".router.groups")
        groups, keep, grouped = gr.int("count", minimum=1), gr.int("keep", minimum=1), True
    if top > experts:
        raise ConfigError(f"{at}: top {top} is more than the {experts} experts")
    if experts % groups or keep > groups or keep * (experts // groups) < top:
        raise ConfigError(f"{at}: {experts} experts in {groups} groups of which {keep} are kept "
                          f"cannot give {top} experts a token")
    shared = _glu(entry["shared"], at + ".shared") if entry.get("shared") is not None else None
    return VifanexMlp("moe", g.ff, g.limit, experts, top, rr.optional_float("scale"), groups,
                      keep, grouped, shared)


def _layer(entry, at) -> VifanexLayer:
    kind = Reader(entry, at).str("type")
    mlp = _mlp(entry["mlp"], at + ".mlp") if entry.get("mlp") is not None else None
    if not isinstance(entry.get("mixer"), dict):
        raise ConfigError(f"{at}: missing key 'mixer'")
    m = Reader(entry["mixer"], at + ".mixer")
    common = dict(heads=m.int("heads", minimum=1), kv_heads=m.int("kv_heads", minimum=1),
                  dim=m.int("dim", minimum=1), vdim=m.int("vdim", minimum=1))
    if common["heads"] % common["kv_heads"]:
        raise ConfigError(f"{at}: invalid head counts: {common['heads']} heads, "
                          f"{common['kv_heads']} kv_heads")
    if kind == ATTENTION:
        window = None
        if entry["mixer"].get("mask") is not None:
            window = Reader(entry["mixer"]["mask"], at + ".mixer.mask").int("size", minimum=1)
        dims, base, scaling = 0, 0.0, None
        if entry["mixer"].get("rot") is not None:
            rot = entry["mixer"]["rot"]
            rr = Reader(rot, at + ".mixer.rot")
            dims, base = rr.int("dims", minimum=0), rr.float("base")
            if dims % 2 or dims > common["dim"] or (dims and common["dim"] % 2) or not base > 0:
                raise ConfigError(f"{at}: rot.dims {dims} must be even and within an even "
                                  f"head size ({common['dim']}), rot.base positive")
            if rot.get("scaling") is not None:
                sr = Reader(rot["scaling"], at + ".mixer.rot.scaling")
                scaling = (sr.float("factor"), sr.float("low"), sr.float("high"),
                           sr.int("original", minimum=1))
                if not (scaling[0] > 0 and scaling[2] > scaling[1]):
                    raise ConfigError(f"{at}: rot.scaling needs factor > 0 and high > low")
        return VifanexLayer(kind, mlp, scale=m.float("scale"), window=window, rot_dims=dims,
                            rot_base=base, rot_scaling=scaling, v_mix=m.bool("v_mix", False),
                            **common)
    if kind == DELTA:
        return VifanexLayer(kind, mlp, taps=m.int("conv", minimum=1),
                            decay_rank=m.optional_int("decay_rank", minimum=1),
                            gate_rank=m.optional_int("gate_rank", minimum=1), **common)
    raise ConfigError(f"{at}: unknown type {kind!r} (known: {ATTENTION!r}, {DELTA!r})")


@dataclass(frozen=True)
class VifanexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[VifanexLayer, ...]
    streams: Optional[int] = None
    embedding_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    torch_dtype: str = "bfloat16"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "VifanexConfig":
        r = Reader(data, where)
        if not isinstance(data.get("layers"), list) or not data["layers"]:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        if not isinstance(data.get("norm"), dict):
            raise ConfigError(f"{where}: missing key 'norm' (an object with 'eps')")
        layers = tuple(_layer(e, f"{where}: layers[{i}]") for i, e in enumerate(data["layers"]))
        mixing = [l for l in layers if l.v_mix]
        if any((l.kv_heads, l.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for l in mixing):
            raise ConfigError(f"{where}: layers with v_mix must agree in kv_heads and vdim")
        scale = None
        if data.get("embedding") is not None:
            scale = Reader(data["embedding"], where + ": embedding").optional_float("scale")
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "streams",
                 "embedding", "logit_softcap", "torch_dtype"}
        name = data.get("architecture")
        if not isinstance(name, str):
            archs = data.get("architectures")
            if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
                raise ConfigError(f"{where}: missing key 'architecture'")
            name = archs[0]
        return cls(architecture=name, vocab=r.int("vocab", minimum=1),
                   width=r.int("width", minimum=1),
                   norm_eps=Reader(data["norm"], where + ": norm").float("eps"), layers=layers,
                   streams=r.optional_int("streams", minimum=1), embedding_scale=scale,
                   logit_softcap=r.optional_float("logit_softcap"),
                   torch_dtype=r.str("torch_dtype", "bfloat16"),
                   extra={k: v for k, v in data.items() if k not in known})

    def with_tensor_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "VifanexConfig":
        """The configuration with the sizes that only the tensor file has: the ranks of each
        delta layer's decay and gate products (rows of `l<i>.mix.a1` and `l<i>.mix.g1`)."""
        layers = []
        for i, l in enumerate(self.layers):
            if l.type == DELTA:
                found = {}
                for key, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    shape = shapes.get(name)
                    have = getattr(l, key)
                    if shape is not None and len(shape) == 2:
                        if have is not None and have != shape[0]:
                            raise ConfigError(f"layers[{i}]: {key} is {have} but tensor {name} "
                                              f"has {shape[0]} rows")
                        found[key] = int(shape[0])
                    elif have is None:
                        raise ConfigError(f"layers[{i}]: the tensor file has no matrix {name} "
                                          f"to take {key} from")
                l = dataclasses.replace(l, **found)
            layers.append(l)
        return dataclasses.replace(self, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        layers = []
        for l in self.layers:
            mixer: Dict[str, Any] = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim,
                                     "vdim": l.vdim}
            if l.type == ATTENTION:
                mixer["scale"] = l.scale
                if l.window is not None:
                    mixer["mask"] = {"size": l.window}
                if l.rot_base:
                    rot: Dict[str, Any] = {"base": l.rot_base, "dims": l.rot_dims}
                    if l.rot_scaling is not None:
                        f, lo, hi, n = l.rot_scaling
                        rot["scaling"] = {"factor": f, "low": lo, "high": hi, "original": n}
                    mixer["rot"] = rot
                if l.v_mix:
                    mixer["v_mix"] = True
            else:
                mixer["conv"] = l.taps
                if l.decay_rank is not None:
                    mixer["decay_rank"] = l.decay_rank
                if l.gate_rank is not None:
                    mixer["gate_rank"] = l.gate_rank
            mlp = None
            if l.mlp is not None and l.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": l.mlp.ff, "limit": l.mlp.limit}
            elif l.mlp is not None:
                router: Dict[str, Any] = {"experts": l.mlp.experts, "top": l.mlp.top}
                if l.mlp.route_scale is not None:
                    router["scale"] = l.mlp.route_scale
                if l.mlp.grouped:
                    router["groups"] = {"count": l.mlp.groups, "keep": l.mlp.keep}
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff, "limit": l.mlp.limit},
                       "router": router}
                if l.mlp.shared is not None:
                    mlp["shared"] = {"ff": l.mlp.shared.ff, "limit": l.mlp.shared.limit}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width,
                 norm={"eps": self.norm_eps}, layers=layers, torch_dtype=self.torch_dtype)
        if self.streams is not None:
            d["streams"] = self.streams
        if self.embedding_scale is not None:
            d["embedding"] = {"scale": self.embedding_scale}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d
