"""The Mevuvik configuration: a list of layers, each a latent attention (queries through a
latent of their own, a turned key part shared by the heads) or two mixers side by side (a gated
grouped-query attention without positions and a matrix memory with exponential gates), each
with a dense or a mixture-of-experts feed-forward or none; a stretch of layers may run several
times with the same weights.

config.json of this design is nested:

    {"architecture": "Mevuvik", "vocab": V, "width": W, "norm": {"eps": e},
     "residual_mult": r, "logit_softcap": c,
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "rot_dim": dr, "vdim": dv, "kv_rank": R,
                           "q_rank": Rq, "scale": s, "rot": {"base": t, "dims": dr}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s},
                           "right": {"heads": H, "dim": d, "vdim": dv, "gate_cap": c},
                           "left_scale": x, "right_scale": y},
                 "mlp": {"kind": "moe", "expert": {"ff": F},
                         "router": {"experts": E, "top": k, "scale": z}}}]}

Every size and constant is read from the file; a key that is absent means the thing does not
exist (no loop: every layer runs once; mlp null: the layer is its mixer alone; no
logit_softcap: logits stay as they are; no residual_mult: 1).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import Reader

LATENT = "latent_attention"
PARALLEL = "parallel"


@dataclass(frozen=True)
class MevuvikMlp:
    kind: str                        # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0


@dataclass(frozen=True)
class MevuvikLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float


@dataclass(frozen=True)
class MevuvikLeft:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float


@dataclass(frozen=True)
class MevuvikRight:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class MevuvikLayer:
    type: str
    mlp: Optional[MevuvikMlp]
    latent: Optional[MevuvikLatent] = None
    left: Optional[MevuvikLeft] = None
    right: Optional[MevuvikRight] = None
    left_scale: float = 1.0
    right_scale: float = 1.0


def _mlp(entry, at) -> MevuvikMlp:
    kind = Reader(entry, at).str("kind")
    if kind == "dense":
        return MevuvikMlp("dense", Reader(entry, at).int("ff", minimum=1))
    if kind != "moe":
        raise ConfigError(f"{at}: unknown kind {kind!r} (known: 'dense', 'moe')")
    if not isinstance(entry.get("expert"), dict) or not isinstance(entry.get("router"), dict):
        raise ConfigError(f"{at}: a mixture needs the objects 'expert' and 'router'")
    ff = Reader(entry["expert"], at + ".expert").int("ff", minimum=1)
    rr = Reader(entry["router"], at + ".router")
    experts, top = rr.int("experts", minimum=1), rr.int("top", minimum=1)
    if top > experts:
        raise ConfigError(f"{at}: top {top} is more than the {experts} experts")
    return MevuvikMlp("moe", ff, experts, top, rr.float("scale", 1.0))


def _latent(entry, at) -> MevuvikLatent:
    m = Reader(entry, at)
    rot_dim = m.int("rot_dim", minimum=0)
    base = 10000.0
    if rot_dim:
        if not isinstance(entry.get("rot"), dict):
            raise ConfigError(f"{at}: a turned part needs the object 'rot'")
        rot = Reader(entry["rot"], at + ".rot")
        base = rot.float("base")
        if rot.int("dims", rot_dim) != rot_dim:
            raise ConfigError(f"{at}: rot.dims must equal rot_dim (the whole part turns)")
        if rot_dim % 2:
            raise ConfigError(f"{at}: rot_dim must be even, got {rot_dim}")
    return MevuvikLatent(heads=m.int("heads", minimum=1), dim=m.int("dim", minimum=1),
                         rot_dim=rot_dim, vdim=m.int("vdim", minimum=1),
                         kv_rank=m.int("kv_rank", minimum=1), q_rank=m.int("q_rank", minimum=1),
                         scale=m.float("scale"), rot_base=base)


def _parallel(entry, at):
    for side in ("left", "right"):
        if not isinstance(entry.get(side), dict):
            raise ConfigError(f"{at}: missing key {side!r}")
    l, r = Reader(entry["left"], at + ".left"), Reader(entry["right"], at + ".right")
    left = MevuvikLeft(heads=l.int("heads", minimum=1), kv_heads=l.int("kv_heads", minimum=1),
                       dim=l.int("dim", minimum=1), vdim=l.int("vdim", minimum=1),
                       scale=l.float("scale"))
    if left.heads % left.kv_heads:
        raise ConfigError(f"{at}.left: invalid attention head counts: {left.heads} query, "
                          f"{left.kv_heads} KV")
    right = MevuvikRight(heads=r.int("heads", minimum=1), dim=r.int("dim", minimum=1),
                         vdim=r.int("vdim", minimum=1), gate_cap=r.float("gate_cap"))
    if not right.gate_cap > 0:
        raise ConfigError(f"{at}.right: gate_cap must be positive")
    m = Reader(entry, at)
    return left, right, m.float("left_scale", 1.0), m.float("right_scale", 1.0)


@dataclass(frozen=True)
class MevuvikConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[MevuvikLayer, ...]
    residual_mult: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)
    logit_softcap: Optional[float] = None
    torch_dtype: str = "bfloat16"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "MevuvikConfig":
        r = Reader(data, where)
        if not isinstance(data.get("layers"), list) or not data["layers"]:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        if not isinstance(data.get("norm"), dict):
            raise ConfigError(f"{where}: missing key 'norm' (an object with 'eps')")
        layers = []
        for i, entry in enumerate(data["layers"]):
            at = f"{where}: layers[{i}]"
            kind = Reader(entry, at).str("type")
            mlp = _mlp(entry["mlp"], at + ".mlp") if entry.get("mlp") is not None else None
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{at}: missing key 'mixer'")
            if kind == LATENT:
                layers.append(MevuvikLayer(kind, mlp, latent=_latent(entry["mixer"], at + ".mixer")))
            elif kind == PARALLEL:
                left, right, ls, rs = _parallel(entry["mixer"], at + ".mixer")
                layers.append(MevuvikLayer(kind, mlp, left=left, right=right, left_scale=ls,
                                           right_scale=rs))
            else:
                raise ConfigError(f"{at}: unknown type {kind!r} (known: {LATENT!r}, {PARALLEL!r})")
        loop = None
        if data.get("loop") is not None:
            lr = Reader(data["loop"], where + ": loop")
            loop = (lr.int("start", minimum=0), lr.int("stop", minimum=0),
                    lr.int("times", minimum=1))
            if not loop[0] < loop[1] <= len(layers):
                raise ConfigError(f"{where}: loop must name layers start < stop <= {len(layers)}")
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "loop",
                 "residual_mult", "logit_softcap", "torch_dtype"}
        name = data.get("architecture")
        if not isinstance(name, str):
            archs = data.get("architectures")
            if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
                raise ConfigError(f"{where}: missing key 'architecture'")
            name = archs[0]
        return cls(architecture=name, vocab=r.int("vocab", minimum=1),
                   width=r.int("width", minimum=1),
                   norm_eps=Reader(data["norm"], where + ": norm").float("eps"),
                   layers=tuple(layers), residual_mult=r.float("residual_mult", 1.0), loop=loop,
                   logit_softcap=r.optional_float("logit_softcap"),
                   torch_dtype=r.str("torch_dtype", "bfloat16"),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        layers = []
        for l in self.layers:
            if l.type == LATENT:
                m = l.latent
                mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim,
                                         "vdim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank,
                                         "scale": m.scale}
                if m.rot_dim:
                    mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dim}
            else:
                a, b = l.left, l.right
                mixer = {"left": {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim,
                                  "vdim": a.vdim, "scale": a.scale},
                         "right": {"heads": b.heads, "dim": b.dim, "vdim": b.vdim,
                                   "gate_cap": b.gate_cap},
                         "left_scale": l.left_scale, "right_scale": l.right_scale}
            mlp = None
            if l.mlp is not None and l.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": l.mlp.ff}
            elif l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                       "router": {"experts": l.mlp.experts, "top": l.mlp.top,
                                  "scale": l.mlp.route_scale}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width,
                 norm={"eps": self.norm_eps}, residual_mult=self.residual_mult, layers=layers,
                 torch_dtype=self.torch_dtype)
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d
