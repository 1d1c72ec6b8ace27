"""Arrangements: how a block wires its norms, mixer and feed-forward.

"pre_norm": h = x + mixer(norm(x)); out = h + ffn(norm(h)) (the reference's
`Layer::forward`, src/model.rs:556-585), with the reference's optional norms of the
mixer's and the feed-forward's output before each addition (src/model.rs:571, 581;
LFM2 uses neither).  The residual stream is float32; each sub-layer's output stays pending and is
added by the next norm's kernel, together with the norm it still has to pass through when
the block has one after the sub-layer.  A block without a feed-forward is its first half.
A block may scale each sub-layer's output channel by channel before the addition (a learned
vector per sub-layer and one factor for the whole model); the scale travels with the pending
rows and is applied by the same kernel.
"""
from __future__ import annotations

from .base import (Arrangement, Stream, feed_forward_class, mixer_class, norm_class,
                   register_arrangement)
import torch

from .spec import BlockSpec, ParamDecl


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def norm_tensor_names(norm, name):
    """{local name: name in the file} of a norm whose place was given `name`: one name is
    the weight's; a mapping is taken as it is."""
    if isinstance(name, str):
        return {"weight": name}
    return dict(name)


def norm_params(norm, name):
    decls = norm_class(norm.kind).params(norm)
    names = norm_tensor_names(norm, name)
    if set(names) != set(decls):
        raise ValueError(f"a {norm.kind} norm has tensors {sorted(decls)}, "
                         f"but names were given for {sorted(names)}")
    return {names[k]: d for k, d in decls.items()}


def build_norm(norm, name, tensors, ops, dtype):
    names = norm_tensor_names(norm, name)
    return norm_class(norm.kind)(norm, {k: tensors[n] for k, n in names.items()}, ops, dtype)


def stream_options(stream: Stream) -> dict:
    """What a norm's `add_norm` has to be told beyond the pending rows: their scale and a vector
    still to be added.  Only norms that take these options are ever given them."""
    options = {}
    if stream.pending_scale is not None and stream.pending is not None:
        options["delta_scale"] = stream.pending_scale
    if stream.pending_add is not None:
        options["add"] = stream.pending_add
    return options


class PreNormBlock(Arrangement):
    REQUIRED = ("mixer", "ffn")
    OPTIONAL = ("post_mixer", "post_ffn")

    @staticmethod
    def _check(spec: BlockSpec):
        places = PreNormBlock.REQUIRED + PreNormBlock.OPTIONAL
        for place in PreNormBlock.REQUIRED:
            if place == "ffn" and spec.feed_forward is None:
                continue
            if place not in spec.norms:
                raise ValueError(f"a pre_norm block needs a norm at {place!r}")
        for place in spec.norms:
            if spec.feed_forward is None and place in ("ffn", "post_ffn"):
                raise ValueError(f"a block without a feed-forward has no place {place!r}")
            if place not in places:
                raise ValueError(f"a pre_norm block has no place {place!r} for a norm "
                                 f"(places: {', '.join(places)})")

    @staticmethod
    def params(spec: BlockSpec, owns_cache: bool = True):
        """Full tensor names -> declarations for one block."""
        PreNormBlock._check(spec)
        out = {}
        mixer = mixer_class(spec.mixer.kind)
        mixer_params = mixer.params(spec.mixer, owns_cache)
        for k, d in mixer_params.items():
            out[spec.mixer_prefix + k] = d
        if spec.feed_forward is not None:
            ff = feed_forward_class(spec.feed_forward.kind).params(spec.feed_forward)
            for k, d in ff.items():
                out[spec.ffn_prefix + k] = d
        for norm, name in spec.norms.values():
            out.update(norm_params(norm, name))
        for place, name in spec.layer_scale.items():
            if place not in ("mixer", "ffn") or (place == "ffn" and spec.feed_forward is None):
                raise ValueError(f"a pre_norm block has no sub-layer {place!r} to scale")
            out[name] = ParamDecl((spec.mixer.hidden,), "norm")
        return out

    def __init__(self, spec: BlockSpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.mixer = mixer_class(spec.mixer.kind)(
            spec.mixer, _sub(tensors, spec.mixer_prefix), ops, dtype)
        self.feed_forward = None if spec.feed_forward is None else \
            feed_forward_class(spec.feed_forward.kind)(
                spec.feed_forward, _sub(tensors, spec.ffn_prefix), ops, dtype)

        def build(place):
            if place not in spec.norms:
                return None
            norm, name = spec.norms[place]
            return build_norm(norm, name, tensors, ops, dtype)

        self.mixer_norm, self.ffn_norm = build("mixer"), build("ffn")
        self.post_mixer, self.post_ffn = build("post_mixer"), build("post_ffn")

        def scale(place):
            """float32 [hidden]: residual_scale times the sub-layer's learned scale, or None."""
            name = spec.layer_scale.get(place)
            if name is None and spec.residual_scale == 1.0:
                return None
            if name is None:
                some = next(iter(tensors.values()))
                return torch.full((spec.mixer.hidden,), float(spec.residual_scale),
                                  dtype=torch.float32, device=some.device)
            return (tensors[name].to(torch.float32) * float(spec.residual_scale)).contiguous()

        self.mixer_scale, self.ffn_scale = scale("mixer"), scale("ffn")

    def forward(self, stream: Stream, ctx, cache) -> Stream:
        normed = self.mixer_norm.add_norm(stream.resid, stream.pending, ctx,
                                          delta_norm=stream.pending_norm, **stream_options(stream))
        mixed = self.mixer.forward(normed, ctx, cache)
        if self.feed_forward is None:
            return Stream(stream.resid, mixed, self.post_mixer, pending_scale=self.mixer_scale)
        options = {} if self.mixer_scale is None else {"delta_scale": self.mixer_scale}
        normed2 = self.ffn_norm.add_norm(stream.resid, mixed, ctx, delta_norm=self.post_mixer,
                                         **options)
        out = self.feed_forward.forward(normed2, ctx)
        return Stream(stream.resid, out, self.post_ffn, pending_scale=self.ffn_scale)


register_arrangement("pre_norm", PreNormBlock)
