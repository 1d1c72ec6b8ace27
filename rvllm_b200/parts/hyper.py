"""Hyper-connections: a pre-norm block over several copies of the residual.

Instead of one residual x there are S streams x_1 .. x_S per token, all equal to the
embedding output at the start.  Sub-layer q of a block has three small tensors, a [S], b [S]
and M [S, S] (indexed [from, to]):

    u   = sum_s a[s] x_s                      what the sub-layer reads
    y   = sublayer(norm(u))
    x_t <- sum_s M[s, t] x_s + b[t] y         all streams at once, from the old ones

and after the last block the model's norm reads the plain sum of the streams.  (The idea of
"Hyper-Connections", Zhu et al., with weights that do not depend on the input.)

The streams are one float32 tensor [N, S, W].  As with the single residual, a sub-layer's
output stays pending: the write-back with M and b, the next read-in with its a and the norm
are one kernel (`ops.hyper_norm`), so the streams are read and written once per sub-layer.
Before the first block the streams are the embedding rows [N, W] themselves; the first
kernel reads them as S equal streams.
"""
from __future__ import annotations

import torch

from .base import (Arrangement, Stream, feed_forward_class, mixer_class, register_arrangement)
from .block import _sub, build_norm, norm_params
from .norm import RMSNorm
from .spec import BlockSpec, ParamDecl


def hyper_between(ops, stream: Stream, in_w, norm, dtype, streams: int, rows=None):
    """Write the pending output back into the streams, read in with `in_w` (None: the plain
    sum) and normalise.  Returns (streams tensor, normalised rows).  With `rows` only those
    rows are formed and the streams stay as they are."""
    if not isinstance(norm, RMSNorm):
        raise ValueError("hyper-connections read through an RMSNorm")
    src = stream.resid
    n = src.shape[0] if rows is None else rows.shape[0]
    out = ops.new_rows(n, norm.spec.size, dtype, src.device)
    dst = None
    if rows is None:
        dst = src if src.dim() == 3 else torch.empty(
            (src.shape[0], streams, src.shape[1]), dtype=torch.float32, device=src.device)
    mix, out_w = stream.pending_hyper if stream.pending is not None else (None, None)
    if in_w is None:
        in_w = torch.ones(streams, dtype=torch.float32, device=src.device) \
            if src.dim() == 2 else None
    ops.hyper_norm(src, dst, stream.pending, mix, out_w, in_w, norm.weight, norm.spec.eps, out,
                   rows)
    return (dst if dst is not None else src), out


class HyperPreNormBlock(Arrangement):
    PLACES = ("mixer", "ffn")

    @staticmethod
    def _check(spec: BlockSpec):
        if spec.streams < 1:
            raise ValueError(f"a block cannot have {spec.streams} residual streams")
        for place in HyperPreNormBlock.PLACES:
            if place == "ffn" and spec.feed_forward is None:
                continue
            if place not in spec.norms or place not in spec.hyper:
                raise ValueError(f"a hyper_pre_norm block needs a norm and stream weights "
                                 f"at {place!r}")
        for place in spec.norms:
            if place not in HyperPreNormBlock.PLACES or \
                    (place == "ffn" and spec.feed_forward is None):
                raise ValueError(f"a hyper_pre_norm block has no place {place!r} for a norm")

    @staticmethod
    def params(spec: BlockSpec, owns_cache: bool = True):
        HyperPreNormBlock._check(spec)
        out = {}
        for k, d in mixer_class(spec.mixer.kind).params(spec.mixer, owns_cache).items():
            out[spec.mixer_prefix + k] = d
        if spec.feed_forward is not None:
            for k, d in feed_forward_class(spec.feed_forward.kind).params(
                    spec.feed_forward).items():
                out[spec.ffn_prefix + k] = d
        s = spec.streams
        for place, (norm, name) in spec.norms.items():
            out.update(norm_params(norm, name))
            prefix = spec.hyper[place]
            out[prefix + ".in"] = ParamDecl((s,), "normal", mean=1.0 / s, std=0.3 / s)
            out[prefix + ".out"] = ParamDecl((s,), "normal", mean=1.0, std=0.3)
            out[prefix + ".mix"] = ParamDecl((s, s), "normal", mean=1.0 / s, std=0.5 / s)
        return out

    def __init__(self, spec: BlockSpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        self.mixer = mixer_class(spec.mixer.kind)(
            spec.mixer, _sub(tensors, spec.mixer_prefix), ops, dtype)
        self.feed_forward = None if spec.feed_forward is None else \
            feed_forward_class(spec.feed_forward.kind)(
                spec.feed_forward, _sub(tensors, spec.ffn_prefix), ops, dtype)
        self.norms, self.weights = {}, {}
        for place, (norm, name) in spec.norms.items():
            self.norms[place] = build_norm(norm, name, tensors, ops, dtype)
            prefix = spec.hyper[place]
            self.weights[place] = tuple(
                tensors[prefix + k].to(torch.float32).contiguous() for k in (".in", ".mix", ".out"))

    def _sublayer(self, stream: Stream, place: str, run, ctx) -> Stream:
        in_w, mix, out_w = self.weights[place]
        resid, normed = hyper_between(self.ops, stream, in_w, self.norms[place], self.dtype,
                                      self.spec.streams)
        return Stream(resid, run(normed), pending_hyper=(mix, out_w))

    def forward(self, stream: Stream, ctx, cache) -> Stream:
        stream = self._sublayer(stream, "mixer", lambda h: self.mixer.forward(h, ctx, cache), ctx)
        if self.feed_forward is not None:
            stream = self._sublayer(stream, "ffn", lambda h: self.feed_forward.forward(h, ctx), ctx)
        return stream


register_arrangement("hyper_pre_norm", HyperPreNormBlock)
