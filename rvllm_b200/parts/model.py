"""The generic model: embedding, the blocks in their run order, final norm and head.

It executes a `ModelSpec` and knows no architecture.  In the reference this is
`Model::hidden` / `lm_head` / `forward_last` (src/model.rs:698-745): embed, run the
layers, keep only the rows whose logits are wanted, final norm, output matrix (the
embedding table when the model has no head of its own, src/weights.rs:339-346).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

import dataclasses

from .base import PagedNeed, Stream, arrangement_class, mixer_class, norm_class
from .block import build_norm, norm_params, stream_options
from .spec import ModelSpec, ParallelSpec, ParamDecl


def block_owns_cache(spec: ModelSpec) -> List[bool]:
    """For each block: does any of its calls own a cache (rather than read another's)?"""
    owns = [False] * len(spec.layers)
    for call in spec.order:
        if call.cache_of is None:
            owns[call.layer] = True
    return owns


def param_decls(spec: ModelSpec) -> Dict[str, ParamDecl]:
    """Every tensor the model reads, by its name in the file."""
    out: Dict[str, ParamDecl] = {
        spec.embedding_name: ParamDecl((spec.vocab_size, spec.hidden), "embedding"),
    }
    out.update(norm_params(spec.final_norm, spec.final_norm_name))
    if spec.embedding_norm is not None:
        out.update(norm_params(*spec.embedding_norm))
    for name, rows in added_rows(spec).items():
        out[name] = ParamDecl((rows, spec.hidden), "bias")
    if spec.head_name is not None:
        out[spec.head_name] = ParamDecl((spec.vocab_size, spec.hidden), "linear")
    used = {call.layer for call in spec.order}
    for i, (b, owns) in enumerate(zip(spec.layers, block_owns_cache(spec))):
        if i in used:
            out.update(arrangement_class(b.arrangement).params(b, owns))
    return out


def added_rows(spec: ModelSpec) -> Dict[str, int]:
    """{tensor name: rows} of the tensors whose rows calls of the run order add to the stream."""
    rows: Dict[str, int] = {}
    for call in spec.order:
        if call.add is not None:
            name, row = call.add
            if row < 0:
                raise ValueError(f"run order: row {row} of {name!r}")
            rows[name] = max(rows.get(name, 0), row + 1)
    return rows


def validate_order(spec: ModelSpec) -> None:
    for b in spec.layers:
        if b.streams != spec.streams:
            raise ValueError(f"a block keeps {b.streams} residual streams, "
                             f"the model {spec.streams}")
        if (b.arrangement == "hyper_pre_norm") != (spec.streams >= 1):
            raise ValueError("blocks with several residual streams are 'hyper_pre_norm' "
                             "blocks, and only they")
    for pos, call in enumerate(spec.order):
        if not 0 <= call.layer < len(spec.layers):
            raise ValueError(f"run order entry {pos} names layer {call.layer}, "
                             f"but the model has {len(spec.layers)} layers")
        if call.cache_of is not None:
            if not 0 <= call.cache_of < pos:
                raise ValueError(f"run order entry {pos} reads the cache of entry "
                                 f"{call.cache_of}, which does not run before it")
            src = spec.order[call.cache_of]
            if src.cache_of is not None:
                raise ValueError(f"run order entry {pos} reads the cache of entry "
                                 f"{call.cache_of}, which owns none")
            if any(isinstance(spec.layers[c.layer].mixer, ParallelSpec) for c in (call, src)):
                raise ValueError(f"run order entry {pos}: a mixer of several mixers keeps "
                                 f"caches of its own")
            a = mixer_class(spec.layers[call.layer].mixer.kind).cache_need(
                spec.layers[call.layer].mixer)
            b = mixer_class(spec.layers[src.layer].mixer.kind).cache_need(
                spec.layers[src.layer].mixer)
            same = a == b
            if isinstance(a, PagedNeed) and isinstance(b, PagedNeed):
                same = a.layout() == b.layout()       # their reach may differ: see cache_needs
            if not same:
                raise ValueError(f"run order entry {pos} reads the cache of entry "
                                 f"{call.cache_of}, whose cache has another shape")


class Model:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], ops, dtype):
        validate_order(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        self.embedding = tensors[spec.embedding_name].contiguous()
        self.head = (tensors[spec.head_name].contiguous() if spec.head_name is not None
                     else self.embedding)
        self.final_norm = build_norm(spec.final_norm, spec.final_norm_name, tensors, ops, dtype)
        self.embedding_norm = None
        if spec.embedding_norm is not None:
            self.embedding_norm = build_norm(*spec.embedding_norm, tensors, ops, dtype)
            if not hasattr(self.embedding_norm, "norm_f32"):
                raise ValueError(f"a {spec.embedding_norm[0].kind} norm cannot normalise the "
                                 f"embedding rows in float32")
        self.added = {name: tensors[name].to(torch.float32).contiguous()
                      for name in added_rows(spec)}
        used = {call.layer for call in spec.order}
        self.blocks = [arrangement_class(b.arrangement)(b, tensors, ops, dtype)
                       if i in used else None for i, b in enumerate(spec.layers)]
        self.device = self.embedding.device

    def cache_needs(self) -> List[Optional[object]]:
        """What each call of the run order has to remember (None: nothing of its own).
        A call that reads another call's pages may look further back than their owner (another
        window or chunk): the owner's pages are then kept for as long as the request lives."""
        needs = []
        for call in self.spec.order:
            m = self.spec.layers[call.layer].mixer
            need = mixer_class(m.kind).cache_need(m)
            if call.cache_of is None:
                needs.append(need)
                continue
            needs.append(None)
            own = needs[call.cache_of]
            if isinstance(own, PagedNeed) and isinstance(need, PagedNeed) and \
                    (own.window, own.chunk) != (need.window, need.chunk):
                needs[call.cache_of] = dataclasses.replace(own, window=None, chunk=None)
        return needs

    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the step's tokens; float32 logits [len(ctx.logit_rows), vocab]."""
        n = ctx.n_tokens
        resid = torch.empty((n, self.spec.hidden), dtype=torch.float32, device=self.device)
        self.ops.embed(self.embedding, ctx.token_ids, resid, self.spec.embedding_scale)
        if self.embedding_norm is not None:
            resid = self.embedding_norm.norm_f32(resid)
        stream = Stream(resid, None)
        for call, cache in zip(self.spec.order, caches):
            if call.add is not None:
                stream.pending_add = self.added[call.add[0]][call.add[1]]
            stream = self.blocks[call.layer].forward(stream, ctx, cache)
        if ctx.logit_rows.shape[0] == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32,
                               device=self.device)
        if self.spec.streams >= 1:
            from .hyper import hyper_between
            _, normed = hyper_between(self.ops, stream, None, self.final_norm, self.dtype,
                                      self.spec.streams, rows=ctx.logit_rows)
        else:
            normed = self.final_norm.add_norm(stream.resid, stream.pending, ctx,
                                              rows=ctx.logit_rows,
                                              delta_norm=stream.pending_norm,
                                              **stream_options(stream))
        logits = self.ops.linear(normed, self.head, out_dtype=torch.float32)
        if self.spec.logit_softcap:
            self.ops.softcap(logits, self.spec.logit_softcap)
        return logits
