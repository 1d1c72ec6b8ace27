"""Several mixers side by side (`ParallelSpec`): every branch reads the same normalised input,
keeps a cache of its own kind (pages, a state record, nothing), and the mixer's output is

    y = sum_j scale_j * branch_j(x)

Any registered mixer can be a branch; a branch's tensors lie under its prefix below the
mixer's own.  The sum of two branches is one elementwise kernel in float32 arithmetic; more
branches are added one at a time.
"""
from __future__ import annotations

from .base import Mixer, SeveralNeeds, mixer_class, register_mixer
from .spec import ParallelSpec


class Parallel(Mixer):
    @staticmethod
    def _check(spec: ParallelSpec):
        n = len(spec.branches)
        if n < 1 or len(spec.scales) != n or len(spec.prefixes) != n:
            raise ValueError("parallel: one factor and one prefix per branch, at least one branch")
        if len(set(spec.prefixes)) != n:
            raise ValueError("parallel: two branches share a prefix")
        for b in spec.branches:
            if b.hidden != spec.hidden:
                raise ValueError("parallel: a branch has another width than the mixer")

    @staticmethod
    def params(spec: ParallelSpec, owns_cache: bool = True):
        Parallel._check(spec)
        out = {}
        for b, prefix in zip(spec.branches, spec.prefixes):
            for k, d in mixer_class(b.kind).params(b, True).items():
                out[prefix + k] = d
        return out

    @staticmethod
    def cache_need(spec: ParallelSpec):
        return SeveralNeeds(tuple(mixer_class(b.kind).cache_need(b) for b in spec.branches))

    @staticmethod
    def workspace_bytes(spec: ParallelSpec, ops, max_requests: int, max_context: int) -> int:
        return max(mixer_class(b.kind).workspace_bytes(b, ops, max_requests, max_context)
                   for b in spec.branches)

    def __init__(self, spec: ParallelSpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        self.branches = []
        for b, prefix in zip(spec.branches, spec.prefixes):
            sub = {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
            self.branches.append(mixer_class(b.kind)(b, sub, ops, dtype))

    def forward(self, normed, ctx, cache):
        if cache is None or cache.parts is None or len(cache.parts) != len(self.branches):
            raise ValueError("parallel: the call's cache has no part per branch")
        outs = [b.forward(normed, ctx, part) for b, part in zip(self.branches, cache.parts)]
        scales = self.spec.scales
        if len(outs) == 1:
            outs.append(outs[0])
            scales = (scales[0], 0.0)
        total = self.ops.new_rows(normed.shape[0], self.spec.hidden, self.dtype, normed.device)
        self.ops.weighted_sum(outs[0], scales[0], outs[1], scales[1], total)
        for y, s in zip(outs[2:], scales[2:]):
            self.ops.weighted_sum(total, 1.0, y, s, total)
        return total


register_mixer("parallel", Parallel)
