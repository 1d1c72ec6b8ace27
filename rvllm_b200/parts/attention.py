"""Grouped-query attention over a paged cache.

In the reference's order (src/model.rs:591-653): q, k, v projections without bias;
per-head RMSNorm of q and k (src/model.rs:608-613); rotation of q and k; k and v
written into the cache at each token's (page, slot) (src/model.rs:631-640); softmax(q
k^T / sqrt(head_dim)) v over the keys at or before the query's position, query heads
[g*G, (g+1)*G) sharing key/value head g (src/model.rs:377-415); output projection.

What differs by design: q, k and v are one [(heads + 2 kv_heads) * head_dim, hidden]
matrix product; norm, rotation and the cache write are one kernel (for a few tokens: the
product's own epilogue); attention reads
the pages through the block table instead of gathering them into a dense batch
(src/kv_storage.rs:157-173), keeps no score matrix and needs no mask tensor
(src/model.rs:347-372): a key at position j is visible to a query at position p iff
j <= p, and with a window iff j > p - window.

A call whose cache belongs to another call (`cache.owns` false) has no k and v of
its own: it projects q only and reads the other call's pages.

Options of the spec, each off at its default.  A value head of its own size.  A sink: the
softmax's denominator holds one more term exp(sink) without a key or a value, a constant
(`sink_score`; 0 gives p_j = exp(s_j) / (1 + sum exp(s_j))) or a learned number per head
(`sinks`).  A unit norm of q and k (`qk_norm` of kind "rms_unit": x / sqrt(mean(x^2) + eps) per
head, no weight).  A query temperature (`q_temp` = (coef, every)): the query at position p is
multiplied by 1 + coef ln(floor((p + 1) / every) + 1), so scores grow slowly with the length
of the context.  With the unit norm, the temperature or a value size of its own, norm,
temperature and the cache write are `ops.qk_unit_write` after the one q|k|v product.  A gate
per head (`head_gate`): head j's result is multiplied by sigmoid(W_g x)_j before the output
product; W_g's rows ride at the end of the q|k|v product and `ops.head_gate` applies them.

A third form (`_prepared`), chosen by any of: biases on the q, k and v projections (`bias`); a
norm over the whole query projection and one over the whole key projection, before the split
into heads (`qk_norm` of kind "rms_full"); a rotation of neighbouring dimensions (position
kind "rope_pairs"); value mixing (`value_mix`): the first such call of a step keeps its values
("source"), every later one caches v <- (1 - l) v + l v_source with its learned scalar l.  The
q|k|v product stays float32 and one kernel (`ops.qkv_full_norm_rope_write`) adds the biases,
normalises, rotates, mixes and writes the cache.  A sink, a window and a value size of its own
go with it.
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, PagedNeed, position_class, register_mixer
from .spec import AttentionSpec, ParamDecl


class Attention(Mixer):
    @staticmethod
    def _names(spec):
        n = spec.names
        return {k: n.get(k, k + ".weight") for k in
                ("q_proj", "k_proj", "v_proj", "out_proj", "q_norm", "k_norm", "sink")} | \
            {"head_gate": n.get("head_gate", "g")} | \
            {k: n.get(k, d) for k, d in (("q_bias", "q_proj.bias"), ("k_bias", "k_proj.bias"),
                                         ("v_bias", "v_proj.bias"), ("vmix", "vmix"))}

    @staticmethod
    def params(spec: AttentionSpec, owns_cache: bool = True):
        n = Attention._names(spec)
        dv = spec.v_head_dim or spec.head_dim
        qd, kd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        p = {n["q_proj"]: ParamDecl((qd, spec.hidden), "linear"),
             n["out_proj"]: ParamDecl((spec.hidden, spec.num_heads * dv), "linear")}
        if owns_cache:
            p[n["k_proj"]] = ParamDecl((kd, spec.hidden), "linear")
            p[n["v_proj"]] = ParamDecl((spec.num_kv_heads * dv, spec.hidden), "linear")
        if Attention._weighted_norm(spec):
            full = spec.qk_norm.kind == "rms_full"
            p[n["q_norm"]] = ParamDecl((qd if full else spec.head_dim,), "norm")
            if owns_cache:
                p[n["k_norm"]] = ParamDecl((kd if full else spec.head_dim,), "norm")
        if spec.bias:
            p[n["q_bias"]] = ParamDecl((qd,), "bias")
            if owns_cache:
                p[n["k_bias"]] = ParamDecl((kd,), "bias")
                p[n["v_bias"]] = ParamDecl((spec.num_kv_heads * dv,), "bias")
        if spec.value_mix is not None:
            if spec.value_mix not in ("source", "mix"):
                raise ValueError(f"attention: value_mix is 'source' or 'mix', "
                                 f"got {spec.value_mix!r}")
            p[n["vmix"]] = ParamDecl((), "normal", mean=0.5, std=0.2)
        if spec.sinks:
            p[n["sink"]] = ParamDecl((spec.num_heads,), "normal", mean=0.0, std=1.0)
        if spec.head_gate:
            if Attention._prepared(spec):
                raise ValueError("attention: a gate per head goes with no bias, whole-projection "
                                 "norm, pairwise rotation or value mixing")
            p[n["head_gate"]] = ParamDecl((spec.num_heads, spec.hidden), "linear")
        return p

    @staticmethod
    def _weighted_norm(spec) -> bool:
        return spec.qk_norm is not None and spec.qk_norm.kind != "rms_unit"

    @staticmethod
    def _prepared(spec) -> bool:
        """Whether the layer takes the form served by `ops.qkv_full_norm_rope_write`."""
        return spec.bias or spec.value_mix is not None or spec.position.kind == "rope_pairs" \
            or (spec.qk_norm is not None and spec.qk_norm.kind == "rms_full")

    @staticmethod
    def _plain(spec) -> bool:
        """Whether the layer is the plain form that the fused q|k|v kernel serves."""
        return (not spec.v_head_dim or spec.v_head_dim == spec.head_dim) and \
            spec.q_temp is None and (spec.qk_norm is None or spec.qk_norm.kind != "rms_unit") \
            and not spec.head_gate

    @staticmethod
    def cache_need(spec: AttentionSpec):
        dv = spec.v_head_dim or spec.head_dim
        return PagedNeed(spec.num_kv_heads, spec.head_dim, spec.window,
                         v_head_dim=dv if dv != spec.head_dim else None)

    @staticmethod
    def workspace_bytes(spec: AttentionSpec, ops, max_requests: int, max_context: int) -> int:
        sizer = getattr(ops, "attention_scratch_bytes", None)
        if sizer is None:
            return 0
        return sizer(max_requests, spec.num_heads, max(spec.head_dim, spec.v_head_dim), max_context)

    def __init__(self, spec: AttentionSpec, tensors, ops, dtype):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"invalid attention head counts: {spec.num_heads} query, "
                             f"{spec.num_kv_heads} KV")
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        q = tensors[n["q_proj"]]
        self.has_kv = n["k_proj"] in tensors
        def fused(parts):
            """The matrices as one; with gate rows at the end, zero rows after them fill the
            product's width up to a multiple of the head size (of 8 at least), so that the rows
            keep the alignment and the shape that the tensor-core attention kernels read."""
            if not spec.head_gate:
                return torch.cat(parts, dim=0).contiguous()
            parts = parts + [tensors[n["head_gate"]].to(q.dtype)]
            rows = sum(p.shape[0] for p in parts)
            unit = spec.head_dim if spec.head_dim % 8 == 0 else 8
            fill = -rows % unit
            if fill:
                parts.append(torch.zeros((fill, spec.hidden), dtype=q.dtype, device=q.device))
            return torch.cat(parts, dim=0).contiguous()

        if self.has_kv:
            self.w_qkv = fused([q, tensors[n["k_proj"]].to(q.dtype),
                                tensors[n["v_proj"]].to(q.dtype)])
        else:
            self.w_qkv = fused([q])
        # a call that reads another call's pages multiplies q (and the gate) only
        self.w_q = self.w_qkv[:spec.num_heads * spec.head_dim] if not spec.head_gate else \
            fused([q])
        self.w_out = tensors[n["out_proj"]].contiguous()
        self.q_norm = self.k_norm = None
        self.v_dim = spec.v_head_dim or spec.head_dim
        self.sinks = None
        if spec.sinks and spec.sink_score is not None:
            raise ValueError("attention: a sink is a constant or learned, not both")
        if spec.sinks:
            self.sinks = tensors[n["sink"]].to(torch.float32).contiguous()
        elif spec.sink_score is not None:
            self.sinks = torch.full((spec.num_heads,), float(spec.sink_score),
                                    dtype=torch.float32, device=q.device)
        if self._weighted_norm(spec):
            self.q_norm = tensors[n["q_norm"]].to(torch.float32).contiguous()
            if self.has_kv:
                self.k_norm = tensors[n["k_norm"]].to(torch.float32).contiguous()
        self.position = position_class(spec.position.kind)(spec.position, q.device)
        self.bias = self.vmix = None
        if self._prepared(spec):
            self._check_prepared(spec)
            if spec.bias:
                self.bias = torch.cat([tensors[n[k]].to(torch.float32) for k in
                                       ("q_bias", "k_bias", "v_bias")]).contiguous()
            if spec.value_mix == "mix":
                self.vmix = tensors[n["vmix"]].to(torch.float32).reshape(1).contiguous()
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)

    def forward(self, normed, ctx, cache):
        s = self.spec
        owns = cache.owns
        if owns and not self.has_kv:
            raise ValueError("attention: this call owns a cache but the block has no "
                             "key and value projections")
        group = ctx.groups[cache.group]
        if self._prepared(s):
            return self._forward_prepared(normed, ctx, cache, group)
        if not self._plain(s):
            return self._forward_options(normed, ctx, cache, group)
        qkv = self.ops.linear_qk_norm_rope_write(
            normed, self.w_qkv if owns else self.w_q, s.num_heads,
            s.num_kv_heads if owns else 0, s.head_dim,
            self.q_norm, self.k_norm if owns else None, s.qk_norm.eps if s.qk_norm else 0.0,
            self.position.rotation_table(), ctx.positions, group.slot_mapping,
            cache.k if owns else None, cache.v if owns else None, out_dtype=self.dtype)
        out = self.ops.new_rows(normed.shape[0], s.num_heads * s.head_dim, self.dtype, normed.device)
        self.ops.paged_attention(qkv, s.num_heads, s.num_kv_heads, s.head_dim,
                                 cache.k, cache.v, ctx, group, self.scale, s.window, out,
                                 sinks=self.sinks)
        return self.ops.linear(out, self.w_out, out_dtype=self.dtype)

    def _forward_options(self, normed, ctx, cache, group):
        s = self.spec
        owns = cache.owns
        if self.q_norm is not None or s.position.kind != "none":
            raise ValueError("attention: a unit norm, a query temperature or a value size of "
                             "its own goes with neither a weighted q/k norm nor a rotation")
        kv = s.num_kv_heads if owns else 0
        rows = self.ops.linear(normed, self.w_qkv if owns else self.w_q, out_dtype=self.dtype)
        self.ops.qk_unit_write(rows, s.num_heads, kv, s.head_dim, self.v_dim,
                               s.qk_norm.eps if s.qk_norm is not None else None, s.q_temp,
                               ctx.positions, group.slot_mapping,
                               cache.k if owns else None, cache.v if owns else None)
        out = self.ops.new_rows(normed.shape[0], s.num_heads * self.v_dim, self.dtype,
                                normed.device)
        self.ops.paged_attention(rows, s.num_heads, s.num_kv_heads, s.head_dim,
                                 cache.k, cache.v, ctx, group, self.scale, s.window, out,
                                 sinks=self.sinks, v_head_dim=self.v_dim)
        if s.head_gate:
            self.ops.head_gate(out, s.num_heads, self.v_dim, rows,
                               s.num_heads * s.head_dim + kv * (s.head_dim + self.v_dim))
        return self.ops.linear(out, self.w_out, out_dtype=self.dtype)


    CARRY_VALUES = "attention.source_values"

    def _check_prepared(self, spec):
        if not self.has_kv:
            raise ValueError("attention: this form makes its own keys and values")
        if spec.q_temp is not None or (spec.qk_norm is not None and
                                       spec.qk_norm.kind not in ("rms_full",)):
            raise ValueError("attention: biases, a whole-projection norm, a pairwise rotation "
                             "and value mixing go with no other q/k norm and no temperature")
        if spec.position.kind not in ("rope_pairs", "none"):
            raise ValueError("attention: this form turns neighbouring dimensions or none")

    def _forward_prepared(self, normed, ctx, cache, group):
        s = self.spec
        if not cache.owns:
            raise ValueError("attention: this form makes its own keys and values")
        n = normed.shape[0]
        rows = self.ops.linear(normed, self.w_qkv, out_dtype=torch.float32)
        q = self.ops.new_rows(n, s.num_heads * s.head_dim, self.dtype, normed.device)
        first_in = first_out = None
        if s.value_mix == "source":
            first_out = torch.empty((n, s.num_kv_heads * self.v_dim), dtype=torch.float32,
                                    device=normed.device)
            ctx.carry[self.CARRY_VALUES] = first_out
        elif s.value_mix == "mix":
            first_in = ctx.carry.get(self.CARRY_VALUES)
            if first_in is None or first_in.shape != (n, s.num_kv_heads * self.v_dim):
                raise ValueError("attention: values are mixed with those of an earlier call of "
                                 "the step, and none of this shape ran")
        freq, rot_dims = (None, 0) if s.position.kind == "none" else self.position.frequencies()
        self.ops.qkv_full_norm_rope_write(
            rows, self.bias, s.num_heads, s.num_kv_heads, s.head_dim, self.v_dim, self.q_norm,
            self.k_norm, s.qk_norm.eps if s.qk_norm is not None else 0.0, freq, rot_dims,
            ctx.positions, group.slot_mapping, q, cache.k, cache.v, first_in, first_out, self.vmix)
        out = self.ops.new_rows(n, s.num_heads * self.v_dim, self.dtype, normed.device)
        self.ops.paged_attention(q, s.num_heads, s.num_kv_heads, s.head_dim, cache.k, cache.v,
                                 ctx, group, self.scale, s.window, out, sinks=self.sinks,
                                 v_head_dim=self.v_dim)
        return self.ops.linear(out, self.w_out, out_dtype=self.dtype)


register_mixer("attention", Attention)
