"""Attention over one small latent row per token (`LatentAttentionSpec`).

A token leaves c = rmsnorm(W_dkv x) * w_c, kv_rank numbers, in the cache; head h's key and
value of that token are W_uk[h] c and W_uv[h] c.  For the query at position p of head h, over
the keys j <= p:

    s_h[j] = scale * <q_h, W_uk[h] c_j>  =  scale * <W_uk[h]^T q_h, c_j>
    w_h[j] = exp(s_h[j]) / (sum_j' exp(s_h[j']) + exp(sink_h))                 (sinks)
    o_h    = sum_j w_h[j] W_uv[h] c_j    =  W_uv[h] (sum_j w_h[j] c_j)
    y      = W_o (concat_h o_h * sigmoid(W_g x))                               (out_gate)

The right-hand forms are what runs: the query is carried into the latent space (one small
product per head), attention is then an ordinary paged attention with ONE key/value head of
size kv_rank shared by all query heads, whose values are its keys, and the result is carried
out of the latent space by W_uv.  Nothing but c is ever stored or re-expanded, whatever the
length of the context or the cut of a prompt, so prompts, portions and single tokens are one
code path.  q, the latent row and the gate are one matrix product; the norm of the latent row
and its cache write are one kernel.

A call whose cache belongs to another call has no W_dkv: it reads that call's latent rows
with its own W_uk, W_uv, queries, sinks and gate.

Two options of the spec.  `q_rank`: queries pass a latent of their own, q = W_uq rmsnorm(W_dq x).
`rot_dim`: a head's query is [d plain | rot_dim turned] dimensions, W_dkv gives rot_dim more
values per token that are turned by the position and shared by all heads as a second key part:

    s_h[j] = scale * ( <W_uk[h]^T q_h[:d], c_j> + <turn_p(q_h[d:]), turn_j(k_rot_j)> )

The page slot of a token then holds [c_j | turn_j(k_rot_j)], kv_rank + rot_dim numbers, and the
query carried into that space is [W_uk[h]^T q_h[:d] | turn_p(q_h[d:])]: one per-head product
with the matrix [[W_uk[h], 0], [0, 1]].  Attention is the same paged attention with one shared
head of size kv_rank + rot_dim whose values are its keys; the turned part of its result meets
zero rows of the matrix that carries it out ([W_uv[h]^T; 0]), so nothing but sizes changed.
W_dq and W_dkv are one product; the two norms, the turn of the key part and the cache write
are one kernel (`ops.latent_prepare`), the turn of the queries another (`ops.rope_heads`).
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, PagedNeed, position_class, register_mixer
from .spec import LatentAttentionSpec, ParamDecl, PositionSpec


class LatentAttention(Mixer):
    LOCAL = ("q", "dkv", "dkv_norm", "uk", "uv", "o", "sink", "g", "dq", "dq_norm", "uq")

    @staticmethod
    def _names(spec):
        return {k: spec.names.get(k, k) for k in LatentAttention.LOCAL}

    @staticmethod
    def params(spec: LatentAttentionSpec, owns_cache: bool = True):
        n = LatentAttention._names(spec)
        H, d, dv, R = spec.num_heads, spec.head_dim, spec.v_head_dim, spec.kv_rank
        rot, qr = spec.rot_dim, spec.q_rank
        if rot < 0 or rot % 2 or qr < 0:
            raise ValueError("latent attention: the turned part has an even size, and ranks "
                             "are not negative")
        p = {n["uk"]: ParamDecl((H * d, R), "normal", mean=0.0, std=R ** -0.5),
             n["uv"]: ParamDecl((H * dv, R), "normal", mean=0.0, std=R ** -0.5),
             n["o"]: ParamDecl((spec.hidden, H * dv), "linear")}
        if qr:
            p[n["dq"]] = ParamDecl((qr, spec.hidden), "linear")
            p[n["dq_norm"]] = ParamDecl((qr,), "norm")
            p[n["uq"]] = ParamDecl((H * (d + rot), qr), "normal", mean=0.0, std=qr ** -0.5)
        else:
            p[n["q"]] = ParamDecl((H * (d + rot), spec.hidden), "linear")
        if owns_cache:
            p[n["dkv"]] = ParamDecl((R + rot, spec.hidden), "linear")
            p[n["dkv_norm"]] = ParamDecl((R,), "norm")
        if spec.sinks:
            p[n["sink"]] = ParamDecl((H,), "normal", mean=0.0, std=1.0)
        if spec.out_gate:
            p[n["g"]] = ParamDecl((H * dv, spec.hidden), "linear")
        return p

    @staticmethod
    def cache_need(spec: LatentAttentionSpec):
        return PagedNeed(1, spec.kv_rank + spec.rot_dim, values=False)

    @staticmethod
    def workspace_bytes(spec: LatentAttentionSpec, ops, max_requests: int, max_context: int) -> int:
        sizer = getattr(ops, "attention_scratch_bytes", None)
        if sizer is None:
            return 0
        return sizer(max_requests, spec.num_heads, spec.kv_rank + spec.rot_dim, max_context)

    def __init__(self, spec: LatentAttentionSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        H, d, dv, R = spec.num_heads, spec.head_dim, spec.v_head_dim, spec.kv_rank
        rot, qr = spec.rot_dim, spec.q_rank
        q = tensors[n["dq"] if qr else n["q"]]
        self.has_kv = n["dkv"] in tensors
        gate = [tensors[n["g"]].to(q.dtype)] if spec.out_gate else []
        # rows of the fused product: q (or the query latent) | gate | latent, so that the gate
        # sits at the same place whether or not the call makes latent rows
        self.w_q_gate = torch.cat([q] + gate, dim=0).contiguous()
        self.w_all = torch.cat([q] + gate + [tensors[n["dkv"]].to(q.dtype)], dim=0).contiguous() \
            if self.has_kv else None
        self.latent_norm = tensors[n["dkv_norm"]].to(torch.float32).contiguous() \
            if self.has_kv else None
        self.q_norm = tensors[n["dq_norm"]].to(torch.float32).contiguous() if qr else None
        self.w_uq = tensors[n["uq"]].contiguous() if qr else None
        w_uk = tensors[n["uk"]].reshape(H, d, R)
        w_uv_t = tensors[n["uv"]].reshape(H, dv, R).transpose(1, 2)
        if rot:
            # [[W_uk, 0], [0, 1]] carries [q plain | q turned] into [latent | turned] space, and
            # [W_uv^T; 0] drops the turned part of what comes back
            uk = torch.zeros((H, d + rot, R + rot), dtype=w_uk.dtype, device=w_uk.device)
            uk[:, :d, :R] = w_uk
            uk[:, d:, R:] = torch.eye(rot, dtype=w_uk.dtype, device=w_uk.device)
            uv = torch.zeros((H, R + rot, dv), dtype=w_uk.dtype, device=w_uk.device)
            uv[:, :R] = w_uv_t
            w_uk, w_uv_t = uk, uv
            self.freq = position_class("rope_partial")(
                PositionSpec("rope_partial", head_dim=rot, theta=spec.rot_theta, rot_dims=rot),
                q.device).frequencies()[0]
        self.w_uk = w_uk.contiguous()                  # [H, d + rot, R + rot]
        self.w_uv_t = w_uv_t.contiguous()              # [H, R + rot, dv]
        self.w_out = tensors[n["o"]].contiguous()
        self.sinks = tensors[n["sink"]].to(torch.float32).contiguous() if spec.sinks else None
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(d)
        self.sizes = (H, d, dv, R)

    def forward(self, normed, ctx, cache):
        s = self.spec
        H, d, dv, R = self.sizes
        rot, qr = s.rot_dim, s.q_rank
        if not rot and not qr:
            return self._forward_plain(normed, ctx, cache)
        owns = cache.owns
        if owns and not self.has_kv:
            raise ValueError("latent attention: this call owns a cache but the block has no "
                             "latent projection")
        group = ctx.groups[cache.group]
        n = normed.shape[0]
        rows = self.ops.linear(normed, self.w_all if owns else self.w_q_gate,
                               out_dtype=self.dtype)
        q_cols = qr if qr else H * (d + rot)
        gate_off = q_cols if s.out_gate else -1
        kv_off = q_cols + (H * dv if s.out_gate else 0)
        cq = self.ops.new_rows(n, qr, self.dtype, normed.device) if qr else None
        if owns:
            self.ops.latent_prepare(rows, 0, qr, self.q_norm, cq, kv_off, R, rot,
                                    self.latent_norm, s.norm_eps, self.freq if rot else None,
                                    ctx.positions, group.slot_mapping, cache.k)
        elif qr:
            cq = self.ops.new_rows(n, qr, self.dtype, normed.device)
            self.ops.add_rmsnorm(None, rows[:, :qr].contiguous(), self.q_norm, s.norm_eps, cq, None)
        q = self.ops.linear(cq, self.w_uq, out_dtype=self.dtype) if qr else rows
        if rot:
            self.ops.rope_heads(q, H, d + rot, d, rot, self.freq, ctx.positions)
        # queries into the space of the page slots: [n, H, d + rot] x [H, d + rot, R + rot]
        q_lat = self.ops.new_rows(n, H * (R + rot), self.dtype, normed.device)
        self.ops.heads_product(q, 0, H, d + rot, self.w_uk, q_lat)
        mixed = self.ops.new_rows(n, H * (R + rot), self.dtype, normed.device)
        self.ops.paged_attention(q_lat, H, 1, R + rot, cache.k, cache.k, ctx, group, self.scale,
                                 None, mixed, sinks=self.sinks)
        out = self.ops.new_rows(n, H * dv, self.dtype, normed.device)
        self.ops.heads_product(mixed, 0, H, R + rot, self.w_uv_t, out,
                               gate_rows=rows if s.out_gate else None, gate_off=gate_off)
        return self.ops.linear(out, self.w_out, out_dtype=self.dtype)

    def _forward_plain(self, normed, ctx, cache):
        s = self.spec
        H, d, dv, R = self.sizes
        owns = cache.owns
        if owns and not self.has_kv:
            raise ValueError("latent attention: this call owns a cache but the block has no "
                             "latent projection")
        group = ctx.groups[cache.group]
        n = normed.shape[0]
        rows = self.ops.linear(normed, self.w_all if owns else self.w_q_gate,
                               out_dtype=self.dtype)
        gate_off = H * d if s.out_gate else -1
        if owns:
            self.ops.latent_norm_write(rows, H * d + (H * dv if s.out_gate else 0), R,
                                       self.latent_norm, s.norm_eps, group.slot_mapping, cache.k)
        # queries into the latent space: [n, H, d] x [H, d, R] -> [n, H, R]
        q_lat = self.ops.new_rows(n, H * R, self.dtype, normed.device)
        self.ops.heads_product(rows, 0, H, d, self.w_uk, q_lat)
        mixed = self.ops.new_rows(n, H * R, self.dtype, normed.device)
        self.ops.paged_attention(q_lat, H, 1, R, cache.k, cache.k, ctx, group, self.scale, None,
                                 mixed, sinks=self.sinks)
        # and out of it: [n, H, R] x [H, R, dv] -> [n, H, dv]
        out = self.ops.new_rows(n, H * dv, self.dtype, normed.device)
        self.ops.heads_product(mixed, 0, H, R, self.w_uv_t, out,
                               gate_rows=rows if s.out_gate else None, gate_off=gate_off)
        return self.ops.linear(out, self.w_out, out_dtype=self.dtype)


register_mixer("attention_latent", LatentAttention)
