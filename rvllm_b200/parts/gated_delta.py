"""The gated delta rule with one decay per key channel: a linear-attention recurrence whose
state is a matrix per head that forgets channel by channel and is corrected, not only
added to, by every token.

For a token with mixer input h (G query/key heads of size d, H value heads of size dv, value
head j reading query/key head j // (H / G)):

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))    causal, per channel
    q <- q / sqrt(sum q^2 + 1e-6) / sqrt(d),  k <- k / sqrt(sum k^2 + 1e-6)        per head
    beta = sigmoid(W_b h)                                                          per head
    g    = exp(-exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias))            per head and channel
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q            per head
    y = W_o [ o / sqrt(mean o^2 + eps) * norm * sigmoid(W_g2 (W_g1 h)) ]

(the delta rule of "Gated Delta Networks", Yang et al., with the decay made a vector.)  S
starts at zero and, with the last taps-1 inputs of the three convolutions, is the request's
record in a state slot: float32 whatever the compute type.

Products: W_q | W_k | W_v | W_b are one matrix whose result stays float32; W_a1 | W_g1 are
another, and the two low-rank second factors one block-diagonal matrix applied to its result.  The
convolution, activations, unit norms, decay, recurrence, output norm and gate are the two
kernels of `ops.gated_delta`, for any mixture of prompt portions and single tokens.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed, register_mixer
from .spec import GatedDeltaSpec, ParamDecl

_LOCAL = ("q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "A_log", "norm", "a1", "a2", "dt_bias",
          "g1", "g2", "o")


class GatedDelta(Mixer):
    @staticmethod
    def _names(spec):
        return {k: spec.names.get(k, k) for k in _LOCAL}

    @staticmethod
    def _check(spec: GatedDeltaSpec):
        if spec.num_kv_heads < 1 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"gated_delta: {spec.num_heads} value heads do not share "
                             f"{spec.num_kv_heads} query/key heads evenly")
        if spec.taps < 1 or spec.decay_rank < 1 or spec.gate_rank < 1:
            raise ValueError("gated_delta: taps and the two ranks must be at least 1")

    @staticmethod
    def record_size(spec: GatedDeltaSpec) -> int:
        channels = 2 * spec.num_kv_heads * spec.head_dim + spec.num_heads * spec.v_head_dim
        return (spec.taps - 1) * channels + spec.num_heads * spec.head_dim * spec.v_head_dim

    @staticmethod
    def params(spec: GatedDeltaSpec, owns_cache: bool = True):
        GatedDelta._check(spec)
        n = GatedDelta._names(spec)
        w, H, G, d, dv = spec.hidden, spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.v_head_dim
        return {
            n["q"]: ParamDecl((G * d, w), "linear"), n["k"]: ParamDecl((G * d, w), "linear"),
            n["v"]: ParamDecl((H * dv, w), "linear"),
            n["q.conv"]: ParamDecl((G * d, spec.taps), "conv"),
            n["k.conv"]: ParamDecl((G * d, spec.taps), "conv"),
            n["v.conv"]: ParamDecl((H * dv, spec.taps), "conv"),
            n["b"]: ParamDecl((H, w), "linear"),
            n["A_log"]: ParamDecl((H,), "normal", mean=-1.0, std=0.5),
            n["norm"]: ParamDecl((dv,), "norm"),
            n["a1"]: ParamDecl((spec.decay_rank, w), "linear"),
            n["a2"]: ParamDecl((H * d, spec.decay_rank), "normal", mean=0.0, std=0.5),
            n["dt_bias"]: ParamDecl((H * d,), "normal", mean=-1.0, std=1.0),
            n["g1"]: ParamDecl((spec.gate_rank, w), "linear"),
            n["g2"]: ParamDecl((H * dv, spec.gate_rank), "normal", mean=0.0, std=0.5),
            n["o"]: ParamDecl((w, H * dv), "linear"),
        }

    @staticmethod
    def cache_need(spec: GatedDeltaSpec):
        return StateNeed((GatedDelta.record_size(spec),))

    def __init__(self, spec: GatedDeltaSpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        q = tensors[n["q"]]
        cat = lambda keys: torch.cat([tensors[n[k]].to(q.dtype) for k in keys], dim=0).contiguous()
        self.w_in = cat(("q", "k", "v", "b"))
        self.w_low = cat(("a1", "g1"))
        H, G, d, dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.v_head_dim
        self.channels = 2 * G * d + H * dv
        ra, rg = spec.decay_rank, spec.gate_rank
        # [a2 0; 0 g2]: one product gives the decays' and the gates' pre-activations
        second = torch.zeros((H * d + H * dv, ra + rg), dtype=q.dtype, device=q.device)
        second[:H * d, :ra] = tensors[n["a2"]].to(q.dtype)
        second[H * d:, ra:] = tensors[n["g2"]].to(q.dtype)
        self.w_second = second.contiguous()
        f32 = lambda k: tensors[n[k]].to(torch.float32).contiguous()
        self.filt = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm = f32("A_log"), f32("dt_bias"), f32("norm")
        self.w_out = tensors[n["o"]].contiguous()

    def forward(self, normed, ctx, cache):
        if cache is None or not cache.owns:
            raise ValueError("gated_delta: a recurrent state cannot be shared between calls")
        s = self.spec
        n = normed.shape[0]
        proj = self.ops.linear(normed, self.w_in, out_dtype=torch.float32)
        low = self.ops.linear(normed, self.w_low, out_dtype=self.dtype)
        lowrank = self.ops.linear(low, self.w_second, out_dtype=torch.float32)
        y = self.ops.new_rows(n, s.num_heads * s.v_head_dim, self.dtype, normed.device)
        self.ops.gated_delta(proj, lowrank, self.filt, self.a_log, self.dt_bias, self.norm,
                             cache.state, ctx, y, s.num_heads, s.num_kv_heads, s.head_dim,
                             s.v_head_dim, s.taps, s.unit_eps, s.norm_eps)
        return self.ops.linear(y, self.w_out, out_dtype=self.dtype)


register_mixer("gated_delta", GatedDelta)
