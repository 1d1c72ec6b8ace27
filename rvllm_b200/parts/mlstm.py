"""The matrix memory with exponential gates (mLSTM, "xLSTM: Extended Long Short-Term Memory",
Beck et al.): a recurrence whose state per head is a matrix C [d, dv], a vector n [d] and a
running maximum m that keeps the exponential gates in range.

For a token with mixer input h, per head (q scaled by d^(-1/2)):

    li = cap tanh((W_i h + b_i) / cap),   lf = logsigmoid(cap tanh((W_f h + b_f) / cap))
    m' = max(lf + m, li);   C <- e^(lf + m - m') C + e^(li - m') k v^T;   n likewise with k
    o  = C^T q / (max(|n . q|, e^(-m')) + 1e-6)
    y  = W_o [ o / sqrt(mean(o^2) + eps) * w * sigmoid(W_g h) ]

C, n and m start at zero and are the request's record in a state slot: float32 whatever the
compute type.  W_q | W_k | W_v | W_i | W_f | W_g are one matrix whose product stays float32, so
that everything that enters the recurrence is 32-bit; gates, recurrence, read-out, norm and
output gate are `ops.mlstm`, for any mixture of prompt portions and single tokens.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed, register_mixer
from .spec import MLSTMSpec, ParamDecl

_LOCAL = ("q", "k", "v", "i", "f", "i.b", "f.b", "g", "norm", "o")


class MLSTM(Mixer):
    @staticmethod
    def _names(spec):
        return {k: spec.names.get(k, k) for k in _LOCAL}

    @staticmethod
    def _check(spec: MLSTMSpec):
        if spec.num_heads < 1 or spec.head_dim < 1 or spec.v_head_dim < 1:
            raise ValueError("mlstm: head count and sizes must be at least 1")
        if not spec.gate_cap > 0:
            raise ValueError(f"mlstm: the gate cap must be positive, got {spec.gate_cap}")

    @staticmethod
    def record_size(spec: MLSTMSpec) -> int:
        """Per head v_head_dim + 1 columns of head_dim rows (the last column is n), then the
        heads' maxima."""
        return spec.num_heads * (spec.v_head_dim + 1) * spec.head_dim + spec.num_heads

    @staticmethod
    def params(spec: MLSTMSpec, owns_cache: bool = True):
        MLSTM._check(spec)
        n = MLSTM._names(spec)
        w, H, d, dv = spec.hidden, spec.num_heads, spec.head_dim, spec.v_head_dim
        return {
            n["q"]: ParamDecl((H * d, w), "linear"), n["k"]: ParamDecl((H * d, w), "linear"),
            n["v"]: ParamDecl((H * dv, w), "linear"), n["g"]: ParamDecl((H * dv, w), "linear"),
            n["i"]: ParamDecl((H, w), "linear"), n["f"]: ParamDecl((H, w), "linear"),
            n["i.b"]: ParamDecl((H,), "normal", mean=0.0, std=1.0),
            n["f.b"]: ParamDecl((H,), "normal", mean=3.0, std=1.0),
            n["norm"]: ParamDecl((H * dv,), "norm"),
            n["o"]: ParamDecl((w, H * dv), "linear"),
        }

    @staticmethod
    def cache_need(spec: MLSTMSpec):
        return StateNeed((MLSTM.record_size(spec),))

    def __init__(self, spec: MLSTMSpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        q = tensors[n["q"]]
        self.w_in = torch.cat([tensors[n[k]].to(q.dtype) for k in ("q", "k", "v", "i", "f", "g")],
                              dim=0).contiguous()
        f32 = lambda k: tensors[n[k]].to(torch.float32).contiguous()
        self.in_bias, self.forget_bias, self.norm = f32("i.b"), f32("f.b"), f32("norm")
        self.w_out = tensors[n["o"]].contiguous()

    def forward(self, normed, ctx, cache):
        if cache is None or not cache.owns:
            raise ValueError("mlstm: a recurrent state cannot be shared between calls")
        s = self.spec
        rows = self.ops.linear(normed, self.w_in, out_dtype=torch.float32)
        y = self.ops.new_rows(normed.shape[0], s.num_heads * s.v_head_dim, self.dtype,
                              normed.device)
        self.ops.mlstm(rows, self.in_bias, self.forget_bias, self.norm, cache.state, ctx, y,
                       s.num_heads, s.head_dim, s.v_head_dim, s.gate_cap, s.norm_eps)
        return self.ops.linear(y, self.w_out, out_dtype=self.dtype)


register_mixer("mlstm", MLSTM)
