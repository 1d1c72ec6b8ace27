"""RMSNorm: x / sqrt(mean(x^2) + eps) * weight, statistics in float32
(the reference's `rms_norm`, src/model.rs:200-214; src/cuda/kernels/rmsnorm.cu:32-38).

The part owns the fusion with the residual addition: the stream's pending sub-layer
output is added to the float32 residual in the same pass that normalises it
(the reference runs `add.cu`, `rmsnorm.cu` and `f32_to_f16.cu` one after the other,
src/cuda/model.rs:685-790).
"""
from __future__ import annotations

import torch

from .base import Norm, register_norm
from .spec import NormSpec, ParamDecl


class RMSNorm(Norm):
    @staticmethod
    def params(spec: NormSpec):
        return {"weight": ParamDecl((spec.size,), "norm")}

    def __init__(self, spec: NormSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        # Norm weights are tiny; float32 keeps a 32-bit file exact and widens a
        # bfloat16 file without loss.
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def add_norm(self, resid, delta, ctx, rows=None, delta_norm=None, delta_scale=None, add=None):
        """`delta_scale` float32 [size] multiplies the pending rows before they are added, `add`
        float32 [size] is added to every row of the stream; both in the same kernel."""
        delta = self._normed_delta(delta, delta_norm, ctx)
        n = resid.shape[0] if rows is None else rows.shape[0]
        out = self.ops.new_rows(n, self.spec.size, self.dtype, resid.device)
        if delta_scale is None and add is None:
            self.ops.add_rmsnorm(resid, delta, self.weight, self.spec.eps, out, rows)
        else:
            self.ops.add_rmsnorm(resid, delta, self.weight, self.spec.eps, out, rows,
                                 delta_scale=delta_scale if delta is not None else None, add=add)
        return out

    def norm_f32(self, x):
        """The normalised float32 rows of float32 `x`: rows that go on as the residual stream."""
        out = torch.empty_like(x)
        self.ops.add_rmsnorm(None, x, self.weight, self.spec.eps, out, None)
        return out

    def norm(self, x, ctx):
        out = self.ops.new_rows(x.shape[0], self.spec.size, self.dtype, x.device)
        self.ops.add_rmsnorm(None, x, self.weight, self.spec.eps, out, None)
        return out


class ScalarRMSNorm(RMSNorm):
    """RMSNorm whose weight is a single number for all coordinates (a tensor without
    dimensions in the file): x / sqrt(mean(x^2) + eps) * g."""

    @staticmethod
    def params(spec: NormSpec):
        return {"weight": ParamDecl((), "norm")}

    def __init__(self, spec: NormSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        g = tensors["weight"].to(torch.float32).reshape(1)
        self.weight = g.expand(spec.size).contiguous()


class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * weight + bias, var the mean squared deviation;
    statistics, the normalised values and the sum with the residual stream in float32.

    `norm(x)` (a norm after a sub-layer) gives float32 rows, because they are on their way
    into the float32 stream; when the next norm of the stream is a LayerNorm too, the two
    and the addition between them are one kernel: x = stream + LN_a(delta); out = LN_b(x).
    """

    @staticmethod
    def params(spec: NormSpec):
        return {"weight": ParamDecl((spec.size,), "norm"),
                "bias": ParamDecl((spec.size,), "bias")}

    def __init__(self, spec: NormSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.bias = tensors["bias"].to(torch.float32).contiguous()

    def add_norm(self, resid, delta, ctx, rows=None, delta_norm=None):
        n = resid.shape[0] if rows is None else rows.shape[0]
        out = self.ops.new_rows(n, self.spec.size, self.dtype, resid.device)
        if delta is not None and isinstance(delta_norm, LayerNorm):
            self.ops.add_layernorm(resid, delta, self.weight, self.bias, self.spec.eps, out, rows,
                                   delta_weight=delta_norm.weight, delta_bias=delta_norm.bias,
                                   delta_eps=delta_norm.spec.eps)
            return out
        delta = self._normed_delta(delta, delta_norm, ctx)
        self.ops.add_layernorm(resid, delta, self.weight, self.bias, self.spec.eps, out, rows)
        return out

    def norm(self, x, ctx):
        out = torch.empty((x.shape[0], self.spec.size), dtype=torch.float32, device=x.device)
        self.ops.add_layernorm(None, x, self.weight, self.bias, self.spec.eps, out, None)
        return out


register_norm("rmsnorm", RMSNorm)
register_norm("rmsnorm_scalar", ScalarRMSNorm)
register_norm("layernorm", LayerNorm)
