"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)) (the reference's `swiglu_ffn`,
src/model.rs:320-335).

gate and up are stored as one [2F, hidden] matrix so that they are one matrix
product; the activation kernel reads both halves of its output row.  (The reference
runs two products and `silu_gate_multiply.cu`, src/cuda/model.rs:740-760.)
"""
from __future__ import annotations

import torch

from .base import FeedForward, feed_forward_class, register_feed_forward
from .spec import DenseSpec, GluClampSpec, MoESpec, ParamDecl, SwiGLUSpec


class SwiGLU(FeedForward):
    @staticmethod
    def params(spec: SwiGLUSpec):
        n = spec.names
        return {
            n.get("gate", "gate.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
            n.get("up", "up.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
            n.get("down", "down.weight"): ParamDecl((spec.hidden, spec.ffn_dim), "linear"),
        }

    def __init__(self, spec: SwiGLUSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = spec.names
        gate = tensors[n.get("gate", "gate.weight")]
        up = tensors[n.get("up", "up.weight")]
        self.gate_up = torch.cat([gate, up.to(gate.dtype)], dim=0).contiguous()
        self.down = tensors[n.get("down", "down.weight")].contiguous()

    def forward(self, normed, ctx):
        gate_up = self.ops.linear(normed, self.gate_up, out_dtype=self.dtype)
        act = self.ops.new_rows(normed.shape[0], self.spec.ffn_dim, self.dtype, normed.device)
        self.ops.swiglu(gate_up, act)
        return self.ops.linear(act, self.down, out_dtype=self.dtype)


register_feed_forward("swiglu", SwiGLU)


class Dense(FeedForward):
    """down(act(up(x))).  Activations by name:

    "xielu": with two learned numbers p, q (tensor "act" [2]),
        z > 0:   softplus(p) z^2 + z/2
        z <= 0:  (1/2 + softplus(q)) (e^z - 1 - z) + z/2
    so the slope at 0 is 1/2 from both sides.
    "relu2": max(z, 0)^2, nothing learned.
    """
    ACTIVATIONS = {"xielu": 2, "relu2": 0}      # name -> how many learned numbers it has

    @staticmethod
    def params(spec: DenseSpec):
        n = spec.names
        if spec.activation not in Dense.ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r} "
                             f"(known: {sorted(Dense.ACTIVATIONS)})")
        p = {n.get("up", "up.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
             n.get("down", "down.weight"): ParamDecl((spec.hidden, spec.ffn_dim), "linear")}
        k = Dense.ACTIVATIONS[spec.activation]
        if k:
            p[n.get("act", "act")] = ParamDecl((k,), "normal", mean=0.0, std=0.5)
        return p

    def __init__(self, spec: DenseSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = spec.names
        self.up = tensors[n.get("up", "up.weight")].contiguous()
        self.down = tensors[n.get("down", "down.weight")].contiguous()
        self.act = tensors[n.get("act", "act")].to(torch.float32).contiguous() \
            if self.ACTIVATIONS[spec.activation] else None

    def forward(self, normed, ctx):
        z = self.ops.linear(normed, self.up, out_dtype=self.dtype)
        act = self.ops.new_rows(normed.shape[0], self.spec.ffn_dim, self.dtype, normed.device)
        if self.spec.activation == "relu2":
            self.ops.relu2(z, act)
        else:
            self.ops.xielu(z, self.act, act)
        return self.ops.linear(act, self.down, out_dtype=self.dtype)


register_feed_forward("dense", Dense)


class GluClamp(FeedForward):
    """down(g * sigmoid(alpha g) * (u + 1)) with g = min(gate(x), limit) and
    u = clamp(up(x), -limit, limit); with `bias` the three products have biases (the tensor's
    name plus ".b").  gate and up are one [2F, hidden] product; their biases, the clamps and
    the activation are one kernel."""

    @staticmethod
    def _names(spec):
        n = spec.names
        return {k: n.get(k, k) for k in ("gate", "up", "down")}

    @staticmethod
    def params(spec: GluClampSpec):
        if not spec.limit > 0:
            raise ValueError(f"glu_clamp: the limit must be positive, got {spec.limit}")
        n = GluClamp._names(spec)
        p = {n["gate"]: ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
             n["up"]: ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
             n["down"]: ParamDecl((spec.hidden, spec.ffn_dim), "linear")}
        if spec.bias:
            p[n["gate"] + ".b"] = ParamDecl((spec.ffn_dim,), "bias")
            p[n["up"] + ".b"] = ParamDecl((spec.ffn_dim,), "bias")
            p[n["down"] + ".b"] = ParamDecl((spec.hidden,), "bias")
        return p

    def __init__(self, spec: GluClampSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        gate = tensors[n["gate"]]
        self.gate_up = torch.cat([gate, tensors[n["up"]].to(gate.dtype)], dim=0).contiguous()
        self.down = tensors[n["down"]].contiguous()
        self.bias_in = self.bias_out = None
        if spec.bias:
            self.bias_in = torch.cat([tensors[n["gate"] + ".b"].to(torch.float32),
                                      tensors[n["up"] + ".b"].to(torch.float32)]).contiguous()
            self.bias_out = tensors[n["down"] + ".b"].to(torch.float32).contiguous()

    def forward(self, normed, ctx):
        gate_up = self.ops.linear(normed, self.gate_up, out_dtype=self.dtype)
        act = self.ops.new_rows(normed.shape[0], self.spec.ffn_dim, self.dtype, normed.device)
        self.ops.glu_clamp(gate_up, self.bias_in, act, self.spec.limit, self.spec.alpha)
        return self.ops.linear(act, self.down, bias=self.bias_out, out_dtype=self.dtype)


register_feed_forward("glu_clamp", GluClamp)


class MoE(FeedForward):
    """A mixture of SwiGLU experts (`MoESpec`).  For a token x:

        s       = sigmoid(W_router x)                           float32
        allowed = experts of the `keep` groups whose `group_top` best scores sum highest
        chosen  = the `top` allowed experts with the largest s  (ties: the lower index)
        y       = sum_{e chosen} s_e / (sum_chosen s + weight_eps) * down_e(silu(gate_e x) * up_e x)

    The router matrix is kept in float32 and its product is formed in float32 whatever the
    compute type, in the kernel that also makes the choice (`ops.moe_route`).  The experts' matrices are stacked ([experts, 2 ffn, hidden] with gate and up rows
    alternating, so that a pair lies in neighbouring rows of a product's tile, and
    [experts, hidden, ffn]); `ops.moe_experts` chooses between a kernel that walks each token's
    experts (few tokens) and grouped matrix products over the tokens sorted by expert.  A
    token's result is a sum over its own experts in the order they were chosen, so it does not
    depend on what else is in the batch.

    Options of the spec: scores that are the softmax of the router logits over all experts;
    chosen scores that are not divided by their sum; a factor on every weight; experts of the
    clamped form (`GluClamp`); a shared feed-forward that every token passes, whose output is
    where the experts' weighted sum starts; experts without a gate, down_e(max(up_e x, 0)^2)
    (`activation` "relu2": no "gate" tensors, the stack is [experts, ffn, hidden]); a learned
    number per expert that is added to the scores where experts are compared and nowhere else
    (`choice_bias`, tensor "correction").
    """
    SCORES = ("sigmoid", "softmax")
    ACTIVATIONS = ("swiglu", "glu_clamp", "relu2")

    @staticmethod
    def _names(spec):
        n = spec.names
        out = {"router": n.get("router", "router"), "correction": n.get("correction", "correction")}
        for e in range(spec.experts):
            for k in ("gate", "up", "down"):
                out[(e, k)] = n.get("expert", "e{e}.{k}").format(e=e, k=k)
        return out

    @staticmethod
    def _check(spec: MoESpec):
        if spec.score not in MoE.SCORES:
            raise ValueError(f"unknown router score {spec.score!r} (known: {MoE.SCORES})")
        if spec.activation not in MoE.ACTIVATIONS:
            raise ValueError(f"unknown expert activation {spec.activation!r} "
                             f"(known: {MoE.ACTIVATIONS})")
        if spec.experts < 1 or not 1 <= spec.top <= spec.experts:
            raise ValueError(f"a mixture of {spec.experts} experts cannot use {spec.top} a token")
        if spec.groups < 1 or spec.experts % spec.groups or not 1 <= spec.keep <= spec.groups:
            raise ValueError(f"{spec.experts} experts do not form {spec.groups} equal groups "
                             f"of which {spec.keep} are kept")
        if spec.keep * (spec.experts // spec.groups) < spec.top:
            raise ValueError(f"{spec.keep} groups of {spec.experts // spec.groups} experts "
                             f"cannot give {spec.top} experts")

    @staticmethod
    def params(spec: MoESpec):
        MoE._check(spec)
        n = MoE._names(spec)
        p = {n["router"]: ParamDecl((spec.experts, spec.hidden), "normal", mean=0.0,
                                    std=spec.hidden ** -0.5)}
        if spec.choice_bias:
            p[n["correction"]] = ParamDecl((spec.experts,), "normal", mean=0.0, std=0.1)
        for e in range(spec.experts):
            if spec.activation != "relu2":
                p[n[(e, "gate")]] = ParamDecl((spec.ffn_dim, spec.hidden), "linear")
            p[n[(e, "up")]] = ParamDecl((spec.ffn_dim, spec.hidden), "linear")
            p[n[(e, "down")]] = ParamDecl((spec.hidden, spec.ffn_dim), "linear")
        if spec.shared is not None:
            for k, d in feed_forward_class(spec.shared.kind).params(spec.shared).items():
                p[MoE.SHARED_PREFIX + k] = d
        return p

    SHARED_PREFIX = "shared."

    def __init__(self, spec: MoESpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        self.router = tensors[n["router"]].to(torch.float32).contiguous()
        self.choice_bias = tensors[n["correction"]].to(torch.float32).contiguous() \
            if spec.choice_bias else None
        first = tensors[n[(0, "up")]]
        if spec.activation == "relu2":
            self.gate_up = torch.stack([tensors[n[(e, "up")]].to(first.dtype)
                                        for e in range(spec.experts)]).contiguous()   # [E, F, W]
        else:
            self.gate_up = torch.stack([
                torch.stack([tensors[n[(e, "gate")]].to(first.dtype),
                             tensors[n[(e, "up")]].to(first.dtype)], dim=1).reshape(
                                 2 * spec.ffn_dim, spec.hidden)
                for e in range(spec.experts)]).contiguous()      # [E, 2F, W]: gate f, up f, ...
        self.down = torch.stack([tensors[n[(e, "down")]].to(first.dtype)
                                 for e in range(spec.experts)]).contiguous()   # [E, W, F]
        self.shared = None
        if spec.shared is not None:
            sub = {k[len(self.SHARED_PREFIX):]: v for k, v in tensors.items()
                   if k.startswith(self.SHARED_PREFIX)}
            self.shared = feed_forward_class(spec.shared.kind)(spec.shared, sub, ops, dtype)

    def forward(self, normed, ctx):
        s = self.spec
        n = normed.shape[0]
        ids = torch.empty((n, s.top), dtype=torch.int32, device=normed.device)
        weights = torch.empty((n, s.top), dtype=torch.float32, device=normed.device)
        # the router's product and the choice: one kernel
        extra = {}
        if s.score != "sigmoid" or not s.renormalize or s.route_scale != 1.0:
            extra = dict(score=s.score, renormalize=s.renormalize, route_scale=s.route_scale)
        if self.choice_bias is not None:
            extra["choice_bias"] = self.choice_bias
        self.ops.moe_route(normed, self.router, s.groups, s.keep, s.group_top, s.weight_eps,
                           ids, weights, **extra)
        out = self.ops.new_rows(n, s.hidden, self.dtype, normed.device)
        extra = {}
        if s.activation != "swiglu":
            extra = dict(activation=s.activation, limit=s.limit, alpha=s.alpha)
        if self.shared is not None:
            extra["addend"] = self.shared.forward(normed, ctx).contiguous()
        self.ops.moe_experts(normed, ids, weights, self.gate_up, self.down, out, **extra)
        return out


register_feed_forward("moe", MoE)
