"""Mevuvik: from its configuration to a `ModelSpec`.

The embedding rows pass an RMS norm whose weight is one number; so do the inputs of every
sub-layer and of the head.  A layer is a pre-norm block whose sub-layer outputs are multiplied
by a learned vector and by one factor of the whole model before they are added:

    x <- x + r * ls1 * mixer(N(x) g1);   x <- x + r * ls2 * ff(N(x) g2)

The mixer is a latent attention (queries through a normed latent of their own; each token
leaves a normed latent row, of which keys and values are projections, and a turned key part
that all heads share) or two mixers side by side whose outputs are added with two factors: a
grouped-query attention without positions whose heads each have a sigmoid gate, and a matrix
memory with exponential gates.  The feed-forward is down(relu(up x)^2), dense or as a mixture
of experts whose sigmoid router compares scores plus a learned correction and weighs with the
scores alone.  Layers [start, stop) may run several times with the same weights: every pass
has caches of its own and begins by adding its row of `loop.step` to the stream.  The head is a
matrix of its own; logits pass c tanh(. / c).

Tensor names: `embed`, `embed.norm`; `loop.step`; `l<i>.norm1`, `.norm2`, `.ls1`, `.ls2`;
`l<i>.mix.*` (`.left.*`, `.right.*` in a parallel layer), `l<i>.mlp.*`; `final.norm`; `head`.
"""
from __future__ import annotations

from ..config.mevuvik import LATENT, MevuvikConfig
from ..config.registry import register_architecture
from ..parts.spec import (AttentionSpec, BlockSpec, DenseSpec, LatentAttentionSpec, LayerCall,
                          MLSTMSpec, ModelSpec, MoESpec, NormSpec, ParallelSpec)

# the design has no longest context: positions are bounded only by what float32 counts exactly
MAX_POSITION = 1 << 24

_LATENT_NAMES = {"dkv_norm": "dkv.norm", "dq_norm": "dq.norm"}
_LEFT_NAMES = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o", "head_gate": "g"}
_DENSE_NAMES = {"up": "up", "down": "down"}
_MOE_NAMES = {"expert": "e{e}.{k}"}
LOOP_STEP = "loop.step"


def run_order(n_layers: int, loop):
    """The calls in order: layers before the stretch, the stretch `times` times (each pass with
    caches of its own, its first call adding the pass's row of `loop.step`), the rest."""
    if loop is None:
        return [LayerCall(i) for i in range(n_layers)]
    start, stop, times = loop
    order = [LayerCall(i) for i in range(start)]
    for t in range(times):
        order += [LayerCall(i, add=(LOOP_STEP, t) if i == start else None)
                  for i in range(start, stop)]
    return order + [LayerCall(i) for i in range(stop, n_layers)]


def build_spec(cfg: MevuvikConfig) -> ModelSpec:
    hidden = cfg.width
    norm = NormSpec("rmsnorm_scalar", hidden, cfg.norm_eps)
    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.type == LATENT:
            m = l.latent
            mixer = LatentAttentionSpec(
                "attention_latent", hidden, num_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim,
                kv_rank=m.kv_rank, scale=m.scale, norm_eps=cfg.norm_eps, q_rank=m.q_rank,
                rot_dim=m.rot_dim, rot_theta=m.rot_base, names=_LATENT_NAMES)
        else:
            a, b = l.left, l.right
            left = AttentionSpec("attention", hidden, num_heads=a.heads, num_kv_heads=a.kv_heads,
                                 head_dim=a.dim, v_head_dim=a.vdim, scale=a.scale, head_gate=True,
                                 names=_LEFT_NAMES)
            right = MLSTMSpec("mlstm", hidden, num_heads=b.heads, head_dim=b.dim,
                              v_head_dim=b.vdim, gate_cap=b.gate_cap, norm_eps=cfg.norm_eps)
            mixer = ParallelSpec("parallel", hidden, branches=(left, right),
                                 scales=(l.left_scale, l.right_scale),
                                 prefixes=("left.", "right."))
        norms = {"mixer": (norm, p + "norm1")}
        scales = {"mixer": p + "ls1"}
        ffn = None
        if l.mlp is not None:
            norms["ffn"] = (norm, p + "norm2")
            scales["ffn"] = p + "ls2"
            if l.mlp.kind == "dense":
                ffn = DenseSpec("dense", hidden, ffn_dim=l.mlp.ff, activation="relu2",
                                names=_DENSE_NAMES)
            else:
                ffn = MoESpec("moe", hidden, ffn_dim=l.mlp.ff, experts=l.mlp.experts,
                              top=l.mlp.top, score="sigmoid", weight_eps=1e-20,
                              route_scale=l.mlp.route_scale, activation="relu2",
                              choice_bias=True, names=_MOE_NAMES)
        layers.append(BlockSpec("pre_norm", mixer, ffn, norms, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "mlp.", layer_scale=scales,
                                residual_scale=cfg.residual_mult))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=hidden,
        max_position=MAX_POSITION, layers=tuple(layers),
        order=tuple(run_order(len(layers), cfg.loop)), final_norm=norm, embedding_name="embed",
        final_norm_name="final.norm", head_name="head", logit_softcap=cfg.logit_softcap,
        embedding_norm=(norm, "embed.norm"))


register_architecture("Mevuvik", MevuvikConfig, build_spec, replace=True)
