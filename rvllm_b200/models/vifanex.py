"""Vifanex: from its configuration to a `ModelSpec`.

The residual is `streams` copies of the embedding output (hyper-connections, or one plain
residual when the configuration names no streams); every layer is a pre-norm block with an
RMSNorm before each sub-layer.  The mixer is a grouped-query attention (biases on q, k and v;
one RMSNorm over the whole query projection and one over the whole key projection; a rotation
of neighbouring dimensions on the first dimensions of each head, with stretched long
wavelengths; a sliding window; values mixed with those of the first such layer) or a gated
delta rule with a decay per key channel.  The feed-forward is the clamped gated form, dense
with biases, or a mixture with a softmax router, groups of experts, scores that are scaled but
not renormalised, and a shared expert.  The head is a matrix of its own after the model's
norm; logits pass c tanh(. / c).

Tensor names: `embed`; `l<i>.norm1`, `.norm2`; `l<i>.hc1.in/.out/.mix`, `l<i>.hc2.*`;
`l<i>.mix.*`, `l<i>.mlp.*`; `final.norm`; `head`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vifanex import ATTENTION, VifanexConfig
from ..errors import ConfigError
from ..parts.spec import (AttentionSpec, BlockSpec, GatedDeltaSpec, GluClampSpec, LayerCall,
                          ModelSpec, MoESpec, NormSpec, PositionSpec)

# the design has no longest context: positions are bounded only by what float32 counts exactly
MAX_POSITION = 1 << 24
GLU_ALPHA = 1.702            # g * sigmoid(1.702 g): the sigmoid form of gelu
UNIT_EPS = 1e-6              # under the root of the delta rule's unit norms

_ATTENTION_NAMES = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o",
                    "q_norm": "q.norm", "k_norm": "k.norm", "q_bias": "q.b", "k_bias": "k.b",
                    "v_bias": "v.b", "vmix": "vmix"}


def _glu(hidden, ff, limit, bias):
    return GluClampSpec("glu_clamp", hidden, ffn_dim=ff, limit=limit, alpha=GLU_ALPHA, bias=bias)


def build_spec(cfg: VifanexConfig) -> ModelSpec:
    hidden = cfg.width
    norm = NormSpec("rmsnorm", hidden, cfg.norm_eps)
    streams = cfg.streams or 0
    layers, order = [], []
    mixing_seen = False
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.type == ATTENTION:
            position = PositionSpec("rope_pairs", l.dim, l.rot_base, MAX_POSITION, l.rot_dims,
                                    l.rot_scaling) if l.rot_dims else PositionSpec("none")
            mixer = AttentionSpec(
                "attention", hidden, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim,
                qk_norm=NormSpec("rms_full", l.dim, cfg.norm_eps), position=position,
                window=l.window, scale=l.scale, names=_ATTENTION_NAMES, v_head_dim=l.vdim,
                bias=True, value_mix=None if not l.v_mix else ("mix" if mixing_seen else "source"))
            mixing_seen = mixing_seen or l.v_mix
        else:
            if l.decay_rank is None or l.gate_rank is None:
                raise ConfigError(f"layers[{i}]: the ranks of the decay and gate products are "
                                  f"not known (they are the rows of l{i}.mix.a1 and l{i}.mix.g1 "
                                  f"in the tensor file, or 'decay_rank' and 'gate_rank')")
            mixer = GatedDeltaSpec(
                "gated_delta", hidden, num_heads=l.heads, num_kv_heads=l.kv_heads,
                head_dim=l.dim, v_head_dim=l.vdim, taps=l.taps, decay_rank=l.decay_rank,
                gate_rank=l.gate_rank, norm_eps=cfg.norm_eps, unit_eps=UNIT_EPS)
        ffn = None
        norms = {"mixer": (norm, p + "norm1")}
        hyper = {"mixer": p + "hc1"}
        if l.mlp is not None:
            m = l.mlp
            if m.kind == "dense":
                ffn = _glu(hidden, m.ff, m.limit, True)
            else:
                ffn = MoESpec(
                    "moe", hidden, ffn_dim=m.ff, experts=m.experts, top=m.top, groups=m.groups,
                    keep=m.keep, group_top=1, score="softmax", renormalize=False,
                    route_scale=1.0 if m.route_scale is None else m.route_scale,
                    activation="glu_clamp", limit=m.limit, alpha=GLU_ALPHA,
                    shared=None if m.shared is None else
                    _glu(hidden, m.shared.ff, m.shared.limit, False))
            norms["ffn"] = (norm, p + "norm2")
            hyper["ffn"] = p + "hc2"
        layers.append(BlockSpec("hyper_pre_norm" if streams else "pre_norm", mixer, ffn, norms,
                                mixer_prefix=p + "mix.", ffn_prefix=p + "mlp.", streams=streams,
                                hyper=hyper if streams else {}))
        order.append(LayerCall(i))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=hidden,
        max_position=MAX_POSITION, layers=tuple(layers), order=tuple(order),
        final_norm=norm, embedding_name="embed", final_norm_name="final.norm",
        head_name="head", embedding_scale=cfg.embedding_scale,
        logit_softcap=cfg.logit_softcap, streams=streams)


register_architecture("Vifanex", VifanexConfig, build_spec, replace=True)
