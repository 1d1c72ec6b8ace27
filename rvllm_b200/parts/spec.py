"""Descriptions of a model as data.

A model is a list of blocks; a block names an arrangement, a mixer, a feed-forward
and its norms; each of these is a small frozen record of sizes and constants.  The
order in which blocks run is a list of `LayerCall`s, so a block can run twice and a
call can read the cache that an earlier call wrote.  Nothing here knows which
architecture it describes: an architecture is a function from its configuration to a
`ModelSpec` (see `rvllm_b200.models`).

The reference expresses the same variability as one parameterised `Layer` with a
`Mixer` enum and optional tensors (src/model.rs:126-195).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class ParamDecl:
    """One tensor a part needs.

    shape      shape the part works with
    init       distribution of the random-weights mode, by name:
               "linear" and "embedding" N(0, 0.02), "conv" N(0, 0.2),
               "norm" 1 + N(0, 0.05), "bias" N(0, 0.02), "zeros";
               or "normal" with the part's own `mean` and `std`
    mean, std  given, they replace the named distribution's values, so a part outside
               this package can ask for any normal distribution
    alt_shapes shapes a file may store instead (same element count; reshaped on load)
    integer    an integer table: kept as int32 whatever the compute dtype
    """
    shape: Tuple[int, ...]
    init: str
    alt_shapes: Tuple[Tuple[int, ...], ...] = ()
    integer: bool = False
    mean: Optional[float] = None
    std: Optional[float] = None


@dataclass(frozen=True)
class NormSpec:
    kind: str
    size: int
    eps: float


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter the attention mixer. kind "none" applies nothing.
    `rot_dims` (kinds "rope_partial", "rope_pairs"): only the first rot_dims dimensions of a
    head turn.  Kind "rope_pairs" turns neighbouring dimensions (2i, 2i + 1) together, and
    `scaling` = (factor, low, high, original) stretches its long wavelengths: with wavelength
    l = 2 pi / f a frequency stays when l < original / high, becomes f / factor when
    l > original / low, and in between is (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low)."""
    kind: str
    head_dim: int = 0
    theta: float = 0.0
    max_position: int = 0
    rot_dims: int = 0
    scaling: Optional[Tuple[float, float, float, int]] = None


@dataclass(frozen=True)
class MixerSpec:
    kind: str
    hidden: int


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: Optional[NormSpec] = None          # per-head norm of q and k before rotation
    position: PositionSpec = PositionSpec("none")
    window: Optional[int] = None                # keys visible: the last `window` positions
    scale: Optional[float] = None               # None: 1/sqrt(head_dim)
    # local tensor name -> suffix in the file
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    # Options that are off at their defaults.  `qk_norm` of kind "rms_unit" divides every query
    # and key head by its root mean square and has no weight.
    v_head_dim: int = 0                         # size of a value head (0: the key size)
    sink_score: Optional[float] = None          # the softmax's denominator holds one more term
                                                # exp(sink_score) that has no key and no value
    sinks: bool = False                         # the same with a learned score per head
                                                # (tensor "sink" [heads])
    q_temp: Optional[Tuple[float, int]] = None  # (coef, every): the query at position p is
                                                # multiplied by 1 + coef ln(floor((p+1)/every) + 1)
    # `qk_norm` of kind "rms_full" is one RMSNorm over the whole query projection (and one over
    # the whole key projection) before the split into heads, with weights of those sizes.
    bias: bool = False                          # q, k and v projections have biases
    value_mix: Optional[str] = None             # "source": this call's values are kept for the
                                                # step; "mix": v <- (1 - l) v + l v_source with
                                                # the learned scalar "vmix", before the cache
    head_gate: bool = False                     # head j's result is multiplied by
                                                # sigmoid(W_g x)_j, one number per head (tensor
                                                # "g" [heads, hidden]), before the output product


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Attention whose keys and values are both projections of one small latent row per token,
    the only thing that is cached: c = rmsnorm(W_dkv x) [kv_rank]; per head k = W_uk c,
    v = W_uv c.  No position encoding.

    sinks       a learned score per head whose exponential joins the softmax's denominator
                (tensor "sink" [heads])
    out_gate    the concatenated heads are multiplied by sigmoid(W_g x) before the output
                product (tensor "g" [heads * v_head_dim, hidden])
    A call that reads another call's latent rows has no W_dkv.

    q_rank      > 0: queries pass a latent of their own, c_q = rmsnorm(W_dq x) [q_rank] with
                weight "dq_norm", q = W_uq c_q (tensors "dq", "dq_norm", "uq" instead of "q")
    rot_dim     > 0: a head's query has `rot_dim` more dimensions after its `head_dim` plain
                ones, W_dkv has `rot_dim` more rows after the latent's, and these parts are
                turned by the position (rotate-half over the whole part, frequencies
                rot_theta^(-2i/rot_dim)); the turned key part is shared by all heads, cached
                beside the latent row, and the score is the sum of both parts' products
    """
    num_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    kv_rank: int = 0
    scale: Optional[float] = None               # None: 1/sqrt(head_dim)
    norm_eps: float = 1e-6
    sinks: bool = False
    out_gate: bool = False
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    q_rank: int = 0
    rot_dim: int = 0
    rot_theta: float = 10000.0


@dataclass(frozen=True)
class MixedAttentionSpec(AttentionSpec):
    """Attention whose heads are not independent of one another, with a few more options;
    each is off at its default.

    v_head_dim  size of a value head (0: the key size)
    chunk       a query sees only the keys of its own chunk of `chunk` positions, counted
                from position 0 of the sequence (None: no such bound)
    head_mix    scores are mixed over the heads before the softmax: s'_h = sum_g M[h, g] s_g
                (tensor "talk" [heads, heads])
    sinks       the softmax's denominator has one more term exp(sink_h) with no key or value
                (tensor "sink" [heads])
    out_gate    the concatenated heads are multiplied by sigmoid(gate(x)) before the output
                product (tensor "g" [heads * v_head_dim, hidden])
    """
    v_head_dim: int = 0
    chunk: Optional[int] = None
    head_mix: bool = False
    sinks: bool = False
    out_gate: bool = False


@dataclass(frozen=True)
class MinGRUSpec(MixerSpec):
    """A gated recurrence whose gates read only the current token; `width` channels."""
    width: int = 0
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class GatedDeltaSpec(MixerSpec):
    """The gated delta rule with one decay per key channel.  `num_kv_heads` query/key heads of
    size `head_dim`, `num_heads` value heads of size `v_head_dim`; q, k and v pass a causal
    convolution of `taps` taps and silu; the decay and the output gate are products of rank
    `decay_rank` and `gate_rank`; `unit_eps` sits under the root of the unit norms of q and
    k, `norm_eps` under that of the output norm."""
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    taps: int = 0
    decay_rank: int = 0
    gate_rank: int = 0
    norm_eps: float = 1e-6
    unit_eps: float = 1e-6
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class MLSTMSpec(MixerSpec):
    """The matrix memory with exponential gates (mLSTM): `num_heads` heads with keys and
    queries of `head_dim` and values of `v_head_dim`; the pre-activations of the input and the
    forget gate are capped as cap * tanh(. / cap) with `gate_cap`; `norm_eps` sits under the
    root of the per-head norm of the read-out."""
    num_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    gate_cap: float = 15.0
    norm_eps: float = 1e-6
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class ParallelSpec(MixerSpec):
    """Several mixers side by side that read the same input; the result is the sum of their
    outputs, each times its factor.  `prefixes[j]` is where branch j's tensors lie below the
    mixer's own prefix.  Every branch keeps a cache of its own."""
    branches: Tuple[MixerSpec, ...] = ()
    scales: Tuple[float, ...] = ()
    prefixes: Tuple[str, ...] = ()


@dataclass(frozen=True)
class ShortConvSpec(MixerSpec):
    taps: int = 0                               # filter length; the state holds taps-1 rows
    bias: bool = False
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str
    hidden: int


@dataclass(frozen=True)
class SwiGLUSpec(FeedForwardSpec):
    ffn_dim: int = 0
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class DenseSpec(FeedForwardSpec):
    """down(act(up(x))) with one of the registered activations ("xielu", "relu2")."""
    ffn_dim: int = 0
    activation: str = "xielu"
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class GluClampSpec(FeedForwardSpec):
    """down(g * sigmoid(alpha g) * (u + 1)) with g = min(gate(x), limit) and
    u = clamp(up(x), -limit, limit); `bias`: the three products have biases."""
    ffn_dim: int = 0
    limit: float = 0.0
    alpha: float = 1.702
    bias: bool = False
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class MoESpec(FeedForwardSpec):
    """A mixture of `experts` SwiGLU feed-forwards of size `ffn_dim`, of which a token uses
    `top`.  score: how router logits become scores ("sigmoid").  `groups` > 1: the experts
    form that many equal groups of neighbours, a group's score is the sum of its
    `group_top` largest scores, and only experts of the `keep` best groups can be chosen.
    The chosen experts' scores, divided by their sum + `weight_eps`, weigh their outputs.
    Tensors: "router" [experts, hidden]; per expert e "e<e>.gate", "e<e>.up" [ffn_dim, hidden],
    "e<e>.down" [hidden, ffn_dim].
    Options: score "softmax" (over all experts); `renormalize` false leaves the chosen scores
    undivided; `route_scale` multiplies every weight; `activation` "glu_clamp" gives the experts
    the clamped form of `GluClampSpec` with `limit` and `alpha`; `shared` is a feed-forward
    that every token passes as well and whose output is added (tensors under "shared.");
    `activation` "relu2": experts without a gate, down_e(max(up_e x, 0)^2); `choice_bias`: a
    learned number per expert (tensor "correction" [experts]) is added to the scores where
    experts are compared, while the weights are made from the scores without it."""
    ffn_dim: int = 0
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    group_top: int = 2
    score: str = "sigmoid"
    weight_eps: float = 1e-20
    renormalize: bool = True
    route_scale: float = 1.0
    activation: str = "swiglu"
    limit: float = 0.0
    alpha: float = 1.702
    shared: Optional[FeedForwardSpec] = None
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    choice_bias: bool = False


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which parts and how they are arranged.

    `norms` maps a place in the block to (norm spec, tensor name in the file); a norm with
    more than one tensor gives a mapping {local name: name in the file} instead of the one
    name.  Which places exist is the arrangement's business.  `feed_forward` None: the block
    is its mixer alone.  "pre_norm" (src/model.rs:556-585):
        h = x + post_mixer(mixer(mixer_norm(x)));  out = h + post_ffn(ffn(ffn_norm(h)))
    with places "mixer" and "ffn" required and "post_mixer", "post_ffn" optional (the
    reference's `post_attn_norm` and `post_ffn_norm`, src/model.rs:571, 581; LFM2 has
    neither).  The *_prefix fields say where the mixer's and the feed-forward's tensors
    are found in the file.

    `layer_scale` maps the places "mixer" and "ffn" to a tensor [hidden] by which that
    sub-layer's output is multiplied, channel by channel, before it is added, and
    `residual_scale` multiplies every sub-layer's output ("pre_norm" blocks):
        h = x + residual_scale * scale_mixer * mixer(...)

    "hyper_pre_norm" keeps `streams` >= 1 copies of the residual (hyper-connections); `hyper` maps
    the places "mixer" and "ffn" to the prefix of that sub-layer's three tensors (".in" [S],
    ".out" [S], ".mix" [S, S]).
    """
    arrangement: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    norms: Mapping[str, Tuple[NormSpec, object]] = field(hash=False)
    mixer_prefix: str = ""
    ffn_prefix: str = ""
    streams: int = 0
    hyper: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    layer_scale: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    residual_scale: float = 1.0


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block `layer`; `cache_of`, if given, is the
    index (in the order list) of an earlier call whose cache this call reads instead of
    owning one.  `add` = (tensor name, row): that row of a tensor [rows, hidden] is added to the
    residual stream right before the call (what a repeated stretch of layers adds at the start
    of each pass)."""
    layer: int
    cache_of: Optional[int] = None
    add: Optional[Tuple[str, int]] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    max_position: int
    layers: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: object                     # a name, or {local name: name in the file}
    head_name: Optional[str]                    # None: the head is the embedding table
    embedding_scale: Optional[float] = None
    logit_softcap: Optional[float] = None       # c: logits <- c tanh(logits / c)
    streams: int = 0                            # copies of the residual (hyper-connections; 0:
                                                # the one plain residual); the final norm
                                                # reads their sum
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    embedding_norm: Optional[Tuple[NormSpec, object]] = None   # (norm, tensor name): the
                                                # embedding rows pass it before the first layer
