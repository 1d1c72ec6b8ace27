"""Small Vifanex configurations for the tests, and helpers around them.

VF_A .. VF_E differ in every size and constant: widths, numbers of residual streams (none,
one, two, three, five), head counts and group sizes of both mixers (1, 2, 3 and 4 heads per
key head), key sizes smaller and larger than value sizes, windows below a page, across pages,
of one token and none, rotations of part of a head, of the whole head and none, with and
without stretched wavelengths, value mixing in some layers, filters of 1 to 5 taps, ranks of
the decay and gate products, dense and mixed feed-forwards and none, experts in one group,
several and as many groups as experts, with and without a shared expert and a factor on the
weights, eps, vocabulary, with and without the embedding factor and the cap on the logits.
VF_C has sizes that no vector access divides.  VF_D and VF_E have sizes the tensor-core
kernels take in bfloat16.
"""
import copy
import os

import numpy as np
import torch

from rvllm_b200.config import config_from_dict
from rvllm_b200.weights import write_random_model


def _attn(heads, kv, dim, vdim, scale, window=None, rot=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        dims, base, scaling = rot
        m["rot"] = {"dims": dims, "base": base}
        if scaling is not None:
            factor, low, high, original = scaling
            m["rot"]["scaling"] = {"factor": factor, "low": low, "high": high,
                                   "original": original}
    if v_mix:
        m["v_mix"] = True
    return m


def _delta(heads, kv, dim, vdim, taps, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps,
            "decay_rank": decay_rank, "gate_rank": gate_rank}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, limit, experts, top, groups=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


VF_A = {
    "architecture": "Vifanex", "vocab": 300, "width": 96, "streams": 3, "norm": {"eps": 1e-5},
    "embedding": {"scale": 4.0}, "logit_softcap": 8.0,
    "layers": [
        {"type": "channel_delta", "mixer": _delta(4, 2, 16, 24, 3, 8, 12),
         "mlp": _moe(48, 1.5, 6, 2, (3, 2), 2.0, (32, 0.7))},
        {"type": "attention",
         "mixer": _attn(6, 2, 32, 16, 0.3, 20, (16, 500.0, (4.0, 1.0, 3.0, 64)), True),
         "mlp": _dense(80, 1.0)},
        {"type": "attention", "mixer": _attn(4, 2, 16, 16, 0.4, 7, (16, 100.0, None), True),
         "mlp": None},
        {"type": "channel_delta", "mixer": _delta(2, 2, 32, 8, 4, 5, 3), "mlp": _moe(32, 3.0, 4, 1)},
        {"type": "attention", "mixer": _attn(2, 2, 48, 16, 0.2, 33, (8, 50.0, None), True),
         "mlp": _moe(24, 0.8, 8, 3, (4, 2), 0.5)},
    ],
}

# no streams (one plain residual), no embedding factor, no cap; a window of one token and none;
# a filter of one tap (no convolution state) and of two; as many groups as experts
VF_B = {
    "architecture": "Vifanex", "vocab": 257, "width": 64, "norm": {"eps": 1e-3},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 1, 16, 48, 1.5, None, (16, 10000.0, (8.0, 1.0, 4.0, 32))),
         "mlp": _moe(96, 1.0, 9, 3, (3, 1), None, (16, 2.0))},
        {"type": "channel_delta", "mixer": _delta(3, 1, 8, 40, 1, 4, 4), "mlp": _dense(40, 0.5)},
        {"type": "attention", "mixer": _attn(2, 2, 8, 8, 0.7, 1), "mlp": None},
        {"type": "channel_delta", "mixer": _delta(4, 4, 24, 16, 2, 16, 2),
         "mlp": _moe(32, 2.5, 5, 2, (5, 3), 1.25)},
        {"type": "attention", "mixer": _attn(3, 3, 32, 24, 0.25, 50, (32, 1000.0, None)),
         "mlp": _dense(72, 4.0)},
    ],
}

# sizes that no vector access divides; one stream with weights of its own; five taps
VF_C = {
    "architecture": "Vifanex", "vocab": 99, "width": 50, "streams": 1, "norm": {"eps": 1e-5},
    "embedding": {"scale": 0.5}, "logit_softcap": 30.0,
    "layers": [
        {"type": "attention", "mixer": _attn(3, 3, 10, 6, 0.6, 5, (6, 30.0, None), True),
         "mlp": _moe(22, 1.0, 3, 3, None, 3.0, (10, 1.0))},
        {"type": "channel_delta", "mixer": _delta(3, 1, 10, 6, 5, 7, 9), "mlp": _dense(34, 2.0)},
        {"type": "attention", "mixer": _attn(6, 3, 14, 6, 0.3, 64, (14, 70.0, (2.0, 0.5, 2.0, 16)), True),
         "mlp": None},
    ],
}

# sizes the tensor-core kernels take in bfloat16; two streams
VF_D = {
    "architecture": "Vifanex", "vocab": 200, "width": 128, "streams": 2, "norm": {"eps": 1e-6},
    "embedding": {"scale": 8.0}, "logit_softcap": 20.0,
    "layers": [
        {"type": "attention",
         "mixer": _attn(8, 2, 64, 64, 0.125, 100, (32, 10000.0, (8.0, 1.0, 4.0, 128)), True),
         "mlp": _moe(128, 2.0, 8, 2, (4, 2), 1.5, (64, 2.0))},
        {"type": "channel_delta", "mixer": _delta(4, 2, 64, 64, 4, 16, 16), "mlp": _dense(256, 1.0)},
        {"type": "attention", "mixer": _attn(12, 2, 32, 32, 0.2, 17, (32, 5000.0, None)),
         "mlp": _moe(64, 1.0, 16, 5, (8, 3), 1.0)},
        {"type": "attention", "mixer": _attn(4, 2, 64, 64, 0.125, 64, (64, 10000.0, None), True),
         "mlp": None},
        {"type": "channel_delta", "mixer": _delta(8, 2, 32, 32, 4, 8, 32),
         "mlp": _moe(128, 2.0, 4, 2, None, None, (128, 1.0))},
    ],
}

# larger heads: key and value heads of 128, a state of 128 x 128, many experts of a size that
# no tile divides, five streams
VF_E = {
    "architecture": "Vifanex", "vocab": 500, "width": 192, "streams": 5, "norm": {"eps": 1e-6},
    "embedding": {"scale": 12.0}, "logit_softcap": 10.0,
    "layers": [
        {"type": "channel_delta", "mixer": _delta(2, 1, 128, 128, 4, 24, 24),
         "mlp": _moe(72, 2.0, 32, 6, (8, 4), 2.0, (200, 2.0))},
        {"type": "attention", "mixer": _attn(4, 4, 128, 128, 0.09, 130, (64, 10000.0, None)),
         "mlp": _dense(200, 1.0)},
        {"type": "channel_delta", "mixer": _delta(3, 3, 64, 96, 3, 6, 40), "mlp": None},
        {"type": "attention", "mixer": _attn(16, 2, 32, 64, 0.2, 31, (16, 300.0, (4.0, 1.0, 2.0, 48)), True),
         "mlp": _moe(72, 1.0, 64, 8, (4, 1), 0.75)},
        {"type": "attention", "mixer": _attn(6, 2, 80, 64, 0.1, 90, (80, 10000.0, None), True),
         "mlp": _dense(64, 3.0)},
    ],
}

CONFIGS = {"A": VF_A, "B": VF_B, "C": VF_C, "D": VF_D, "E": VF_E}
SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34, "E": 35}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write(folder: str, name: str) -> str:
    return write_random_model(os.path.join(folder, "vf_" + name), config_from_dict(config(name)),
                              SEEDS[name])


def read_tensors(folder: str):
    """The file's tensors by name as float64 arrays, through the package's format reader."""
    from rvllm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return {n: f.tensor(n).to(torch.float64).numpy().copy() for n in f.names()}


def plain_logits(folder: str, name: str, tokens, cfg=None, tensors=None):
    import plain_vifanex
    out = plain_vifanex.forward(cfg or config(name), tensors or read_tensors(folder), tokens)
    return torch.from_numpy(np.asarray(out))
