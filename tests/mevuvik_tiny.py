"""Small Mevuvik configurations for the tests, and helpers around them.

MV_A and MV_B differ in every size and constant: widths, head counts and group sizes (1, 2
and 4 query heads per key/value head), key sizes smaller and larger than value sizes, latent
ranks for keys and for queries, turned parts of 2 to 16 dimensions with other bases, scales,
gate caps, branch factors, dense and routed feed-forwards and none, experts of which one, some
or all are chosen, a repeated stretch at the start, in the middle and none, run 1, 2 and 3
times, a residual factor of 1 and others, eps, vocabulary, with and without a cap on the logits.
MV_C has sizes that no vector access divides.  MV_D has sizes the tensor-core kernels take.
"""
import copy
import os

import numpy as np
import torch

from rvllm_b200.config import config_from_dict
from rvllm_b200.weights import write_random_model


def _latent(heads, dim, rot, vdim, rank, q_rank, scale, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
            "q_rank": q_rank, "scale": scale, "rot": {"base": base, "dims": rot}}


def _parallel(left, right, ls, rs):
    heads, kv, dim, vdim, scale = left
    rh, rd, rv, cap = right
    return {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale},
            "right": {"heads": rh, "dim": rd, "vdim": rv, "gate_cap": cap},
            "left_scale": ls, "right_scale": rs}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale}}


MV_A = {
    "architecture": "Mevuvik", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
    "residual_mult": 0.7, "logit_softcap": 8.0, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(4, 16, 8, 24, 32, 40, 0.3, 500.0),
         "mlp": _moe(48, 6, 2, 1.5)},
        {"type": "parallel", "mixer": _parallel((6, 2, 32, 16, 0.25), (2, 24, 16, 8.0), 0.8, 1.3),
         "mlp": _dense(80)},
        {"type": "latent_attention", "mixer": _latent(2, 24, 16, 8, 16, 24, 0.2), "mlp": None},
        {"type": "parallel", "mixer": _parallel((3, 3, 16, 32, 0.4), (3, 8, 40, 15.0), 1.1, 0.6),
         "mlp": _moe(32, 8, 8, 1.0)},
    ],
}

MV_B = {
    "architecture": "Mevuvik", "vocab": 257, "width": 64, "norm": {"eps": 1e-3},
    "residual_mult": 1.0,
    "layers": [
        {"type": "parallel", "mixer": _parallel((4, 1, 16, 48, 0.5), (1, 32, 32, 4.0), 1.0, 1.0),
         "mlp": _moe(96, 5, 1, 2.5)},
        {"type": "latent_attention", "mixer": _latent(3, 32, 2, 16, 48, 16, 0.15, 10.0),
         "mlp": _dense(40)},
        {"type": "parallel", "mixer": _parallel((2, 2, 8, 8, 1.0), (4, 16, 8, 30.0), 0.5, 2.0),
         "mlp": None},
    ],
}

# sizes that no vector access divides: keys of 10 and 6, values of 6 and 5, ranks of 14 and 9, a
# width of 50; the repeated stretch is the whole model, run twice
MV_C = {
    "architecture": "Mevuvik", "vocab": 99, "width": 50, "norm": {"eps": 1e-5},
    "residual_mult": 0.4, "logit_softcap": 25.0, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 10, 6, 6, 14, 9, 0.3, 2e5),
         "mlp": _moe(34, 3, 2, 1.8)},
        {"type": "parallel", "mixer": _parallel((3, 3, 10, 6, 0.6), (2, 6, 5, 7.0), 1.4, 0.75),
         "mlp": _dense(22)},
    ],
}

# sizes the tensor-core kernels take in bfloat16; a stretch that runs once
MV_D = {
    "architecture": "Mevuvik", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "residual_mult": 0.6, "logit_softcap": 20.0, "loop": {"start": 2, "stop": 3, "times": 1},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(8, 32, 16, 48, 48, 64, 0.18, 1e4),
         "mlp": _moe(64, 16, 4, 2.0)},
        {"type": "parallel", "mixer": _parallel((8, 2, 64, 64, 0.2), (4, 64, 64, 11.0), 1.0, 1.0),
         "mlp": _dense(256)},
        {"type": "latent_attention", "mixer": _latent(4, 64, 32, 32, 96, 32, 0.12, 3e5),
         "mlp": _moe(128, 4, 2, 1.0)},
        {"type": "parallel", "mixer": _parallel((4, 4, 32, 32, 0.3), (2, 128, 32, 10.0), 0.7, 1.4),
         "mlp": None},
    ],
}

CONFIGS = {"A": MV_A, "B": MV_B, "C": MV_C, "D": MV_D}
SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write(folder: str, name: str) -> str:
    return write_random_model(os.path.join(folder, "mv_" + name), config_from_dict(config(name)),
                              SEEDS[name])


def read_tensors(folder: str):
    """The file's tensors by name as float64 arrays, through the package's format reader."""
    from rvllm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return {n: f.tensor(n).to(torch.float64).numpy().copy() for n in f.names()}


def plain_logits(folder: str, name: str, tokens, cfg=None, tensors=None):
    import plain_mevuvik
    out = plain_mevuvik.forward(cfg or config(name), tensors or read_tensors(folder), tokens)
    return torch.from_numpy(np.asarray(out))
