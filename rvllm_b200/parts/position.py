"""Position encodings for the attention mixer.

"rope": rotate-half rotation by angle pos * theta^(-2j/head_dim) for the pair
(j, j + head_dim/2) (the reference's `rope_cos_sin` and `rope_apply`,
src/model.rs:224-263).  Frequencies, angles, cosines and sines are float32, as in the
reference; the table is built once per (theta, head_dim, max_position) and indexed by
absolute position in the kernel, where the reference rebuilds it for every forward
call (src/model.rs:487-492).
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position
from .spec import PositionSpec

_TABLES = {}


class Rope(PositionEncoding):
    def __init__(self, spec: PositionSpec, device):
        if spec.head_dim % 2:
            raise ValueError(f"rope needs an even head size, got {spec.head_dim}")
        self.spec = spec
        key = (spec.theta, spec.head_dim, spec.max_position, str(device))
        if key not in _TABLES:
            half = spec.head_dim // 2
            j = torch.arange(half, dtype=torch.float32)
            freq = torch.pow(torch.tensor(spec.theta, dtype=torch.float32),
                             -2.0 * j / spec.head_dim)
            pos = torch.arange(spec.max_position, dtype=torch.float32).unsqueeze(1)
            angles = pos * freq.unsqueeze(0)
            _TABLES[key] = (angles.cos().to(device).contiguous(),
                            angles.sin().to(device).contiguous())
        self.cos, self.sin = _TABLES[key]

    def rotation_table(self):
        return self.cos, self.sin


class PartialRope(PositionEncoding):
    """The rotate-half rotation on the first `rot_dims` dimensions of a head only: dimension
    i turns with i + rot_dims/2 by the angle pos * theta^(-2i/rot_dims); the others pass.
    There is no table over positions: the kernels form the angle (float32) from the position
    and `frequencies()`, so no longest context has to be known."""

    def __init__(self, spec: PositionSpec, device):
        dims = spec.rot_dims or spec.head_dim
        if dims % 2 or dims > spec.head_dim or dims < 0:
            raise ValueError(f"rope_partial needs an even number of turning dimensions within "
                             f"the head's {spec.head_dim}, got {dims}")
        self.spec = spec
        self.rot_dims = dims
        i = torch.arange(dims // 2, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(spec.theta, dtype=torch.float64),
                                  -2.0 * i / max(dims, 1)).to(torch.float32).to(device).contiguous()

    def rotation_table(self):
        return None

    def frequencies(self):
        """(float32 [rot_dims/2] angle per position of each pair, rot_dims)"""
        return self.inv_freq, self.rot_dims


class PairRope(PositionEncoding):
    """A rotation of neighbouring dimensions: in each head the pair (2i, 2i + 1), i < rot_dims/2,
    at position p turns by p * f_i with f_i = theta^(-2i/rot_dims); the dimensions from rot_dims
    on pass.  With `scaling` = (factor, low, high, original) long wavelengths are stretched
    (see `PositionSpec`).  As with `PartialRope` the kernels form the angle in float32 from
    the position and `frequencies()`, so no longest context has to be known."""

    def __init__(self, spec: PositionSpec, device):
        dims = spec.rot_dims or spec.head_dim
        if dims % 2 or dims > spec.head_dim or dims < 0 or spec.head_dim % 2:
            raise ValueError(f"rope_pairs needs an even number of turning dimensions within an "
                             f"even head size, got {dims} of {spec.head_dim}")
        self.spec = spec
        self.rot_dims = dims
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(spec.theta, dtype=torch.float64), -2.0 * i / max(dims, 1))
        if spec.scaling is not None:
            factor, low, high, original = spec.scaling
            if not (factor > 0 and high > low and original > 0):
                raise ValueError("rope_pairs: the scaling needs factor > 0, high > low and a "
                                 "positive original length")
            wavelength = 2.0 * torch.pi / f
            s = (original / wavelength - low) / (high - low)
            between = (1.0 - s) * f / factor + s * f
            f = torch.where(wavelength < original / high, f,
                            torch.where(wavelength > original / low, f / factor, between))
        self.inv_freq = f.to(torch.float32).to(device).contiguous()

    def rotation_table(self):
        return None

    def frequencies(self):
        """(float32 [rot_dims/2] angle per position of each pair, rot_dims)"""
        return self.inv_freq, self.rot_dims


class NoPosition(PositionEncoding):
    def __init__(self, spec: PositionSpec, device):
        self.spec = spec

    def rotation_table(self):
        return None


register_position("rope", Rope)
register_position("rope_partial", PartialRope)
register_position("rope_pairs", PairRope)
register_position("none", NoPosition)
