"""Position encodings."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..config import register_part
from .base import PositionEncoding


class RotaryEmbedding(PositionEncoding):
    """Rotary positions: pair ``i`` of a head turns by ``pos * theta^(-2i / rotary_dim)``.

    The reference computes ``pos / powf(theta, 2i/hd)`` in float on the host for every layer
    (src/engine/engine_server.cpp:1570-1578) and rotates NeoX pairs ``(i, i + hd/2)``
    (src/ops/rope.cu:54-59).  Here the inverse frequencies are computed once in float64 and
    rounded to float32; the angle is the float32 product ``pos * inv_freq`` inside the kernel.
    ``style`` is ``"neox"`` (half-split pairs) or ``"interleaved"`` (adjacent pairs);
    ``rotary_dim`` below ``head_dim`` leaves the upper dimensions unrotated.

    ``scaling = {"factor", "original", "fast", "slow"}`` stretches the slow pairs for contexts beyond the ``original``
    length (YaRN): with ``turns(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)`` the pair index at which a
    pair makes ``t`` turns over the original length, ``lo = max(floor(turns(fast)), 0)``, ``hi = min(ceil(turns(slow)),
    rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair ``i`` turns by
    ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and cos and sin are multiplied by ``magnitude = 0.1 ln(factor) + 1``.
    The kernels that take a table from :meth:`rotary_table` alone rotate with magnitude 1; a mixer whose kernel knows the
    factor reads ``magnitude``."""

    graph_safe = True

    def __init__(self, prefix: str, head_dim: int, theta: float, rotary_dim: Optional[int] = None,
                 style: str = "neox", scaling: Optional[dict] = None):
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and in (0, head_dim={head_dim}]")
        if style not in ("neox", "interleaved"):
            raise ValueError(f"rotary style must be 'neox' or 'interleaved', got {style!r}")
        self.head_dim, self.rotary_dim, self.theta, self.style = head_dim, rotary_dim, float(theta), style
        exponents = np.arange(0, rotary_dim, 2, dtype=np.float64) / rotary_dim
        freq = 1.0 / np.power(np.float64(theta), exponents)
        self.magnitude = 1.0
        self.scaling = dict(scaling) if scaling else None
        if scaling:
            import math
            factor = float(scaling["factor"])
            turns = lambda t: rotary_dim * math.log(float(scaling["original"]) / (2 * math.pi * float(t))) \
                / (2 * math.log(float(theta)))
            lo = max(math.floor(turns(scaling["fast"])), 0)
            hi = min(math.ceil(turns(scaling["slow"])), rotary_dim - 1)
            ramp = np.clip((np.arange(rotary_dim // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            freq = freq / factor * ramp + freq * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.inv_freq_host = freq.astype(np.float32)
        self.inv_freq = None

    def bind(self, tensors, dtype, device) -> None:
        self.inv_freq = torch.from_numpy(self.inv_freq_host).to(device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim, self.style == "interleaved"

    def step_table(self, ctx, transposed: bool = False):
        """(cos, sin) of every token of the step, computed once per step and shared by all layers
        whose encoding has the same frequencies: ``[T, pairs, 2]``, or ``[pairs, T, 2]`` with ``transposed``."""
        from ..csrc import ops
        if self.magnitude != 1.0:
            raise NotImplementedError("the shared cos/sin table has magnitude 1; scaled rotary positions go through "
                                      "a kernel that takes the magnitude")
        key = ("rope_table", self.rotary_dim, self.theta, transposed, tuple(sorted((self.scaling or {}).items())))
        hit = ctx.memo.get(key)
        if hit is None:
            hit = ctx.memo[key] = ops.rope_table(ctx.positions, self.inv_freq, transposed)
        return hit


class NoPositionEncoding(PositionEncoding):
    """Leaves q and k as they are."""

    graph_safe = True

    def __init__(self, prefix: str = ""):
        pass


register_part("position", "rotary", RotaryEmbedding)
register_part("position", "none", NoPositionEncoding)
