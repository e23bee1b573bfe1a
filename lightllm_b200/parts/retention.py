"""Retention: linear attention with a fixed decay per head, run as a recurrence over a per-request state."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheSpec, StateSpec
from ..config import PartSpec, part_class, register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import CacheView, LazyNorm, Mixer


class RetentionMixer(Mixer):
    """``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head, with no softmax and no denominator.

    q and k are rotated by position (``position``: a rotary part spec, or none), k is then multiplied by ``k_scale``
    (default ``head_dim ** -0.5``); each head's o is divided by its root mean square (``norm_eps`` inside the root, no
    weight), the heads are multiplied element by element by ``act(W_g x)`` and projected by ``W_o``.

    The state ``[heads, head_dim, v_head_dim]`` lives in float32 in the request's state slot: it is zero before the
    request's first token and carried from span to span, so the result does not depend on how the tokens were cut.
    Everything from the rotation to the normalised output is float32 in both precisions."""

    graph_safe = True
    accepts_lazy_norm = False

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int,
                 decay: Sequence[float], position: Optional[PartSpec] = None, k_scale: Optional[float] = None,
                 norm_eps: float = 1e-6, gate_act: str = "silu", names: Optional[Dict[str, str]] = None,
                 weight_suffix: str = ".weight"):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        if gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"gate_act must be 'sigmoid' or 'silu', got {gate_act!r}")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.num_heads, self.head_dim, self.v_head_dim = num_heads, head_dim, v_head_dim
        self.decay_host = [float(d) for d in decay]
        self.k_scale = float(k_scale) if k_scale is not None else head_dim ** -0.5
        self.norm_eps, self.gate_act = float(norm_eps), gate_act
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "g_proj", "o": "o_proj"}
        self.names.update(names or {})
        self.weight_suffix = weight_suffix
        position = position or PartSpec("none")
        self.position = part_class("position", position.kind)(position.prefix, **position.params)
        self.w_fused = self.w_o = self.decay = None

    def _n(self, which: str) -> str:
        return f"{self.prefix}.{self.names[which]}{self.weight_suffix}"

    def children(self):
        return [self.position]

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(state=StateSpec((self.num_heads, self.head_dim, self.v_head_dim), "float32"))

    def weight_specs(self) -> List[WeightSpec]:
        D, H, hd, vd = self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim
        return [WeightSpec(self._n("q"), (H * hd, D)), WeightSpec(self._n("k"), (H * hd, D)),
                WeightSpec(self._n("v"), (H * vd, D)), WeightSpec(self._n("g"), (H * vd, D)),
                WeightSpec(self._n("o"), (D, H * vd))] + self.position.weight_specs()

    def bind(self, tensors, dtype, device) -> None:
        ws = [tensors[self._n(p)] for p in "qkvg"]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_fused = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        self.w_o = tensors[self._n("o")]
        self.decay = torch.tensor(self.decay_host, dtype=torch.float32, device=device)
        self.position.bind(tensors, dtype, device)

    # A span longer than this is cut into pieces that run side by side (csrc/retention.cu); the pieces are made as long as
    # the step's tokens allow while still filling the GPU with warps.
    MIN_PIECE = 32
    WARPS_PER_SM = 16

    @property
    def prepare_key(self):
        return ("retention", self.num_heads, self.head_dim, self.v_head_dim)

    def _pieces(self, ctx):
        """(item_span, item_c, span_first, num_items, chunk) for this step: which pieces the spans are cut into."""
        key = ("retention_pieces", self.num_heads, self.head_dim, self.v_head_dim)
        hit = ctx.memo.get(key)
        if hit is not None:
            return hit
        longest = max(s.length for s in ctx.spans)
        chunk = 1 << 30
        if longest > 2 * self.MIN_PIECE:
            dg = 1 if self.head_dim <= 64 else 2 if self.head_dim <= 128 else 4 if self.head_dim <= 256 else 8
            warps = self.num_heads * -(-self.v_head_dim * dg // 32)             # of one piece
            wanted = max(1, L.num_sms(ctx.device) * self.WARPS_PER_SM // warps)   # pieces in flight
            total = sum(s.length for s in ctx.spans)
            chunk = max(self.MIN_PIECE, -(-(-(-total // wanted)) // 16) * 16)
        counts = [-(-s.length // chunk) for s in ctx.spans]
        if max(counts) == 1:
            hit = (ctx.iota, ctx.zeros, ctx.iota, len(ctx.spans), 1 << 30)
        else:
            item_span = np.repeat(np.arange(len(counts), dtype=np.int32), counts)
            first = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int32)
            item_c = (np.arange(len(item_span), dtype=np.int32) - first[item_span]).astype(np.int32)
            items = ctx.stage(np.stack([item_span, item_c]))
            hit = (items[0], items[1], ctx.stage(first), int(len(item_span)), int(chunk))
        ctx.shape_key.append(("retention", hit[3], hit[4]))
        ctx.memo[key] = hit
        return hit

    def prepare(self, ctx, cache=None) -> None:
        self._pieces(ctx)

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if cache is None or cache.state is None:
            raise ops.KernelError("retention: the run has no state plane")
        if not cache.writes:
            raise ops.KernelError("retention: a run cannot read another run's state (the recurrence advances it)")
        T = x.shape[0]
        H, hd, vd = self.num_heads, self.head_dim, self.v_head_dim
        fused = L.linear(x, self.w_fused, None, L.STORE)           # [T, q | k | v | gate]
        table = self.position.rotary_table() or (None, 0, False)
        inv_freq, rotary_dim, interleaved = table
        o = torch.empty((T, H * vd), dtype=torch.float32, device=x.device)
        ops.retention(fused, 0, H * hd, 2 * H * hd, ctx.span_row, ctx.span_len, ctx.span_pos, ctx.span_slot,
                      ctx.num_spans, H, hd, vd, self.decay, inv_freq, rotary_dim, interleaved, self.k_scale,
                      cache.state, o, pieces=self._pieces(ctx))
        gated = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        g0 = 2 * H * hd + H * vd
        ops.head_gate(o, fused[:, g0: g0 + H * vd], gated, H, vd, False, self.gate_act, unit_rms=True, eps=self.norm_eps)
        L.linear(gated, self.w_o, None, L.RESIDUAL, residual=residual)


register_part("mixer", "retention", RetentionMixer)
