"""Feed-forward layers made of routed experts."""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import FeedForward, LazyNorm
from .mlp import ACTIVATIONS


class RoutedExperts(FeedForward):
    """``h += sum over the chosen experts e of w_e * W_down_e (act(W_gate_e x) * (W_up_e x))``.

    Routing (float32): logits ``z = W_r x``, scores ``sigmoid(z)`` (or a softmax over the experts with
    ``score="softmax"``), the ``top`` experts with the largest ``score + correction`` (``correction``: a per-expert
    tensor that takes part in the choice only, or none), weights = the chosen experts' scores, divided by their sum
    with ``renormalize``, times ``route_scale``.

    Three ways to run the experts, all with launches whose shapes follow from the step's token count alone, so that steps
    replay from CUDA graphs:

    * **every expert on every row** (few rows, float32, odd sizes): gate and up of all experts are the rows of one matrix
      (interleaved pair by pair, the gated activation in the contraction's epilogue), the activations of expert e are
      multiplied by w_e (zero for the experts a token did not choose) and the down matrices, side by side along the inner
      dimension, add the weighted sum into the stream: ``sum_e w_e W_down_e a_e = [W_down_0 .. W_down_E-1] [w_0 a_0; ..;
      w_E-1 a_E-1]``.  A decode step reads every expert's weights once, as it would anyway from about ``E / top`` rows on.
    * **pair by pair** (bfloat16, fewer (token, expert) pairs than experts: a decode step of a few rows): every pair streams
      its own expert's weights through a CUDA-core kernel and the experts nobody chose are not read.
    * **grouped** (bfloat16 on the tensor cores, from ``GROUPED_MIN_ROWS`` rows on or where it needs less arithmetic): the
      (token, expert) pairs are sorted by expert on the device, every expert's rows padded to whole tiles of 128, the rows
      gathered, and two grouped contractions (each row tile takes its expert's weights) make the experts' outputs in
      float, which are then added into the stream token by token with the routing weights, in the order of the choice.
      The padded row count is bounded by ``T * top + 128 * E`` on the host, so nothing is read back from the device."""

    graph_safe = True
    accepts_lazy_norm = False
    GROUPED = True               # False: every expert on every row, always (for comparisons)
    # From this many rows on the grouped contractions are taken whatever the arithmetic says: measured at the 0.5B sizes
    # with 8 experts of which 2 are chosen, a decode step of 64 rows takes 1.10 ms grouped against 1.19 ms with every
    # expert on every row (the few-row contraction streams 4 times the weights at a quarter of the memory bandwidth),
    # one of 8 rows 0.98 against 0.91.
    GROUPED_MIN_ROWS = 48

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 route_scale: float = 1.0, score: str = "sigmoid", renormalize: bool = False, correction: bool = False,
                 activation: str = "silu", names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight",
                 expert_prefix: str = "experts."):
        if not 0 < top <= num_experts:
            raise ValueError(f"top {top} of {num_experts} experts")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"score must be 'sigmoid' or 'softmax', got {score!r}")
        if activation != "silu":
            raise ValueError(f"routed experts implement the SiLU gate, not {activation!r}")
        self.prefix, self.hidden_size, self.intermediate_size = prefix, hidden_size, intermediate_size
        self.num_experts, self.top, self.route_scale = num_experts, top, float(route_scale)
        self.score, self.renormalize, self.has_correction = score, bool(renormalize), bool(correction)
        self.activation = ACTIVATIONS[activation]
        self.names = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj", "router": "router",
                      "correction": "correction"}
        self.names.update(names or {})
        self.weight_suffix, self.expert_prefix = weight_suffix, expert_prefix
        self.w_router = self.correction = self.w_gate_up = self.w_down = self.w_down_rows = None

    def _e(self, e: int, which: str) -> str:
        return f"{self.prefix}.{self.expert_prefix}{e}.{self.names[which]}{self.weight_suffix}"

    def weight_specs(self) -> List[WeightSpec]:
        D, I = self.hidden_size, self.intermediate_size
        specs = [WeightSpec(f"{self.prefix}.{self.names['router']}{self.weight_suffix}", (self.num_experts, D), init=("normal", 0.1))]
        if self.has_correction:
            specs.append(WeightSpec(f"{self.prefix}.{self.names['correction']}", (self.num_experts,), init=("normal", 0.1)))
        for e in range(self.num_experts):
            specs += [WeightSpec(self._e(e, "gate"), (I, D)), WeightSpec(self._e(e, "up"), (I, D)),
                      WeightSpec(self._e(e, "down"), (D, I))]
        return specs

    def bind(self, tensors, dtype, device) -> None:
        E, I, D = self.num_experts, self.intermediate_size, self.hidden_size
        self.w_router = tensors[f"{self.prefix}.{self.names['router']}{self.weight_suffix}"].float().contiguous()
        if self.has_correction:
            self.correction = tensors[f"{self.prefix}.{self.names['correction']}"].float().contiguous()
        gates, ups = [tensors[self._e(e, "gate")] for e in range(E)], [tensors[self._e(e, "up")] for e in range(E)]
        downs = [tensors[self._e(e, "down")] for e in range(E)]
        wide = any(w.dtype == torch.float32 for w in gates + ups + downs)
        wdt = torch.float32 if wide else gates[0].dtype
        # rows: expert by expert, (gate_j, up_j) adjacent, so that the epilogue writes act(gate) * up in expert order
        self.w_gate_up = torch.stack([torch.stack([g.to(wdt), u.to(wdt)], dim=1).reshape(2 * I, D)
                                      for g, u in zip(gates, ups)]).reshape(E * 2 * I, D).contiguous()
        self.w_down = torch.cat([w.to(wdt) for w in downs], dim=1).contiguous()          # [D, E * I]
        if wdt == torch.bfloat16 and dtype == torch.bfloat16 and self.top < E and D % 8 == 0 and I % 8 == 0:
            self.w_down_rows = torch.cat(downs, dim=0).contiguous()                     # [E * D, I]: expert by expert
            self._iota = torch.arange(E, dtype=torch.int32, device=device)              # each pair's own row, pair by pair
        L.reserve_fused_scratch(device, E * 2 * I)

    def route(self, x):
        """(ids [T, top] int32, weights [T, top], dense weights [T, E]) of the rows of x."""
        T = x.shape[0]
        ids = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        dense = torch.empty((T, self.num_experts), dtype=torch.float32, device=x.device)
        ops.moe_route(x, self.w_router, self.correction, self.top, self.route_scale, ids, weights, dense,
                      softmax=self.score == "softmax", renormalize=self.renormalize)
        return ids, weights, dense

    def grouped_pays(self, rows: int) -> bool:
        """Whether the grouped contractions need less arithmetic than every expert on every row: ``rows * top`` pairs plus
        half a tile of padding an expert, against ``rows * experts``.  ``LLB_MOE_GROUPED=always|never`` in the environment
        overrides the rule (for comparisons)."""
        if not (self.GROUPED and self.w_down_rows is not None and ops.has_tcgen05()):
            return False
        forced = os.environ.get("LLB_MOE_GROUPED", "")
        if forced in ("always", "never"):
            return forced == "always"
        return rows >= self.GROUPED_MIN_ROWS or rows * self.top + 64 * self.num_experts < rows * self.num_experts

    def _forward_pairs(self, x, residual) -> None:
        T = x.shape[0]
        ids, weights, _ = self.route(x)
        pairs = T * self.top
        act = torch.empty((pairs, self.intermediate_size), dtype=x.dtype, device=x.device)
        y = torch.empty((pairs, self.hidden_size), dtype=torch.float32, device=x.device)
        ops.moe_pairs(x, ids, self.w_gate_up, self.w_down_rows, act, y)
        ops.moe_combine(y, self._iota[:pairs], weights, residual)

    def _forward_grouped(self, x, residual) -> None:
        T, E, I, D = x.shape[0], self.num_experts, self.intermediate_size, self.hidden_size
        ids, weights, _ = self.route(x)
        tiles = ops.moe_sorted_tiles(T * self.top, E)
        rows = tiles * ops.MOE_TILE_ROWS
        slot = torch.empty(T * self.top, dtype=torch.int32, device=x.device)
        tile_group = torch.empty(tiles, dtype=torch.int32, device=x.device)
        ops.moe_sort(ids, E, slot, tile_group)
        xs = torch.empty((rows, D), dtype=x.dtype, device=x.device)          # padding rows keep what the memory held:
        ops.moe_gather(x, slot, self.top, xs)                               # a row's result depends on that row alone
        act = torch.empty((rows, I), dtype=x.dtype, device=x.device)
        ops.gemm_tcgen05_grouped(xs, self.w_gate_up, act, ops.EPI_SWIGLU, E, tile_group)
        y = torch.empty((rows, D), dtype=torch.float32, device=x.device)
        ops.gemm_tcgen05_grouped(act, self.w_down_rows, y, ops.EPI_STORE_F32, E, tile_group)
        ops.moe_combine(y, slot, weights, residual)

    def forward(self, x, residual, ctx=None) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if x.dtype == torch.bfloat16 and self.w_down_rows is not None and self.GROUPED and \
                x.shape[0] * self.top < self.num_experts and os.environ.get("LLB_MOE_GROUPED", "") != "never":
            self._forward_pairs(x, residual)
            return
        if x.dtype == torch.bfloat16 and self.grouped_pays(x.shape[0]):
            self._forward_grouped(x, residual)
            return
        _, _, dense = self.route(x)
        act = L.linear(x, self.w_gate_up, None, L.SWIGLU)           # [T, E * I]
        ops.moe_scale(act, dense, self.num_experts, self.intermediate_size)
        L.linear(act, self.w_down, None, L.RESIDUAL, residual=residual)


register_part("ffn", "routed_experts", RoutedExperts)
