"""The gated delta rule with a decay per key channel, run as a recurrence over a per-request state."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache import CacheSpec, StateSpec
from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import CacheView, LazyNorm, Mixer
from .conv_attention import span_arrays


class ChannelDeltaMixer(Mixer):
    """Per head, with a state ``S [head_dim, v_head_dim]`` that is zero before a request's first token::

        S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t

    * q, k (``num_qk_heads`` heads, shared by ``num_heads / num_qk_heads`` value heads each) and v pass a causal
      convolution of ``conv_taps`` taps over time and SiLU; q and k are then made unit vectors (``1e-6`` inside the
      root), q times ``head_dim ** -0.5``;
    * ``beta = sigmoid(W_b x)``, one per head;
    * ``g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 x) + dt_bias))``, one per head and key channel;
    * each head's o is divided by its root mean square (``norm_eps``), multiplied by a weight shared by the heads and
      by ``sigmoid(W_g2 (W_g1 x))``, then projected by ``W_o``.

    One contraction makes everything that reads x (q | k | v | beta | the two low-rank inputs); the request's state
    slot holds S and the inputs of the last ``conv_taps - 1`` positions, both float32.  Everything from the
    convolution's output to the normed head is float32 in both precisions."""

    graph_safe = True
    accepts_lazy_norm = False
    UNIT_EPS = 1e-6

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, v_head_dim: int,
                 conv_taps: int, decay_rank: int, gate_rank: int, norm_eps: float = 1e-6,
                 names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight", conv_ending: str = "conv"):
        if num_heads % num_qk_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_qk_heads} q/k heads")
        if conv_taps < 0:
            raise ValueError(f"a convolution has a number of taps (or 0 for none), got {conv_taps}")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.num_heads, self.num_qk_heads, self.head_dim, self.v_head_dim = num_heads, num_qk_heads, head_dim, v_head_dim
        self.conv_taps, self.decay_rank, self.gate_rank, self.norm_eps = int(conv_taps), decay_rank, gate_rank, float(norm_eps)
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "b": "b_proj", "a1": "a_down", "a2": "a_up",
                      "g1": "g_down", "g2": "g_up", "o": "o_proj", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm"}
        self.names.update(names or {})
        self.weight_suffix, self.conv_ending = weight_suffix, conv_ending
        self.channels = 2 * num_qk_heads * head_dim + num_heads * v_head_dim          # what the convolution sees
        self.state_floats = num_heads * head_dim * v_head_dim
        self.w_fused = self.w_conv = self.w_a2 = self.w_g2 = self.w_o = self.rate = self.dt_bias = self.norm_w = None

    def _n(self, which: str, weight: bool = True) -> str:
        return f"{self.prefix}.{self.names[which]}" + (self.weight_suffix if weight else "")

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(state=StateSpec((self.state_floats + max(0, self.conv_taps - 1) * self.channels,), "float32"))

    def weight_specs(self) -> List[WeightSpec]:
        D, H, G, hd, vd = self.hidden_size, self.num_heads, self.num_qk_heads, self.head_dim, self.v_head_dim
        rows = {"q": G * hd, "k": G * hd, "v": H * vd}
        specs = [WeightSpec(self._n(p), (n, D)) for p, n in rows.items()]
        if self.conv_taps > 0:
            specs += [WeightSpec(f"{self._n(p, False)}.{self.conv_ending}", (n, self.conv_taps), init=("normal", 0.5))
                      for p, n in rows.items()]
        specs += [WeightSpec(self._n("b"), (H, D)), WeightSpec(self._n("a1"), (self.decay_rank, D)),
                  WeightSpec(self._n("a2"), (H * hd, self.decay_rank), init=("normal", 0.2)),
                  WeightSpec(self._n("g1"), (self.gate_rank, D)),
                  WeightSpec(self._n("g2"), (H * vd, self.gate_rank), init=("normal", 0.2)),
                  WeightSpec(self._n("A_log", False), (H,), init=("normal", 0.5)),
                  WeightSpec(self._n("dt_bias", False), (H * hd,), init=("normal", 0.5)),
                  WeightSpec(self._n("norm", False), (vd,), init=("one_plus_normal", 0.1)),
                  WeightSpec(self._n("o"), (D, H * vd))]
        return specs

    def bind(self, tensors, dtype, device) -> None:
        ws = [tensors[self._n(p)] for p in ("q", "k", "v", "b", "a1", "g1")]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_fused = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        if self.conv_taps > 0:
            self.w_conv = torch.cat([tensors[f"{self._n(p, False)}.{self.conv_ending}"].float() for p in "qkv"], dim=0).contiguous()
        else:          # no convolution: one tap of weight one
            self.w_conv = torch.ones((self.channels, 1), dtype=torch.float32, device=device)
        self.w_a2, self.w_g2 = tensors[self._n("a2")].contiguous(), tensors[self._n("g2")].contiguous()
        self.w_o = tensors[self._n("o")]
        self.rate = torch.exp(tensors[self._n("A_log", False)].float()).contiguous()
        self.dt_bias = tensors[self._n("dt_bias", False)].float().contiguous()
        self.norm_w = tensors[self._n("norm", False)].float().contiguous()

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if cache is None or cache.state is None or not cache.writes:
            raise ops.KernelError("delta rule: the run needs a state plane of its own (the recurrence advances it)")
        T = x.shape[0]
        H, G, hd, vd = self.num_heads, self.num_qk_heads, self.head_dim, self.v_head_dim
        f32 = dict(dtype=torch.float32, device=x.device)
        fused = L.linear(x, self.w_fused, None, L.STORE)           # [T, q | k | v | beta | decay rank | gate rank]
        q, k, v = torch.empty((T, G * hd), **f32), torch.empty((T, G * hd), **f32), torch.empty((T, H * vd), **f32)
        segments = [ops.ConvSegment(0, G, hd, q, act="silu", norm="unit", eps=self.UNIT_EPS, scale=hd ** -0.5),
                    ops.ConvSegment(G * hd, G, hd, k, act="silu", norm="unit", eps=self.UNIT_EPS),
                    ops.ConvSegment(2 * G * hd, H, vd, v, act="silu")]
        spans = span_arrays(ctx)
        tail_off = self.state_floats
        ops.conv_prepare(fused, 0, self.channels, self.w_conv, segments, spans, cache.state, tail_off,
                         fuse_tail=ctx.decode_only)
        if not ctx.decode_only and self.conv_taps > 1:
            ops.conv_tail_update(fused, 0, self.channels, self.conv_taps, spans, cache.state, tail_off)
        c = self.channels
        decay = torch.empty((T, H * hd), **f32)
        ops.low_rank_up(fused, c + H, self.w_a2, decay, bias=self.dt_bias, mode="log_decay", rate=self.rate)
        gate = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        ops.low_rank_up(fused, c + H + self.decay_rank, self.w_g2, gate)
        o = torch.empty((T, H * vd), **f32)
        # a step with portions of prompts walks its spans in blocks of tokens; a step of single tokens token by token
        # (the choice follows from what a CUDA graph's key holds)
        ops.delta_rule(q, k, v, decay, fused[:, c: c + H], spans, H, G, hd, vd, cache.state, 0, o,
                       blocked=not ctx.decode_only)
        gated = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        ops.head_gate(o, gate, gated, H, vd, False, "sigmoid", unit_rms=True, eps=self.norm_eps, norm_weight=self.norm_w)
        L.linear(gated, self.w_o, None, L.RESIDUAL, residual=residual)


register_part("mixer", "channel_delta", ChannelDeltaMixer)
