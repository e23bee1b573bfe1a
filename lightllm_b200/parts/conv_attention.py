"""Attention whose q, k and v pass a short causal convolution over time before the heads are formed."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache import CacheSpec, KVSpec, StateSpec
from ..config import PartSpec, register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .attention import AttentionMixer
from .base import CacheView, LazyNorm


def span_arrays(ctx):
    return ctx.span_row, ctx.span_len, ctx.span_pos, ctx.span_slot, ctx.num_spans


class ConvAttentionMixer(AttentionMixer):
    """Grouped-query attention over the paged cache in which

    * every channel of q, k and v (bias included) first passes a causal convolution of ``conv_taps`` taps over time
      (``<projection>.conv``, ``[channels, taps]``, the last tap on the current token, zeros before the sequence;
      ``conv_taps = 0``: no convolution and no such tensors);
    * q and k are then rotated by position (``position``: adjacent or half-split pairs, optionally YaRN-scaled, with
      its magnitude applied) and, with ``qk_unit_rms``, divided head by head by their root mean square;
    * values may be of another width than keys (``v_head_dim``); ``scale``, ``window`` and ``chunk`` as the plain mixer;
    * the output projection may have a bias.

    One contraction makes q, k and v (bias in its epilogue); one kernel convolves, rotates, norms, writes q and the
    cache rows of the new tokens.  A request keeps the inputs of its last ``conv_taps - 1`` positions in its state
    slot (float32, ``[taps - 1, channels]``), so any cutting of its tokens gives the same result.  Convolution sums,
    angles, norms and the softmax are float32 in both precisions."""

    graph_safe = True
    accepts_lazy_norm = False
    takes_rotary_magnitude = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: Optional[int] = None, position: Optional[PartSpec] = None, conv_taps: int = 1,
                 qkv_bias: bool = True, out_bias: bool = True, window: Optional[int] = None, chunk: Optional[int] = None,
                 scale: Optional[float] = None, qk_unit_rms: bool = False, qk_norm_eps: float = 1e-6,
                 names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight", bias_ending: str = "bias",
                 conv_ending: str = "conv"):
        if conv_taps < 0:
            raise ValueError(f"a convolution has a number of taps (or 0 for none), got {conv_taps}")
        super().__init__(prefix, hidden_size, num_heads, num_kv_heads, head_dim, position=position, qkv_bias=qkv_bias,
                         out_bias=out_bias, window=window, scale=scale, names=names, weight_suffix=weight_suffix,
                         v_head_dim=v_head_dim, chunk=chunk)
        self.conv_taps, self.qk_unit_rms, self.qk_norm_eps = int(conv_taps), bool(qk_unit_rms), float(qk_norm_eps)
        self.bias_ending, self.conv_ending = bias_ending, conv_ending
        self.channels = (num_heads + num_kv_heads) * head_dim + num_kv_heads * self.v_head_dim
        self.w_conv = None
        table = self.position.rotary_table()
        if table is not None and table[1] and not table[2]:
            raise ValueError("the convolution kernel rotates adjacent pairs (the interleaved layout) only")

    def cache_spec(self) -> CacheSpec:
        kv = super().cache_spec().kv
        state = None
        if self.conv_taps > 1:
            state = StateSpec(((self.conv_taps - 1) * self.channels,), "float32")
        return CacheSpec(kv=kv, state=state)

    def weight_specs(self) -> List[WeightSpec]:
        D, H, G, hd, vd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        rows = {"q": H * hd, "k": G * hd, "v": G * vd}
        specs = [WeightSpec(self._n(p, "weight"), (n, D)) for p, n in rows.items()]
        specs.append(WeightSpec(self._n("o", "weight"), (D, H * vd)))
        if self.qkv_bias:
            specs += [WeightSpec(self._n(p, self.bias_ending), (n,)) for p, n in rows.items()]
        if self.out_bias:
            specs.append(WeightSpec(self._n("o", self.bias_ending), (D,)))
        if self.conv_taps > 0:
            specs += [WeightSpec(self._n(p, self.conv_ending), (n, self.conv_taps), init=("normal", 0.5)) for p, n in rows.items()]
        return specs + self.position.weight_specs()

    def bind(self, tensors, dtype, device) -> None:
        ws = [tensors[self._n(p, "weight")] for p in "qkv"]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_qkv = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        self.w_o = tensors[self._n("o", "weight")]
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[self._n(p, self.bias_ending)].float() for p in "qkv"]).contiguous()
        if self.out_bias:
            self.b_o = tensors[self._n("o", self.bias_ending)].float().contiguous()
        if self.conv_taps > 0:
            self.w_conv = torch.cat([tensors[self._n(p, self.conv_ending)].float() for p in "qkv"], dim=0).contiguous()
        else:          # no convolution: one tap of weight one
            self.w_conv = torch.ones((self.channels, 1), dtype=torch.float32, device=device)
        self.position.bind(tensors, dtype, device)

    def prepare(self, ctx, cache=None) -> None:
        self._plan(ctx, ctx.dtype)

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if cache is None or not cache.writes or (self.conv_taps > 1 and cache.state is None):
            raise ops.KernelError("convolved attention: the run needs cache planes and a state plane of its own")
        T = x.shape[0]
        H, G, hd, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        fused = L.linear(x, self.w_qkv, self.b_qkv, L.STORE)           # [T, q | k | v]
        table = self.position.rotary_table() or (None, 0, True)
        freq, rotary_dim, _ = table
        norm = "rms" if self.qk_unit_rms else None
        q = torch.empty((T, H * hd), dtype=x.dtype, device=x.device)
        segments = [ops.ConvSegment(0, H, hd, q, rotary_dim=rotary_dim, norm=norm, eps=self.qk_norm_eps),
                    ops.ConvSegment(H * hd, G, hd, cache.k, to_cache=True, rotary_dim=rotary_dim, norm=norm,
                                    eps=self.qk_norm_eps),
                    ops.ConvSegment((H + G) * hd, G, vd, cache.v, to_cache=True)]
        spans = span_arrays(ctx)
        ops.conv_prepare(fused, 0, self.channels, self.w_conv, segments, spans, cache.state, 0,
                         ctx.slot_mapping[cache.group], freq, getattr(self.position, "magnitude", 1.0),
                         fuse_tail=ctx.decode_only)
        if self.conv_taps > 1 and not ctx.decode_only:
            ops.conv_tail_update(fused, 0, self.channels, self.conv_taps, spans, cache.state, 0)          # (its taps: w_conv's)
        attn = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        self.attend(q, cache, ctx, attn)
        L.linear(attn, self.w_o, self.b_o, L.RESIDUAL, residual=residual)


register_part("mixer", "conv_attention", ConvAttentionMixer)
