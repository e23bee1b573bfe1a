"""Attention mixers beyond the plain one: q/k normalisation over the whole projection, output gates, values of
another width than the keys, and attention over a shared low-rank latent with learned sinks."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import PartSpec, register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .attention import AttentionMixer
from .base import CacheView, LazyNorm

GATES = (None, "elementwise", "per_head")


class GatedAttentionMixer(AttentionMixer):
    """Grouped-query attention over the paged cache with

    * ``qk_norm``: q and k are RMS-normalised over their WHOLE projection (all heads at once, one weight per
      column, ``<q>.norm`` / ``<k>.norm``) before the rotation;
    * ``gate``: the heads' outputs are multiplied by ``act(W_g x)`` before the output projection, element by element
      (``W_g`` has ``heads * v_head_dim`` rows) or one number per head (``heads`` rows);
    * ``v_head_dim``: values (and outputs) of another width than keys;
    * ``window`` and ``scale`` as the plain mixer.

    One contraction makes q, k, v and the gate's input from the same x; one kernel norms, rotates and writes the
    cache; the gate is applied in place on the attention's output.  Norm statistics, angles and the softmax are float32."""

    graph_safe = True
    accepts_lazy_norm = False

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: Optional[int] = None, position: Optional[PartSpec] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, qk_norm: bool = False, qk_norm_eps: float = 1e-6,
                 gate: Optional[str] = None, gate_act: str = "sigmoid", names: Optional[Dict[str, str]] = None,
                 weight_suffix: str = ".weight"):
        if gate not in GATES:
            raise ValueError(f"gate must be one of {GATES}, got {gate!r}")
        if gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"gate_act must be 'sigmoid' or 'silu', got {gate_act!r}")
        base = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "g": "g_proj"}
        base.update(names or {})
        super().__init__(prefix, hidden_size, num_heads, num_kv_heads, head_dim, position=position, qkv_bias=False,
                         out_bias=False, window=window, scale=scale, names=base, weight_suffix=weight_suffix,
                         v_head_dim=v_head_dim)
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.gate, self.gate_act = gate, gate_act
        self.w_fused = self.q_norm_w = self.k_norm_w = None

    def _gate_rows(self) -> int:
        return 0 if self.gate is None else (self.num_heads if self.gate == "per_head" else self.num_heads * self.v_head_dim)

    def weight_specs(self) -> List[WeightSpec]:
        D, H, G, hd, vd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        specs = [WeightSpec(self._n("q", "weight"), (H * hd, D)), WeightSpec(self._n("k", "weight"), (G * hd, D)),
                 WeightSpec(self._n("v", "weight"), (G * vd, D)), WeightSpec(self._n("o", "weight"), (D, H * vd))]
        if self.gate is not None:
            specs.append(WeightSpec(self._n("g", "weight"), (self._gate_rows(), D)))
        if self.qk_norm:
            specs += [WeightSpec(self._n("q", "norm"), (H * hd,), init=("one_plus_normal", 0.1)),
                      WeightSpec(self._n("k", "norm"), (G * hd,), init=("one_plus_normal", 0.1))]
        return specs + self.position.weight_specs()

    def bind(self, tensors, dtype, device) -> None:
        ws = [tensors[self._n(p, "weight")] for p in ("q", "k", "v") + (("g",) if self.gate is not None else ())]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_fused = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        self.w_o = tensors[self._n("o", "weight")]
        if self.qk_norm:
            self.q_norm_w = tensors[self._n("q", "norm")].float().contiguous()
            self.k_norm_w = tensors[self._n("k", "norm")].float().contiguous()
        self.position.bind(tensors, dtype, device)

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        T = x.shape[0]
        H, G, hd, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        fused = L.linear(x, self.w_fused, None, L.STORE)
        table = self.position.rotary_table()
        if table is None:
            table = (None, 0, False)
        inv_freq, rotary_dim, interleaved = table
        q = torch.empty((T, H * hd), dtype=x.dtype, device=x.device)
        writes = cache.writes
        ops.qkv_prepare(fused, 0, H * hd, (H + G) * hd, H, G if writes else 0, hd, vd, ctx.positions,
                        ctx.slot_mapping[cache.group] if writes else None, q, cache.k if writes else None,
                        cache.v if writes else None, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, inv_freq,
                        rotary_dim, interleaved)
        attn = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        self.attend(q, cache, ctx, attn)
        if self.gate is not None:
            g0 = (H + G) * hd + G * vd
            ops.head_gate(attn, fused[:, g0: g0 + self._gate_rows()], attn, H, vd, self.gate == "per_head", self.gate_act)
        L.linear(attn, self.w_o, None, L.RESIDUAL, residual=residual)


class LatentAttentionMixer(AttentionMixer):
    """Attention whose keys and values are up-projections of one low-rank latent per token, so that only the latent is
    cached: ``c = rms(W_dkv x) * g`` (``rank`` numbers a token), per head ``k = W_uk c``, ``v = W_uv c``.

    The up-projections are folded onto the query and the output (``q.k = (W_uk^T q).c`` and ``sum p v = W_uv (sum p c)``),
    so the kernels see multi-query attention with ONE kv head of width ``rank`` whose value rows are its key rows, and
    nothing of the context is ever expanded.  ``sinks``: a learned logit per head (``<prefix>.sink``) that joins the
    softmax denominator once, without key or value and unscaled.  ``gate`` as :class:`GatedAttentionMixer`.  No positions.

    ``fold``: multiply the up-projections into the neighbouring matrices when the model is bound
    (``W_q' = blockdiag(W_uk^T) W_q`` with ``heads * rank`` rows, ``W_o' = W_o blockdiag(W_uv)``; a gate of one number a
    head commutes with ``W_uv``), so that a layer is two contractions around the attention like any other; without it
    the two per-head contractions run as kernels of their own.  ``None`` folds when the latent is at most twice as wide
    as a head's keys and values (the folded matrices are ``rank / head_dim`` times the size of the plain ones)."""

    graph_safe = True
    accepts_lazy_norm = False

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, rank: int,
                 norm_eps: float = 1e-6, scale: Optional[float] = None, window: Optional[int] = None,
                 sinks: bool = False, gate: Optional[str] = None, gate_act: str = "sigmoid",
                 names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight", fold: Optional[bool] = None):
        if gate not in GATES:
            raise ValueError(f"gate must be one of {GATES}, got {gate!r}")
        if fold and gate == "elementwise":
            raise ValueError("a gate on every element does not commute with the value up-projection: fold=False")
        if fold is None:
            fold = gate != "elementwise" and rank <= 2 * head_dim and rank <= 2 * v_head_dim
        self.fold = bool(fold)
        base = {"q": "q_proj", "dkv": "kv_down", "uk": "k_up", "uv": "v_up", "o": "o_proj", "g": "g_proj", "sink": "sink"}
        base.update(names or {})
        # the attention kernels' geometry: one kv head of `rank`, values in the key rows
        super().__init__(prefix, hidden_size, num_heads, 1, rank, position=None, qkv_bias=False, out_bias=False,
                         window=window, scale=scale if scale is not None else head_dim ** -0.5, names=base,
                         weight_suffix=weight_suffix, v_head_dim=rank)
        self.values_in_keys = True
        self.q_dim, self.out_dim, self.rank = int(head_dim), int(v_head_dim), int(rank)
        self.norm_eps, self.has_sinks, self.gate, self.gate_act = float(norm_eps), bool(sinks), gate, gate_act
        self.w_fused = self.w_q_up = self.w_v_up = self.c_norm_w = None

    def _gate_rows(self) -> int:
        return 0 if self.gate is None else (self.num_heads if self.gate == "per_head" else self.num_heads * self.out_dim)

    def weight_specs(self) -> List[WeightSpec]:
        D, H, r = self.hidden_size, self.num_heads, self.rank
        specs = [WeightSpec(self._n("q", "weight"), (H * self.q_dim, D)), WeightSpec(self._n("dkv", "weight"), (r, D)),
                 WeightSpec(self._n("dkv", "norm"), (r,), init=("one_plus_normal", 0.1)),
                 WeightSpec(self._n("uk", "weight"), (H * self.q_dim, r)),
                 WeightSpec(self._n("uv", "weight"), (H * self.out_dim, r)),
                 WeightSpec(self._n("o", "weight"), (D, H * self.out_dim))]
        if self.has_sinks:
            specs.append(WeightSpec(f"{self.prefix}.{self.names['sink']}", (H,), init=("normal", 1.0)))
        if self.gate is not None:
            specs.append(WeightSpec(self._n("g", "weight"), (self._gate_rows(), D)))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        H, r = self.num_heads, self.rank
        ws = [tensors[self._n(p, "weight")] for p in ("q", "dkv") + (("g",) if self.gate is not None else ())]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        uk = tensors[self._n("uk", "weight")].view(H, self.q_dim, r)
        uv = tensors[self._n("uv", "weight")].view(H, self.out_dim, r)
        self.w_o = tensors[self._n("o", "weight")]
        if self.fold:          # products in float64, rounded once to the weights' dtype
            D = self.hidden_size
            wq = ws[0].double().view(H, self.q_dim, D)
            ws[0] = torch.einsum("hdr,hdk->hrk", uk.double(), wq).reshape(H * r, D)
            wo = self.w_o.double().view(D, H, self.out_dim)
            self.w_o = torch.einsum("khe,her->khr", wo, uv.double()).reshape(D, H * r).to(self.w_o.dtype).contiguous()
        else:
            # [H, rank, dim]: row o of head h is column o of that head's key up-projection.  The per-head contraction
            # takes its weights in the activations' dtype (also where a checkpoint stores them in 32 bits)
            self.w_q_up = uk.to(dtype).transpose(1, 2).contiguous()
            self.w_v_up = uv.to(dtype).contiguous()
        self.w_fused = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        self.c_norm_w = tensors[self._n("dkv", "norm")].float().contiguous()
        if self.has_sinks:
            self.sinks = tensors[f"{self.prefix}.{self.names['sink']}"].float().contiguous()

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        T = x.shape[0]
        H, r = self.num_heads, self.rank
        fused = L.linear(x, self.w_fused, None, L.STORE)           # [T, q | rank | gate]
        q = torch.empty((T, H * r), dtype=x.dtype, device=x.device)
        slots = ctx.slot_mapping[cache.group] if cache.writes else None
        if self.fold:
            # q is already W_uk^T q; one kernel copies it out of the fused rows and writes the normed latent to the
            # cache rows of the new tokens
            ops.qkv_prepare(fused, 0, H * r, -1, H, 1 if cache.writes else 0, r, r, ctx.positions, slots, q,
                            cache.k if cache.writes else None, None, None, self.c_norm_w if cache.writes else None,
                            self.norm_eps)
            mixed = torch.empty((T, H * r), dtype=x.dtype, device=x.device)
            self.attend(q, cache, ctx, mixed)                      # sum_j p_ij c_j
            if self.gate is not None:
                g0 = H * r + r
                ops.head_gate(mixed, fused[:, g0: g0 + self._gate_rows()], mixed, H, r, True, self.gate_act)
            L.linear(mixed, self.w_o, None, L.RESIDUAL, residual=residual)
            return
        if cache.writes:          # the normed latent goes to the cache rows of the new tokens
            ops.qkv_prepare(fused, 0, H * self.q_dim, -1, 0, 1, r, r, ctx.positions, slots, None,
                            cache.k, None, None, self.c_norm_w, self.norm_eps)
        ops.head_linear(fused, 0, self.w_q_up, q)                  # W_uk^T q, head by head
        mixed = torch.empty((T, H * r), dtype=x.dtype, device=x.device)
        self.attend(q, cache, ctx, mixed)                          # sum_j p_ij c_j
        out = torch.empty((T, H * self.out_dim), dtype=x.dtype, device=x.device)
        ops.head_linear(mixed, 0, self.w_v_up, out)                # W_uv (...)
        if self.gate is not None:
            g0 = H * self.q_dim + r
            ops.head_gate(out, fused[:, g0: g0 + self._gate_rows()], out, H, self.out_dim, self.gate == "per_head",
                          self.gate_act)
        L.linear(out, self.w_o, None, L.RESIDUAL, residual=residual)


register_part("mixer", "gated_attention", GatedAttentionMixer)
register_part("mixer", "latent_attention", LatentAttentionMixer)
