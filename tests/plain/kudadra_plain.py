"""A plain, slow implementation of the Kudadra decoder: whole sequences, no cache, on the CPU, one function
for each mechanism, in float64 by default.  It shares no code with the engine.

The design in this file's notation (x is the residual stream, one row per token, positions from 0):

    x <- x + LN1(mixer(x));  x <- x + LN2(ff(x))          the norm sits on the branch's OUTPUT; branches read x itself
    LN(y) = (y - mean) / sqrt(var + eps) * w + b           var = mean of squared deviations
    rms(y) = y / sqrt(mean(y^2) + eps)

Mixers (all project the same input h = x):
  latent attention   q = Wq h;  c = rms(Wdkv h) * g;  per head k = Wuk c, v = Wuv c;  s_ij = scale q_i.k_j for j <= i;
                     p_ij = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij'));  out = Wo concat_h(sigmoid(Wg h)_h * sum_j p_ij v_j)
  window attention   q, k, v = Wq h, Wk h, Wv h;  q = rms(q) * gq over ALL heads at once, k likewise;  rotary on the first
                     `dims` of each head;  j visible iff 0 <= i - j < window;  softmax;  out = Wo (sigmoid(Wg h) * concat heads)
  retention          q, k rotated, k *= dim^-1/2;  S_t = decay_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;
                     out = Wo (concat_h rms(o_t,h) * silu(Wg h))
Feed-forward          g = min(Wgate h, L);  u = clamp(Wup h, -L, L);  out = Wdown (g * sigmoid(1.702 g) * (u + 1))
Rotary               pair (i, i + dims/2), angle = p * base^(-2i/dims):  (a, b) -> (a cos - b sin, b cos + a sin)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def plain_layer_norm(y, w, b, eps):
    mean = y.mean(-1, keepdim=True)
    var = ((y - mean) ** 2).mean(-1, keepdim=True)
    return (y - mean) / torch.sqrt(var + eps) * w + b


def plain_rms(y, eps, w=None):
    out = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return out if w is None else out * w


def plain_rotate(x, positions, dims: int, base: float):
    """x [T, H, d]: the first ``dims`` of each head are turned, pair (i, i + dims/2)."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.pow(torch.tensor(base, dtype=x.dtype), -2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]          # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def plain_latent_attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    T = h.shape[0]
    H, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q = (h @ w["q"].T).view(T, H, dim)
    c = plain_rms(h @ w["dkv"].T, eps, w["dkv.norm"])            # [T, rank]: all that a cache has to keep
    k = (c @ w["uk"].T).view(T, H, dim)
    v = (c @ w["uv"].T).view(T, H, vdim)
    gate = torch.sigmoid(h @ w["g"].T)                            # [T, H]
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh].T) * m["scale"]
        s = s.masked_fill(torch.ones(T, T).triu(1).bool(), -math.inf)
        big = torch.maximum(s.max(-1, keepdim=True).values, w["sink"][hh])
        e = torch.exp(s - big)
        den = e.sum(-1, keepdim=True) + torch.exp(w["sink"][hh] - big)
        out[:, hh] = (e / den) @ v[:, hh] * gate[:, hh:hh + 1]
    return out.reshape(T, H * vdim) @ w["o"].T


def plain_window_attention(h, w, m: dict, eps: float):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = plain_rms(h @ w["q"].T, eps, w["q.norm"]).view(T, H, dim)
    k = plain_rms(h @ w["k"].T, eps, w["k.norm"]).view(T, G, dim)
    v = (h @ w["v"].T).view(T, G, vdim)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q, k = plain_rotate(q, pos, rot["dims"], rot["base"]), plain_rotate(k, pos, rot["dims"], rot["base"])
    d = pos[:, None] - pos[None, :]
    hidden = (d < 0) | (d >= m["mask"]["size"])
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = ((q[:, hh] @ k[:, g].T) * m["scale"]).masked_fill(hidden, -math.inf)
        out[:, hh] = torch.softmax(s, dim=-1) @ v[:, g]
    return (out.reshape(T, H * vdim) * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def plain_retention(h, w, m: dict, eps: float):
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = plain_rotate((h @ w["q"].T).view(T, H, dim), pos, rot["dims"], rot["base"])
    k = plain_rotate((h @ w["k"].T).view(T, H, dim), pos, rot["dims"], rot["base"]) * dim ** -0.5
    v = (h @ w["v"].T).view(T, H, vdim)
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(T):
            S = m["decay"][hh] * S + torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    out = plain_rms(out, eps).reshape(T, H * vdim)
    z = h @ w["g"].T
    return (out * (z * torch.sigmoid(z))) @ w["o"].T


def plain_feed_forward(h, w, f: dict):
    L = f["limit"]
    g = torch.clamp(h @ w["gate"].T, max=L)
    u = torch.clamp(h @ w["up"].T, min=-L, max=L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


MIXERS = {"latent_attention": plain_latent_attention, "attention": plain_window_attention,
          "retention": plain_retention}


def _sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def plain_forward(tokens: List[int], weights: Dict[str, torch.Tensor], config: dict, dtype=torch.float64,
                  layers_out: Optional[list] = None):
    """Logits [T, vocab] of one sequence; ``layers_out`` receives the stream after every layer."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](x, _sub(W, p + "mix."), layer["mixer"], eps)
        x = x + plain_layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            y = plain_feed_forward(x, _sub(W, p + "mlp."), layer["mlp"])
            x = x + plain_layer_norm(y, W[p + "norm2"], W[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = plain_layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return x @ W["head"].T
