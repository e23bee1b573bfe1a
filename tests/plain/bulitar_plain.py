"""A plain, slow evaluation of the Bulitar design: one function a mechanism, written from the design's equations in
float64 torch on the CPU.  It shares no code with the engine; the tests compare the engine with it.

``tensors`` maps checkpoint names to tensors; ``cfg`` is the config.json dictionary.  Every function takes whole
sequences (positions 0 .. T-1 of one request).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c]`` with zeros before the first token."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotary_frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    """(frequency of each pair, factor on cos and sin)."""
    dims, base = rot["dims"], float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])

    def turn_dim(t):
        return dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
    lo = max(math.floor(turn_dim(sc["fast"])), 0)
    hi = min(math.ceil(turn_dim(sc["slow"])), dims - 1)
    out = []
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(float(f[i]) / factor * ramp + float(f[i]) * (1 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x ``[T, heads, dim]``: dimensions 2i and 2i+1 of the first ``dims`` form a pair."""
    if not rot or rot["dims"] == 0:
        return x
    f, m = rotary_frequencies(rot)
    dims = rot["dims"]
    a = positions.to(F)[:, None] * f[None, :]                  # [T, dims/2]
    c, s = (torch.cos(a) * m)[:, None, :], (torch.sin(a) * m)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def chunked_softmax_attention(q, k, v, scale: float, chunk: Optional[int]) -> torch.Tensor:
    """q ``[T, H, dim]``, k ``[T, G, dim]``, v ``[T, G, vdim]``; row i sees j <= i in its own chunk of positions."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = (i // chunk) * chunk if chunk else 0
            s = (k[lo: i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[lo: i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)

    def proj(name):
        y = h @ W[f"{p}.{name}"].T + W[f"{p}.{name}.b"]
        return short_conv(y, W[f"{p}.{name}.conv"]) if f"{p}.{name}.conv" in W else y
    q = proj("q").view(T, H, dim)
    k = proj("k").view(T, G, dim)
    v = proj("v").view(T, G, vdim)
    q = unit_rms(rotate_pairs(q, pos, m.get("rot")), eps)
    k = unit_rms(rotate_pairs(k, pos, m.get("rot")), eps)
    chunk = (m.get("mask") or {}).get("size")
    o = chunked_softmax_attention(q, k, v, float(m["scale"]), chunk)
    return o.reshape(T, H * vdim) @ W[f"{p}.o"].T + W[f"{p}.o.b"]


def delta_rule(q, k, v, g, beta) -> torch.Tensor:
    """One head.  q, k, g ``[T, dim]``, v ``[T, vdim]``, beta ``[T]``; the state ``[dim, vdim]`` starts at zero."""
    T, dim = q.shape
    S = torch.zeros(dim, v.shape[1], dtype=q.dtype)
    out = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def proj(name):
        y = short_conv(h @ W[f"{p}.{name}"].T, W[f"{p}.{name}.conv"])
        return y * torch.sigmoid(y)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q = unit(proj("q").view(T, G, dim)) * dim ** -0.5
    k = unit(proj("k").view(T, G, dim))
    v = proj("v").view(T, H, vdim)
    beta = torch.sigmoid(h @ W[f"{p}.b"].T)                                           # [T, H]
    a = (h @ W[f"{p}.a1"].T) @ W[f"{p}.a2"].T + W[f"{p}.dt_bias"]                      # [T, H*dim]
    rate = torch.exp(W[f"{p}.A_log"])                                                  # [H]
    g = torch.exp(-rate[None, :, None] * torch.nn.functional.softplus(a.view(T, H, dim)))
    o = torch.zeros(T, H, vdim, dtype=h.dtype)
    for i in range(H):
        j = i // (H // G)
        o[:, i] = delta_rule(q[:, j], k[:, j], v[:, i], g[:, i], beta[:, i])
    o = unit_rms(o, eps) * W[f"{p}.norm"]
    gate = torch.sigmoid((h @ W[f"{p}.g1"].T) @ W[f"{p}.g2"].T).view(T, H, vdim)
    return (o * gate).reshape(T, H * vdim) @ W[f"{p}.o"].T


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, r: dict) -> Tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts ``[T, top]``, their weights)."""
    s = torch.sigmoid(h @ W[f"{p}.router"].T)
    choice = s + W[f"{p}.correction"]
    idx = torch.topk(choice, r["top"], dim=-1).indices
    return idx, torch.gather(s, 1, idx) * float(r["scale"])


def moe(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    idx, wts = route(h, W, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wts[t]):
            z = W[f"{p}.e{e}.gate"] @ h[t]
            a = z * torch.sigmoid(z) * (W[f"{p}.e{e}.up"] @ h[t])
            out[t] += w * (W[f"{p}.e{e}.down"] @ a)
    return out


def run_list(cfg: dict) -> List[Tuple[int, Optional[int]]]:
    """(layer, pass number if the layer opens a pass of the loop else None) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            out.append((i, t if i == loop["start"] else None))
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(tokens, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=F):
    """Logits ``[T, vocab]`` of one whole sequence, and the stream after every run of a layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    x0 = x.clone()
    streams = []
    for i, opens in run_list(cfg):
        if opens is not None:
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].T + W["loop.step"][opens]
        layer, p = cfg["layers"][i], f"l{i}"
        h = layer_norm(x, W[f"{p}.norm1"], eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(h, W, f"{p}.mix", layer["mixer"], eps)
        elif layer["type"] == "channel_delta":
            x = x + channel_delta_mixer(h, W, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + moe(layer_norm(x, W[f"{p}.norm2"], eps), W, f"{p}.mlp", layer["mlp"])
        streams.append(x.clone())
    logits = layer_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(streams)
