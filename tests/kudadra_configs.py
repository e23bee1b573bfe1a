"""Tiny Kudadra configurations for the tests, and random weights for them drawn here (names and shapes restated from
the design, not taken from the engine).  The configurations differ in every size, in the order of the layers, in which
values happen to be equal or 1, and in which kernels the engine picks for them."""
import copy
import json
import os
from typing import Dict

import torch


def _latent(heads, dim, vdim, rank, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale or dim ** -0.5}}


def _attn(heads, kv_heads, dim, vdim, window, rot_dims, base=10000.0, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                      "rot": {"dims": rot_dims, "base": base}, "scale": scale or dim ** -0.5}}


def _ret(heads, dim, vdim, decay, rot_dims, base=1000000.0):
    return {"type": "retention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"dims": rot_dims, "base": base}}}


def _with_mlp(layer, ff, limit):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}
    return layer


# P: odd sizes everywhere (CUDA-core kernels in both precisions): values narrower and wider than keys, partial rotation,
# a window shorter than a page, a layer without feed-forward, sizes that are no multiples of 8.
KUD_P = {"architecture": "Kudadra", "vocab": 301, "width": 44, "norm": {"eps": 1e-5}, "layers": [
    _with_mlp(_attn(4, 2, 12, 20, 11, 6, base=500.0), 52, 1.5),
    _with_mlp(_ret(3, 12, 20, [0.9, 0.97, 0.995], 8), None, 0),
    _with_mlp(_latent(3, 12, 20, 28, scale=0.4), 36, 0.75),
    _with_mlp(_attn(3, 3, 20, 12, 40, 20), 52, 7.0),
]}
# Q: the sizes the tensor-core kernels take in bfloat16 (heads of 64 and 128, a window longer than a tile), a latent of
# 128 with narrow heads and one of 64 with heads as wide (whose up-projections the engine folds into its matrices),
# retention heads of 128 (two threads a column) and 256 (four).
KUD_Q = {"architecture": "Kudadra", "vocab": 517, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    _with_mlp(_latent(4, 32, 48, 128), 192, 1.0),
    _with_mlp(_attn(4, 1, 64, 64, 150, 32), 192, 1.0),
    _with_mlp(_ret(2, 128, 64, [0.96875, 0.999], 64), 192, 2.0),
    _with_mlp(_attn(2, 2, 128, 128, 300, 128, base=1000000.0), None, 0),
    _with_mlp(_ret(1, 256, 32, [0.99], 0), 192, 1.0),
    _with_mlp(_latent(3, 64, 64, 64), 192, 1.0),
]}
# R: recurrent layers only (no pages at all), one head, decay 1 (nothing is ever forgotten) and a fast decay.
KUD_R = {"architecture": "Kudadra", "vocab": 97, "width": 32, "norm": {"eps": 1e-5}, "layers": [
    _with_mlp(_ret(1, 16, 16, [1.0], 16, base=100.0), 40, 1.0),
    _with_mlp(_ret(2, 8, 24, [0.5, 0.875], 4), 40, 1.0),
]}
# S: attention only, a window of one token (a position sees itself alone) and one that no test sequence fills.
KUD_S = {"architecture": "Kudadra", "vocab": 211, "width": 40, "norm": {"eps": 1e-5}, "layers": [
    _with_mlp(_attn(2, 1, 8, 8, 1, 8), 24, 1.0),
    _with_mlp(_latent(1, 8, 8, 8), 24, 1.0),
    _with_mlp(_attn(2, 2, 16, 8, 100000, 0), 24, 1.0),
    _with_mlp(_latent(5, 16, 8, 40), None, 0),
]}
# T: widths that are multiples of nothing (no 16-byte row anywhere: every kernel's scalar path), odd head sizes, a
# feed-forward of odd width, a vocabulary of a prime.
KUD_T = {"architecture": "Kudadra", "vocab": 79, "width": 50, "norm": {"eps": 1e-5}, "layers": [
    _with_mlp(_ret(2, 10, 7, [0.75, 0.9375], 6, base=300.0), 33, 1.0),
    _with_mlp(_attn(3, 1, 10, 7, 9, 4), 33, 2.0),
    _with_mlp(_latent(3, 6, 5, 11), 33, 0.5),
]}
CONFIGS = {"P": KUD_P, "Q": KUD_Q, "R": KUD_R, "S": KUD_S, "T": KUD_T}
PAGE_SIZE = {"P": 16, "Q": 16, "R": 16, "S": 8, "T": 16}


def config(name):
    return copy.deepcopy(CONFIGS[name])


def tensor_shapes(cfg) -> Dict[str, tuple]:
    """Every tensor of a model of this design, by the naming rule of its checkpoints."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "head": (V, D), "final.norm": (D,), "final.norm.b": (D,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1.b"] = (D,)
        H, dim, vdim = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "latent_attention":
            r = m["kv_rank"]
            out.update({p + "mix.q": (H * dim, D), p + "mix.dkv": (r, D), p + "mix.dkv.norm": (r,),
                        p + "mix.uk": (H * dim, r), p + "mix.uv": (H * vdim, r), p + "mix.sink": (H,),
                        p + "mix.g": (H, D), p + "mix.o": (D, H * vdim)})
        elif layer["type"] == "attention":
            G = m["kv_heads"]
            out.update({p + "mix.q": (H * dim, D), p + "mix.k": (G * dim, D), p + "mix.v": (G * vdim, D),
                        p + "mix.q.norm": (H * dim,), p + "mix.k.norm": (G * dim,), p + "mix.g": (H * vdim, D),
                        p + "mix.o": (D, H * vdim)})
        else:
            out.update({p + "mix.q": (H * dim, D), p + "mix.k": (H * dim, D), p + "mix.v": (H * vdim, D),
                        p + "mix.g": (H * vdim, D), p + "mix.o": (D, H * vdim)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            out[p + "norm2"] = out[p + "norm2.b"] = (D,)
            out.update({p + "mlp.gate": (ff, D), p + "mlp.up": (ff, D), p + "mlp.down": (D, ff)})
    return out


def random_weights(cfg, seed: int, sharp: float = 1.0, sink: float = None, store=torch.float32) -> Dict[str, torch.Tensor]:
    """Weights that keep activations of order one (matrices N(0, 1/in)); ``sharp`` multiplies every q and k projection
    (sharp attention: one key can stand out), ``sink`` sets every sink to one value.  Rounded once to ``store``."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        tail = name.split(".")[-1]
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif tail == "b":
            t = 0.1 * torch.randn(shape, generator=g)
        elif tail == "sink":
            t = torch.randn(shape, generator=g) if sink is None else torch.full(shape, float(sink))
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
            if tail in ("q", "k") and ".mix." in name:
                t = t * sharp
        out[name] = t.to(store).contiguous()
    return out


def write_model(cfg, weights, out_dir: str) -> str:
    from lightllm_b200.weights import save_file
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(weights, os.path.join(out_dir, "model.safetensors"))
    return out_dir
