"""Tiny Bulitar configurations for the tests, and random weights for them drawn here (names and shapes restated from
the design, not taken from the engine).  The configurations differ in every size, in the order of the layers, in where
the loop lies, in which values happen to be equal or 1, and in which kernels the engine picks for them."""
import copy
import json
import os
from typing import Dict

import torch


def _attn(heads, kv_heads, dim, vdim, conv, chunk, rot_dims, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5}
    if conv is not None:          # (no 'conv': the layer has no convolution and no such tensors)
        m["conv"] = conv
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot_dims is not None:
        m["rot"] = {"dims": rot_dims, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": m}


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def _moe(layer, ff, experts, top, scale):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top,
                                                                                         "scale": scale}}
    return layer


YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}

# U: odd sizes everywhere (CUDA-core kernels in both precisions): values wider and narrower than keys, partial rotation
# with scaled frequencies, a chunk shorter than a page and one that is no multiple of anything, taps 2 and 3, a layer
# without feed-forward, a loop of two layers run three times in the middle of the model.
BUL_U = {"architecture": "Bulitar", "vocab": 301, "width": 44, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
         "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    _moe(_attn(4, 2, 12, 20, 3, 11, 6, base=500.0, scaling=YARN), 20, 5, 2, 1.5),
    _moe(_delta(4, 2, 12, 20, 2, 5, 7), 20, 5, 2, 1.5),
    _moe(_attn(3, 3, 20, 12, 2, 37, 20), None, 0, 0, 0),
    _moe(_delta(3, 1, 10, 6, 3, 3, 4), 28, 3, 1, 0.5),
]}
# V: the sizes the tensor-core kernels take in bfloat16 (heads of 64 and 128 with values as wide, chunks longer than a
# tile and across page borders), delta heads of 64, 128 and 256 key channels, four taps, every expert chosen (top =
# experts), the whole model inside the loop.
BUL_V = {"architecture": "Bulitar", "vocab": 517, "width": 128, "embedding": {"scale": 12.0}, "norm": {"eps": 1e-6},
         "loop": {"start": 0, "stop": 5, "times": 2}, "layers": [
    _moe(_attn(4, 1, 64, 64, 4, 150, 32, scaling={"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0}), 64, 4, 4, 1.0),
    _moe(_delta(2, 2, 128, 64, 4, 16, 8), 64, 6, 2, 2.5),
    _moe(_attn(2, 2, 128, 128, 3, 300, 128, base=1000000.0), None, 0, 0, 0),
    _moe(_delta(4, 1, 64, 32, 3, 24, 24), 64, 6, 2, 2.5),
    _moe(_delta(1, 1, 256, 16, 2, 8, 8), 64, 4, 1, 1.0),
]}
# W: what the others make unequal is equal, 1 or absent here: no loop, no convolution in one layer and one tap in the
# others (no convolution state at all), no mask, no rotation in one layer and a full one in the other, one expert, one head.
BUL_W = {"architecture": "Bulitar", "vocab": 97, "width": 32, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "layers": [
    _moe(_attn(1, 1, 16, 16, None, None, None), 24, 1, 1, 1.0),
    _moe(_delta(1, 1, 16, 16, 1, 4, 4), 24, 2, 2, 1.0),
    _moe(_attn(2, 1, 8, 8, 1, 5, 8), 24, 3, 2, 1.0),
]}
# X: a loop that is run once, at the model's end; widths that are multiples of nothing; a chunk of one position (a
# token sees itself alone).
BUL_X = {"architecture": "Bulitar", "vocab": 79, "width": 50, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
         "loop": {"start": 1, "stop": 3, "times": 1}, "layers": [
    _moe(_delta(2, 2, 10, 7, 3, 3, 5), 33, 4, 3, 2.0),
    _moe(_attn(3, 1, 10, 7, 3, 1, 4), 33, 4, 3, 2.0),
    _moe(_attn(2, 2, 6, 9, 2, 9, 6, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}), 33, 7, 2, 0.7),
]}
CONFIGS = {"U": BUL_U, "V": BUL_V, "W": BUL_W, "X": BUL_X}
PAGE_SIZE = {"U": 16, "V": 16, "W": 8, "X": 16}


def config(name):
    return copy.deepcopy(CONFIGS[name])


def tensor_shapes(cfg) -> Dict[str, tuple]:
    """Every tensor of a model of this design, by the naming rule of its checkpoints."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "head": (V, D), "final.norm": (D,)}
    if cfg.get("loop"):
        out["loop.in"] = (D, 2 * D)
        out["loop.step"] = (cfg["loop"]["times"], D)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (D,)
        H, G, dim, vdim, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv")
        if layer["type"] == "attention":
            rows = {"q": H * dim, "k": G * dim, "v": G * vdim}
            for n, r in rows.items():
                out[p + f"mix.{n}"], out[p + f"mix.{n}.b"] = (r, D), (r,)
                if taps:
                    out[p + f"mix.{n}.conv"] = (r, taps)
            out[p + "mix.o"], out[p + "mix.o.b"] = (D, H * vdim), (D,)
        else:
            rows = {"q": G * dim, "k": G * dim, "v": H * vdim}
            for n, r in rows.items():
                out[p + f"mix.{n}"], out[p + f"mix.{n}.conv"] = (r, D), (r, taps)
            ra, rg = m["decay_rank"], m["gate_rank"]
            out.update({p + "mix.b": (H, D), p + "mix.A_log": (H,), p + "mix.norm": (vdim,), p + "mix.a1": (ra, D),
                        p + "mix.a2": (H * dim, ra), p + "mix.dt_bias": (H * dim,), p + "mix.g1": (rg, D),
                        p + "mix.g2": (H * vdim, rg), p + "mix.o": (D, H * vdim)})
        mlp = layer.get("mlp")
        if mlp is not None:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            out[p + "norm2"] = (D,)
            out[p + "mlp.router"], out[p + "mlp.correction"] = (E, D), (E,)
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (ff, D), p + f"mlp.e{e}.up": (ff, D), p + f"mlp.e{e}.down": (D, ff)})
    return out


def random_weights(cfg, seed: int, store=torch.float32) -> Dict[str, torch.Tensor]:
    """Weights that keep activations of order one (matrices N(0, 1/in), convolutions near the identity).  q and k of
    the attention layers are normed head by head, so how sharp the attention is lies in the configuration's ``scale``.
    Rounded once to ``store``."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        tail = name.split(".")[-1]
        if tail in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif tail in ("b",) and len(shape) == 1:
            t = 0.1 * torch.randn(shape, generator=g)
        elif tail == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
            t[:, -1] += 1.0
        elif tail in ("A_log", "dt_bias"):
            t = 0.5 * torch.randn(shape, generator=g) - (1.0 if tail == "dt_bias" else 0.0)
        elif tail == "correction":
            t = 0.2 * torch.randn(shape, generator=g)
        elif tail == "step":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif tail == "router":
            t = 2.0 * torch.randn(shape, generator=g) / shape[1] ** 0.5
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        out[name] = t.to(store).contiguous()
    return out


def file_config(cfg):
    """The configuration as a checkpoint's config.json has it: the ranks of the low-rank pairs are left to the tensors."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    return cfg


def write_model(cfg, weights, out_dir: str) -> str:
    from lightllm_b200.weights import save_file
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(file_config(cfg), f)
    save_file(weights, os.path.join(out_dir, "model.safetensors"))
    return out_dir
