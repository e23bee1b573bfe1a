"""``Kudadra``: a decoder whose layers each pick one of three mixers (attention over a shared low-rank latent with
learned sinks, windowed grouped-query attention with whole-projection q/k norms, retention with a per-request state),
with the norms on the branches' OUTPUTS: ``h += LN(mixer(h)); h += LN(ff(h))``.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list of
``{"type", "mixer": {...sizes and constants...}, "mlp": {"kind": "dense", "ff", "limit"} | null}``.  Tensors:
``embed``, ``head``, ``final.norm`` (+ ``.b``), and per layer i ``l<i>.norm1|norm2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``;
linear weights are ``[out, in]`` without a ``.weight`` ending.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..config import (ConfigError, ConfigReader, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, SubBlock,
                      architecture_name, register_architecture)

# The design has no table of positions: rotations are computed from the position itself.  The engine still wants a
# bound for its buffers; float32 angles stay exact integers times a frequency far beyond it.
MAX_POSITIONS = 1 << 20
# Constants that the design fixes (not read from config.json).
SWISH_ALPHA = 1.702
UP_SHIFT = 1.0
MIXER_TYPES = ("latent_attention", "attention", "retention")


@dataclass(frozen=True)
class KudadraLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass(frozen=True)
class KudadraConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    layers: Tuple[KudadraLayer, ...] = field(default_factory=tuple)

    @staticmethod
    def _rot(r: ConfigReader, where: str, dim: int) -> Optional[Dict[str, Any]]:
        raw = r.raw.get("rot")
        if raw is None:
            return None
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: 'rot' must be an object")
        rr = ConfigReader(raw, f"{where}.rot")
        dims = rr.integer("dims", minimum=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{where}.rot: 'dims' {dims} must be even and at most 'dim' {dim}")
        return {"dims": dims, "base": rr.real("base")}

    @staticmethod
    def _mixer(kind: str, raw: Any, where: str) -> Dict[str, Any]:
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: 'mixer' must be an object")
        r = ConfigReader(raw, where)
        out: Dict[str, Any] = {"heads": r.integer("heads"), "dim": r.integer("dim"), "vdim": r.integer("vdim")}
        if kind == "latent_attention":
            out.update(kv_rank=r.integer("kv_rank"), scale=r.real("scale"))
        elif kind == "attention":
            out.update(kv_heads=r.integer("kv_heads"), scale=r.real("scale"), rot=KudadraConfig._rot(r, where, out["dim"]))
            if out["heads"] % out["kv_heads"]:
                raise ConfigError(f"{where}: 'heads' {out['heads']} is not a multiple of 'kv_heads' {out['kv_heads']}")
            mask = raw.get("mask")
            if mask is not None:
                if not isinstance(mask, dict):
                    raise ConfigError(f"{where}: 'mask' must be an object")
                out["window"] = ConfigReader(mask, f"{where}.mask").integer("size")
            else:
                out["window"] = None
        else:
            decay = raw.get("decay")
            if not isinstance(decay, list) or len(decay) != out["heads"] or \
                    not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                raise ConfigError(f"{where}: 'decay' must list one number for each of the {out['heads']} heads")
            out.update(decay=[float(d) for d in decay], rot=KudadraConfig._rot(r, where, out["dim"]))
        return out

    @staticmethod
    def from_dict(raw: Dict[str, Any], where: str = "config.json") -> "KudadraConfig":
        r = ConfigReader(raw, where)
        arch = architecture_name(raw, where)
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError(f"{where}: required key 'norm' must be an object with 'eps'")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: required key 'layers' must be a non-empty list")
        layers: List[KudadraLayer] = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            if not isinstance(lr, dict):
                raise ConfigError(f"{w} must be an object")
            kind = ConfigReader(lr, w).string("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{w}: unknown 'type' {kind!r}; known: {list(MIXER_TYPES)}")
            mlp = lr.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{w}: 'mlp' must be an object or null")
                mr = ConfigReader(mlp, f"{w}.mlp")
                if mr.string("kind") != "dense":
                    raise ConfigError(f"{w}.mlp: 'kind' must be 'dense', got {mlp.get('kind')!r}")
                mlp = {"ff": mr.integer("ff"), "limit": mr.real("limit")}
            layers.append(KudadraLayer(kind, KudadraConfig._mixer(kind, lr.get("mixer"), f"{w}.mixer"), mlp))
        return KudadraConfig(architecture=arch, raw=dict(raw), vocab=r.integer("vocab"), width=r.integer("width"),
                             norm_eps=ConfigReader(norm, f"{where}: norm").real("eps"), layers=tuple(layers))


def _rotary(rot: Optional[Dict[str, Any]], dim: int) -> Optional[PartSpec]:
    if not rot or rot["dims"] == 0:
        return None
    return PartSpec("rotary", {"head_dim": dim, "theta": rot["base"], "rotary_dim": rot["dims"], "style": "neox"})


def kudadra_spec(cfg: KudadraConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    plain_names = {"weight_suffix": ""}

    def layer_norm(prefix: str) -> PartSpec:
        return PartSpec("layernorm", {"hidden_size": D, "eps": eps, "weight_name": "", "bias_name": "b"}, prefix)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        if layer.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "num_heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
                "rank": m["kv_rank"], "norm_eps": eps, "scale": m["scale"], "sinks": True, "gate": "per_head",
                "gate_act": "sigmoid",
                "names": {"q": "q", "dkv": "dkv", "uk": "uk", "uv": "uv", "o": "o", "g": "g", "sink": "sink"},
                **plain_names}, f"{p}.mix")
        elif layer.type == "attention":
            mixer = PartSpec("gated_attention", {
                "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "position": _rotary(m["rot"], m["dim"]), "window": m["window"],
                "scale": m["scale"], "qk_norm": True, "qk_norm_eps": eps, "gate": "elementwise", "gate_act": "sigmoid",
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}, **plain_names}, f"{p}.mix")
        else:
            mixer = PartSpec("retention", {
                "hidden_size": D, "num_heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
                "decay": m["decay"], "position": _rotary(m["rot"], m["dim"]), "k_scale": m["dim"] ** -0.5,
                "norm_eps": eps, "gate_act": "silu",
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}, **plain_names}, f"{p}.mix")
        subs = [SubBlock("mixer", mixer, norm_after=layer_norm(f"{p}.norm1"), after="branch")]
        if layer.mlp is not None:
            ffn = PartSpec("gated_mlp", {
                "hidden_size": D, "intermediate_size": layer.mlp["ff"], "activation": "clamped_swish",
                "alpha": SWISH_ALPHA, "limit": layer.mlp["limit"], "up_shift": UP_SHIFT,
                "names": {"gate": "gate", "up": "up", "down": "down"}, **plain_names}, f"{p}.mlp")
            subs.append(SubBlock("ffn", ffn, norm_after=layer_norm(f"{p}.norm2"), after="branch"))
        layers.append(LayerSpec(sub_blocks=subs, arrangement="sequential"))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "embed"}, ""),
        layers=layers, run=[RunEntry(i) for i in range(len(layers))],
        final_norm=layer_norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "head"}, ""))


register_architecture("Kudadra", KudadraConfig.from_dict, kudadra_spec)
