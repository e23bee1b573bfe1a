"""``Bulitar``: a pre-norm decoder (``h += mixer(LN(h)); h += experts(LN(h))``, layer norms with a weight and no bias)
whose layers each pick one of two mixers (chunked grouped-query attention whose q, k, v pass a short causal
convolution, with YaRN-scaled rotary positions on adjacent pairs and unit-RMS q and k; the gated delta rule with a
decay per key channel), whose feed-forwards are routed experts with sigmoid scores, and in which a stretch of layers
may run several times in a row with the same weights: before every pass the stream is mixed again with the embedding
output (``h <- W_in [h; e] + step[pass]``), and every pass has cache and state of its own.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` (a list of
``{"type", "mixer": {...sizes and constants...}, "mlp": {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top",
"scale"}} | null}``) and ``loop`` ``{"start", "stop", "times"}``.  The ranks of the delta rule's two low-rank pairs are
not in config.json: they are the row counts of ``l<i>.mix.a1`` and ``l<i>.mix.g1`` in the checkpoint (a configuration
that is not read beside a checkpoint gives them as ``decay_rank`` / ``gate_rank`` in the mixer's object).  Tensors:
``embed``, ``head``, ``final.norm``, ``loop.in``, ``loop.step`` and per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.*``,
``l<i>.mlp.router|correction|e<j>.gate|up|down``; linear weights are ``[out, in]`` without a ``.weight`` ending.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..config import (ConfigError, ConfigReader, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, SubBlock,
                      architecture_name, register_architecture)

# Rotations are computed from the position itself; the engine only wants a bound for its buffers.
MAX_POSITIONS = 1 << 20
MIXER_TYPES = ("attention", "channel_delta")


def _object(raw: Any, key: str, where: str, required: bool = True) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {'required ' if required else ''}key '{key}' must be an object")
    return v


@dataclass(frozen=True)
class BulitarLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass(frozen=True)
class BulitarConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0
    layers: Tuple[BulitarLayer, ...] = field(default_factory=tuple)
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)

    @staticmethod
    def _rot(raw: Dict[str, Any], where: str, dim: int) -> Optional[Dict[str, Any]]:
        rot = _object(raw, "rot", where, required=False)
        if rot is None:
            return None
        rr = ConfigReader(rot, f"{where}.rot")
        dims = rr.integer("dims", minimum=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{where}.rot: 'dims' {dims} must be even and at most 'dim' {dim}")
        out: Dict[str, Any] = {"dims": dims, "base": rr.real("base"), "scaling": None}
        sc = _object(rot, "scaling", f"{where}.rot", required=False)
        if sc is not None:
            sr = ConfigReader(sc, f"{where}.rot.scaling")
            out["scaling"] = {"factor": sr.real("factor"), "original": sr.real("original"), "fast": sr.real("fast"),
                              "slow": sr.real("slow")}
        return out

    @staticmethod
    def _mixer(kind: str, raw: Any, where: str, index: int, shapes: Optional[Dict[str, tuple]]) -> Dict[str, Any]:
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: 'mixer' must be an object")
        r = ConfigReader(raw, where)
        out: Dict[str, Any] = {"heads": r.integer("heads"), "kv_heads": r.integer("kv_heads"), "dim": r.integer("dim"),
                               "vdim": r.integer("vdim"), "conv": r.integer("conv", None)}          # no 'conv': no convolution
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"{where}: 'heads' {out['heads']} is not a multiple of 'kv_heads' {out['kv_heads']}")
        if kind == "attention":
            out.update(scale=r.real("scale"), rot=BulitarConfig._rot(raw, where, out["dim"]), chunk=None)
            mask = _object(raw, "mask", where, required=False)
            if mask is not None:
                out["chunk"] = ConfigReader(mask, f"{where}.mask").integer("size")
        else:
            for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
                name = f"l{index}.mix.{tensor}"
                if raw.get(key) is not None:
                    out[key] = r.integer(key)
                elif shapes is not None and name in shapes and len(shapes[name]) == 2:
                    out[key] = int(shapes[name][0])
                else:
                    raise ConfigError(f"{where}: the rank '{key}' is neither in the configuration nor given by the "
                                      f"shape of a tensor '{name}' in a checkpoint beside it")
        return out

    @staticmethod
    def _mlp(raw: Any, where: str) -> Optional[Dict[str, Any]]:
        if raw is None:
            return None
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        kind = ConfigReader(raw, where).string("kind")
        if kind != "moe":
            raise ConfigError(f"{where}: 'kind' must be 'moe', got {kind!r}")
        expert = ConfigReader(_object(raw, "expert", where), f"{where}.expert")
        router = ConfigReader(_object(raw, "router", where), f"{where}.router")
        out = {"ff": expert.integer("ff"), "experts": router.integer("experts"), "top": router.integer("top"),
               "scale": router.real("scale")}
        if out["top"] > out["experts"]:
            raise ConfigError(f"{where}.router: 'top' {out['top']} exceeds 'experts' {out['experts']}")
        return out

    @staticmethod
    def from_dict(raw: Dict[str, Any], where: str = "config.json",
                  tensor_shapes: Optional[Dict[str, tuple]] = None) -> "BulitarConfig":
        r = ConfigReader(raw, where)
        arch = architecture_name(raw, where)
        norm = ConfigReader(_object(raw, "norm", where), f"{where}: norm")
        emb = _object(raw, "embedding", where, required=False)
        scale = ConfigReader(emb, f"{where}: embedding").real("scale", 1.0) if emb is not None else 1.0
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: required key 'layers' must be a non-empty list")
        layers: List[BulitarLayer] = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            if not isinstance(lr, dict):
                raise ConfigError(f"{w} must be an object")
            kind = ConfigReader(lr, w).string("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{w}: unknown 'type' {kind!r}; known: {list(MIXER_TYPES)}")
            layers.append(BulitarLayer(kind, BulitarConfig._mixer(kind, lr.get("mixer"), f"{w}.mixer", i, tensor_shapes),
                                       BulitarConfig._mlp(lr.get("mlp"), f"{w}.mlp")))
        loop = None
        lp = _object(raw, "loop", where, required=False)
        if lp is not None:
            lr_ = ConfigReader(lp, f"{where}: loop")
            start, stop, times = lr_.integer("start", minimum=0), lr_.integer("stop"), lr_.integer("times")
            if not 0 <= start <= stop <= len(layers):
                raise ConfigError(f"{where}: loop: layers {start} .. {stop} - 1 are not a stretch of the {len(layers)} layers")
            loop = (start, stop, times) if stop > start else None          # an empty stretch: nothing is run again
        # the ranks read from tensor shapes are written back, so that the configuration stands on its own
        raw_out = dict(raw)
        if tensor_shapes is not None:
            raw_out["layers"] = [dict(lr, mixer=dict(lr["mixer"], **{k: l.mixer[k] for k in ("decay_rank", "gate_rank")
                                                                   if k in l.mixer}))
                                 for lr, l in zip(layers_raw, layers)]
        return BulitarConfig(architecture=arch, raw=raw_out, vocab=r.integer("vocab"), width=r.integer("width"),
                             norm_eps=norm.real("eps"), embedding_scale=scale, layers=tuple(layers), loop=loop)


def bulitar_spec(cfg: BulitarConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    plain = {"weight_suffix": ""}

    def layer_norm(prefix: str) -> PartSpec:
        return PartSpec("layernorm", {"hidden_size": D, "eps": eps, "weight_name": "", "bias_name": None}, prefix)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        if layer.type == "attention":
            rot = m["rot"]
            position = None
            if rot and rot["dims"]:
                position = PartSpec("rotary", {"head_dim": m["dim"], "theta": rot["base"], "rotary_dim": rot["dims"],
                                               "style": "interleaved", "scaling": rot["scaling"]})
            mixer = PartSpec("conv_attention", {
                "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "position": position, "conv_taps": m["conv"] or 0, "qkv_bias": True, "out_bias": True,
                "chunk": m["chunk"], "scale": m["scale"], "qk_unit_rms": True, "qk_norm_eps": eps,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "bias_ending": "b", "conv_ending": "conv", **plain},
                f"{p}.mix")
        else:
            mixer = PartSpec("channel_delta", {
                "hidden_size": D, "num_heads": m["heads"], "num_qk_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "conv_taps": m["conv"] or 0, "decay_rank": m["decay_rank"], "gate_rank": m["gate_rank"],
                "norm_eps": eps, "conv_ending": "conv",
                "names": {"q": "q", "k": "k", "v": "v", "b": "b", "a1": "a1", "a2": "a2", "g1": "g1", "g2": "g2", "o": "o",
                          "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm"}, **plain}, f"{p}.mix")
        subs = [SubBlock("mixer", mixer, norm_before=layer_norm(f"{p}.norm1"))]
        if layer.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": D, "intermediate_size": layer.mlp["ff"], "num_experts": layer.mlp["experts"],
                "top": layer.mlp["top"], "route_scale": layer.mlp["scale"], "score": "sigmoid", "renormalize": False,
                "correction": True, "activation": "silu", "expert_prefix": "e",
                "names": {"gate": "gate", "up": "up", "down": "down", "router": "router", "correction": "correction"},
                **plain}, f"{p}.mlp")
            subs.append(SubBlock("ffn", ffn, norm_before=layer_norm(f"{p}.norm2")))
        layers.append(LayerSpec(sub_blocks=subs, arrangement="sequential"))

    n = len(layers)
    if cfg.loop is None:
        run = [RunEntry(i) for i in range(n)]
    else:
        start, stop, times = cfg.loop
        run = [RunEntry(i) for i in range(start)]
        for t in range(times):
            enter = PartSpec("reinjection", {"hidden_size": D, "weight_name": "loop.in", "step_name": "loop.step",
                                             "steps": times, "index": t}, "")
            run += [RunEntry(i, enter=enter if i == start else None) for i in range(start, stop)]
        run += [RunEntry(i) for i in range(stop, n)]
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "embed",
                                               "scale": cfg.embedding_scale, "keep_output": cfg.loop is not None}, ""),
        layers=layers, run=run, final_norm=layer_norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "head"}, ""),
        # a model without a loop (or with an empty one) may still carry the loop's tensors
        ignored_suffixes=("loop.in", "loop.step") if cfg.loop is None else ())


register_architecture("Bulitar", BulitarConfig.from_dict, bulitar_spec, reads_shapes=True)
