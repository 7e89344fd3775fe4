"""Typed configuration of the Kagorax decoder and its plan.

``config.json`` of this design is nested: ``architecture`` (the string ``Kagorax``), ``vocab``,
``width``, ``embedding.scale``, ``norm.eps`` and ``layers``, a list with one object per layer:
``type`` (the mixer's kind; ``attention`` is the one there is), ``mixer`` (its sizes) and ``mlp``
(the feed-forward, or null).  Nothing has a default: a missing size or constant is an error.

The layer the plan stands for: ``h = RMSNorm(x)``; ``x += mixer(h) + ffn(h)`` (one norm, both
sublayers read it).  The mixer is grouped-query attention without rotation, with biased
projections, unit-RMS queries and keys, a learned bias per (head, distance bucket), a window that
keeps the first tokens, and a sigmoid output gate (``parts/gated_attention.py``); a layer with
``kv_from: j`` reads layer ``j``'s keys and values.  The feed-forward is a sigmoid-routed
mixture of gated experts with an optional gated shared expert (``parts/moe.py``).  The
embedding is scaled and gets a sinusoidal position wave; the head is the embedding table.

Tensor names: ``embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.mix.{q,q.b,k,k.b,v,v.b,rel,g,o}``,
``l<i>.mlp.{router, e<n>.gate, e<n>.up, e<n>.down, shared.gate, shared.up, shared.down, shared.sg}``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from .registry import Architecture, ConfigError, register_architecture

MAX_POSITION = 1 << 17        # the design names no longest context; the engine's tables need a bound


def _get(cfg: Mapping[str, Any], path: str):
    node: Any = cfg
    for key in path.split("."):
        if not isinstance(node, Mapping) or key not in node or node[key] is None:
            raise ConfigError(f"config.json lacks '{path}'")
        node = node[key]
    return node


def _int(cfg, path: str, minimum: int = 1) -> int:
    v = _get(cfg, path)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"'{path}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"'{path}' must be >= {minimum}, got {v}")
    return v


def _positive(cfg, path: str) -> float:
    v = _get(cfg, path)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ConfigError(f"'{path}' must be a positive number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class KagoraxMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int
    window: int
    keep_first: int
    kv_from: Optional[int] = None
    bias_rows: Optional[int] = None      # rows of the distance table: the stored tensor's size; a
                                         # configuration names it only for random weights


@dataclass(frozen=True)
class KagoraxMlp:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int] = None


@dataclass(frozen=True)
class KagoraxLayer:
    mixer: KagoraxMixer
    mlp: Optional[KagoraxMlp]


@dataclass(frozen=True)
class KagoraxConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple[KagoraxLayer, ...]
    source: Mapping[str, Any]

    ARCHITECTURE = "Kagorax"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "KagoraxConfig":
        vocab, width = _int(cfg, "vocab"), _int(cfg, "width")
        raw = _get(cfg, "layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"'{where}' must be an object")
            if entry.get("type") != "attention":
                raise ConfigError(f"'{where}.type' is {entry.get('type')!r}; known: 'attention'")
            heads, kv_heads = _int(entry, "mixer.heads"), _int(entry, "mixer.kv_heads")
            if heads % kv_heads:
                raise ConfigError(f"'{where}': {heads} heads cannot share {kv_heads} kv heads evenly")
            kv_from = entry["mixer"].get("kv_from")
            if kv_from is not None:
                if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < i:
                    raise ConfigError(f"'{where}.mixer.kv_from' must name an earlier layer, got {kv_from!r}")
                src = layers[kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"'{where}.mixer.kv_from' names layer {kv_from}, which has no keys of its own")
            mixer = KagoraxMixer(
                heads=heads, kv_heads=kv_heads, dim=_int(entry, "mixer.dim"), vdim=_int(entry, "mixer.vdim"),
                scale=_positive(entry, "mixer.scale"), bias_max=_int(entry, "mixer.bias_max", 2),
                window=_int(entry, "mixer.mask.size"), keep_first=_int(entry, "mixer.mask.keep_first", 0),
                kv_from=kv_from,
                bias_rows=None if entry["mixer"].get("bias_rows") is None else _int(entry, "mixer.bias_rows", 2))
            if kv_from is not None:
                src = layers[kv_from].mixer
                if (src.kv_heads, src.dim, src.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                    raise ConfigError(f"'{where}' reads layer {kv_from}'s keys and values but its kv heads "
                                      f"or head sizes differ")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
                    raise ConfigError(f"'{where}.mlp.kind' is {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}; known: 'moe'")
                experts, top = _int(mlp, "router.experts"), _int(mlp, "router.top")
                if top > experts:
                    raise ConfigError(f"'{where}.mlp.router': top {top} of {experts} experts")
                shared = mlp.get("shared")
                mlp = KagoraxMlp(experts=experts, top=top, expert_ff=_int(mlp, "expert.ff"),
                                 shared_ff=None if shared is None else _int(mlp, "shared.ff"))
            layers.append(KagoraxLayer(mixer, mlp))
        return KagoraxConfig(vocab=vocab, width=width, embedding_scale=_positive(cfg, "embedding.scale"),
                             norm_eps=_positive(cfg, "norm.eps"), layers=tuple(layers), source=dict(cfg))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.source)


def build_plan(cfg: KagoraxConfig) -> ModelPlan:
    norm_eps = cfg.norm_eps
    # a cache slot keeps what its widest reader needs
    need: dict[int, list[int]] = {}
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        owner = i if m.kv_from is None else m.kv_from
        w, k = need.setdefault(owner, [0, 0])
        need[owner] = [max(w, m.window), max(k, m.keep_first)]
    slots = {owner: n for n, owner in enumerate(sorted(need))}
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        owner = i if m.kv_from is None else m.kv_from
        mixer = PartSpec("gated_bias_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
            "head_dim": m.dim, "v_head_dim": m.vdim, "scale": m.scale, "qk_norm_eps": norm_eps,
            "window": m.window, "keep_first": m.keep_first, "bias_rows": m.bias_rows, "bias_far": m.bias_max,
            "own_kv": m.kv_from is None, "cache_window": need[owner][0], "cache_keep_first": need[owner][1]})
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": cfg.width, "experts": layer.mlp.experts, "top": layer.mlp.top,
                "expert_size": layer.mlp.expert_ff, "shared_size": layer.mlp.shared_ff})
        p = f"l{i}."
        layers.append(LayerPlan(
            block=PartSpec("parallel"), mixer=mixer, ffn=ffn,
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.width, "eps": norm_eps, "tensor": "norm1"}),
            ffn_norm=None, names={"mixer": p + "mix.", "ffn": p + "mlp.", "mixer_norm": p}))
        schedule.append(ScheduleEntry(layer=i, cache_slot=slots[owner], writes_cache=m.kv_from is None))
    return ModelPlan(
        architecture=cfg.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab,
        max_position=MAX_POSITION, layers=layers, schedule=schedule,
        embedding=PartSpec("scaled_sinusoid", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                               "scale": cfg.embedding_scale, "tensor": "embed"}),
        final_norm=PartSpec("rmsnorm", {"size": cfg.width, "eps": norm_eps, "tensor": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": True}),
        names={"embedding": "", "final_norm": "", "head": "head."})


register_architecture(Architecture(
    name=KagoraxConfig.ARCHITECTURE, from_dict=KagoraxConfig.from_dict, build_plan=build_plan,
    aliases=("kagorax",)))
