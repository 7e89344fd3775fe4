"""Typed configuration of the Ruvuvik decoder and its plan.

``config.json`` of this design is nested: ``architecture`` (the string ``Ruvuvik``), ``vocab``,
``width``, ``norm.eps`` and ``layers``, a list with one object per layer: ``type`` (the mixer's
kind), ``mixer`` (its sizes and constants), ``mlp`` (``{"kind": "dense", "ff": n}`` or null) and
optionally ``weights_of: j``: the layer then has no tensors of its own and runs with layer j's
(mixer, feed-forward and norms) on a cache or state of its own.  Nothing has a default.

The layer: ``x += mixer(norm1(x))``, then ``x += ff(norm2(x))`` where there is a feed-forward; the
norms are RMS norms whose weights are stored minus one.  The embedding's rows pass through such a
norm too (``embed.norm``), the head has a table of its own behind ``final.norm``.  Mixers:

``attention``         grouped-query attention inside chunks of ``mask.size`` positions, norm over the
                      whole query and key rows, neighbouring-pair rotation of the first ``rot.dims``
                      elements of every head, a score factor per head, ``softcap``, a sigmoid gate per
                      head (``parts/chunked_attention.py``)
``latent_attention``  keys and values made from one cached latent row per token, one shared rotated
                      key part, a sink in the softmax (``parts/latent_attention.py``)
``wkv``               a recurrent mixer with a decaying matrix state per head (``parts/wkv.py``)

The feed-forward is ``Wdown xIELU(Wup h)`` (``parts/mlp.py``).

Tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``head``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*`` (attention: ``q k v g o q.norm k.norm temp``; latent attention: ``q dkv dkv.norm uk uv
sink o``; wkv: ``mu.{r,k,v,g,w} r k v g w1 w2 w0 u norm o``), ``l<i>.mlp.{up,down,act}``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .kagorax import MAX_POSITION, _get, _int, _positive
from .plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from .registry import Architecture, ConfigError, register_architecture

MIXER_TYPES = ("attention", "latent_attention", "wkv")


@dataclass(frozen=True)
class RuvuvikLayer:
    type: str
    mixer: Mapping[str, Any]           # the validated sizes and constants of the mixer, flat
    ff: Optional[int]                  # None: no feed-forward
    weights_of: Optional[int]          # the layer whose tensors this one uses (None: its own)


def _rotation(entry, where: str, head_dim: int) -> tuple[int, float]:
    dims, base = _int(entry, "mixer.rot.dims", 0), _positive(entry, "mixer.rot.base")
    if dims % 2 or dims > head_dim:
        raise ConfigError(f"'{where}.mixer.rot.dims' must be even and at most {head_dim}, got {dims}")
    return dims, base


def _mixer(entry, where: str, kind: str) -> dict:
    heads, dim = _int(entry, "mixer.heads"), _int(entry, "mixer.dim")
    if kind == "attention":
        kv_heads = _int(entry, "mixer.kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"'{where}': {heads} heads cannot share {kv_heads} kv heads evenly")
        dims, base = _rotation(entry, where, dim)
        # a constant that the configuration does not name does not exist: no cap, no chunks
        m = entry["mixer"]
        return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": _int(entry, "mixer.vdim"),
                "scale": _positive(entry, "mixer.scale"),
                "softcap": None if m.get("softcap") is None else _positive(entry, "mixer.softcap"),
                "chunk": None if m.get("mask") is None else _int(entry, "mixer.mask.size"),
                "rot_dims": dims, "rot_base": base}
    if kind == "latent_attention":
        rot_dim = _int(entry, "mixer.rot_dim", 0)
        dims, base = _rotation(entry, where, rot_dim)
        if dims != rot_dim:
            raise ConfigError(f"'{where}.mixer.rot.dims' is {dims}, the rotated part has {rot_dim} elements")
        return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": _int(entry, "mixer.vdim"),
                "kv_rank": _int(entry, "mixer.kv_rank"), "scale": _positive(entry, "mixer.scale"),
                "rot_base": base}
    out = {"heads": heads, "dim": dim}
    if entry["mixer"].get("decay_rank") is not None:       # only random weights need it
        out["decay_rank"] = _int(entry, "mixer.decay_rank")
    return out


@dataclass(frozen=True)
class RuvuvikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[RuvuvikLayer, ...]
    source: Mapping[str, Any]

    ARCHITECTURE = "Ruvuvik"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "RuvuvikConfig":
        vocab, width = _int(cfg, "vocab"), _int(cfg, "width")
        raw = _get(cfg, "layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"'{where}' must be an object")
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"'{where}.type' is {kind!r}; known: {', '.join(MIXER_TYPES)}")
            mlp = entry.get("mlp")
            if mlp is not None and (not isinstance(mlp, Mapping) or mlp.get("kind") != "dense"):
                raise ConfigError(f"'{where}.mlp.kind' is {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}; "
                                  f"known: 'dense'")
            owner = entry.get("weights_of")
            if owner is not None and (isinstance(owner, bool) or not isinstance(owner, int)
                                      or not 0 <= owner < len(raw) or owner == i):
                raise ConfigError(f"'{where}.weights_of' must name another layer, got {owner!r}")
            layers.append(RuvuvikLayer(kind, _mixer(entry, where, kind),
                                       None if mlp is None else _int(mlp, "ff"), owner))
        for i, layer in enumerate(layers):
            if layer.weights_of is None:
                continue
            src = layers[layer.weights_of]
            if src.weights_of is not None:
                raise ConfigError(f"'layers[{i}].weights_of' names layer {layer.weights_of}, which has no "
                                  f"tensors of its own")
            if (src.type, dict(src.mixer), src.ff) != (layer.type, dict(layer.mixer), layer.ff):
                raise ConfigError(f"'layers[{i}]' uses layer {layer.weights_of}'s tensors but its type, sizes "
                                  f"or constants differ")
        return RuvuvikConfig(vocab=vocab, width=width, norm_eps=_positive(cfg, "norm.eps"),
                             layers=tuple(layers), source=dict(cfg))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.source)


def _mixer_spec(cfg: RuvuvikConfig, layer: RuvuvikLayer) -> PartSpec:
    m = layer.mixer
    if layer.type == "attention":
        return PartSpec("chunked_attention", {
            "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
            "head_dim": m["dim"], "v_head_dim": m["vdim"], "scale": m["scale"], "qk_norm_eps": cfg.norm_eps,
            "chunk": m["chunk"], "softcap": m["softcap"],
            "position": PartSpec("rope_interleaved", {"head_dim": m["dim"], "theta": m["rot_base"],
                                                      "rotary_dim": m["rot_dims"]})
            if m["rot_dims"] else PartSpec("none", {"head_dim": m["dim"]})})
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
            "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": m["scale"], "norm_eps": cfg.norm_eps,
            "position": PartSpec("rope_interleaved", {"head_dim": m["rot_dim"], "theta": m["rot_base"]})
            if m["rot_dim"] else PartSpec("none", {"head_dim": 0})})
    return PartSpec("wkv", {"hidden_size": cfg.width, "num_heads": m["heads"], "head_dim": m["dim"],
                            "norm_eps": cfg.norm_eps, "decay_rank": m.get("decay_rank")})


def build_plan(cfg: RuvuvikConfig) -> ModelPlan:
    def norm(tensor: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "tensor": tensor, "one_plus": True})

    # the plan's layers are the layers that own tensors; the schedule runs one entry per layer of
    # the configuration, each with a cache slot of its own
    index_of: dict[int, int] = {}
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        index_of[i] = len(layers)
        p = f"l{i}."
        layers.append(LayerPlan(
            block=PartSpec("prenorm"), mixer=_mixer_spec(cfg, layer),
            ffn=None if layer.ff is None else PartSpec("xielu_mlp", {"hidden_size": cfg.width,
                                                                      "intermediate_size": layer.ff}),
            mixer_norm=norm("norm1"), ffn_norm=None if layer.ff is None else norm("norm2"),
            names={"mixer": p + "mix.", "ffn": p + "mlp.", "mixer_norm": p, "ffn_norm": p}))
    schedule = [ScheduleEntry(layer=index_of[i if layer.weights_of is None else layer.weights_of], cache_slot=i)
                for i, layer in enumerate(cfg.layers)]
    return ModelPlan(
        architecture=cfg.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab,
        max_position=MAX_POSITION, layers=layers, schedule=schedule,
        embedding=PartSpec("normed", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "eps": cfg.norm_eps,
                                      "tensor": "embed", "norm_tensor": "embed.norm", "one_plus": True}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False,
                                  "tensor": "head"}),
        names={"embedding": "", "final_norm": "", "head": ""})


register_architecture(Architecture(
    name=RuvuvikConfig.ARCHITECTURE, from_dict=RuvuvikConfig.from_dict, build_plan=build_plan,
    aliases=("ruvuvik",)))
