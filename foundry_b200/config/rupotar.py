"""Typed configuration of the Rupotar decoder, read from config.json.

A Rupotar model is a list of layers, each with one of three mixers
(`attention`, `wkv`, `channel_delta`) and a dense or routed feed-forward (or
none), an embedding with a constant scale and sinusoidal positions, layer
norms on both sides of every part, and optionally a group of layers that runs
several times with the same weights (`loop`). Keys:

    architecture: "Rupotar", vocab, width, embedding.scale, norm.eps,
    layers[i]: {type, mixer: {...sizes...}, mlp: null | {kind: "dense", ff} |
                {kind: "moe", expert: {ff, limit}, router: {experts, top}}},
    loop: null | {start, stop, times}

Two sizes are not in config.json but in the tensors' shapes: the ranks of the
low-rank projections inside the recurrent mixers. `complete_from_files` reads
them there; a configuration written by this library (`to_json`) carries them
as `decay_rank` / `gate_rank` in the mixer's entry.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Dict, Mapping, Optional, Tuple

from . import errors
from .fields import need as _need, positive as _positive
from .files import decode_json

ARCHITECTURE = "Rupotar"
MIXER_TYPES = ("attention", "wkv", "channel_delta")
# No key bounds the positions (the position vector is computed, not stored);
# 2^24 keeps every position exactly representable in 32-bit floats.
MAX_POSITIONS = 1 << 24


@dataclass(frozen=True)
class RupotarMlp:
    kind: str  # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0
    limit: float = 0.0

    def to_json(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class RupotarLayer:
    type: str
    heads: int
    dim: int
    kv_heads: int = 0      # attention, channel_delta
    vdim: int = 0          # attention, channel_delta
    scale: float = 0.0     # attention
    window: Optional[int] = None   # attention: mask.size
    keep_first: int = 0            # attention: mask.keep_first
    taps: int = 0          # channel_delta: conv
    decay_rank: Optional[int] = None  # wkv, channel_delta (from the tensors' shapes)
    gate_rank: Optional[int] = None   # channel_delta (from the tensors' shapes)
    mlp: Optional[RupotarMlp] = None

    def to_json(self) -> dict:
        m: Dict[str, Any] = {"heads": self.heads, "dim": self.dim}
        if self.type in ("attention", "channel_delta"):
            m.update(kv_heads=self.kv_heads, vdim=self.vdim)
        if self.type == "attention":
            m["scale"] = self.scale
            if self.window is not None:
                m["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.type == "channel_delta":
            m["conv"] = self.taps
        if self.decay_rank is not None:
            m["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            m["gate_rank"] = self.gate_rank
        return {"type": self.type, "mixer": m, "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class RupotarConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[RupotarLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:  # the name other parts of the library ask for
        return self.vocab

    @classmethod
    def parse(cls, source) -> "RupotarConfig":
        doc = decode_json(source)
        if doc.get("architecture") != ARCHITECTURE:
            raise errors.ModelType(f"architecture is {doc.get('architecture')!r}, "
                                   f"expected {ARCHITECTURE!r}")
        width = _positive(doc, "width", "config")
        if width % 2:
            raise errors.ConfigJson(f"width {width} must be even (sin/cos position pairs)")
        layers_doc = _need(doc, "layers", list, "config")
        if not layers_doc:
            raise errors.ConfigJson("config: no layers")
        layers = tuple(_parse_layer(entry, f"layers[{i}]") for i, entry in enumerate(layers_doc))
        loop = None
        if doc.get("loop") is not None:
            ld = _need(doc, "loop", dict, "config")
            start, stop = _need(ld, "start", int, "loop"), _need(ld, "stop", int, "loop")
            times = _positive(ld, "times", "loop")
            if not 0 <= start < stop <= len(layers):
                raise errors.ConfigJson(f"loop: layers {start}..{stop - 1} of {len(layers)}")
            loop = (start, stop, times)
        known = {"architecture", "vocab", "width", "embedding", "norm", "layers", "loop"}
        return cls(
            vocab=_positive(doc, "vocab", "config"), width=width,
            embedding_scale=_need(_need(doc, "embedding", dict, "config"), "scale", float,
                                  "embedding"),
            norm_eps=_need(_need(doc, "norm", dict, "config"), "eps", float, "norm"),
            layers=layers, loop=loop, extra={k: v for k, v in doc.items() if k not in known})

    def to_json(self) -> dict:
        doc = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_json() for layer in self.layers]}
        if self.loop is not None:
            doc["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return doc

    def with_default_ranks(self, rank: int = 16) -> "RupotarConfig":
        """Ranks that no file gives (a model made from this configuration alone)."""
        return replace(self, layers=tuple(
            replace(layer,
                    decay_rank=layer.decay_rank if layer.decay_rank is not None or
                    layer.type == "attention" else rank,
                    gate_rank=layer.gate_rank if layer.gate_rank is not None or
                    layer.type != "channel_delta" else rank)
            for layer in self.layers))


def _parse_layer(entry, where: str) -> RupotarLayer:
    if not isinstance(entry, dict):
        raise errors.ConfigJson(f"{where} is not an object")
    kind = _need(entry, "type", str, where)
    if kind not in MIXER_TYPES:
        raise errors.UnsupportedOption(f"{where}: mixer type {kind!r}; known: {MIXER_TYPES}")
    m = _need(entry, "mixer", dict, where)
    w = f"{where}.mixer"
    fields: Dict[str, Any] = dict(type=kind, heads=_positive(m, "heads", w), dim=_positive(m, "dim", w))
    if kind in ("attention", "channel_delta"):
        fields.update(kv_heads=_positive(m, "kv_heads", w), vdim=_positive(m, "vdim", w))
        if fields["heads"] % fields["kv_heads"]:
            raise errors.HeadRatio(f"{w}: {fields['heads']} heads over {fields['kv_heads']} kv heads")
    if kind == "attention":
        fields["scale"] = _need(m, "scale", float, w)
        mask = m.get("mask")
        if mask is not None:
            if not isinstance(mask, dict):
                raise errors.ConfigJson(f"{w}.mask is not an object")
            if mask.get("size") is not None:
                fields["window"] = _positive(mask, "size", f"{w}.mask")
                keep = mask.get("keep_first") or 0
                if not isinstance(keep, int) or keep < 0:
                    raise errors.ConfigJson(f"{w}.mask.keep_first = {keep!r}")
                fields["keep_first"] = keep
    if kind == "channel_delta":
        fields["taps"] = _positive(m, "conv", w)
    for key in ("decay_rank", "gate_rank"):
        if m.get(key) is not None:
            fields[key] = _positive(m, key, w)
    mlp = entry.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict):
            raise errors.ConfigJson(f"{where}.mlp is not an object")
        mk = _need(mlp, "kind", str, f"{where}.mlp")
        if mk == "dense":
            fields["mlp"] = RupotarMlp("dense", _positive(mlp, "ff", f"{where}.mlp"))
        elif mk == "moe":
            ex = _need(mlp, "expert", dict, f"{where}.mlp")
            ro = _need(mlp, "router", dict, f"{where}.mlp")
            experts, top = _positive(ro, "experts", "router"), _positive(ro, "top", "router")
            if top > experts:
                raise errors.ConfigJson(f"{where}.mlp: {top} of {experts} experts")
            fields["mlp"] = RupotarMlp("moe", _positive(ex, "ff", "expert"), experts, top,
                                       _need(ex, "limit", float, "expert"))
        else:
            raise errors.UnsupportedOption(f"{where}.mlp.kind {mk!r}; known: dense, moe")
    return RupotarLayer(**fields)


def complete_from_files(config: RupotarConfig, files) -> RupotarConfig:
    """Fill the sizes that only the tensors' shapes give (`files`: anything with
    `in` and `entry(name).shape`, i.e. the opened weight files)."""
    layers = []
    for i, layer in enumerate(config.layers):
        def rows(name, current):
            full = f"l{i}.mix.{name}"
            return int(files.entry(full).shape[0]) if full in files else current
        if layer.type == "wkv":
            layer = replace(layer, decay_rank=rows("w1", layer.decay_rank))
        elif layer.type == "channel_delta":
            layer = replace(layer, decay_rank=rows("a1", layer.decay_rank),
                            gate_rank=rows("g1", layer.gate_rank))
        layers.append(layer)
    return replace(config, layers=tuple(layers))
