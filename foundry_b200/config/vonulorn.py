"""Typed configuration of the Vonulorn decoder, read from config.json.

A Vonulorn model is a list of layers, each with one of three mixers (`delta`:
the gated delta rule with a decay per head; `attention`: differential
attention with a query temperature and a score cap; `latent_attention`:
attention through a cached low-rank latent with a rotated key part and a
learned sink) and a dense gated feed-forward or none, RMS norms in front of
every part, and one constant on every part's output. Keys:

    architecture: "Vonulorn", vocab, width, norm.eps, residual_mult,
    layers[i]: {type, mixer: {...sizes and constants...}, mlp: null | {kind: "dense", ff}}
    delta:            heads, kv_heads, dim, vdim, conv
    attention:        heads, kv_heads, dim, vdim, scale, softcap, diff, q_temp: {coef, every}
    latent_attention: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from . import errors
from .fields import need as _need, positive as _positive
from .files import decode_json

ARCHITECTURE = "Vonulorn"
MIXER_TYPES = ("delta", "attention", "latent_attention")
# No key bounds the positions; 2^24 keeps every position exact in 32-bit floats.
MAX_POSITIONS = 1 << 24


@dataclass(frozen=True)
class VonulornLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0        # delta, attention
    taps: int = 0            # delta: conv
    scale: float = 0.0       # attention, latent_attention
    softcap: float = 0.0     # attention
    diff: float = 0.0        # attention
    temp_coef: float = 0.0   # attention: q_temp.coef
    temp_every: int = 0      # attention: q_temp.every
    rot_dim: int = 0         # latent_attention
    kv_rank: int = 0
    q_rank: int = 0
    rot_base: float = 0.0    # latent_attention: rot.base
    rot_dims: int = 0        # latent_attention: rot.dims
    ff: Optional[int] = None  # the dense feed-forward's inner width; None: no feed-forward

    def to_json(self) -> dict:
        m: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == "delta":
            m.update(kv_heads=self.kv_heads, conv=self.taps)
        elif self.type == "attention":
            m.update(kv_heads=self.kv_heads, scale=self.scale, softcap=self.softcap,
                     diff=self.diff, q_temp={"coef": self.temp_coef, "every": self.temp_every})
        else:
            m.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank, q_rank=self.q_rank,
                     scale=self.scale, rot={"base": self.rot_base, "dims": self.rot_dims})
        return {"type": self.type, "mixer": m,
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class VonulornConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[VonulornLayer, ...]
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:  # the name other parts of the library ask for
        return self.vocab

    @classmethod
    def parse(cls, source) -> "VonulornConfig":
        doc = decode_json(source)
        if doc.get("architecture") != ARCHITECTURE:
            raise errors.ModelType(f"architecture is {doc.get('architecture')!r}, "
                                   f"expected {ARCHITECTURE!r}")
        layers_doc = _need(doc, "layers", list, "config")
        if not layers_doc:
            raise errors.ConfigJson("config: no layers")
        known = {"architecture", "vocab", "width", "norm", "residual_mult", "layers"}
        return cls(
            vocab=_positive(doc, "vocab", "config"), width=_positive(doc, "width", "config"),
            norm_eps=_need(_need(doc, "norm", dict, "config"), "eps", float, "norm"),
            residual_mult=_need(doc, "residual_mult", float, "config"),
            layers=tuple(_parse_layer(e, f"layers[{i}]") for i, e in enumerate(layers_doc)),
            extra={k: v for k, v in doc.items() if k not in known})

    def to_json(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "layers": [layer.to_json() for layer in self.layers]}


def _parse_layer(entry, where: str) -> VonulornLayer:
    if not isinstance(entry, dict):
        raise errors.ConfigJson(f"{where} is not an object")
    kind = _need(entry, "type", str, where)
    if kind not in MIXER_TYPES:
        raise errors.UnsupportedOption(f"{where}: mixer type {kind!r}; known: {MIXER_TYPES}")
    m = _need(entry, "mixer", dict, where)
    w = f"{where}.mixer"
    fields: Dict[str, Any] = dict(type=kind, heads=_positive(m, "heads", w),
                                  dim=_positive(m, "dim", w), vdim=_positive(m, "vdim", w))
    if kind in ("delta", "attention"):
        fields["kv_heads"] = _positive(m, "kv_heads", w)
        if fields["heads"] % fields["kv_heads"]:
            raise errors.HeadRatio(f"{w}: {fields['heads']} heads over {fields['kv_heads']} kv heads")
    if kind == "delta":
        fields["taps"] = _positive(m, "conv", w)
    elif kind == "attention":
        temp = _need(m, "q_temp", dict, w)
        fields.update(scale=_need(m, "scale", float, w), softcap=_need(m, "softcap", float, w),
                      diff=_need(m, "diff", float, w),
                      temp_coef=_need(temp, "coef", float, f"{w}.q_temp"),
                      temp_every=_positive(temp, "every", f"{w}.q_temp"))
        if fields["softcap"] <= 0.0:
            raise errors.ConfigJson(f"{w}: softcap {fields['softcap']} must be positive")
    else:
        rot = _need(m, "rot", dict, w)
        fields.update(rot_dim=_positive(m, "rot_dim", w), kv_rank=_positive(m, "kv_rank", w),
                      q_rank=_positive(m, "q_rank", w), scale=_need(m, "scale", float, w),
                      rot_base=_need(rot, "base", float, f"{w}.rot"),
                      rot_dims=_positive(rot, "dims", f"{w}.rot"))
        if fields["rot_dims"] % 2 or fields["rot_dims"] > fields["rot_dim"]:
            raise errors.ConfigJson(f"{w}: rot.dims {fields['rot_dims']} must be even and at most "
                                    f"rot_dim {fields['rot_dim']}")
    mlp = entry.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict):
            raise errors.ConfigJson(f"{where}.mlp is not an object")
        mk = _need(mlp, "kind", str, f"{where}.mlp")
        if mk != "dense":
            raise errors.UnsupportedOption(f"{where}.mlp.kind {mk!r}; known: dense")
        fields["ff"] = _positive(mlp, "ff", f"{where}.mlp")
    return VonulornLayer(**fields)
