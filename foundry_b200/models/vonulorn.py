"""The Vonulorn decoder as data: config.json -> `ModelSpec`.

A plain table lookup as embedding; layers in the order the configuration
lists them, each `x <- x + m * mixer(norm1(x))` and, where it has a
feed-forward, `x <- x + m * ff(norm2(x))` with RMS norms and one constant m
for the whole model (`scaled_pre_norm_residual`); three mixers (`gated_delta`,
`differential_attention`, `latent_attention`); the feed-forward is the gated
one with the tanh form of GELU; a final RMS norm and a separate output head.
Tensor names: `embed`, `head`, `final.norm`, `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule
from ..config.vonulorn import ARCHITECTURE, MAX_POSITIONS, VonulornConfig, VonulornLayer

NAMES = {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1", "feed_forward_norm": "norm2"}
UNIT_EPS = 1e-6  # inside the root of the delta mixer's unit-length heads


def _mixer(config: VonulornConfig, layer: VonulornLayer) -> PartSpec:
    if layer.type == "delta":
        return PartSpec("gated_delta", {
            "width": config.width, "heads": layer.heads, "kv_heads": layer.kv_heads,
            "dim": layer.dim, "vdim": layer.vdim, "taps": layer.taps, "eps": config.norm_eps,
            "unit_eps": UNIT_EPS, "gate": "silu"})
    if layer.type == "attention":
        return PartSpec("differential_attention", {
            "width": config.width, "heads": layer.heads, "kv_heads": layer.kv_heads,
            "dim": layer.dim, "vdim": layer.vdim, "scale": layer.scale, "eps": config.norm_eps,
            "diff": layer.diff, "softcap": layer.softcap, "temp_coef": layer.temp_coef,
            "temp_every": layer.temp_every})
    return PartSpec("latent_attention", {
        "width": config.width, "heads": layer.heads, "dim": layer.dim, "rot_dim": layer.rot_dim,
        "vdim": layer.vdim, "kv_rank": layer.kv_rank, "q_rank": layer.q_rank,
        "scale": layer.scale, "eps": config.norm_eps, "rot_base": layer.rot_base,
        "rot_dims": layer.rot_dims, "sink": True})


def build_vonulorn_spec(config: VonulornConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"size": config.width, "eps": config.norm_eps, "weight_suffix": ""})
    block = PartSpec("scaled_pre_norm_residual", {"residual_scale": config.residual_mult})
    layers = []
    for i, layer in enumerate(config.layers):
        ff = None
        if layer.ff is not None:
            ff = PartSpec("swiglu", {"hidden_size": config.width, "intermediate_size": layer.ff,
                                     "names": ("gate", "up", "down"), "suffix": "",
                                     "activation": "gelu_tanh"})
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=_mixer(config, layer),
                                feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff is not None else None, names=NAMES))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=config.width, vocab_size=config.vocab,
        max_positions=MAX_POSITIONS, layers=tuple(layers),
        schedule=default_schedule(len(layers)), final_norm=norm, embedding_name="embed",
        final_norm_prefix="final.norm", output_head_name="head",
        ignorable_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(config.layers)
                                if layer.ff is None))
    spec.validate()
    return spec


VONULORN = register_architecture(Architecture(
    name=ARCHITECTURE, model_type="vonulorn", parse_config=VonulornConfig.parse,
    build_spec=build_vonulorn_spec), replace=True)
