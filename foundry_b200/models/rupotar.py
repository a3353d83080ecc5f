"""The Rupotar decoder as data: config.json -> `ModelSpec`.

Embedding times a constant plus a sinusoidal position vector; layers with a
layer norm in front of and behind each part (`sandwich_norm_residual`); three
mixers (attention with distance bias, window, kept first tokens and a sink;
RWKV-style time mixing; the gated delta rule with channel-wise decay); dense
SwiGLU or routed experts behind them; a group of layers that may run several
times with the same weights, each pass with cache entries of its own and a
`loop_input` junction in front; a final layer norm and a separate output head.
Tensor names: `embed`, `head`, `final.norm[.b]`, `loop.in`, `loop.step`, and
`l<i>.{norm1,norm1b,norm2,norm2b}[.b]`, `l<i>.mix.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.rupotar import (ARCHITECTURE, MAX_POSITIONS, RupotarConfig, RupotarLayer,
                              complete_from_files)
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NAMES = {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1", "mixer_post_norm": "norm1b",
         "feed_forward_norm": "norm2", "feed_forward_post_norm": "norm2b"}
BIAS_STEEPNESS = 8.0     # slope_h = 2^(-8 (h + 1) / heads)
EXPERT_ALPHA = 1.702     # g * sigmoid(1.702 g)
UNIT_EPS = 1e-6          # inside the root of the unit-length heads
POSITION_BASE = 10000.0


def _mixer(config: RupotarConfig, layer: RupotarLayer) -> PartSpec:
    if layer.type == "attention":
        return PartSpec("sink_window_attention", {
            "width": config.width, "heads": layer.heads, "kv_heads": layer.kv_heads,
            "dim": layer.dim, "vdim": layer.vdim, "scale": layer.scale, "eps": config.norm_eps,
            "window": layer.window, "keep_first": layer.keep_first, "steep": BIAS_STEEPNESS,
            "sink": True})
    if layer.type == "wkv":
        return PartSpec("wkv_time_mix", {
            "width": config.width, "heads": layer.heads, "dim": layer.dim, "eps": config.norm_eps,
            "decay_rank": layer.decay_rank})
    return PartSpec("gated_delta_channel", {
        "width": config.width, "heads": layer.heads, "kv_heads": layer.kv_heads, "dim": layer.dim,
        "vdim": layer.vdim, "taps": layer.taps, "eps": config.norm_eps,
        "decay_rank": layer.decay_rank, "gate_rank": layer.gate_rank, "unit_eps": UNIT_EPS})


def _feed_forward(config: RupotarConfig, layer: RupotarLayer):
    mlp = layer.mlp
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return PartSpec("swiglu", {"hidden_size": config.width, "intermediate_size": mlp.ff,
                                   "names": ("gate", "up", "down"), "suffix": ""})
    return PartSpec("routed_experts", {"width": config.width, "ff": mlp.ff, "experts": mlp.experts,
                                       "top": mlp.top, "limit": mlp.limit, "alpha": EXPERT_ALPHA})


def build_rupotar_spec(config: RupotarConfig) -> ModelSpec:
    config = config.with_default_ranks()
    norm = PartSpec("layer_norm", {"size": config.width, "eps": config.norm_eps,
                                   "weight_suffix": "", "bias_suffix": ".b"})
    layers = []
    for i, layer in enumerate(config.layers):
        ff = _feed_forward(config, layer)
        layers.append(LayerSpec(
            prefix=f"l{i}", block=PartSpec("sandwich_norm_residual", {}),
            mixer=_mixer(config, layer), feed_forward=ff, mixer_norm=norm,
            feed_forward_norm=norm if ff is not None else None, names=NAMES,
            mixer_post_norm=norm, feed_forward_post_norm=norm if ff is not None else None))
    # the order of runs: a looped group's passes follow one another, each pass with
    # cache entries of its own and the junction in front of its first layer
    runs = []
    junctions = ()
    n = len(config.layers)
    if config.loop is None:
        runs = [(i, None) for i in range(n)]
    else:
        start, stop, times = config.loop
        junctions = (PartSpec("loop_input", {"width": config.width, "times": times}),)
        runs = [(i, None) for i in range(start)]
        for t in range(times):
            runs += [(i, (0, t) if i == start else None) for i in range(start, stop)]
        runs += [(i, None) for i in range(stop, n)]
    schedule = tuple(ScheduleEntry(layer=i, cache=c, junction=j) for c, (i, j) in enumerate(runs))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=config.width, vocab_size=config.vocab,
        max_positions=MAX_POSITIONS, layers=tuple(layers), schedule=schedule, final_norm=norm,
        embedding_name="embed", final_norm_prefix="final.norm", output_head_name="head",
        # a layer without a feed-forward has no use for the norms around one; a file
        # that carries them all the same is still this model
        ignorable_tensors=tuple(f"l{i}.norm2{tail}" for i, layer in enumerate(config.layers)
                                if layer.mlp is None for tail in ("", ".b", "b", "b.b")),
        embedding=PartSpec("scaled_sinusoidal", {"width": config.width,
                                                 "scale": config.embedding_scale,
                                                 "base": POSITION_BASE}),
        junctions=junctions, junction_prefixes=("loop",) * len(junctions))
    spec.validate()
    return spec


RUPOTAR = register_architecture(Architecture(
    name=ARCHITECTURE, model_type="rupotar", parse_config=RupotarConfig.parse,
    build_spec=build_rupotar_spec, complete_from_files=complete_from_files), replace=True)
