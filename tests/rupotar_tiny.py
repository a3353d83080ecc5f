"""Small Rupotar configurations for the tests, and random weights for them.

The two differ from each other in every size: widths, head counts and
groupings, key and value sizes (unequal in one, equal in the other), taps, ranks, experts and how many are
chosen (also one), windows (shorter than a page, longer than a page, none),
kept first tokens (none, some), layers without feed-forward, the order of the
mixers, a loop of three passes over the first layers, and no loop.
"""
import torch

CONFIGS = {
    "looped": {
        "architecture": "Rupotar", "vocab": 200, "width": 96,
        "embedding": {"scale": 5.0}, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "wkv", "mixer": {"heads": 3, "dim": 16},
             "mlp": {"kind": "dense", "ff": 136}},
            {"type": "attention",
             "mixer": {"heads": 6, "kv_heads": 3, "dim": 16, "vdim": 24, "scale": 0.3,
                       "mask": {"size": 9, "keep_first": 2}},
             "mlp": {"kind": "moe", "expert": {"ff": 40, "limit": 0.8},
                     "router": {"experts": 5, "top": 3}}},
            {"type": "channel_delta",
             "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "conv": 3}, "mlp": None},
            {"type": "attention",
             "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 8, "scale": 0.2},
             "mlp": {"kind": "dense", "ff": 72}},
        ],
        "loop": {"start": 0, "stop": 2, "times": 3},
    },
    "straight": {
        "architecture": "Rupotar", "vocab": 130, "width": 64,
        "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "channel_delta",
             "mixer": {"heads": 2, "kv_heads": 2, "dim": 40, "vdim": 48, "conv": 2},
             "mlp": {"kind": "moe", "expert": {"ff": 24, "limit": 2.5},
                     "router": {"experts": 3, "top": 1}}},
            {"type": "attention",
             "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.5,
                       "mask": {"size": 70, "keep_first": 0}},
             "mlp": None},
            {"type": "wkv", "mixer": {"heads": 2, "dim": 40},
             "mlp": {"kind": "dense", "ff": 100}},
        ],
        "loop": None,
    },
}
RANKS = {"looped": (8, 12), "straight": (24, 8)}  # (decay rank, gate rank) of the low-rank projections


def tensor_shapes(cfg, decay_rank, gate_rank):
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "head": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    if cfg.get("loop"):
        shapes["loop.in"] = (W, 2 * W)
        shapes["loop.step"] = (cfg["loop"]["times"], W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        norms = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer["mlp"] else [])
        for n in norms:
            shapes[f"{p}.{n}"] = shapes[f"{p}.{n}.b"] = (W,)
        H, d = m["heads"], m["dim"]
        if layer["type"] == "attention":
            G, e = m["kv_heads"], m["vdim"]
            shapes.update({f"{p}.mix.q": (H * d, W), f"{p}.mix.k": (G * d, W),
                           f"{p}.mix.v": (G * e, W), f"{p}.mix.q.norm": (H * d,),
                           f"{p}.mix.k.norm": (G * d,), f"{p}.mix.o": (W, H * e)})
        elif layer["type"] == "wkv":
            for s in "rkvgw":
                shapes[f"{p}.mix.mu.{s}"] = (W,)
            for s in "rkvg":
                shapes[f"{p}.mix.{s}"] = (H * d, W)
            shapes.update({f"{p}.mix.w1": (decay_rank, W), f"{p}.mix.w2": (H * d, decay_rank),
                           f"{p}.mix.w0": (H * d,), f"{p}.mix.u": (H, d),
                           f"{p}.mix.norm": (H * d,), f"{p}.mix.o": (W, H * d)})
        else:
            G, e, taps = m["kv_heads"], m["vdim"], m["conv"]
            shapes.update({f"{p}.mix.q": (G * d, W), f"{p}.mix.q.conv": (G * d, taps),
                           f"{p}.mix.k": (G * d, W), f"{p}.mix.k.conv": (G * d, taps),
                           f"{p}.mix.v": (H * e, W), f"{p}.mix.v.conv": (H * e, taps),
                           f"{p}.mix.b": (H, W), f"{p}.mix.A_log": (H,), f"{p}.mix.norm": (e,),
                           f"{p}.mix.a1": (decay_rank, W), f"{p}.mix.a2": (H * d, decay_rank),
                           f"{p}.mix.dt_bias": (H * d,), f"{p}.mix.g1": (gate_rank, W),
                           f"{p}.mix.g2": (H * e, gate_rank), f"{p}.mix.o": (W, H * e)})
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            shapes.update({f"{p}.mlp.gate": (mlp["ff"], W), f"{p}.mlp.up": (mlp["ff"], W),
                           f"{p}.mlp.down": (W, mlp["ff"])})
        elif mlp:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            shapes[f"{p}.mlp.router"], shapes[f"{p}.mlp.router.b"] = (E, W), (E,)
            for x in range(E):
                shapes.update({f"{p}.mlp.e{x}.gate": (ff, W), f"{p}.mlp.e{x}.up": (ff, W),
                               f"{p}.mlp.e{x}.down": (W, ff)})
    return shapes


def random_weights(name, seed=0):
    """bfloat16-representable float32 tensors by file name. Matrices are wide
    enough that a wrong key, state or expert moves the logits; norm weights lie
    around one, biases and mixing coefficients in sensible ranges."""
    cfg = CONFIGS[name]
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for key, shape in tensor_shapes(cfg, *RANKS[name]).items():
        leaf = key.split(".")[-1]
        r = torch.randn(shape, generator=gen)
        if key.endswith(".b") and "norm" in key or leaf in ("dt_bias", "w0", "step") or key.endswith("router.b"):
            t = 0.3 * r
        elif leaf in ("norm", "norm1", "norm1b", "norm2", "norm2b") and len(shape) == 1:
            t = 1.0 + 0.2 * r
        elif leaf in "rkvgw" and ".mu." in key:
            t = torch.rand(shape, generator=gen)
        elif leaf == "A_log":
            t = -0.5 + 0.5 * r
        elif leaf == "conv":
            t = 0.5 * r
        elif leaf == "u":
            t = 0.5 * r
        elif leaf in ("embed",):
            t = 0.5 * r
        else:
            t = r / (shape[-1] ** 0.5) * 1.5
        out[key] = t.to(torch.bfloat16).to(torch.float32)
    return out


def write_folder(folder, name, seed=0):
    """A model folder as the loader reads it: config.json + model.safetensors (bfloat16)."""
    import json
    import os
    from foundry_b200.weights.safetensors_io import SINGLE_FILE, save_file
    os.makedirs(folder, exist_ok=True)
    weights = random_weights(name, seed)
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()},
              os.path.join(folder, SINGLE_FILE), metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(CONFIGS[name], handle)
    return folder, weights
