"""Small Vonulorn configurations for the tests, and random weights for them.

The two differ from each other in every size and constant: widths, head
counts and groupings (also one head, and as many key heads as heads), key and
value sizes (multiples of 8 and not), taps, ranks, rotated sizes, scales, the
score cap (one that bites and one that hardly does), the query temperature's
period (shorter and longer than a page), the residual constant (also 1),
layers without feed-forward, and the order of the mixers.
"""
import json
import os

import torch

CONFIGS = {
    "mixed": {
        "architecture": "Vonulorn", "vocab": 210, "width": 96, "norm": {"eps": 1e-5},
        "residual_mult": 0.7,
        "layers": [
            {"type": "latent_attention",
             "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "q_rank": 48,
                       "scale": 0.2, "rot": {"base": 10000.0, "dims": 8}},
             "mlp": {"kind": "dense", "ff": 136}},
            {"type": "delta",
             "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 24, "conv": 4}, "mlp": None},
            {"type": "attention",
             "mixer": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3,
                       "softcap": 2.0, "diff": 0.35, "q_temp": {"coef": 0.2, "every": 7}},
             "mlp": {"kind": "dense", "ff": 72}},
            {"type": "delta",
             "mixer": {"heads": 2, "kv_heads": 1, "dim": 40, "vdim": 8, "conv": 2},
             "mlp": {"kind": "dense", "ff": 64}},
        ],
    },
    "other": {
        "architecture": "Vonulorn", "vocab": 130, "width": 64, "norm": {"eps": 3e-6},
        "residual_mult": 1.0,
        "layers": [
            {"type": "attention",
             "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.25,
                       "softcap": 50.0, "diff": 0.25, "q_temp": {"coef": 0.5, "every": 70}},
             "mlp": None},
            {"type": "latent_attention",
             "mixer": {"heads": 1, "dim": 32, "rot_dim": 16, "vdim": 16, "kv_rank": 64, "q_rank": 24,
                       "scale": 0.15, "rot": {"base": 500000.0, "dims": 16}},
             "mlp": {"kind": "dense", "ff": 100}},
            {"type": "delta",
             "mixer": {"heads": 3, "kv_heads": 1, "dim": 24, "vdim": 48, "conv": 3},
             "mlp": {"kind": "dense", "ff": 40}},
        ],
    },
}


def mixer_shapes(kind, m, W):
    """Tensor shapes of one mixer by the names under its prefix."""
    H, d, e = m["heads"], m["dim"], m["vdim"]
    if kind == "delta":
        G, taps = m["kv_heads"], m["conv"]
        return {"q": (G * d, W), "q.conv": (G * d, taps), "k": (G * d, W), "k.conv": (G * d, taps),
                "v": (H * e, W), "v.conv": (H * e, taps), "b": (H, W), "A_log": (H,), "norm": (e,),
                "a": (H, W), "dt_bias": (H,), "g": (H * e, W), "o": (W, H * e)}
    if kind == "attention":
        G = m["kv_heads"]
        return {"q": (H * 2 * d, W), "k": (G * 2 * d, W), "v": (G * e, W), "lq1": (d,), "lk1": (d,),
                "lq2": (d,), "lk2": (d,), "o": (W, H * e)}
    r, c, qr = m["kv_rank"], m["rot_dim"], m["q_rank"]
    return {"dq": (qr, W), "dq.norm": (qr,), "uq": (H * (d + c), qr), "dkv": (r + c, W),
            "dkv.norm": (r,), "uk": (H * d, r), "uv": (H * e, r), "sink": (H,), "o": (W, H * e)}


def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        shapes[f"{p}.norm1"] = (W,)
        for name, shape in mixer_shapes(layer["type"], layer["mixer"], W).items():
            shapes[f"{p}.mix.{name}"] = shape
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            shapes[f"{p}.norm2"] = (W,)
            shapes.update({f"{p}.mlp.gate": (ff, W), f"{p}.mlp.up": (ff, W), f"{p}.mlp.down": (W, ff)})
    return shapes


def draw(key, shape, gen):
    """One bfloat16-representable float32 tensor in a range that lets its mechanism
    matter: decays well inside (0, 1), sinks that take a real share of the sum,
    a lambda away from its constant part, norm weights around one."""
    leaf = key.split(".")[-1]
    r = torch.randn(shape, generator=gen)
    if leaf in ("dt_bias",):
        t = 0.3 * r
    elif leaf == "norm" or leaf in ("norm1", "norm2"):
        t = 1.0 + 0.2 * r
    elif leaf == "A_log":
        t = -0.5 + 0.5 * r
    elif leaf == "conv":
        t = 0.5 * r
    elif leaf == "sink":
        t = 1.0 + r
    elif leaf in ("lq1", "lk1", "lq2", "lk2"):
        t = 0.35 * r
    elif leaf == "embed":
        t = 0.5 * r
    else:
        t = r / (shape[-1] ** 0.5) * 1.5
    return t.to(torch.bfloat16).to(torch.float32)


def random_weights(name, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return {key: draw(key, shape, gen) for key, shape in tensor_shapes(CONFIGS[name]).items()}


def random_mixer(kind, m, W, prefix="a", seed=0):
    gen = torch.Generator().manual_seed(seed)
    return {f"{prefix}.{n}": draw(f"{prefix}.{n}", s, gen) for n, s in mixer_shapes(kind, m, W).items()}


def write_folder(folder, name, seed=0):
    """A model folder as the loader reads it: config.json + model.safetensors (bfloat16)."""
    from foundry_b200.weights.safetensors_io import SINGLE_FILE, save_file
    os.makedirs(folder, exist_ok=True)
    weights = random_weights(name, seed)
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()},
              os.path.join(folder, SINGLE_FILE), metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(CONFIGS[name], handle)
    return folder, weights
