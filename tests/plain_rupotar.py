"""The Rupotar decoder, plainly: float64, whole sequences, no cache, no state
carried between calls, one function per mechanism. It takes a decoded
config.json document and a dict of tensors by their file names, and shares no
code with `foundry_b200`. `*_stepwise` variants walk a sequence token by token
with explicit state and guard the whole-sequence forms (tests/test_rupotar_cpu.py).

Notation: T tokens, W width, H heads, G key/value heads, d key size, e value size.
"""
import math

import torch

F = torch.float64


def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def position_vector(positions, width, base=10000.0):
    p = torch.as_tensor(positions, dtype=F)[:, None]
    i = torch.arange(width // 2, dtype=F)[None, :]
    angle = p * torch.pow(torch.tensor(base, dtype=F), -2.0 * i / width)
    out = torch.zeros(len(positions), width, dtype=F)
    out[:, 0::2], out[:, 1::2] = torch.sin(angle), torch.cos(angle)
    return out


def embedding(cfg, w, tokens, first_position=0):
    rows = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    return rows + position_vector(range(first_position, first_position + len(tokens)), cfg["width"])


def visible(i, j, window, keep_first):
    return j <= i and (window is None or i - j < window or j < keep_first)


def sink_attention(m, w, p, h, eps, steep=8.0):
    """Attention with whole-projection q/k norm, distance bias, window with kept
    first tokens, and one added to the softmax's denominator."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit(h @ w[p + ".q"].T, eps) * w[p + ".q.norm"]
    k = rms_unit(h @ w[p + ".k"].T, eps) * w[p + ".k.norm"]
    v = h @ w[p + ".v"].T
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, e)
    mask = m.get("mask") or {}
    window, keep = mask.get("size"), mask.get("keep_first") or 0
    seen = torch.tensor([[visible(i, j, window, keep) for j in range(T)] for i in range(T)])
    distance = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F)
    out = torch.zeros(T, H, e, dtype=F)
    for a in range(H):
        g = a // (H // G)
        slope = 2.0 ** (-steep * (a + 1) / H)
        s = (q[:, a] @ k[:, g].T) * m["scale"] - slope * distance
        s = torch.where(seen, s, torch.tensor(-math.inf, dtype=F))
        top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)  # the sink's score is 0
        ex = torch.exp(s - top)
        prob = ex / (torch.exp(-top) + ex.sum(-1, keepdim=True))
        out[:, a] = prob @ v[:, g]
    return out.reshape(T, H * e) @ w[p + ".o"].T


def wkv_time_mix(m, w, p, h, eps):
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, W, dtype=F), h[:-1]], 0)

    def mixed(s):
        return h + (before - h) * w[f"{p}.mu.{s}"]
    r = (mixed("r") @ w[p + ".r"].T).view(T, H, d)
    k = (mixed("k") @ w[p + ".k"].T).view(T, H, d)
    v = (mixed("v") @ w[p + ".v"].T).view(T, H, d)
    gate = silu(mixed("g") @ w[p + ".g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mixed("w") @ w[p + ".w1"].T) @ w[p + ".w2"].T
                                 + w[p + ".w0"])).view(T, H, d)
    bonus = w[p + ".u"]
    S = torch.zeros(H, d, d, dtype=F)
    o = torch.zeros(T, H, d, dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = ((S + bonus[:, :, None] * kv) * r[t][:, :, None]).sum(1)
        S = decay[t][:, :, None] * S + kv
    y = rms_unit(o, eps).reshape(T, H * d) * w[p + ".norm"] * gate
    return y @ w[p + ".o"].T


def causal_conv(x, taps_w):
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], 0)
    return sum(padded[a:a + T] * taps_w[:, a] for a in range(taps))


def gated_delta(m, w, p, h, eps, unit_eps=1e-6):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])).view(T, H, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    beta = torch.sigmoid(h @ w[p + ".b"].T)
    raw = (h @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".dt_bias"]
    g = torch.exp(-torch.exp(w[p + ".A_log"])[None, :, None]
                  * torch.log1p(torch.exp(raw)).view(T, H, d))
    S = torch.zeros(H, d, e, dtype=F)
    o = torch.zeros(T, H, e, dtype=F)
    for t in range(T):
        for a in range(H):
            kk, qq = k[t, a // (H // G)], q[t, a // (H // G)]
            S[a] = g[t, a][:, None] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ kk)
            S[a] = S[a] + kk[:, None] * u[None, :]
            o[t, a] = S[a].T @ qq
    gate = torch.sigmoid((h @ w[p + ".g1"].T) @ w[p + ".g2"].T).view(T, H, e)
    y = rms_unit(o, eps) * w[p + ".norm"] * gate
    return y.reshape(T, H * e) @ w[p + ".o"].T


def dense_feed_forward(w, p, h):
    return (silu(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


def routed_experts(mlp, w, p, h, alpha=1.702):
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    z = h @ w[p + ".router"].T + w[p + ".router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))[:top]
        share = torch.softmax(torch.stack([z[t, e] for e in order]), 0)
        for c, e in enumerate(order):
            g = torch.clamp(h[t] @ w[f"{p}.e{e}.gate"].T, max=limit)
            u = torch.clamp(h[t] @ w[f"{p}.e{e}.up"].T, -limit, limit)
            out[t] += share[c] * ((g * torch.sigmoid(alpha * g) * (u + 1.0)) @ w[f"{p}.e{e}.down"].T)
    return out


MIXERS = {"attention": lambda cfg, m, w, p, h: sink_attention(m, w, p, h, cfg["norm"]["eps"]),
          "wkv": lambda cfg, m, w, p, h: wkv_time_mix(m, w, p, h, cfg["norm"]["eps"]),
          "channel_delta": lambda cfg, m, w, p, h: gated_delta(m, w, p, h, cfg["norm"]["eps"])}


def layer(cfg, w, i, x):
    spec, p, eps = cfg["layers"][i], f"l{i}", cfg["norm"]["eps"]

    def norm(name, y):
        return layer_norm(y, w[f"{p}.{name}"], w[f"{p}.{name}.b"], eps)
    x = x + norm("norm1b", MIXERS[spec["type"]](cfg, spec["mixer"], w, p + ".mix", norm("norm1", x)))
    mlp = spec.get("mlp")
    if mlp:
        h = norm("norm2", x)
        y = dense_feed_forward(w, p + ".mlp", h) if mlp["kind"] == "dense" else \
            routed_experts(mlp, w, p + ".mlp", h)
        x = x + norm("norm2b", y)
    return x


def run_order(cfg):
    """[(layer, pass number or None)]: the pass number stands at a pass's first layer."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] of a whole sequence; `streams` collects the residual
    stream after every layer run."""
    x0 = embedding(cfg, w, tokens)
    x = x0
    for i, number in run_order(cfg):
        if number is not None:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T + w["loop.step"][number]
        x = layer(cfg, w, i, x)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"]) @ w["head"].T


def greedy_generate(cfg, w, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits = forward(cfg, w, tokens)[-1]
        tokens.append(int(torch.argmax(logits)))  # the lowest index among equals
    return tokens[len(prompt):]


# ---------------------------------------------------------- token by token
def wkv_stepwise(m, w, p, h, eps):
    """The same mixer one token at a time over explicit state (previous input, S)."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    before, S, outs = torch.zeros(W, dtype=F), torch.zeros(H, d, d, dtype=F), []
    for t in range(T):
        x = h[t]
        mix = {s: x + (before - x) * w[f"{p}.mu.{s}"] for s in "rkvgw"}
        r, k, v = ((w[f"{p}.{s}"] @ mix[s]).view(H, d) for s in "rkv")
        gate = silu(w[p + ".g"] @ mix["g"])
        decay = torch.exp(-torch.exp(w[p + ".w2"] @ torch.tanh(w[p + ".w1"] @ mix["w"])
                                     + w[p + ".w0"])).view(H, d)
        kv = k[:, :, None] * v[:, None, :]
        o = ((S + w[p + ".u"][:, :, None] * kv) * r[:, :, None]).sum(1)
        S = decay[:, :, None] * S + kv
        before = x
        outs.append(w[p + ".o"] @ (rms_unit(o, eps).reshape(-1) * w[p + ".norm"] * gate))
    return torch.stack(outs)


def gated_delta_stepwise(m, w, p, h, eps, unit_eps=1e-6):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    taps = w[p + ".q.conv"].shape[1]
    hist = {s: torch.zeros(taps - 1, w[f"{p}.{s}"].shape[0], dtype=F) for s in "qkv"}
    S, outs = torch.zeros(H, d, e, dtype=F), []
    for t in range(T):
        x = h[t]
        cur = {}
        for s in "qkv":
            rows = torch.cat([hist[s], (w[f"{p}.{s}"] @ x)[None]], 0)
            cur[s] = silu((rows * w[f"{p}.{s}.conv"].T).sum(0))
            hist[s] = rows[1:]
        q, k, v = cur["q"].view(G, d), cur["k"].view(G, d), cur["v"].view(H, e)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * d ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
        beta = torch.sigmoid(w[p + ".b"] @ x)
        raw = w[p + ".a2"] @ (w[p + ".a1"] @ x) + w[p + ".dt_bias"]
        g = torch.exp(-torch.exp(w[p + ".A_log"])[:, None] * torch.log1p(torch.exp(raw)).view(H, d))
        o = torch.zeros(H, e, dtype=F)
        for a in range(H):
            kk, qq = k[a // (H // G)], q[a // (H // G)]
            S[a] = g[a][:, None] * S[a]
            S[a] = S[a] + kk[:, None] * (beta[a] * (v[a] - S[a].T @ kk))[None, :]
            o[a] = S[a].T @ qq
        gate = torch.sigmoid(w[p + ".g2"] @ (w[p + ".g1"] @ x)).view(H, e)
        outs.append(w[p + ".o"] @ (rms_unit(o, eps) * w[p + ".norm"] * gate).reshape(-1))
    return torch.stack(outs)
