"""The Vonulorn decoder, plainly: float64, whole sequences, no cache, no state
carried between calls, one function per mechanism. It takes a decoded
config.json document and a dict of tensors by their file names, and shares no
code with `foundry_b200`. The `*_stepwise` variants walk a sequence token by
token with explicit state or explicit key lists and guard the whole-sequence
forms (tests/test_vonulorn_cpu.py).

Notation: T tokens, W width, H heads, G key heads, d key size, e value size,
r latent size, c rotated size.
"""
import math

import torch

F = torch.float64
UNIT_EPS = 1e-6  # inside the root of the unit-length heads of the delta mixer


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_feed_forward(w, p, h):
    return (gelu_tanh(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


# ------------------------------------------------------------------ delta mixer
def causal_conv(x, taps_w):
    """y[t, c] = sum_a taps_w[c, a] x[t - (A - 1 - a), c], zeros in front of t = 0."""
    T, C = x.shape
    A = taps_w.shape[1]
    padded = torch.cat([torch.zeros(A - 1, C, dtype=F), x], 0)
    y = torch.zeros(T, C, dtype=F)
    for a in range(A):
        y += padded[a:a + T] * taps_w[:, a]
    return y


def delta_inputs(m, w, p, h):
    """What enters the recurrence: q, k [T, G, d] (unit length, q also / sqrt d),
    v [T, H, e], step sizes beta [T, H], decays g [T, H]."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def branch(name):
        return silu(causal_conv(h @ w[f"{p}.{name}"].T, w[f"{p}.{name}.conv"]))

    def unit(x):
        return x / torch.sqrt((x * x).sum(-1, keepdim=True) + UNIT_EPS)

    q = unit(branch("q").view(T, G, d)) * d ** -0.5
    k = unit(branch("k").view(T, G, d))
    v = branch("v").view(T, H, e)
    beta = torch.sigmoid(h @ w[p + ".b"].T)
    g = torch.exp(-torch.exp(w[p + ".A_log"]) * softplus(h @ w[p + ".a"].T + w[p + ".dt_bias"]))
    return q, k, v, beta, g


def delta_recurrence(q, k, v, beta, g, state=None):
    """S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, per head, in this
    order. q, k [T, G, d]; v [T, H, e]; beta, g [T, H]. Returns o [T, H, e] and S."""
    T, H, e = v.shape
    G, d = q.shape[1], q.shape[2]
    S = torch.zeros(H, d, e, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, e, dtype=F)
    for t in range(T):
        for a in range(H):
            kk, qq = k[t, a // (H // G)], q[t, a // (H // G)]
            S[a] = S[a] * g[t, a]
            u = beta[t, a] * (v[t, a] - S[a].T @ kk)
            S[a] = S[a] + torch.outer(kk, u)
            o[t, a] = S[a].T @ qq
    return o, S


def delta_mixer(m, w, p, h, eps):
    T = h.shape[0]
    H, e = m["heads"], m["vdim"]
    o, _ = delta_recurrence(*delta_inputs(m, w, p, h))
    gate = silu(h @ w[p + ".g"].T).view(T, H, e)
    y = rms_unit(o, eps) * w[p + ".norm"] * gate
    return y.reshape(T, H * e) @ w[p + ".o"].T


# ------------------------------------------------------- differential attention
def query_temperature(positions, coef, every):
    p = torch.as_tensor(positions, dtype=torch.int64)
    return 1.0 + coef * torch.log(torch.div(p + 1, every, rounding_mode="floor").to(F) + 1.0)


def soft_cap(s, cap):
    return cap * torch.tanh(s / cap)


def differential_lambda(m, w, p):
    return (math.exp(float((w[p + ".lq1"] * w[p + ".lk1"]).sum()))
            - math.exp(float((w[p + ".lq2"] * w[p + ".lk2"]).sum())) + m["diff"])


def differential_attention(m, w, p, h, eps, first_position=0):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    temp = query_temperature(range(first_position, first_position + T), m["q_temp"]["coef"],
                             m["q_temp"]["every"])
    q = (h @ w[p + ".q"].T).view(T, H, 2, d) * temp[:, None, None, None]
    k = (h @ w[p + ".k"].T).view(T, G, 2, d)
    v = (h @ w[p + ".v"].T).view(T, G, e)
    lam = differential_lambda(m, w, p)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, e, dtype=F)
    for a in range(H):
        g = a // (H // G)
        maps = []
        for which in range(2):
            s = soft_cap((q[:, a, which] @ k[:, g, which].T) * m["scale"], m["softcap"])
            s = torch.where(causal, s, torch.tensor(-math.inf, dtype=F))
            maps.append(torch.softmax(s, -1) @ v[:, g])
        out[:, a] = rms_unit(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    return out.reshape(T, H * e) @ w[p + ".o"].T


# ------------------------------------------------------------ latent attention
def rotate_pairs(x, positions, base, dims):
    """The first `dims` elements of the last axis turn in neighbouring pairs
    (2i, 2i + 1) by the angle position * base^(-2i / dims); the rest stay."""
    p = torch.as_tensor(positions, dtype=F)
    i = torch.arange(dims // 2, dtype=F)
    angle = p[:, None] * torch.pow(torch.tensor(base, dtype=F), -2.0 * i / dims)
    shape = [len(positions)] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def latent_attention(m, w, p, h, eps, first_position=0):
    T = h.shape[0]
    H, d, c, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = range(first_position, first_position + T)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    cq = rms_norm(h @ w[p + ".dq"].T, w[p + ".dq.norm"], eps)
    q = (cq @ w[p + ".uq"].T).view(T, H, d + c)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], positions, base, dims)
    down = h @ w[p + ".dkv"].T
    latent = rms_norm(down[:, :r], w[p + ".dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, r:], positions, base, dims)       # one for all heads
    k_plain = (latent @ w[p + ".uk"].T).view(T, H, d)
    v = (latent @ w[p + ".uv"].T).view(T, H, e)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, e, dtype=F)
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        s = torch.where(causal, s, torch.tensor(-math.inf, dtype=F))
        sink = w[p + ".sink"][a]
        top = torch.maximum(s.max(-1, keepdim=True).values, sink)
        ex = torch.exp(s - top)
        out[:, a] = (ex / (torch.exp(sink - top) + ex.sum(-1, keepdim=True))) @ v[:, a]
    return out.reshape(T, H * e) @ w[p + ".o"].T


MIXERS = {"delta": lambda m, w, p, h, eps: delta_mixer(m, w, p, h, eps),
          "attention": differential_attention, "latent_attention": latent_attention}


# ----------------------------------------------------------------- the model
def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence from position 0 (and, if asked,
    the residual stream after every layer [layers, T, W])."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens)]
    seen = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        mixed = MIXERS[layer["type"]](layer["mixer"], w, p + ".mix", rms_norm(x, w[p + ".norm1"], eps), eps)
        x = x + mult * mixed
        if layer.get("mlp") is not None:
            x = x + mult * gated_feed_forward(w, p + ".mlp", rms_norm(x, w[p + ".norm2"], eps))
        seen.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(seen)) if return_layers else logits


# ------------------------------------------------- token-by-token counterparts
def delta_mixer_stepwise(m, w, p, h, eps):
    """The delta mixer one token at a time: explicit convolution tails and state."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    taps = w[p + ".q.conv"].shape[1]
    tails = {n: torch.zeros(taps - 1, w[f"{p}.{n}"].shape[0], dtype=F) for n in "qkv"}
    S = torch.zeros(H, d, e, dtype=F)
    rows = []
    for t in range(T):
        x = h[t]
        act = {}
        for n in "qkv":
            window = torch.cat([tails[n], (w[f"{p}.{n}"] @ x)[None]], 0)   # [taps, C], newest last
            act[n] = silu((window * w[f"{p}.{n}.conv"].T).sum(0))
            tails[n] = window[1:]
        q = act["q"].view(G, d)
        k = act["k"].view(G, d)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_EPS) * d ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
        v = act["v"].view(H, e)
        beta = torch.sigmoid(w[p + ".b"] @ x)
        g = torch.exp(-torch.exp(w[p + ".A_log"]) * softplus(w[p + ".a"] @ x + w[p + ".dt_bias"]))
        o, S = delta_recurrence(q[None], k[None], v[None], beta[None], g[None], S)
        y = rms_unit(o[0], eps) * w[p + ".norm"] * silu(w[p + ".g"] @ x).view(H, e)
        rows.append(w[p + ".o"] @ y.reshape(H * e))
    return torch.stack(rows)


def latent_attention_stepwise(m, w, p, h, eps):
    """Latent attention one token at a time over a list of (latent, rotated key)
    rows, with the key and value expansions folded into the query and the output."""
    T = h.shape[0]
    H, d, c, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    uk, uv = w[p + ".uk"].view(H, d, r), w[p + ".uv"].view(H, e, r)
    kept = []
    rows = []
    for t in range(T):
        x = h[t:t + 1]
        q = (rms_norm(x @ w[p + ".dq"].T, w[p + ".dq.norm"], eps) @ w[p + ".uq"].T).view(1, H, d + c)
        q_rot = rotate_pairs(q[..., d:], [t], base, dims)[0]
        down = x @ w[p + ".dkv"].T
        kept.append(torch.cat([rms_norm(down[:, :r], w[p + ".dkv.norm"], eps)[0],
                               rotate_pairs(down[:, r:], [t], base, dims)[0]]))
        rows_kept = torch.stack(kept)                                  # [t + 1, r + c]
        heads = []
        for a in range(H):
            q_lat = uk[a].T @ q[0, a, :d]                              # [r]
            s = (rows_kept[:, :r] @ q_lat + rows_kept[:, r:] @ q_rot[a]) * m["scale"]
            sink = w[p + ".sink"][a]
            top = torch.maximum(s.max(), sink)
            ex = torch.exp(s - top)
            mixed = (ex / (torch.exp(sink - top) + ex.sum())) @ rows_kept[:, :r]
            heads.append(uv[a] @ mixed)
        rows.append(w[p + ".o"] @ torch.cat(heads))
    return torch.stack(rows)
