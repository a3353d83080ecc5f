"""Grouped-query attention with a distance bias, a sliding window that keeps
the first tokens, and a softmax with a sink, as a mixer.

    q = Wq h, k = Wk h, v = Wv h   (one product), no biases
    q, k: RMS norm over the WHOLE projection of a token (all heads at once), weights wq, wk
    s_ij = (q_i . k_j) * scale - slope_h (i - j),   slope_h = 2^(-steep (h + 1) / heads)
    j visible to i iff j <= i and (i - j < window or j < keep_first)
    p_ij = exp(s_ij) / (1 + sum_j exp(s_ij))        (the 1 is exp(0): one more term in the sum that adds nothing to the output)
    out = Wo [heads' outputs side by side]

Keys have `dim` elements a head, values `vdim`. No rotation: positions enter
through the bias and the mask only; the bias of a kept token is by the distance it really has.
Every constant (scale, steep, window, keep_first, the sink) is a parameter; the
tensor names under the mixer's prefix are `q k v o` and `q.norm k.norm` unless
given otherwise.

The cache keeps every key (the kept first tokens stay readable for ever, so a
ring over the window alone would lose them); the kernels walk only the kept
prefix and the window.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.store import KVRequest, KVView
from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_mixer
from .linear import Linear
from .products import product_f32


@register_mixer("sink_window_attention")
class SinkWindowAttention(Part):
    replay_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, window: Optional[int] = None, keep_first: int = 0,
                 steep: float = 8.0, sink: bool = True, suffix: str = "", *,
                 dtype: torch.dtype, device: torch.device):
        if kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key-value heads")
        if not 1 <= dim <= 256 or not 1 <= vdim <= 256:
            raise ValueError(f"key size {dim} and value size {vdim} must be at most 256")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.eps = float(scale), float(eps)
        self.window, self.keep_first = (int(window) if window else 0), int(keep_first or 0)
        self.steep, self.sink = float(steep), bool(sink)
        self.dtype, self.device = dtype, device
        self.nq, self.nk, self.nv = heads * dim, kv_heads * dim, kv_heads * vdim
        self.suffix = suffix
        self.qkv = Linear(width, [("q", self.nq), ("k", self.nk), ("v", self.nv)], dtype=dtype,
                          device=device, suffix=suffix)
        self.o = Linear(heads * vdim, [("o", width)], dtype=dtype, device=device, suffix=suffix)
        self.q_norm = self.k_norm = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {**self.qkv.expected_tensors(prefix), **self.o.expected_tensors(prefix),
                f"{prefix}.q.norm": ExpectedTensor((self.nq,)),
                f"{prefix}.k.norm": ExpectedTensor((self.nk,))}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.qkv.load(prefix, fetch)
        self.o.load(prefix, fetch)
        self.q_norm = fetch(f"{prefix}.q.norm").to(torch.float32).contiguous()
        self.k_norm = fetch(f"{prefix}.k.norm").to(torch.float32).contiguous()

    def cache_request(self) -> KVRequest:
        return KVRequest(self.kv_heads, self.dim, None, self.vdim)

    def first_weight(self):
        return self.qkv.weight

    def context_flops(self, token_counts, starts) -> float:
        pairs = 0.0
        for n, start in zip(token_counts, starts):
            for p in (start, start + n - 1):
                seen = p + 1
                if self.window:
                    seen = min(seen, self.window + min(self.keep_first, max(0, p + 1 - self.window)))
                pairs += 0.5 * n * seen
        return 2.0 * self.heads * (self.dim + self.vdim) * pairs

    def forward(self, ctx, x, cache: KVView):
        table = ctx.page_table(cache.group)
        qkv = product_f32(x, self.qkv.weight)
        q = torch.empty((x.shape[0], self.nq), dtype=x.dtype, device=x.device)
        ops.qk_norm_cache_write(qkv, q, self.q_norm, self.k_norm, self.eps, ctx.positions,
                                ctx.seq_of_token, table, cache.k, cache.v, self.heads,
                                self.kv_heads, self.dim, self.vdim, write_cache=cache.writes)
        attn = torch.empty((x.shape[0], self.heads * self.vdim), dtype=x.dtype, device=x.device)
        ops.attention_sink(ctx, q, attn, table, cache.k, cache.v, self.heads, self.kv_heads,
                           self.dim, self.vdim, self.scale, window=self.window,
                           keep_first=self.keep_first, sink=self.sink, steep=self.steep)
        return product_f32(attn, self.o.weight)
