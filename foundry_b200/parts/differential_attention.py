"""Differential attention over the cache, as a mixer.

A query head has two query vectors and a key head two key vectors of `dim`
elements, laid out head by head as [map 1 | map 2]; each map is a causal
softmax attention of its own over the same values (`vdim` a head), and a
head's output is their weighted difference, normalised:

    q = Wq h (heads x 2 dim),  k = Wk h (kv_heads x 2 dim),  v = Wv h (kv_heads x vdim)
    q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))          at position p
    s_m = cap((q_m . k_m) * scale),  cap(x) = softcap * tanh(x / softcap);  a_m = softmax(s_m) v
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff               one number for the layer
    o = a_1 - lambda a_2;  o <- o / sqrt(mean(o^2) + eps) * (1 - diff);  out = Wo [heads' o]

No rotation: positions enter through the query temperature only. Every
constant (scale, softcap, coef, every, diff) is a parameter; softcap 0 means
no cap and every 0 no temperature.

The cache keeps a token's two key vectors as one row of 2 dim elements per key
head, beside its value row, so one walk over the pages serves both maps: the
kernel carries two running softmaxes and loads every value row once.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..cache.store import KVRequest, KVView
from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_mixer
from .linear import Linear
from .products import product_f32, product_to_residual


@register_mixer("differential_attention")
class DifferentialAttention(Part):
    replay_safe = True
    accepts_row_scaled = True  # the first product applies a deferred norm's row scale

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, diff: float, softcap: float = 0.0, temp_coef: float = 0.0,
                 temp_every: int = 0, suffix: str = "", *, dtype: torch.dtype,
                 device: torch.device):
        if kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key-value heads")
        if not 1 <= 2 * dim <= 1024 or not 1 <= vdim <= 256:
            raise ValueError(f"key size 2 x {dim} (at most 1024) and value size {vdim} (at most 256)")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.eps, self.diff = float(scale), float(eps), float(diff)
        self.softcap, self.temp_coef, self.temp_every = float(softcap), float(temp_coef), int(temp_every)
        self.dtype, self.device = dtype, device
        self.nq, self.nk, self.nv = heads * 2 * dim, kv_heads * 2 * dim, kv_heads * vdim
        self.qkv = Linear(width, [("q", self.nq), ("k", self.nk), ("v", self.nv)], dtype=dtype,
                          device=device, suffix=suffix)
        self.o = Linear(heads * vdim, [("o", width)], dtype=dtype, device=device, suffix=suffix)
        self.lam = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        small = {f"{prefix}.{n}": ExpectedTensor((self.dim,)) for n in ("lq1", "lk1", "lq2", "lk2")}
        return {**self.qkv.expected_tensors(prefix), **self.o.expected_tensors(prefix), **small}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.qkv.load(prefix, fetch)
        self.o.load(prefix, fetch)
        # a constant of the loaded weights: worked out once, in 32-bit
        v = {n: fetch(f"{prefix}.{n}").to(torch.float32) for n in ("lq1", "lk1", "lq2", "lk2")}
        first = torch.exp((v["lq1"] * v["lk1"]).sum())
        second = torch.exp((v["lq2"] * v["lk2"]).sum())
        self.lam = float(first - second + torch.tensor(self.diff, dtype=torch.float32))

    def cache_request(self) -> KVRequest:
        return KVRequest(self.kv_heads, 2 * self.dim, None, self.vdim)

    def first_weight(self):
        return self.qkv.weight

    def context_flops(self, token_counts, starts) -> float:
        pairs = sum(0.5 * n * (2 * start + n + 1) for n, start in zip(token_counts, starts))
        return 2.0 * self.heads * 2 * (self.dim + self.vdim) * pairs

    def forward(self, ctx, x, cache: KVView):
        table = ctx.page_table(cache.group)
        qkv = product_f32(x, self.qkv.weight)
        q = torch.empty((x.shape[0], self.nq), dtype=x.dtype, device=x.device)
        ops.q_temp_cache_write(qkv, q, self.temp_coef, self.temp_every, ctx.positions,
                               ctx.seq_of_token, table, cache.k, cache.v, self.kv_heads,
                               2 * self.dim, self.vdim, write_cache=cache.writes)
        attn = torch.empty((x.shape[0], self.heads * self.vdim), dtype=x.dtype, device=x.device)
        ops.attention_sink(ctx, q, attn, table, cache.k, cache.v, self.heads, self.kv_heads,
                           self.dim, self.vdim, self.scale, softcap=self.softcap, maps=2,
                           combine=(self.lam, self.eps, 1.0 - self.diff))
        return product_to_residual(ctx, attn, self.o.weight)
