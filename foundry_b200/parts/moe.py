"""A feed-forward of routed experts.

    z = W_router h + b   (32-bit);  the `top` experts with the largest z are chosen
    (the lower index among equals) and weighted by the softmax over the chosen z only
    expert:  g = min(W_gate h, limit);  u = clamp(W_up h, -limit, limit)
             y = W_down (g * sigmoid(alpha g) * (u + 1))
    out = sum over the chosen experts of weight * y

The experts' tensors are `<prefix>.e<i>.gate|up|down`, the router's
`<prefix>.router` and `<prefix>.router.b`; they are stacked at load time so
that a kernel reaches any expert by index. `limit` and `alpha` are parameters.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_feed_forward
from .products import product_f32


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    replay_safe = True

    def __init__(self, width: int, ff: int, experts: int, top: int, limit: float,
                 alpha: float = 1.702, *, dtype: torch.dtype, device: torch.device):
        if not 1 <= top <= min(experts, 32) or experts > 256:
            raise ValueError(f"{top} of {experts} experts: the router takes up to 256 experts and "
                             f"chooses up to 32")
        self.width, self.ff, self.experts, self.top = width, ff, experts, top
        self.limit, self.alpha = float(limit), float(alpha)
        self.dtype, self.device = dtype, device

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        out = {f"{prefix}.router": ExpectedTensor((self.experts, self.width)),
               f"{prefix}.router.b": ExpectedTensor((self.experts,))}
        for e in range(self.experts):
            out[f"{prefix}.e{e}.gate"] = ExpectedTensor((self.ff, self.width))
            out[f"{prefix}.e{e}.up"] = ExpectedTensor((self.ff, self.width))
            out[f"{prefix}.e{e}.down"] = ExpectedTensor((self.width, self.ff))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.router = fetch(f"{prefix}.router").contiguous()
        self.router_bias = fetch(f"{prefix}.router.b").to(torch.float32).contiguous()
        # [E, 2 ff, W]: an expert's gate rows, then its up rows;  [E, W, ff]
        self.gate_up = torch.stack([torch.cat([fetch(f"{prefix}.e{e}.gate"),
                                               fetch(f"{prefix}.e{e}.up")], 0)
                                    for e in range(self.experts)], 0).contiguous()
        self.down = torch.stack([fetch(f"{prefix}.e{e}.down") for e in range(self.experts)],
                                0).contiguous()

    def first_weight(self):
        return self.router

    def forward(self, ctx, x):
        T = x.shape[0]
        z = product_f32(x, self.router)
        chosen = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        ops.moe_route(z, self.router_bias, self.top, chosen, weights)
        out = torch.empty((T, self.width), dtype=torch.float32, device=x.device)
        return ops.moe_experts_rows(x, self.gate_up, self.down, chosen, weights, out, self.limit,
                                    self.alpha)
