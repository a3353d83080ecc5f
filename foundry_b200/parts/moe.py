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
from .linear import matmul_nt
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
        if not (ops.moe_grouped_fits(self.width) and ops.moe_grouped_fits(self.ff)):
            # sizes the grouped kernels do not take: every token streams its own experts
            return ops.moe_experts_rows(x, self.gate_up, self.down, chosen, weights, out,
                                        self.limit, self.alpha)
        order = ops.ExpertOrder(chosen, self.experts)
        if T >= self.LIBRARY_ROWS and getattr(ctx, "cu_tokens_host", None) is not None:
            y = self._per_expert_products(ops.moe_gather(x, order), order)
        elif ops.moe_grouped_mma_fits(x, self.width, self.ff):
            act = ops.moe_grouped_mma(x, self.gate_up, order, True, self.limit, self.alpha,
                                      by_token=True)
            y = ops.moe_grouped_mma(act, self.down, order, False)
        else:
            act = ops.moe_grouped(x, self.gate_up, order, True, self.limit, self.alpha,
                                  by_token=True)
            y = ops.moe_grouped(act, self.down, order, False)
        return ops.moe_combine(y, order, weights, out)

    # From this many tokens on, a step that is launched plainly (its context has the
    # host copies; such a step is never captured) runs every expert's rows through
    # the tensor-core products, which needs the experts' counts on the host.
    LIBRARY_ROWS = 128

    def _per_expert_products(self, rows, order):
        starts = order.starts.tolist()  # waits for the routing
        pairs, dev = order.pairs, rows.device
        gate_up = torch.empty((pairs, 2 * self.ff), dtype=torch.float32, device=dev)
        for e in range(self.experts):
            a, b = starts[e], starts[e + 1]
            if b > a:
                matmul_nt(rows[a:b], self.gate_up[e], gate_up[a:b])
        act = torch.empty((pairs, self.ff), dtype=rows.dtype, device=dev)
        ops.moe_glu(gate_up, act, order, self.limit, self.alpha)
        y = torch.empty((pairs, self.width), dtype=torch.float32, device=dev)
        for e in range(self.experts):
            a, b = starts[e], starts[e + 1]
            if b > a:
                matmul_nt(act[a:b], self.down[e], y[a:b])
        return y
