"""Parts that rewrite the whole residual stream between two layer runs.

`loop_input` stands in front of every pass of a group of layers that runs
several times with the same weights:

    x <- W_in [x ; x0] + step[t]

x0 being the stream as the embedding left it and t the number of the pass;
W_in is [width, 2 width] with the columns of x first, `step` is [times, width].
The product reads the two streams side by side in the activation type and the
new stream is 32-bit like the old one.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, Registry
from .linear import matmul_nt

JUNCTIONS = Registry("junction")
register_junction = JUNCTIONS.register


@register_junction("loop_input")
class LoopInput(Part):
    replay_safe = True
    needs_embedding_output = True

    def __init__(self, width: int, times: int, weight_name: str = "in", step_name: str = "step", *,
                 dtype: torch.dtype, device: torch.device):
        self.width, self.times = width, times
        self.weight_name, self.step_name = weight_name, step_name
        self.dtype, self.device = dtype, device
        self.weight = self.step = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{self.weight_name}": ExpectedTensor((self.width, 2 * self.width)),
                f"{prefix}.{self.step_name}": ExpectedTensor((self.times, self.width))}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.weight = fetch(f"{prefix}.{self.weight_name}").contiguous()
        self.step = fetch(f"{prefix}.{self.step_name}").to(torch.float32).contiguous()

    def first_weight(self):
        return self.weight

    def forward(self, ctx, resid: torch.Tensor, delta, x0: torch.Tensor, number: int):
        """Rewrites `resid` in place from (resid + delta) and `x0`; returns the
        new un-added output (None)."""
        if not 0 <= number < self.times:
            raise ValueError(f"pass {number} of a loop of {self.times}")
        if isinstance(delta, ops.NormedDelta):
            delta = delta.settle(resid)
        elif delta is not None:
            delta = ops.NormedDelta(ops.plain(delta), None, None, 1.0).settle(resid)
        both = torch.empty((resid.shape[0], 2 * self.width), dtype=self.dtype, device=resid.device)
        ops.concat_cast(resid, x0, both)
        matmul_nt(both, self.weight, resid)
        ops.add_row_vector(resid, self.step[number])
        return None
