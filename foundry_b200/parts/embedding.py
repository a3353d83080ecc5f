"""From token ids to the first residual rows.

`lookup` is the plain table gather (src/nn/linear.rs:54-69). `scaled_sinusoidal`
multiplies the table row by a constant and adds a sinusoidal position vector:

    x[2i] = E[token][2i] * scale + sin(p * base^(-2i / width)),  x[2i+1] = ... + cos(same)

with p the token's own position (from 0 in each sequence). The frequencies are
held in double precision and the angle is their double-precision product with
the position, so the vector is exact to 32 bits however far the sequence runs.
The table itself belongs to the model (it may also be the output head); a part
here only says how a row becomes the stream.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..kernels import ops
from .base import Part, Registry

EMBEDDINGS = Registry("embedding")
register_embedding = EMBEDDINGS.register


@register_embedding("lookup")
class Lookup(Part):
    replay_safe = True

    def __init__(self, *, dtype: torch.dtype, device: torch.device):
        self.dtype, self.device = dtype, device

    def forward(self, ctx, table: torch.Tensor, out: torch.Tensor,
                copy: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops.embed_gather(table, ctx.token_ids, out)
        if copy is not None:
            copy.copy_(out)
        return out


@register_embedding("scaled_sinusoidal")
class ScaledSinusoidal(Part):
    replay_safe = True

    def __init__(self, width: int, scale: float, base: float = 10000.0, *, dtype: torch.dtype,
                 device: torch.device):
        if width % 2:
            raise ValueError(f"a sinusoidal position vector needs an even width, not {width}")
        self.width, self.scale, self.base = width, float(scale), float(base)
        self.dtype, self.device = dtype, device
        freq = np.power(np.float64(base), -2.0 * np.arange(width // 2, dtype=np.float64) / width)
        self.freq = torch.from_numpy(freq).to(device)

    def forward(self, ctx, table: torch.Tensor, out: torch.Tensor,
                copy: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.embed_sinusoid(table, ctx.token_ids, ctx.positions, self.freq, self.scale, out,
                                  copy)
