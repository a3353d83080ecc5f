"""A product whose result feeds 32-bit arithmetic: float32 out, any shape."""
from __future__ import annotations

import torch

from ..kernels import ops
from .linear import matmul_nt

SMALL_K = 64  # below one K block of the tensor-core products the CUDA-core product runs


def product_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, K] @ w [N, K]^T accumulated and returned in float32. The operands
    are in the run's element type (bfloat16 products round nothing but their
    inputs). Low-rank projections (K below a tensor-core K block) and views
    that TMA cannot address take the CUDA-core product."""
    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
    if x.shape[0] == 0:
        return out
    if x.dtype == torch.float32 or x.shape[1] < SMALL_K:
        return ops.gemm_simt(ops.plain(x), w, out)
    y = matmul_nt(x, w, out)
    return y if isinstance(y, torch.Tensor) else out


def product_to_residual(ctx, x: torch.Tensor, w: torch.Tensor):
    """A part's last product, whose result joins the residual: float32 as
    `product_f32` gives it, or, where the block offers the next norm's sink
    (`ctx.residual_sink`, single-token steps in bfloat16), the sum and the norm's
    preparation made in the product's epilogue (an `ops.NormPending` comes back)."""
    sink = getattr(ctx, "residual_sink", None)
    if sink is None or x.dtype == torch.float32 or x.shape[1] < SMALL_K or x.shape[0] == 0:
        return product_f32(x, w)
    return matmul_nt(x, w, out_dtype=torch.float32, residual=sink,
                     then_reads=getattr(ctx, "reads_after_part", None))
