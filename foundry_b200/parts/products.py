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
        return ops.gemm_simt(x, w, out)
    y = matmul_nt(x, w, out)
    return y if isinstance(y, torch.Tensor) else out
