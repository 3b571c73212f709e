"""Matrix products of the parts: ``out = epilogue(x . w^T)``.

One function, so that which kernel runs is decided in one place.  float32
always takes the CUDA-core kernel (true 32-bit).  bfloat16 takes the tcgen05
tensor-core kernel when the shapes meet its alignment rules and the CUDA-core
kernel otherwise; ``ctx.options["gemm"] = "plain"`` forces the latter.
"""
from __future__ import annotations

import torch

from .. import kernels as K

EPI_STORE, EPI_F32, EPI_ADD, EPI_SWIGLU = K.EPI_STORE, K.EPI_F32, K.EPI_ADD, K.EPI_SWIGLU


def matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, ctx) -> None:
    if w.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain":
        fast = getattr(K, "gemm_tc", None)
        if fast is not None and K.gemm_tc_accepts(x, w, out, epi):
            fast(x, w, out, epi, ctx.stream, ordered=bool(ctx.options.get("reproducible", False)))
            return
    K.gemm_simt(x, w, out, epi, ctx.stream)
