"""bfloat16 matrix products y = x · Wᵀ (+ bias) on the tensor cores.

The plain product of a part that does not fuse anything into it.  Up to ``ops.GEMV_MAX_ROWS`` rows go to this
library's weight-streaming kernel (csrc/gemv_bf16.cu); beyond that the route is cuBLASLt, called directly by the
library with the algorithm of every (rows, columns, depth, output type) kept after its first use (``mm_blas_gemm_nt``,
csrc/exec/core.cu: the product the step executor uses; the reference's bf16 library route is cuBLASLt too,
src/compute/cuda/GpuMatmul.cpp:786-884) and the bias in the library's epilogue; accumulation is fp32 inside
the product and the result is rounded once to the requested dtype.  ``torch.mm`` remains for what that call does not
take (a bias whose type is not the output's).  The products with fused epilogues (the decode
layer's, csrc/gemv_bf16.cu and csrc/gemm_skinny_tcgen05.cu; the prefill gate/up product, csrc/gemm_tcgen05.cu) are
called by the parts directly.
"""
from __future__ import annotations

from typing import Optional

import torch


USE_LIBRARY_CALL = True       # False: the products of more than a few rows go through torch.mm (tests compare the two)


def matmul_nt(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    from . import ops
    if ops.gemv_supported(x.shape[0], weight.shape[0], weight.shape[1]):
        return ops.gemv_bf16(x, weight, bias, out_dtype)          # a handful of rows: weight streaming
    if USE_LIBRARY_CALL and x.is_contiguous() and weight.is_contiguous() and out_dtype in (torch.float32, torch.bfloat16) \
            and (bias is None or (bias.dtype == out_dtype and bias.is_contiguous())):
        m, k = x.shape
        n = weight.shape[0]
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        if m == 0:
            return out
        ops.check(ops._lib.load().mm_blas_gemm_nt(x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                                                  out.data_ptr(), ops.dtype_code(out_dtype), m, n, k, ops._stream()), "blas_gemm_nt")
        return out
    if out_dtype == torch.float32:
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias.float()
        return y
    if bias is not None:
        return torch.addmm(bias.to(x.dtype), x, weight.t())
    return torch.mm(x, weight.t())
