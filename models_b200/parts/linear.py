"""Matrix products y = x . W^T for row-major W [out, in] (integrallis/models,
backend-java/.../ops/TensorOps.java:61-63), chosen by the weight's storage.

bfloat16 weights: with up to 8 activation rows (decode) this package's own weight-streaming kernel
(csrc/skinny_gemm.cu; it takes up to 32 rows but pays off up to 8); with 9 to 128 rows its tcgen05 kernel
with the weights as the 128-row operand and K split over a thread-block cluster
(csrc/wide_gemm_tcgen05.cu); with more rows (prefill) its tcgen05 kernel csrc/gemm_tcgen05.cu.  What is
left -- a matrix whose sizes are no multiples of 8, which TMA cannot address -- falls to a library product
(bfloat16 inputs, float accumulation), the place where the reference too calls a library (its matmul is
VectorUtil.batchDotProduct of an external artifact).
float32 weights: this package's own true-32-bit kernel, in both modes -- a matrix stored in 32-bit is
multiplied in 32-bit.
"""

from __future__ import annotations

import torch

from ..kernels import ops


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    if not x.is_cuda:
        raise ops.KernelError("models_b200 runs on a CUDA device only; there is no CPU path")
    if weight.dtype == torch.float32:
        a = x if x.dtype == torch.float32 else x.float()
        out = ops.gemm_f32(a, weight)
        return out if out_dtype == torch.float32 else out.to(out_dtype)
    if weight.dtype != torch.bfloat16:
        raise ops.KernelError(f"matrices are bfloat16 or float32, got {weight.dtype}")
    a = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if ops.skinny_pays(weight, a.shape[0]) and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 \
            and out_dtype in (torch.bfloat16, torch.float32):
        # decode: few rows, the weights stream once through this package's own kernel
        return ops.skinny_gemm(weight, ops.EPI_F32 if out_dtype == torch.float32 else ops.EPI_BF16, x=a)
    if (ops.gemm_tcgen05_takes(weight, rows=a.shape[0]) and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
            and out_dtype in (torch.bfloat16, torch.float32)):
        # many rows: this package's tcgen05 kernels (wide decode form up to 128 rows, prefill form above)
        return ops.tensor_core_gemm(a, weight, ops.EPI_F32 if out_dtype == torch.float32 else ops.EPI_BF16)
    if out_dtype == torch.float32:
        return torch.mm(a, weight.t(), out_dtype=torch.float32)
    return torch.mm(a, weight.t())
