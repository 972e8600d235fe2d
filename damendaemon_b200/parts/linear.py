"""Matrix products of the parts: one call that picks the kernel for the engine dtype."""
from __future__ import annotations

import torch

from .. import kernels


def linear(runtime, a, w, bias=None, residual=None, activation=None, out_dtype=None, out=None):
    """act(a @ w.T + bias) (+ residual). float32 engine: CUDA-core float32 kernel.
    bfloat16 engine: the tcgen05 tensor-core kernel, unless the runtime asks for 'simt' or the
    reduction width is no multiple of 8 (then the CUDA-core kernel with bfloat16 operands)."""
    if a.dtype == torch.float32 or runtime.gemm == "simt":
        return kernels.gemm_simt(a, w, bias, residual, activation, out_dtype, out)
    if a.shape[1] % 8 or a.stride(0) % 8 or w.stride(0) % 8:
        # TMA wants 16-byte rows; a reduction width that is no multiple of 8 runs on the CUDA cores instead
        return kernels.gemm_simt(a, w, bias, residual, activation, out_dtype or torch.bfloat16, out)
    return kernels.gemm_tcgen05(a, w, bias, residual, activation, out_dtype, out)
