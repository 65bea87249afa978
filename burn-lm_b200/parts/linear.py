"""The matrix product y = x W^T of a weight stored [out, in], picked by the weight's dtype.

bfloat16 weights go through the library product (cuBLAS via torch.mm), as the reference's engine
uses its library's `Linear` (crates/burn-lm-llama/src/nn/attention/mha.rs:124-126).  float32
weights go through this package's own fp32 kernel, which has no reduced-precision mode: that is the
32-bit path, and also what a layer stored in 32-bit inside a bfloat16 model gets.
"""
from __future__ import annotations

import torch

from .. import kernels as K


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError("a linear weight is [out, in]")
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        w = self.weight
        out_dtype = out_dtype or x.dtype
        if w.dtype == torch.float32:
            xf = x
            if x.dtype != torch.float32:
                xf = torch.empty(x.shape, dtype=torch.float32, device=x.device)
                K.convert(x, xf)
            y = K.gemm_f32(xf, w)
            if out_dtype != torch.float32:
                yo = torch.empty(y.shape, dtype=out_dtype, device=y.device)
                K.convert(y, yo)
                return yo
            return y
        if x.dtype != w.dtype:
            xc = torch.empty(x.shape, dtype=w.dtype, device=x.device)
            K.convert(x, xc)
            x = xc
        if not x.is_cuda:
            raise K.KernelError("burn-lm_b200 runs on a CUDA device only")
        if out_dtype == w.dtype:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)
