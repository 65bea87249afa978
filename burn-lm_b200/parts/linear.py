"""The matrix product y = x W^T of a weight stored [out, in], picked by the weight's dtype and the
number of tokens.

bfloat16 weights: steps of up to 16 tokens run this package's skinny kernel (weights streamed once,
tensor-core accumulation in fp32), which can also take the RMS norm in front of it and the gated
activation or the residual add behind it; for prompts the gated gate/up product runs this package's
tcgen05 kernel (accumulator in tensor memory, activation in the epilogue) and the plain products go
through the library product (cuBLAS via torch.mm), as the reference's engine uses its library's
`Linear` (crates/burn-lm-llama/src/nn/attention/mha.rs:124-126).  float32 weights go through this package's
own fp32 kernel, which has no reduced-precision mode: that is the 32-bit path, and also what a
layer stored in 32-bit inside a bfloat16 model gets.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K

SKINNY_TOKENS = 16        # the skinny kernel takes up to this many tokens
FUSED_NORM_TOKENS = 16    # ... and normalises them in its prologue (every block redoes it)
TENSOR_CORE_TOKENS = 128  # from this many tokens the gated product runs this package's tcgen05 kernel


@dataclass
class NormedStream:
    """An RMS norm not yet computed: rows of the fp32 residual stream, to be normalised with gamma.
    A consumer that can normalise on the fly takes it as it is; `materialize()` runs the norm."""
    resid: torch.Tensor
    gamma: torch.Tensor
    eps: float
    rows: Optional[torch.Tensor]
    dtype: torch.dtype

    @property
    def n_tokens(self) -> int:
        return self.rows.numel() if self.rows is not None else self.resid.shape[0]

    def materialize(self) -> torch.Tensor:
        out = torch.empty((self.n_tokens, self.resid.shape[1]), dtype=self.dtype, device=self.resid.device)
        K.add_rmsnorm(self.resid, None, self.gamma, self.eps, out, self.rows)
        return out


class Linear:
    def __init__(self, weight: torch.Tensor, gate_tile: int = 0):
        """gate_tile: for a fused gate/up weight, how its rows are laid out: 0 = all gate rows then all up
        rows; n = tiles of n gate rows followed by the n up rows of the same outputs."""
        if weight.dim() != 2:
            raise ValueError("a linear weight is [out, in]")
        self.weight = weight
        self.gate_tile = gate_tile
        self.out_features, self.in_features = weight.shape

    def _skinny(self, n_tokens: int, m: int) -> bool:
        w = self.weight
        return (w.dtype == torch.bfloat16 and w.is_cuda and n_tokens <= SKINNY_TOKENS
                and K.gemv_supported(n_tokens, m, self.in_features))

    @staticmethod
    def _tokens(x) -> int:
        return x.n_tokens if isinstance(x, NormedStream) else x.shape[0]

    def _source(self, x):
        """Keyword arguments that hand x (a tensor or a pending norm) to the skinny kernel."""
        if isinstance(x, NormedStream):
            if x.n_tokens <= FUSED_NORM_TOKENS:
                return dict(stream_rows=x.resid, gamma=x.gamma, eps=x.eps, rows=x.rows)
            x = x.materialize()
        if x.dtype != torch.bfloat16:
            xc = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
            K.convert(x, xc)
            x = xc
        return dict(x=x)

    def __call__(self, x, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        n = self._tokens(x)
        if self._skinny(n, self.out_features):
            out_dtype = out_dtype or torch.bfloat16
            if out_dtype in (torch.bfloat16, torch.float32):
                out = torch.empty((n, self.out_features), dtype=out_dtype, device=self.weight.device)
                K.gemv(self.weight, n, out=out, **self._source(x))
                return out
        if isinstance(x, NormedStream):
            x = x.materialize()
        return self._library(x, out_dtype or x.dtype)

    def into_stream(self, x, stream: Optional[torch.Tensor], out_dtype: torch.dtype):
        """The product added into the fp32 residual stream when the skinny kernel can do that itself
        (returns None); otherwise the product, for the next norm to add."""
        n = self._tokens(x)
        if stream is not None and self._skinny(n, self.out_features):
            K.gemv(self.weight, n, add_into=stream, **self._source(x))
            return None
        return self(x, out_dtype)

    def gated(self, x, out_dtype: torch.dtype) -> torch.Tensor:
        """silu(x Wgate^T) * (x Wup^T) for a fused [gate; up] weight."""
        n = self._tokens(x)
        inner = self.out_features // 2
        act = torch.empty((n, inner), dtype=out_dtype, device=self.weight.device)
        if out_dtype == torch.bfloat16 and self.gate_tile == K.GATE_TILE and self._skinny(n, inner):
            K.gemv(self.weight, n, out=act, swiglu=True, **self._source(x))
            return act
        if (out_dtype == torch.bfloat16 and self.gate_tile == K.GATE_TILE and self.weight.dtype == torch.bfloat16
                and n >= TENSOR_CORE_TOKENS and K.gemm_tc_supported(n, self.out_features, self.in_features)):
            # prompts: the tcgen05 product with the gated activation in its epilogue
            if isinstance(x, NormedStream):
                x = x.materialize()
            if x.dtype == torch.bfloat16 and x.is_contiguous():
                K.gemm_tc(x, self.weight, act, swiglu=True)
                return act
        K.swiglu(self(x, out_dtype), act, tile=self.gate_tile)
        return act

    def _library(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        w = self.weight
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
