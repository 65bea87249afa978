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

import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K

SKINNY_TOKENS = 16        # the skinny kernel takes up to this many tokens
FUSED_NORM_TOKENS = 16    # ... and normalises them in its prologue (every block redoes it)
# BURN_LM_B200_SK_TOKENS=n: steps of more tokens than that, up to n (at most 128), run the tcgen05 product whose
# wide operand is the weight (kernels.gemm_sk: K cut over a cluster, sums met in distributed shared memory, the
# same fused ends as the skinny kernel).  Off by default (16): measured on the 1B shape at 64 tokens its products
# take 13 / 10 / 25 / 20 us (qkv / output / gate-up / down, with their fused ends) against 5.7 / 5.9 / 13.6 / 13.7 us
# for the library's, which more than eats what the four launches it saves a layer are worth (a batch-64 decode
# step: 1.52 ms against 1.14 ms).
SK_TOKENS = int(os.environ.get("BURN_LM_B200_SK_TOKENS", "16"))
# From this many tokens the gated product runs this package's tcgen05 kernel.  Measured inside CUDA graphs on
# the 1B shape (16,384 x 2,048 weight): with fewer tokens its 128 x 256 tiles fill the SMs unevenly and the
# library's product followed by the activation kernel is faster (384 tokens: 28 against 36 us; 1,024: 61
# against 60; 2,048: 119 against 103).
TENSOR_CORE_TOKENS = 1024
# BURN_LM_B200_OWN_PRODUCTS=1: the plain products of a prompt (qkv, output, down, head) run this package's
# tcgen05 kernel too, from 128 tokens, instead of the library, and the two that feed the residual stream add
# into it in their epilogue (fp32, in place).  Off by default: measured at 2,048 tokens they reach 0.88 (qkv),
# 0.83 (output) and 0.94 (down) of the library's speed, the whole prompt step takes 5.1 ms against 4.3 ms, and
# the adding epilogue does not win that back: output product + norm 37 us against 27 us for the library's product
# and the norm kernel that also adds, down 78 against 58 us (a thread of the epilogue owns a row of the tile, so
# its 64-byte reads and writes of the stream lie a row apart).
OWN_PRODUCTS = os.environ.get("BURN_LM_B200_OWN_PRODUCTS", "") == "1"
OWN_PRODUCTS_TOKENS = 128


@dataclass
class HandedNorm:
    """What the writer of the stream left for the norm that reads it next: `scaled` = bfloat16(stream * gamma)
    [N, width] and `squares` [parts, 16], the rows' sums of squares in parts.  Only the division by the root
    mean square is left, and that commutes with the product that follows."""
    scaled: torch.Tensor
    squares: torch.Tensor


class NormHandoff:
    """A step's letterbox between the part that adds into the residual stream last and the norm that reads
    the stream next.  The block says which norm comes next (`expect`); a product that can leaves the norm's
    input with its sum (`leave`); the norm picks it up (`claim`).  Nothing left, nothing claimed: the norm
    is computed from the stream as ever."""

    def __init__(self):
        self.wanted = None
        self.left = None

    def expect(self, norm) -> None:
        """`norm`: a part with `gamma` and `spec.eps` that can take a handed-over input, or None."""
        self.wanted = norm if getattr(norm, "takes_handed_norm", False) else None
        self.left = None

    def leave(self, stream, gamma, handed: HandedNorm) -> None:
        self.left = (stream, gamma, handed)

    def claim(self, stream, gamma) -> Optional[HandedNorm]:
        left, self.left, self.wanted = self.left, None, None
        if left is not None and left[0] is stream and left[1] is gamma:
            return left[2]
        return None


@dataclass
class NormedStream:
    """An RMS norm not yet computed: rows of the fp32 residual stream, to be normalised with gamma.
    A consumer that can normalise on the fly takes it as it is; `materialize()` runs the norm."""
    resid: torch.Tensor
    gamma: torch.Tensor
    eps: float
    rows: Optional[torch.Tensor]
    dtype: torch.dtype
    handed: Optional[HandedNorm] = None

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

    def _skinny(self, n_tokens: int, m: int, x=None) -> bool:
        w = self.weight
        plain = isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16
        return (w.dtype == torch.bfloat16 and w.is_cuda and n_tokens <= SKINNY_TOKENS
                and K.gemv_supported(n_tokens, m, self.in_features, plain_tokens=plain))

    def _sk(self, n_tokens: int) -> bool:
        """Whether the step runs kernels.gemm_sk (asked after _skinny has said no)."""
        w = self.weight
        return (w.dtype == torch.bfloat16 and w.is_cuda and w.is_contiguous() and n_tokens <= min(SK_TOKENS, K.SK_TOKENS)
                and K.gemm_sk_supported(n_tokens, self.out_features, self.in_features))

    @staticmethod
    def _sk_source(x):
        """Keyword arguments that hand x (a tensor or a pending norm) to gemm_sk: dense bfloat16 rows, or a norm
        that the writer of the stream handed over in gemm_sk's layout."""
        if isinstance(x, NormedStream):
            h = x.handed
            if h is not None and x.rows is None and h.squares.shape[1] == K.SK_SQUARES_ROWS:
                return dict(x=h.scaled, squares=h.squares, eps=x.eps)
            x = x.materialize()
        if x.dtype != torch.bfloat16:
            xc = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
            K.convert(x, xc)
            x = xc
        return dict(x=x if x.is_contiguous() else x.contiguous())

    @staticmethod
    def _tokens(x) -> int:
        return x.n_tokens if isinstance(x, NormedStream) else x.shape[0]

    def _source(self, x):
        """Keyword arguments that hand x (a tensor or a pending norm) to the skinny kernel."""
        if isinstance(x, NormedStream):
            if x.handed is not None and x.n_tokens <= SKINNY_TOKENS and x.handed.squares.shape[1] == K.SQUARES_ROWS:
                return dict(x=x.handed.scaled, squares=x.handed.squares, eps=x.eps, rows=x.rows)
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
        if self._skinny(n, self.out_features, x):
            out_dtype = out_dtype or torch.bfloat16
            if out_dtype in (torch.bfloat16, torch.float32):
                out = torch.empty((n, self.out_features), dtype=out_dtype, device=self.weight.device)
                K.gemv(self.weight, n, out=out, **self._source(x))
                return out
        elif self._sk(n) and (out_dtype or torch.bfloat16) in (torch.bfloat16, torch.float32):
            out = torch.empty((n, self.out_features), dtype=out_dtype or torch.bfloat16, device=self.weight.device)
            K.gemm_sk(self.weight, out=out, **self._sk_source(x))
            return out
        if isinstance(x, NormedStream):
            x = x.materialize()
        return self._library(x, out_dtype or x.dtype)

    def into_stream(self, x, stream: Optional[torch.Tensor], out_dtype: torch.dtype, handoff: Optional[NormHandoff] = None):
        """The product added into the fp32 residual stream when the skinny kernel can do that itself
        (returns None); otherwise the product, for the next norm to add.  With a `handoff` that expects a
        norm, the kernel also leaves that norm's input there."""
        n = self._tokens(x)
        if stream is not None and self._skinny(n, self.out_features, x):
            hand_over = None
            norm = handoff.wanted if handoff is not None else None
            if norm is not None and n <= K.SQUARES_ROWS and norm.gamma.numel() == self.out_features:
                handed = HandedNorm(torch.empty((n, self.out_features), dtype=torch.bfloat16, device=stream.device),
                                    torch.empty(((self.out_features + 15) // 16, K.SQUARES_ROWS), dtype=torch.float32,
                                                device=stream.device))
                hand_over = (norm.gamma, handed.scaled, handed.squares)
            K.gemv(self.weight, n, add_into=stream, hand_over=hand_over, **self._source(x))
            if hand_over is not None:
                handoff.leave(stream, norm.gamma, handed)
            return None
        if stream is not None and self._sk(n):
            hand_over = None
            norm = handoff.wanted if handoff is not None else None
            if norm is not None and n <= K.SK_SQUARES_ROWS and norm.gamma.numel() == self.out_features:
                handed = HandedNorm(torch.empty((n, self.out_features), dtype=torch.bfloat16, device=stream.device),
                                    torch.empty(((self.out_features + 15) // 16, K.SK_SQUARES_ROWS), dtype=torch.float32,
                                                device=stream.device))
                hand_over = (norm.gamma, handed.scaled, handed.squares)
            K.gemm_sk(self.weight, add_into=stream, hand_over=hand_over, **self._sk_source(x))
            if hand_over is not None:
                handoff.leave(stream, norm.gamma, handed)
            return None
        if (OWN_PRODUCTS and stream is not None and self.weight.dtype == torch.bfloat16 and n >= OWN_PRODUCTS_TOKENS
                and K.gemm_tc_supported(n, self.out_features, self.in_features)):
            if isinstance(x, NormedStream):
                x = x.materialize()
            if x.dtype == torch.bfloat16 and x.is_contiguous() and tuple(stream.shape) == (n, self.out_features) and stream.is_contiguous():
                K.gemm_tc(x, self.weight, add_into=stream)        # prompts: the tcgen05 product adds into the stream itself
                return None
        return self(x, out_dtype)

    def with_rotary(self, x, q_out: torch.Tensor, rope: dict) -> str:
        """For a [q; k; v] weight whose q and k rows are in kernels.tiled_pair_order(): when one of this package's
        skinny products takes the step, it rotates q and k and appends k and v to the cache in its epilogue, writes q
        to `q_out`, and this returns which one did ("skinny": kernels.gemv, "cluster": kernels.gemm_sk); else nothing
        is done and "" comes back."""
        n = self._tokens(x)
        if q_out.dtype != torch.bfloat16:
            return ""
        if self._skinny(n, self.out_features, x):
            K.gemv(self.weight, n, out=q_out, rope=rope, **self._source(x))
            return "skinny"
        if self._sk(n):
            K.gemm_sk(self.weight, out=q_out, rope=rope, **self._sk_source(x))
            return "cluster"
        return ""

    def gated(self, x, out_dtype: torch.dtype) -> torch.Tensor:
        """silu(x Wgate^T) * (x Wup^T) for a fused [gate; up] weight."""
        n = self._tokens(x)
        inner = self.out_features // 2
        act = torch.empty((n, inner), dtype=out_dtype, device=self.weight.device)
        if out_dtype == torch.bfloat16 and self.gate_tile == K.GATE_TILE and self._skinny(n, inner, x):
            K.gemv(self.weight, n, out=act, swiglu=True, **self._source(x))
            return act
        if out_dtype == torch.bfloat16 and self.gate_tile == K.GATE_TILE and self._sk(n):
            K.gemm_sk(self.weight, out=act, swiglu=True, **self._sk_source(x))
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
        if (OWN_PRODUCTS and w.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and x.shape[0] >= OWN_PRODUCTS_TOKENS
                and x.is_contiguous() and K.gemm_tc_supported(x.shape[0], w.shape[0], w.shape[1])):
            y = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
            K.gemm_tc(x, w, y)
            return y
        if out_dtype == w.dtype:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)
