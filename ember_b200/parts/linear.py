"""A weight matrix [out, in] on the device and the product y = x . W^T with a fused epilogue.

The kernel is chosen by dtype and shape: the tcgen05 tensor-core kernel for bfloat16 weights
and activations whose sizes it takes, the fp32 SIMT kernel otherwise (always on the float32
path: that is the true 32-bit product).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight = weight            # [N, K], float32 or bfloat16, on the device
        self.bias = bias                # float32 [N] or None
        self.n, self.k = weight.shape
        if weight.is_cuda and weight.dtype == torch.bfloat16:
            # the small-M tensor-core product sums its K parts in a shared fp32 scratch of up to 128 x N: made
            # now, so that no step (least of all one inside a captured graph's lifetime) has to grow it
            ops.reserve_scratch(weight.device, 128 * self.n)

    @classmethod
    def from_host(cls, w: torch.Tensor, rt: Runtime, bias: Optional[torch.Tensor] = None) -> "Linear":
        dev = rt.to_device(w, rt.weight_dtype(w.dtype))
        b = rt.to_device(bias, torch.float32) if bias is not None else None
        return cls(dev, b)

    def __call__(self, ctx, x: torch.Tensor, out: torch.Tensor, m: int, epilogue: int = ops.EPI_STORE) -> None:
        if m <= 0:
            return
        if ops.gemm_tc_usable(x, self.weight, self.bias, epilogue):
            ops.gemm_tc(x, self.weight, out, m, epilogue, err=ctx.err, stream=ctx.stream)
        else:
            ops.gemm_simt(x, self.weight, out, m, epilogue, bias=self.bias, stream=ctx.stream)
