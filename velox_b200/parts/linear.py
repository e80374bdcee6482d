"""y = x W^T (+ b) with W stored [out, in], as the reference's linears
(src/paged/qwen3.rs:120-132, 226-239).

The one place where a matrix product is chosen:
  float32   the engine's own multiply-add kernel on the CUDA cores: true 32-bit,
            every output element summed over k in ascending order, so a row's
            result does not depend on the rows beside it.
  bfloat16  the tensor-core product (see `matmul`).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


def matmul(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        return ops.gemm_nt_simt(x, weight, bias, out_dtype)
    return ops.gemm_bf16(x, weight, bias, out_dtype)


class Linear:
    """A weight [out, in] and an optional float32 bias, already on the device."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight, self.bias = weight, bias

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return matmul(x, self.weight, self.bias, out_dtype)
