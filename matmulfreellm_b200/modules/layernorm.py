"""RMSNorm with the reference's module interface (mmfreelm/modules/layernorm.py:586-623)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import kernels

__all__ = ["RMSNorm", "rms_norm_fn"]


def rms_norm_fn(x, weight, bias, residual=None, eps=1e-6, prenorm=False, residual_in_fp32=False):
    """layernorm.py:534-543: y = rmsnorm(x [+ residual]) * weight; with prenorm also returns x + residual."""
    if bias is not None:
        raise NotImplementedError("RMSNorm bias is never used on the HGRNBit path")
    return kernels.rmsnorm(x, weight, eps, residual=residual, prenorm=prenorm, residual_in_fp32=residual_in_fp32)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-5):
        super().__init__()
        self.hidden_size = hidden_size
        self.elementwise_affine = elementwise_affine
        self.eps = eps
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(hidden_size))
        else:
            self.register_parameter("weight", None)
        self.register_parameter("bias", None)

    def __repr__(self) -> str:
        s = f"{self.__class__.__name__}({self.hidden_size}"
        if not self.elementwise_affine:
            s += f", elementwise_affine={self.elementwise_affine}"
        return s + f", eps={self.eps})"

    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        return rms_norm_fn(x, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm,
                           residual_in_fp32=residual_in_fp32)
