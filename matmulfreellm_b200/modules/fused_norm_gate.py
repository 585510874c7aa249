"""FusedRMSNormSwishGate with the reference's interface (mmfreelm/modules/fused_norm_gate.py:514-536)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import kernels

__all__ = ["FusedRMSNormSwishGate", "rms_norm_fn"]


def rms_norm_fn(x, o, weight, bias, residual=None, prenorm=False, residual_in_fp32=False, eps=1e-6):
    """fused_norm_gate.py:510-511: y = rmsnorm(x) * weight * o * sigmoid(o)."""
    if bias is not None or residual is not None or prenorm:
        raise NotImplementedError("only the plain gated form used by HGRNBitAttention is provided")
    return kernels.rmsnorm_swishgate(x, o, weight, eps)


class FusedRMSNormSwishGate(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.register_parameter("bias", None)

    def reset_parameters(self):
        nn.init.ones_(self.weight)

    def forward(self, x, o, residual=None, prenorm=False, residual_in_fp32=False):
        return rms_norm_fn(x, o, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm,
                           residual_in_fp32=residual_in_fp32)
