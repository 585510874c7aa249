"""HGRN recurrence ops with the reference's signatures (mmfreelm/ops/hgrn/__init__.py:3-9)."""
from typing import Optional, Tuple

import torch

from ... import kernels

__all__ = ["chunk_hgrn", "fused_recurrent_hgrn"]


def _check(x, g):
    if x.dim() != 4 or x.shape != g.shape:
        raise AssertionError("x and g must both be [B, H, T, D]")


def fused_recurrent_hgrn(x: torch.Tensor, g: torch.Tensor, initial_state: Optional[torch.Tensor] = None,
                         output_final_state: bool = False,
                         state_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """h_t = g_t * h_{t-1} + x_t with the forget gate g in the LINEAR domain (0,1).

    Mirrors mmfreelm/ops/hgrn/recurrent_fuse.py:176-185: x, g are [B,H,T,D]; returns (o, final_state) with
    final_state [B,H,D] or None.  The state is carried in fp32 on the device; `state_dtype` chooses how the
    returned final state is stored (default: x.dtype, as the reference's `x.new_empty`, recurrent_fuse.py:145)."""
    _check(x, g)
    B, H, T, D = x.shape
    o, ht = kernels.hgrn_scan(x, g, initial_state, output_final_state, gate_is_log=False,
                              state_dtype=state_dtype or x.dtype)
    return o, ht


def chunk_hgrn(x: torch.Tensor, g: torch.Tensor, initial_state: Optional[torch.Tensor] = None,
               output_final_state: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Same recurrence with g the LOG forget gate: h_t = exp(g_t) * h_{t-1} + x_t.

    Mirrors mmfreelm/ops/hgrn/chunk.py:287-296; the final state is fp32 as there (chunk.py:233,251)."""
    _check(x, g)
    o, ht = kernels.hgrn_scan(x, g, initial_state, output_final_state, gate_is_log=True, state_dtype=torch.float32)
    return o, ht
