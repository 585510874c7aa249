"""HGRNBitAttention: the gated-recurrence token mixer (mmfreelm/layers/hgrn_bit.py:22-162), default branch
(no short convolution)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import kernels
from ..modules import FusedRMSNormSwishGate
from ..modules.activations import swiglu
from ..ops.fusedbitnet import FusedBitLinear as BitLinear


class HGRNBitAttention(nn.Module):
    def __init__(self, mode: str = "fused_recurrent", hidden_size: int = 1024, num_heads: Optional[int] = None,
                 expand_ratio: Optional[int] = 1, use_short_conv: bool = False, conv_size: int = 4,
                 conv_bias: bool = False, share_conv_kernel: bool = True, layernorm_eps: float = 1e-5,
                 layer_idx: int = None):
        super().__init__()
        if mode != "fused_recurrent":
            raise AssertionError(f"Not supported mode `{mode}`.")
        if use_short_conv:
            raise NotImplementedError("use_short_conv=True is outside the inference hot path (off by default "
                                      "in HGRNBitConfig and unusable in the reference)")
        num_heads = num_heads or 1
        if hidden_size % num_heads:
            raise AssertionError(f"hidden size must be divisible by num_heads of {num_heads}")
        self.mode, self.hidden_size, self.num_heads, self.expand_ratio = mode, hidden_size, num_heads, expand_ratio
        self.input_dim = int(hidden_size * expand_ratio)
        self.head_dim = self.input_dim // num_heads
        self.use_short_conv, self.conv_size, self.conv_bias = use_short_conv, conv_size, conv_bias
        self.share_conv_kernel, self.layer_idx = share_conv_kernel, layer_idx

        self.i_proj = BitLinear(hidden_size, self.input_dim, bias=False)
        self.f_proj = BitLinear(hidden_size, self.input_dim, bias=False)
        self.g_proj = BitLinear(hidden_size, self.input_dim, bias=False)
        self.g_norm = FusedRMSNormSwishGate(self.input_dim, layernorm_eps)
        self.o_proj = BitLinear(self.input_dim, hidden_size, bias=False)
        for m in (self.i_proj, self.f_proj, self.g_proj, self.o_proj):   # hgrn_bit.py:74-81
            nn.init.xavier_uniform_(m.weight, gain=2 ** -2.5)

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                past_key_values=None, use_cache: Optional[bool] = False, output_attentions: Optional[bool] = False,
                lower_bound: Optional[torch.Tensor] = None, **kwargs):
        B, T, _ = hidden_states.shape
        last_state = past_key_values[self.layer_idx] if use_cache else None
        i = self.i_proj(hidden_states)
        f = self.f_proj(hidden_states).sigmoid()
        if lower_bound is not None and self.layer_idx > 0:          # first layer's bound is zero
            f = lower_bound + (1 - lower_bound) * f
        i = swiglu(i, 1 - f)
        if attention_mask is not None:                              # left padding
            i = i.mul_(attention_mask.unsqueeze(-1))
        # [B, T, H*D] -> independent (b, h) sequences; H == 1 by default so this is a view
        H, D = self.num_heads, self.head_dim
        if H == 1:
            xi, xf = i, f
        else:
            xi = i.view(B, T, H, D).transpose(1, 2).contiguous()
            xf = f.view(B, T, H, D).transpose(1, 2).contiguous()
        h0 = last_state[-1] if use_cache else None
        o, state = kernels.hgrn_scan(xi.view(B * H, T, D), xf.view(B * H, T, D), h0, bool(use_cache), gate_is_log=False,
                                     state_dtype=torch.float32)
        if H > 1:
            o = o.view(B, H, T, D).transpose(1, 2).reshape(B, T, H * D)
        else:
            o = o.view(B, T, D)
        if past_key_values is not None and use_cache:
            past_key_values.update((state.view(B, H, D),), self.layer_idx, T)
        o = self.g_norm(self.g_proj(hidden_states), o)
        return self.o_proj(o), None, past_key_values

    def init_state(self, batch_size: int) -> Tuple[torch.Tensor]:
        """Zero recurrent state [B, num_heads, head_dim]; kept in fp32 whatever the parameter dtype."""
        param = next(self.parameters())
        return (torch.zeros(batch_size, self.num_heads, self.head_dim, dtype=torch.float32, device=param.device),)

    def state_size(self, **kwargs) -> int:
        return self.hidden_size
