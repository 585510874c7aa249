"""BitLinear / FusedBitLinear with the reference's interface (mmfreelm/ops/fusedbitnet.py).

The reference fake-quantises in floating point on every call; here the weight is ternarised and 2-bit
packed once ("offline") from the fp32 latent weight and each forward runs RMSNorm + int8 quantisation and
an integer contraction on the GPU.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import kernels
from ..modules.layernorm import RMSNorm

__all__ = ["activation_quant", "weight_quant", "BitLinear", "FusedBitLinear", "layer_norm_linear_quant_fn"]


def activation_quant(x: torch.Tensor) -> torch.Tensor:
    """Per-token int8 absmax fake quantisation (fusedbitnet.py:15-29): returns the dequantised tensor."""
    shape = x.shape
    q, dq, _ = kernels.act_quant(x.reshape(-1, shape[-1]).contiguous(), None, 0.0, use_norm=False)
    return (q.float() * dq[:, None]).to(x.dtype).reshape(shape)


def weight_quant(w: torch.Tensor) -> torch.Tensor:
    """Per-tensor absmean ternary fake quantisation (fusedbitnet.py:32-46): returns codes * mean|w|.
    Needs in_features % 64 == 0 (the packed layout's chunk size)."""
    pw = kernels.pack_weight(w)
    return (kernels.unpack_codes(pw).float() * pw.scale).to(w.dtype)


class BitLinear(nn.Linear):
    """nn.Linear whose forward is RMSNorm -> int8 activation codes -> ternary-weight contraction.

    Same constructor, parameters (`weight [N,K]`, `norm.weight [K]`) and state-dict keys as
    fusedbitnet.py:539-581.  `eps` of the fused RMSNorm is 1e-8 as in BitLinear (its `self.norm`)."""
    NORM_EPS = 1e-8

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__(in_features, out_features, bias=bias)
        self.norm = RMSNorm(in_features, eps=1e-8)
        self._packed: Optional[kernels.PackedWeight] = None
        self._packed_from = None    # (parameter object, its _version, its dtype, packed by an explicit call) at pack time
        self._norm_w32: Optional[torch.Tensor] = None
        self._norm_version = None

    # -- offline packing -------------------------------------------------------------------------
    def _pack(self, explicit: bool) -> kernels.PackedWeight:
        w = self.weight
        self._packed = kernels.pack_weight(w)
        self._packed_from = (w, w._version, w.dtype, explicit)
        return self._packed

    def pack_weights(self) -> kernels.PackedWeight:
        """(Re)build the 2-bit packed weight from the current latent weight. Called lazily by forward; call it
        yourself before casting the module to half precision so the codes come from the fp32 weights."""
        return self._pack(explicit=True)

    def packed(self) -> kernels.PackedWeight:
        """The packed weight that matches the CURRENT latent weight.  The reference re-ternarises on every forward
        (fusedbitnet.py:456); here the codes are rebuilt whenever the weight was replaced or modified in place
        (load_state_dict, weight.mul_, re-initialisation) since they were made.  A dtype cast alone (.half(),
        .bfloat16()) keeps codes that pack_weights() made from the higher-precision weight; codes packed lazily by
        a forward are rebuilt from the cast weight, which is what the reference would ternarise.  A module loaded
        from a packed checkpoint has no latent weight (numel 0) and keeps its codes."""
        w = self.weight
        if self._packed is None:
            return self._pack(explicit=False)
        if w.numel() == 0 or self._packed_from is None:
            if self._packed.device != w.device:
                self._packed = self._moved(w.device)
            return self._packed
        src, version, dtype, explicit = self._packed_from
        if src is not w or w._version != version or (w.dtype != dtype and not explicit):
            return self._pack(explicit=False)
        if self._packed.device != w.device:     # the module moved: the codes move with it
            self._packed = self._moved(w.device)
        return self._packed

    def _moved(self, device) -> kernels.PackedWeight:
        p = self._packed
        return kernels.PackedWeight(p.packed.to(device), p.scale.to(device), p.N, p.K, p.groups,
                                    None if p.slabs is None else p.slabs.to(device))

    def norm_weight_f32(self) -> torch.Tensor:
        w = self.norm.weight
        key = (w._version, w.data_ptr())
        if self._norm_w32 is None or self._norm_version != key:
            self._norm_w32 = w.detach().float().contiguous()
            self._norm_version = key
        return self._norm_w32

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        pw = self.packed()
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        q, dq, rs = kernels.act_quant(x2, self.norm_weight_f32(), self.NORM_EPS)
        y = kernels.bitlinear(q, dq, rs, pw, x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*shape[:-1], self.out_features)


class FusedBitLinear(BitLinear):
    """As BitLinear, with eps = 1e-6: the reference's fused call does not forward the module's eps, so the
    default of layer_norm_linear_quant_fn applies (fusedbitnet.py:520, :603-610)."""
    NORM_EPS = 1e-6


def layer_norm_linear_quant_fn(x, norm_weight, norm_bias, linear_weight, linear_bias, residual=None, eps=1e-6,
                               prenorm=False, residual_in_fp32=False, is_rms_norm=False):
    """Functional form (fusedbitnet.py:513-536), RMS branch without residual only — the combination the
    model uses.  The weight is ternarised and packed on every call, as the reference does."""
    if not is_rms_norm or norm_bias is not None or residual is not None or prenorm:
        raise NotImplementedError("only the RMSNorm, no-residual form used by FusedBitLinear is provided")
    pw = kernels.pack_weight(linear_weight)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).contiguous()
    q, dq, rs = kernels.act_quant(x2, None if norm_weight is None else norm_weight.detach().float().contiguous(), eps)
    y = kernels.bitlinear(q, dq, rs, pw, x.dtype)
    if linear_bias is not None:
        y = y + linear_bias.to(y.dtype)
    return y.reshape(*shape[:-1], linear_weight.shape[0])
