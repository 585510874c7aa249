from .fused_norm_gate import FusedRMSNormSwishGate
from .layernorm import RMSNorm

__all__ = ["RMSNorm", "FusedRMSNormSwishGate"]
