from .hgrn_bit import HGRNBitAttention

__all__ = ["HGRNBitAttention"]
