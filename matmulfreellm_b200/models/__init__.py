from .hgrn_bit import HGRNBitConfig, HGRNBitForCausalLM, HGRNBitModel

__all__ = ["HGRNBitConfig", "HGRNBitForCausalLM", "HGRNBitModel"]
