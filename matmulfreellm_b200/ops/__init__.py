from .hgrn import chunk_hgrn, fused_recurrent_hgrn

__all__ = ["fused_recurrent_hgrn", "chunk_hgrn"]
