"""HGRNBitConfig, field for field as mmfreelm/models/hgrn_bit/configuration_hgrn_bit.py:8-64."""
from typing import Optional

from transformers.configuration_utils import PretrainedConfig


class HGRNBitConfig(PretrainedConfig):
    model_type = "hgrn_bit"
    keys_to_ignore_at_inference = ["past_key_values"]

    def __init__(self, vocab_size: int = 32000, hidden_size: int = 2048, num_hidden_layers: int = 24,
                 attn_mode: str = "fused_recurrent", num_heads: Optional[int] = 1, expand_ratio: Optional[int] = 1,
                 use_short_conv: bool = False, conv_size: int = 4, share_conv_kernel: bool = True,
                 use_lower_bound: bool = True, hidden_ratio: Optional[int] = 4,
                 intermediate_size: Optional[int] = None, hidden_act: str = "swish",
                 max_position_embeddings: int = 2048, rms_norm_eps: float = 1e-6, use_cache: bool = True,
                 pad_token_id: int = None, bos_token_id: int = 1, eos_token_id: int = 2,
                 tie_word_embeddings: bool = False, initializer_range: float = 0.02,
                 fuse_cross_entropy: bool = True, **kwargs):
        for key, value in dict(vocab_size=vocab_size, max_position_embeddings=max_position_embeddings,
                               hidden_size=hidden_size, num_hidden_layers=num_hidden_layers, attn_mode=attn_mode,
                               num_heads=num_heads, expand_ratio=expand_ratio, use_short_conv=use_short_conv,
                               conv_size=conv_size, share_conv_kernel=share_conv_kernel,
                               use_lower_bound=use_lower_bound, hidden_ratio=hidden_ratio,
                               intermediate_size=intermediate_size, hidden_act=hidden_act, rms_norm_eps=rms_norm_eps,
                               use_cache=use_cache, initializer_range=initializer_range,
                               fuse_cross_entropy=fuse_cross_entropy).items():
            setattr(self, key, value)
        super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                         tie_word_embeddings=tie_word_embeddings, **kwargs)
