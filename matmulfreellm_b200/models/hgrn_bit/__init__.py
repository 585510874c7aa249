from transformers import AutoConfig, AutoModel, AutoModelForCausalLM

from .configuration_hgrn_bit import HGRNBitConfig
from .modeling_hgrn_bit import HGRNBitForCausalLM, HGRNBitModel

# same registrations as mmfreelm/models/hgrn_bit/__init__.py:8-10; tolerate a second registration
# (e.g. when the reference package is imported in the same process)
for _reg, _args in ((AutoConfig, (HGRNBitConfig.model_type, HGRNBitConfig)), (AutoModel, (HGRNBitConfig, HGRNBitModel)),
                    (AutoModelForCausalLM, (HGRNBitConfig, HGRNBitForCausalLM))):
    try:
        _reg.register(*_args)
    except ValueError:
        pass

__all__ = ["HGRNBitConfig", "HGRNBitForCausalLM", "HGRNBitModel"]
