"""matmulfreellm_b200 — the MatMul-free LM inference hot path on NVIDIA B200 (sm_100a).

The package mirrors the import layout of the reference's `mmfreelm` package for the modules on
that path (ops.fusedbitnet, ops.hgrn, modules, layers, models), so that
`matmulfreellm_b200.install_as_mmfreelm()` makes `import mmfreelm...` resolve here.  All
arithmetic runs in hand-written CUDA behind the C ABI of libmmfree_b200.so; there is no
Triton, no backend dispatch and no CPU fallback.
"""
__version__ = "0.1"

_MIRRORED = ["", ".ops", ".ops.fusedbitnet", ".ops.hgrn", ".modules", ".modules.activations", ".modules.layernorm",
             ".modules.fused_norm_gate", ".layers", ".layers.hgrn_bit", ".models", ".models.utils",
             ".models.hgrn_bit", ".models.hgrn_bit.configuration_hgrn_bit", ".models.hgrn_bit.modeling_hgrn_bit"]


def install_as_mmfreelm() -> None:
    """Register this package under the name `mmfreelm` (and its mirrored submodules) in sys.modules."""
    import importlib
    import sys
    for suffix in _MIRRORED:
        sys.modules["mmfreelm" + suffix] = importlib.import_module(__name__ + suffix)


def __getattr__(name):
    if name in ("HGRNBitModel", "HGRNBitForCausalLM", "HGRNBitConfig"):
        from . import models
        return getattr(models, name)
    raise AttributeError(name)
