"""swiglu with the reference's call form (mmfreelm/modules/activations.py:178)."""
from .. import kernels

__all__ = ["swiglu"]


def swiglu(x, y):
    """x * sigmoid(x) * y computed in fp32 and returned in x.dtype (activations.py:115-119)."""
    return kernels.swiglu(x, y)
