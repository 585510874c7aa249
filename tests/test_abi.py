"""CPU-side checks of the C-ABI shared library: it builds, loads, exports every symbol the header declares,
and validates its arguments before touching a device.  No GPU needed (nvcc cross-compiles)."""
import ctypes
import re
from pathlib import Path

import pytest

from matmulfreellm_b200 import _build, _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "mmfree_b200.h"


@pytest.fixture(scope="module")
def lib():
    _build.build_library()
    return _lib.load()


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"\b(mmf_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.PROTOTYPES, f"{name} has no ctypes prototype"
    assert sorted(_lib.PROTOTYPES) == names


def test_abi_version_and_constants(lib):
    assert lib.mmf_abi_version() == _lib.ABI_VERSION
    text = HEADER.read_text()
    assert f"#define MMF_ABI_VERSION {_lib.ABI_VERSION}" in text
    assert f"#define MMF_TILE_ROWS {_lib.TILE_ROWS}" in text and f"#define MMF_TILE_K {_lib.TILE_K}" in text
    assert lib.mmf_packed_bytes(128, 64) == 128 * 16
    assert lib.mmf_packed_bytes(200, 192) == 2 * 3 * 128 * 16
    assert lib.mmf_packed_bytes(128, 100) == 0          # K must be a multiple of 64
    assert lib.mmf_hgrn_workspace_bytes(8, 2048, 2048) == 0
    assert lib.mmf_hgrn_workspace_bytes(1, 8192, 128) > 0
    assert lib.mmf_bitlinear_workspace_bytes(1, 2048, 2048) % 256 == 0


def test_argument_validation_needs_no_device(lib):
    """Bad arguments are rejected on the host with a status code and a message (no CUDA call is made)."""
    with pytest.raises(_lib.MMFreeError) as e:
        _lib.call("mmf_act_quant", None, 1, 64, None, 1, 1e-6, None, None, None, 1, 64, None)
    assert e.value.code == -1 and "null" in str(e.value)
    buf = (ctypes.c_char * 4096)()
    p = (ctypes.addressof(buf) + 15) & ~15
    with pytest.raises(_lib.MMFreeError) as e:   # K not a multiple of 16
        _lib.call("mmf_act_quant", p, 1, 40, None, 1, 1e-6, p, p, p, 1, 40, None)
    assert e.value.code == -2
    with pytest.raises(_lib.MMFreeError) as e:   # misaligned x
        _lib.call("mmf_act_quant", p + 2, 1, 64, None, 1, 1e-6, p, p, p, 1, 64, None)
    assert e.value.code == -3
    with pytest.raises(_lib.MMFreeError) as e:   # unknown dtype
        _lib.call("mmf_rmsnorm", p, 7, None, 7, None, 1e-6, p, None, 1, 64, None)
    assert e.value.code == -1
    with pytest.raises(_lib.MMFreeError) as e:   # K % 64 != 0
        _lib.call("mmf_pack_ternary", p, 128, 96, p, p, None)
    assert e.value.code == -2
    with pytest.raises(_lib.MMFreeError) as e:   # groups must split N into multiples of 128
        _lib.call("mmf_bitlinear", p, p, p, p, p, 3, p, 1, 300, None, 1, 300, 64, None, 0, 0, None)
    assert e.value.code == -2
    with pytest.raises(_lib.MMFreeError) as e:   # D % 8
        _lib.call("mmf_hgrn_scan", p, 1, p, 1, None, None, 0, p, 1, 4, 12, 0, None, 0, None)
    assert e.value.code == -2
    # empty problems are accepted without a launch
    _lib.call("mmf_act_quant", p, 1, 64, None, 1, 1e-6, p, p, p, 0, 64, None)
    _lib.call("mmf_hgrn_scan", p, 1, p, 1, None, None, 0, p, 0, 4, 16, 0, None, 0, None)


def test_cpu_tensors_are_refused():
    import torch
    from matmulfreellm_b200 import kernels
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernels.rmsnorm(torch.zeros(2, 64), torch.ones(64), 1e-6)


def test_kernels_refuse_tensors_of_another_device(monkeypatch):
    """The C entry points launch on the current CUDA device; tensors that live on another GPU must be refused before
    anything is launched (checked with stand-in tensor objects: no GPU needed)."""
    import types

    import pytest
    import torch

    from matmulfreellm_b200 import _lib, kernels
    monkeypatch.setattr(kernels, "_raw_device", lambda: 0)
    monkeypatch.setattr(_lib, "require_device", lambda idx: None)
    t0 = types.SimpleNamespace(is_cuda=True, device=torch.device("cuda", 0))
    t1 = types.SimpleNamespace(is_cuda=True, device=torch.device("cuda", 1))
    cpu = types.SimpleNamespace(is_cuda=False, device=torch.device("cpu"))
    assert kernels._need_cuda(t0, None, t0) == torch.device("cuda", 0)
    with pytest.raises(RuntimeError, match="current device is cuda:0"):
        kernels._need_cuda(t1)
    with pytest.raises(RuntimeError, match="different devices"):
        kernels._need_cuda(t0, t1)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernels._need_cuda(cpu)
