"""ctypes binding of libmmfree_b200.so (the C ABI declared in include/mmfree_b200.h).

There is no CPU or PyTorch fallback behind these bindings: if the shared library is
missing, or the device is not a B200-class GPU, the calls raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmmfree_b200.so"

F32, BF16, F16 = 0, 1, 2
KERNEL_AUTO, KERNEL_GEMV, KERNEL_MMA = 0, 1, 2
KERNEL_STREAM = 3   # Python-level selector: the mma.sync decode experiment (mmf_bitlinear_decode, experiments build only)
STREAM_MAX_M = 64
TILE_ROWS, TILE_K = 128, 64
ABSMEAN_PARTIALS = 1024
ABI_VERSION = 2

_ERR_NAMES = {
    -1: "MMF_ERR_BAD_ARG", -2: "MMF_ERR_BAD_SHAPE", -3: "MMF_ERR_ALIGN", -4: "MMF_ERR_CUDA",
    -5: "MMF_ERR_ARCH", -6: "MMF_ERR_WORKSPACE", -7: "MMF_ERR_TIMEOUT",
}

# name -> (restype, argtypes); must list every symbol include/mmfree_b200.h declares
PROTOTYPES = {
    "mmf_last_error": (c_char_p, []),
    "mmf_abi_version": (c_int, []),
    "mmf_check_device": (c_int, []),
    "mmf_absmean_f32": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "mmf_packed_bytes": (c_int64, [c_int64, c_int64]),
    "mmf_pack_ternary": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "mmf_unpack_ternary": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "mmf_act_quant": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
                              c_int64, c_int64, c_void_p]),
    "mmf_bitlinear_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "mmf_bitlinear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64,
                              c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int, c_void_p]),
    "mmf_bitlinear_gemv_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64,
                                          c_int64, c_int64, c_int64, c_void_p]),
    "mmf_int8_mma_peak": (c_int, [c_int, c_int, c_void_p, c_void_p]),
    "mmf_sync_probe": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "mmf_hgrn_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "mmf_hgrn_scan": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int64,
                              c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p]),
    "mmf_hgrn_status": (c_int, [c_void_p]),
    "mmf_hgrn_gated": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                               c_int64, c_void_p, c_int64, c_void_p]),
    "mmf_hgrn_gated_masked": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_int64, c_int64, c_void_p, c_int64, c_void_p]),
    "mmf_prenorm_quant": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_float, c_void_p,
                                  c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                  c_int64, c_int64, c_void_p]),
    "mmf_gatenorm_quant": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_float, c_void_p, c_float,
                                   c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "mmf_decode_mix": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p,
                               c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "mmf_decode_mix_masked": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float,
                                      c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "mmf_swiglu_quant": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                 c_int64, c_int64, c_void_p]),
    "mmf_rmsnorm": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int64,
                            c_int64, c_void_p]),
    "mmf_rmsnorm_swishgate": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int64, c_int64,
                                      c_void_p]),
    "mmf_swiglu": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64,
                           c_void_p]),
    "mmf_argmax_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "mmf_sample_top_p": (c_int, [c_void_p, c_int, c_int64, c_float, c_float, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "mmf_embedding": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
}


class MMFreeError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, code: int, text: str):
        self.code = code
        super().__init__(f"{fn} failed with {_ERR_NAMES.get(code, code)}: {text}")


_lib = None
EXPERIMENTS_LIB_PATH = LIB_PATH.with_name("libmmfree_b200_experiments.so")
_EXPERIMENT_PROTOTYPES = {
    "mmf_tuning": (c_int, [c_int, c_int]), "mmf_row_trace": (c_int, [c_void_p]),
    "mmf_repack_slabs": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "mmf_bitlinear_decode_fits": (c_int, [c_int64, c_int64]),
    "mmf_bitlinear_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64,
                                     c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
}


def _open(path: Path, prototypes) -> ctypes.CDLL:
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in prototypes.items():
        fn = getattr(lib, name)  # AttributeError here = header and library out of sync
        fn.restype = res
        fn.argtypes = args
    if lib.mmf_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{path.name} ABI {lib.mmf_abi_version()} != binding ABI {ABI_VERSION}")
    return lib


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach prototypes. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing. Build it with `python -m matmulfreellm_b200._build` "
            "(needs nvcc); there is no fallback implementation.")
    _lib = _open(LIB_PATH, PROTOTYPES)
    return _lib


class experiments_library:
    """Context manager for kernel experiments and the configuration-sweep tests: inside it every call of this module
    goes to libmmfree_b200_experiments.so (the same sources built with -DMMF_EXPERIMENTS), which also exports
    mmf_tuning; on exit all overrides are reset and the product library is current again."""

    KNOBS = 13
    _handle = None

    def __enter__(self):
        global _lib
        cls = experiments_library
        if cls._handle is None:
            if not EXPERIMENTS_LIB_PATH.exists():
                raise RuntimeError(f"{EXPERIMENTS_LIB_PATH} is missing: python -m matmulfreellm_b200._build")
            cls._handle = _open(EXPERIMENTS_LIB_PATH, {**PROTOTYPES, **_EXPERIMENT_PROTOTYPES})
        self._saved = load()
        _lib = cls._handle
        return cls._handle

    def __exit__(self, *exc):
        global _lib
        for k in range(self.KNOBS):
            experiments_library._handle.mmf_tuning(k, 0)
        _lib = self._saved
        return False


# kernels each entry point launches per successful call (for launch accounting in benchmarks)
_LAUNCHES = {"mmf_absmean_f32": 2}
launch_count = 0


def call(name: str, *args) -> None:
    """Invoke an int-returning entry point and raise MMFreeError on a negative status."""
    global launch_count
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise MMFreeError(name, rc, lib.mmf_last_error().decode(errors="replace"))
    launch_count += _LAUNCHES.get(name, 1)


_device_checked = set()


def require_device(index: int) -> None:
    """Fail loudly (once per device) unless `index` is a compute-capability-10.x GPU."""
    if index in _device_checked:
        return
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("matmulfreellm_b200 needs a CUDA device (B200, sm_100a); none is available")
    with torch.cuda.device(index):
        call("mmf_check_device")
    _device_checked.add(index)
