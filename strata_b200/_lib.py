"""ctypes binding of libstrata_b200.so (the C ABI declared in include/strata_b200.h).

There is no CPU or eager fallback: if the library is missing or an entry point reports an
error, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p, POINTER, Structure
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libstrata_b200.so"
_lib = None


class StrataLibraryError(RuntimeError):
    pass


class BlockWeights(Structure):
    """struct strata_block_weights (device pointers)."""
    _fields_ = [(n, c_void_p) for n in ("w_qkv", "b_qkv", "w_proj", "b_proj", "w_gate", "b_gate",
                                        "w_fc1", "b_fc1", "w_fc2", "b_fc2")]


_SIGNATURES = {
    "strata_abi_version": (c_int, []),
    "strata_error_string": (c_char_p, [c_int]),
    "strata_device_status": (c_int, [POINTER(c_int), c_int]),
    "strata_layernorm_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_float,
                                      c_void_p]),
    "strata_linear_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                   c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                   c_void_p]),
    "strata_qkv_rope_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                     c_int64, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                     c_int, c_float, c_void_p]),
    "strata_na3d_fwd_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                     c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_int, c_float, c_void_p]),
    "strata_block_workspace_bytes": (c_int64, [c_int64, c_int, c_int]),
    "strata_block_forward_bf16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_int, c_int, POINTER(BlockWeights),
                                          c_void_p, c_int, c_float, c_float, c_void_p,
                                          c_int64, c_void_p]),
    "strata_halo_gather_tokens_bf16": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                               c_void_p]),
    "strata_halo_gather_fields_f32": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_void_p, c_void_p,
                                              c_int, c_int, c_int, c_int64, c_void_p]),
    "strata_halo_gather_kv_bf16": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_int64, c_void_p]),
    "strata_qkv_rope_padded_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                            c_int64, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                            c_int, c_float, c_int, c_int, c_int, c_void_p]),
    "strata_na3d_fwd_region_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                            c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                            c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                            c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "strata_halo_gather_knn_fields_f32": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_void_p, c_void_p,
                                                  c_int, c_int, c_int, c_int, c_int64, c_void_p]),
    "strata_halo_adjoint_fields_f32": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                               c_int64, c_void_p]),
    "strata_preprocess_patches_bf16": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                               c_int, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "strata_postprocess_fields_f32": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                              c_int, c_int, c_int, c_void_p, c_void_p]),
    "strata_adaln_rows_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                       c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p,
                                       c_int64, c_int, c_int, c_float, c_void_p]),
    "strata_qk_norm_rows_bf16": (c_int, [c_void_p, c_int64, c_int64, c_int, c_float, c_void_p]),
    "strata_adaln_cond_bf16": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p,
                                       c_void_p, c_void_p]),
    "strata_adaln_cond_table_floats": (c_int64, [c_int, c_int, c_int]),
    "strata_dealias_patches_bf16": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                            c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int64,
                                            c_void_p]),
    "strata_halo_barrier": (c_int, [POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p]),
    "strata_ipc_alloc": (c_int, [c_int64, POINTER(c_void_p), c_void_p]),
    "strata_ipc_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "strata_ipc_close": (c_int, [c_void_p]),
    "strata_ipc_free": (c_int, [c_void_p]),
    "strata_block_forward_static_scratch_bf16": (c_int, [
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
        POINTER(BlockWeights), c_void_p, c_int, c_float, c_float, c_void_p]),
}


def lib_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise StrataLibraryError(
            f"{_LIB_PATH} is missing: build it with `python -m strata_b200.build` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def exported_names() -> list[str]:
    return sorted(_SIGNATURES)


def check(code: int, what: str) -> None:
    """Raise for a non-zero return code of an entry point."""
    if code == 0:
        return
    msg = load().strata_error_string(code).decode()
    if code in (-1,):
        raise ValueError(f"{what}: {msg} (code {code})")
    raise StrataLibraryError(f"{what}: {msg} (code {code})")


def device_status(reset: bool = True) -> int:
    """Synchronise and return the device status word (0 = ok)."""
    st = c_int(0)
    check(load().strata_device_status(ctypes.byref(st), 1 if reset else 0), "strata_device_status")
    return st.value
