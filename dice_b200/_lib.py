"""ctypes binding of ``libdice_b200.so`` (declarations: ``include/dice_b200.h``).

There is no fallback: if the library has not been built, or an entry point is
missing, importing a symbol raises.  Build with ``python -m dice_b200.build``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_uint32, c_void_p

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libdice_b200.so")

# name -> (restype, argtypes); mirrors include/dice_b200.h one to one
SIGNATURES = {
    "dice_abi_version": (c_int, []),
    "dice_strerror": (c_char_p, [c_int]),
    "dice_status_message": (c_char_p, [c_uint32]),
    "dice_kernel_launches": (ctypes.c_uint64, []),
    "dice_router_top2": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p],
    ),
    "dice_top2_from_logits": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "dice_permute_scratch_bytes": (c_size_t, [c_int64, c_int]),
    "dice_permute_plan": (
        c_int,
        [c_void_p, c_int64, c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "dice_permute_plan_chunked": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
         c_void_p],
    ),
    "dice_permute_plan_static": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "dice_permute_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p]),
    "dice_unpermute_combine": (
        c_int,
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
         c_int, c_int64, c_int, c_int, c_void_p, c_void_p],
    ),
    "dice_ln_modulate": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, ctypes.c_float, c_int, c_int, c_void_p, c_void_p],
    ),
    "dice_w13_rows": (c_int64, [c_int]),
    "dice_pack_w13": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "dice_grouped_gemm": (
        c_int,
        [c_void_p, c_int64, c_int, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
         c_int, c_int, c_void_p, c_void_p],
    ),
    "dice_grouped_ffn": (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
         c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
         c_void_p],
    ),
    "dice_grouped_ffn_combine": (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
         c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    ),
    "dice_grouped_ffn_f32": (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
         c_void_p, c_void_p],
    ),
    "dice_ep_meta_ints": (c_int, [c_int, c_int]),
    "dice_ep_exchange_counts": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_uint32, c_void_p, c_void_p]),
    "dice_ep_dispatch_rows": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
         c_int, c_int, c_uint32, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "dice_ep_wait_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_uint32, c_void_p, c_void_p]),
    "dice_ep_wait_flags": (c_int, [c_void_p, c_int, c_uint32, c_int, c_void_p, c_void_p]),
    "dice_ep_return_rows": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_uint32, c_int,
         c_void_p, c_void_p]),
    "dice_ep_set_wait_limit_ms": (c_int, [c_int]),
    "dice_ep_return_rows_following": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_uint32, c_int,
         c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "dice_grouped_ffn_return": (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_uint32, c_int, c_void_p, c_void_p]),
    "dice_ipc_export": (c_int, [c_void_p, c_void_p, c_void_p]),
    "dice_ipc_import": (c_int, [c_void_p, ctypes.c_uint64, c_void_p]),
    "dice_ipc_close": (c_int, [c_void_p, ctypes.c_uint64]),
}

ABI_VERSION = 2
_lib = None


class DiceLibraryError(RuntimeError):
    pass


def library_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the native library (once) and bind every declared entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise DiceLibraryError(
            f"{_LIB_PATH} is missing: the CUDA extension has not been built "
            "(run `python -m dice_b200.build`); dice_b200 has no CPU or PyTorch fallback"
        )
    lib = ctypes.CDLL(_LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise DiceLibraryError(f"{_LIB_PATH} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    got = lib.dice_abi_version()
    if got != ABI_VERSION:
        raise DiceLibraryError(f"ABI version mismatch: library {got}, binding {ABI_VERSION}")
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    """Raise on a negative return code of an entry point."""
    if code != 0:
        msg = load().dice_strerror(code).decode()
        raise DiceLibraryError(f"{what} failed: {msg} (code {code})")
