"""ctypes binding of ``libb200_trimul.so`` (the C ABI declared in ``include/b200_trimul.h``).

There is no fallback: if the library is missing or a call fails, a ``RuntimeError`` is raised.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200_trimul.so"

BIDIRECTIONAL = 0
OUTGOING = 1
INCOMING = 2
DTYPE_BF16 = 0
DTYPE_F32 = 1

# name -> (restype, argtypes); must list every symbol declared in include/b200_trimul.h
SIGNATURES = {
    "b200_trimul_version": (c_int, []),
    "b200_trimul_strerror": (c_char_p, [c_int]),
    "b200_trimul_last_cuda_error": (c_int, []),
    "b200_trimul_workspace_bytes": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(c_size_t)]),
    "b200_trimul_workspace_layout": (c_int, [c_int, c_int, POINTER(c_size_t)]),
    "b200_trimul_packed_bytes": (c_size_t, []),
    "b200_trimul_pack_weights": (
        c_int,
        [c_void_p] * 6 + [c_int] + [c_void_p] * 4 + [POINTER(c_void_p), c_void_p, c_void_p],
    ),
    "b200_trimul_prologue": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_contract": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_contract_backward": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_backward_workspace_bytes": (c_int, [c_int, c_int, c_int, POINTER(c_size_t)]),
    "b200_trimul_backward_workspace_layout": (c_int, [c_int, c_int, c_int, POINTER(c_size_t)]),
    "b200_trimul_backward": (
        c_int,
        [c_void_p] * 8 + [c_int] + [c_void_p] * 4 + [c_void_p] * 5 + [c_void_p] * 2 + [c_void_p] * 4
        + [c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
    ),
    "b200_trimul_contract_partial": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_prologue_push": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_reduce_partials": (
        c_int,
        [c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p],
    ),
    "b200_trimul_prologue_channels": (
        c_int,
        [c_void_p, c_void_p, c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_contract_channels": (
        c_int,
        [c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_epilogue_groups": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_peer_barrier": (
        c_int,
        [POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_epilogue": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_forward": (
        c_int,
        [c_void_p] * 7
        + [c_int]
        + [c_void_p] * 4
        + [POINTER(c_void_p), c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]
        + [c_int] * 5
        + [c_float, c_float, c_int, c_void_p],
    ),
    "b200_trimul_forward_ex": (
        c_int,
        [c_void_p] * 7
        + [c_int]
        + [c_void_p] * 4
        + [POINTER(c_void_p), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]
        + [c_int] * 5
        + [c_float, c_float, c_int, c_void_p],
    ),
    "b200_trimul_pack_weights_bidir": (
        c_int,
        [c_void_p] * 6 + [c_int] + [c_void_p] * 4 + [POINTER(c_void_p), c_void_p, c_void_p, c_void_p],
    ),
    "b200_trimul_epilogue_wide": (
        c_int,
        [c_void_p] * 7 + [c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p],
    ),
    "b200_trimul_forward_static": (
        c_int,
        [c_void_p] * 7
        + [c_int]
        + [c_void_p] * 4
        + [POINTER(c_void_p), c_void_p, c_void_p, c_void_p]
        + [c_int] * 5
        + [c_float, c_float, c_int, POINTER(c_void_p), c_void_p],
    ),
    "b200_transition_packed_bytes": (c_size_t, []),
    "b200_transition_pack_weights": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_transition_forward": (
        c_int,
        [c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    ),
    "b200_transition_backward_workspace_bytes": (c_int, [ctypes.c_longlong, POINTER(c_size_t)]),
    "b200_transition_backward": (
        c_int,
        [c_void_p] * 5 + [c_int] + [c_void_p] * 8 + [c_void_p, c_size_t, ctypes.c_longlong, c_int, c_int, c_float, c_int, c_void_p],
    ),
    "b200_trimul_clear_status": (c_int, [c_void_p, c_void_p]),
    "b200_trimul_read_status": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m miniworld_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().b200_trimul_strerror(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        lib = load()
        extra = ""
        if code == -6:
            extra = f" (cuda error {lib.b200_trimul_last_cuda_error()})"
        raise RuntimeError(f"{what}: {strerror(code)} [{code}]{extra}")
