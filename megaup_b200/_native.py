"""ctypes binding of libmegaup.so (declarations: include/megaup.h).

The library is the only compute path of this package: there is no PyTorch or
CPU fallback. Loading fails loudly when the shared object is missing.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

# MEGAUP_LIBRARY names another build of the library (A/B comparisons of kernel variants).
LIB_PATH = Path(os.environ.get("MEGAUP_LIBRARY") or Path(__file__).resolve().parent / "_lib" / "libmegaup.so")

MUP_OK = 0
ERROR_NAMES = {
    -1: "MUP_ERR_BAD_ARG",
    -2: "MUP_ERR_CUDA",
    -3: "MUP_ERR_UNSUPPORTED",
    -4: "MUP_ERR_DRIVER",
    -5: "MUP_ERR_DEVICE_STATUS",
}
STATUS_NAMES = {
    0: "ok",
    1: "TMA producer timed out waiting for a free shared-memory stage",
    2: "MMA warp timed out waiting for a filled shared-memory stage",
    3: "MMA warp timed out waiting for a free accumulator",
    4: "epilogue timed out waiting for a finished accumulator",
    5: "TMA producer timed out waiting for pulled rows",
    6: "dynamic shared memory is not 1024-byte aligned",
    7: "slot hand-off flag was not raised by a peer in time",
    8: "a role timed out waiting for its next work item",
}

class MupSync(ctypes.Structure):
    """``mup_sync`` of include/megaup.h: a hand-off folded into a launch."""

    _fields_ = [
        ("peer_flags", POINTER(c_void_p)),
        ("up", c_int),
        ("rank", c_int),
        ("wait_epoch", c_uint32),
        ("signal_epoch", c_uint32),
        ("done_counter", c_void_p),
        ("done_before", c_uint64),
        ("done_after", c_uint64),
        ("status_device_ptr", c_void_p),
        ("timeout_ns", c_uint64),
    ]


# name -> (restype, argtypes); must list every symbol include/megaup.h declares.
SIGNATURES: dict[str, tuple[object, tuple[object, ...]]] = {
    "mup_abi_version": (c_int, ()),
    "mup_last_error": (c_char_p, ()),
    "mup_device_supported": (c_int, (c_int, POINTER(c_int))),
    "mup_shape_rule": (c_int, (c_int64, c_int)),
    "mup_peer_n_rotation": (c_int, (c_int, c_int, c_int, c_int)),
    "mup_schedule_preview": (
        c_int,
        (
            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_uint32), c_int,
            POINTER(c_int), POINTER(c_int), POINTER(ctypes.c_double),
        ),
    ),
    "mup_set_max_active_ctas": (c_int, (c_int,)),
    "mup_status_create": (c_int, (POINTER(POINTER(c_uint32)), POINTER(c_void_p))),
    "mup_status_destroy": (c_int, (POINTER(c_uint32),)),
    "mup_arena_create": (c_int, (c_int, c_uint64, POINTER(c_void_p))),
    "mup_arena_import": (c_int, (c_int, c_int, c_uint64, POINTER(c_void_p))),
    "mup_arena_info": (c_int, (c_void_p, POINTER(c_void_p), POINTER(c_uint64), POINTER(c_int))),
    "mup_arena_destroy": (c_int, (c_void_p,)),
    "mup_flag_barrier": (
        c_int,
        (POINTER(c_void_p), c_int, c_int, c_uint32, c_void_p, c_uint64, c_void_p),
    ),
    "mup_peer_write_plan_create": (
        c_int,
        (
            POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int, c_int,
            c_void_p, c_void_p, POINTER(c_void_p), c_int, c_void_p, c_uint64,
        ),
    ),
    "mup_peer_write_launch": (c_int, (c_void_p, c_void_p, c_void_p)),
    "mup_peer_write_launch_synced": (c_int, (c_void_p, c_void_p, c_void_p, POINTER(MupSync))),
    "mup_peer_write_plan_info": (
        c_int,
        (c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int)),
    ),
    "mup_peer_write_plan_set_trace": (c_int, (c_void_p, c_void_p)),
    "mup_peer_write_plan_destroy": (c_int, (c_void_p,)),
    "mup_pull_workspace_bytes": (c_uint64, (c_int,)),
    "mup_pull_plan_create": (
        c_int,
        (
            POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int, c_int, c_int,
            c_void_p, c_void_p, POINTER(c_void_p), c_void_p, c_void_p, c_void_p,
            c_int, c_void_p, c_uint64,
        ),
    ),
    "mup_pull_launch": (c_int, (c_void_p, c_void_p)),
    "mup_pull_launch_synced": (c_int, (c_void_p, c_void_p, POINTER(MupSync))),
    "mup_pull_plan_reset": (c_int, (c_void_p, c_void_p)),
    "mup_pull_ticket_shape": (c_int, (c_int, POINTER(c_int), POINTER(c_int))),
    "mup_pull_plan_info": (
        c_int,
        (c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_uint64), POINTER(c_int), POINTER(c_int)),
    ),
    "mup_pull_plan_set_trace": (c_int, (c_void_p, c_void_p)),
    "mup_pull_plan_destroy": (c_int, (c_void_p,)),
    "mup_pull_gemm_noalloc": (
        c_int,
        (
            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
            POINTER(c_void_p), c_void_p, c_void_p, c_int, c_void_p, c_uint64, c_void_p,
        ),
    ),
    "mup_gather_rows": (c_int, (c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p)),
    "mup_gather_rows_synced": (
        c_int,
        (c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, POINTER(MupSync)),
    ),
    "mup_regroup_rows_synced": (
        c_int,
        (c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_void_p, POINTER(MupSync)),
    ),
    "mup_probe_load_latency": (c_int, (c_void_p, c_int, c_void_p, c_void_p)),
    "mup_regroup_rows": (
        c_int,
        (c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_void_p),
    ),
}

_LIB: ctypes.CDLL | None = None


class NativeError(RuntimeError):
    """A libmegaup.so call returned a negative code."""

    def __init__(self, function: str, code: int, message: str) -> None:
        self.function = function
        self.code = code
        name = ERROR_NAMES.get(code, str(code))
        super().__init__(f"{function} failed with {name}: {message}")


def lib() -> ctypes.CDLL:
    """Load libmegaup.so once and attach the argument types."""

    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m megaup_b200.build` "
                "(there is no fallback path)"
            )
        loaded = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(loaded, name)
            function.restype = restype
            function.argtypes = list(argtypes)
        _LIB = loaded
    return _LIB


def check(function: str, code: int) -> None:
    if code != MUP_OK:
        message = lib().mup_last_error()
        raise NativeError(function, code, message.decode() if message else "")


def call(function: str, *args: object) -> None:
    """Call an int-returning entry point and raise on a negative code."""

    check(function, getattr(lib(), function)(*args))


def pointer_array(addresses: list[int] | tuple[int, ...]) -> ctypes.Array:
    return (c_void_p * len(addresses))(*addresses)


def decode_status(word: int) -> str:
    code, detail = word >> 24, word & 0xFFFFFF
    return f"{STATUS_NAMES.get(code, f'code {code}')} (detail {detail})"
