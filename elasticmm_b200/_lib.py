"""ctypes binding of libemm_kv.so (the C ABI in include/emm_kv.h).

The library is loaded from the package directory. There is no fallback: if
the shared object is missing or fails to load, importing this module raises,
and every data-path call raises when no CUDA device is usable.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent / "libemm_kv.so"

IPC_HANDLE_BYTES = 64
NOALLOC_MAX_IDS = 16384
NOALLOC_MAX_LAYERS = 256
NCCL_UNIQUE_ID_BYTES = 128

# enum emm_status
OK = 0
ERR_BAD_ARG = 1
ERR_ID_RANGE = 2
ERR_LENGTH = 3
ERR_CUDA = 4
ERR_TIMEOUT = 5
ERR_ALIGN = 6
ERR_DUPLICATE = 7
ERR_OVERLAP = 8
ERR_TOO_LARGE = 9
ERR_NOMEM = 10
ERR_NCCL = 11

# enum emm_copy_variant
COPY_AUTO, COPY_BULK, COPY_LDG = 0, 1, 2

# enum emm_option
OPT_COPY_VARIANT = 0
OPT_CHUNK_BYTES = 1
OPT_STAGES = 2
OPT_WARPS = 3
OPT_CTAS_PER_SM = 4
OPT_LDG_UNROLL = 5
OPT_MAX_CTAS = 6
OPT_REMOTE_VARIANT = 7
OPT_L2_HINT = 8
OPT_WAIT_LIMIT_NS = 9
OPT_PDL = 10


class PoolDesc(C.Structure):
    """struct emm_pool_desc."""

    _fields_ = [
        ("num_layers", C.c_int32),
        ("num_blocks", C.c_int32),
        ("block_size", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_size", C.c_int32),
        ("elem_size", C.c_int32),
        ("plane_stride", C.c_int64),
        ("block_stride", C.c_int64),
        ("token_stride", C.c_int64),
        ("head_stride", C.c_int64),
        ("num_planes", C.c_int32),
        ("reserved", C.c_int32),
    ]


class EmmError(RuntimeError):
    """A non-zero status from the C ABI."""

    def __init__(self, status: int, message: str):
        super().__init__(f"emm_kv status {status}: {message}")
        self.status = status
        self.message = message


_P = C.c_void_p
_I32P = C.POINTER(C.c_int32)
_I64P = C.POINTER(C.c_int64)

# name -> (restype, argtypes). This table is also what the symbol test checks
# against the header.
SIGNATURES = {
    "emm_abi_version": (C.c_int, []),
    "emm_status_string": (C.c_char_p, [C.c_int]),
    "emm_last_error": (C.c_char_p, []),
    "emm_ctx_create": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "emm_ctx_destroy": (C.c_int, [_P]),
    "emm_ctx_set_option": (C.c_int, [_P, C.c_int, C.c_int64]),
    "emm_ctx_get_option": (C.c_int, [_P, C.c_int, _I64P]),
    "emm_ctx_launch_count": (C.c_int64, [_P]),
    "emm_ctx_status": (C.c_int, [_P, _P, _I64P]),
    "emm_pool_desc_nhd": (C.c_int, [C.POINTER(PoolDesc)] + [C.c_int] * 6),
    "emm_pool_desc_hnd": (C.c_int, [C.POINTER(PoolDesc)] + [C.c_int] * 6),
    "emm_pool_desc_blocks": (C.c_int, [C.POINTER(PoolDesc)] + [C.c_int] * 5),
    "emm_pool_create": (C.c_int, [_P, C.POINTER(PoolDesc), C.POINTER(_P), C.POINTER(_P)]),
    "emm_pool_destroy": (C.c_int, [_P]),
    "emm_pool_get_desc": (C.c_int, [_P, C.POINTER(PoolDesc)]),
    "emm_pool_page_bytes": (C.c_int64, [_P]),
    "emm_gather": (C.c_int, [_P, _P, C.c_int32, _P, C.c_uint64, _P]),
    "emm_scatter": (C.c_int, [_P, _P, C.c_int32, _P, C.c_uint64, _P]),
    "emm_gather_layers": (C.c_int, [_P, C.c_int32, C.c_int32, _P, C.c_int32, _P, C.c_uint64, _P]),
    "emm_scatter_layers": (C.c_int, [_P, C.c_int32, C.c_int32, _P, C.c_int32, _P, C.c_uint64, _P]),
    "emm_gather_many": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, _P, C.c_uint64, _P]),
    "emm_scatter_many": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, _P, C.c_uint64, _P]),
    "emm_gather_many_layers": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, C.c_int32, C.c_int32, _P, C.c_uint64, _P]),
    "emm_scatter_many_layers": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, C.c_int32, C.c_int32, _P, C.c_uint64, _P]),
    "emm_test_gather_expect_overcount": (C.c_int, [_P, _P, C.c_int32, _P, C.c_uint64, C.c_uint32, _P]),
    "emm_copy_blocks": (C.c_int, [_P, _P, _P, _P, C.c_int32, _P]),
    "emm_gather_h": (C.c_int, [_P, _P, C.c_int32, _P, C.c_uint64, _P]),
    "emm_scatter_h": (C.c_int, [_P, _P, C.c_int32, _P, C.c_uint64, _P]),
    "emm_copy_blocks_h": (C.c_int, [_P, _P, _P, _P, C.c_int32, _P]),
    "emm_gather_noalloc": (C.c_int, [C.c_int, C.POINTER(PoolDesc), C.POINTER(_P), _P, C.c_int32, _P, C.c_uint64, _P]),
    "emm_append": (C.c_int, [_P, C.c_int32, _P, _P, C.c_int64, C.c_int64, _P, C.c_int32, _P]),
    "emm_append_all_layers": (
        C.c_int,
        [_P, _P, _P, C.c_int64, C.c_int64, C.c_int64, C.c_int64, _P, C.c_int32, _P],
    ),
    "emm_append_bind": (C.c_int, [_P, _P, _P, C.c_int64, C.c_int64, C.c_int64, C.c_int64, _P, C.c_int32, C.POINTER(_P)]),
    "emm_append_bound": (C.c_int, [_P, C.c_int32, _P]),
    "emm_append_unbind": (C.c_int, [_P]),
    "emm_upload_ids": (C.c_int, [_P, _P, C.c_int32, _P, _P]),
    "emm_compact_plan": (C.c_int, [_I64P, C.c_int64, C.c_int64, _I64P, _I64P, _I64P, _I64P]),
    "emm_nccl_unique_id": (C.c_int, [C.c_char_p]),
    "emm_nccl_comm_init": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int, C.POINTER(_P)]),
    "emm_nccl_comm_destroy": (C.c_int, [_P]),
    "emm_send_packed": (C.c_int, [_P, _P, C.c_uint64, C.c_int, _P]),
    "emm_recv_packed": (C.c_int, [_P, _P, C.c_uint64, C.c_int, _P]),
    "emm_exchange": (C.c_int, [_P, C.c_int32, _I32P, C.POINTER(_P), C.POINTER(C.c_uint64), _I32P, _P]),
    "emm_send_blocks": (C.c_int, [_P, _P, C.c_int, _P, C.c_int32, _P, C.c_uint64, C.c_int32, _P]),
    "emm_recv_blocks": (C.c_int, [_P, _P, C.c_int, _P, C.c_int32, _P, C.c_uint64, C.c_int32, _P]),
    "emm_enable_peer_access": (C.c_int, [_P, C.c_int]),
    "emm_ipc_export": (C.c_int, [_P, _P, C.c_char_p, C.POINTER(C.c_uint64)]),
    "emm_ipc_open": (C.c_int, [_P, C.c_char_p, C.c_uint64, C.POINTER(_P)]),
}

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Loads the shared library once and sets the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m elasticmm_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is absent
        fn.restype = restype
        fn.argtypes = argtypes
    got = lib.emm_abi_version()
    if got != 1:
        raise ImportError(f"libemm_kv.so ABI version {got}, binding expects 1")
    _lib = lib
    return lib


def last_error() -> str:
    return load().emm_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raises EmmError for a non-zero status."""
    if status != OK:
        raise EmmError(status, last_error())
