"""ctypes face of oracle/kv_oracle.c on torch CPU tensors.  TEST INFRASTRUCTURE ONLY.

Used as a second, independently written checker and as the multi-threaded
CPU baseline (plain memcpy per page on all host cores).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path
from typing import List, Sequence, Tuple

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "libkv_oracle.so"
_lib = None


def build() -> Path:
    """Compiles the C restatement with the Makefile beside it."""
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    return LIB


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        _lib = C.CDLL(str(LIB))
        _lib.kvo_compact_plan.restype = C.c_int64
    return _lib


def _geom(layers: Sequence[torch.Tensor]) -> Tuple[C.Array, int, int, int]:
    t = layers[0]
    e = t.element_size()
    ptrs = (C.c_void_p * len(layers))(*[x.data_ptr() for x in layers])
    page = t.shape[2] * t.shape[3] * t.shape[4] * e
    assert t.stride(1) * e >= page and t[0, 0].is_contiguous(), "pages must be dense"
    return ptrs, t.stride(0) * e, t.stride(1) * e, page


def _ids(ids) -> np.ndarray:
    return np.ascontiguousarray(ids, dtype=np.int64)


def gather(layers: Sequence[torch.Tensor], ids, threads: int = 1) -> torch.Tensor:
    t = layers[0]
    ptrs, plane, block, page = _geom(layers)
    a = _ids(ids)
    out = torch.empty((len(layers), 2, len(a)) + tuple(t.shape[2:]), dtype=t.dtype)
    load().kvo_gather(ptrs, C.c_int64(len(layers)), C.c_int64(plane), C.c_int64(block), C.c_int64(page),
                      a.ctypes.data_as(C.c_void_p), C.c_int64(len(a)), C.c_void_p(out.data_ptr()),
                      C.c_int(threads))
    return out


def scatter(layers: Sequence[torch.Tensor], ids, packed: torch.Tensor, threads: int = 1) -> None:
    ptrs, plane, block, page = _geom(layers)
    a = _ids(ids)
    assert packed.is_contiguous() and packed.shape[2] == len(a)
    load().kvo_scatter(ptrs, C.c_int64(len(layers)), C.c_int64(plane), C.c_int64(block), C.c_int64(page),
                       a.ctypes.data_as(C.c_void_p), C.c_int64(len(a)), C.c_void_p(packed.data_ptr()),
                       C.c_int(threads))


def copy_blocks(src: Sequence[torch.Tensor], dst: Sequence[torch.Tensor], src_ids, dst_ids,
                threads: int = 1) -> None:
    sp, splane, sblock, page = _geom(src)
    dp, dplane, dblock, dpage = _geom(dst)
    assert page == dpage and len(src) == len(dst)
    a, b = _ids(src_ids), _ids(dst_ids)
    assert len(a) == len(b)
    load().kvo_copy_blocks(sp, dp, C.c_int64(len(src)), C.c_int64(splane), C.c_int64(sblock),
                           C.c_int64(dplane), C.c_int64(dblock), C.c_int64(page),
                           a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), C.c_int64(len(a)),
                           C.c_int(threads))


def append(layer_kv: torch.Tensor, key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    e = layer_kv.element_size()
    assert layer_kv[0, 0, 0].is_contiguous(), "token rows must be contiguous (token-major layout)"
    row = layer_kv.shape[3] * layer_kv.shape[4] * e
    s = np.ascontiguousarray(slot_mapping.numpy(), dtype=np.int64)
    load().kvo_append(C.c_void_p(layer_kv.data_ptr()), C.c_int64(layer_kv.stride(0) * e),
                      C.c_int64(layer_kv.stride(1) * e), C.c_int64(layer_kv.stride(2) * e),
                      C.c_int64(layer_kv.shape[2]), C.c_int64(row), C.c_void_p(key.data_ptr()),
                      C.c_void_p(value.data_ptr()), C.c_int64(key.stride(0) * e),
                      C.c_int64(value.stride(0) * e), s.ctypes.data_as(C.c_void_p), C.c_int64(len(s)))


def compact_plan(table_ids, num_blocks: int) -> Tuple[List[int], List[int], List[int]]:
    a = _ids(table_ids)
    n = len(a)
    new = np.empty(n, dtype=np.int64)
    src = np.empty(n, dtype=np.int64)
    dst = np.empty(n, dtype=np.int64)
    m = load().kvo_compact_plan(a.ctypes.data_as(C.c_void_p), C.c_int64(n), C.c_int64(num_blocks),
                                new.ctypes.data_as(C.c_void_p), src.ctypes.data_as(C.c_void_p),
                                dst.ctypes.data_as(C.c_void_p))
    if m < 0:
        raise ValueError("bad table: id out of range, duplicate, or more ids than blocks")
    return new.tolist(), src[:m].tolist(), dst[:m].tolist()
