"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

import pytest

from elasticmm_b200 import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(__file__)), "include", "emm_kv.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(emm_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} declared in emm_kv.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes prototype"
    assert sorted(_lib.SIGNATURES) == names


def test_abi_version_and_status_strings():
    lib = _lib.load()
    assert lib.emm_abi_version() == 1
    assert lib.emm_status_string(_lib.OK) == b"ok"
    seen = {lib.emm_status_string(c) for c in range(0, 12)}
    assert len(seen) == 12 and b"unknown status" not in seen
    assert lib.emm_status_string(99) == b"unknown status"


def test_status_codes_match_header():
    text = open(HEADER).read()
    for name, value in re.findall(r"(EMM_(?:OK|ERR_[A-Z_]+))\s*=\s*(\d+)", text):
        py = name[len("EMM_"):]
        assert getattr(_lib, py) == int(value), name


def test_pool_desc_presets_need_no_gpu():
    lib = _lib.load()
    assert C.sizeof(_lib.PoolDesc) == 64  # struct emm_pool_desc; the C client below checks the C side
    d = _lib.PoolDesc()
    assert lib.emm_pool_desc_nhd(C.byref(d), 32, 2048, 16, 32, 128, 2) == 0
    page = 16 * 32 * 128 * 2
    assert (d.block_stride, d.plane_stride, d.token_stride, d.head_stride) == (page, page * 2048, 32 * 256, 256)
    assert lib.emm_pool_desc_hnd(C.byref(d), 28, 64, 16, 4, 128, 2) == 0
    assert (d.token_stride, d.head_stride) == (256, 16 * 256)
    assert lib.emm_pool_desc_nhd(C.byref(d), 0, 1, 1, 1, 1, 2) == _lib.ERR_BAD_ARG
    assert lib.emm_pool_desc_nhd(C.byref(d), 1, 1, 1, 1, 1, 3) == _lib.ERR_BAD_ARG
    assert b"elem_size" in lib.emm_last_error()


def test_context_creation_fails_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    lib = _lib.load()
    h = C.c_void_p()
    rc = lib.emm_ctx_create(0, C.byref(h))
    assert rc == _lib.ERR_CUDA and not h.value
    assert lib.emm_last_error() != b""
    from elasticmm_b200 import get_context
    from elasticmm_b200.engine.v0 import V0Worker

    with pytest.raises(RuntimeError, match="no CPU path"):
        get_context(0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        V0Worker()


def test_nccl_entries_validate_arguments_without_a_gpu():
    lib = _lib.load()
    assert lib.emm_send_packed(None, None, 16, 0, None) == _lib.ERR_BAD_ARG
    assert lib.emm_recv_packed(None, None, 16, 0, None) == _lib.ERR_BAD_ARG
    assert lib.emm_exchange(None, 1, None, None, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.emm_nccl_comm_destroy(None) == _lib.OK
    assert lib.emm_send_blocks(None, None, 0, None, 0, None, 0, 1, None) == _lib.ERR_BAD_ARG


C_CLIENT = r"""
#include <stdio.h>
#include "emm_kv.h"

int main(void) {
  emm_pool_desc d;
  int64_t table[5] = {9, 1, 7, 0, 4}, new_ids[5], src[5], dst[5], moves = -1;
  if (emm_abi_version() != EMM_KV_ABI_VERSION) return 1;
  if (sizeof(emm_pool_desc) != 64) return 6;
  if (emm_pool_desc_hnd(&d, 28, 64, 16, 4, 128, 2) != EMM_OK) return 2;
  if (d.token_stride != 256 || d.head_stride != 16 * 256 || d.num_planes != 2) return 3;
  if (emm_pool_desc_nhd(&d, 1, 1, 1, 1, 1, 3) != EMM_ERR_BAD_ARG) return 4;
  if (emm_compact_plan(table, 5, 10, new_ids, src, dst, &moves) != EMM_OK || moves != 2) return 5;
  printf("%lld->%lld %lld->%lld %s\n", (long long)src[0], (long long)dst[0], (long long)src[1],
         (long long)dst[1], emm_status_string(EMM_ERR_TIMEOUT));
  return 0;
}
"""


def test_header_is_plain_c_and_a_c_program_links_against_the_library(tmp_path):
    """An integrator may bind the ABI from C: the header must compile as C99 and
    as C++ without warnings, and a C client must link and run (host-only entries)."""
    import shutil
    import subprocess

    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    inc = os.path.dirname(HEADER)
    _lib.load()
    libdir = str(_lib.LIB_PATH.parent)
    src = tmp_path / "client.c"
    src.write_text(C_CLIENT)
    flags = ["-Wall", "-Wextra", "-pedantic", "-Werror", "-I", inc]
    subprocess.run(["gcc", "-std=c99", *flags, "-fsyntax-only", str(src)], check=True)
    if shutil.which("g++"):
        subprocess.run(["g++", "-std=c++11", *flags, "-fsyntax-only", "-x", "c++", str(src)], check=True)
    exe = tmp_path / "client"
    subprocess.run(["gcc", "-std=c99", *flags, str(src), "-o", str(exe), "-L", libdir, "-lemm_kv",
                    f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    assert out.strip() == "9->2 7->3 device-side wait timed out"
