"""The ctypes binding printed in INTEGRATION.md (Option B) is executed as written:
its struct must have the size of the C struct, and on a GPU its two methods must
give what the reference's extract_kv_blocks / write_kv_blocks give."""
import ctypes as C
import os
import re
import shutil
import subprocess

import pytest
import torch

from elasticmm_b200 import _lib
from oracle import kv_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def option_b_namespace():
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    section = text[text.index("## Option B"):]
    block = re.search(r"```python\n(.*?)```", section, flags=re.S).group(1)
    _lib.load()  # the library is built
    block = block.replace('"elasticmm_b200/libemm_kv.so"', repr(str(_lib.LIB_PATH)))
    ns = {}
    exec(compile(block, "INTEGRATION.md:OptionB", "exec"), ns)
    return ns


def c_sizeof_pool_desc(tmp_path):
    src = tmp_path / "size.c"
    src.write_text('#include <stdio.h>\n#include "emm_kv.h"\n'
                   'int main(void) { printf("%zu %zu\\n", sizeof(emm_pool_desc), '
                   '(size_t)((char *)&((emm_pool_desc *)0)->num_planes - (char *)0)); return 0; }\n')
    exe = tmp_path / "size"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    size, off = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    return int(size), int(off)


def test_documented_struct_matches_the_header(tmp_path):
    ns = option_b_namespace()
    doc, mine = ns["PoolDesc"], _lib.PoolDesc
    assert C.sizeof(doc) == C.sizeof(mine) == 64
    assert [n for n, _ in doc._fields_] == [n for n, _ in mine._fields_]
    assert [getattr(doc, n).offset for n, _ in doc._fields_] == [getattr(mine, n).offset for n, _ in mine._fields_]
    if shutil.which("gcc"):
        size, off = c_sizeof_pool_desc(tmp_path)
        assert size == 64 and off == doc.num_planes.offset == 56
    # the presets write every field of the struct, the last two included
    d = doc(num_planes=7, reserved=7)
    assert ns["lib"].emm_pool_desc_nhd(C.byref(d), 2, 8, 4, 2, 8, 2) == 0
    assert (d.num_planes, d.reserved) == (2, 0)
    assert ns["lib"].emm_last_error.restype is C.c_char_p


@pytest.mark.gpu
def test_documented_binding_runs_and_matches_the_oracle():
    ns = option_b_namespace()
    L, NB, BS, H, D = 3, 24, 16, 4, 64
    src_cpu = kv_oracle.make_pool(L, NB, BS, H, D, torch.bfloat16, 5)
    dst_cpu = kv_oracle.make_pool(L, NB, BS, H, D, torch.bfloat16, 0, fill="guard")
    src = ns["B200KV"]([t.cuda() for t in src_cpu])
    dst = ns["B200KV"]([t.cuda() for t in dst_cpu])
    g = torch.Generator().manual_seed(5)
    s_ids = torch.randperm(NB, generator=g)[:11].tolist()
    d_ids = torch.randperm(NB, generator=g)[:11].tolist()
    packed = src.extract_kv_blocks(s_ids)
    dst.write_kv_blocks(d_ids, packed)
    dst.sync_and_check()
    want = kv_oracle.extract_kv_blocks(src_cpu, s_ids)
    assert kv_oracle.bit_equal(packed.cpu(), want)
    kv_oracle.write_kv_blocks(dst_cpu, d_ids, want)
    assert all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(dst.kv, dst_cpu))
    with pytest.raises(RuntimeError, match="outside"):
        src.extract_kv_blocks([0, NB])
