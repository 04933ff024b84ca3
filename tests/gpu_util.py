"""Helpers shared by the GPU parity tests."""
from elasticmm_b200 import _lib
from oracle import kv_oracle

VARIANTS = [
    dict(variant=_lib.COPY_BULK, chunk_bytes=0, stages=2, warps=0),
    dict(variant=_lib.COPY_BULK, chunk_bytes=0, stages=4, warps=4),
    dict(variant=_lib.COPY_BULK, chunk_bytes=4096, stages=2, warps=1),
    dict(variant=_lib.COPY_BULK, chunk_bytes=16384, stages=3, warps=2),
    dict(variant=_lib.COPY_BULK, chunk_bytes=1024, stages=8, warps=8),
    dict(variant=_lib.COPY_LDG, chunk_bytes=0, ldg_unroll=4),
    dict(variant=_lib.COPY_LDG, chunk_bytes=2048, ldg_unroll=1),
    dict(variant=_lib.COPY_LDG, chunk_bytes=65536, ldg_unroll=8),
]
BULK_DEFAULT = VARIANTS[0]
LDG_DEFAULT = next(v for v in VARIANTS if v["variant"] == _lib.COPY_LDG)
DEFAULTS = dict(variant=_lib.COPY_AUTO, chunk_bytes=0, stages=2, warps=0, ctas_per_sm=0, ldg_unroll=2, max_ctas=0)


def vid(v):
    name = {_lib.COPY_BULK: "bulk", _lib.COPY_LDG: "ldg", _lib.COPY_AUTO: "auto"}[v["variant"]]
    return name + "-" + "-".join(f"{k[0]}{val}" for k, val in v.items() if k != "variant")


def configure(ctx, **opts):
    ctx.configure(**{**DEFAULTS, **opts})


def to_gpu(pool_cpu, device="cuda:0"):
    return [t.to(device) for t in pool_cpu]


def pools_equal(gpu_layers, cpu_layers):
    return all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(gpu_layers, cpu_layers))


def assert_clean(ctx):
    rc, detail = ctx.status()
    assert rc == _lib.OK, f"device status {rc} detail {detail}: {_lib.last_error()}"
