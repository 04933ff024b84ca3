"""Imports the reference's own KV functions, unmodified, for CPU use.  TEST INFRASTRUCTURE ONLY.

The reference tree is only present where the fixtures are generated; nothing
that runs on a GPU box may call this. `ray` is not installed, and the
reference's worker module decorates its class with `@ray.remote` at import
time, so a minimal stand-in module is placed in sys.modules first:
`ray.remote(...)` becomes an identity decorator. The reference classes
themselves are not modified; a worker is created without running its
constructor (which imports vLLM and creates CUDA streams) and given CPU
tensors as its `kv_cache`.
"""
from __future__ import annotations

import importlib
import os
import sys
import types
from typing import Sequence

import torch

# The reference checkout sits beside this repository unless ELASTICMM_REFERENCE_ROOT says otherwise.
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_ROOT = os.environ.get("ELASTICMM_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference"))


def reference_available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "elasticmm", "engine", "v0"))


def _install_ray_stub() -> None:
    if "ray" in sys.modules:
        return
    ray = types.ModuleType("ray")

    def remote(*args, **kwargs):
        if len(args) == 1 and callable(args[0]) and not kwargs:
            return args[0]
        return lambda cls: cls

    ray.remote = remote
    ray.get = lambda x, timeout=None: x
    ray.get_gpu_ids = lambda: [0]
    ray.is_initialized = lambda: False
    util = types.ModuleType("ray.util")
    collective = types.ModuleType("ray.util.collective")
    util.collective = collective
    ray.util = util
    sys.modules["ray"] = ray
    sys.modules["ray.util"] = util
    sys.modules["ray.util.collective"] = collective


_modules = {}


def load(name: str):
    """Imports `elasticmm.engine.v0.<name>` from the reference tree."""
    if not reference_available():
        raise RuntimeError(f"reference tree not found under {REFERENCE_ROOT}")
    if name in _modules:
        return _modules[name]
    _install_ray_stub()
    if REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, REFERENCE_ROOT)
    # Import the leaf modules directly: the package __init__ pulls in the stage
    # engines and the backend, which need vLLM's V0 API.
    pkg_name = "elasticmm.engine.v0"
    for pkg, path in (("elasticmm", "elasticmm"), ("elasticmm.engine", "elasticmm/engine"),
                      (pkg_name, "elasticmm/engine/v0")):
        if pkg not in sys.modules:
            mod = types.ModuleType(pkg)
            mod.__path__ = [os.path.join(REFERENCE_ROOT, path)]
            sys.modules[pkg] = mod
    mod = importlib.import_module(f"{pkg_name}.{name}")
    _modules[name] = mod
    return mod


def make_worker(kv_cache: Sequence[torch.Tensor]):
    """A reference V0Worker over CPU tensors, constructor bypassed."""
    V0Worker = load("worker").V0Worker
    w = object.__new__(V0Worker)
    w.device = torch.device("cpu")
    w.kv_cache = list(kv_cache)
    return w


def make_block_manager(stage: str, num_gpu_blocks: int, num_cpu_blocks: int, block_size: int):
    return load("block_manager").V0BlockManager(stage, num_gpu_blocks, num_cpu_blocks, block_size)


def make_request(request_id: str, num_tokens: int):
    Request = load("utils").Request
    return Request(request_id=request_id, prompt="", max_tokens=1, prompt_token_ids=[0] * num_tokens)
