"""Python face of the C ABI: device contexts and paged KV pools.

`Context` wraps one `emm_ctx` (one per process and GPU); `KVPool` wraps one
`emm_pool` built from the tensors a worker already owns. torch is used for
device memory and streams only; every byte of KV data is moved by the CUDA
kernels in libemm_kv.so. Nothing here computes on the CPU, and nothing falls
back to torch indexing when the library or a GPU is missing.

Pool tensors follow the reference: a list of L tensors, logical shape
[2, NB, BS, H, D] (elasticmm/engine/v0/worker.py:388-394,593-594). The byte
strides are read off each tensor, so a head-major pool is passed as the
permuted view `t.permute(0, 1, 3, 2, 4)` of a [2, NB, H, BS, D] allocation
and a single 6-D tensor [L, 2, NB, BS, H, D]
(elasticmm/engine/v0/nccl_transfer.py:215) as `list(t.unbind(0))`.
"""
from __future__ import annotations

import ctypes as C
import functools
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib

IdList = Union[Sequence[int], np.ndarray, torch.Tensor]


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class Context:
    """One emm_ctx: device status word, id staging ring, kernel options."""

    def __init__(self, device: Union[int, torch.device]):
        if not torch.cuda.is_available():
            raise RuntimeError("elasticmm_b200 needs a CUDA device; there is no CPU path")
        dev = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        if dev.type != "cuda":
            raise ValueError(f"KV pools live on CUDA devices, got {dev}")
        index = dev.index if dev.index is not None else torch.cuda.current_device()
        self.device = torch.device("cuda", index)
        self._lib = _lib.load()
        torch.cuda.init()
        with torch.cuda.device(self.device):
            torch.zeros(1, device=self.device)  # make sure the primary context exists
            handle = C.c_void_p()
            _lib.check(self._lib.emm_ctx_create(index, C.byref(handle)))
        self._h = handle
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count

    # -- options ---------------------------------------------------------
    def set_option(self, option: int, value: int) -> None:
        _lib.check(self._lib.emm_ctx_set_option(self._h, option, int(value)))

    def get_option(self, option: int) -> int:
        out = C.c_int64()
        _lib.check(self._lib.emm_ctx_get_option(self._h, option, C.byref(out)))
        return out.value

    def configure(self, *, variant: Optional[int] = None, chunk_bytes: Optional[int] = None,
                  stages: Optional[int] = None, warps: Optional[int] = None,
                  ctas_per_sm: Optional[int] = None, ldg_unroll: Optional[int] = None,
                  max_ctas: Optional[int] = None, remote_variant: Optional[int] = None,
                  l2_hint: Optional[int] = None) -> None:
        """Sets copy-kernel options; None leaves an option as it is."""
        pairs = [
            (_lib.OPT_COPY_VARIANT, variant), (_lib.OPT_CHUNK_BYTES, chunk_bytes),
            (_lib.OPT_STAGES, stages), (_lib.OPT_WARPS, warps),
            (_lib.OPT_CTAS_PER_SM, ctas_per_sm), (_lib.OPT_LDG_UNROLL, ldg_unroll),
            (_lib.OPT_MAX_CTAS, max_ctas), (_lib.OPT_REMOTE_VARIANT, remote_variant),
            (_lib.OPT_L2_HINT, l2_hint),
        ]
        for opt, val in pairs:
            if val is not None:
                self.set_option(opt, val)

    @property
    def launch_count(self) -> int:
        return int(self._lib.emm_ctx_launch_count(self._h))

    def status(self) -> Tuple[int, int]:
        """Synchronises the current stream; returns (status, detail) and clears it."""
        detail = C.c_int64()
        rc = self._lib.emm_ctx_status(self._h, C.c_void_p(_stream_ptr(self.device)), C.byref(detail))
        return rc, detail.value

    def check_status(self) -> None:
        """Raises EmmError if a kernel recorded a bad id, slot or a timeout."""
        rc, _ = self.status()
        _lib.check(rc)

    # -- peer mapping ------------------------------------------------------
    def ipc_export(self, tensor: torch.Tensor) -> Tuple[bytes, int]:
        """(handle, offset) naming `tensor`'s storage for another process."""
        buf = C.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        off = C.c_uint64()
        _lib.check(self._lib.emm_ipc_export(self._h, C.c_void_p(tensor.data_ptr()), buf, C.byref(off)))
        return bytes(buf.raw), off.value

    def ipc_open(self, handle: bytes, offset: int) -> int:
        """Maps a peer allocation; returns the device address in this process."""
        out = C.c_void_p()
        _lib.check(self._lib.emm_ipc_open(self._h, handle, C.c_uint64(offset), C.byref(out)))
        return int(out.value)

    def enable_peer_access(self, peer_device: Union[int, torch.device]) -> None:
        """Lets this device's kernels address another GPU of the same process."""
        index = peer_device if isinstance(peer_device, int) else torch.device(peer_device).index
        _lib.check(self._lib.emm_enable_peer_access(self._h, int(index)))

    # -- NCCL communicator owned by the library ------------------------------------
    def nccl_unique_id(self) -> bytes:
        """A fresh NCCL unique id (rank 0 makes it and ships it to the other ranks)."""
        buf = C.create_string_buffer(_lib.NCCL_UNIQUE_ID_BYTES)
        _lib.check(self._lib.emm_nccl_unique_id(buf))
        return bytes(buf.raw)

    def nccl_comm_init(self, unique_id: bytes, nranks: int, rank: int) -> int:
        """Collective: every rank calls it with the same id. Returns the ncclComm_t as an int."""
        comm = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self._lib.emm_nccl_comm_init(self._h, unique_id, nranks, rank, C.byref(comm)))
        return int(comm.value)

    def nccl_comm_destroy(self, comm: int) -> None:
        _lib.check(self._lib.emm_nccl_comm_destroy(C.c_void_p(comm)))

    def send_packed(self, comm: int, buf: torch.Tensor, peer: int) -> None:
        """Stream-ordered ncclSend of a contiguous device tensor's bytes."""
        _lib.check(self._lib.emm_send_packed(C.c_void_p(comm), C.c_void_p(buf.data_ptr()),
                                             buf.numel() * buf.element_size(), peer,
                                             C.c_void_p(_stream_ptr(self.device))))

    def recv_packed(self, comm: int, buf: torch.Tensor, peer: int) -> None:
        _lib.check(self._lib.emm_recv_packed(C.c_void_p(comm), C.c_void_p(buf.data_ptr()),
                                             buf.numel() * buf.element_size(), peer,
                                             C.c_void_p(_stream_ptr(self.device))))

    def exchange(self, comm: int, ops: Sequence[Tuple[bool, torch.Tensor, int]]) -> None:
        """One grouped exchange; ops are (is_send, contiguous device tensor, peer)."""
        n = len(ops)
        flags = (C.c_int32 * n)(*[1 if o[0] else 0 for o in ops])
        bufs = (C.c_void_p * n)(*[o[1].data_ptr() for o in ops])
        sizes = (C.c_uint64 * n)(*[o[1].numel() * o[1].element_size() for o in ops])
        peers = (C.c_int32 * n)(*[o[2] for o in ops])
        _lib.check(self._lib.emm_exchange(C.c_void_p(comm), n, flags, bufs, sizes, peers,
                                          C.c_void_p(_stream_ptr(self.device))))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            self._lib.emm_ctx_destroy(self._h)
            self._h = None


_contexts: Dict[int, Context] = {}


def get_context(device: Union[int, torch.device, None] = None) -> Context:
    """The process-wide Context of a device (created on first use)."""
    if device is None:
        if not torch.cuda.is_available():
            raise RuntimeError("elasticmm_b200 needs a CUDA device; there is no CPU path")
        index = torch.cuda.current_device()
    elif isinstance(device, int):
        index = device
    else:
        d = torch.device(device)
        index = d.index if d.index is not None else torch.cuda.current_device()
    ctx = _contexts.get(index)
    if ctx is None:
        ctx = Context(index)
        _contexts[index] = ctx
    return ctx


def _as_host_ids(ids: IdList) -> np.ndarray:
    if isinstance(ids, torch.Tensor):
        ids = ids.detach().cpu().numpy()
    arr = np.ascontiguousarray(ids, dtype=np.int64)
    if arr.ndim != 1:
        raise ValueError("block ids must be a flat list")
    return arr


class KVPool:
    """A paged KV pool known to the library.

    `layers` are the L per-layer tensors of logical shape [2, NB, BS, H, D]
    with the innermost dimension contiguous, or, for a single-plane block pool
    such as the vision-embedding block cache
    (elasticmm/engine/v0/nccl_transfer.py:295-368), tensors [NB, rows, cols];
    packed buffers of a block pool are [L, 1, n, rows, 1, cols]. For a pool that is not torch
    memory (a peer GPU's pool mapped by Context.ipc_open, a pinned host pool)
    use `KVPool.from_pointers`.
    """

    def __init__(self, layers: Sequence[torch.Tensor], ctx: Optional[Context] = None):
        layers = list(layers)
        if not layers:
            raise ValueError("a pool needs at least one layer tensor")
        first = layers[0]
        block_pool = first.dim() == 3  # [NB, rows, cols]: a single-plane block pool (vision embeddings)
        if not block_pool and (first.dim() != 5 or first.shape[0] != 2):
            raise ValueError(f"layer tensors must be [2, NB, BS, H, D] or [NB, rows, cols], got {tuple(first.shape)}")
        for t in layers:
            if t.shape != first.shape or t.dtype != first.dtype or t.stride() != first.stride():
                raise ValueError("all layer tensors must share shape, dtype and strides")
            if t.stride(-1) != 1:
                raise ValueError("the innermost dimension must be contiguous")
        device = first.device
        if device.type == "cuda":
            self.ctx = ctx or get_context(device)
        else:
            if ctx is None or not first.is_pinned():
                raise ValueError("a host pool must be pinned and needs an explicit Context")
            self.ctx = ctx
        e = first.element_size()
        if block_pool:
            desc = _lib.PoolDesc(
                num_layers=len(layers), num_blocks=first.shape[0], block_size=first.shape[1], num_kv_heads=1,
                head_size=first.shape[2], elem_size=e, plane_stride=0, block_stride=first.stride(0) * e,
                token_stride=first.stride(1) * e, head_stride=first.shape[2] * e, num_planes=1, reserved=0,
            )
        else:
            desc = _lib.PoolDesc(
                num_layers=len(layers), num_blocks=first.shape[1], block_size=first.shape[2],
                num_kv_heads=first.shape[3], head_size=first.shape[4], elem_size=e,
                plane_stride=first.stride(0) * e, block_stride=first.stride(1) * e,
                token_stride=first.stride(2) * e, head_stride=first.stride(3) * e, num_planes=2, reserved=0,
            )
        self._layers = layers  # keeps the memory alive
        self.dtype = first.dtype
        self._init_handle(desc, [t.data_ptr() for t in layers])

    @classmethod
    def from_pointers(cls, ctx: Context, desc: "_lib.PoolDesc", layer_ptrs: Sequence[int],
                      dtype: torch.dtype) -> "KVPool":
        """A pool over raw addresses (peer-mapped or host-pinned memory)."""
        self = cls.__new__(cls)
        self.ctx = ctx
        self._layers = None
        self.dtype = dtype
        self._init_handle(desc, list(layer_ptrs))
        return self

    def _init_handle(self, desc: "_lib.PoolDesc", ptrs: List[int]) -> None:
        lib = self.ctx._lib
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        handle = C.c_void_p()
        _lib.check(lib.emm_pool_create(self.ctx._h, C.byref(desc), arr, C.byref(handle)))
        self._h = handle
        self.desc = desc
        self.layer_ptrs = ptrs
        self.num_layers = desc.num_layers
        self.num_blocks = desc.num_blocks
        self.block_size = desc.block_size
        self.num_kv_heads = desc.num_kv_heads
        self.head_size = desc.head_size
        self.elem_size = desc.elem_size
        self.num_planes = 1 if desc.num_planes == 1 else 2
        self.page_bytes = int(lib.emm_pool_page_bytes(handle))
        self._append_sigs: Dict[tuple, int] = {}
        self._emm_append = lib.emm_append
        # head-major pages: tokens step by D, heads by BS*D
        self.head_major = (desc.num_kv_heads > 1 and desc.block_size > 1
                           and desc.token_stride == desc.head_size * desc.elem_size)

    # -- helpers ---------------------------------------------------------
    @property
    def device(self) -> torch.device:
        return self.ctx.device

    @property
    def layers(self) -> Optional[List[torch.Tensor]]:
        return self._layers

    def block_bytes(self) -> int:
        """Bytes of one block over all layers, K and V."""
        return self.num_planes * self.num_layers * self.page_bytes

    def packed_bytes(self, n: int, layer_count: Optional[int] = None) -> int:
        lc = self.num_layers if layer_count is None else layer_count
        return lc * self.num_planes * n * self.page_bytes

    def packed_shape(self, n: int, layer_count: Optional[int] = None) -> Tuple[int, ...]:
        lc = self.num_layers if layer_count is None else layer_count
        if self.head_major:
            return (lc, self.num_planes, n, self.num_kv_heads, self.block_size, self.head_size)
        return (lc, self.num_planes, n, self.block_size, self.num_kv_heads, self.head_size)

    def _logical(self, packed: torch.Tensor) -> torch.Tensor:
        """[.., n, BS, H, D] view of a packed buffer, whatever the page order."""
        return packed.permute(0, 1, 2, 4, 3, 5) if self.head_major else packed

    def new_packed(self, n: int, layer_count: Optional[int] = None) -> torch.Tensor:
        """An uninitialised packed buffer; logical shape [L, 2, n, BS, H, D]."""
        return self._logical(torch.empty(self.packed_shape(n, layer_count), dtype=self.dtype,
                                         device=self.device))

    def _packed_ptr(self, packed: torch.Tensor, n: int, layer_count: int) -> Tuple[int, int]:
        want = (layer_count, self.num_planes, n, self.block_size, self.num_kv_heads, self.head_size)
        if tuple(packed.shape) != want:
            raise ValueError(f"packed tensor has shape {tuple(packed.shape)}, expected {want}")
        if packed.dtype != self.dtype:
            raise ValueError(f"packed tensor dtype {packed.dtype} differs from pool dtype {self.dtype}")
        if packed.device != self.device:
            raise ValueError(f"packed tensor on {packed.device}, pool on {self.device}")
        phys = self._logical(packed)  # permute is its own inverse here
        if not phys.is_contiguous():
            raise ValueError("packed tensor must be contiguous in the pool's page order")
        return phys.data_ptr(), phys.numel() * phys.element_size()

    def upload_ids(self, ids: IdList) -> torch.Tensor:
        """int32 device table from a host list: staged through the library's pinned ring and
        copied on the current stream, with no pinned allocation and no synchronisation per call."""
        host = _as_host_ids(ids)
        n = host.shape[0]
        dev = torch.empty(n, dtype=torch.int32, device=self.device)
        if n:
            _lib.check(self.ctx._lib.emm_upload_ids(self.ctx._h, host.ctypes.data, n, dev.data_ptr(),
                                                    _stream_ptr(self.device)))
        return dev

    @staticmethod
    def _check_table(t: torch.Tensor, device: torch.device) -> None:
        if t.dtype != torch.int32 or t.dim() != 1 or not t.is_contiguous() or t.device != device:
            raise ValueError("device id tables must be contiguous 1-D int32 tensors on the pool's device")

    # -- whole-block movement -----------------------------------------------
    def gather(self, ids: IdList, out: Optional[torch.Tensor] = None,
               layer_begin: int = 0, layer_count: Optional[int] = None) -> torch.Tensor:
        """packed[l, p, i] = pool[l][p, ids[i]]; one launch for all layers.

        `ids` is a host list (range checked on the host, uploaded on the
        current stream) or an int32 device tensor (checked by the kernel).
        """
        lc = self.num_layers - layer_begin if layer_count is None else layer_count
        lib = self.ctx._lib
        st = _stream_ptr(self.device)
        if isinstance(ids, torch.Tensor) and ids.is_cuda:
            self._check_table(ids, self.device)
            n = ids.numel()
            out = self.new_packed(n, lc) if out is None else out
            ptr, nbytes = self._packed_ptr(out, n, lc)
            _lib.check(lib.emm_gather_layers(self._h, layer_begin, lc, C.c_void_p(ids.data_ptr()), n,
                                             C.c_void_p(ptr), nbytes, st))
            return out
        host = _as_host_ids(ids)
        n = host.shape[0]
        if layer_begin != 0 or lc != self.num_layers:
            return self.gather(self.upload_ids(self._validated(host)), out, layer_begin, lc)
        out = self.new_packed(n, lc) if out is None else out
        ptr, nbytes = self._packed_ptr(out, n, lc)
        rc = lib.emm_gather_h(self._h, host.ctypes.data, n, ptr, nbytes, st)
        if rc:
            _lib.check(rc)
        return out

    def scatter(self, ids: IdList, packed: torch.Tensor,
                layer_begin: int = 0, layer_count: Optional[int] = None) -> None:
        """pool[l][p, ids[i]] = packed[l, p, i]; one launch for all layers."""
        lc = self.num_layers - layer_begin if layer_count is None else layer_count
        lib = self.ctx._lib
        st = _stream_ptr(self.device)
        if isinstance(ids, torch.Tensor) and ids.is_cuda:
            self._check_table(ids, self.device)
            n = ids.numel()
            ptr, nbytes = self._packed_ptr(packed, n, lc)
            _lib.check(lib.emm_scatter_layers(self._h, layer_begin, lc, C.c_void_p(ids.data_ptr()), n,
                                              C.c_void_p(ptr), nbytes, st))
            return
        host = _as_host_ids(ids)
        n = host.shape[0]
        if layer_begin != 0 or lc != self.num_layers:
            host = self._validated(host, unique=True)
            return self.scatter(self.upload_ids(host), packed, layer_begin, lc)
        ptr, nbytes = self._packed_ptr(packed, n, lc)
        rc = lib.emm_scatter_h(self._h, host.ctypes.data, n, ptr, nbytes, st)
        if rc:
            _lib.check(rc)

    # -- several requests per launch ---------------------------------------------------
    def _many_tables(self, id_lists: Sequence[IdList], unique: bool):
        hosts = [_as_host_ids(x) for x in id_lists]
        counts = [h.shape[0] for h in hosts]
        flat = np.concatenate(hosts) if hosts else np.empty(0, dtype=np.int64)
        self._validated(flat, unique=unique)
        prefix = np.zeros(len(counts) + 1, dtype=np.int64)
        np.cumsum(counts, out=prefix[1:])
        dev = self.upload_ids(np.concatenate([flat, prefix]))  # one staged copy for the table and its prefix sums
        return counts, int(prefix[-1]), dev[: flat.shape[0]], dev[flat.shape[0]:]

    def gather_many(self, id_lists: Sequence[IdList]) -> List[torch.Tensor]:
        """extract_kv_blocks for several requests in one launch.

        Returns one tensor [L, 2, n_r, BS, H, D] per request; they are views of a
        single allocation in which the requests' buffers lie end to end.
        """
        counts, total, ids, prefix = self._many_tables(id_lists, unique=False)
        flat = torch.empty(self.packed_bytes(total) // self.elem_size, dtype=self.dtype, device=self.device)
        if total:
            _lib.check(self.ctx._lib.emm_gather_many(
                self._h, C.c_void_p(ids.data_ptr()), C.c_void_p(prefix.data_ptr()), len(counts), total,
                C.c_void_p(flat.data_ptr()), flat.numel() * self.elem_size, C.c_void_p(_stream_ptr(self.device))))
        return self._split_many(flat, counts)

    def many_tables(self, id_lists: Sequence[IdList], unique: bool = False):
        """Uploads the tables of several requests once: (counts, n_total, ids, prefix), for
        gather_many_into / scatter_many_from when the same tables are used repeatedly."""
        return self._many_tables(id_lists, unique)

    def gather_many_into(self, tables, flat: torch.Tensor) -> List[torch.Tensor]:
        """gather_many with tables from many_tables and a caller-owned flat buffer."""
        counts, total, ids, prefix = tables
        nbytes = self.packed_bytes(total)
        if flat.numel() * flat.element_size() < nbytes or flat.dtype != self.dtype or not flat.is_contiguous():
            raise ValueError("flat buffer too small, of another dtype, or not contiguous")
        if total:
            _lib.check(self.ctx._lib.emm_gather_many(
                self._h, C.c_void_p(ids.data_ptr()), C.c_void_p(prefix.data_ptr()), len(counts), total,
                C.c_void_p(flat.data_ptr()), nbytes, C.c_void_p(_stream_ptr(self.device))))
        return self._split_many(flat, counts)

    def scatter_many_from(self, tables, flat: torch.Tensor) -> None:
        """scatter_many with tables from many_tables and the flat buffer gather_many_into filled."""
        counts, total, ids, prefix = tables
        nbytes = self.packed_bytes(total)
        if flat.numel() * flat.element_size() < nbytes or flat.dtype != self.dtype or not flat.is_contiguous():
            raise ValueError("flat buffer too small, of another dtype, or not contiguous")
        if total:
            _lib.check(self.ctx._lib.emm_scatter_many(
                self._h, C.c_void_p(ids.data_ptr()), C.c_void_p(prefix.data_ptr()), len(counts), total,
                C.c_void_p(flat.data_ptr()), nbytes, C.c_void_p(_stream_ptr(self.device))))

    def gather_segments(self, tables, flat: torch.Tensor, layer_begin: int, layer_count: int) -> None:
        """Packs `layer_count` layers of several segments' blocks into `flat`, one contiguous
        [layer_count, planes, n_r, page] run per segment (tables from many_tables): the packed side of a
        rebalancing exchange, where a segment is everything one peer gets of this chunk of layers."""
        counts, total, ids, prefix = tables
        nbytes = self.packed_bytes(total, layer_count)
        if flat.numel() * flat.element_size() < nbytes or not flat.is_contiguous():
            raise ValueError("flat buffer too small or not contiguous")
        if total:
            _lib.check(self.ctx._lib.emm_gather_many_layers(
                self._h, layer_begin, layer_count, ids.data_ptr(), prefix.data_ptr(), len(counts), total,
                flat.data_ptr(), nbytes, _stream_ptr(self.device)))

    def scatter_segments(self, tables, flat: torch.Tensor, layer_begin: int, layer_count: int) -> None:
        """The inverse of gather_segments on the receiving pool."""
        counts, total, ids, prefix = tables
        nbytes = self.packed_bytes(total, layer_count)
        if flat.numel() * flat.element_size() < nbytes or not flat.is_contiguous():
            raise ValueError("flat buffer too small or not contiguous")
        if total:
            _lib.check(self.ctx._lib.emm_scatter_many_layers(
                self._h, layer_begin, layer_count, ids.data_ptr(), prefix.data_ptr(), len(counts), total,
                flat.data_ptr(), nbytes, _stream_ptr(self.device)))

    def _split_many(self, flat: torch.Tensor, counts: Sequence[int]) -> List[torch.Tensor]:
        out, pos = [], 0
        per_block = self.packed_bytes(1) // self.elem_size
        for n in counts:
            piece = flat[pos: pos + n * per_block]
            out.append(self._logical(piece.view(self.packed_shape(n))))
            pos += n * per_block
        return out

    def scatter_many(self, id_lists: Sequence[IdList], packed: Union[torch.Tensor, Sequence[torch.Tensor]]) -> None:
        """write_kv_blocks for several requests in one launch.

        `packed` is the list gather_many returned (buffers end to end in one
        allocation) or that allocation as one flat tensor.
        """
        counts, total, ids, prefix = self._many_tables(id_lists, unique=True)
        if isinstance(packed, torch.Tensor):
            flat = packed.reshape(-1)
        else:
            pieces = [self._logical(t) for t in packed]
            if [t.shape[2] for t in packed] != list(counts):
                raise ValueError("packed buffers do not match the block counts of the id lists")
            filled = [t for t in pieces if t.numel()]
            pos = 0
            for t in filled:  # the buffers must lie end to end, as gather_many lays them out
                if not t.is_contiguous() or t.data_ptr() != filled[0].data_ptr() + pos:
                    raise ValueError("packed buffers must be contiguous and adjacent (use gather_many's result)")
                if t.dtype != self.dtype or t.device != self.device:
                    raise ValueError("packed buffers must have the pool's dtype and device")
                pos += t.numel() * t.element_size()
            flat = filled[0] if filled else torch.empty(0, dtype=self.dtype, device=self.device)
        nbytes = self.packed_bytes(total)
        if total:
            _lib.check(self.ctx._lib.emm_scatter_many(
                self._h, C.c_void_p(ids.data_ptr()), C.c_void_p(prefix.data_ptr()), len(counts), total,
                C.c_void_p(flat.data_ptr()), nbytes, C.c_void_p(_stream_ptr(self.device))))

    def _validated(self, host: np.ndarray, unique: bool = False) -> np.ndarray:
        if host.size and (host.min() < 0 or host.max() >= self.num_blocks):
            raise _lib.EmmError(_lib.ERR_ID_RANGE, f"block id outside [0, {self.num_blocks})")
        if unique and np.unique(host).size != host.size:
            raise _lib.EmmError(_lib.ERR_DUPLICATE, "duplicate destination block id")
        return host

    def copy_blocks(self, dst: "KVPool", src_ids: IdList, dst_ids: IdList,
                    max_ctas: Optional[int] = None) -> None:
        """dst[l][p, dst_ids[i]] = self[l][p, src_ids[i]] with no staging buffer.

        `max_ctas` caps this launch's grid (used when several link-bound copies
        run side by side on different streams)."""
        if dst.ctx is not self.ctx:
            raise ValueError("both pools must belong to the same Context")
        if max_ctas is not None:
            before = self.ctx.get_option(_lib.OPT_MAX_CTAS)
            self.ctx.set_option(_lib.OPT_MAX_CTAS, max_ctas)
            try:
                return self.copy_blocks(dst, src_ids, dst_ids)
            finally:
                self.ctx.set_option(_lib.OPT_MAX_CTAS, before)
        lib = self.ctx._lib
        st = _stream_ptr(self.device)
        dev_tables = isinstance(src_ids, torch.Tensor) and src_ids.is_cuda
        if dev_tables != (isinstance(dst_ids, torch.Tensor) and dst_ids.is_cuda):
            raise ValueError("src_ids and dst_ids must both be host lists or both device tensors")
        if dev_tables:
            self._check_table(src_ids, self.device)
            self._check_table(dst_ids, self.device)
            if src_ids.numel() != dst_ids.numel():
                raise _lib.EmmError(_lib.ERR_LENGTH, "src_ids and dst_ids differ in length")
            _lib.check(lib.emm_copy_blocks(self._h, dst._h, C.c_void_p(src_ids.data_ptr()),
                                           C.c_void_p(dst_ids.data_ptr()), src_ids.numel(), st))
            return
        hs, hd = _as_host_ids(src_ids), _as_host_ids(dst_ids)
        if hs.shape != hd.shape:
            raise _lib.EmmError(_lib.ERR_LENGTH, "src_ids and dst_ids differ in length")
        rc = lib.emm_copy_blocks_h(self._h, dst._h, hs.ctypes.data, hd.ctypes.data, hs.shape[0], st)
        if rc:
            _lib.check(rc)

    # -- staged transport over a library-owned or host-owned ncclComm_t --------------
    def send_blocks(self, comm: int, peer: int, ids: torch.Tensor, staging: torch.Tensor,
                    layers_per_msg: int) -> None:
        """Pack -> ncclSend pipeline of all layers in messages of `layers_per_msg` layers."""
        self._check_table(ids, self.device)
        _lib.check(self.ctx._lib.emm_send_blocks(
            self._h, C.c_void_p(comm), peer, C.c_void_p(ids.data_ptr()), ids.numel(),
            C.c_void_p(staging.data_ptr()), staging.numel() * staging.element_size(), layers_per_msg,
            C.c_void_p(_stream_ptr(self.device))))

    def recv_blocks(self, comm: int, peer: int, ids: torch.Tensor, staging: torch.Tensor,
                    layers_per_msg: int) -> None:
        """ncclRecv -> unpack pipeline, the mirror of send_blocks."""
        self._check_table(ids, self.device)
        _lib.check(self.ctx._lib.emm_recv_blocks(
            self._h, C.c_void_p(comm), peer, C.c_void_p(ids.data_ptr()), ids.numel(),
            C.c_void_p(staging.data_ptr()), staging.numel() * staging.element_size(), layers_per_msg,
            C.c_void_p(_stream_ptr(self.device))))

    # -- per-token append ------------------------------------------------------
    def _check_kv(self, key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor,
                  lead: int) -> int:
        want_tail = (self.num_kv_heads, self.head_size)
        for name, t in (("key", key), ("value", value)):
            if t.dim() != lead + 3 or tuple(t.shape[-2:]) != want_tail:
                raise ValueError(f"{name} must be [{'L, ' if lead else ''}T, H, D] with H, D = {want_tail}")
            if t.dtype != self.dtype or t.device != self.device:
                raise ValueError(f"{name} must have the pool's dtype and device")
            if t.stride(-1) != 1 or t.stride(-2) != self.head_size:
                raise ValueError(f"{name} heads must be contiguous ([H, D] dense per token)")
        if key.shape != value.shape:
            raise ValueError("key and value shapes differ")
        T = key.shape[lead]
        if (slot_mapping.dtype != torch.int64 or slot_mapping.dim() != 1 or slot_mapping.numel() != T
                or slot_mapping.device != self.device or not slot_mapping.is_contiguous()):
            raise ValueError("slot_mapping must be a contiguous int64 device tensor with one entry per token")
        return T

    def append(self, layer: int, key: torch.Tensor, value: torch.Tensor,
               slot_mapping: torch.Tensor) -> None:
        """reshape_and_cache for one layer; slot < 0 entries are skipped."""
        # Called once per layer per step: argument checks are cached by signature.
        sig = (key.shape, key.stride(), key.dtype, key.device, value.shape, value.stride(), value.dtype,
               value.device, slot_mapping.shape, slot_mapping.stride(), slot_mapping.dtype, slot_mapping.device)
        T = self._append_sigs.get(sig)
        if T is None:
            T = self._check_kv(key, value, slot_mapping, 0)
            if len(self._append_sigs) < 64:
                self._append_sigs[sig] = T
        e = self.elem_size
        rc = self._emm_append(
            self._h, layer, key.data_ptr(), value.data_ptr(), key.stride(0) * e, value.stride(0) * e,
            slot_mapping.data_ptr(), T, torch.cuda.current_stream(self.ctx.device).cuda_stream)
        if rc:
            _lib.check(rc)

    def bind_append(self, key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor):
        """Pre-validated per-layer append over static buffers.

        `key` / `value` are [L, T, H, D] buffers and `slot_mapping` a [T] int64
        buffer that the caller refills in place every step (the usual shape of
        a graph-captured decode step). Returns `append(layer, stream=None)`,
        which launches reshape_and_cache for that layer at the cost of one
        three-argument foreign call (emm_append_bound). `stream` is a raw
        cudaStream_t handle (`torch.cuda.current_stream().cuda_stream`); a
        runner that issues all layers of a step on one stream looks it up once
        per step and passes it in, otherwise the current stream is looked up
        on every call.
        """
        T = self._check_kv(key, value, slot_mapping, 1)
        if key.shape[0] != self.num_layers:
            raise ValueError(f"key has {key.shape[0]} layers, pool has {self.num_layers}")
        e = self.elem_size
        lib = self.ctx._lib
        handle = C.c_void_p()
        _lib.check(lib.emm_append_bind(self._h, key.data_ptr(), value.data_ptr(), key.stride(0) * e, key.stride(1) * e,
                                       value.stride(0) * e, value.stride(1) * e, slot_mapping.data_ptr(), T,
                                       C.byref(handle)))
        fn, h = lib.emm_append_bound, handle.value
        device = self.ctx.device
        current_stream = torch.cuda.current_stream

        def append(layer: int, stream: Optional[int] = None) -> None:
            rc = fn(h, layer, current_stream(device).cuda_stream if stream is None else stream)
            if rc:
                _lib.check(rc)

        append.buffers = (key, value, slot_mapping, self)  # the closure keeps the buffers and the pool alive
        append.release = lambda: lib.emm_append_unbind(h)
        # the bare foreign call for hot loops: raw(layer, stream) returns the status code (0 = ok)
        append.raw = functools.partial(fn, h)
        return append

    def append_all_layers(self, key: torch.Tensor, value: torch.Tensor,
                          slot_mapping: torch.Tensor) -> None:
        """reshape_and_cache for every layer in one launch; key/value are [L, T, H, D]."""
        T = self._check_kv(key, value, slot_mapping, 1)
        if key.shape[0] != self.num_layers:
            raise ValueError(f"key has {key.shape[0]} layers, pool has {self.num_layers}")
        e = self.elem_size
        _lib.check(self.ctx._lib.emm_append_all_layers(
            self._h, C.c_void_p(key.data_ptr()), C.c_void_p(value.data_ptr()),
            key.stride(0) * e, key.stride(1) * e, value.stride(0) * e, value.stride(1) * e,
            C.c_void_p(slot_mapping.data_ptr()), T, C.c_void_p(_stream_ptr(self.device))))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            self.ctx._lib.emm_pool_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


def compact_plan(table_ids: Sequence[int], num_blocks: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Minimal-move defragmentation plan (host only, emm_compact_plan).

    Returns (new_table_ids, move_src, move_dst). Needs no GPU.
    """
    lib = _lib.load()
    ids = np.ascontiguousarray(table_ids, dtype=np.int64)
    n = ids.shape[0]
    new_ids = np.empty(n, dtype=np.int64)
    src = np.empty(n, dtype=np.int64)
    dst = np.empty(n, dtype=np.int64)
    moves = C.c_int64()
    p = lambda a: a.ctypes.data_as(C.POINTER(C.c_int64))
    _lib.check(lib.emm_compact_plan(p(ids), n, int(num_blocks), p(new_ids), p(src), p(dst), C.byref(moves)))
    m = moves.value
    return new_ids, src[:m].copy(), dst[:m].copy()
