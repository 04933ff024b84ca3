"""CPU oracle for the paged KV-cache movement path.  TEST INFRASTRUCTURE ONLY.

This module restates, on CPU tensors, what the reference computes on its KV
movement path. It exists to check the CUDA library and to serve as the timed
CPU baseline. Nothing in the product package imports it: only tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline / reference legs do.

Parity status
  * gather / scatter / block tables: PINNED. The functions below are checked
    against the reference's own V0Worker.extract_kv_blocks /
    write_kv_blocks and V0BlockManager, imported unmodified (ref_loader.py),
    through the fixtures under tests/golden/ (made by tests/golden/make_golden.py)
    and, where the reference tree is present, live in tests/test_oracle_vs_reference.py.
  * 6-D single-tensor transfer and GPU<->CPU swap: restated from the source
    (the reference functions need a process group / CUDA streams and cannot
    run on CPU); pinned indirectly, because they must equal gather->scatter.
  * append (reshape_and_cache): PINNED against the third-party op the
    reference runs. The arithmetic lives in vLLM (requirement `vllm>=0.10.1`),
    which is not part of the reference tree; the reference reaches it under
    model_runner.execute_model (elasticmm/engine/v0/worker_steps.py:281,438).
    vLLM's reshape_and_cache_flash (the op for the [2, NB, BS, H, D] pool the
    reference binds, elasticmm/engine/v0/worker.py:380-412) was run on a B200
    (vLLM 0.22.0) by tests/golden/make_append_golden.py on the seeded inputs of
    tests/golden/cases.py; its output pools are the fixture
    tests/golden/append_golden.npz, which tests/test_oracle_golden.py checks
    this restatement against (slot s -> block s // BS, offset s % BS; negative
    slots are padding). Head rows that are not multiples of 16 bytes are outside
    what vLLM's kernel accepts (it raised "misaligned address" on 10-byte rows)
    and stay restatement-only.
  * compaction: no reference implementation exists; defined as
    extract_kv_blocks(old ids) followed by write_kv_blocks(new ids).

All payload is moved as opaque words; comparisons are bit-exact on int views.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ---------------------------------------------------------------------------
# gather / scatter
# ---------------------------------------------------------------------------

def extract_kv_blocks(kv_cache: Sequence[torch.Tensor], block_indices: Sequence[int]) -> torch.Tensor:
    """elasticmm/engine/v0/worker.py:578-610.

    For each per-layer tensor [2, NB, BS, H, D] select `[:, ids]` with an
    int64 index tensor, then stack the L results: [L, 2, n, BS, H, D].
    """
    idx = torch.tensor(list(block_indices), dtype=torch.long, device=kv_cache[0].device)
    per_layer = [layer_kv[:, idx, :, :, :] for layer_kv in kv_cache]
    return torch.stack(per_layer, dim=0)


def write_kv_blocks(kv_cache: Sequence[torch.Tensor], block_indices: Sequence[int],
                    kv_data: torch.Tensor) -> None:
    """elasticmm/engine/v0/worker.py:612-633: `layer_kv[:, ids] = kv_data[layer]`."""
    assert kv_data.shape[2] == len(block_indices), (
        f"Block count mismatch: {kv_data.shape[2]} vs {len(block_indices)}")
    idx = torch.tensor(list(block_indices), dtype=torch.long, device=kv_cache[0].device)
    for layer_idx, layer_kv in enumerate(kv_cache):
        layer_kv[:, idx, :, :, :] = kv_data[layer_idx]


def send_recv_per_layer(src_cache: Sequence[torch.Tensor], dst_cache: Sequence[torch.Tensor],
                        src_blocks: Sequence[int], dst_blocks: Sequence[int]) -> int:
    """Payload semantics of p2p_send_kv + p2p_recv_kv without the wire
    (elasticmm/engine/v0/worker.py:676-682,715-722): per layer, the message
    is `layer_kv[:, src_ids].contiguous()` and the sink does
    `layer_kv[:, dst_ids] = message`. Returns total bytes, as the reference
    reports them."""
    sidx = torch.tensor(list(src_blocks), dtype=torch.long)
    didx = torch.tensor(list(dst_blocks), dtype=torch.long)
    total = 0
    for s_layer, d_layer in zip(src_cache, dst_cache):
        msg = s_layer[:, sidx, :, :, :].contiguous()
        d_layer[:, didx, :, :, :] = msg
        total += msg.numel() * msg.element_size()
    return total


def transfer_blocks_6d(src_kv: torch.Tensor, dst_kv: torch.Tensor, src_blocks: Sequence[int],
                       dst_blocks: Sequence[int]) -> torch.Tensor:
    """elasticmm/engine/v0/nccl_transfer.py:241-247,282-289 on a single
    [L, 2, NB, BS, H, D] tensor: stack per-block slices along dim 2, flatten
    (the message), reshape on the sink, write block by block."""
    kv_data = torch.stack([src_kv[:, :, b, :, :, :] for b in src_blocks], dim=2)
    flat = kv_data.flatten()
    L, P, _, BS, H, D = src_kv.shape
    recv = flat.view(L, P, len(dst_blocks), BS, H, D)
    for i, b in enumerate(dst_blocks):
        dst_kv[:, :, b, :, :, :] = recv[:, :, i, :, :, :]
    return recv


def swap_blocks(kv_cache: Sequence[torch.Tensor], kv_swap: Sequence[torch.Tensor],
                source_block_ids: Sequence[int], target_block_ids: Sequence[int],
                is_swap_in: bool) -> None:
    """elasticmm/engine/v0/worker.py:516-526, per-block copy of all layers'
    K and V between the host pool and the GPU pool (the reference indexes a
    6-D tensor; per-layer lists are equivalent)."""
    for src_idx, tgt_idx in zip(source_block_ids, target_block_ids):
        for layer_gpu, layer_cpu in zip(kv_cache, kv_swap):
            if is_swap_in:
                layer_gpu[:, tgt_idx] = layer_cpu[:, src_idx]
            else:
                layer_cpu[:, tgt_idx] = layer_gpu[:, src_idx]


def copy_blocks(src_cache: Sequence[torch.Tensor], dst_cache: Sequence[torch.Tensor],
                src_ids: Sequence[int], dst_ids: Sequence[int]) -> None:
    """Block copy defined as extract on the source, write on the sink."""
    write_kv_blocks(dst_cache, dst_ids, extract_kv_blocks(src_cache, src_ids))


def transfer_vision_blocks(src_cache: torch.Tensor, dst_cache: torch.Tensor, src_blocks: Sequence[int],
                           dst_blocks: Sequence[int]) -> torch.Tensor:
    """elasticmm/engine/v0/nccl_transfer.py:328-363 on a block cache
    [blocks, embed_tokens, embed_dim]: stack the source blocks, flatten (the
    message), reshape on the sink and write block by block. Restated from the
    source (the reference function needs a process group)."""
    ve_data = torch.stack([src_cache[b] for b in src_blocks], dim=0)
    flat = ve_data.flatten()
    recv = flat.view(len(dst_blocks), src_cache.shape[1], src_cache.shape[2])
    for i, b in enumerate(dst_blocks):
        dst_cache[b] = recv[i]
    return recv


# ---------------------------------------------------------------------------
# append (pinned against vLLM's op through tests/golden/append_golden.npz, see the module docstring)
# ---------------------------------------------------------------------------

def reshape_and_cache(key: torch.Tensor, value: torch.Tensor, layer_kv: torch.Tensor,
                      slot_mapping: torch.Tensor) -> None:
    """Writes key/value [T, H, D] into one layer's pool [2, NB, BS, H, D].

    Call site in the reference: the cache op under
    model_runner.execute_model (elasticmm/engine/v0/worker_steps.py:281,438);
    slots come from the block tables passed at :219,411. Each plane is viewed
    as [NB*BS, H, D]; rows with slot >= 0 are stored at their slot.
    """
    valid = slot_mapping >= 0
    slots = slot_mapping[valid]
    nb, bs = layer_kv.shape[1], layer_kv.shape[2]
    blk = torch.div(slots, bs, rounding_mode="floor")
    off = slots - blk * bs
    layer_kv[0, blk, off] = key[valid]
    layer_kv[1, blk, off] = value[valid]


def slot_mapping_from_table(table: Sequence[int], positions: Sequence[int], block_size: int) -> List[int]:
    """slot = table[pos // BS] * BS + pos % BS."""
    return [table[p // block_size] * block_size + p % block_size for p in positions]


# ---------------------------------------------------------------------------
# compaction
# ---------------------------------------------------------------------------

def compact_plan(table_ids: Sequence[int], num_blocks: int) -> Tuple[List[int], List[int], List[int]]:
    """Minimal-move plan: live ids >= n_live move, in table order, into the
    free ids < n_live in ascending order. Returns (new_ids, move_src, move_dst)."""
    ids = [int(x) for x in table_ids]
    n_live = len(ids)
    live = set(ids)
    assert len(live) == n_live, "a block belongs to two table entries"
    assert all(0 <= b < num_blocks for b in ids)
    holes = iter(b for b in range(n_live) if b not in live)
    new_ids, move_src, move_dst = [], [], []
    for b in ids:
        if b < n_live:
            new_ids.append(b)
        else:
            h = next(holes)
            new_ids.append(h)
            move_src.append(b)
            move_dst.append(h)
    return new_ids, move_src, move_dst


def compact(kv_cache: Sequence[torch.Tensor], move_src: Sequence[int], move_dst: Sequence[int]) -> None:
    """Executes a plan with the reference's copy path (worker.py:578-633)."""
    if len(move_src):
        write_kv_blocks(kv_cache, move_dst, extract_kv_blocks(kv_cache, move_src))


# ---------------------------------------------------------------------------
# block tables
# ---------------------------------------------------------------------------

class BlockTables:
    """elasticmm/engine/v0/block_manager.py:102-142,174-256 with plain lists:
    allocation slices the head of the free list, freeing appends at the tail,
    a table only grows."""

    def __init__(self, num_gpu_blocks: int, block_size: int):
        self.block_size = block_size
        self.free: List[int] = list(range(num_gpu_blocks))
        self.table: Dict[str, List[int]] = {}

    def _take(self, n: int) -> List[int]:
        assert len(self.free) >= n
        out, self.free = self.free[:n], self.free[n:]
        return out

    def allocate(self, request_id: str, num_tokens: int, num_blocks: Optional[int] = None) -> None:
        need = -(-num_tokens // self.block_size) if num_blocks is None else num_blocks
        if request_id not in self.table:
            self.table[request_id] = self._take(need)
        elif len(self.table[request_id]) < need:
            self.table[request_id] += self._take(need - len(self.table[request_id]))

    def expand(self, request_id: str, seq_len: int) -> List[int]:
        need = -(-seq_len // self.block_size)
        cur = len(self.table[request_id])
        if cur < need:
            self.table[request_id] += self._take(need - cur)
        return self.table[request_id]

    def release(self, request_id: str) -> None:
        self.free += self.table.pop(request_id)


# ---------------------------------------------------------------------------
# helpers for tests and the bench
# ---------------------------------------------------------------------------

def bits(t: torch.Tensor) -> torch.Tensor:
    """Integer view of a tensor for bit-exact comparison."""
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return t.contiguous().view(view)


def bit_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and a.dtype == b.dtype and torch.equal(bits(a.cpu()), bits(b.cpu()))


def make_pool(num_layers: int, num_blocks: int, block_size: int, num_heads: int, head_size: int,
              dtype: torch.dtype, seed: int, fill: str = "normal") -> List[torch.Tensor]:
    """Seeded CPU pool in the reference layout: L tensors [2, NB, BS, H, D]."""
    g = torch.Generator().manual_seed(seed)
    shape = (2, num_blocks, block_size, num_heads, head_size)
    out = []
    for _ in range(num_layers):
        if fill == "normal":
            out.append(torch.randn(shape, generator=g, dtype=torch.float32).to(dtype))
        else:  # guard pattern: every 16-bit word 0x7FFF (a NaN payload nothing computes)
            t = torch.full(shape, 0, dtype=dtype)
            bits(t).fill_(0x7FFF if t.element_size() == 2 else 0x7F)
            out.append(t)
    return out
