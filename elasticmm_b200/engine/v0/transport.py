"""Layer-chunked, double-buffered point-to-point transport of packed KV pages.

The reference moves a request one layer per message, strictly serially:
gather layer l, blocking send, next layer; the receiver allocates a buffer,
blocks in recv, then scatters (elasticmm/engine/v0/worker.py:676-682,804-820).
Here the same per-layer message order is kept but grouped into chunks of
consecutive layers and pipelined: while chunk c is on the wire, chunk c+1 is
being packed on the source and chunk c-1 unpacked on the sink. Both sides
derive the identical chunk schedule from (L, n, page_bytes), so no metadata
is exchanged beyond what the reference exchanges (the two block-id lists,
host side).

The functions are written against callables (`pack`, `unpack`, `isend`,
`irecv`) so the schedule and the buffer-reuse protocol do not depend on where
the bytes live. On a GPU the callables are KVPool.gather / KVPool.scatter and
torch.distributed P2P on the NCCL backend, and `Work.wait()` orders streams
without blocking the host.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

Chunk = Tuple[int, int]  # (layer_begin, layer_count)

DEFAULT_MESSAGE_BYTES = 512 << 20  # NCCL reaches its upper point-to-point rate from about half a gibibyte per message
PIPELINE_DEPTH = 2


def plan_chunks(num_layers: int, n_blocks: int, page_bytes: int,
                target_bytes: int = DEFAULT_MESSAGE_BYTES, taper: bool = False) -> List[Chunk]:
    """Splits the L layers into consecutive chunks of about `target_bytes` each.

    One layer of n blocks is 2*n*page_bytes on the wire. At least two chunks
    are produced whenever L >= 2 so that packing and sending can overlap. With
    `taper` the first and the last chunk are a single layer: the first chunk's
    pack and the last chunk's unpack are the only parts of a pipelined transfer
    that nothing overlaps, so they should be short.
    """
    if num_layers <= 0 or n_blocks <= 0:
        return []
    layer_bytes = 2 * n_blocks * page_bytes
    per_chunk = max(1, min(num_layers, target_bytes // max(1, layer_bytes)))
    if num_layers >= 2:
        per_chunk = min(per_chunk, (num_layers + 1) // 2)
    if taper and per_chunk > 1 and num_layers >= 3:
        inner = [(1 + b, min(per_chunk, num_layers - 2 - b)) for b in range(0, num_layers - 2, per_chunk)]
        return [(0, 1)] + inner + [(num_layers - 1, 1)]
    return [(b, min(per_chunk, num_layers - b)) for b in range(0, num_layers, per_chunk)]


def max_chunk_layers(chunks: Sequence[Chunk]) -> int:
    return max((c for _, c in chunks), default=0)


def pipelined_send(chunks: Sequence[Chunk], buffer_for: Callable[[int, int], object],
                   pack: Callable[[object, int, int], None],
                   isend: Callable[[object], object], depth: int = PIPELINE_DEPTH) -> int:
    """Packs and sends every chunk; returns the number of messages sent.

    `buffer_for(slot, layer_count)` returns the staging buffer of ring slot
    `slot` shaped for `layer_count` layers. A slot is packed again only after
    the send that read it has completed.
    """
    works: List[object] = []
    for c, (begin, count) in enumerate(chunks):
        if c >= depth:
            works[c - depth].wait()
        buf = buffer_for(c % depth, count)
        pack(buf, begin, count)
        works.append(isend(buf))
    for w in works[-depth:]:
        w.wait()
    return len(works)


def pipelined_recv(chunks: Sequence[Chunk], buffer_for: Callable[[int, int], object],
                   irecv: Callable[[object], object],
                   unpack: Callable[[object, int, int], None], depth: int = PIPELINE_DEPTH) -> int:
    """Receives and unpacks every chunk; returns the number of messages received.

    Up to `depth` receives are posted ahead; the receive for chunk c+depth is
    posted after chunk c has been unpacked from the slot it will land in.
    """
    posted: Dict[int, Tuple[object, object]] = {}

    def post(c: int) -> None:
        buf = buffer_for(c % depth, chunks[c][1])
        posted[c] = (buf, irecv(buf))

    for c in range(min(depth, len(chunks))):
        post(c)
    for c, (begin, count) in enumerate(chunks):
        buf, work = posted.pop(c)
        work.wait()
        unpack(buf, begin, count)
        if c + depth < len(chunks):
            post(c + depth)
    return len(chunks)


@dataclass(frozen=True)
class Transfer:
    """One request's move: the unit the reference passes to transfer_kv_cache
    (elasticmm/engine/v0/kv_transfer.py:224-231)."""

    request_id: str
    src_rank: int
    dst_rank: int
    src_blocks: Tuple[int, ...]
    dst_blocks: Tuple[int, ...]

    def __post_init__(self):
        if len(self.src_blocks) != len(self.dst_blocks):
            raise ValueError(
                f"Block count mismatch: src={len(self.src_blocks)}, dst={len(self.dst_blocks)}")


class MigrationPlan:
    """All transfers of one role switch, grouped by (source, sink) pair.

    The reference migrates a GPU's requests one awaited RPC at a time
    (elasticmm/engine/v0/backend.py:674-718). Grouping the same tuples by
    pair lets each pair move as one long table: per pair the block lists are
    concatenated in plan order, which is also the page order on the wire.
    """

    def __init__(self, transfers: Sequence[Transfer] = ()):
        self.transfers: List[Transfer] = []
        self._tables = {}
        for t in transfers:
            self.add(t)

    def add(self, t: Transfer) -> None:
        if t.src_rank == t.dst_rank:
            raise ValueError(f"{t.request_id}: source and sink rank are both {t.src_rank}")
        self.transfers.append(t)
        self._tables: Dict[Tuple[int, int], Tuple[List[int], List[int]]] = {}  # derived data is rebuilt lazily

    def pairs(self) -> List[Tuple[int, int]]:
        """(src, dst) pairs in a fixed order every rank agrees on."""
        return sorted({(t.src_rank, t.dst_rank) for t in self.transfers})

    def ordered_pairs(self) -> List[Tuple[int, int]]:
        """Pairs in the order every rank serves them.

        Source number i starts at sink number i and walks the sinks cyclically,
        so concurrent sources meet different sinks first. Sorting all pairs by
        (step, source) gives one total order; a rank that serves its own pairs
        in that order can never be part of a circular wait, because the
        globally first unfinished pair is first for both of its ends.
        """
        pairs = self.pairs()
        sources = sorted({s for s, _ in pairs})
        sinks = sorted({d for _, d in pairs})
        m = len(sinks)
        step = lambda sd: (sinks.index(sd[1]) - sources.index(sd[0])) % m
        return sorted(pairs, key=lambda sd: (step(sd), sd[0], sd[1]))

    def pull_order(self, sink: int) -> List[int]:
        """Sources of `sink`, rotated so that sink number j lists source number j first.

        A sink launches its pulls in this order (side by side, with capped grids);
        the rotation spreads the first requests over the sources.
        """
        sinks = sorted({d for _, d in self.pairs()})
        mine = sorted(s for s, d in self.pairs() if d == sink)
        if not mine:
            return []
        k = sinks.index(sink) % len(mine)
        return mine[k:] + mine[:k]

    def push_order(self, source: int) -> List[int]:
        """Sinks of `source` in the order it should push to them, one at a time
        (the mirror image of pull_order: one flow per source, starts spread out)."""
        sources = sorted({s for s, _ in self.pairs()})
        mine = sorted(d for s, d in self.pairs() if s == source)
        if not mine:
            return []
        k = (sources.index(source) * max(1, len(mine) // len(sources))) % len(mine)
        return mine[k:] + mine[:k]

    def tables(self, src_rank: int, dst_rank: int) -> Tuple[List[int], List[int]]:
        """Concatenated (src_blocks, dst_blocks) of one pair, in plan order."""
        cached = self._tables.get((src_rank, dst_rank))
        if cached is not None:
            return cached
        src: List[int] = []
        dst: List[int] = []
        for t in self.transfers:
            if t.src_rank == src_rank and t.dst_rank == dst_rank:
                src += t.src_blocks
                dst += t.dst_blocks
        self._tables[(src_rank, dst_rank)] = (src, dst)
        return src, dst

    def tables_np(self, src_rank: int, dst_rank: int):
        """The same two tables as contiguous int64 arrays (made once; what the C ABI takes)."""
        import numpy as np

        key = ("np", src_rank, dst_rank)
        cached = self._tables.get(key)
        if cached is None:
            s, d = self.tables(src_rank, dst_rank)
            cached = self._tables[key] = (np.asarray(s, dtype=np.int64), np.asarray(d, dtype=np.int64))
        return cached

    def outgoing(self, rank: int) -> List[int]:
        return [d for s, d in self.pairs() if s == rank]

    def incoming(self, rank: int) -> List[int]:
        return [s for s, d in self.pairs() if d == rank]

    def total_blocks(self) -> int:
        return sum(len(t.src_blocks) for t in self.transfers)

    def validate(self, num_blocks_of_rank: Callable[[int], int]) -> None:
        """Range-checks every id and rejects a destination block used twice."""
        seen_dst: Dict[int, set] = {}
        for t in self.transfers:
            nb_s, nb_d = num_blocks_of_rank(t.src_rank), num_blocks_of_rank(t.dst_rank)
            if any(b < 0 or b >= nb_s for b in t.src_blocks):
                raise ValueError(f"{t.request_id}: source block outside [0, {nb_s})")
            if any(b < 0 or b >= nb_d for b in t.dst_blocks):
                raise ValueError(f"{t.request_id}: destination block outside [0, {nb_d})")
            used = seen_dst.setdefault(t.dst_rank, set())
            for b in t.dst_blocks:
                if b in used:
                    raise ValueError(f"{t.request_id}: destination block {b} on rank {t.dst_rank} assigned twice")
                used.add(b)


class WaveLedger:
    """Host-side record of which (wave, source) moves have finished, shared by all ranks.

    A role switch that does not fit the pools moves in waves. The reference has
    no such record: it awaits every request's RPC before the next
    (elasticmm/engine/v0/backend.py:674-718) and frees source blocks without
    waiting for the copy (elasticmm/engine/v0/stage_engine.py:1336). Here every
    sink posts one completion per (wave, source) once its copy of that source's
    blocks has finished on the device; a source may reuse a wave's blocks when
    all of its sinks of that wave have posted, and a sink starts wave w of a
    source only when wave w - depth of that source is complete everywhere. No
    rank waits for ranks it does not exchange data with, and nobody meets at a
    barrier between waves.

    `store` is any torch.distributed key-value store (TCPStore, FileStore,
    HashStore, PrefixStore); counters live under `prefix`, which must be unique
    per migration (epoch) because counters are never reset.
    """

    def __init__(self, store, prefix: str, poll_s: float = 20e-6, timeout_s: float = 30.0):
        self.store = store
        self.prefix = prefix
        self.poll_s = poll_s
        self.timeout_s = timeout_s

    def _key(self, wave: int, source: int) -> str:
        return f"{self.prefix}/w{wave}/s{source}"

    def post(self, wave: int, source: int) -> int:
        """This sink's copy of `source`'s blocks of `wave` has finished; returns the new count."""
        return int(self.store.add(self._key(wave, source), 1))

    def count(self, wave: int, source: int) -> int:
        return int(self.store.add(self._key(wave, source), 0))

    def failed(self) -> Optional[str]:
        if int(self.store.add(f"{self.prefix}/failed_flag", 0)):
            return self.store.get(f"{self.prefix}/failed").decode("utf-8", "replace")
        return None

    def mark_failed(self, reason: str) -> None:
        """Marks the migration as failed so that ranks waiting in wait() stop waiting."""
        self.store.set(f"{self.prefix}/failed", reason.encode("utf-8", "replace")[:200])
        self.store.add(f"{self.prefix}/failed_flag", 1)

    def wait(self, wave: int, source: int, expected: int) -> None:
        """Returns once `expected` sinks have posted (wave, source); raises TimeoutError after
        `timeout_s`, RuntimeError if another rank marked the migration as failed."""
        if expected <= 0:
            return
        import time

        deadline = time.monotonic() + self.timeout_s
        spins, pause = 0, self.poll_s
        while self.count(wave, source) < expected:
            spins += 1
            if spins % 16 == 0:
                why = self.failed()
                if why is not None:
                    raise RuntimeError(f"migration failed on another rank: {why}")
            if time.monotonic() > deadline:
                raise TimeoutError(f"wave {wave} of source {source}: {self.count(wave, source)} of {expected} "
                                   f"sinks finished within {self.timeout_s} s")
            if pause:
                time.sleep(pause)
                pause = min(pause * 2, 200e-6)  # a long wait polls the store gently


def run_waves(plans: Sequence["MigrationPlan"], rank: int, ledger: WaveLedger, depth: int,
              launch: Callable[[int, int, List[object]], object],
              wait_done: Callable[[object], float],
              on_wave_landed: Optional[Callable[[int], None]] = None,
              wait_for_readers: bool = True) -> List[float]:
    """Drives one rank through a sequence of waves without a barrier between waves.

    Sink side. For wave w and each of its sources (in the plan's pull order):
    wait until all sinks have posted wave w - depth of that source, then
    `launch(w, source, earlier)` starts this sink's copy of that source's blocks,
    ordered after the handles in `earlier` (this sink's own copies of wave
    w - depth, whose destination blocks wave w may reuse); it returns a handle.
    After wave w has been launched, the waves up to w - depth + 1 are completed:
    `wait_done(handle)` blocks until a copy has finished and returns its
    duration in ms, `on_wave_landed` runs, and the wave is posted in the ledger.
    So with depth 2 a sink always has the next wave queued behind the running
    one, and runs at most `depth` waves ahead of the slowest sink that shares a
    source with it; depth 1 degenerates to one wave at a time.

    Source side. A source returns once every one of its waves is complete
    everywhere: from then on all the blocks it offered may be freed. A caller
    that ends the migration with a meeting of all ranks anyway passes
    wait_for_readers=False and lets that meeting carry the same guarantee.

    Returns this rank's per-wave durations (the longest copy of each wave, one
    entry per wave; empty for a rank that receives nothing in any wave).
    """
    if depth < 1:
        raise ValueError("depth must be at least 1")
    launched: List[List[Tuple[int, object]]] = []
    wave_ms: List[float] = []
    finished = 0  # waves [0, finished) of this rank are complete and posted
    is_sink = any(plan.incoming(rank) for plan in plans)

    def finish(w: int) -> None:
        longest = 0.0
        for _, handle in launched[w]:
            longest = max(longest, float(wait_done(handle)))
        if on_wave_landed is not None:
            on_wave_landed(w)
        if wait_for_readers or w + depth < len(plans):  # nobody reads the record of the last waves otherwise
            for source, _ in launched[w]:
                ledger.post(w, source)
        if is_sink:
            wave_ms.append(longest)  # 0.0 for a wave in which this sink receives nothing

    for w, plan in enumerate(plans):
        this_wave: List[Tuple[int, object]] = []
        earlier = [h for _, h in launched[w - depth]] if w >= depth else []
        for source in plan.pull_order(rank):
            if w >= depth:
                ledger.wait(w - depth, source, len(plans[w - depth].outgoing(source)))
            this_wave.append((source, launch(w, source, earlier)))
        launched.append(this_wave)
        while finished <= w - depth + 1:  # keep at most `depth` waves of this rank unposted
            finish(finished)
            finished += 1
    while finished < len(plans):
        finish(finished)
        finished += 1
    if wait_for_readers:
        for w, plan in enumerate(plans):
            n = len(plan.outgoing(rank))
            if n:
                ledger.wait(w, rank, n)
    return wave_ms
