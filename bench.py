#!/usr/bin/env python
"""KV-migration benchmark: payload GB/s of moving paged KV blocks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" migrates every request of the workload once.
  N = 1   Llama-7B-shaped pool (32 layers, 32 KV heads, fp16, 2048 blocks), 64 requests: each request is
          gathered from pool A into a contiguous buffer and scattered into pool B
          under an independent block table, in waves that fit the 2048-block pool.
  N = 2   Qwen2.5-VL-7B-shaped pool (28 layers, 4 KV heads, bf16), 128 requests with a 576-token image
          prefix: rank 0 -> rank 1 (the sink pulls).
  N = 4   LLaVA-13B-shaped pool (40 layers, 40 KV heads, fp16), 512 requests: 2 sources -> 2 sinks.
  N = 8   the same 512 requests: 2 sources -> 6 sinks. The KV of all requests exceeds the pools, so it
          moves in waves of half a pool; waves are not separated by a barrier (a completion ledger lets a
          sink start the next wave of a source as soon as the wave before the last is done everywhere).
For N > 1 launch under torchrun (one rank per GPU). The line's `value` is the
whole-job payload rate with tables resident on the device; `e2e` is the same
workload through the engine/v0 worker API with host block-id lists, table upload
and a device->host status read inside the timed region. Decode-time append (256 tokens
x 32 layers, 8 KV heads) and eviction + compaction (70B-shaped GQA pool) are reported as
extra objects at N = 1.

All data is synthetic: seeded N(0,1) values with the named shapes; no model
weights or datasets are involved. `--impl reference` times the CPU restatement
of the reference's torch index/copy path (oracle/) on the host cores.

Every line carries `verified_bit_exact`: before anything is timed, every request of every
wave is moved once and compared bit for bit on the device with the reference's own
indexing expression (`dst_layer[:, dst_ids]` against `src_layer[:, src_ids]`,
elasticmm/engine/v0/worker.py:604,633); for N > 1 the expected bytes travel from the
source to the sink through torch.distributed, independently of the kernels under test.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

GIB = float(1 << 30)

WORKLOADS = {
    "llama7b_cfg1": dict(L=32, H=32, D=128, BS=16, NB=2048, dtype="float16", requests=64,
                         tokens=("uniform", 128, 2048), prefix=0),
    "qwen25vl7b_cfg3": dict(L=28, H=4, D=128, BS=16, NB=16384, dtype="bfloat16", requests=128,
                            tokens=("uniform", 32, 1024), prefix=576),
    "llava13b_cfg4": dict(L=40, H=40, D=128, BS=16, NB=4096, dtype="float16", requests=512,
                          tokens=("loguniform", 256, 8192), prefix=0),
    "append_cfg2": dict(L=32, H=8, D=128, BS=16, NB=16384, dtype="bfloat16", T=256, pad_frac=0.01),
    "gqa70b_cfg5": dict(L=80, H=8, D=128, BS=16, NB=8192, dtype="bfloat16", occupancy=0.85,
                        evict_frac=0.30, tokens=("uniform", 512, 16384)),
}
DT = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def page_bytes(w):
    return w["BS"] * w["H"] * w["D"] * 2


def block_bytes(w):
    return 2 * w["L"] * page_bytes(w)


def request_blocks(w, seed):
    """Seeded request lengths -> block counts."""
    g = torch.Generator().manual_seed(seed)
    kind, lo, hi = w["tokens"]
    n = w["requests"]
    if kind == "uniform":
        toks = torch.randint(lo, hi + 1, (n,), generator=g)
    else:
        u = torch.rand(n, generator=g, dtype=torch.float64)
        toks = torch.exp(math.log(lo) + u * (math.log(hi) - math.log(lo))).round().long()
    toks = toks + w["prefix"]
    return [-(-int(t) // w["BS"]) for t in toks]


def make_waves(counts, capacity):
    waves, cur, used = [], [], 0
    for i, n in enumerate(counts):
        if used + n > capacity and cur:
            waves.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += n
    if cur:
        waves.append(cur)
    return waves


def build_requests(w, seed=1):
    """(counts, waves, reqs): seeded request sizes, the waves that fit the pool, and per request (in wave
    order) the source and destination block tables, slices of one seeded permutation per wave and side.
    Shared by the GPU arm and the CPU reference arm so that both move the same tables."""
    counts = request_blocks(w, seed)
    waves = make_waves(counts, w["NB"])
    g = torch.Generator().manual_seed(seed)
    reqs = []
    for wave in waves:
        sperm, dperm = torch.randperm(w["NB"], generator=g).tolist(), torch.randperm(w["NB"], generator=g).tolist()
        pos = 0
        for i in wave:
            reqs.append((sperm[pos:pos + counts[i]], dperm[pos:pos + counts[i]]))
            pos += counts[i]
    return counts, waves, reqs


def mem_available_gib():
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) / (1 << 20)
    except OSError:
        pass
    return 0.0


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with NVML while the timed region runs (read only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            try:  # CUDA index and NVML index differ under CUDA_VISIBLE_DEVICES
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def gpu_pool(w, device, seed, guard=False):
    shape = (2, w["NB"], w["BS"], w["H"], w["D"])
    dt = DT[w["dtype"]]
    if guard:
        out = []
        for _ in range(w["L"]):
            t = torch.empty(shape, device=device, dtype=dt)
            t.view(torch.int16).fill_(0x7FFF)
            out.append(t)
        return out
    g = torch.Generator(device=device).manual_seed(seed)
    return [torch.randn(shape, generator=g, device=device, dtype=dt) for _ in range(w["L"])]


def block_checksums(layers):
    total = None
    for t in layers:
        s = t.view(torch.int16).reshape(2, t.shape[1], -1).sum(dim=2, dtype=torch.int64).sum(dim=0)
        total = s if total is None else total + s
    return total


def timed(fn, steps, warmup, device, barrier=None):
    """Runs fn() warmup + steps times; returns total milliseconds of the timed steps (CUDA events)."""
    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize(device)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize(device)
    if barrier:
        barrier()
    return a.elapsed_time(b)


# ---------------------------------------------------------------------------
# CPU baseline (oracle port of the reference's torch index/copy path)
# ---------------------------------------------------------------------------

def cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


class CpuPath:
    """gather -> scatter of a workload on host tensors with the oracle port of the reference's torch
    index/copy path (extract_kv_blocks then write_kv_blocks), all torch threads.

    When the host has the memory, the pools have the workload's full block count and the requests use the
    same seeded tables as the GPU arm; otherwise the pool is cut to `nb` blocks (stated in the result) and the
    requests keep their sizes with tables drawn inside the smaller pool."""

    def __init__(self, wname, full=True, seed=1):
        from oracle import kv_oracle

        self.oracle = kv_oracle
        self.wname = wname
        # torchrun pins OMP_NUM_THREADS to 1 per rank; the CPU legs run on one rank only and may use every core
        torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))
        w = self.w = WORKLOADS[wname]
        pool_gib = w["NB"] * block_bytes(w) / GIB
        need_gib = 2 * pool_gib + 3 * max(request_blocks(w, seed)) * block_bytes(w) / GIB + 8
        self.full = bool(full and mem_available_gib() >= need_gib)
        self.nb = nb = w["NB"] if self.full else min(w["NB"], max(64, int(3 * GIB // block_bytes(w))))
        dt = DT[w["dtype"]]
        shape = (2, nb, w["BS"], w["H"], w["D"])
        tile = torch.randn(1 << 16).to(dt)
        self.src, self.dst = [], []
        for _ in range(w["L"]):
            t = torch.empty(shape, dtype=dt)
            flat = t.view(-1)
            whole = flat.numel() // tile.numel() * tile.numel()
            flat[:whole].view(-1, tile.numel())[:] = tile
            flat[whole:] = 0
            self.src.append(t)
            self.dst.append(torch.zeros(shape, dtype=dt))
        if self.full:
            self.counts, _, self.reqs = build_requests(w, seed)
            self.reqs = list(self.reqs)
        else:
            counts = [min(c, nb // 2) for c in request_blocks(w, seed)]
            gen = torch.Generator().manual_seed(seed)
            self.reqs = [(torch.randperm(nb, generator=gen)[:c].tolist(), torch.randperm(nb, generator=gen)[:c].tolist())
                         for c in counts]
        self.threads = torch.get_num_threads()
        # warm-up on one small request
        kv_oracle.write_kv_blocks(self.dst, [0, 1], kv_oracle.extract_kv_blocks(self.src, [2, 3]))

    def describe(self, reqs, moved):
        w = self.w
        pool = (f"the full {self.nb}-block host pools, seeded permutation tables"
                + (" (the GPU arm's)" if self.wname == "llama7b_cfg1" else "") if self.full
                else f"host pools cut to {self.nb} blocks (of {w['NB']}; host memory), request sizes kept")
        return (f"{reqs} of {len(self.reqs)} requests ({moved} blocks, {moved * block_bytes(w) / GIB:.1f} GiB payload) of "
                f"{self.wname} on {pool}; extract_kv_blocks then write_kv_blocks restated with torch CPU indexing; "
                f"{self.threads} torch threads, {os.cpu_count()} host cpus")

    def run(self, budget_s=None, max_requests=None):
        """One pass over the requests (all of them, or the first `max_requests`, or as many as fit `budget_s`)."""
        w = self.w
        moved, reqs, t_total = 0, 0, 0.0
        for s, d in self.reqs[: max_requests or len(self.reqs)]:
            t0 = time.perf_counter()
            self.oracle.write_kv_blocks(self.dst, d, self.oracle.extract_kv_blocks(self.src, s))
            t_total += time.perf_counter() - t0
            moved += len(s)
            reqs += 1
            if budget_s is not None and t_total > budget_s:
                break
        gbs = moved * block_bytes(w) / t_total / 1e9
        return {"value": round(gbs, 3), "unit": "GB/s", "cores": self.threads, "kind": "port",
                "sample": self.describe(reqs, moved), "requests": reqs, "blocks": moved,
                "nb_reduced_to": None if self.full else self.nb,
                "seconds": round(t_total, 2), "blocks_per_s": round(moved / t_total, 1), "cpu_model": cpu_model()}

    def run_c(self, budget_s):
        """The same requests with the plain-C restatement (one memcpy per page, all host threads)."""
        from oracle import kv_oracle_c

        threads = os.cpu_count() or 1
        w = self.w
        moved, t_total = 0, 0.0
        for s, d in self.reqs:
            t0 = time.perf_counter()
            kv_oracle_c.scatter(self.dst, d, kv_oracle_c.gather(self.src, s, threads=threads), threads=threads)
            t_total += time.perf_counter() - t0
            moved += len(s)
            if t_total > budget_s:
                break
        return {"value": round(moved * block_bytes(w) / t_total / 1e9, 3), "unit": "GB/s", "cores": threads,
                "kind": "port", "what": "plain-C restatement, one memcpy per page on pthreads",
                "seconds": round(t_total, 2)}


def cpu_baseline(wname, budget_s=12.0):
    """The bounded CPU leg printed beside the GPU line (about 20 s of CPU work on a 3 GiB pool)."""
    path = CpuPath(wname, full=False)
    out = path.run(budget_s)
    threads = torch.get_num_threads()
    try:  # the same path on one thread (a few seconds)
        torch.set_num_threads(1)
        path.threads = 1
        one = path.run(min(budget_s, 3.0))
        out["single_thread"] = {"value": one["value"], "unit": "GB/s", "cores": 1, "seconds": one["seconds"]}
    finally:
        torch.set_num_threads(threads)
        path.threads = threads
    try:
        out["alt_c_memcpy"] = path.run_c(min(budget_s, 6.0))
    except Exception as e:  # the C checker is optional for the baseline
        out["alt_c_memcpy"] = {"error": f"{type(e).__name__}: {e}"}
    return out


REFERENCE_ARM_BUDGET_S = 240.0  # CPU seconds the whole --impl reference run may take (steps + warm-up)


def reference_arm(args):
    """The reference's own torch index/copy path on the host cores, on the GPU arm's workload: at N = 1
    BASELINE config 1 as worded (2048-block pools, 64 requests, the same seeded tables) whenever the host
    has the memory and a full step fits the time budget; otherwise a bounded sample, named in `config`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wname = {1: "llama7b_cfg1", 2: "qwen25vl7b_cfg3"}.get(args.gpus, "llava13b_cfg4")
    w = WORKLOADS[wname]
    n_runs = max(1, args.steps + args.warmup)
    # Full-size host pools only where a whole step can fit the budget at all (assuming a generous 10 GB/s): the
    # 900 GiB of config 4 cannot, and 100 GiB of host pools would be filled for a sample that never needs them.
    seed = 1 if args.gpus == 1 else 4  # the request sizes of the GPU arm at this N
    workload_blocks = sum(request_blocks(w, seed))
    whole_gib = workload_blocks * block_bytes(w) / GIB
    path = CpuPath(wname, full=whole_gib * n_runs / 10.0 <= REFERENCE_ARM_BUDGET_S, seed=seed)
    probe = path.run(max_requests=2)  # sizes the step: seconds per block on this host
    total_blocks = sum(len(s) for s, _ in path.reqs)
    est_full = probe["seconds"] / max(1, probe["blocks"]) * total_blocks
    if est_full * n_runs <= REFERENCE_ARM_BUDGET_S:
        per_step = dict(max_requests=None)
    else:
        per_step = dict(budget_s=max(2.0, REFERENCE_ARM_BUDGET_S / n_runs))
    vals, base = [], None
    for i in range(args.warmup + args.steps):
        base = path.run(**per_step)
        if i >= args.warmup:
            vals.append(base)
    value = sum(v["value"] for v in vals) / len(vals)
    secs = sum(v["seconds"] for v in vals) / len(vals)
    base["value"] = round(value, 3)
    whole = base["requests"] == len(path.reqs) and path.full
    line = {
        "impl": "reference", "metric": "kv_migration_payload_GBps", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(secs * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": wname, "geometry": {k: w[k] for k in ("L", "H", "D", "BS", "NB", "dtype")},
                   "requests": w["requests"], "blocks_per_step": workload_blocks,
                   "sample_requests": base["requests"], "sample_blocks": base["blocks"],
                   "nb_reduced_to": base["nb_reduced_to"], "whole_workload_per_step": whole,
                   "path": "gather -> packed buffer -> scatter",
                   "note": "CPU restatement of the reference's torch index/copy path on host cores; the reference "
                           "is pure Python+torch on this path and needs Ray and vLLM to run as shipped; the "
                           "transport leg of a multi-GPU migration has no CPU counterpart"},
        "cpu_baseline": base,
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# N = 1
# ---------------------------------------------------------------------------

def bench_single(args):
    from elasticmm_b200 import KVPool, _lib, compact_plan, get_context
    from elasticmm_b200.engine.v0 import V0Worker

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    ctx = get_context(0)
    wname = args.workload
    w = WORKLOADS[wname]
    src_worker = V0Worker(dtype=w["dtype"], device=device, kv_cache=gpu_pool(w, device, 1))
    dst_worker = V0Worker(dtype=w["dtype"], device=device, kv_cache=gpu_pool(w, device, 0, guard=True))
    src, dst = src_worker.pool, dst_worker.pool
    counts, waves, reqs = build_requests(w, 1)  # (src ids, dst ids) per request, in wave order
    total_blocks = sum(counts)
    payload = total_blocks * block_bytes(w)
    dev_tables = [(src.upload_ids(s), dst.upload_ids(d)) for s, d in reqs]
    packed = src.new_packed(max(counts))
    flat = packed.view(-1)

    def packed_for(n):
        return flat[: src.packed_bytes(n) // 2].view(src.packed_shape(n))

    def step_device():
        for (s, d) in dev_tables:
            buf = packed_for(s.numel())
            src.gather(s, out=buf)
            dst.scatter(d, buf)

    def step_e2e():
        for (s, d) in reqs:
            dst_worker.write_kv_blocks(d, src_worker.extract_kv_blocks(s))
        rc, _ = ctx.status()  # device -> host read of the status word, synchronises
        assert rc == 0

    # Correctness gate before timing: every request of every wave is moved once and compared bit for bit on
    # the device with the reference's own indexing expression, dst_layer[:, dst_ids] against
    # src_layer[:, src_ids] per layer (waves reuse destination blocks, so each wave is checked before the next).
    verified, verified_requests, pos = True, 0, 0
    for wave in waves:
        for k in range(len(wave)):
            s_dev, d_dev = dev_tables[pos + k]
            buf = packed_for(s_dev.numel())
            src.gather(s_dev, out=buf)
            dst.scatter(d_dev, buf)
        rc, detail = ctx.status()
        assert rc == 0, f"device status {rc} ({detail})"
        for k in range(len(wave)):
            s_idx = torch.tensor(reqs[pos + k][0], device=device)
            d_idx = torch.tensor(reqs[pos + k][1], device=device)
            for ls, ld in zip(src.layers, dst.layers):
                verified = verified and bool(torch.equal(ld[:, d_idx].view(torch.int16), ls[:, s_idx].view(torch.int16)))
            verified_requests += 1
        pos += len(wave)
    assert verified, "gather -> scatter differs from the reference's indexing expression"

    l0 = ctx.launch_count
    with ClockSampler(0) as clocks:
        ms = timed(step_device, args.steps, args.warmup, device)
    launches = ctx.launch_count - l0 - args.warmup * 2 * len(reqs)
    value = payload * args.steps / (ms / 1e3) / 1e9
    peak, peak_kind = measured_peak()
    # gather reads and writes the payload once, scatter does the same: 4 x payload of HBM bytes per step
    achieved = 4 * payload * args.steps / (ms / 1e3) / 1e9
    def step_direct():
        for (s, d) in dev_tables:
            src.copy_blocks(dst, s, d)

    ms_direct = timed(step_direct, max(3, args.steps // 2), 3, device)
    direct_steps = max(3, args.steps // 2)
    # the same copies batched: one launch per wave over the concatenated tables (what a plan-level call issues)
    wave_tables, pos = [], 0
    for wave in waves:
        s_cat = torch.cat([dev_tables[pos + k][0] for k in range(len(wave))])
        d_cat = torch.cat([dev_tables[pos + k][1] for k in range(len(wave))])
        wave_tables.append((s_cat, d_cat))
        pos += len(wave)

    def step_direct_waves():
        for (s, d) in wave_tables:
            src.copy_blocks(dst, s, d)

    ms_dw = timed(step_direct_waves, direct_steps, 3, device)
    # gather -> per-request packed buffers -> scatter with one launch per wave for each direction
    many, pos = [], 0
    for wave in waves:
        s_lists = [reqs[pos + k][0] for k in range(len(wave))]
        d_lists = [reqs[pos + k][1] for k in range(len(wave))]
        many.append((src.many_tables(s_lists), dst.many_tables(d_lists, unique=True)))
        pos += len(wave)
    many_flat = torch.empty(max(src.packed_bytes(t[0][1]) for t in many) // 2, dtype=src.dtype, device=device)

    def step_many():
        for s_tab, d_tab in many:
            src.gather_many_into(s_tab, many_flat)
            dst.scatter_many_from(d_tab, many_flat)

    ms_many = timed(step_many, direct_steps, 3, device)
    del many_flat
    # the same through the worker methods with host id lists (tables built, staged and uploaded inside the timed region)
    wave_lists, pos = [], 0
    for wave in waves:
        wave_lists.append(([reqs[pos + k][0] for k in range(len(wave))], [reqs[pos + k][1] for k in range(len(wave))]))
        pos += len(wave)

    def step_many_api():
        for s_lists, d_lists in wave_lists:
            dst_worker.write_kv_blocks_many(d_lists, src_worker.extract_kv_blocks_many(s_lists))
        rc, _ = ctx.status()
        assert rc == 0

    ms_many_api = timed(step_many_api, direct_steps, 3, device)
    ms_e2e = timed(step_e2e, max(3, args.steps // 4), 3, device)
    e2e_steps = max(3, args.steps // 4)
    e2e_value = payload * e2e_steps / (ms_e2e / 1e3) / 1e9
    h2d = sum(4 * (len(s) + len(d)) for s, d in reqs)

    # What the reference itself executes on a GPU today: torch indexing per layer, torch.stack, index_put per
    # layer, with the synchronous upload of the id list (elasticmm/engine/v0/worker.py:597-608,628-633).
    def step_torch_index():
        for (s_ids, d_ids) in reqs:
            idx = torch.tensor(s_ids, dtype=torch.long, device=device)
            data = torch.stack([layer[:, idx] for layer in src.layers], dim=0)
            idx = torch.tensor(d_ids, dtype=torch.long, device=device)
            for l, layer in enumerate(dst.layers):
                layer[:, idx] = data[l]

    del packed, flat
    torch.cuda.empty_cache()
    ti_steps = max(2, args.steps // 10)
    try:
        ms_ti = timed(step_torch_index, ti_steps, 1, device)
        torch_index = {"value": round(payload * ti_steps / (ms_ti / 1e3) / 1e9, 2), "unit": "GB/s",
                       "ms_per_step": round(ms_ti / ti_steps, 3), "steps": ti_steps,
                       "path": "the reference's own expression on CUDA tensors: layer[:, idx] per layer, torch.stack, "
                               "layer[:, idx] = data per layer (torch indexing kernels, not this library)"}
    except Exception as e:
        torch_index = {"error": f"{type(e).__name__}: {e}"}
    torch.cuda.empty_cache()

    del dev_tables, wave_tables, many
    extras = {}
    if not args.skip_extras:
        src_worker = dst_worker = src = dst = None
        torch.cuda.empty_cache()
        extras["append"] = bench_append(ctx, device, args)
        torch.cuda.empty_cache()
        extras["compaction"] = bench_compaction(ctx, device, args)
        torch.cuda.empty_cache()
        extras["small_transfer"] = bench_small_transfer(ctx, device, args)
        torch.cuda.empty_cache()
    cpu = cpu_baseline(wname) if not args.skip_cpu else None
    kernel_name = "page_copy_ldg" if ctx.get_option(_lib.OPT_COPY_VARIANT) == _lib.COPY_LDG else "page_copy_bulk"

    line = {
        "metric": "kv_migration_payload_GBps", "value": round(value, 2), "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": wname, "geometry": {k: w[k] for k in ("L", "H", "D", "BS", "NB", "dtype")},
                   "requests": w["requests"], "blocks_per_step": total_blocks, "waves": len(waves), "small": args.small,
                   "payload_gib_per_step": round(payload / GIB, 2), "path": "gather -> packed buffer -> scatter",
                   "l2": f"inputs larger than L2 (two {w['NB'] * block_bytes(w) / GIB:.0f} GiB pools, "
                         f"{min(counts) * block_bytes(w) >> 20}..{max(counts) * block_bytes(w) >> 20} MiB per launch)",
                   "blocks_per_s": round(total_blocks * args.steps / (ms / 1e3), 1)},
        "verified_bit_exact": verified, "verified_waves": len(waves), "waves": len(waves),
        "verified_requests": verified_requests,
        "verified_how": "torch.equal of dst_layer[:, dst_ids] and src_layer[:, src_ids] (int16 views) per layer, "
                        "every request of every wave, on the device before timing",
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": round(TRAFFIC_RATIO["page_copy"] * 2 * payload / len(reqs)),
                     "peak_kind": f"of {peak_kind}", "frac_of_8tbs_nominal": round(achieved / 8000.0, 4),
                     "kernel": kernel_name, "algorithmic_bytes_per_launch":
                         round(2 * payload / len(reqs)), "avg_launch_us": round(ms * 1e3 / launches, 2)},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 16,
                "api": "V0Worker.extract_kv_blocks + write_kv_blocks per request, host id lists (tables of up to 128 ids "
                       "reach the device in the kernel arguments, longer ones through a pinned staging copy)",
                "steps": e2e_steps, "ms_per_step": round(ms_e2e / e2e_steps, 3)},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "cpu_baseline": cpu,
        "variants": {"torch_index_gpu": torch_index, "direct_block_copy": {
            "value": round(payload * direct_steps / (ms_direct / 1e3) / 1e9, 2), "unit": "GB/s",
            "hbm_gbs": round(2 * payload * direct_steps / (ms_direct / 1e3) / 1e9, 1),
            "ms_per_step": round(ms_direct / direct_steps, 3),
            "path": "pool A -> pool B in one launch per request, no packed buffer (the form used between GPUs)"},
            "direct_block_copy_per_wave": {
                "value": round(payload * direct_steps / (ms_dw / 1e3) / 1e9, 2), "unit": "GB/s",
                "hbm_gbs": round(2 * payload * direct_steps / (ms_dw / 1e3) / 1e9, 1),
                "ms_per_step": round(ms_dw / direct_steps, 3), "launches_per_step": len(waves),
                "path": "the same copies with one launch per wave over concatenated tables (plan-level batching)"},
            "gather_scatter_many_per_wave": {
                "value": round(payload * direct_steps / (ms_many / 1e3) / 1e9, 2), "unit": "GB/s",
                "hbm_gbs": round(4 * payload * direct_steps / (ms_many / 1e3) / 1e9, 1),
                "ms_per_step": round(ms_many / direct_steps, 3), "launches_per_step": 2 * len(waves),
                "path": "gather into one contiguous buffer per request, then scatter, all requests of a wave in one "
                        "launch per direction (emm_gather_many / emm_scatter_many)",
                "through_worker_api": {
                    "value": round(payload * direct_steps / (ms_many_api / 1e3) / 1e9, 2), "unit": "GB/s",
                    "ms_per_step": round(ms_many_api / direct_steps, 3),
                    "api": "V0Worker.extract_kv_blocks_many + write_kv_blocks_many per wave, host id lists, "
                           "output tensors allocated per call"}}},
    }
    line.update(extras)
    print(json.dumps(line))


# DRAM bytes (read + written, ncu dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic bytes for one
# page_copy_bulk launch: 880.88 MB read and 832.83 MB written for 2 x 880.80 MB algorithmic, captured on a 105-block
# launch of the --small case. Traffic grows in proportion to the blocks a launch moves, so the ratio is applied to
# this run's mean launch.
TRAFFIC_RATIO = {"page_copy": (880.883456 + 832.828416) / (2 * 880.80384)}


def bench_append(ctx, device, args):
    """Decode-time append: reshape_and_cache of [256, 8, 128] bf16 per layer into a 32-layer, 16384-block pool.
    Successive steps take their new-token K/V from a ring of buffers larger than L2 and fresh slot sets, so
    that the rows are read from HBM as in a decode loop (one step's 33 MB of rows would otherwise stay in L2)."""
    from elasticmm_b200 import KVPool

    w = WORKLOADS["append_cfg2"]
    pool = KVPool(gpu_pool(w, device, 2), ctx)
    L, T, H, D = w["L"], w["T"], w["H"], w["D"]
    g = torch.Generator().manual_seed(2)
    # a fresh slot set per step (decode advances), cycled from 16 precomputed mappings
    maps = []
    for _ in range(16):
        s = torch.randperm(w["NB"] * w["BS"], generator=g)[:T].clone()
        s[torch.randperm(T, generator=g)[: max(1, round(w["pad_frac"] * T))]] = -1
        maps.append(s.to(device))
    valid = int((maps[0] >= 0).sum())
    gd = torch.Generator(device=device).manual_seed(3)
    ring = 8  # 8 x (16.8 MB key + 16.8 MB value) = 268 MB, more than the 126 MB L2
    keys = [torch.randn(L, T, H, D, generator=gd, device=device, dtype=torch.bfloat16) for _ in range(ring)]
    values = [torch.randn(L, T, H, D, generator=gd, device=device, dtype=torch.bfloat16) for _ in range(ring)]
    it = {"i": 0}

    def per_layer():
        i = it["i"]
        it["i"] += 1
        s, key, value = maps[i % 16], keys[i % ring], values[i % ring]
        for l in range(L):
            pool.append(l, key[l], value[l], s)

    def all_layers():
        i = it["i"]
        it["i"] += 1
        pool.append_all_layers(keys[i % ring], values[i % ring], maps[i % 16])

    steps = max(args.steps, 50)
    out = {"workload": "append_cfg2", "tokens_per_step": T, "valid_tokens": valid, "layers": L,
           "l2": f"key/value rotate over {ring} buffer pairs ({ring * 2 * keys[0].numel() * 2 >> 20} MiB), slots over 16 sets"}
    ms = timed(all_layers, steps, 5, device)
    row = H * D * 2
    algo = valid * L * (4 * row + 8)  # K and V rows read and written, plus the slot
    peak, kind = measured_peak()
    out["all_layers_call"] = {"tokens_per_s": round(T * steps / (ms / 1e3)), "us_per_step": round(ms * 1e3 / steps, 2),
                              "launches_per_step": 1, "hbm_gbs": round(algo * steps / (ms / 1e3) / 1e9, 1),
                              "frac_of_peak": round(algo * steps / (ms / 1e3) / 1e9 / peak, 4), "peak_kind": f"of {kind}"}
    # the same launches replayed from a CUDA graph (16 steps on rotating buffers per graph): the kernel's own
    # rate, without the host time of the Python call between launches
    try:
        stream = torch.cuda.Stream(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            all_layers()
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(16):
                    all_layers()
        reps = max(4, steps // 4)
        ms = timed(graph.replay, reps, 3, device)
        n = reps * 16
        out["all_layers_graph_replay"] = {"tokens_per_s": round(T * n / (ms / 1e3)), "us_per_step": round(ms * 1e3 / n, 2),
                                          "launches_per_step": 1, "hbm_gbs": round(algo * n / (ms / 1e3) / 1e9, 1),
                                          "frac_of_peak": round(algo * n / (ms / 1e3) / 1e9 / peak, 4),
                                          "peak_kind": f"of {kind}"}
    except Exception as e:
        out["all_layers_graph_replay"] = {"error": f"{type(e).__name__}: {e}"}
    ms = timed(per_layer, steps, 5, device)
    out["per_layer_calls"] = {"tokens_per_s": round(T * steps / (ms / 1e3)), "us_per_step": round(ms * 1e3 / steps, 2),
                              "launches_per_step": L}
    # static buffers refilled in place every step, validated once; the step's stream is looked up once per step
    key_buf, value_buf, slot_buf = keys[0].clone(), values[0].clone(), maps[0].clone()
    bound = pool.bind_append(key_buf, value_buf, slot_buf)

    def per_layer_bound():
        slot_buf.copy_(maps[it["i"] % 16])
        it["i"] += 1
        stream = torch.cuda.current_stream(device).cuda_stream
        launch = bound.raw
        for l in range(L):
            if launch(l, stream):
                bound(l, stream)  # raises with the library's message

    ms = timed(per_layer_bound, steps, 5, device)
    out["per_layer_bound_calls"] = {"tokens_per_s": round(T * steps / (ms / 1e3)),
                                    "us_per_step": round(ms * 1e3 / steps, 2), "launches_per_step": L,
                                    "what": "static key/value/slot buffers validated once (KVPool.bind_append -> "
                                            "emm_append_bound), one three-argument foreign call per layer"}
    # CUDA-graph replay of the per-layer sequence (how a captured decode step issues it)
    try:
        stream = torch.cuda.Stream(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            for l in range(L):
                bound(l, stream.cuda_stream)
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                for l in range(L):
                    bound(l, stream.cuda_stream)
        ms = timed(graph.replay, steps, 5, device)
        out["per_layer_graph_replay"] = {"tokens_per_s": round(T * steps / (ms / 1e3)),
                                         "us_per_step": round(ms * 1e3 / steps, 2), "launches_per_step": L}
    except Exception as e:  # graph capture is a reporting extra, not part of the contract
        out["per_layer_graph_replay"] = {"error": f"{type(e).__name__}: {e}"}
    bound.release()
    return out


def bench_small_transfer(ctx, device, args):
    """Wall-clock cost of moving one short request through the manager API, device synchronised per
    transfer as the reference's manager does: 15 blocks (a 234-token Qwen2.5-VL request, the example
    size the reference's engine README quotes) between two pools on this GPU."""
    from elasticmm_b200.engine.v0 import KVTransferMetrics, TransferMethod, V0KVTransferManager, V0Worker

    w = dict(WORKLOADS["qwen25vl7b_cfg3"], NB=1024)
    src = V0Worker(dtype=w["dtype"], device=device, kv_cache=gpu_pool(w, device, 7))
    dst = V0Worker(dtype=w["dtype"], device=device, kv_cache=gpu_pool(w, device, 0, guard=True))
    g = torch.Generator().manual_seed(7)
    out = {"workload": "15 blocks of qwen25vl7b geometry (13.1 MiB payload)", "blocks": 15}
    for name, method in (("p2p_copy", TransferMethod.P2P_COPY), ("b200_peer", TransferMethod.B200_PEER)):
        metrics = KVTransferMetrics("decoding", block_bytes=src.pool.block_bytes())
        mgr = V0KVTransferManager(transfer_method=method, metrics_callback=metrics.record_kv_transfer)
        mgr.register_worker(0, src, "prefill")
        mgr.register_worker(1, dst, "decoding")
        n_iter = 300
        tables = [(torch.randperm(w["NB"], generator=g)[:15].tolist(), torch.randperm(w["NB"], generator=g)[:15].tolist())
                  for _ in range(n_iter)]
        for s_ids, d_ids in tables[:20]:
            mgr.transfer_kv_cache_sync("warm", 0, 1, s_ids, d_ids)
        t0 = time.perf_counter()
        for s_ids, d_ids in tables:
            assert mgr.transfer_kv_cache_sync("r", 0, 1, s_ids, d_ids)
        dt = time.perf_counter() - t0
        out[name] = {"us_per_transfer": round(dt / n_iter * 1e6, 1), "blocks_per_s": round(15 * n_iter / dt),
                     "payload_gbs": round(15 * src.pool.block_bytes() * n_iter / dt / 1e9, 1)}
    out["gain_cost_params"] = {k: round(v, 7) for k, v in metrics.gain_cost_params().items()}
    return out


def bench_compaction(ctx, device, args):
    """Eviction + defragmentation: evict 30 % of the requests of an 85 %-full 8192-block pool, compact the survivors."""
    from elasticmm_b200 import KVPool, compact_plan

    w = WORKLOADS["gqa70b_cfg5"]
    pool = KVPool(gpu_pool(w, device, 5), ctx)
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(w["NB"], generator=g).tolist()
    tables, used = [], 0
    while True:
        n = -(-int(torch.randint(w["tokens"][1], w["tokens"][2] + 1, (1,), generator=g)) // w["BS"])
        if used + n > w["occupancy"] * w["NB"]:
            break
        tables.append(perm[used:used + n])
        used += n
    stamps = torch.rand(len(tables), generator=g)
    evict = set(torch.argsort(stamps)[: max(1, round(w["evict_frac"] * len(tables)))].tolist())
    flat = [b for i, t in enumerate(tables) if i not in evict for b in t]
    t0 = time.perf_counter()
    new_ids, move_src, move_dst = compact_plan(flat, w["NB"])
    plan_ms = (time.perf_counter() - t0) * 1e3
    s_dev, d_dev = pool.upload_ids(move_src), pool.upload_ids(move_dst)
    before = block_checksums(pool.layers)
    # Re-running the same plan copies the same source blocks to the same holes: identical traffic every step.
    steps = max(5, args.steps // 4)
    ms = timed(lambda: pool.copy_blocks(pool, s_dev, d_dev), steps, 3, device)
    after = block_checksums(pool.layers)
    ok = bool(torch.equal(after[torch.tensor(new_ids.tolist(), device=device)],
                          before[torch.tensor(flat, device=device)]))
    moved = len(move_src)
    algo = 2 * moved * block_bytes(w)
    peak, kind = measured_peak()
    gbs = algo * steps / (ms / 1e3) / 1e9
    return {"workload": "gqa70b_cfg5", "requests": len(tables), "evicted": len(evict), "live_blocks": len(flat),
            "moved_blocks": moved, "plan_ms_host": round(plan_ms, 3), "ms_per_compaction": round(ms / steps, 3),
            "hbm_gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4), "peak_kind": f"of {kind}",
            "blocks_per_s": round(moved * steps / (ms / 1e3), 1), "verified_checksum": ok}


# ---------------------------------------------------------------------------
# N > 1
# ---------------------------------------------------------------------------

NVLINK_NOMINAL_GBS = 900.0  # NVLink 5, per direction per GPU


def build_wave_plans(w, sources, sinks, seed=4):
    """Splits the workload's requests over the sources, assigns each a seeded sink, and packs them into waves.

    When everything fits the pools at once there is a single wave. Otherwise a wave may occupy half of every
    pool (source and sink blocks of wave k are reused by wave k + 2, so two waves can be in flight). Within a wave a source fills its half so that its sinks receive about the same
    number of blocks: it repeatedly gives the sink that has the least so far the largest remaining request
    that still fits. Block tables are seeded permutations of the half the wave may use."""
    from elasticmm_b200.engine.v0 import MigrationPlan, Transfer

    counts = request_blocks(w, seed)
    g = torch.Generator().manual_seed(seed)
    assign = torch.randint(0, len(sinks), (len(counts),), generator=g).tolist()
    per_source = [sum(c for i, c in enumerate(counts) if i % len(sources) == k) for k in range(len(sources))]
    per_sink = [sum(c for i, c in enumerate(counts) if assign[i] == j) for j in range(len(sinks))]
    one_wave = max(per_source) <= w["NB"] and max(per_sink) <= w["NB"]  # everything fits the pools at once
    half = w["NB"] if one_wave else w["NB"] // 2
    remaining = {s: {d: sorted((i for i in range(len(counts)) if i % len(sources) == k and sinks[assign[i]] == d),
                               key=lambda i: -counts[i]) for d in sinks} for k, s in enumerate(sources)}
    plans, wv = [], 0
    carry = {s: {d: 0.0 for d in sinks} for s in sources}  # blocks a sink is behind (+) or ahead (-) of its fair share
    while any(lst for per in remaining.values() for lst in per.values()):
        base = 0 if one_wave else (wv % 2) * half
        plan = MigrationPlan()
        sink_used = {d: 0 for d in sinks}
        sink_perm = {d: (torch.randperm(half, generator=torch.Generator().manual_seed(77 * wv + d)) + base).tolist()
                     for d in sinks}
        for s in sources:
            perm = (torch.randperm(half, generator=torch.Generator().manual_seed(1000 * wv + s)) + base).tolist()
            pos, given = 0, {d: 0 for d in sinks}
            # A sink's fair share of this source's wave is proportional to what it still has to receive from the
            # source (so that all sinks finish together), plus what it is owed from earlier waves.
            owed = {d: sum(counts[i] for i in remaining[s][d]) for d in sinks}
            left = sum(owed.values())
            budget = {d: (min(half, left) * owed[d] / left if left else 0.0) + carry[s][d] for d in sinks}

            def give(d, i):
                nonlocal pos
                n = counts[i]
                plan.add(Transfer(f"req{i}", s, d, tuple(perm[pos:pos + n]),
                                  tuple(sink_perm[d][sink_used[d]:sink_used[d] + n])))
                pos += n
                sink_used[d] += n
                given[d] += n
                remaining[s][d].remove(i)

            def fits(d, i):
                return pos + counts[i] <= half and sink_used[d] + counts[i] <= half

            # first every sink's share, largest requests first, the sink that is owed most first ...
            for d in sorted(sinks, key=lambda d: -budget[d]):
                for i in list(remaining[s][d]):
                    if fits(d, i) and given[d] + counts[i] <= budget[d]:
                        give(d, i)
            # ... then the rest of the source's half, always to the sink that is furthest below its share
            while True:
                pick = None
                for d in sorted(sinks, key=lambda d: given[d] - budget[d]):
                    pick = next(((d, i) for i in remaining[s][d] if fits(d, i)), None)
                    if pick:
                        break
                if pick is None:
                    break
                give(*pick)
            for d in sinks:
                carry[s][d] = max(-half, min(half, budget[d] - given[d])) if remaining[s][d] else 0.0
        assert plan.transfers, "a request does not fit an empty wave"
        plans.append(plan)
        wv += 1
    return plans


def bench_multi(args):
    import hashlib

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # send/recv and peer loads only: no NVLink multicast binding
    import torch.distributed as dist

    from elasticmm_b200.engine.v0 import V0Worker
    from elasticmm_b200.engine.v0.transport import WaveLedger

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    store = dist.distributed_c10d._get_default_store()
    t_start = time.monotonic()

    if world == 2:
        wname, sources, sinks = "qwen25vl7b_cfg3", [0], [1]
    elif world == 4:
        wname, sources, sinks = "llava13b_cfg4", [0, 1], [2, 3]
    else:
        wname, sources, sinks = "llava13b_cfg4", [0, 1], list(range(2, world))
    w = WORKLOADS[wname]
    is_src = rank in sources
    worker = V0Worker(worker_id=rank, dtype=w["dtype"], device=device, global_rank=rank, world_size=world,
                      kv_cache=gpu_pool(w, device, 100 + rank, guard=not is_src))
    worker.init_global_nccl()
    handles = [None] * world
    dist.all_gather_object(handles, (worker.get_ipc_handles(), worker.get_pool_desc()))
    for peer in (sinks if is_src else sources):  # sources map sinks (push variant), sinks map sources (pull)
        worker.attach_peer_pool(peer, handles[peer][0], handles[peer][1])
    nxt = (rank + 1) % world  # ring neighbour, for the all-ranks exchange variant
    if nxt not in worker.peer_pools:
        worker.attach_peer_pool(nxt, handles[nxt][0], handles[nxt][1])

    plans = build_wave_plans(w, sources, sinks)
    total_blocks = sum(p.total_blocks() for p in plans)
    payload = total_blocks * block_bytes(w)
    kv = worker.kv_cache

    # device-resident tables per wave: a sink holds (src ids, dst ids) per source, a source per sink (push variant)
    pull_tables = [{s: tuple(worker.pool.upload_ids(t) for t in plan.tables(s, rank)) for s in plan.incoming(rank)}
                   for plan in plans]
    push_tables = [[(d,) + tuple(worker.pool.upload_ids(t) for t in plan.tables(rank, d)) for d in plan.push_order(rank)]
                   for plan in plans]
    epoch = {"n": 0}

    def ledger(tag):
        epoch["n"] += 1
        return WaveLedger(store, f"bench/{tag}/{epoch['n']}")

    def barrier():
        dist.barrier()

    def max_ms(ms):
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(flag):
        t = torch.tensor([1 if flag else 0], device=device, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    wave_times = []

    def step_pull():
        res = worker.migrate_waves(plans, ledger("pull"), depth=2, tables=pull_tables)
        assert "error" not in res, res
        wave_times.append(res["wave_ms"])

    def step_e2e():
        res = worker.migrate_waves(plans, ledger("e2e"), depth=2)
        assert "error" not in res, res

    def step_method(method):
        def run():
            for plan in plans:
                res = worker.migrate(plan, method=method)
                assert "error" not in res, res
        return run

    def step_push_resident():
        for per in push_tables:
            for peer, si, di in per:  # one sink at a time, sources start at different sinks
                worker.pool.copy_blocks(worker.peer_pools[peer], si, di)
            torch.cuda.synchronize(device)
            dist.barrier()  # blocks of a wave are reused only after every copy of the wave has landed

    # ---- correctness gates (nothing here is timed) --------------------------------------------------------
    def verify_wave(plan):
        """Full bit compare of one wave: for every transfer, in the plan's order on every rank, the source
        evaluates the reference's expression on its own pool (stack of layer[:, src_ids]) and ships it with
        torch.distributed; the sink evaluates the same expression on what landed (layer[:, dst_ids]) and
        compares with torch.equal."""
        ok = True
        for t in plan.transfers:
            if t.src_rank == rank:
                idx = torch.tensor(t.src_blocks, dtype=torch.long, device=device)
                dist.send(torch.stack([layer[:, idx] for layer in kv], dim=0), dst=t.dst_rank)
                torch.cuda.current_stream(device).synchronize()  # one request's copy in flight at a time
            elif t.dst_rank == rank:
                idx = torch.tensor(t.dst_blocks, dtype=torch.long, device=device)
                got = torch.stack([layer[:, idx] for layer in kv], dim=0)
                want = torch.empty_like(got)
                dist.recv(want, src=t.src_rank)
                ok = ok and bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
        return ok

    def reset_sinks():
        if not is_src:
            for layer in kv:
                layer.view(torch.int16).fill_(0x7FFF)
        torch.cuda.synchronize(device)
        dist.barrier()

    def sample_of(plan, sink):
        """The sampled request of a (wave, sink): its smallest transfer, first 8 blocks."""
        mine = [t for t in plan.transfers if t.dst_rank == sink]
        if not mine:
            return None
        t = min(mine, key=lambda t: (len(t.src_blocks), t.request_id))
        return t.src_rank, t.src_blocks[:8], t.dst_blocks[:8]

    def digest(blocks):
        idx = torch.tensor(blocks, dtype=torch.long, device=device)
        data = torch.stack([layer[:, idx] for layer in kv], dim=0).view(torch.int16).cpu()
        return hashlib.sha256(data.numpy().tobytes()).hexdigest()

    verified = {}
    # 1. the timed path itself (waves in flight two deep): SHA-256 of a sampled request per wave and sink, taken
    #    when the wave has landed and while later waves are running, against the source's digest of the same blocks
    landed = {}

    def on_wave_landed(wv):
        smp = sample_of(plans[wv], rank)
        if smp is not None:
            landed[wv] = digest(smp[2])

    res = worker.migrate_waves(plans, ledger("gate"), depth=2, tables=pull_tables, on_wave_landed=on_wave_landed)
    assert "error" not in res, res
    expected = {}
    for wv, plan in enumerate(plans):
        for d in sinks:
            smp = sample_of(plan, d)
            if smp is not None and smp[0] == rank:
                expected[(wv, d)] = digest(smp[1])
    gathered = [None] * world
    dist.all_gather_object(gathered, (expected, landed))
    want_all = {k: v for e, _ in gathered for k, v in e.items()}
    ok = all(gathered[d][1].get(wv) == h for (wv, d), h in want_all.items())
    verified["pull_waves_in_flight_sha256_samples"] = all_true(ok and len(want_all) > 0)
    sampled = len(want_all)
    # 2. every request of every wave, bit for bit, for each transport
    verified_waves = {}
    for method in ("pull", "alltoall", "nccl"):
        if method == "alltoall":
            try:
                worker.init_native_nccl()
            except Exception as e:
                verified[method] = f"unavailable: {type(e).__name__}: {e}"
                continue
        reset_sinks()
        ok, n_ok = True, 0
        for plan in plans:
            r = worker.migrate(plan, method=method)
            good = "error" not in r and verify_wave(plan)
            ok = ok and good
            n_ok += 1 if all_true(good) else 0
        verified[method] = all_true(ok)
        verified_waves[method] = n_ok
    verified_all = all(v is True for v in verified.values())

    # ---- reference rates measured in this run --------------------------------------------------------------
    probe = {}
    one_gib = torch.empty(1 << 30, dtype=torch.uint8, device=device)
    two_gib = torch.empty(1 << 30, dtype=torch.uint8, device=device)
    if worker._nccl_comm is not None:
        # raw ncclSend/ncclRecv between the first source and the first sink, no pack or unpack: the library's ceiling
        table = {}
        for mib in (64, 256, 1024):
            n = mib << 20

            def nccl_pair():
                if rank == sources[0]:
                    worker.ctx.send_packed(worker._nccl_comm, one_gib[:n], sinks[0])
                elif rank == sinks[0]:
                    worker.ctx.recv_packed(worker._nccl_comm, one_gib[:n], sources[0])

            def nccl_both():
                if rank in (sources[0], sinks[0]):
                    other = sinks[0] if rank == sources[0] else sources[0]
                    worker.ctx.exchange(worker._nccl_comm, [(True, one_gib[:n], other), (False, two_gib[:n], other)])

            ms_p = max_ms(timed(nccl_pair, 5, 2, device, barrier))
            ms_b = max_ms(timed(nccl_both, 5, 2, device, barrier))
            table[f"{mib}MiB"] = {"one_way": round(n * 5 / (ms_p / 1e3) / 1e9, 1),
                                  "both_ways_per_direction": round(n * 5 / (ms_b / 1e3) / 1e9, 1)}
        probe["nccl_sendrecv_gbs"] = table
        probe["nccl_sendrecv_1gib_gbs"] = table["1024MiB"]["one_way"]
    del one_gib, two_gib
    # one contiguous flow through the copy kernel: the first sink loads the first quarter of the first source's pool
    quarter = w["NB"] // 4
    flow_ids = worker.pool.upload_ids(list(range(quarter)))

    def one_flow():
        if rank == sinks[0]:
            worker.peer_pools[sources[0]].copy_blocks(worker.pool, flow_ids, flow_ids)

    ms_f = max_ms(timed(one_flow, 3, 1, device, barrier))
    probe["single_flow_contiguous_pull_gbs"] = round(quarter * block_bytes(w) * 3 / (ms_f / 1e3) / 1e9, 1)

    # ---- timed: headline, end to end -------------------------------------------------------------------------
    l0 = worker.ctx.launch_count
    wave_times.clear()
    with ClockSampler(local) as clocks:
        ms = max_ms(timed(step_pull, args.steps, args.warmup, device, barrier))
    launches = worker.ctx.launch_count - l0 - args.warmup * sum(len(t) for t in pull_tables)
    lt = torch.tensor([launches], device=device, dtype=torch.int64)
    dist.all_reduce(lt)
    value = payload * args.steps / (ms / 1e3) / 1e9
    # per wave: how far apart the sinks' device times are (mean over the timed steps)
    mine = [sum(col) / len(col) for col in zip(*wave_times[-args.steps:])] if wave_times and wave_times[-1] else []
    all_waves = [None] * world
    dist.all_gather_object(all_waves, mine)
    per_wave = [[aw[k] for aw in all_waves if len(aw) > k] for k in range(len(plans))]
    spread = [max(c) - min(c) for c in per_wave if c]
    longest = [max(c) for c in per_wave if c]

    e2e_steps = max(2, args.steps // 4)
    ms_e = max_ms(timed(step_e2e, e2e_steps, 2, device, barrier))
    h2d = sum(8 * len(t.src_blocks) for p in plans for t in p.transfers)

    variants = {}
    deadline = t_start + float(os.environ.get("EMM_BENCH_TIME_LIMIT_S", "420"))

    def time_left():
        """Every rank takes rank 0's view of the clock, so that all skip the same variants."""
        t = torch.tensor([1 if time.monotonic() < deadline else 0], device=device, dtype=torch.int32)
        dist.broadcast(t, src=0)
        return bool(t.item())

    def variant(name, fn, steps, path, extra=None):
        if not time_left():
            variants.setdefault("skipped_for_time", []).append(name)
            return
        try:
            ms_v = max_ms(timed(fn, steps, 2, device, barrier))
            variants[name] = {"value": round(payload * steps / (ms_v / 1e3) / 1e9, 2), "unit": "GB/s",
                              "per_source_egress_gbs": round(payload * steps / (ms_v / 1e3) / 1e9 / len(sources), 2),
                              "ms_per_step": round(ms_v / steps, 3), "path": path}
            if extra:
                variants[name].update(extra)
        except Exception as e:  # a variant is an extra; its failure is reported, the headline stands
            variants[name] = {"error": f"{type(e).__name__}: {e}"}

    if not args.skip_extras:
        v_steps = max(2, args.steps // 4)
        variant("pull_wave_at_a_time", step_method("pull"), v_steps,
                "the same direct loads with every wave closed by an agreement of all ranks before the next starts")
        variant("peer_push", step_push_resident, v_steps,
                "sources store into the sinks' peer-mapped pools (same kernel, other direction), a barrier per wave")
        if worker._nccl_comm is not None:
            variant("nccl_alltoall_pipelined", step_method("alltoall"), v_steps,
                    "per layer chunk: one gather laid out [sink][layer][plane][blocks], one grouped exchange with one "
                    "ncclSend per sink and one ncclRecv per source, one scatter; three streams, two staging slots",
                    {"verified_bit_exact": verified.get("alltoall")})
            variant("nccl_staged", step_method("nccl"), v_steps,
                    "per pair: emm_send_blocks / emm_recv_blocks, pack -> ncclSend, ncclRecv -> unpack on library streams",
                    {"verified_bit_exact": verified.get("nccl")})
        # Every rank a source and a sink at once (the rebalancing exchange): rank r loads the lower half of
        # rank r+1's pool into the upper half of its own. Last, because it overwrites pool contents.
        half = w["NB"] // 2
        ring_src = worker.pool.upload_ids(torch.randperm(half, generator=torch.Generator().manual_seed(rank)).tolist())
        ring_dst = worker.pool.upload_ids((torch.randperm(half, generator=torch.Generator().manual_seed(50 + rank)) + half).tolist())

        def step_ring():
            worker.peer_pools[nxt].copy_blocks(worker.pool, ring_src, ring_dst)
            torch.cuda.synchronize(device)
            dist.barrier()

        if time_left():
            ring_steps = max(3, args.steps // 2)
            ms_r = max_ms(timed(step_ring, ring_steps, 2, device, barrier))
            ring_bytes = world * half * block_bytes(w)
            variants["ring_exchange_all_ranks"] = {
                "value": round(ring_bytes * ring_steps / (ms_r / 1e3) / 1e9, 2), "unit": "GB/s",
                "per_gpu_ingress_gbs": round(ring_bytes / world * ring_steps / (ms_r / 1e3) / 1e9, 2),
                "ms_per_step": round(ms_r / ring_steps, 3),
                "path": "every rank pulls half of the next rank's pool into its own at the same time"}

    if rank == 0:
        per_src_gbs = value / len(sources)
        line = {
            "metric": "kv_migration_payload_GBps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
            "config": {"workload": wname, "geometry": {k: w[k] for k in ("L", "H", "D", "BS", "NB", "dtype")},
                       "requests": w["requests"], "blocks_per_step": total_blocks, "waves": len(plans),
                       "payload_gib_per_step": round(payload / GIB, 2), "sources": sources, "sinks": sinks,
                       "path": "one direct-load kernel per (wave, source, sink) launched by the sink, its sources side by "
                               "side on separate streams with grids capped to one CTA per SM in total: NVLink loads "
                               "from the source's peer-mapped pool, local stores; waves of half a pool, two in flight, "
                               "ordered by a completion ledger instead of a barrier", "l2": "inputs larger than L2",
                       "per_source_egress_gbs": round(per_src_gbs, 2),
                       "per_sink_ingress_gbs": round(value / len(sinks), 2),
                       "per_pair_mean_gbs": round(value / (len(sources) * len(sinks)), 2),
                       "per_sink_ingress_frac_of_900": round(value / len(sinks) / NVLINK_NOMINAL_GBS, 4),
                       "blocks_per_s": round(total_blocks * args.steps / (ms / 1e3), 1),
                       "wave_sink_ms": {"longest_mean": round(sum(longest) / max(1, len(longest)), 3),
                                        "max_minus_min_mean": round(sum(spread) / max(1, len(spread)), 3),
                                        "max_minus_min_worst": round(max(spread), 3) if spread else None}},
            "verified_bit_exact": verified_all, "verified_waves": verified_waves, "waves": len(plans),
            "verified_methods": verified, "verified_sha256_samples": sampled,
            "verified_how": "before timing: (1) the timed path with two waves in flight, SHA-256 of a sampled request per "
                            "wave and sink taken while later waves run, against the source's digest; (2) per transport, "
                            "every request of every wave: the source ships stack(layer[:, src_ids]) through "
                            "torch.distributed and the sink compares it with stack(layer[:, dst_ids]) by torch.equal",
            "roofline": {"bound": "nvlink", "achieved": round(per_src_gbs, 1), "peak": NVLINK_NOMINAL_GBS,
                         "unit": "GB/s", "frac": round(per_src_gbs / NVLINK_NOMINAL_GBS, 4), "traffic": None,
                         "peak_kind": "of nominal NVLink 5 per direction per GPU (source egress is the bound)",
                         "measured_in_this_run": probe, "kernel": "page_copy_ldg (peer loads)"},
            "e2e": {"value": round(payload * e2e_steps / (ms_e / 1e3) / 1e9, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 16 * len(sinks),
                    "api": "V0Worker.migrate_waves(plans, ledger) with host id lists", "steps": e2e_steps},
            "gpu_launches": int(lt.item()),
            "clocks": clocks.summary(),
            "variants": variants,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true",
                    help="N=1: the same geometries on pools of a few GiB and 8 requests (the case profiled under ncu)")
    ap.add_argument("--workload", default="llama7b_cfg1",
                    choices=["llama7b_cfg1", "qwen25vl7b_cfg3", "llava13b_cfg4"],
                    help="N=1: pool geometry and request mix of the gather -> scatter step (default: the headline one)")
    ap.add_argument("--skip-extras", action="store_true", help="N=1: skip the append and compaction objects")
    ap.add_argument("--skip-cpu", action="store_true", help="N=1: skip the CPU baseline leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.small:
        WORKLOADS["llama7b_cfg1"].update(NB=256, requests=8)
        WORKLOADS["qwen25vl7b_cfg3"].update(NB=4096, requests=16)
        WORKLOADS["llava13b_cfg4"].update(NB=256, requests=8, tokens=("loguniform", 256, 2048))
        WORKLOADS["append_cfg2"].update(NB=1024)
        WORKLOADS["gqa70b_cfg5"].update(NB=512, tokens=("uniform", 512, 2048))
    if args.impl == "reference":
        reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        bench_single(args)
    else:
        bench_multi(args)


if __name__ == "__main__":
    main()
