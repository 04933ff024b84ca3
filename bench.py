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
  N = 8   the same 512 requests: 2 sources -> 6 sinks, in waves bounded by the pools.
For N > 1 launch under torchrun (one rank per GPU). The line's `value` is the
whole-job payload rate with tables resident on the device; `e2e` is the same
workload through the engine/v0 worker API with host block-id lists, table upload
and a device->host status read inside the timed region. Decode-time append (256 tokens
x 32 layers, 8 KV heads) and eviction + compaction (70B-shaped GQA pool) are reported as
extra objects at N = 1.

All data is synthetic: seeded N(0,1) values with the named shapes; no model
weights or datasets are involved. `--impl reference` times the CPU restatement
of the reference's torch index/copy path (oracle/) on the host cores.
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


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


NVLINK_PEER_COPY_GBS = 770.0  # measured peer copy per direction per GPU on this pool


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
    """gather -> scatter of a workload's geometry on host tensors with the oracle port of the
    reference's torch index/copy path, all torch threads. Bounded: a reduced pool (about 3 GiB)
    and as many requests as fit a time budget."""

    def __init__(self, wname):
        from oracle import kv_oracle

        self.oracle = kv_oracle
        self.wname = wname
        # torchrun pins OMP_NUM_THREADS to 1 per rank; the CPU legs run on one rank only and may use every core
        torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))
        w = self.w = WORKLOADS[wname]
        self.nb = nb = min(w["NB"], max(64, int(3 * GIB // block_bytes(w))))
        dt = DT[w["dtype"]]
        shape = (2, nb, w["BS"], w["H"], w["D"])
        tile = torch.randn(1 << 16).to(dt)
        self.src, self.dst = [], []
        for _ in range(w["L"]):
            t = torch.zeros(shape, dtype=dt)
            flat = t.view(-1)
            whole = flat.numel() // tile.numel() * tile.numel()
            flat[:whole].view(-1, tile.numel())[:] = tile
            self.src.append(t)
            self.dst.append(torch.zeros(shape, dtype=dt))
        self.counts = [min(c, nb // 2) for c in request_blocks(w, 1)]
        self.gen = torch.Generator().manual_seed(1)
        self.threads = torch.get_num_threads()
        # warm-up on one small request
        kv_oracle.write_kv_blocks(self.dst, [0, 1], kv_oracle.extract_kv_blocks(self.src, [2, 3]))

    def run(self, budget_s):
        w, nb = self.w, self.nb
        moved, reqs, t_total = 0, 0, 0.0
        for c in self.counts:
            s = torch.randperm(nb, generator=self.gen)[:c].tolist()
            d = torch.randperm(nb, generator=self.gen)[:c].tolist()
            t0 = time.perf_counter()
            self.oracle.write_kv_blocks(self.dst, d, self.oracle.extract_kv_blocks(self.src, s))
            t_total += time.perf_counter() - t0
            moved += c
            reqs += 1
            if t_total > budget_s:
                break
        gbs = moved * block_bytes(w) / t_total / 1e9
        return {"value": round(gbs, 3), "unit": "GB/s", "cores": self.threads, "kind": "port",
                "sample": f"{reqs} requests ({moved} blocks, {moved * block_bytes(w) / GIB:.1f} GiB payload) of "
                          f"{self.wname} geometry on a {nb}-block host pool; extract_kv_blocks then write_kv_blocks "
                          f"restated with torch CPU indexing; {self.threads} torch threads, {os.cpu_count()} host cpus",
                "seconds": round(t_total, 2), "blocks_per_s": round(moved / t_total, 1), "cpu_model": cpu_model()}

    def run_c(self, budget_s):
        """The same requests with the plain-C restatement (one memcpy per page, all host threads)."""
        from oracle import kv_oracle_c

        threads = os.cpu_count() or 1
        w, nb = self.w, self.nb
        gen = torch.Generator().manual_seed(1)
        moved, t_total = 0, 0.0
        for c in self.counts:
            s = torch.randperm(nb, generator=gen)[:c].tolist()
            d = torch.randperm(nb, generator=gen)[:c].tolist()
            t0 = time.perf_counter()
            kv_oracle_c.scatter(self.dst, d, kv_oracle_c.gather(self.src, s, threads=threads), threads=threads)
            t_total += time.perf_counter() - t0
            moved += c
            if t_total > budget_s:
                break
        return {"value": round(moved * block_bytes(w) / t_total / 1e9, 3), "unit": "GB/s", "cores": threads,
                "kind": "port", "what": "plain-C restatement, one memcpy per page on pthreads",
                "seconds": round(t_total, 2)}


def cpu_baseline(wname, budget_s=12.0):
    path = CpuPath(wname)
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


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wname = {1: "llama7b_cfg1", 2: "qwen25vl7b_cfg3"}.get(args.gpus, "llava13b_cfg4")
    per_step = max(2.0, min(10.0, 120.0 / max(1, args.steps + args.warmup)))
    path = CpuPath(wname)
    vals = []
    base = None
    for i in range(args.warmup + args.steps):
        base = path.run(per_step)
        if i >= args.warmup:
            vals.append(base)
    value = sum(v["value"] for v in vals) / len(vals)
    secs = sum(v["seconds"] for v in vals) / len(vals)
    base["value"] = round(value, 3)
    line = {
        "impl": "reference", "metric": "kv_migration_payload_GBps", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(secs * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": wname, "note": "CPU restatement of the reference's torch index/copy path on host "
                   "cores; the reference is pure Python+torch on this path and needs Ray and vLLM to run as shipped; "
                   "the transport leg has no CPU counterpart"},
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
    counts = request_blocks(w, 1)
    waves = make_waves(counts, w["NB"])
    g = torch.Generator().manual_seed(1)
    reqs = []  # (src ids, dst ids) per request, in wave order
    for wave in waves:
        sperm, dperm = torch.randperm(w["NB"], generator=g).tolist(), torch.randperm(w["NB"], generator=g).tolist()
        pos = 0
        for i in wave:
            reqs.append((sperm[pos:pos + counts[i]], dperm[pos:pos + counts[i]]))
            pos += counts[i]
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

    # correctness gate before timing: per-block checksums of the last wave
    step_device()
    rc, detail = ctx.status()
    assert rc == 0, f"device status {rc} ({detail})"
    s_sum, d_sum = block_checksums(src.layers), block_checksums(dst.layers)
    last = waves[-1]
    s_last = torch.tensor([b for i in range(len(reqs) - len(last), len(reqs)) for b in reqs[i][0]], device=device)
    d_last = torch.tensor([b for i in range(len(reqs) - len(last), len(reqs)) for b in reqs[i][1]], device=device)
    verified = bool(torch.equal(s_sum[s_last], d_sum[d_last]))

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

    del packed, flat, dev_tables, wave_tables, many
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
        "verified_bit_exact_checksum": verified,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": round(TRAFFIC_RATIO["page_copy"] * 2 * payload / len(reqs)),
                     "peak_kind": f"of {peak_kind}", "frac_of_8tbs_nominal": round(achieved / 8000.0, 4),
                     "kernel": kernel_name, "algorithmic_bytes_per_launch":
                         round(2 * payload / len(reqs)), "avg_launch_us": round(ms * 1e3 / launches, 2)},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 16,
                "api": "V0Worker.extract_kv_blocks + write_kv_blocks per request, host id lists",
                "steps": e2e_steps, "ms_per_step": round(ms_e2e / e2e_steps, 3)},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "cpu_baseline": cpu,
        "variants": {"direct_block_copy": {
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


# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes for page_copy_bulk, from the ncu capture
# summarised in profiles/page_copy_bulk_llama7b_small.md (105-block launch of the --small case); traffic grows in
# proportion to the blocks a launch moves, so the ratio is scaled to this run's mean launch.
TRAFFIC_RATIO = {"page_copy": (880.883456 + 832.828416) / (2 * 880.80384)}


def bench_append(ctx, device, args):
    """Decode-time append: reshape_and_cache of [256, 8, 128] bf16 per layer into a 32-layer, 16384-block pool."""
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
    key = torch.randn(L, T, H, D, generator=gd, device=device, dtype=torch.bfloat16)
    value = torch.randn(L, T, H, D, generator=gd, device=device, dtype=torch.bfloat16)
    it = {"i": 0}

    def per_layer():
        s = maps[it["i"] % 16]
        it["i"] += 1
        for l in range(L):
            pool.append(l, key[l], value[l], s)

    def all_layers():
        s = maps[it["i"] % 16]
        it["i"] += 1
        pool.append_all_layers(key, value, s)

    steps = max(args.steps, 50)
    out = {"workload": "append_cfg2", "tokens_per_step": T, "valid_tokens": valid, "layers": L}
    ms = timed(all_layers, steps, 5, device)
    row = H * D * 2
    algo = valid * L * (4 * row + 8)  # K and V rows read and written, plus the slot
    peak, kind = measured_peak()
    out["all_layers_call"] = {"tokens_per_s": round(T * steps / (ms / 1e3)), "us_per_step": round(ms * 1e3 / steps, 2),
                              "launches_per_step": 1, "hbm_gbs": round(algo * steps / (ms / 1e3) / 1e9, 1),
                              "frac_of_peak": round(algo * steps / (ms / 1e3) / 1e9 / peak, 4), "peak_kind": f"of {kind}"}
    ms = timed(per_layer, steps, 5, device)
    out["per_layer_calls"] = {"tokens_per_s": round(T * steps / (ms / 1e3)), "us_per_step": round(ms * 1e3 / steps, 2),
                              "launches_per_step": L}
    slot_buf = maps[0].clone()
    bound = pool.bind_append(key, value, slot_buf)

    def per_layer_bound():
        slot_buf.copy_(maps[it["i"] % 16])
        it["i"] += 1
        for l in range(L):
            bound(l)

    ms = timed(per_layer_bound, steps, 5, device)
    out["per_layer_bound_calls"] = {"tokens_per_s": round(T * steps / (ms / 1e3)),
                                    "us_per_step": round(ms * 1e3 / steps, 2), "launches_per_step": L,
                                    "what": "static key/value/slot buffers validated once (KVPool.bind_append)"}
    # CUDA-graph replay of the per-layer sequence (how a captured decode step issues it)
    try:
        stream = torch.cuda.Stream(device)
        graph = torch.cuda.CUDAGraph()
        s0 = maps[0]
        with torch.cuda.stream(stream):
            for l in range(L):
                pool.append(l, key[l], value[l], s0)
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                for l in range(L):
                    pool.append(l, key[l], value[l], s0)
        ms = timed(graph.replay, steps, 5, device)
        out["per_layer_graph_replay"] = {"tokens_per_s": round(T * steps / (ms / 1e3)),
                                         "us_per_step": round(ms * 1e3 / steps, 2), "launches_per_step": L}
    except Exception as e:  # graph capture is a reporting extra, not part of the contract
        out["per_layer_graph_replay"] = {"error": f"{type(e).__name__}: {e}"}
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

def bench_multi(args):
    import torch.distributed as dist

    from elasticmm_b200 import _lib
    from elasticmm_b200.engine.v0 import MigrationPlan, Transfer, V0Worker

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)

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

    # Requests are split evenly over the sources; each gets a seeded sink. A wave is bounded by the
    # source pool (blocks live at once) and by each sink's pool; source and sink tables are seeded
    # permutations of the pool's block ids.
    counts = request_blocks(w, 4)
    g = torch.Generator().manual_seed(4)
    assign = torch.randint(0, len(sinks), (len(counts),), generator=g).tolist()
    per_src = {s: [i for i in range(len(counts)) if i % len(sources) == k] for k, s in enumerate(sources)}

    def build_plans():
        """First-fit waves: in each wave every source takes, in order, each of its remaining requests
        that still fits its own pool and the pool of the sink the request is assigned to (requests are
        independent, so their order is free). Fuller waves mean fewer barriers and less imbalance."""
        out = []
        remaining = {s: list(per_src[s]) for s in sources}
        wv = 0
        while any(remaining.values()):
            plan = MigrationPlan()
            sink_used = {d: 0 for d in sinks}
            sink_perm = {d: torch.randperm(w["NB"], generator=torch.Generator().manual_seed(77 * wv + d)).tolist()
                         for d in sinks}
            for s in sources:
                perm = torch.randperm(w["NB"], generator=torch.Generator().manual_seed(1000 * wv + s)).tolist()
                pos, later = 0, []
                for i in remaining[s]:
                    d, n = sinks[assign[i]], counts[i]
                    if pos + n > w["NB"] or sink_used[d] + n > w["NB"]:
                        later.append(i)
                        continue
                    plan.add(Transfer(f"req{i}", s, d, tuple(perm[pos:pos + n]),
                                      tuple(sink_perm[d][sink_used[d]:sink_used[d] + n])))
                    pos += n
                    sink_used[d] += n
                remaining[s] = later
            assert plan.transfers, "a request does not fit an empty wave"
            out.append(plan)
            wv += 1
        return out

    plans = build_plans()
    total_blocks = sum(p.total_blocks() for p in plans)
    payload = total_blocks * block_bytes(w)

    # device-resident tables per wave, in the order this rank serves its peers: sinks hold
    # (source, src ids, dst ids) for the pull path, sources hold (sink, ...) for the push variant
    push_tables, pull_tables = [], []
    for plan in plans:
        pull = [(s,) + tuple(worker.pool.upload_ids(t) for t in plan.tables(s, rank)) for s in plan.pull_order(rank)]
        push = [(d,) + tuple(worker.pool.upload_ids(t) for t in plan.tables(rank, d)) for d in plan.push_order(rank)]
        pull_tables.append(pull)
        push_tables.append(push)

    def barrier():
        dist.barrier()

    streams = {p: torch.cuda.Stream(device) for p in range(world)}
    sm_count = torch.cuda.get_device_properties(device).multi_processor_count

    def run_waves(tables, pull):
        main = torch.cuda.current_stream(device)
        for per in tables:
            if pull:
                # all sources of this sink at once, grids capped to one CTA per SM in total (measured:
                # uncapped side-by-side pulls halve the NVSwitch rate, capped ones run at link speed)
                cap = max(24, sm_count // max(1, len(per))) if len(per) > 1 else None
                for peer, si, di in per:
                    streams[peer].wait_stream(main)
                    with torch.cuda.stream(streams[peer]):
                        worker.peer_pools[peer].copy_blocks(worker.pool, si, di, max_ctas=cap)
                for peer, _, _ in per:
                    main.wait_stream(streams[peer])
            else:
                for peer, si, di in per:  # one sink at a time, sources start at different sinks
                    worker.pool.copy_blocks(worker.peer_pools[peer], si, di)
            torch.cuda.synchronize(device)
            dist.barrier()  # wave boundary: blocks are reused only after every copy of the wave landed

    def step_pull():
        run_waves(pull_tables, True)

    def step_push():
        run_waves(push_tables, False)

    def step_nccl():
        for plan in plans:
            res = worker.migrate(plan, method="nccl")
            assert "error" not in res, res
            dist.barrier()

    # correctness gate: checksums of what landed against what was sent (last wave)
    step_pull()
    sums = block_checksums(worker.pool.layers).cpu()
    all_sums = [None] * world
    dist.all_gather_object(all_sums, sums)
    verified = True
    for t in plans[-1].transfers:
        if t.dst_rank == rank:
            a = all_sums[t.src_rank][list(t.src_blocks)]
            b = sums[list(t.dst_blocks)]
            verified = verified and bool(torch.equal(a, b))
    flags = [None] * world
    dist.all_gather_object(flags, verified)
    verified = all(flags)

    def max_ms(ms):
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    l0 = worker.ctx.launch_count
    with ClockSampler(local) as clocks:
        ms = max_ms(timed(step_pull, args.steps, args.warmup, device, barrier))
    launches = worker.ctx.launch_count - l0 - args.warmup * sum(len(p) for p in pull_tables)
    lt = torch.tensor([launches], device=device, dtype=torch.int64)
    dist.all_reduce(lt)
    value = payload * args.steps / (ms / 1e3) / 1e9

    # end to end through the worker API with host id lists (tables uploaded inside the timed region)
    def step_e2e():
        for plan in plans:
            res = worker.migrate(plan, method="pull")
            assert "error" not in res, res

    e2e_steps = max(2, args.steps // 4)
    ms_e = max_ms(timed(step_e2e, e2e_steps, 2, device, barrier))
    h2d = sum(8 * len(t.src_blocks) for p in plans for t in p.transfers)

    variants = {}
    line = None
    if rank == 0:
        per_src_gbs = value / len(sources)
        line = {
            "metric": "kv_migration_payload_GBps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
            "config": {"workload": wname, "geometry": {k: w[k] for k in ("L", "H", "D", "BS", "NB", "dtype")},
                       "requests": w["requests"], "blocks_per_step": total_blocks, "waves": len(plans),
                       "payload_gib_per_step": round(payload / GIB, 2), "sources": sources, "sinks": sinks,
                       "path": "one direct-load kernel per (source, sink) launched by the sink, its sources side by "
                               "side on separate streams with grids capped to one CTA per SM in total: NVLink loads "
                               "from the source's peer-mapped pool, local stores", "l2": "inputs larger than L2",
                       "per_source_egress_gbs": round(per_src_gbs, 2),
                       "per_sink_ingress_gbs": round(value / len(sinks), 2),
                       "per_pair_mean_gbs": round(value / (len(sources) * len(sinks)), 2),
                       "per_sink_ingress_frac_of_900": round(value / len(sinks) / 900.0, 4),
                       "blocks_per_s": round(total_blocks * args.steps / (ms / 1e3), 1)},
            "verified_bit_exact_checksum": verified,
            "roofline": {"bound": "nvlink", "achieved": round(per_src_gbs, 1), "peak": NVLINK_PEER_COPY_GBS,
                         "unit": "GB/s", "frac": round(per_src_gbs / NVLINK_PEER_COPY_GBS, 4), "traffic": None,
                         "peak_kind": "of measured peer copy per direction per GPU (900 nominal)",
                         "frac_of_900_nominal": round(per_src_gbs / 900.0, 4), "kernel": "page_copy_ldg (peer loads)"},
            "e2e": {"value": round(payload * e2e_steps / (ms_e / 1e3) / 1e9, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 16 * len(plans) * len(sources),
                    "api": "V0Worker.migrate(plan, method='pull') with host id lists", "steps": e2e_steps},
            "gpu_launches": int(lt.item()),
            "clocks": clocks.summary(),
            "variants": variants,
        }
    def run_variants():
        nccl_steps = max(2, args.steps // 4)
        ms_p = max_ms(timed(step_push, nccl_steps, 2, device, barrier))
        variants["peer_push"] = {"value": round(payload * nccl_steps / (ms_p / 1e3) / 1e9, 2), "unit": "GB/s",
                                 "ms_per_step": round(ms_p / nccl_steps, 3),
                                 "path": "sources store into the sinks' peer-mapped pools (same kernel, other direction)"}
        try:
            ms_n = max_ms(timed(step_nccl, nccl_steps, 2, device, barrier))
            variants["nccl_staged"] = {"value": round(payload * nccl_steps / (ms_n / 1e3) / 1e9, 2), "unit": "GB/s",
                                       "ms_per_step": round(ms_n / nccl_steps, 3),
                                       "path": "pack -> NCCL send/recv -> unpack, layer-chunk pipeline"}
        except Exception as e:
            variants["nccl_staged"] = {"error": f"{type(e).__name__}: {e}"}

        try:  # the same staged pipeline run inside the C library on its own communicator and streams
            worker.init_native_nccl()
            ms_nn = max_ms(timed(step_nccl, nccl_steps, 2, device, barrier))
            variants["nccl_staged_native"] = {"value": round(payload * nccl_steps / (ms_nn / 1e3) / 1e9, 2), "unit": "GB/s",
                                              "ms_per_step": round(ms_nn / nccl_steps, 3),
                                              "path": "emm_send_blocks / emm_recv_blocks: pack -> ncclSend, ncclRecv -> "
                                                      "unpack on library streams"}
            def step_a2a():
                for plan in plans:
                    res = worker.migrate(plan, method="alltoall")
                    assert "error" not in res, res

            ms_a = max_ms(timed(step_a2a, nccl_steps, 2, device, barrier))
            variants["nccl_alltoall_pipelined"] = {
                "value": round(payload * nccl_steps / (ms_a / 1e3) / 1e9, 2), "unit": "GB/s",
                "ms_per_step": round(ms_a / nccl_steps, 3),
                "path": "per layer chunk: one gather for all sinks, one grouped ncclSend/ncclRecv exchange among all "
                        "ranks, one scatter for all sources; three streams, two staging slots"}
        except Exception as e:
            variants["nccl_staged_native"] = {"error": f"{type(e).__name__}: {e}"}

        # Every rank a source and a sink at once (the rebalancing exchange): rank r loads the lower half of
        # rank r+1's pool into the upper half of its own. Run last among the device-resident variants because
        # it overwrites pool contents.
        half = w["NB"] // 2
        ring_src = worker.pool.upload_ids(torch.randperm(half, generator=torch.Generator().manual_seed(rank)).tolist())
        ring_dst = worker.pool.upload_ids((torch.randperm(half, generator=torch.Generator().manual_seed(50 + rank)) + half).tolist())

        def step_ring():
            worker.peer_pools[nxt].copy_blocks(worker.pool, ring_src, ring_dst)
            torch.cuda.synchronize(device)
            dist.barrier()

        ring_steps = max(3, args.steps // 2)
        ms_r = max_ms(timed(step_ring, ring_steps, 2, device, barrier))
        ring_bytes = world * half * block_bytes(w)
        variants["ring_exchange_all_ranks"] = {
            "value": round(ring_bytes * ring_steps / (ms_r / 1e3) / 1e9, 2), "unit": "GB/s",
            "per_gpu_ingress_gbs": round(ring_bytes / world * ring_steps / (ms_r / 1e3) / 1e9, 2),
            "ms_per_step": round(ms_r / ring_steps, 3),
            "path": "every rank pulls half of the next rank's pool into its own at the same time"}


    # The variants are extras: if one of them stalls (an NCCL path on an unusual fabric), the headline
    # line is still printed and the job ends instead of hanging until an outer limit kills it.
    done = threading.Event()

    def give_up():
        if done.is_set():
            return
        if rank == 0:
            variants["timed_out"] = True
            print(json.dumps(line), flush=True)
        os._exit(0)

    watchdog = threading.Timer(float(os.environ.get("EMM_BENCH_VARIANT_LIMIT_S", "240")), give_up)
    watchdog.daemon = True
    watchdog.start()
    if not args.skip_extras:
        run_variants()
    done.set()
    watchdog.cancel()
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def probe_fabric(args):
    """Peer-copy patterns over NVSwitch (N >= 2 ranks): one flow with different grid sizes, and with
    N >= 4 two sources -> all other ranks as sinks, pulled side by side with full grids, with grids capped
    to one CTA per SM in total, and one source at a time. One JSON line per pattern on rank 0. These
    measurements fixed the schedule V0Worker.migrate uses."""
    import torch.distributed as dist

    from elasticmm_b200.engine.v0 import V0Worker

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    w = dict(WORKLOADS["llava13b_cfg4"], NB=1024)
    n = 512  # blocks per flow: 6.25 GiB
    worker = V0Worker(worker_id=rank, dtype=w["dtype"], device=device, global_rank=rank, world_size=world,
                      kv_cache=gpu_pool(w, device, rank))
    worker.init_global_nccl()
    handles = [None] * world
    dist.all_gather_object(handles, (worker.get_ipc_handles(), worker.get_pool_desc()))
    for peer in range(world):
        if peer != rank:
            worker.attach_peer_pool(peer, handles[peer][0], handles[peer][1])
    g = torch.Generator().manual_seed(rank)
    tabs = {p: (worker.pool.upload_ids(torch.randperm(w["NB"] // 2, generator=g)[:n].tolist()),
                worker.pool.upload_ids((torch.randperm(w["NB"] // 2, generator=g)[:n] + w["NB"] // 2).tolist()))
            for p in range(world)}
    streams = {p: torch.cuda.Stream(device) for p in range(world)}
    flow_bytes = n * block_bytes(w)

    def run(name, ops, flows, cap=None, serial=False, iters=3):
        """ops: [(kind, peer)] this rank runs; 'pull' loads peer -> here, 'push' stores here -> peer."""
        def step():
            main = torch.cuda.current_stream(device)
            for kind, peer in ops:
                st = main if serial else streams[peer]
                if not serial:
                    st.wait_stream(main)
                with torch.cuda.stream(st):
                    si, di = tabs[peer]
                    if kind == "pull":
                        worker.peer_pools[peer].copy_blocks(worker.pool, si, di, max_ctas=cap)
                    else:
                        worker.pool.copy_blocks(worker.peer_pools[peer], si, di, max_ctas=cap)
            if not serial:
                for _, peer in ops:
                    main.wait_stream(streams[peer])
        step()
        torch.cuda.synchronize(device)
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            step()
        b.record()
        torch.cuda.synchronize(device)
        ms = torch.tensor([a.elapsed_time(b) / iters], device=device, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
        if rank == 0:
            print(json.dumps({"probe": name, "flows": flows, "ms": round(ms.item(), 3),
                              "total_gbs": round(flows * flow_bytes / ms.item() / 1e6, 1)}))

    for cap in (None, 74, 48, 37, 24):
        run(f"one pull flow 1<-0, grid cap {cap}", [("pull", 0)] if rank == 1 else [], 1, cap=cap)
        run(f"one push flow 0->1, grid cap {cap}", [("push", 1)] if rank == 0 else [], 1, cap=cap)
    if world >= 4:
        srcs, snks = [0, 1], list(range(2, world))
        j = snks.index(rank) if rank in snks else 0
        pulls = [("pull", s) for s in srcs] if rank in snks else []
        run(f"pull 2->{len(snks)}, both sources at once, full grids", pulls, 2 * len(snks))
        for cap in (120, 100, 74, 48):
            run(f"pull 2->{len(snks)}, both sources at once, grid cap {cap} each", pulls, 2 * len(snks), cap=cap)
        run(f"pull 2->{len(snks)}, one source at a time, rotated start",
            [("pull", srcs[(j + k) % 2]) for k in range(2)] if rank in snks else [], 2 * len(snks), serial=True)
        run(f"pull 2->{len(snks)}, one source at a time, same start", pulls, 2 * len(snks), serial=True)
        pushes = [("push", d) for d in snks] if rank in srcs else []
        run(f"push 2->{len(snks)}, all sinks at once, full grids", pushes, 2 * len(snks))
        i = srcs.index(rank) if rank in srcs else 0
        k0 = i * (len(snks) // 2)
        run(f"push 2->{len(snks)}, one sink at a time, rotated start",
            [("push", snks[(k0 + k) % len(snks)]) for k in range(len(snks))] if rank in srcs else [],
            2 * len(snks), serial=True)
        run("ring: every rank pulls from the next", [("pull", (rank + 1) % world)], world)
        run("ring: every rank pushes to the next", [("push", (rank + 1) % world)], world)
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
    ap.add_argument("--probe-fabric", action="store_true",
                    help="N>1: measure peer-copy patterns over NVSwitch instead of the migration workload")
    ap.add_argument("--variant", type=int, default=None, help="copy kernel family (1 bulk, 2 ldg)")
    ap.add_argument("--chunk", type=int, default=None)
    ap.add_argument("--stages", type=int, default=None)
    ap.add_argument("--warps", type=int, default=None)
    ap.add_argument("--ctas-per-sm", type=int, default=None)
    ap.add_argument("--unroll", type=int, default=None)
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
    from elasticmm_b200 import get_context

    if any(v is not None for v in (args.variant, args.chunk, args.stages, args.warps, args.ctas_per_sm, args.unroll)):
        dev = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(dev)
        get_context(dev).configure(variant=args.variant, chunk_bytes=args.chunk, stages=args.stages,
                                   warps=args.warps, ctas_per_sm=args.ctas_per_sm, ldg_unroll=args.unroll)
    if args.probe_fabric:
        probe_fabric(args)
    elif args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        bench_single(args)
    else:
        bench_multi(args)


if __name__ == "__main__":
    main()
