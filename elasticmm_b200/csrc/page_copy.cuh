// Page-copy kernels for sm_100a: the one data mover behind gather, scatter,
// block copy (compaction / swap) and direct stores into a peer GPU's pool.
//
// A work item ("chunk") is a run of at most `chunk_bytes` bytes inside one
// page, a page being one block of one plane (K or V; a block pool has a
// single plane) of one layer. Chunks are
// numbered with the chunk-in-page index fastest, then the block position i in
// the table, then the plane, then the layer, so that neighbouring CTAs touch
// neighbouring bytes of the packed side and the table is read once per page.
//
//   address(side, l, p, i, c) = layer_base(side, l) + p*plane_stride
//                             + id(side, i)*block_stride + c*chunk_bytes
//   id(side, i) = ids ? ids[i] : i              (identity on the packed side)
//   layer_base  = layers ? layers[l] : base + l*layer_stride
//
// Two kernel families implement the same contract:
//   * page_copy_bulk: each warp's lane 0 drives a ring of shared-memory
//     buffers with cp.async.bulk (global -> shared, completion on an
//     mbarrier) and cp.async.bulk (shared -> global, bulk groups). No data
//     passes through registers; two to eight lanes per SM keep 32-64 KiB of
//     loads in flight, which is where B200's HBM throughput peaks.
//   * page_copy_ldg<V, U>: vector loads/stores through registers; also the
//     path for geometries whose pages are not 16-byte granular, and for
//     destinations that are not ordinary device memory of this GPU.
//
// Neither kernel traps: an id outside [0, num_blocks) records
// EMM_ERR_ID_RANGE in the status word and the page is skipped; a wait that
// runs out records EMM_ERR_TIMEOUT and the warp drains what it has in flight
// and returns.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace emm {

struct CopySide {
  const uint64_t *layers;  // device array of per-layer base addresses, or nullptr
  uint64_t base;           // used when layers == nullptr
  uint64_t layer_stride;   // used when layers == nullptr
  uint64_t plane_stride;
  uint64_t block_stride;
  const int32_t *ids;      // device table of n ids, or nullptr for identity
  uint32_t num_blocks;     // bound for ids (ignored for identity)
  // Segmented packed side (several requests, each with its own [layers, planes, n_r, page]
  // buffer laid end to end): prefix sums of the requests' block counts, or nullptr.
  const uint32_t *seg_prefix;  // device array of num_segs + 1 entries, seg_prefix[0] == 0
  uint32_t num_segs;
  uint64_t seg_stride;         // bytes one block occupies over the moved layers and planes
};

constexpr int kInlineIds = 128;  // longest table carried in the kernel arguments (2 x 512 B of the 4 KiB argument space)

struct PageCopyArgs {
  CopySide src;
  CopySide dst;
  uint32_t n;                // table length
  uint32_t plane_shift;      // 1: K and V planes per layer; 0: single-plane block pool
  uint32_t layer_begin;      // first layer of the pools to move
  uint32_t layer_count;      // number of layers to move
  uint32_t page_bytes;       // bytes per page
  uint32_t chunk_bytes;      // bytes per chunk (multiple of the vector width)
  uint32_t chunks_per_page;  // ceil(page_bytes / chunk_bytes)
  uint64_t total_chunks;     // layer_count * planes * n * chunks_per_page
  int *status;               // [0] = sticky status code, [1..2] = detail (lo, hi)
  // Short tables travel in the kernel arguments instead of device memory (no staging copy before the
  // launch): when inline_count > 0, a side with use_inline set reads its ids from inline_ids[side].
  uint32_t inline_count;
  uint32_t src_inline, dst_inline;
  int32_t inline_ids[2][kInlineIds];
  uint64_t wait_limit_ns;    // bulk family: longest a lane waits for one load before it gives up
  uint32_t tx_overcount;     // bulk family, test hook: bytes added to every expected transaction count
                             // (0 in every product path; non-zero makes each wait run out)
};

// Status codes duplicated from emm_kv.h so that device code needs no C header.
constexpr int kStatusIdRange = 2;
constexpr int kStatusTimeout = 5;

constexpr int kMaxStages = 8;
constexpr int kMaxWarps = 8;
constexpr uint64_t kDefaultWaitLimitNs = 2000000000ull;  // 2 s per bounded wait unless the context says otherwise

struct ChunkAddr {
  uint64_t src;
  uint64_t dst;
  uint32_t len;  // 0 = skip (id out of range)
};

__device__ __forceinline__ void report(int *status, int code, long long detail) {
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = (int)(detail & 0xffffffffll);
    status[2] = (int)(detail >> 32);
  }
}

// Address of page (lrel, p, i) on a segmented packed side: request r with
// seg_prefix[r] <= i < seg_prefix[r+1] owns a [layers, planes, n_r, page] buffer that
// starts seg_prefix[r] * seg_stride bytes into the allocation.
__device__ __forceinline__ uint64_t segmented_address(const CopySide &sd, uint32_t i, uint32_t lrel,
                                                      uint32_t p, uint32_t planes) {
  uint32_t lo = 0, hi = sd.num_segs;
  while (hi - lo > 1) {
    const uint32_t mid = (lo + hi) >> 1;
    if (sd.seg_prefix[mid] <= i) lo = mid;
    else hi = mid;
  }
  const uint32_t start = sd.seg_prefix[lo];
  const uint32_t n_r = sd.seg_prefix[lo + 1] - start;
  return sd.base + (uint64_t)start * sd.seg_stride +
         ((uint64_t)(lrel * planes + p) * n_r + (i - start)) * sd.block_stride;
}

// Decodes chunk g into addresses. Uniform across the threads that call it
// with the same g (table and layer-pointer reads are broadcasts).
template <bool kSeg>
__device__ __forceinline__ ChunkAddr decode_chunk(const PageCopyArgs &a, uint64_t g) {
  uint64_t page = g / a.chunks_per_page;
  uint32_t c = (uint32_t)(g - page * a.chunks_per_page);
  uint64_t t = page / a.n;
  uint32_t i = (uint32_t)(page - t * a.n);
  uint32_t p = (uint32_t)(t & a.plane_shift);                   // plane_shift is 0 or 1: also the plane mask
  uint32_t lrel = (uint32_t)(t >> a.plane_shift);               // index on a linear (packed) side
  uint32_t l = a.layer_begin + lrel;                            // index into the pools' layer arrays

  ChunkAddr r;
  uint32_t off = c * a.chunk_bytes;
  uint32_t rem = a.page_bytes - off;
  r.len = rem < a.chunk_bytes ? rem : a.chunk_bytes;

  const bool s_tab = a.src.ids || a.src_inline, d_tab = a.dst.ids || a.dst_inline;
  int32_t sid = a.src.ids ? a.src.ids[i] : (a.src_inline ? a.inline_ids[0][i] : (int32_t)i);
  int32_t did = a.dst.ids ? a.dst.ids[i] : (a.dst_inline ? a.inline_ids[1][i] : (int32_t)i);
  bool bad = (s_tab && (uint32_t)sid >= a.src.num_blocks) || (d_tab && (uint32_t)did >= a.dst.num_blocks);
  if (bad) {
    report(a.status, kStatusIdRange, (s_tab && (uint32_t)sid >= a.src.num_blocks) ? sid : did);
    r.len = 0;
    r.src = 0;
    r.dst = 0;
    return r;
  }
  // kSeg kernels serve the several-requests-per-launch entries: the packed side (the one without
  // a layer-pointer array) is then addressed through the segment table.
  if (kSeg && a.src.seg_prefix) {
    r.src = segmented_address(a.src, i, lrel, p, a.plane_shift + 1u) + off;
  } else {
    const uint64_t sbase = a.src.layers ? a.src.layers[l] : a.src.base + (uint64_t)lrel * a.src.layer_stride;
    r.src = sbase + (uint64_t)p * a.src.plane_stride + (uint64_t)(uint32_t)sid * a.src.block_stride + off;
  }
  if (kSeg && a.dst.seg_prefix) {
    r.dst = segmented_address(a.dst, i, lrel, p, a.plane_shift + 1u) + off;
  } else {
    const uint64_t dbase = a.dst.layers ? a.dst.layers[l] : a.dst.base + (uint64_t)lrel * a.dst.layer_stride;
    r.dst = dbase + (uint64_t)p * a.dst.plane_stride + (uint64_t)(uint32_t)did * a.dst.block_stride + off;
  }
  return r;
}

// ---------------------------------------------------------------------------
// PTX wrappers (sm_90+/sm_100a bulk-copy and mbarrier instructions)
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Waits for the phase with the given parity, for at most limit_ns.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = global_timer_ns();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
}

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, uint64_t gsrc, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void bulk_store(uint64_t gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_src), "r"(bytes)
               : "memory");
}

// Variants with an L2 eviction-priority hint (the pages are touched once).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void bulk_load_hint(uint32_t smem_dst, uint64_t gsrc, uint32_t bytes,
                                               uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void bulk_store_hint(uint64_t gdst, uint32_t smem_src, uint32_t bytes,
                                                uint64_t policy) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(gdst),
               "r"(smem_src), "r"(bytes), "l"(policy)
               : "memory");
}

__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may start
// while its predecessor in the stream is still draining; it must not touch global memory before
// grid_dependency_wait(), which returns once the predecessor has completed and its writes are visible.
// Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Bulk-copy ring kernel
// ---------------------------------------------------------------------------
//
// Dynamic shared memory: warps * stages * chunk_bytes (each warp owns a ring).
// Chunk stream of warp w in CTA b: g = (j*gridDim.x + b)*warps + w, j = 0,1,..
//
// Per ring slot s the sequence over time is
//   load(j) -> [mbarrier phase] -> store(j) -> [bulk group read done] -> load(j+stages)
// The loop keeps stages-1 loads in flight: in iteration j it waits for load j,
// issues store j, then waits until store j-1 has finished reading its slot and
// refills that slot with load j+stages-1. Addresses for the next load are
// decoded one iteration early so the table read is off the critical path.
template <bool kSeg>
__global__ void __launch_bounds__(kMaxWarps * 32)
page_copy_bulk(const __grid_constant__ PageCopyArgs a, const uint32_t stages, const uint32_t l2_hint) {
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(8) uint64_t bars[kMaxWarps * kMaxStages];
  __shared__ uint64_t slot_dst[kMaxWarps * kMaxStages];
  __shared__ uint32_t slot_len[kMaxWarps * kMaxStages];

  const uint32_t warp = threadIdx.x >> 5;
  grid_launch_dependents();  // the next copy in the stream may set up while this one runs
  if ((threadIdx.x & 31) != 0) return;  // one issuing lane per warp
  const uint32_t warps = blockDim.x >> 5;

  const uint32_t ring = smem_u32(ring_mem) + warp * stages * a.chunk_bytes;
  uint64_t *my_bars = bars + warp * kMaxStages;
  uint64_t *my_dst = slot_dst + warp * kMaxStages;
  uint32_t *my_len = slot_len + warp * kMaxStages;

  for (uint32_t s = 0; s < stages; ++s) mbar_init(smem_u32(&my_bars[s]), 1);
  mbar_init_fence();
  // l2_hint bit 0: loads evict-first, bit 1: stores evict-first
  const uint64_t policy = l2_hint ? l2_evict_first_policy() : 0;

  const uint64_t stream_id = (uint64_t)blockIdx.x * warps + warp;
  const uint64_t stream_step = (uint64_t)gridDim.x * warps;
  if (stream_id >= a.total_chunks) return;
  const uint64_t n_mine = (a.total_chunks - stream_id + stream_step - 1) / stream_step;
  grid_dependency_wait();  // everything below reads or writes global memory

  // Issues the load of this stream's chunk into ring slot s.
  auto issue = [&](const ChunkAddr &ca, uint32_t s) {
    const uint32_t bar = smem_u32(&my_bars[s]);
    my_dst[s] = ca.dst;
    my_len[s] = ca.len;
    if (ca.len) {
      mbar_expect_tx(bar, ca.len + a.tx_overcount);
      if (l2_hint & 1) bulk_load_hint(ring + s * a.chunk_bytes, ca.src, ca.len, bar, policy);
      else bulk_load(ring + s * a.chunk_bytes, ca.src, ca.len, bar);
    } else {
      mbar_arrive(bar);  // skipped page: complete the phase with no bytes
    }
  };

  const uint64_t prologue = n_mine < (uint64_t)(stages - 1) ? n_mine : (uint64_t)(stages - 1);
  for (uint64_t j = 0; j < prologue; ++j)
    issue(decode_chunk<kSeg>(a, stream_id + j * stream_step), (uint32_t)j);

  uint64_t jn = prologue;  // next chunk of this stream to load
  ChunkAddr next_ca;
  next_ca.src = next_ca.dst = 0;
  next_ca.len = 0;
  if (jn < n_mine) next_ca = decode_chunk<kSeg>(a, stream_id + jn * stream_step);

  bool timed_out = false;
  uint32_t s = 0;       // slot of chunk j
  uint32_t parity = 0;  // phase parity of slot s for chunk j
  uint64_t j = 0;
  for (; j < n_mine; ++j) {
    // Decode one load ahead: these global reads complete while we wait below.
    const ChunkAddr cur_ca = next_ca;
    if (jn + 1 < n_mine) next_ca = decode_chunk<kSeg>(a, stream_id + (jn + 1) * stream_step);

    if (!mbar_wait_bounded(smem_u32(&my_bars[s]), parity, a.wait_limit_ns)) {
      report(a.status, kStatusTimeout, (long long)(stream_id + j * stream_step));
      timed_out = true;
      break;
    }
    if (my_len[s]) {
      if (l2_hint & 2) bulk_store_hint(my_dst[s], ring + s * a.chunk_bytes, my_len[s], policy);
      else bulk_store(my_dst[s], ring + s * a.chunk_bytes, my_len[s]);
    }
    bulk_commit();

    if (jn < n_mine) {
      // Slot of chunk j-1 (== slot of chunk jn): its store must have read the
      // buffer before the next load overwrites it.
      bulk_wait_read<1>();
      const uint32_t sn = (s == 0) ? stages - 1 : s - 1;
      issue(cur_ca, sn);
      ++jn;
    }
    if (++s == stages) {
      s = 0;
      parity ^= 1;
    }
  }

  if (timed_out) {
    // Loads j .. jn-1 may still be writing this CTA's shared memory: give
    // each one more bounded wait before the CTA may retire.
    for (uint64_t q = j; q < jn; ++q) {
      const uint32_t qs = (uint32_t)(q % stages);
      const uint32_t qp = (uint32_t)((q / stages) & 1);
      if (!mbar_wait_bounded(smem_u32(&my_bars[qs]), qp, a.wait_limit_ns)) break;
    }
  }
  bulk_wait_all();  // stores complete (and have left shared memory) before exit
}

// ---------------------------------------------------------------------------
// Register (LDG/STG) kernel
// ---------------------------------------------------------------------------

template <typename V>
__device__ __forceinline__ V load_stream(const V *p) {
  return *p;
}
template <typename V>
__device__ __forceinline__ void store_stream(V *p, const V &v) {
  *p = v;
}
template <>
__device__ __forceinline__ uint4 load_stream<uint4>(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
template <>
__device__ __forceinline__ void store_stream<uint4>(uint4 *p, const uint4 &v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// One CTA per chunk, grid-stride. Each thread moves up to U vectors of type V
// per pass; all U loads are issued before the first store.
template <typename V, int U, bool kSeg>
__global__ void __launch_bounds__(256) page_copy_ldg(const __grid_constant__ PageCopyArgs a) {
  grid_launch_dependents();
  grid_dependency_wait();
  for (uint64_t g = blockIdx.x; g < a.total_chunks; g += gridDim.x) {
    const ChunkAddr ca = decode_chunk<kSeg>(a, g);
    if (ca.len == 0) continue;
    const V *__restrict__ sp = reinterpret_cast<const V *>(ca.src);
    V *__restrict__ dp = reinterpret_cast<V *>(ca.dst);
    const uint32_t nvec = ca.len / (uint32_t)sizeof(V);
    for (uint32_t base = 0; base < nvec; base += 256u * U) {
      V v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t k = base + (uint32_t)u * 256u + threadIdx.x;
        if (k < nvec) v[u] = load_stream<V>(sp + k);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t k = base + (uint32_t)u * 256u + threadIdx.x;
        if (k < nvec) store_stream<V>(dp + k, v[u]);
      }
    }
  }
}

}  // namespace emm
