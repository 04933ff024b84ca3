// C ABI of the paged KV-cache movement library: contexts, pool descriptors,
// argument validation and kernel launches. Declarations and the reference
// methods each entry replaces are in include/emm_kv.h.
#include "emm_kv.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "append.cuh"
#include "page_copy.cuh"

namespace {

thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define EMM_CUDA(call)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (call);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return fail(EMM_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_),  \
                  __FILE__, __LINE__);                                                   \
  } while (0)

// Largest power of two (capped at 256) dividing v; 256 for v == 0.
uint32_t pow2_align(uint64_t v) {
  if (v == 0) return 256;
  uint64_t a = v & (~v + 1);
  return a > 256 ? 256u : (uint32_t)a;
}

constexpr int kRingSlots = 8;

struct IdSlot {
  int32_t *h = nullptr;  // pinned
  int32_t *d = nullptr;
  size_t cap = 0;        // ids
  cudaEvent_t ev = nullptr;
  bool pending = false;
};

struct IpcMapping {
  unsigned char handle[EMM_IPC_HANDLE_BYTES];
  void *base;
};

class DeviceGuard {
 public:
  explicit DeviceGuard(int dev) {
    ok_ = cudaGetDevice(&prev_) == cudaSuccess;
    if (ok_ && prev_ != dev) ok_ = cudaSetDevice(dev) == cudaSuccess;
    changed_ = ok_ && prev_ != dev;
  }
  ~DeviceGuard() {
    if (changed_) cudaSetDevice(prev_);
  }
  bool ok() const { return ok_; }

 private:
  int prev_ = 0;
  bool ok_ = false;
  bool changed_ = false;
};

}  // namespace

struct emm_ctx {
  int device = 0;
  int sm_count = 0;
  int max_smem_optin = 0;
  int *d_status = nullptr;  // 4 ints: code, detail lo, detail hi, pad
  int *h_status = nullptr;  // pinned mirror
  int64_t launches = 0;
  // options
  int copy_variant = EMM_COPY_AUTO;
  int64_t chunk_bytes = 0;  // 0 = per-variant default
  int stages = 2;
  int warps = 0;            // 0 = sized from the chunk (see launch_page_copy)
  int ctas_per_sm = 0;      // 0 = per-variant default
  int ldg_unroll = 2;
  int max_ctas = 0;
  int remote_variant = EMM_COPY_LDG;  // family used when a side is peer or host memory
  int l2_hint = 0;                    // bulk family: bit 0 loads, bit 1 stores carry an L2 evict-first hint
  uint64_t wait_limit_ns = emm::kDefaultWaitLimitNs;  // bulk family: bound of each device-side wait
  int pdl = 1;                 // copy kernels are launched with programmatic stream serialisation
  IdSlot ring[kRingSlots];
  int next_slot = 0;
  std::vector<uint64_t> bitmap;  // scratch for duplicate / overlap checks
  std::vector<IpcMapping> ipc;
  // staged transport: a packing/unpacking stream, a wire stream and their events (made on first use)
  cudaStream_t copy_stream = nullptr;
  cudaStream_t wire_stream = nullptr;
  cudaEvent_t ev_entry = nullptr;
  cudaEvent_t ev_copied[2] = {nullptr, nullptr};
  cudaEvent_t ev_wired[2] = {nullptr, nullptr};
  cudaEvent_t ev_done[2] = {nullptr, nullptr};
};

struct emm_pool {
  emm_ctx *ctx = nullptr;
  int device = 0;  // copy of ctx->device: destroying a pool must not need a live context
  emm_pool_desc desc{};
  uint64_t *d_layers = nullptr;
  std::vector<uint64_t> h_layers;
  int64_t page_bytes = 0;
  int planes = 2;
  uint32_t align = 1;   // power-of-two alignment shared by all page addresses
  bool device_local = true;  // every layer pointer is plain memory of ctx->device
};

namespace {

using emm::CopySide;
using emm::PageCopyArgs;

// Checks the descriptor; on success *dense_page says whether a block of a
// plane is one dense run of BS*H*D*e bytes.
int check_desc(const emm_pool_desc &d, bool *dense_page) {
  if (d.num_layers <= 0 || d.num_blocks <= 0 || d.block_size <= 0 || d.num_kv_heads <= 0 ||
      d.head_size <= 0)
    return fail(EMM_ERR_BAD_ARG, "pool geometry must be positive (L=%d NB=%d BS=%d H=%d D=%d)",
                d.num_layers, d.num_blocks, d.block_size, d.num_kv_heads, d.head_size);
  if (d.elem_size != 1 && d.elem_size != 2 && d.elem_size != 4 && d.elem_size != 8)
    return fail(EMM_ERR_BAD_ARG, "elem_size %d not in {1,2,4,8}", d.elem_size);
  if (d.num_planes < 0 || d.num_planes > 2 || d.reserved != 0)
    return fail(EMM_ERR_BAD_ARG, "num_planes must be 0, 1 or 2 and reserved must be 0");
  const int64_t e = d.elem_size;
  const int64_t head_bytes = (int64_t)d.head_size * e;
  const int64_t page = (int64_t)d.block_size * d.num_kv_heads * head_bytes;
  if (page > (int64_t)0x7fffffff) return fail(EMM_ERR_TOO_LARGE, "page of %lld bytes", (long long)page);
  const bool two_planes = d.num_planes != 1;
  if ((two_planes && d.plane_stride < page) || d.block_stride < page || d.token_stride < head_bytes ||
      d.head_stride < head_bytes)
    return fail(EMM_ERR_BAD_ARG, "strides smaller than the data they step over");
  if (d.plane_stride % e || d.block_stride % e || d.token_stride % e || d.head_stride % e)
    return fail(EMM_ERR_ALIGN, "strides must be multiples of elem_size");
  const bool nhd = d.head_stride == head_bytes && d.token_stride == head_bytes * d.num_kv_heads;
  const bool hnd = d.token_stride == head_bytes && d.head_stride == head_bytes * d.block_size;
  *dense_page = nhd || hnd;
  if (!*dense_page) {
    // A strided page still supports append; whole-block moves are refused later.
    const int64_t tok_span = (int64_t)(d.block_size - 1) * d.token_stride;
    const int64_t head_span = (int64_t)(d.num_kv_heads - 1) * d.head_stride;
    if (tok_span + head_span + head_bytes > d.block_stride)
      return fail(EMM_ERR_BAD_ARG, "token/head strides run past block_stride");
  }
  return EMM_OK;
}

int acquire_slot(emm_ctx *ctx, size_t n_ids, IdSlot **out) {
  IdSlot &s = ctx->ring[ctx->next_slot];
  ctx->next_slot = (ctx->next_slot + 1) % kRingSlots;
  if (s.pending) {
    EMM_CUDA(cudaEventSynchronize(s.ev));  // normally long complete
    s.pending = false;
  }
  if (!s.ev) EMM_CUDA(cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming));
  if (s.cap < n_ids) {
    size_t cap = std::max<size_t>(4096, s.cap * 2);
    while (cap < n_ids) cap *= 2;
    if (s.h) cudaFreeHost(s.h);
    if (s.d) cudaFree(s.d);
    s.h = nullptr;
    s.d = nullptr;
    s.cap = 0;
    EMM_CUDA(cudaMallocHost(&s.h, cap * sizeof(int32_t)));
    EMM_CUDA(cudaMalloc(&s.d, cap * sizeof(int32_t)));
    s.cap = cap;
  }
  *out = &s;
  return EMM_OK;
}

// Marks ids in the scratch bitmap. Returns false on the first id already set.
bool bitmap_mark(std::vector<uint64_t> &bm, const int64_t *ids, int32_t n, int64_t *dup) {
  for (int32_t i = 0; i < n; ++i) {
    uint64_t w = (uint64_t)ids[i] >> 6, b = 1ull << (ids[i] & 63);
    if (bm[w] & b) {
      *dup = ids[i];
      return false;
    }
    bm[w] |= b;
  }
  return true;
}
int bitmap_reserve(std::vector<uint64_t> &bm, int64_t num_blocks) {
  const size_t words = ((size_t)num_blocks + 63) / 64;
  if (bm.size() >= words) return EMM_OK;
  try {
    bm.resize(words);
  } catch (const std::bad_alloc &) {
    return fail(EMM_ERR_NOMEM, "no host memory for a bitmap of %lld blocks", (long long)num_blocks);
  }
  return EMM_OK;
}
void bitmap_clear(std::vector<uint64_t> &bm, const int64_t *ids, int32_t n) {
  for (int32_t i = 0; i < n; ++i) bm[(uint64_t)ids[i] >> 6] = 0;
}

int check_ids_host(const int64_t *ids, int32_t n, int64_t nb, const char *what) {
  for (int32_t i = 0; i < n; ++i)
    if (ids[i] < 0 || ids[i] >= nb)
      return fail(EMM_ERR_ID_RANGE, "%s id %lld at position %d outside [0, %lld)", what,
                  (long long)ids[i], i, (long long)nb);
  return EMM_OK;
}

// One side of a copy backed by a pool.
CopySide pool_side(const emm_pool *p, const int32_t *ids) {
  CopySide s;
  s.layers = p->d_layers;
  s.base = 0;
  s.layer_stride = 0;
  s.plane_stride = (uint64_t)p->desc.plane_stride;
  s.block_stride = (uint64_t)p->desc.block_stride;
  s.ids = ids;
  s.num_blocks = (uint32_t)p->desc.num_blocks;
  s.seg_prefix = nullptr;
  s.num_segs = 0;
  s.seg_stride = 0;
  return s;
}

// One side backed by the packed buffer [layers, 2, n, page].
CopySide packed_side(const void *packed, int32_t n, int64_t page, int planes = 2) {
  CopySide s;
  s.layers = nullptr;
  s.base = (uint64_t)packed;
  s.layer_stride = (uint64_t)planes * (uint64_t)n * (uint64_t)page;
  s.plane_stride = (uint64_t)n * (uint64_t)page;
  s.block_stride = (uint64_t)page;
  s.ids = nullptr;
  s.num_blocks = (uint32_t)n;
  s.seg_prefix = nullptr;
  s.num_segs = 0;
  s.seg_stride = 0;
  return s;
}

// The dynamic shared-memory limit of a kernel belongs to (kernel, device) and is
// shared by every context and entry point of the process, so it is tracked per
// device and only ever raised: lowering it under a caller that already sized
// its launches for the larger value would make those launches fail.
constexpr int kMaxTrackedDevices = 64;
std::atomic<int> g_bulk_smem_limit[kMaxTrackedDevices];
std::mutex g_bulk_smem_mutex;

// Call with `device` current.
int ensure_bulk_smem(int device, int smem) {
  const bool tracked = device >= 0 && device < kMaxTrackedDevices;
  if (tracked && smem <= g_bulk_smem_limit[device].load(std::memory_order_acquire)) return EMM_OK;
  std::lock_guard<std::mutex> lock(g_bulk_smem_mutex);
  int current = tracked ? g_bulk_smem_limit[device].load(std::memory_order_relaxed) : 0;
  if (!tracked) {
    cudaFuncAttributes fa;
    EMM_CUDA(cudaFuncGetAttributes(&fa, emm::page_copy_bulk<false>));
    current = fa.maxDynamicSharedSizeBytes;
  }
  if (smem <= current) return EMM_OK;
  EMM_CUDA(cudaFuncSetAttribute(emm::page_copy_bulk<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  EMM_CUDA(cudaFuncSetAttribute(emm::page_copy_bulk<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  if (tracked) g_bulk_smem_limit[device].store(smem, std::memory_order_release);
  return EMM_OK;
}

template <typename V, bool kSeg>
int launch_ldg_typed(emm_ctx *ctx, const PageCopyArgs &a, int grid, cudaStream_t st) {
  switch (ctx->ldg_unroll) {
    case 1: emm::page_copy_ldg<V, 1, kSeg><<<grid, 256, 0, st>>>(a); break;
    case 2: emm::page_copy_ldg<V, 2, kSeg><<<grid, 256, 0, st>>>(a); break;
    case 8: emm::page_copy_ldg<V, 8, kSeg><<<grid, 256, 0, st>>>(a); break;
    default: emm::page_copy_ldg<V, 4, kSeg><<<grid, 256, 0, st>>>(a); break;
  }
  return EMM_OK;
}

template <bool kSeg>
void launch_ldg(emm_ctx *ctx, const PageCopyArgs &a, int grid, uint32_t align, cudaStream_t st) {
  if (align >= 16) launch_ldg_typed<uint4, kSeg>(ctx, a, grid, st);
  else if (align >= 8) launch_ldg_typed<uint2, kSeg>(ctx, a, grid, st);
  else if (align >= 4) launch_ldg_typed<uint32_t, kSeg>(ctx, a, grid, st);
  else if (align >= 2) launch_ldg_typed<uint16_t, kSeg>(ctx, a, grid, st);
  else launch_ldg_typed<uint8_t, kSeg>(ctx, a, grid, st);
}

// Launches the page copy described by (src, dst). `align` is the common
// power-of-two alignment of every address and length involved; `local` says
// both sides are ordinary memory of this GPU.
int launch_page_copy(emm_ctx *ctx, CopySide src, CopySide dst, int32_t n, int32_t layer_begin,
                     int32_t layer_count, int64_t page_bytes, uint32_t align, bool local,
                     cudaStream_t st, int planes = 2, uint32_t tx_overcount = 0,
                     const int64_t *inline_src = nullptr, const int64_t *inline_dst = nullptr) {
  if (n == 0 || layer_count == 0) return EMM_OK;
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);

  int variant = ctx->copy_variant;
  if (variant == EMM_COPY_AUTO) variant = EMM_COPY_BULK;
  if (!local) variant = ctx->remote_variant;
  if (tx_overcount) variant = EMM_COPY_BULK;  // the test hook exists for the bulk family's wait only
  if (align < 16) variant = EMM_COPY_LDG;

  PageCopyArgs a;
  a.src = src;
  a.dst = dst;
  a.n = (uint32_t)n;
  a.plane_shift = planes == 2 ? 1u : 0u;
  a.layer_begin = (uint32_t)layer_begin;
  a.layer_count = (uint32_t)layer_count;
  a.page_bytes = (uint32_t)page_bytes;
  a.status = ctx->d_status;
  a.wait_limit_ns = ctx->wait_limit_ns;
  a.tx_overcount = tx_overcount;
  a.inline_count = 0;
  a.src_inline = a.dst_inline = 0;
  if ((inline_src || inline_dst) && n <= emm::kInlineIds) {
    a.inline_count = (uint32_t)n;
    if (inline_src) {
      a.src_inline = 1;
      for (int32_t i = 0; i < n; ++i) a.inline_ids[0][i] = (int32_t)inline_src[i];
    }
    if (inline_dst) {
      a.dst_inline = 1;
      for (int32_t i = 0; i < n; ++i) a.inline_ids[1][i] = (int32_t)inline_dst[i];
    }
  }
  const bool segmented = src.seg_prefix != nullptr || dst.seg_prefix != nullptr;

  int64_t chunk = ctx->chunk_bytes;
  if (chunk <= 0) chunk = (variant == EMM_COPY_BULK) ? 32768 : 65536;
  if (chunk > page_bytes) chunk = page_bytes;
  int warps = ctx->warps;
  int auto_ctas_per_sm = 0;
  if (variant == EMM_COPY_BULK) {
    if (warps <= 0) {
      // Measured on B200 with a 2-deep ring: throughput peaks sharply at two
      // lanes per SM for 32 KiB chunks, three for 16 KiB, five for 8 KiB and
      // eight for 4 KiB (one lane more or fewer costs 5-25 %), that is at
      // about 32 KiB of loads in flight per SM beyond one chunk.
      const int64_t in_flight = (int64_t)(ctx->stages - 1) * chunk;
      int lanes = (int)(1 + (32 * 1024 + in_flight / 2) / in_flight);
      lanes = std::max(1, std::min(lanes, 16));
      warps = std::min(lanes, emm::kMaxWarps);
      auto_ctas_per_sm = (lanes + warps - 1) / warps;
    }
    // The ring of warps*stages chunks must fit the opt-in shared memory.
    const int64_t budget = (int64_t)ctx->max_smem_optin - 2048;
    while ((int64_t)warps * ctx->stages * chunk > budget && chunk > 1024) chunk /= 2;
    chunk &= ~(int64_t)15;
    if (chunk < 16 || (int64_t)warps * ctx->stages * chunk > budget)
      return fail(EMM_ERR_BAD_ARG, "bulk ring of %d x %d chunks does not fit shared memory",
                  warps, ctx->stages);
  }
  a.chunk_bytes = (uint32_t)chunk;
  a.chunks_per_page = (uint32_t)((page_bytes + chunk - 1) / chunk);
  a.total_chunks = (uint64_t)layer_count * (uint64_t)planes * (uint64_t)n * a.chunks_per_page;

  if (variant == EMM_COPY_BULK) {
    const int smem = (int)((int64_t)warps * ctx->stages * chunk);
    if (int rc = ensure_bulk_smem(ctx->device, smem)) return rc;
    const int fit = std::max(1, (int)((ctx->max_smem_optin - 2048) / (smem + 1024)));
    int per_sm = ctx->ctas_per_sm > 0 ? ctx->ctas_per_sm : (auto_ctas_per_sm > 0 ? auto_ctas_per_sm : fit);
    per_sm = std::min(std::min(per_sm, fit), 2048 / (warps * 32));
    uint64_t want = (a.total_chunks + warps - 1) / warps;
    uint64_t cap = (uint64_t)ctx->sm_count * per_sm;
    if (ctx->max_ctas > 0) cap = std::min<uint64_t>(cap, ctx->max_ctas);
    const int grid = (int)std::min<uint64_t>(want, cap);
    // Launched with programmatic stream serialisation: when the previous kernel in the stream is another
    // copy of this library, this grid's CTAs are placed and set up their rings while that one drains.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)(warps * 32));
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    const uint32_t stages_arg = (uint32_t)ctx->stages, hint_arg = (uint32_t)ctx->l2_hint;
    if (segmented) EMM_CUDA(cudaLaunchKernelEx(&cfg, emm::page_copy_bulk<true>, a, stages_arg, hint_arg));
    else EMM_CUDA(cudaLaunchKernelEx(&cfg, emm::page_copy_bulk<false>, a, stages_arg, hint_arg));
  } else {
    // A copy to or from a peer GPU or pinned host memory is bound by the link, not
    // by HBM: 48 CTAs already saturate NVLink (measured), and side-by-side copies
    // from several peers only keep the link rate when together they hold at most
    // one CTA per SM, so the default is one per SM and callers cap it further.
    const int per_sm = ctx->ctas_per_sm > 0 ? ctx->ctas_per_sm : (local ? 4 : 1);
    uint64_t cap = (uint64_t)ctx->sm_count * per_sm;
    if (ctx->max_ctas > 0) cap = std::min<uint64_t>(cap, ctx->max_ctas);
    const int grid = (int)std::min<uint64_t>(a.total_chunks, cap);
    if (segmented) launch_ldg<true>(ctx, a, grid, align, st);
    else launch_ldg<false>(ctx, a, grid, align, st);
  }
  EMM_CUDA(cudaGetLastError());
  ctx->launches += 1;
  return EMM_OK;
}

int check_pool_for_pages(const emm_pool *p, const char *what) {
  if (!p) return fail(EMM_ERR_BAD_ARG, "%s: null pool", what);
  if (p->page_bytes == 0)
    return fail(EMM_ERR_BAD_ARG, "%s: pool pages are not dense; whole-block moves unsupported", what);
  return EMM_OK;
}

int check_layer_range(const emm_pool *p, int32_t begin, int32_t count) {
  if (begin < 0 || count < 0 || (int64_t)begin + count > p->desc.num_layers)
    return fail(EMM_ERR_BAD_ARG, "layer range [%d, %d) outside [0, %d)", begin, begin + count,
                p->desc.num_layers);
  return EMM_OK;
}

int packed_copy(emm_pool *pool, bool to_packed, int32_t layer_begin, int32_t layer_count,
                const int32_t *d_ids, int32_t n, const void *d_packed, uint64_t packed_bytes,
                void *stream, const uint32_t *d_seg_prefix = nullptr, int32_t num_segs = 0,
                uint32_t tx_overcount = 0, const int64_t *h_inline_ids = nullptr) {
  const char *what = to_packed ? "gather" : "scatter";
  if (int rc = check_pool_for_pages(pool, what)) return rc;
  if (int rc = check_layer_range(pool, layer_begin, layer_count)) return rc;
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "%s: negative block count %d", what, n);
  const uint64_t want = (uint64_t)layer_count * (uint64_t)pool->planes * (uint64_t)n * (uint64_t)pool->page_bytes;
  if (packed_bytes != want)
    return fail(EMM_ERR_LENGTH, "%s: packed buffer holds %llu bytes, %d blocks need %llu", what,
                (unsigned long long)packed_bytes, n, (unsigned long long)want);
  if (n == 0 || layer_count == 0) return EMM_OK;
  if ((!d_ids && !h_inline_ids) || !d_packed) return fail(EMM_ERR_BAD_ARG, "%s: null pointer", what);
  const uint32_t align = std::min(pool->align, pow2_align((uint64_t)d_packed));
  if (align < (uint32_t)pool->desc.elem_size)
    return fail(EMM_ERR_ALIGN, "%s: packed buffer not aligned to elem_size", what);
  CopySide ps = pool_side(pool, d_ids);
  CopySide bs = packed_side(d_packed, n, pool->page_bytes, pool->planes);
  if (d_seg_prefix) {
    bs.seg_prefix = d_seg_prefix;
    bs.num_segs = (uint32_t)num_segs;
    bs.seg_stride = (uint64_t)layer_count * (uint64_t)pool->planes * (uint64_t)pool->page_bytes;
  }
  if (tx_overcount && align < 16) return fail(EMM_ERR_ALIGN, "%s: the wait test needs 16-byte granular pages", what);
  return to_packed ? launch_page_copy(pool->ctx, ps, bs, n, layer_begin, layer_count,
                                      pool->page_bytes, align, pool->device_local,
                                      (cudaStream_t)stream, pool->planes, tx_overcount, h_inline_ids, nullptr)
                   : launch_page_copy(pool->ctx, bs, ps, n, layer_begin, layer_count,
                                      pool->page_bytes, align, pool->device_local,
                                      (cudaStream_t)stream, pool->planes, tx_overcount, nullptr, h_inline_ids);
}

// Uploads host ids (already validated) into a ring slot; returns the device
// pointers of the first and (optional) second table.
int upload_ids(emm_ctx *ctx, const int64_t *a, const int64_t *b, int32_t n, cudaStream_t st,
               IdSlot **slot_out, const int32_t **d_a, const int32_t **d_b) {
  IdSlot *s = nullptr;
  const size_t total = (size_t)n * (b ? 2 : 1);
  if (int rc = acquire_slot(ctx, total, &s)) return rc;
  for (int32_t i = 0; i < n; ++i) s->h[i] = (int32_t)a[i];
  if (b)
    for (int32_t i = 0; i < n; ++i) s->h[n + i] = (int32_t)b[i];
  EMM_CUDA(cudaMemcpyAsync(s->d, s->h, total * sizeof(int32_t), cudaMemcpyHostToDevice, st));
  *d_a = s->d;
  if (d_b) *d_b = b ? s->d + n : nullptr;
  *slot_out = s;
  return EMM_OK;
}

int finish_slot(IdSlot *s, cudaStream_t st) {
  EMM_CUDA(cudaEventRecord(s->ev, st));
  s->pending = true;
  return EMM_OK;
}

}  // namespace

extern "C" {

int emm_abi_version(void) { return EMM_KV_ABI_VERSION; }

const char *emm_status_string(int status) {
  switch (status) {
    case EMM_OK: return "ok";
    case EMM_ERR_BAD_ARG: return "bad argument";
    case EMM_ERR_ID_RANGE: return "block id or slot out of range";
    case EMM_ERR_LENGTH: return "length mismatch";
    case EMM_ERR_CUDA: return "CUDA error";
    case EMM_ERR_TIMEOUT: return "device-side wait timed out";
    case EMM_ERR_ALIGN: return "misaligned pointer or stride";
    case EMM_ERR_DUPLICATE: return "duplicate destination id";
    case EMM_ERR_OVERLAP: return "source and destination ids overlap";
    case EMM_ERR_TOO_LARGE: return "size exceeds capacity";
    case EMM_ERR_NOMEM: return "out of memory";
    case EMM_ERR_NCCL: return "NCCL unavailable or failed";
    default: return "unknown status";
  }
}

const char *emm_last_error(void) { return g_last_error.c_str(); }

int emm_ctx_create(int device, emm_ctx **out) {
  if (!out) return fail(EMM_ERR_BAD_ARG, "emm_ctx_create: null out");
  *out = nullptr;
  int count = 0;
  EMM_CUDA(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count)
    return fail(EMM_ERR_BAD_ARG, "device %d not in [0, %d)", device, count);
  DeviceGuard guard(device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", device);
  emm_ctx *ctx = new (std::nothrow) emm_ctx();
  if (!ctx) return fail(EMM_ERR_NOMEM, "emm_ctx_create: host allocation failed");
  ctx->device = device;
  cudaError_t e = cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e == cudaSuccess)
    e = cudaDeviceGetAttribute(&ctx->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  if (e == cudaSuccess) e = cudaMalloc(&ctx->d_status, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(&ctx->h_status, 4 * sizeof(int));
  if (e != cudaSuccess) {
    if (ctx->d_status) cudaFree(ctx->d_status);
    delete ctx;
    return fail(EMM_ERR_CUDA, "emm_ctx_create: %s", cudaGetErrorString(e));
  }
  *out = ctx;
  return EMM_OK;
}

int emm_ctx_destroy(emm_ctx *ctx) {
  if (!ctx) return EMM_OK;
  DeviceGuard guard(ctx->device);
  cudaDeviceSynchronize();
  for (IdSlot &s : ctx->ring) {
    if (s.h) cudaFreeHost(s.h);
    if (s.d) cudaFree(s.d);
    if (s.ev) cudaEventDestroy(s.ev);
  }
  for (IpcMapping &m : ctx->ipc) cudaIpcCloseMemHandle(m.base);
  if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
  if (ctx->wire_stream) cudaStreamDestroy(ctx->wire_stream);
  for (cudaEvent_t e : {ctx->ev_entry, ctx->ev_copied[0], ctx->ev_copied[1], ctx->ev_wired[0], ctx->ev_wired[1],
                        ctx->ev_done[0], ctx->ev_done[1]})
    if (e) cudaEventDestroy(e);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  delete ctx;
  return EMM_OK;
}

int emm_ctx_set_option(emm_ctx *ctx, int option, int64_t value) {
  if (!ctx) return fail(EMM_ERR_BAD_ARG, "null context");
  switch (option) {
    case EMM_OPT_COPY_VARIANT:
      if (value < EMM_COPY_AUTO || value > EMM_COPY_LDG)
        return fail(EMM_ERR_BAD_ARG, "copy variant %lld unknown", (long long)value);
      ctx->copy_variant = (int)value;
      return EMM_OK;
    case EMM_OPT_CHUNK_BYTES:
      if (value < 0 || value % 16 || value > (1 << 20))
        return fail(EMM_ERR_BAD_ARG, "chunk bytes must be a multiple of 16 in [0, 1 MiB]");
      ctx->chunk_bytes = value;
      return EMM_OK;
    case EMM_OPT_STAGES:
      if (value < 2 || value > emm::kMaxStages)
        return fail(EMM_ERR_BAD_ARG, "stages must be in [2, %d]", emm::kMaxStages);
      ctx->stages = (int)value;
      return EMM_OK;
    case EMM_OPT_WARPS:
      if (value < 0 || value > emm::kMaxWarps)
        return fail(EMM_ERR_BAD_ARG, "warps must be in [0, %d] (0 = automatic)", emm::kMaxWarps);
      ctx->warps = (int)value;
      return EMM_OK;
    case EMM_OPT_CTAS_PER_SM:
      if (value < 0 || value > 32) return fail(EMM_ERR_BAD_ARG, "CTAs per SM must be in [0, 32]");
      ctx->ctas_per_sm = (int)value;
      return EMM_OK;
    case EMM_OPT_LDG_UNROLL:
      if (value != 1 && value != 2 && value != 4 && value != 8)
        return fail(EMM_ERR_BAD_ARG, "LDG unroll must be 1, 2, 4 or 8");
      ctx->ldg_unroll = (int)value;
      return EMM_OK;
    case EMM_OPT_MAX_CTAS:
      if (value < 0 || value > (1 << 20)) return fail(EMM_ERR_BAD_ARG, "max CTAs out of range");
      ctx->max_ctas = (int)value;
      return EMM_OK;
    case EMM_OPT_L2_HINT:
      if (value < 0 || value > 3) return fail(EMM_ERR_BAD_ARG, "L2 hint must be in [0, 3]");
      ctx->l2_hint = (int)value;
      return EMM_OK;
    case EMM_OPT_PDL:
      if (value != 0 && value != 1) return fail(EMM_ERR_BAD_ARG, "PDL option must be 0 or 1");
      ctx->pdl = (int)value;
      return EMM_OK;
    case EMM_OPT_WAIT_LIMIT_NS:
      if (value < 1000 || value > 60000000000ll)
        return fail(EMM_ERR_BAD_ARG, "wait limit must be between 1 us and 60 s (in ns)");
      ctx->wait_limit_ns = (uint64_t)value;
      return EMM_OK;
    case EMM_OPT_REMOTE_VARIANT:
      if (value != EMM_COPY_BULK && value != EMM_COPY_LDG)
        return fail(EMM_ERR_BAD_ARG, "remote variant must be EMM_COPY_BULK or EMM_COPY_LDG");
      ctx->remote_variant = (int)value;
      return EMM_OK;
    default:
      return fail(EMM_ERR_BAD_ARG, "unknown option %d", option);
  }
}

int emm_ctx_get_option(emm_ctx *ctx, int option, int64_t *value) {
  if (!ctx || !value) return fail(EMM_ERR_BAD_ARG, "null argument");
  switch (option) {
    case EMM_OPT_COPY_VARIANT: *value = ctx->copy_variant; return EMM_OK;
    case EMM_OPT_CHUNK_BYTES: *value = ctx->chunk_bytes; return EMM_OK;
    case EMM_OPT_STAGES: *value = ctx->stages; return EMM_OK;
    case EMM_OPT_WARPS: *value = ctx->warps; return EMM_OK;
    case EMM_OPT_CTAS_PER_SM: *value = ctx->ctas_per_sm; return EMM_OK;
    case EMM_OPT_LDG_UNROLL: *value = ctx->ldg_unroll; return EMM_OK;
    case EMM_OPT_MAX_CTAS: *value = ctx->max_ctas; return EMM_OK;
    case EMM_OPT_REMOTE_VARIANT: *value = ctx->remote_variant; return EMM_OK;
    case EMM_OPT_L2_HINT: *value = ctx->l2_hint; return EMM_OK;
    case EMM_OPT_WAIT_LIMIT_NS: *value = (int64_t)ctx->wait_limit_ns; return EMM_OK;
    case EMM_OPT_PDL: *value = ctx->pdl; return EMM_OK;
    default: return fail(EMM_ERR_BAD_ARG, "unknown option %d", option);
  }
}

int64_t emm_ctx_launch_count(emm_ctx *ctx) { return ctx ? ctx->launches : -1; }

int emm_ctx_status(emm_ctx *ctx, void *stream, int64_t *detail) {
  if (!ctx) return fail(EMM_ERR_BAD_ARG, "null context");
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  cudaStream_t st = (cudaStream_t)stream;
  EMM_CUDA(cudaMemcpyAsync(ctx->h_status, ctx->d_status, 4 * sizeof(int), cudaMemcpyDeviceToHost, st));
  EMM_CUDA(cudaMemsetAsync(ctx->d_status, 0, 4 * sizeof(int), st));
  EMM_CUDA(cudaStreamSynchronize(st));
  const int code = ctx->h_status[0];
  const int64_t d = (int64_t)(((uint64_t)(uint32_t)ctx->h_status[2] << 32) | (uint32_t)ctx->h_status[1]);
  if (detail) *detail = d;
  if (code != EMM_OK)
    return fail(code, "device reported '%s' (detail %lld)", emm_status_string(code), (long long)d);
  return EMM_OK;
}

static int fill_desc(emm_pool_desc *d, int L, int NB, int BS, int H, int D, int e, bool hnd) {
  if (!d) return fail(EMM_ERR_BAD_ARG, "null descriptor");
  d->num_layers = L;
  d->num_blocks = NB;
  d->block_size = BS;
  d->num_kv_heads = H;
  d->head_size = D;
  d->elem_size = e;
  d->num_planes = 2;
  d->reserved = 0;
  const int64_t head_bytes = (int64_t)D * e;
  const int64_t page = (int64_t)BS * H * head_bytes;
  d->block_stride = page;
  d->plane_stride = page * NB;
  if (hnd) {
    d->token_stride = head_bytes;
    d->head_stride = head_bytes * BS;
  } else {
    d->token_stride = head_bytes * H;
    d->head_stride = head_bytes;
  }
  bool dense;
  return check_desc(*d, &dense);
}

int emm_pool_desc_nhd(emm_pool_desc *desc, int L, int NB, int BS, int H, int D, int elem_size) {
  return fill_desc(desc, L, NB, BS, H, D, elem_size, false);
}

int emm_pool_desc_hnd(emm_pool_desc *desc, int L, int NB, int BS, int H, int D, int elem_size) {
  return fill_desc(desc, L, NB, BS, H, D, elem_size, true);
}

int emm_pool_desc_blocks(emm_pool_desc *desc, int L, int NB, int rows, int cols, int elem_size) {
  if (!desc) return fail(EMM_ERR_BAD_ARG, "null descriptor");
  desc->num_layers = L;
  desc->num_blocks = NB;
  desc->block_size = rows;
  desc->num_kv_heads = 1;
  desc->head_size = cols;
  desc->elem_size = elem_size;
  desc->num_planes = 1;
  desc->reserved = 0;
  const int64_t row_bytes = (int64_t)cols * elem_size;
  desc->token_stride = row_bytes;
  desc->head_stride = row_bytes;
  desc->block_stride = row_bytes * rows;
  desc->plane_stride = 0;
  bool dense;
  return check_desc(*desc, &dense);
}

int emm_pool_create(emm_ctx *ctx, const emm_pool_desc *desc, const void *const *layer_ptrs,
                    emm_pool **out) {
  if (!ctx || !desc || !layer_ptrs || !out) return fail(EMM_ERR_BAD_ARG, "emm_pool_create: null argument");
  *out = nullptr;
  bool dense = false;
  if (int rc = check_desc(*desc, &dense)) return rc;
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);

  emm_pool *p = new (std::nothrow) emm_pool();
  if (!p) return fail(EMM_ERR_NOMEM, "emm_pool_create: host allocation failed");
  p->ctx = ctx;
  p->device = ctx->device;
  p->desc = *desc;
  p->planes = desc->num_planes == 1 ? 1 : 2;
  p->desc.num_planes = p->planes;
  p->page_bytes = dense ? (int64_t)desc->block_size * desc->num_kv_heads * desc->head_size * desc->elem_size : 0;
  uint32_t align = pow2_align((uint64_t)desc->block_stride);
  if (p->planes == 2) align = std::min(align, pow2_align((uint64_t)desc->plane_stride));
  if (dense) align = std::min(align, pow2_align((uint64_t)p->page_bytes));
  p->h_layers.resize(desc->num_layers);
  for (int l = 0; l < desc->num_layers; ++l) {
    if (!layer_ptrs[l]) {
      delete p;
      return fail(EMM_ERR_BAD_ARG, "layer %d base pointer is null", l);
    }
    p->h_layers[l] = (uint64_t)layer_ptrs[l];
    align = std::min(align, pow2_align(p->h_layers[l]));
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, layer_ptrs[l]);
    if (e != cudaSuccess) {
      cudaGetLastError();
      p->device_local = false;
    } else if (attr.type != cudaMemoryTypeDevice || attr.device != ctx->device) {
      p->device_local = false;
    }
  }
  if (align < (uint32_t)desc->elem_size) {
    delete p;
    return fail(EMM_ERR_ALIGN, "layer base pointers not aligned to elem_size");
  }
  p->align = align;
  cudaError_t e = cudaMalloc(&p->d_layers, sizeof(uint64_t) * desc->num_layers);
  if (e == cudaSuccess)
    e = cudaMemcpy(p->d_layers, p->h_layers.data(), sizeof(uint64_t) * desc->num_layers,
                   cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (p->d_layers) cudaFree(p->d_layers);
    delete p;
    return fail(EMM_ERR_CUDA, "emm_pool_create: %s", cudaGetErrorString(e));
  }
  *out = p;
  return EMM_OK;
}

int emm_pool_destroy(emm_pool *pool) {
  if (!pool) return EMM_OK;
  DeviceGuard guard(pool->device);
  if (pool->d_layers) cudaFree(pool->d_layers);
  delete pool;
  return EMM_OK;
}

int emm_pool_get_desc(const emm_pool *pool, emm_pool_desc *desc) {
  if (!pool || !desc) return fail(EMM_ERR_BAD_ARG, "null argument");
  *desc = pool->desc;
  return EMM_OK;
}

int64_t emm_pool_page_bytes(const emm_pool *pool) { return pool ? pool->page_bytes : -1; }

int emm_gather(emm_pool *pool, const int32_t *d_ids, int32_t n, void *d_packed,
               uint64_t packed_bytes, void *stream) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "gather: null pool");
  return packed_copy(pool, true, 0, pool->desc.num_layers, d_ids, n, d_packed, packed_bytes, stream);
}

int emm_scatter(emm_pool *pool, const int32_t *d_ids, int32_t n, const void *d_packed,
                uint64_t packed_bytes, void *stream) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "scatter: null pool");
  return packed_copy(pool, false, 0, pool->desc.num_layers, d_ids, n, d_packed, packed_bytes, stream);
}

int emm_gather_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count,
                      const int32_t *d_ids, int32_t n, void *d_packed, uint64_t packed_bytes,
                      void *stream) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "gather: null pool");
  return packed_copy(pool, true, layer_begin, layer_count, d_ids, n, d_packed, packed_bytes, stream);
}

int emm_scatter_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count,
                       const int32_t *d_ids, int32_t n, const void *d_packed,
                       uint64_t packed_bytes, void *stream) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "scatter: null pool");
  return packed_copy(pool, false, layer_begin, layer_count, d_ids, n, d_packed, packed_bytes, stream);
}

int emm_test_gather_expect_overcount(emm_pool *pool, const int32_t *d_ids, int32_t n, void *d_packed,
                                     uint64_t packed_bytes, uint32_t extra_tx_bytes, void *stream) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "gather: null pool");
  if (extra_tx_bytes == 0 || extra_tx_bytes > (1u << 20))
    return fail(EMM_ERR_BAD_ARG, "extra_tx_bytes must be in [1, 1 MiB]");
  return packed_copy(pool, true, 0, pool->desc.num_layers, d_ids, n, d_packed, packed_bytes, stream, nullptr, 0,
                     extra_tx_bytes);
}

static int many_impl(emm_pool *pool, bool to_packed, int32_t layer_begin, int32_t layer_count,
                     const int32_t *d_ids, const uint32_t *d_seg_prefix, int32_t num_segs, int32_t n_total,
                     const void *d_packed, uint64_t packed_bytes, void *stream) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "gather/scatter_many: null pool");
  if (num_segs < 0 || n_total < 0) return fail(EMM_ERR_BAD_ARG, "gather/scatter_many: negative count");
  if (n_total > 0 && (num_segs == 0 || !d_seg_prefix))
    return fail(EMM_ERR_BAD_ARG, "gather/scatter_many: blocks without segments");
  if (layer_count < 0) layer_count = pool->desc.num_layers - layer_begin;
  return packed_copy(pool, to_packed, layer_begin, layer_count, d_ids, n_total, d_packed, packed_bytes, stream,
                     d_seg_prefix, num_segs);
}

int emm_gather_many(emm_pool *pool, const int32_t *d_ids, const uint32_t *d_seg_prefix, int32_t num_segs,
                    int32_t n_total, void *d_packed, uint64_t packed_bytes, void *stream) {
  return many_impl(pool, true, 0, -1, d_ids, d_seg_prefix, num_segs, n_total, d_packed, packed_bytes, stream);
}

int emm_scatter_many(emm_pool *pool, const int32_t *d_ids, const uint32_t *d_seg_prefix, int32_t num_segs,
                     int32_t n_total, const void *d_packed, uint64_t packed_bytes, void *stream) {
  return many_impl(pool, false, 0, -1, d_ids, d_seg_prefix, num_segs, n_total, d_packed, packed_bytes, stream);
}

int emm_gather_many_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count, const int32_t *d_ids,
                           const uint32_t *d_seg_prefix, int32_t num_segs, int32_t n_total, void *d_packed,
                           uint64_t packed_bytes, void *stream) {
  if (layer_count < 0) return fail(EMM_ERR_BAD_ARG, "gather_many_layers: negative layer count");
  return many_impl(pool, true, layer_begin, layer_count, d_ids, d_seg_prefix, num_segs, n_total, d_packed,
                   packed_bytes, stream);
}

int emm_scatter_many_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count, const int32_t *d_ids,
                            const uint32_t *d_seg_prefix, int32_t num_segs, int32_t n_total,
                            const void *d_packed, uint64_t packed_bytes, void *stream) {
  if (layer_count < 0) return fail(EMM_ERR_BAD_ARG, "scatter_many_layers: negative layer count");
  return many_impl(pool, false, layer_begin, layer_count, d_ids, d_seg_prefix, num_segs, n_total, d_packed,
                   packed_bytes, stream);
}

}  // extern "C"

static int copy_blocks_impl(emm_pool *src, emm_pool *dst, const int32_t *d_src_ids, const int32_t *d_dst_ids,
                            const int64_t *h_src_inline, const int64_t *h_dst_inline, int32_t n, void *stream) {
  if (int rc = check_pool_for_pages(src, "copy_blocks(src)")) return rc;
  if (int rc = check_pool_for_pages(dst, "copy_blocks(dst)")) return rc;
  if (src->ctx != dst->ctx) return fail(EMM_ERR_BAD_ARG, "copy_blocks: pools of different contexts");
  if (src->page_bytes != dst->page_bytes || src->desc.num_layers != dst->desc.num_layers ||
      src->planes != dst->planes)
    return fail(EMM_ERR_LENGTH, "copy_blocks: pools differ in page size (%lld vs %lld), layers (%d vs %d) or planes",
                (long long)src->page_bytes, (long long)dst->page_bytes, src->desc.num_layers,
                dst->desc.num_layers);
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "copy_blocks: negative block count");
  if (n == 0) return EMM_OK;
  if ((!d_src_ids || !d_dst_ids) && (!h_src_inline || !h_dst_inline))
    return fail(EMM_ERR_BAD_ARG, "copy_blocks: null id table");
  return launch_page_copy(src->ctx, pool_side(src, d_src_ids), pool_side(dst, d_dst_ids), n, 0,
                          src->desc.num_layers, src->page_bytes, std::min(src->align, dst->align),
                          src->device_local && dst->device_local, (cudaStream_t)stream, src->planes, 0,
                          h_src_inline, h_dst_inline);
}

extern "C" {

int emm_copy_blocks(emm_pool *src, emm_pool *dst, const int32_t *d_src_ids,
                    const int32_t *d_dst_ids, int32_t n, void *stream) {
  return copy_blocks_impl(src, dst, d_src_ids, d_dst_ids, nullptr, nullptr, n, stream);
}

int emm_gather_h(emm_pool *pool, const int64_t *h_ids, int32_t n, void *d_packed,
                 uint64_t packed_bytes, void *stream) {
  if (int rc = check_pool_for_pages(pool, "gather")) return rc;
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "gather: negative block count");
  if (n > 0 && !h_ids) return fail(EMM_ERR_BAD_ARG, "gather: null id list");
  if (int rc = check_ids_host(h_ids, n, pool->desc.num_blocks, "gather")) return rc;
  if (n == 0) return packed_copy(pool, true, 0, pool->desc.num_layers, nullptr, 0, d_packed, packed_bytes, stream);
  if (n <= emm::kInlineIds)  // a short table rides in the kernel arguments: no staging copy
    return packed_copy(pool, true, 0, pool->desc.num_layers, nullptr, n, d_packed, packed_bytes, stream, nullptr, 0, 0,
                       h_ids);
  DeviceGuard guard(pool->ctx->device);
  IdSlot *slot;
  const int32_t *d_ids;
  if (int rc = upload_ids(pool->ctx, h_ids, nullptr, n, (cudaStream_t)stream, &slot, &d_ids, nullptr)) return rc;
  int rc = packed_copy(pool, true, 0, pool->desc.num_layers, d_ids, n, d_packed, packed_bytes, stream);
  int rc2 = finish_slot(slot, (cudaStream_t)stream);
  return rc ? rc : rc2;
}

int emm_scatter_h(emm_pool *pool, const int64_t *h_ids, int32_t n, const void *d_packed,
                  uint64_t packed_bytes, void *stream) {
  if (int rc = check_pool_for_pages(pool, "scatter")) return rc;
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "scatter: negative block count");
  if (n > 0 && !h_ids) return fail(EMM_ERR_BAD_ARG, "scatter: null id list");
  if (int rc = check_ids_host(h_ids, n, pool->desc.num_blocks, "scatter")) return rc;
  if (n == 0) return packed_copy(pool, false, 0, pool->desc.num_layers, nullptr, 0, d_packed, packed_bytes, stream);
  emm_ctx *ctx = pool->ctx;
  if (int rc = bitmap_reserve(ctx->bitmap, pool->desc.num_blocks)) return rc;
  int64_t dup = -1;
  const bool unique = bitmap_mark(ctx->bitmap, h_ids, n, &dup);
  bitmap_clear(ctx->bitmap, h_ids, n);
  if (!unique) return fail(EMM_ERR_DUPLICATE, "scatter: destination id %lld appears twice", (long long)dup);
  if (n <= emm::kInlineIds)
    return packed_copy(pool, false, 0, pool->desc.num_layers, nullptr, n, d_packed, packed_bytes, stream, nullptr, 0,
                       0, h_ids);
  DeviceGuard guard(ctx->device);
  IdSlot *slot;
  const int32_t *d_ids;
  if (int rc = upload_ids(ctx, h_ids, nullptr, n, (cudaStream_t)stream, &slot, &d_ids, nullptr)) return rc;
  int rc = packed_copy(pool, false, 0, pool->desc.num_layers, d_ids, n, d_packed, packed_bytes, stream);
  int rc2 = finish_slot(slot, (cudaStream_t)stream);
  return rc ? rc : rc2;
}

int emm_copy_blocks_h(emm_pool *src, emm_pool *dst, const int64_t *h_src_ids,
                      const int64_t *h_dst_ids, int32_t n, void *stream) {
  if (int rc = check_pool_for_pages(src, "copy_blocks(src)")) return rc;
  if (int rc = check_pool_for_pages(dst, "copy_blocks(dst)")) return rc;
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "copy_blocks: negative block count");
  if (n == 0) return EMM_OK;
  if (!h_src_ids || !h_dst_ids) return fail(EMM_ERR_BAD_ARG, "copy_blocks: null id list");
  if (int rc = check_ids_host(h_src_ids, n, src->desc.num_blocks, "copy_blocks source")) return rc;
  if (int rc = check_ids_host(h_dst_ids, n, dst->desc.num_blocks, "copy_blocks destination")) return rc;
  emm_ctx *ctx = src->ctx;
  if (int rc = bitmap_reserve(ctx->bitmap, std::max(src->desc.num_blocks, dst->desc.num_blocks))) return rc;
  int64_t dup = -1;
  bool ok = bitmap_mark(ctx->bitmap, h_dst_ids, n, &dup);
  int rc_check = EMM_OK;
  if (!ok) {
    rc_check = fail(EMM_ERR_DUPLICATE, "copy_blocks: destination id %lld appears twice", (long long)dup);
  } else if (src == dst || (src->h_layers == dst->h_layers)) {
    // Same memory: a source that is also a destination would be read and
    // written by different CTAs in an undefined order.
    for (int32_t i = 0; i < n; ++i) {
      const uint64_t w = (uint64_t)h_src_ids[i] >> 6, b = 1ull << (h_src_ids[i] & 63);
      if (ctx->bitmap[w] & b) {
        rc_check = fail(EMM_ERR_OVERLAP, "copy_blocks: block %lld is both source and destination",
                        (long long)h_src_ids[i]);
        break;
      }
    }
  }
  bitmap_clear(ctx->bitmap, h_dst_ids, n);
  if (rc_check) return rc_check;
  if (n <= emm::kInlineIds) return copy_blocks_impl(src, dst, nullptr, nullptr, h_src_ids, h_dst_ids, n, stream);
  DeviceGuard guard(ctx->device);
  IdSlot *slot;
  const int32_t *d_s, *d_d;
  if (int rc = upload_ids(ctx, h_src_ids, h_dst_ids, n, (cudaStream_t)stream, &slot, &d_s, &d_d)) return rc;
  int rc = emm_copy_blocks(src, dst, d_s, d_d, n, stream);
  int rc2 = finish_slot(slot, (cudaStream_t)stream);
  return rc ? rc : rc2;
}

int emm_upload_ids(emm_ctx *ctx, const int64_t *h_values, int32_t n, int32_t *d_out, void *stream) {
  if (!ctx) return fail(EMM_ERR_BAD_ARG, "upload_ids: null context");
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "upload_ids: negative count");
  if (n == 0) return EMM_OK;
  if (!h_values || !d_out) return fail(EMM_ERR_BAD_ARG, "upload_ids: null pointer");
  for (int32_t i = 0; i < n; ++i)
    if (h_values[i] < 0 || h_values[i] > 0x7fffffffll)
      return fail(EMM_ERR_ID_RANGE, "upload_ids: value %lld at position %d does not fit a non-negative int32",
                  (long long)h_values[i], i);
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  IdSlot *s = nullptr;
  if (int rc = acquire_slot(ctx, (size_t)n, &s)) return rc;
  for (int32_t i = 0; i < n; ++i) s->h[i] = (int32_t)h_values[i];
  EMM_CUDA(cudaMemcpyAsync(d_out, s->h, (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return finish_slot(s, (cudaStream_t)stream);
}

// Validates an append and fills the kernel arguments; *align_out receives the common
// power-of-two alignment of every address and stride involved.
static int append_prepare(emm_pool *pool, int32_t layer_begin, int32_t layer_count, const void *d_key,
                          const void *d_value, int64_t kls, int64_t kts, int64_t vls, int64_t vts,
                          const int64_t *d_slots, int32_t T, emm::AppendArgs *out, uint32_t *align_out) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "append: null pool");
  if (int rc = check_layer_range(pool, layer_begin, layer_count)) return rc;
  if (pool->planes != 2) return fail(EMM_ERR_BAD_ARG, "append: needs a KV pool (two planes)");
  if (T < 0) return fail(EMM_ERR_BAD_ARG, "append: negative token count");
  if (T > 0 && layer_count > 0 && (!d_key || !d_value || !d_slots)) return fail(EMM_ERR_BAD_ARG, "append: null pointer");
  const emm_pool_desc &d = pool->desc;
  const int64_t head_bytes = (int64_t)d.head_size * d.elem_size;
  const int64_t row_bytes = head_bytes * d.num_kv_heads;
  if (kts < row_bytes || vts < row_bytes)
    return fail(EMM_ERR_BAD_ARG, "append: token stride smaller than a token row (%lld bytes)", (long long)row_bytes);
  if (layer_count > 1 && (kls < (int64_t)T * row_bytes || vls < (int64_t)T * row_bytes))
    return fail(EMM_ERR_BAD_ARG, "append: layer stride smaller than one layer of rows");

  uint32_t align = pow2_align((uint64_t)head_bytes);
  for (int l = 0; l < d.num_layers; ++l) align = std::min(align, pow2_align(pool->h_layers[l]));
  const uint64_t parts[] = {(uint64_t)d.plane_stride, (uint64_t)d.block_stride, (uint64_t)d.token_stride,
                            (uint64_t)d.head_stride,  (uint64_t)d_key,          (uint64_t)d_value,
                            (uint64_t)kts,            (uint64_t)vts,
                            layer_count > 1 ? (uint64_t)kls : 0, layer_count > 1 ? (uint64_t)vls : 0};
  for (uint64_t v : parts) align = std::min(align, pow2_align(v));
  if (align < (uint32_t)d.elem_size) return fail(EMM_ERR_ALIGN, "append: key/value not aligned to elem_size");
  if ((uint64_t)layer_count * (uint64_t)T * 2ull > 0x3fffffffull)
    return fail(EMM_ERR_TOO_LARGE, "append: %d layers x %d tokens", layer_count, T);

  emm::AppendArgs &a = *out;
  a.layers = pool->d_layers;
  a.plane_stride = (uint64_t)d.plane_stride;
  a.block_stride = (uint64_t)d.block_stride;
  a.token_stride = (uint64_t)d.token_stride;
  a.head_stride = (uint64_t)d.head_stride;
  a.num_slots = (uint64_t)d.num_blocks * (uint64_t)d.block_size;
  a.block_size = (uint32_t)d.block_size;
  a.head_bytes = (uint32_t)head_bytes;
  a.row_bytes = (uint32_t)row_bytes;
  a.layer_begin = (uint32_t)layer_begin;
  a.layer_count = (uint32_t)layer_count;
  a.num_tokens = (uint32_t)T;
  a.key = (uint64_t)d_key;
  a.value = (uint64_t)d_value;
  a.key_layer_stride = (uint64_t)kls;
  a.key_token_stride = (uint64_t)kts;
  a.value_layer_stride = (uint64_t)vls;
  a.value_token_stride = (uint64_t)vts;
  a.slots = d_slots;
  a.status = pool->ctx->d_status;
  *align_out = align;
  return EMM_OK;
}

// Launches the append kernel for prepared arguments. Call with the context's device current.
static int append_launch(emm_ctx *ctx, const emm::AppendArgs &a, uint32_t align, cudaStream_t st) {
  if (a.num_tokens == 0 || a.layer_count == 0) return EMM_OK;
  const uint64_t rows = (uint64_t)a.layer_count * (uint64_t)a.num_tokens * 2ull;
  const int grid = (int)((rows + emm::kAppendWarps - 1) / emm::kAppendWarps);
  const int block = emm::kAppendWarps * 32;
  if (align >= 16) emm::append_rows<uint4, 4><<<grid, block, 0, st>>>(a);
  else if (align >= 8) emm::append_rows<uint2, 4><<<grid, block, 0, st>>>(a);
  else if (align >= 4) emm::append_rows<uint32_t, 4><<<grid, block, 0, st>>>(a);
  else if (align >= 2) emm::append_rows<uint16_t, 4><<<grid, block, 0, st>>>(a);
  else emm::append_rows<uint8_t, 4><<<grid, block, 0, st>>>(a);
  EMM_CUDA(cudaGetLastError());
  ctx->launches += 1;
  return EMM_OK;
}

static int append_impl(emm_pool *pool, int32_t layer_begin, int32_t layer_count, const void *d_key,
                       const void *d_value, int64_t kls, int64_t kts, int64_t vls, int64_t vts,
                       const int64_t *d_slots, int32_t T, void *stream) {
  emm::AppendArgs a;
  uint32_t align = 1;
  if (int rc = append_prepare(pool, layer_begin, layer_count, d_key, d_value, kls, kts, vls, vts, d_slots, T, &a,
                              &align))
    return rc;
  DeviceGuard guard(pool->ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", pool->ctx->device);
  return append_launch(pool->ctx, a, align, (cudaStream_t)stream);
}

int emm_append(emm_pool *pool, int32_t layer, const void *d_key, const void *d_value,
               int64_t key_token_stride, int64_t value_token_stride,
               const int64_t *d_slot_mapping, int32_t num_tokens, void *stream) {
  return append_impl(pool, layer, 1, d_key, d_value, 0, key_token_stride, 0, value_token_stride,
                     d_slot_mapping, num_tokens, stream);
}

int emm_append_all_layers(emm_pool *pool, const void *d_key, const void *d_value,
                          int64_t key_layer_stride, int64_t key_token_stride,
                          int64_t value_layer_stride, int64_t value_token_stride,
                          const int64_t *d_slot_mapping, int32_t num_tokens, void *stream) {
  if (!pool) return fail(EMM_ERR_BAD_ARG, "append: null pool");
  return append_impl(pool, 0, pool->desc.num_layers, d_key, d_value, key_layer_stride,
                     key_token_stride, value_layer_stride, value_token_stride, d_slot_mapping,
                     num_tokens, stream);
}

}  // extern "C"

// A per-layer append over static buffers, validated once: what a decode loop that refills the
// same key/value/slot buffers every step calls once per layer.
struct emm_append_binding {
  emm_pool *pool = nullptr;
  emm::AppendArgs args{};   // layer 0, one layer; the launch fills in the layer
  uint32_t align = 1;
  uint64_t key0 = 0, value0 = 0, key_layer_stride = 0, value_layer_stride = 0;
  int32_t num_layers = 0;
};

extern "C" {

int emm_append_bind(emm_pool *pool, const void *d_key, const void *d_value, int64_t key_layer_stride,
                    int64_t key_token_stride, int64_t value_layer_stride, int64_t value_token_stride,
                    const int64_t *d_slot_mapping, int32_t num_tokens, emm_append_binding **out) {
  if (!out) return fail(EMM_ERR_BAD_ARG, "append_bind: null out");
  *out = nullptr;
  if (!pool) return fail(EMM_ERR_BAD_ARG, "append_bind: null pool");
  emm_append_binding *b = new (std::nothrow) emm_append_binding();
  if (!b) return fail(EMM_ERR_NOMEM, "append_bind: host allocation failed");
  // Validated as the all-layers call (every layer's rows must exist), launched one layer at a time.
  if (int rc = append_prepare(pool, 0, pool->desc.num_layers, d_key, d_value, key_layer_stride, key_token_stride,
                              value_layer_stride, value_token_stride, d_slot_mapping, num_tokens, &b->args,
                              &b->align)) {
    delete b;
    return rc;
  }
  b->pool = pool;
  b->key0 = (uint64_t)d_key;
  b->value0 = (uint64_t)d_value;
  b->key_layer_stride = (uint64_t)key_layer_stride;
  b->value_layer_stride = (uint64_t)value_layer_stride;
  b->num_layers = pool->desc.num_layers;
  b->args.layer_count = 1;
  b->args.key_layer_stride = 0;
  b->args.value_layer_stride = 0;
  *out = b;
  return EMM_OK;
}

int emm_append_bound(emm_append_binding *b, int32_t layer, void *stream) {
  if (!b) return fail(EMM_ERR_BAD_ARG, "append_bound: null binding");
  if (layer < 0 || layer >= b->num_layers)
    return fail(EMM_ERR_BAD_ARG, "append_bound: layer %d outside [0, %d)", layer, b->num_layers);
  emm_ctx *ctx = b->pool->ctx;
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  emm::AppendArgs a = b->args;
  a.layer_begin = (uint32_t)layer;
  a.key = b->key0 + (uint64_t)layer * b->key_layer_stride;
  a.value = b->value0 + (uint64_t)layer * b->value_layer_stride;
  return append_launch(ctx, a, b->align, (cudaStream_t)stream);
}

int emm_append_unbind(emm_append_binding *b) {
  delete b;
  return EMM_OK;
}

int emm_compact_plan(const int64_t *table_ids, int64_t n_ids, int64_t num_blocks,
                     int64_t *new_table_ids, int64_t *move_src, int64_t *move_dst,
                     int64_t *n_moves) {
  if (n_ids < 0 || num_blocks <= 0 || !n_moves) return fail(EMM_ERR_BAD_ARG, "compact_plan: bad argument");
  *n_moves = 0;
  if (n_ids == 0) return EMM_OK;
  if (!table_ids || !new_table_ids || !move_src || !move_dst)
    return fail(EMM_ERR_BAD_ARG, "compact_plan: null pointer");
  if (n_ids > num_blocks)
    return fail(EMM_ERR_LENGTH, "compact_plan: %lld live ids in a pool of %lld blocks", (long long)n_ids,
                (long long)num_blocks);
  // seen[b]: block b is live; for b < n_ids it already sits in the dense prefix.
  std::vector<uint8_t> seen;
  try {
    seen.assign((size_t)num_blocks, 0);
  } catch (const std::bad_alloc &) {
    return fail(EMM_ERR_NOMEM, "compact_plan: no host memory for %lld flags", (long long)num_blocks);
  }
  for (int64_t i = 0; i < n_ids; ++i) {
    const int64_t id = table_ids[i];
    if (id < 0 || id >= num_blocks)
      return fail(EMM_ERR_ID_RANGE, "compact_plan: id %lld at position %lld outside [0, %lld)", (long long)id,
                  (long long)i, (long long)num_blocks);
    if (seen[(size_t)id])
      return fail(EMM_ERR_DUPLICATE, "compact_plan: block %lld belongs to two table entries", (long long)id);
    seen[(size_t)id] = 1;
  }
  int64_t hole = 0;  // next candidate free id inside the prefix
  int64_t moves = 0;
  for (int64_t i = 0; i < n_ids; ++i) {
    const int64_t id = table_ids[i];
    if (id < n_ids) {
      new_table_ids[i] = id;
      continue;
    }
    while (seen[(size_t)hole]) ++hole;  // a hole exists: #live outside prefix == #holes inside
    move_src[moves] = id;
    move_dst[moves] = hole;
    new_table_ids[i] = hole;
    ++hole;
    ++moves;
  }
  *n_moves = moves;
  return EMM_OK;
}

int emm_ipc_export(emm_ctx *ctx, const void *d_ptr, unsigned char handle[EMM_IPC_HANDLE_BYTES],
                   uint64_t *offset) {
  if (!ctx || !d_ptr || !handle || !offset) return fail(EMM_ERR_BAD_ARG, "ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == EMM_IPC_HANDLE_BYTES, "IPC handle size");
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  // The handle names the whole allocation; find its base through the driver.
  typedef int (*GetRangeFn)(unsigned long long *, size_t *, unsigned long long);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  EMM_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
  if (!fn || qres != cudaDriverEntryPointSuccess)
    return fail(EMM_ERR_CUDA, "ipc_export: driver entry point cuMemGetAddressRange unavailable");
  unsigned long long base = 0;
  size_t size = 0;
  const int drc = ((GetRangeFn)fn)(&base, &size, (unsigned long long)d_ptr);
  if (drc != 0) return fail(EMM_ERR_CUDA, "ipc_export: cuMemGetAddressRange returned %d", drc);
  cudaIpcMemHandle_t h;
  EMM_CUDA(cudaIpcGetMemHandle(&h, (void *)base));
  memcpy(handle, &h, EMM_IPC_HANDLE_BYTES);
  *offset = (uint64_t)d_ptr - (uint64_t)base;
  return EMM_OK;
}

int emm_ipc_open(emm_ctx *ctx, const unsigned char handle[EMM_IPC_HANDLE_BYTES], uint64_t offset,
                 void **d_ptr) {
  if (!ctx || !handle || !d_ptr) return fail(EMM_ERR_BAD_ARG, "ipc_open: null argument");
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  for (const IpcMapping &m : ctx->ipc) {
    if (memcmp(m.handle, handle, EMM_IPC_HANDLE_BYTES) == 0) {
      *d_ptr = (char *)m.base + offset;
      return EMM_OK;
    }
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, EMM_IPC_HANDLE_BYTES);
  void *base = nullptr;
  EMM_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  IpcMapping m;
  memcpy(m.handle, handle, EMM_IPC_HANDLE_BYTES);
  m.base = base;
  ctx->ipc.push_back(m);
  *d_ptr = (char *)base + offset;
  return EMM_OK;
}


int emm_enable_peer_access(emm_ctx *ctx, int peer_device) {
  if (!ctx) return fail(EMM_ERR_BAD_ARG, "enable_peer_access: null context");
  if (peer_device == ctx->device) return EMM_OK;
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  int can = 0;
  EMM_CUDA(cudaDeviceCanAccessPeer(&can, ctx->device, peer_device));
  if (!can) return fail(EMM_ERR_CUDA, "device %d cannot address device %d", ctx->device, peer_device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();  // clear the sticky "already enabled"
    return EMM_OK;
  }
  if (e != cudaSuccess) return fail(EMM_ERR_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
  return EMM_OK;
}

// ---------------------------------------------------------------------------
// Staged transport over NCCL (entry points resolved with dlopen / dlsym)
// ---------------------------------------------------------------------------
}  // extern "C"

namespace {

struct NcclUniqueId {
  char internal[EMM_NCCL_UNIQUE_ID_BYTES];
};
typedef int (*nccl_get_unique_id_fn)(NcclUniqueId *);
typedef int (*nccl_comm_init_rank_fn)(void **, int, NcclUniqueId, int);
typedef int (*nccl_comm_destroy_fn)(void *);
typedef int (*nccl_send_fn)(const void *, size_t, int, int, void *, cudaStream_t);
typedef int (*nccl_recv_fn)(void *, size_t, int, int, void *, cudaStream_t);
typedef int (*nccl_group_fn)(void);
typedef const char *(*nccl_error_string_fn)(int);
constexpr int kNcclInt8 = 0;  // ncclInt8 / ncclChar

struct NcclApi {
  std::once_flag once;
  void *lib = nullptr;
  nccl_get_unique_id_fn get_unique_id = nullptr;
  nccl_comm_init_rank_fn comm_init_rank = nullptr;
  nccl_comm_destroy_fn comm_destroy = nullptr;
  nccl_send_fn send = nullptr;
  nccl_recv_fn recv = nullptr;
  nccl_group_fn group_start = nullptr;
  nccl_group_fn group_end = nullptr;
  nccl_error_string_fn error_string = nullptr;
};
NcclApi g_nccl;

int nccl_api(NcclApi **out) {
  NcclApi &a = g_nccl;
  std::call_once(a.once, [&a] {
    const char *override_path = getenv("EMM_NCCL_LIB");
    // Prefer the copy the process has already loaded (the host framework's), then the search path.
    if (override_path && *override_path) a.lib = dlopen(override_path, RTLD_NOW | RTLD_GLOBAL);
    if (!a.lib) a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!a.lib) a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (a.lib) {
      a.get_unique_id = (nccl_get_unique_id_fn)dlsym(a.lib, "ncclGetUniqueId");
      a.comm_init_rank = (nccl_comm_init_rank_fn)dlsym(a.lib, "ncclCommInitRank");
      a.comm_destroy = (nccl_comm_destroy_fn)dlsym(a.lib, "ncclCommDestroy");
      a.send = (nccl_send_fn)dlsym(a.lib, "ncclSend");
      a.recv = (nccl_recv_fn)dlsym(a.lib, "ncclRecv");
      a.group_start = (nccl_group_fn)dlsym(a.lib, "ncclGroupStart");
      a.group_end = (nccl_group_fn)dlsym(a.lib, "ncclGroupEnd");
      a.error_string = (nccl_error_string_fn)dlsym(a.lib, "ncclGetErrorString");
    }
  });
  if (!a.lib || !a.get_unique_id || !a.comm_init_rank || !a.comm_destroy || !a.send || !a.recv ||
      !a.group_start || !a.group_end)
    return fail(EMM_ERR_NCCL, "libnccl.so.2 could not be loaded (set EMM_NCCL_LIB to its path): %s",
                a.lib ? "a symbol is missing" : "not found");
  *out = &a;
  return EMM_OK;
}

int nccl_fail(NcclApi *a, const char *what, int rc) {
  return fail(EMM_ERR_NCCL, "%s failed: %s (%d)", what, a->error_string ? a->error_string(rc) : "?", rc);
}

#define EMM_NCCL(api, call)                          \
  do {                                               \
    int r_ = (call);                                 \
    if (r_ != 0) return nccl_fail((api), #call, r_); \
  } while (0)

int transport_setup(emm_ctx *ctx) {
  if (ctx->copy_stream) return EMM_OK;
  EMM_CUDA(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
  EMM_CUDA(cudaStreamCreateWithFlags(&ctx->wire_stream, cudaStreamNonBlocking));
  cudaEvent_t *evs[] = {&ctx->ev_entry,    &ctx->ev_copied[0], &ctx->ev_copied[1], &ctx->ev_wired[0],
                        &ctx->ev_wired[1], &ctx->ev_done[0],   &ctx->ev_done[1]};
  for (cudaEvent_t *e : evs) EMM_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
  return EMM_OK;
}

int check_blocks_args(emm_pool *pool, void *comm, const int32_t *d_ids, int32_t n, void *d_staging,
                      uint64_t staging_bytes, int32_t layers_per_msg, const char *what) {
  if (int rc = check_pool_for_pages(pool, what)) return rc;
  if (!comm) return fail(EMM_ERR_BAD_ARG, "%s: null communicator", what);
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "%s: negative block count", what);
  if (n == 0) return EMM_OK;
  if (!d_ids || !d_staging) return fail(EMM_ERR_BAD_ARG, "%s: null pointer", what);
  if (layers_per_msg < 1 || layers_per_msg > pool->desc.num_layers)
    return fail(EMM_ERR_BAD_ARG, "%s: layers_per_msg %d outside [1, %d]", what, layers_per_msg,
                pool->desc.num_layers);
  const uint64_t msg = (uint64_t)layers_per_msg * pool->planes * (uint64_t)n * (uint64_t)pool->page_bytes;
  if (staging_bytes < 2 * msg)
    return fail(EMM_ERR_LENGTH, "%s: staging buffer holds %llu bytes, two messages need %llu", what,
                (unsigned long long)staging_bytes, (unsigned long long)(2 * msg));
  return EMM_OK;
}

}  // namespace

extern "C" {

int emm_nccl_unique_id(unsigned char id[EMM_NCCL_UNIQUE_ID_BYTES]) {
  if (!id) return fail(EMM_ERR_BAD_ARG, "nccl_unique_id: null output");
  NcclApi *api;
  if (int rc = nccl_api(&api)) return rc;
  NcclUniqueId u;
  EMM_NCCL(api, api->get_unique_id(&u));
  memcpy(id, u.internal, EMM_NCCL_UNIQUE_ID_BYTES);
  return EMM_OK;
}

int emm_nccl_comm_init(emm_ctx *ctx, const unsigned char id[EMM_NCCL_UNIQUE_ID_BYTES], int nranks,
                       int rank, void **comm) {
  if (!ctx || !id || !comm) return fail(EMM_ERR_BAD_ARG, "nccl_comm_init: null argument");
  if (nranks < 1 || rank < 0 || rank >= nranks)
    return fail(EMM_ERR_BAD_ARG, "nccl_comm_init: rank %d of %d", rank, nranks);
  NcclApi *api;
  if (int rc = nccl_api(&api)) return rc;
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  NcclUniqueId u;
  memcpy(u.internal, id, EMM_NCCL_UNIQUE_ID_BYTES);
  *comm = nullptr;
  EMM_NCCL(api, api->comm_init_rank(comm, nranks, u, rank));
  return EMM_OK;
}

int emm_nccl_comm_destroy(void *comm) {
  if (!comm) return EMM_OK;
  NcclApi *api;
  if (int rc = nccl_api(&api)) return rc;
  EMM_NCCL(api, api->comm_destroy(comm));
  return EMM_OK;
}

int emm_send_packed(void *comm, const void *d_buf, uint64_t bytes, int peer, void *stream) {
  if (!comm || (!d_buf && bytes)) return fail(EMM_ERR_BAD_ARG, "send_packed: null argument");
  NcclApi *api;
  if (int rc = nccl_api(&api)) return rc;
  if (bytes == 0) return EMM_OK;
  EMM_NCCL(api, api->send(d_buf, (size_t)bytes, kNcclInt8, peer, comm, (cudaStream_t)stream));
  return EMM_OK;
}

int emm_recv_packed(void *comm, void *d_buf, uint64_t bytes, int peer, void *stream) {
  if (!comm || (!d_buf && bytes)) return fail(EMM_ERR_BAD_ARG, "recv_packed: null argument");
  NcclApi *api;
  if (int rc = nccl_api(&api)) return rc;
  if (bytes == 0) return EMM_OK;
  EMM_NCCL(api, api->recv(d_buf, (size_t)bytes, kNcclInt8, peer, comm, (cudaStream_t)stream));
  return EMM_OK;
}

int emm_exchange(void *comm, int32_t n_ops, const int32_t *is_send, void *const *bufs,
                 const uint64_t *bytes, const int32_t *peers, void *stream) {
  if (!comm || n_ops < 0) return fail(EMM_ERR_BAD_ARG, "exchange: bad argument");
  if (n_ops == 0) return EMM_OK;
  if (!is_send || !bufs || !bytes || !peers) return fail(EMM_ERR_BAD_ARG, "exchange: null array");
  NcclApi *api;
  if (int rc = nccl_api(&api)) return rc;
  EMM_NCCL(api, api->group_start());
  int first_error = 0;
  for (int32_t k = 0; k < n_ops && !first_error; ++k) {
    if (bytes[k] == 0) continue;
    first_error = is_send[k] ? api->send(bufs[k], (size_t)bytes[k], kNcclInt8, peers[k], comm, (cudaStream_t)stream)
                             : api->recv(bufs[k], (size_t)bytes[k], kNcclInt8, peers[k], comm, (cudaStream_t)stream);
  }
  const int end_rc = api->group_end();  // always close the group
  if (first_error) return nccl_fail(api, "ncclSend/ncclRecv inside the group", first_error);
  if (end_rc) return nccl_fail(api, "ncclGroupEnd", end_rc);
  return EMM_OK;
}

// Shared body of emm_send_blocks / emm_recv_blocks.
static int staged_blocks(emm_pool *pool, void *comm, int peer, const int32_t *d_ids, int32_t n,
                         void *d_staging, uint64_t staging_bytes, int32_t layers_per_msg, void *stream,
                         bool sending) {
  const char *what = sending ? "send_blocks" : "recv_blocks";
  if (int rc = check_blocks_args(pool, comm, d_ids, n, d_staging, staging_bytes, layers_per_msg, what)) return rc;
  if (n == 0) return EMM_OK;
  NcclApi *api;
  if (int rc = nccl_api(&api)) return rc;
  emm_ctx *ctx = pool->ctx;
  DeviceGuard guard(ctx->device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", ctx->device);
  if (int rc = transport_setup(ctx)) return rc;
  // The pack / unpack kernels run beside the NCCL kernel, whose CTAs need an SM almost to themselves: unless
  // the caller set a cap, leave 48 SMs free for it (measured: ~630 instead of ~565 GB/s per pair).
  struct CapGuard {
    emm_ctx *c;
    int saved;
    ~CapGuard() { c->max_ctas = saved; }
  } cap_guard{ctx, ctx->max_ctas};
  if (ctx->max_ctas == 0) ctx->max_ctas = std::max(16, ctx->sm_count - 48);

  const int L = pool->desc.num_layers;
  const uint64_t layer_bytes = (uint64_t)pool->planes * (uint64_t)n * (uint64_t)pool->page_bytes;
  const uint64_t slot_bytes = (uint64_t)layers_per_msg * layer_bytes;
  char *slots[2] = {(char *)d_staging, (char *)d_staging + slot_bytes};
  cudaStream_t user = (cudaStream_t)stream, copy = ctx->copy_stream, wire = ctx->wire_stream;

  // Everything below is ordered after what the caller has queued on `stream`.
  EMM_CUDA(cudaEventRecord(ctx->ev_entry, user));
  EMM_CUDA(cudaStreamWaitEvent(copy, ctx->ev_entry, 0));
  EMM_CUDA(cudaStreamWaitEvent(wire, ctx->ev_entry, 0));

  int c = 0;
  for (int begin = 0; begin < L; begin += layers_per_msg, ++c) {
    const int count = std::min(layers_per_msg, L - begin);
    const uint64_t bytes = (uint64_t)count * layer_bytes;
    const int s = c & 1;
    if (sending) {
      // pack message c once the send that last read this slot is done, then put it on the wire
      if (c >= 2) EMM_CUDA(cudaStreamWaitEvent(copy, ctx->ev_wired[s], 0));
      if (int rc = packed_copy(pool, true, begin, count, d_ids, n, slots[s], bytes, copy)) return rc;
      EMM_CUDA(cudaEventRecord(ctx->ev_copied[s], copy));
      EMM_CUDA(cudaStreamWaitEvent(wire, ctx->ev_copied[s], 0));
      EMM_NCCL(api, api->send(slots[s], (size_t)bytes, kNcclInt8, peer, comm, wire));
      EMM_CUDA(cudaEventRecord(ctx->ev_wired[s], wire));
    } else {
      // receive message c once the unpack that last read this slot is done, then scatter it
      if (c >= 2) EMM_CUDA(cudaStreamWaitEvent(wire, ctx->ev_copied[s], 0));
      EMM_NCCL(api, api->recv(slots[s], (size_t)bytes, kNcclInt8, peer, comm, wire));
      EMM_CUDA(cudaEventRecord(ctx->ev_wired[s], wire));
      EMM_CUDA(cudaStreamWaitEvent(copy, ctx->ev_wired[s], 0));
      if (int rc = packed_copy(pool, false, begin, count, d_ids, n, slots[s], bytes, copy)) return rc;
      EMM_CUDA(cudaEventRecord(ctx->ev_copied[s], copy));
    }
  }
  // Join both helper streams back into the caller's stream.
  EMM_CUDA(cudaEventRecord(ctx->ev_done[0], copy));
  EMM_CUDA(cudaEventRecord(ctx->ev_done[1], wire));
  EMM_CUDA(cudaStreamWaitEvent(user, ctx->ev_done[0], 0));
  EMM_CUDA(cudaStreamWaitEvent(user, ctx->ev_done[1], 0));
  return EMM_OK;
}

int emm_send_blocks(emm_pool *pool, void *comm, int peer, const int32_t *d_ids, int32_t n,
                    void *d_staging, uint64_t staging_bytes, int32_t layers_per_msg, void *stream) {
  return staged_blocks(pool, comm, peer, d_ids, n, d_staging, staging_bytes, layers_per_msg, stream, true);
}

int emm_recv_blocks(emm_pool *pool, void *comm, int peer, const int32_t *d_ids, int32_t n,
                    void *d_staging, uint64_t staging_bytes, int32_t layers_per_msg, void *stream) {
  return staged_blocks(pool, comm, peer, d_ids, n, d_staging, staging_bytes, layers_per_msg, stream, false);
}

// ---------------------------------------------------------------------------
// Gather without any allocation (see emm_gather_noalloc in emm_kv.h)
// ---------------------------------------------------------------------------
}  // extern "C"

namespace {

// Fixed scratch inside the library image: [0,16) status word, then the layer
// pointer array, then the id table. Every GPU that loads the library holds it.
constexpr size_t kNaStatusBytes = 256;
constexpr size_t kNaLayersBytes = EMM_NOALLOC_MAX_LAYERS * sizeof(uint64_t);
constexpr size_t kNaIdsBytes = EMM_NOALLOC_MAX_IDS * sizeof(int32_t);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaStatusBytes + kNaLayersBytes + kNaIdsBytes];

constexpr int kNaMaxDevices = 64;
struct NoAllocDevice {
  std::once_flag once;
  int setup_rc = EMM_OK;
  std::string setup_error;
  unsigned char *scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int sm_count = 0;
  int max_smem_optin = 0;
};
NoAllocDevice g_noalloc_dev[kNaMaxDevices];

// Once per device (threads racing on the first call are serialised), with that
// device current. In host code the array's name is only a handle; the address
// a kernel can use comes from cudaGetSymbolAddress.
int noalloc_setup(int device, NoAllocDevice **out) {
  if (device < 0 || device >= kNaMaxDevices)
    return fail(EMM_ERR_BAD_ARG, "gather_noalloc: device %d outside [0, %d)", device, kNaMaxDevices);
  NoAllocDevice &d = g_noalloc_dev[device];
  std::call_once(d.once, [&d, device] {
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess)
      e = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (e != cudaSuccess) {
      d.setup_rc = EMM_ERR_CUDA;
      d.setup_error = std::string("gather_noalloc: set-up on device failed: ") + cudaGetErrorString(e);
      return;
    }
    d.scratch = static_cast<unsigned char *>(ptr);
  });
  if (d.setup_rc != EMM_OK) return fail(d.setup_rc, "%s", d.setup_error.c_str());
  *out = &d;
  return EMM_OK;
}

}  // namespace

extern "C" {

int emm_gather_noalloc(int device, const emm_pool_desc *desc, const void *const *h_layer_ptrs,
                       const int64_t *h_ids, int32_t n, void *d_packed, uint64_t packed_bytes,
                       void *stream) {
  if (!desc || !h_layer_ptrs) return fail(EMM_ERR_BAD_ARG, "gather_noalloc: null descriptor or layer array");
  bool dense = false;
  if (int rc = check_desc(*desc, &dense)) return rc;
  if (!dense) return fail(EMM_ERR_BAD_ARG, "gather_noalloc: pool pages are not dense");
  if (desc->num_layers > EMM_NOALLOC_MAX_LAYERS)
    return fail(EMM_ERR_TOO_LARGE, "gather_noalloc: %d layers exceed the fixed maximum of %d",
                desc->num_layers, EMM_NOALLOC_MAX_LAYERS);
  if (n < 0) return fail(EMM_ERR_BAD_ARG, "gather_noalloc: negative block count");
  if (n > EMM_NOALLOC_MAX_IDS)
    return fail(EMM_ERR_TOO_LARGE, "gather_noalloc: %d block ids exceed the fixed maximum of %d", n,
                EMM_NOALLOC_MAX_IDS);
  const int64_t page = (int64_t)desc->block_size * desc->num_kv_heads * desc->head_size * desc->elem_size;
  const int planes = desc->num_planes == 1 ? 1 : 2;
  const uint64_t want = (uint64_t)desc->num_layers * (uint64_t)planes * (uint64_t)n * (uint64_t)page;
  if (packed_bytes != want)
    return fail(EMM_ERR_LENGTH, "gather_noalloc: packed buffer holds %llu bytes, %d blocks need %llu",
                (unsigned long long)packed_bytes, n, (unsigned long long)want);
  if (n == 0) return EMM_OK;
  if (!h_ids || !d_packed) return fail(EMM_ERR_BAD_ARG, "gather_noalloc: null pointer");
  if (int rc = check_ids_host(h_ids, n, desc->num_blocks, "gather_noalloc")) return rc;

  DeviceGuard guard(device);
  if (!guard.ok()) return fail(EMM_ERR_CUDA, "cannot select device %d", device);
  NoAllocDevice *nd = nullptr;
  if (int rc = noalloc_setup(device, &nd)) return rc;
  // The table and the layer addresses are read from host memory at call time;
  // a capturing stream would record the copies, not perform them, and a later
  // replay would read host memory that no longer holds them.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  EMM_CUDA(cudaStreamIsCapturing((cudaStream_t)stream, &capturing));
  if (capturing != cudaStreamCaptureStatusNone)
    return fail(EMM_ERR_BAD_ARG, "gather_noalloc: the stream is capturing; this entry uploads its table at call time");

  uint32_t align = pow2_align((uint64_t)desc->block_stride);
  if (planes == 2) align = std::min(align, pow2_align((uint64_t)desc->plane_stride));
  align = std::min(align, std::min(pow2_align((uint64_t)page), pow2_align((uint64_t)d_packed)));
  uint64_t layer_addr[EMM_NOALLOC_MAX_LAYERS];
  for (int l = 0; l < desc->num_layers; ++l) {
    if (!h_layer_ptrs[l]) return fail(EMM_ERR_BAD_ARG, "gather_noalloc: layer %d base pointer is null", l);
    layer_addr[l] = (uint64_t)h_layer_ptrs[l];
    align = std::min(align, pow2_align(layer_addr[l]));
  }
  if (align < (uint32_t)desc->elem_size) return fail(EMM_ERR_ALIGN, "gather_noalloc: pointers not aligned to elem_size");
  int32_t ids32[EMM_NOALLOC_MAX_IDS];
  for (int32_t i = 0; i < n; ++i) ids32[i] = (int32_t)h_ids[i];

  cudaStream_t st = (cudaStream_t)stream;
  unsigned char *d_status = nd->scratch;
  unsigned char *d_layers = nd->scratch + kNaStatusBytes;
  unsigned char *d_ids = d_layers + kNaLayersBytes;
  // The array keeps the previous call's contents: the status word must start
  // at zero; the layer array and the table are overwritten up to what is read.
  EMM_CUDA(cudaMemsetAsync(d_status, 0, 16, st));
  // Pageable sources: the runtime has copied them out before these calls return,
  // which it can only do once earlier work on `st` has finished (the host waits for it).
  EMM_CUDA(cudaMemcpyAsync(d_layers, layer_addr, sizeof(uint64_t) * desc->num_layers, cudaMemcpyHostToDevice, st));
  EMM_CUDA(cudaMemcpyAsync(d_ids, ids32, sizeof(int32_t) * n, cudaMemcpyHostToDevice, st));

  PageCopyArgs a;
  a.src.layers = reinterpret_cast<const uint64_t *>(d_layers);
  a.src.base = 0;
  a.src.layer_stride = 0;
  a.src.plane_stride = (uint64_t)desc->plane_stride;
  a.src.block_stride = (uint64_t)desc->block_stride;
  a.src.ids = reinterpret_cast<const int32_t *>(d_ids);
  a.src.num_blocks = (uint32_t)desc->num_blocks;
  a.src.seg_prefix = nullptr;
  a.src.num_segs = 0;
  a.src.seg_stride = 0;
  a.dst = packed_side(d_packed, n, page, planes);
  a.n = (uint32_t)n;
  a.plane_shift = planes == 2 ? 1u : 0u;
  a.layer_begin = 0;
  a.layer_count = (uint32_t)desc->num_layers;
  a.page_bytes = (uint32_t)page;
  a.status = reinterpret_cast<int *>(d_status);
  a.wait_limit_ns = emm::kDefaultWaitLimitNs;
  a.tx_overcount = 0;
  a.inline_count = 0;
  a.src_inline = a.dst_inline = 0;

  if (align >= 16) {
    int64_t chunk = std::min<int64_t>(32768, page);
    const int stages = 2;
    int lanes = (int)(1 + (32 * 1024 + chunk / 2) / chunk);
    lanes = std::max(1, std::min(lanes, 16));
    const int warps = std::min(lanes, emm::kMaxWarps);
    const int per_sm = (lanes + warps - 1) / warps;
    a.chunk_bytes = (uint32_t)chunk;
    a.chunks_per_page = (uint32_t)((page + chunk - 1) / chunk);
    a.total_chunks = (uint64_t)desc->num_layers * (uint64_t)planes * (uint64_t)n * a.chunks_per_page;
    const int smem = (int)(warps * stages * chunk);
    if (smem > nd->max_smem_optin - 2048)
      return fail(EMM_ERR_BAD_ARG, "gather_noalloc: ring does not fit shared memory");
    if (int rc = ensure_bulk_smem(device, smem)) return rc;
    const uint64_t want_ctas = (a.total_chunks + warps - 1) / warps;
    const int grid = (int)std::min<uint64_t>(want_ctas, (uint64_t)nd->sm_count * per_sm);
    emm::page_copy_bulk<false><<<grid, warps * 32, smem, st>>>(a, (uint32_t)stages, 0u);
  } else {
    int64_t chunk = std::min<int64_t>(65536, page);
    a.chunk_bytes = (uint32_t)chunk;
    a.chunks_per_page = (uint32_t)((page + chunk - 1) / chunk);
    a.total_chunks = (uint64_t)desc->num_layers * (uint64_t)planes * (uint64_t)n * a.chunks_per_page;
    const int grid = (int)std::min<uint64_t>(a.total_chunks, (uint64_t)nd->sm_count * 4);
    if (align >= 8) emm::page_copy_ldg<uint2, 2, false><<<grid, 256, 0, st>>>(a);
    else if (align >= 4) emm::page_copy_ldg<uint32_t, 2, false><<<grid, 256, 0, st>>>(a);
    else if (align >= 2) emm::page_copy_ldg<uint16_t, 2, false><<<grid, 256, 0, st>>>(a);
    else emm::page_copy_ldg<uint8_t, 2, false><<<grid, 256, 0, st>>>(a);
  }
  EMM_CUDA(cudaGetLastError());
  return EMM_OK;
}

}  // extern "C"
