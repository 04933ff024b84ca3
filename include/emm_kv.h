/*
 * emm_kv.h -- C ABI of the paged KV-cache movement library (sm_100a).
 *
 * One shared library, plain C types only. Every data entry point takes raw
 * device pointers, element counts and a CUDA stream (passed as void*, it is a
 * cudaStream_t). Launches are asynchronous and stream ordered; nothing here
 * synchronises the device except emm_ctx_status() and the *_create/_destroy
 * calls. Errors are returned as int status codes (0 = ok), never thrown; the
 * text of the last failure on the calling thread is kept for
 * emm_last_error(). This mirrors the reference's convention of returning
 * {"error": ..., "bytes": 0} from its data path instead of raising
 * (elasticmm/engine/v0/worker.py:686-691,726-731,860-871).
 *
 * The reference has no FFI for this path: its data plane is a set of Python
 * methods on the V0Worker actor built from torch indexing kernels. Each entry
 * below names the reference method whose device work it replaces.
 *
 * Pool layout. A pool is L per-layer allocations. Inside a layer:
 *   address(plane p, block b, token t, head h) =
 *       layer_ptr[l] + p*plane_stride + b*block_stride + t*token_stride + h*head_stride
 * with head_size*elem_size contiguous bytes at that address. The reference
 * layout is a list of L tensors [2, NB, BS, H, D]
 * (elasticmm/engine/v0/worker.py:388-394,593-594): plane_stride = NB*page,
 * block_stride = page, token_stride = H*D*e, head_stride = D*e, where
 * page = BS*H*D*e. Whole-block operations need the BS*H*D*e bytes of one
 * block of one plane to be one dense run ("page"); both the reference order
 * (token-major) and the head-major order satisfy that.
 *
 * Packed transfer buffer: [L, 2, n, page] contiguous, the byte image of the
 * tensor [L, 2, n, BS, H, D] that extract_kv_blocks returns
 * (elasticmm/engine/v0/worker.py:578-610).
 */
#ifndef EMM_KV_H
#define EMM_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EMM_KV_ABI_VERSION 1

typedef struct emm_ctx emm_ctx;   /* one per process and device; not thread safe */
typedef struct emm_pool emm_pool; /* geometry + per-layer base pointers of one pool */
typedef struct emm_append_binding emm_append_binding; /* a validated per-layer append over static buffers */

enum emm_status {
  EMM_OK = 0,
  EMM_ERR_BAD_ARG = 1,    /* null pointer, negative count, unsupported geometry */
  EMM_ERR_ID_RANGE = 2,   /* a block id or slot outside the pool */
  EMM_ERR_LENGTH = 3,     /* buffer size / block count mismatch */
  EMM_ERR_CUDA = 4,       /* a CUDA runtime call failed; text in emm_last_error */
  EMM_ERR_TIMEOUT = 5,    /* a bounded device-side wait ran out */
  EMM_ERR_ALIGN = 6,      /* pointer or stride alignment below element size */
  EMM_ERR_DUPLICATE = 7,  /* duplicate destination ids (write order undefined) */
  EMM_ERR_OVERLAP = 8,    /* source and destination id sets overlap in one pool */
  EMM_ERR_TOO_LARGE = 9,  /* request exceeds a fixed capacity */
  EMM_ERR_NOMEM = 10,     /* host or device allocation failed */
  EMM_ERR_NCCL = 11       /* the NCCL library is missing or one of its calls failed */
};

typedef struct emm_pool_desc {
  int32_t num_layers;   /* L */
  int32_t num_blocks;   /* NB, blocks per layer and plane */
  int32_t block_size;   /* BS, tokens per block */
  int32_t num_kv_heads; /* H */
  int32_t head_size;    /* D */
  int32_t elem_size;    /* bytes per element: 2 for fp16/bf16, 1 for fp8, 4 for fp32 */
  int64_t plane_stride; /* bytes from the K plane to the V plane of a layer */
  int64_t block_stride; /* bytes between consecutive blocks of a plane */
  int64_t token_stride; /* bytes between consecutive tokens of a block */
  int64_t head_stride;  /* bytes between consecutive heads of a token */
  int32_t num_planes;   /* 2 for a KV pool (K plane, V plane); 1 for a single-plane block pool; 0 means 2 */
  int32_t reserved;     /* must be 0 */
} emm_pool_desc;

/* Copy-kernel families, for emm_ctx_set_option(ctx, EMM_OPT_COPY_VARIANT, v). */
enum emm_copy_variant {
  EMM_COPY_AUTO = 0, /* library default */
  EMM_COPY_BULK = 1, /* cp.async.bulk global->shared->global ring, one issuing lane per warp */
  EMM_COPY_LDG = 2   /* 16-byte vector loads/stores through registers */
};

enum emm_option {
  EMM_OPT_COPY_VARIANT = 0,  /* enum emm_copy_variant */
  EMM_OPT_CHUNK_BYTES = 1,   /* bytes per work item of the copy kernels (multiple of 16) */
  EMM_OPT_STAGES = 2,        /* shared-memory ring depth per warp, bulk variant (2..8) */
  EMM_OPT_WARPS = 3,         /* issuing warps per CTA, bulk variant (1..8; 0 = sized from the chunk) */
  EMM_OPT_CTAS_PER_SM = 4,   /* resident CTAs per SM the grid is sized for */
  EMM_OPT_LDG_UNROLL = 5,    /* 16-byte loads in flight per thread, LDG variant (1,2,4,8) */
  EMM_OPT_MAX_CTAS = 6,      /* cap on the grid (0 = none) */
  EMM_OPT_REMOTE_VARIANT = 7, /* family used when a side is a peer GPU's or pinned host memory (default LDG) */
  EMM_OPT_L2_HINT = 8,        /* bulk variant: bit 0 loads, bit 1 stores carry an L2 evict-first hint (default 0) */
  EMM_OPT_PDL = 10,                /* bulk variant: launch with programmatic stream serialisation, so that a copy
                                      sets up while the previous copy in the stream drains (default 1) */
  EMM_OPT_WAIT_LIMIT_NS = 9   /* bulk variant: longest one device-side wait for a load may last, in ns
                                 (default 2 s, range 1 us .. 60 s); when it runs out the kernel records
                                 EMM_ERR_TIMEOUT in the status word, drains and returns */
};

/* ---- library ---------------------------------------------------------- */

int emm_abi_version(void);
const char *emm_status_string(int status);
/* Text of the most recent failure on this thread ("" if none). */
const char *emm_last_error(void);

/* ---- context ---------------------------------------------------------- */

/* Binds to `device`, creates the device status word and the id staging ring.
 * Replaces nothing in the reference (it keeps no native state). */
int emm_ctx_create(int device, emm_ctx **out);
int emm_ctx_destroy(emm_ctx *ctx);
int emm_ctx_set_option(emm_ctx *ctx, int option, int64_t value);
int emm_ctx_get_option(emm_ctx *ctx, int option, int64_t *value);
/* Number of kernels this context has launched so far. */
int64_t emm_ctx_launch_count(emm_ctx *ctx);
/* Waits for `stream`, then returns and clears the sticky device-side status
 * (EMM_OK, EMM_ERR_ID_RANGE, EMM_ERR_TIMEOUT). The kernels never trap: a bad
 * id is recorded here and the page is skipped. `detail` (may be NULL)
 * receives the offending id or slot. */
int emm_ctx_status(emm_ctx *ctx, void *stream, int64_t *detail);

/* ---- pools ------------------------------------------------------------ */

/* Fills `desc` with the reference layout [2, NB, BS, H, D] per layer
 * (elasticmm/engine/v0/worker.py:593-594). */
int emm_pool_desc_nhd(emm_pool_desc *desc, int L, int NB, int BS, int H, int D, int elem_size);
/* Same geometry with heads before tokens inside a block: [2, NB, H, BS, D]. */
int emm_pool_desc_hnd(emm_pool_desc *desc, int L, int NB, int BS, int H, int D, int elem_size);

/* Single-plane block pool [NB, rows, cols] per layer, e.g. the vision-embedding
 * block cache [blocks, embed_tokens, embed_dim] that
 * V0NCCLTransferManager.transfer_vision_embeddings gathers and scatters
 * (elasticmm/engine/v0/nccl_transfer.py:295-368). A block is one page of
 * rows*cols*elem_size bytes; the packed buffer is [L, 1, n, page]. Gather,
 * scatter and block copy apply; append does not. */
int emm_pool_desc_blocks(emm_pool_desc *desc, int L, int NB, int rows, int cols, int elem_size);

/* `layer_ptrs` is a HOST array of L device (or device-visible) base
 * addresses; the library keeps a device copy. A single 6-D tensor
 * [L, 2, NB, BS, H, D] (elasticmm/engine/v0/nccl_transfer.py:215,241-244) is
 * passed as L pointers base + l*layer_bytes. The memory stays owned by the
 * caller. Also the source of get_kv_cache_layout
 * (elasticmm/engine/v0/worker.py:635-647). */
int emm_pool_create(emm_ctx *ctx, const emm_pool_desc *desc, const void *const *layer_ptrs,
                    emm_pool **out);
/* Frees the library's part of a pool (its device copy of the layer pointers). A pool may be
 * destroyed after its context, but must not be used for a launch after it. */
int emm_pool_destroy(emm_pool *pool);
int emm_pool_get_desc(const emm_pool *pool, emm_pool_desc *desc);
/* Bytes of one block of one plane of one layer (BS*H*D*elem_size). */
int64_t emm_pool_page_bytes(const emm_pool *pool);

/* ---- whole-block movement --------------------------------------------- */

/* Gather: packed[l][p][i] = pool[l][p][ids[i]] for all layers and both
 * planes, one launch. `d_ids` is a DEVICE int32 array of n block ids.
 * `packed_bytes` must equal L*planes*n*page (planes = 2 for a KV pool).
 * Replaces the L index launches plus
 * torch.stack of V0Worker.extract_kv_blocks
 * (elasticmm/engine/v0/worker.py:578-610) and the gather half of p2p_send_kv
 * (:676-678) and of V0NCCLTransferManager.transfer_kv_cache_blocks
 * (elasticmm/engine/v0/nccl_transfer.py:241-247). */
int emm_gather(emm_pool *pool, const int32_t *d_ids, int32_t n, void *d_packed,
               uint64_t packed_bytes, void *stream);

/* Scatter: pool[l][p][ids[i]] = packed[l][p][i]. Duplicate ids give an
 * undefined winner, as in the reference. Replaces the L index_put launches of
 * V0Worker.write_kv_blocks (elasticmm/engine/v0/worker.py:612-633), the
 * scatter half of p2p_recv_kv / p2p_coordinated_transfer_kv (:721,819) and
 * the per-block loop at elasticmm/engine/v0/nccl_transfer.py:288-289. */
int emm_scatter(emm_pool *pool, const int32_t *d_ids, int32_t n, const void *d_packed,
                uint64_t packed_bytes, void *stream);

/* Same two operations on a layer range [layer_begin, layer_begin+layer_count):
 * the packed pointer addresses that range only ([layer_count, 2, n, page]).
 * This is the per-layer message of the reference's pipelined send/recv
 * (elasticmm/engine/v0/worker.py:676-682,804-820). */
int emm_gather_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count,
                      const int32_t *d_ids, int32_t n, void *d_packed, uint64_t packed_bytes,
                      void *stream);
int emm_scatter_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count,
                       const int32_t *d_ids, int32_t n, const void *d_packed,
                       uint64_t packed_bytes, void *stream);

/* Several requests in one launch, each with its own packed buffer. `d_ids`
 * holds the requests' tables one after the other (n_total ids),
 * `d_seg_prefix` is a DEVICE array of num_segs + 1 prefix sums of their block
 * counts (first entry 0, last n_total). Request r's buffer [L, 2, n_r, page]
 * starts L*2*page*seg_prefix[r] bytes into `d_packed`, so the buffers lie end
 * to end and `packed_bytes` is L*2*n_total*page. One launch instead of one per
 * request is what the reference's batching branch aims at when it merges the
 * transfers of a worker pair (elasticmm/engine/v0/kv_transfer.py:342-418),
 * here without giving up one contiguous tensor per request. */
int emm_gather_many(emm_pool *pool, const int32_t *d_ids, const uint32_t *d_seg_prefix, int32_t num_segs,
                    int32_t n_total, void *d_packed, uint64_t packed_bytes, void *stream);
int emm_scatter_many(emm_pool *pool, const int32_t *d_ids, const uint32_t *d_seg_prefix, int32_t num_segs,
                     int32_t n_total, const void *d_packed, uint64_t packed_bytes, void *stream);

/* The same on a layer range: segment r holds [layer_count, planes, n_r, page]
 * and starts layer_count*planes*page*seg_prefix[r] bytes into `d_packed`
 * (`packed_bytes` = layer_count*planes*n_total*page). With one segment per
 * peer this is the packed side of a rebalancing exchange: a source packs a
 * chunk of layers as [sink][layer][plane][n_sink][page], so that each sink's
 * share is ONE contiguous message, and a sink unpacks [source][layer][plane]
 * [n_source][page] the same way. The reference sends one message per layer
 * (elasticmm/engine/v0/worker.py:676-682). */
int emm_gather_many_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count, const int32_t *d_ids,
                           const uint32_t *d_seg_prefix, int32_t num_segs, int32_t n_total, void *d_packed,
                           uint64_t packed_bytes, void *stream);
int emm_scatter_many_layers(emm_pool *pool, int32_t layer_begin, int32_t layer_count, const int32_t *d_ids,
                            const uint32_t *d_seg_prefix, int32_t num_segs, int32_t n_total,
                            const void *d_packed, uint64_t packed_bytes, void *stream);

/* Block copy: dst[l][p][dst_ids[i]] = src[l][p][src_ids[i]] with no staging
 * buffer. src and dst may be the same pool (compaction; id sets must not
 * overlap), two pools on one GPU, a pool in pinned host memory (swap), or a
 * peer GPU's pool mapped into this process (migration by direct store). Both
 * pools must have equal page size and layer count. Replaces the per-block
 * copy loop of V0Worker.swap_blocks (elasticmm/engine/v0/worker.py:520-526)
 * and extract_kv_blocks followed by write_kv_blocks. */
int emm_copy_blocks(emm_pool *src, emm_pool *dst, const int32_t *d_src_ids,
                    const int32_t *d_dst_ids, int32_t n, void *stream);

/* Host-id forms: `h_ids` are HOST int64 arrays (the reference passes Python
 * lists and uploads them with a synchronous torch.tensor(..., device=...),
 * elasticmm/engine/v0/worker.py:597,628). The ids are range checked (and,
 * for destinations, checked for duplicates) on the host. A list of up to 128
 * ids travels inside the kernel arguments (no copy precedes the launch); a
 * longer one is staged through a pinned ring and uploaded on `stream` without
 * a device synchronisation. */
int emm_gather_h(emm_pool *pool, const int64_t *h_ids, int32_t n, void *d_packed,
                 uint64_t packed_bytes, void *stream);
int emm_scatter_h(emm_pool *pool, const int64_t *h_ids, int32_t n, const void *d_packed,
                  uint64_t packed_bytes, void *stream);
int emm_copy_blocks_h(emm_pool *src, emm_pool *dst, const int64_t *h_src_ids,
                      const int64_t *h_dst_ids, int32_t n, void *stream);

/* Uploads a HOST int64 list as int32 into caller-owned device memory `d_out`
 * (n entries) through the context's pinned staging ring, stream ordered, with
 * no allocation in steady state and no device synchronisation. For tables a
 * caller keeps on the device across calls (the device-table entries above and
 * the seg_prefix arrays); values must lie in [0, 2^31). The reference uploads
 * its id lists with a synchronous torch.tensor(..., device=...)
 * (elasticmm/engine/v0/worker.py:597,628). */
int emm_upload_ids(emm_ctx *ctx, const int64_t *h_values, int32_t n, int32_t *d_out, void *stream);

/* Gather for callers that must not allocate device memory. No counterpart in
 * the reference. Some hosts cannot afford a cudaMalloc on this path: a serving
 * process that has already handed nearly all HBM to its own caching allocator
 * (a raw allocation may fail or fragment it), or a latency-critical section
 * where the implicit device synchronisation of cudaMalloc / cudaFree is not
 * acceptable. This entry needs no emm_ctx and no emm_pool (both allocate): the
 * pool is described by `desc` plus a HOST array of `desc->num_layers` layer
 * base addresses, the ids are a HOST int64 list, and the device copies of both
 * live in a fixed array inside the library image (about 66 KiB of device
 * memory on every GPU that loads the library, held until the process exits).
 * Limits: n <= EMM_NOALLOC_MAX_IDS, num_layers <= EMM_NOALLOC_MAX_LAYERS;
 * larger requests return EMM_ERR_TOO_LARGE. Ids are range checked on the host.
 * The result equals emm_gather_h. The first call on a device looks up the
 * array's device address and the device's limits; make that first call before
 * any stream capture begins. All calls share the one array: two calls whose
 * kernels may overlap on the GPU (different streams, no ordering) race on it;
 * calls on one stream are safe. Nothing in this call invokes cudaMalloc,
 * cudaFree or any allocating library routine. The table and the layer
 * addresses are uploaded from ordinary (pageable) host memory, so the call
 * waits on the host until earlier work on `stream` has finished before it
 * returns; what it saves is the allocation, not that wait. A stream that is
 * being captured is refused with EMM_ERR_BAD_ARG, because the upload happens at
 * call time. Ids are checked on the host, so the kernel has no bad id to
 * report; a device-side wait that runs out is not reported through this entry
 * (it has no context whose status word could be read). */
#define EMM_NOALLOC_MAX_IDS 16384
#define EMM_NOALLOC_MAX_LAYERS 256
int emm_gather_noalloc(int device, const emm_pool_desc *desc, const void *const *h_layer_ptrs,
                       const int64_t *h_ids, int32_t n, void *d_packed, uint64_t packed_bytes,
                       void *stream);

/* Test hook, not for production use: emm_gather with `extra_tx_bytes` added to
 * the byte count every load is expected to deliver, so that no device-side
 * wait of the bulk-copy kernel can complete. Each lane gives up after the
 * context's EMM_OPT_WAIT_LIMIT_NS, records EMM_ERR_TIMEOUT in the status word
 * and returns; every load it issued has long landed by then, so nothing is in
 * flight when the kernel ends, the packed buffer is left partly written and
 * the context stays usable. It lets a test run the time-out path without a
 * fault, a trap or an unbounded wait. No counterpart in the reference (its
 * time-out is the host-side poll at elasticmm/engine/v0/worker.py:806-812). */
int emm_test_gather_expect_overcount(emm_pool *pool, const int32_t *d_ids, int32_t n, void *d_packed,
                                     uint64_t packed_bytes, uint32_t extra_tx_bytes, void *stream);

/* ---- per-token append -------------------------------------------------- */

/* reshape_and_cache for one layer: for each token t with s = slot_mapping[t],
 * s < 0 is skipped, otherwise K[s / BS][s % BS][:, :] = key[t] and the same
 * for V. key/value are [T, H, D] with the given token stride in bytes (heads
 * contiguous: head stride D*elem_size). `d_slot_mapping` is a DEVICE int64
 * array. In the reference this is vLLM's cache op reached under
 * model_runner.execute_model (elasticmm/engine/v0/worker_steps.py:281,438);
 * the slot mapping derives from the reference's block tables (:219,411). */
int emm_append(emm_pool *pool, int32_t layer, const void *d_key, const void *d_value,
               int64_t key_token_stride, int64_t value_token_stride,
               const int64_t *d_slot_mapping, int32_t num_tokens, void *stream);

/* All layers of one decode step in one launch: key/value are [L, T, H, D]
 * with the given layer and token strides in bytes; one slot mapping is
 * shared by all layers (every layer of a request uses the same block table,
 * elasticmm/engine/v0/worker_steps.py:406-420). */
int emm_append_all_layers(emm_pool *pool, const void *d_key, const void *d_value,
                          int64_t key_layer_stride, int64_t key_token_stride,
                          int64_t value_layer_stride, int64_t value_token_stride,
                          const int64_t *d_slot_mapping, int32_t num_tokens, void *stream);

/* The per-layer call for a decode loop that refills the SAME key / value /
 * slot-mapping buffers every step (the shape of a graph-captured or
 * static-buffer model runner): emm_append_bind validates the buffers once
 * ([L, T, H, D] key and value with the given strides in bytes, one [T] int64
 * slot mapping) and emm_append_bound(binding, layer, stream) then costs one
 * short foreign call plus the launch. Same kernel and same result as
 * emm_append(pool, layer, key + layer*key_layer_stride, ...). The binding
 * keeps pointers only: the buffers and the pool must outlive it. The
 * reference reaches vLLM's op once per layer in the same way
 * (elasticmm/engine/v0/worker_steps.py:281,438). */
int emm_append_bind(emm_pool *pool, const void *d_key, const void *d_value, int64_t key_layer_stride,
                    int64_t key_token_stride, int64_t value_layer_stride, int64_t value_token_stride,
                    const int64_t *d_slot_mapping, int32_t num_tokens, emm_append_binding **out);
int emm_append_bound(emm_append_binding *binding, int32_t layer, void *stream);
int emm_append_unbind(emm_append_binding *binding);

/* ---- compaction planning (host only) ---------------------------------- */

/* Minimal-move defragmentation plan. `table_ids` holds the concatenated
 * block tables of the live requests, `n_ids` entries in total, each id in
 * [0, num_blocks) and unique. After the plan every live block has an id in
 * [0, n_ids): live blocks whose id is already < n_ids stay; the others move,
 * in table order, into the free ids < n_ids in ascending order (so source
 * and destination sets are disjoint). Outputs: `new_table_ids[n_ids]` (the
 * rewritten tables), `move_src` / `move_dst` (capacity n_ids each) and
 * `*n_moves`. The reference has no compaction; its free list only ever
 * appends freed ids (elasticmm/engine/v0/block_manager.py:247-256), which is
 * what fragments the tables. */
int emm_compact_plan(const int64_t *table_ids, int64_t n_ids, int64_t num_blocks,
                     int64_t *new_table_ids, int64_t *move_src, int64_t *move_dst,
                     int64_t *n_moves);

/* ---- staged transport over NCCL (multi-GPU, one process per GPU) ------- */

/* The NCCL entry points are resolved at run time from the libnccl.so.2 the
 * process already has loaded (or can load); the library does not link NCCL.
 * `comm` below is an ncclComm_t passed as void*: one made by
 * emm_nccl_comm_init, or any communicator the host application owns. */
#define EMM_NCCL_UNIQUE_ID_BYTES 128
/* Rank 0 creates the id and ships it to the other ranks by any host channel;
 * the reference rendezvous is tcp://127.0.0.1:29600
 * (elasticmm/engine/v0/nccl_coordinator.py:179-186, worker.py:225-230). */
int emm_nccl_unique_id(unsigned char id[EMM_NCCL_UNIQUE_ID_BYTES]);
/* Collective over all `nranks` ranks (ncclCommInitRank) with ctx's device current. */
int emm_nccl_comm_init(emm_ctx *ctx, const unsigned char id[EMM_NCCL_UNIQUE_ID_BYTES], int nranks,
                       int rank, void **comm);
int emm_nccl_comm_destroy(void *comm);

/* Stream-ordered send / receive of a packed buffer (bytes). Replace the
 * per-layer torch.distributed.send / recv of p2p_send_kv / p2p_recv_kv
 * (elasticmm/engine/v0/worker.py:681,718,816). */
int emm_send_packed(void *comm, const void *d_buf, uint64_t bytes, int peer, void *stream);
int emm_recv_packed(void *comm, void *d_buf, uint64_t bytes, int peer, void *stream);
/* One grouped exchange (ncclGroupStart .. ncclGroupEnd): operation k sends
 * (is_send[k] != 0) or receives bytes[k] bytes at bufs[k] to / from peers[k].
 * This is the all-to-all-v step of a rebalancing round; the reference has no
 * collective of this kind. */
int emm_exchange(void *comm, int32_t n_ops, const int32_t *is_send, void *const *bufs,
                 const uint64_t *bytes, const int32_t *peers, void *stream);

/* Whole pipelines, ordered after `stream` on entry and joined back into it on
 * return (asynchronous to the host): the L layers move in messages of
 * `layers_per_msg` layers through the two halves of `d_staging`
 * (`staging_bytes` >= 2 * layers_per_msg * 2 * n * page); packing message c+1
 * overlaps sending message c, receiving c+1 overlaps unpacking c. Both ends
 * must pass the same n and layers_per_msg. These are p2p_send_kv and
 * p2p_recv_kv (elasticmm/engine/v0/worker.py:665-731) without the per-layer
 * serialisation. */
int emm_send_blocks(emm_pool *pool, void *comm, int peer, const int32_t *d_ids, int32_t n,
                    void *d_staging, uint64_t staging_bytes, int32_t layers_per_msg, void *stream);
int emm_recv_blocks(emm_pool *pool, void *comm, int peer, const int32_t *d_ids, int32_t n,
                    void *d_staging, uint64_t staging_bytes, int32_t layers_per_msg, void *stream);

/* ---- peer mapping (multi-GPU, one process per GPU) --------------------- */

#define EMM_IPC_HANDLE_BYTES 64

/* Exports the allocation containing `d_ptr` for another process on the same
 * node: `handle` names the allocation, `*offset` is d_ptr's distance from
 * its base. The reference only sketches this (register_ipc_handle,
 * elasticmm/engine/v0/kv_transfer.py:89-111; get_ipc_handles returns [],
 * elasticmm/engine/v0/worker.py:415-437). */
int emm_ipc_export(emm_ctx *ctx, const void *d_ptr, unsigned char handle[EMM_IPC_HANDLE_BYTES],
                   uint64_t *offset);
/* Maps a peer allocation and returns the peer address of the exported
 * pointer. A handle is opened once per process and cached; emm_ctx_destroy
 * closes the mappings. */
int emm_ipc_open(emm_ctx *ctx, const unsigned char handle[EMM_IPC_HANDLE_BYTES], uint64_t offset,
                 void **d_ptr);

/* One process driving several GPUs: lets kernels of ctx's device address memory
 * of `peer_device` directly (cudaDeviceEnablePeerAccess; already-enabled is not
 * an error). A pool of the other GPU is then described to this context with
 * emm_pool_create over the same device pointers; no IPC handle is involved. */
int emm_enable_peer_access(emm_ctx *ctx, int peer_device);

#ifdef __cplusplus
}
#endif
#endif /* EMM_KV_H */
