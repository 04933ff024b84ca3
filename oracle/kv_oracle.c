/*
 * kv_oracle.c -- plain C restatement of the KV movement path on host memory.
 * TEST INFRASTRUCTURE ONLY: a checker and a timed CPU baseline, never linked
 * into or called by the product library.
 *
 * Each function restates the byte movement of a reference function for the
 * reference pool layout (L per-layer tensors [2, NB, BS, H, D], a "page" being
 * the BS*H*D*e contiguous bytes of one block of one plane):
 *   kvo_gather        V0Worker.extract_kv_blocks  elasticmm/engine/v0/worker.py:578-610
 *   kvo_scatter       V0Worker.write_kv_blocks    elasticmm/engine/v0/worker.py:612-633
 *   kvo_copy_blocks   gather followed by scatter; per-block copy of V0Worker.swap_blocks
 *                                                 elasticmm/engine/v0/worker.py:520-526
 *   kvo_append        the cache op under execute_model (vLLM; checked against a fixture its op produced)
 *                                                 elasticmm/engine/v0/worker_steps.py:281,438
 *   kvo_compact_plan  no reference counterpart; the free list it repairs is
 *                                                 elasticmm/engine/v0/block_manager.py:247-256
 * Pages are independent, so the work is split over `threads` POSIX threads.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  uint8_t *const *src_layers; /* L base pointers, or NULL: src is packed */
  uint8_t *const *dst_layers; /* L base pointers, or NULL: dst is packed */
  uint8_t *packed;
  int64_t src_plane, src_block, dst_plane, dst_block, page;
  const int64_t *src_ids; /* NULL = identity */
  const int64_t *dst_ids; /* NULL = identity */
  int64_t L, n;
  int64_t begin, end; /* page range of this thread */
} job_t;

static void *run_pages(void *arg) {
  job_t *j = (job_t *)arg;
  for (int64_t g = j->begin; g < j->end; ++g) {
    int64_t i = g % j->n, t = g / j->n, p = t & 1, l = t >> 1;
    int64_t sid = j->src_ids ? j->src_ids[i] : i;
    int64_t did = j->dst_ids ? j->dst_ids[i] : i;
    const uint8_t *s = j->src_layers
                           ? j->src_layers[l] + p * j->src_plane + sid * j->src_block
                           : j->packed + ((l * 2 + p) * j->n + i) * j->page;
    uint8_t *d = j->dst_layers ? j->dst_layers[l] + p * j->dst_plane + did * j->dst_block
                               : j->packed + ((l * 2 + p) * j->n + i) * j->page;
    memcpy(d, s, (size_t)j->page);
  }
  return NULL;
}

static void run(job_t proto, int threads) {
  int64_t total = proto.L * 2 * proto.n;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  if (total < threads) threads = total > 0 ? (int)total : 1;
  pthread_t tid[256];
  job_t jobs[256];
  for (int k = 0; k < threads; ++k) {
    jobs[k] = proto;
    jobs[k].begin = total * k / threads;
    jobs[k].end = total * (k + 1) / threads;
    if (k > 0) pthread_create(&tid[k], NULL, run_pages, &jobs[k]);
  }
  run_pages(&jobs[0]);
  for (int k = 1; k < threads; ++k) pthread_join(tid[k], NULL);
}

void kvo_gather(uint8_t *const *layers, int64_t L, int64_t plane_stride, int64_t block_stride,
                int64_t page, const int64_t *ids, int64_t n, uint8_t *packed, int threads) {
  job_t j = {layers, NULL, packed, plane_stride, block_stride, 0, 0, page, ids, NULL, L, n, 0, 0};
  run(j, threads);
}

void kvo_scatter(uint8_t *const *layers, int64_t L, int64_t plane_stride, int64_t block_stride,
                 int64_t page, const int64_t *ids, int64_t n, uint8_t *packed, int threads) {
  job_t j = {NULL, layers, packed, 0, 0, plane_stride, block_stride, page, NULL, ids, L, n, 0, 0};
  run(j, threads);
}

void kvo_copy_blocks(uint8_t *const *src_layers, uint8_t *const *dst_layers, int64_t L,
                     int64_t src_plane, int64_t src_block, int64_t dst_plane, int64_t dst_block,
                     int64_t page, const int64_t *src_ids, const int64_t *dst_ids, int64_t n,
                     int threads) {
  job_t j = {src_layers, dst_layers, NULL, src_plane, src_block, dst_plane, dst_block,
             page,       src_ids,    dst_ids, L,       n,         0,         0};
  run(j, threads);
}

/* One layer: key/value [T, H, D] rows of row_bytes with the given token
 * strides; slot < 0 skipped; pool rows at block*block_stride + tok*token_stride
 * (token-major layout: a row is contiguous). */
void kvo_append(uint8_t *layer, int64_t plane_stride, int64_t block_stride, int64_t token_stride,
                int64_t block_size, int64_t row_bytes, const uint8_t *key, const uint8_t *value,
                int64_t key_token_stride, int64_t value_token_stride, const int64_t *slots,
                int64_t T) {
  for (int64_t t = 0; t < T; ++t) {
    int64_t s = slots[t];
    if (s < 0) continue;
    int64_t blk = s / block_size, tok = s % block_size;
    uint8_t *d = layer + blk * block_stride + tok * token_stride;
    memcpy(d, key + t * key_token_stride, (size_t)row_bytes);
    memcpy(d + plane_stride, value + t * value_token_stride, (size_t)row_bytes);
  }
}

/* Returns the number of moves, or -1 on a bad table (range / duplicate). */
int64_t kvo_compact_plan(const int64_t *ids, int64_t n, int64_t num_blocks, int64_t *new_ids,
                         int64_t *move_src, int64_t *move_dst) {
  if (n > num_blocks) return -1;
  uint8_t *live = (uint8_t *)calloc((size_t)num_blocks, 1);
  if (!live) return -1;
  for (int64_t i = 0; i < n; ++i) {
    if (ids[i] < 0 || ids[i] >= num_blocks || live[ids[i]]) {
      free(live);
      return -1;
    }
    live[ids[i]] = 1;
  }
  int64_t hole = 0, m = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (ids[i] < n) {
      new_ids[i] = ids[i];
      continue;
    }
    while (live[hole]) ++hole;
    move_src[m] = ids[i];
    move_dst[m] = hole;
    new_ids[i] = hole++;
    ++m;
  }
  free(live);
  return m;
}
