// Slot-mapped per-token append (reshape_and_cache) for sm_100a.
//
// One warp moves one row: the H*D*e bytes of one token of one plane (K or V)
// of one layer. Rows are numbered plane fastest, then token, then layer. A
// row is contiguous in the source ([T, H, D] with a token stride); in the
// pool it is contiguous for the token-major layout and H runs of D*e bytes
// for the head-major layout, which the explicit token/head strides cover.
//
// slot < 0 is padding and skipped; slot >= num_blocks*block_size records
// EMM_ERR_ID_RANGE in the status word and is skipped. No trap, no early exit
// of the CTA.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "page_copy.cuh"

namespace emm {

struct AppendArgs {
  const uint64_t *layers;  // device array of the pool's per-layer base addresses
  uint64_t plane_stride;
  uint64_t block_stride;
  uint64_t token_stride;
  uint64_t head_stride;
  uint64_t num_slots;    // num_blocks * block_size
  uint32_t block_size;
  uint32_t head_bytes;   // D * elem_size
  uint32_t row_bytes;    // H * D * elem_size
  uint32_t layer_begin;  // first pool layer written
  uint32_t layer_count;
  uint32_t num_tokens;
  uint64_t key;          // base address of key[layer_begin]
  uint64_t value;
  uint64_t key_layer_stride;
  uint64_t key_token_stride;
  uint64_t value_layer_stride;
  uint64_t value_token_stride;
  const int64_t *slots;  // device, num_tokens entries
  int *status;
};

// Rows (warps) per CTA. Measured on B200 for the 2 KiB-row decode batch (32 layers x 256 tokens, rows
// read from HBM): 1, 2, 4, 8 and 16 rows per CTA all take 12.5 us per launch, 32 take 13.2 us.
constexpr int kAppendWarps = 8;

template <typename V, int U>
__global__ void __launch_bounds__(kAppendWarps * 32) append_rows(const AppendArgs a) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t row = (uint64_t)blockIdx.x * kAppendWarps + (threadIdx.x >> 5);
  const uint64_t rows = (uint64_t)a.layer_count * a.num_tokens * 2;
  if (row >= rows) return;
  const uint32_t p = (uint32_t)(row & 1);
  const uint64_t tl = row >> 1;
  const uint32_t lrel = (uint32_t)(tl / a.num_tokens);
  const uint32_t t = (uint32_t)(tl - (uint64_t)lrel * a.num_tokens);

  // The source row does not depend on the slot: issue its first loads before the
  // slot is known so the two global-memory latencies overlap instead of adding up
  // (a padding row costs a wasted load, padding is ~1 % of a batch).
  const uint64_t src = p ? a.value + (uint64_t)lrel * a.value_layer_stride + (uint64_t)t * a.value_token_stride
                         : a.key + (uint64_t)lrel * a.key_layer_stride + (uint64_t)t * a.key_token_stride;
  const uint32_t head_vecs = a.head_bytes / (uint32_t)sizeof(V);
  const uint32_t row_vecs = a.row_bytes / (uint32_t)sizeof(V);
  V v[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint32_t k = (uint32_t)u * 32u + lane;
    if (k < row_vecs) v[u] = *reinterpret_cast<const V *>(src + (uint64_t)k * sizeof(V));
  }

  const int64_t slot = a.slots[t];
  if (slot < 0) return;  // padding entry
  if ((uint64_t)slot >= a.num_slots) {
    if (lane == 0) report(a.status, kStatusIdRange, slot);
    return;
  }
  const uint64_t blk = (uint64_t)slot / a.block_size;
  const uint64_t tok = (uint64_t)slot - blk * a.block_size;
  const uint64_t dst = a.layers[a.layer_begin + lrel] + (uint64_t)p * a.plane_stride +
                       blk * a.block_stride + tok * a.token_stride;
  const bool dense = a.head_stride == a.head_bytes;  // token row contiguous in the pool

  for (uint32_t base = 0; base < row_vecs; base += 32u * U) {
    if (base != 0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t k = base + (uint32_t)u * 32u + lane;
        if (k < row_vecs) v[u] = *reinterpret_cast<const V *>(src + (uint64_t)k * sizeof(V));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k = base + (uint32_t)u * 32u + lane;
      if (k < row_vecs) {
        uint64_t off;
        if (dense) {
          off = (uint64_t)k * sizeof(V);
        } else {
          const uint32_t h = k / head_vecs;
          off = (uint64_t)h * a.head_stride + (uint64_t)(k - h * head_vecs) * sizeof(V);
        }
        *reinterpret_cast<V *>(dst + off) = v[u];
      }
    }
  }
}

}  // namespace emm
