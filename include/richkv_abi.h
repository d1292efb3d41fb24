/* richkv_abi.h — byte layout of paged KV storage and of the per-lane kernel
 * parameters, shared by host C/C++ code, the CUDA kernels and the CPU oracle.
 *
 * Layout-compatible with the reference's host/shader ABI:
 *   runtime/metal/abi/KvExtent.h:16-111          (page entry, element and extent offsets)
 *   runtime/metal/abi/PagedAttention.h:14-87     (parameter blocks, 8/8/24/32/36 bytes)
 *   runtime/metal/abi/ExecutionGeometry.h:5-40   (page size, limits)
 *   runtime/ops/PagedKv.hpp:16,125-168           (formats and byte accounting)
 * A reference-side caller can pass its own structs through a reinterpret_cast;
 * the static assertions below pin every size and field offset.
 */
#ifndef RICHKV_ABI_H
#define RICHKV_ABI_H

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define RK_HD __host__ __device__ __forceinline__
#else
#define RK_HD static inline
#endif

/* ---- geometry constants (ExecutionGeometry.h) ---------------------------- */
#define RK_PAGE_TOKENS 32u                 /* tokens per KV page                      */
#define RK_VERIFY_ROWS 8u                  /* rows of a chain verify lane             */
#define RK_TREE_NODES 16u                  /* row capacity of a tree verify lane      */
#define RK_MAX_CONTEXT_TOKENS 262144u
#define RK_SCRATCH_TOKENS (RK_TREE_NODES - 1u)
#define RK_MAX_PHYSICAL_TOKENS (RK_MAX_CONTEXT_TOKENS + RK_SCRATCH_TOKENS)
#define RK_PREFILL_TOKEN_BUDGET 2048u      /* rows of one prefill chunk               */
#define RK_VERIFY_CHUNK_STRIDE RK_PAGE_TOKENS
#define RK_PREFILL_TILE_ROWS 8u
#define RK_PREFILL_MAX_SPLITS 32u
#define RK_VERIFY_MAX_SPLITS 128u
#define RK_REFERENCE_BATCH_WIDTH 4u        /* lanes the reference binds per dispatch  */

/* ---- page entries (KvExtent.h:16-20,107-111) ------------------------------ */
/* One page as kernels address it: the address of the extent that holds it,
 * 16 KiB-aligned, with the page's index inside the extent in the low 14 bits. */
typedef uint64_t rk_page_entry;
#define RK_PAGE_INDEX_BITS 14u
#define RK_PAGE_INDEX_MASK ((1u << RK_PAGE_INDEX_BITS) - 1u)

/* Tensors of one layer in the order they sit in the layer's region. */
#define RK_TENSOR_KEYS 0u
#define RK_TENSOR_KEY_SCALES 1u
#define RK_TENSOR_VALUES 2u
#define RK_TENSOR_VALUE_SCALES 3u

/* ---- formats (PagedKv.hpp:16) ---------------------------------------------- */
enum rk_format {
  RK_FORMAT_INT8 = 1,
  RK_FORMAT_BF16 = 2,
  RK_FORMAT_INT4 = 3,
  RK_FORMAT_FP8E4M3 = 4
};

/* Where one attention layer's region starts inside every extent of a pool
 * (KvExtent.h:93-105). */
typedef struct rk_kv_layer {
  uint32_t extent_pages;
  uint32_t offset;
} rk_kv_layer;

/* Chunk store parameters of one lane (PagedAttention.h:39-48). */
typedef struct rk_chunk_params {
  uint32_t committed_tokens;
  uint32_t chunk_tokens;
  uint32_t chunk_stride;
  uint32_t page_table_entries;
  rk_kv_layer kv;
} rk_chunk_params;

/* Prefill attention parameters of one sequence (PagedAttention.h:52-64). */
typedef struct rk_prefill_params {
  uint32_t committed_tokens;
  uint32_t rows;
  uint32_t chunk_stride;
  uint32_t page_table_entries;
  rk_kv_layer kv;
  uint32_t split_count;
  float score_scale; /* 0 selects 1/sqrt(head_dim) */
} rk_prefill_params;

/* Verify (and decode) attention parameters of one lane (PagedAttention.h:73-87). */
typedef struct rk_verify_params {
  uint32_t committed_tokens;
  uint32_t page_table_entries;
  rk_kv_layer kv;
  uint32_t split_count;
  uint32_t slot_splits;
  uint32_t active_rows;
  uint32_t row_capacity;
  float score_scale; /* 0 selects 1/sqrt(head_dim) */
} rk_verify_params;

/* A page whose content goes to another page (PagedKv.hpp:49-53). */
typedef struct rk_page_copy {
  uint32_t from;
  uint32_t to;
} rk_page_copy;

#if defined(__cplusplus)
static_assert(sizeof(rk_kv_layer) == 8, "layer placement is 8 bytes");
static_assert(sizeof(rk_chunk_params) == 24, "chunk store parameters are 24 bytes");
static_assert(sizeof(rk_prefill_params) == 32, "prefill parameters are 32 bytes");
static_assert(sizeof(rk_verify_params) == 36, "verify parameters are 36 bytes");
static_assert(sizeof(rk_page_copy) == 8, "page copy is 8 bytes");
static_assert(offsetof(rk_chunk_params, kv) == 16, "chunk kv offset");
static_assert(offsetof(rk_prefill_params, kv) == 16 &&
                  offsetof(rk_prefill_params, split_count) == 24 &&
                  offsetof(rk_prefill_params, score_scale) == 28,
              "prefill field offsets");
static_assert(offsetof(rk_verify_params, kv) == 8 &&
                  offsetof(rk_verify_params, split_count) == 16 &&
                  offsetof(rk_verify_params, slot_splits) == 20 &&
                  offsetof(rk_verify_params, active_rows) == 24 &&
                  offsetof(rk_verify_params, row_capacity) == 28 &&
                  offsetof(rk_verify_params, score_scale) == 32,
              "verify field offsets");
#endif

/* ---- byte accounting (PagedKv.hpp:144-168) --------------------------------- */
RK_HD int rk_format_valid(uint32_t format) {
  return format == RK_FORMAT_INT8 || format == RK_FORMAT_BF16 ||
         format == RK_FORMAT_INT4 || format == RK_FORMAT_FP8E4M3;
}
RK_HD int rk_format_quantized(uint32_t format) { return format != RK_FORMAT_BF16; }

/* Bytes of K (or V) data one page holds in one layer. */
RK_HD uint32_t rk_data_bytes(uint32_t format, uint32_t kv_heads, uint32_t head_dim) {
  const uint32_t elements = RK_PAGE_TOKENS * kv_heads * head_dim;
  if (format == RK_FORMAT_BF16) return elements * 2u;
  if (format == RK_FORMAT_INT4) return elements / 2u;
  return elements;
}
/* Bytes of K (or V) scales one page holds in one layer; zero for bf16. */
RK_HD uint32_t rk_scale_bytes(uint32_t format, uint32_t kv_heads) {
  return rk_format_quantized(format) ? RK_PAGE_TOKENS * kv_heads * 4u : 0u;
}
RK_HD uint64_t rk_layer_page_bytes(uint32_t format, uint32_t kv_heads, uint32_t head_dim) {
  return 2ull * ((uint64_t)rk_data_bytes(format, kv_heads, head_dim) +
                 rk_scale_bytes(format, kv_heads));
}
/* KV bytes one token occupies in one layer: 1056 / 2080 / 2080 / 4096 at
 * 4 heads x 256 (the unit of every bandwidth figure). */
RK_HD uint64_t rk_token_layer_bytes(uint32_t format, uint32_t kv_heads, uint32_t head_dim) {
  return rk_layer_page_bytes(format, kv_heads, head_dim) / RK_PAGE_TOKENS;
}

/* ---- element placement inside a page's slab (KvExtent.h:41-74) -------------- */
/* Keys are token-major, values dimension-major, one scale per (head, token).
 * INT4 packs two elements per byte (even element in the low nibble) and keeps
 * BOTH tensors token-major: byte index = key_element / 2. */
RK_HD uint64_t rk_key_element(uint32_t head, uint32_t token, uint32_t dim, uint32_t head_dim) {
  return ((uint64_t)head * RK_PAGE_TOKENS + token) * head_dim + dim;
}
RK_HD uint64_t rk_value_element(uint32_t head, uint32_t token, uint32_t dim, uint32_t head_dim) {
  return ((uint64_t)head * head_dim + dim) * RK_PAGE_TOKENS + token;
}
RK_HD uint64_t rk_scale_element(uint32_t head, uint32_t token) {
  return (uint64_t)head * RK_PAGE_TOKENS + token;
}

/* Bytes one page holds of `tensor` in one layer. */
RK_HD uint32_t rk_tensor_page_bytes(uint32_t data_bytes, uint32_t scale_bytes, uint32_t tensor) {
  return (tensor & 1u) ? scale_bytes : data_bytes;
}

/* Byte offset of (layer, tensor, page index) inside an extent (KvExtent.h:80-89):
 * per layer a region of [K data x pages][K scales x pages][V data x pages][V scales x pages]. */
RK_HD uint64_t rk_extent_offset(uint32_t extent_pages, uint32_t data_bytes, uint32_t scale_bytes,
                                uint32_t layer, uint32_t tensor, uint32_t index) {
  const uint64_t region = (uint64_t)layer * extent_pages * 2u * ((uint64_t)data_bytes + scale_bytes);
  const uint64_t before = (uint64_t)((tensor + 1u) / 2u) * data_bytes + (uint64_t)(tensor / 2u) * scale_bytes;
  return region + (uint64_t)extent_pages * before +
         (uint64_t)index * rk_tensor_page_bytes(data_bytes, scale_bytes, tensor);
}

RK_HD rk_kv_layer rk_make_layer(uint32_t extent_pages, uint32_t data_bytes, uint32_t scale_bytes,
                                uint32_t layer) {
  rk_kv_layer placed;
  placed.extent_pages = extent_pages;
  placed.offset = (uint32_t)rk_extent_offset(extent_pages, data_bytes, scale_bytes, layer, RK_TENSOR_KEYS, 0u);
  return placed;
}

RK_HD rk_page_entry rk_make_entry(uint64_t extent_address, uint32_t index) {
  return extent_address | index;
}
RK_HD uint32_t rk_entry_index(rk_page_entry entry) { return (uint32_t)entry & RK_PAGE_INDEX_MASK; }
RK_HD uint64_t rk_entry_extent(rk_page_entry entry) { return entry & ~(uint64_t)RK_PAGE_INDEX_MASK; }

/* Address of `tensor`'s bytes of one page in one layer, from its table entry. */
RK_HD uint64_t rk_tensor_address(rk_page_entry entry, rk_kv_layer layer, uint32_t data_bytes,
                                 uint32_t scale_bytes, uint32_t tensor) {
  const uint64_t before = (uint64_t)((tensor + 1u) / 2u) * data_bytes + (uint64_t)(tensor / 2u) * scale_bytes;
  return rk_entry_extent(entry) + layer.offset + (uint64_t)layer.extent_pages * before +
         (uint64_t)rk_entry_index(entry) * rk_tensor_page_bytes(data_bytes, scale_bytes, tensor);
}

/* The softmax scale a kernel applies: the parameter when non-zero, else
 * 1/sqrt(head_dim) for 64 / 128 / 256 (paged_attention_tile.h:122-126). */
RK_HD float rk_score_scale(float requested, uint32_t head_dim) {
  if (requested != 0.0f) return requested;
  return head_dim == 64u ? 0.125f : (head_dim == 128u ? 0.08838834764831845f : 0.0625f);
}

/* ---- contracts (paged_store_row.h:14-29, paged_attention_tile.h:28-59) ------- */
RK_HD uint32_t rk_pages_for(uint32_t tokens) { return (tokens + RK_PAGE_TOKENS - 1u) / RK_PAGE_TOKENS; }

RK_HD int rk_chunk_contract_valid(const rk_chunk_params *p) {
  return p->committed_tokens <= RK_MAX_PHYSICAL_TOKENS && p->chunk_tokens > 0u &&
         p->chunk_tokens <= RK_PREFILL_TOKEN_BUDGET &&
         (uint64_t)p->committed_tokens + p->chunk_tokens <= RK_MAX_PHYSICAL_TOKENS &&
         p->chunk_stride >= p->chunk_tokens && p->chunk_stride <= RK_PREFILL_TOKEN_BUDGET &&
         p->chunk_stride % RK_PAGE_TOKENS == 0u &&
         p->page_table_entries >= rk_pages_for(p->committed_tokens + p->chunk_tokens) &&
         p->kv.extent_pages > 0u;
}

RK_HD int rk_prefill_contract_valid(const rk_prefill_params *p) {
  return p->rows > 0u && p->rows <= RK_PREFILL_TOKEN_BUDGET && p->chunk_stride >= p->rows &&
         p->chunk_stride <= RK_PREFILL_TOKEN_BUDGET && p->chunk_stride % RK_PAGE_TOKENS == 0u &&
         (uint64_t)p->committed_tokens + p->rows <= RK_MAX_PHYSICAL_TOKENS &&
         p->page_table_entries >= rk_pages_for(p->committed_tokens + p->rows) &&
         p->kv.extent_pages > 0u && p->split_count > 0u && p->split_count <= RK_PREFILL_MAX_SPLITS;
}

RK_HD int rk_verify_contract_valid(const rk_verify_params *p) {
  return p->active_rows > 0u && p->active_rows <= p->row_capacity &&
         p->row_capacity <= RK_TREE_NODES &&
         (uint64_t)p->committed_tokens + p->active_rows <= RK_MAX_PHYSICAL_TOKENS &&
         p->page_table_entries >= rk_pages_for(p->committed_tokens + p->active_rows) &&
         p->kv.extent_pages > 0u && p->split_count > 0u && p->split_count <= RK_VERIFY_MAX_SPLITS &&
         p->slot_splits >= p->split_count && p->slot_splits <= RK_VERIFY_MAX_SPLITS;
}

/* Balanced split partition shared by split and reduce
 * (paged_attention_tile.h:63-69,225-231). */
RK_HD uint32_t rk_pages_per_split(uint32_t pages, uint32_t splits) { return (pages + splits - 1u) / splits; }

#endif /* RICHKV_ABI_H */
