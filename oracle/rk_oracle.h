/* rk_oracle.h — CPU restatement of the reference's paged-KV algorithms.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product library links, imports or
 * calls this file; it is the checker the parity tests, the smoke test and the
 * benchmark's cpu_baseline leg compare the CUDA path against.
 *
 * Every function works on HOST memory laid out exactly like device memory:
 * page tables hold rk_page_entry values whose address part is a host pointer
 * to a 16 KiB-aligned extent. Each function cites the reference lines it
 * restates (paths relative to the reference project root).
 */
#ifndef RK_ORACLE_H
#define RK_ORACLE_H

#include "../include/richkv_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* bf16 <-> fp32, round-to-nearest-even, NaN kept quiet
 * (dev/tests/engine/Q8PageFormatReference.hpp:66-80). */
uint16_t rko_f32_to_bf16(float value);
float rko_bf16_to_f32(uint16_t bits);

/* e4m3 encode (RNE, saturating to 448) and decode
 * (dev/tests/engine/Fp8PageFormatReference.hpp:27-63). */
uint8_t rko_f32_to_e4m3(float value);
float rko_e4m3_to_f32(uint8_t code);
/* bf16 -> fp16 -> fp32: the fp8 tile's query staging
 * (dev/tests/engine/Fp8PageFormatReference.hpp:67-69). */
float rko_query_stage_f16(float value);

/* Append + quantize one lane's chunk rows into their final page slots
 * (runtime/metal/kernels/common/paged_store_row.h:47-147,
 *  runtime/metal/kernels/common/paged_store_row_fp8.h:28-78).
 * chunk_keys is [kv_heads][stride][head_dim] bf16 and chunk_values
 * [kv_heads][head_dim][stride] bf16, both already offset to the lane.
 * Returns 0, or -1 when the contract (paged_store_row.h:14-29) fails, in
 * which case nothing is written. */
int rko_store_chunk(uint32_t format, uint32_t kv_heads, uint32_t head_dim,
                    const uint16_t *chunk_keys, const uint16_t *chunk_values,
                    const rk_page_entry *table, const rk_chunk_params *params);

/* Verify store of `lanes` lanes (decode/paged_attention_store.metal:3-45):
 * lane l's staging begins l*kv_heads*32*head_dim elements in, stride 32,
 * at most 16 rows. tables[l] is lane l's table. */
int rko_store_verify(uint32_t format, uint32_t kv_heads, uint32_t head_dim, uint32_t lanes,
                     const uint16_t *chunk_keys, const uint16_t *chunk_values,
                     const rk_page_entry *const *tables, const rk_chunk_params *params);

/* Reference attention of one (lane, kv head) tile: softmax over the admitted
 * tokens of (q . dequantized K) * score_scale, times dequantized V, evaluated
 * in fp64 (shape of dev/tests/engine/q8_flash_attention_metal_test.mm:289-338;
 * admission rule runtime/metal/kernels/common/paged_attention_tile.h:103-143).
 *   queries: bf16 [row][group][head_dim] of this tile (row stride = group*head_dim)
 *   row_masks: null for the causal chain, else one 32-bit ancestor mask per row
 *   q_fp16: non-zero stages each query element through fp16 (fp8 tile)
 *   out: fp32 [row_capacity*group][head_dim]; rows >= active_rows are zero. */
int rko_attention_tile(uint32_t format, uint32_t kv_heads, uint32_t group, uint32_t head_dim,
                       uint32_t kv_head, const uint16_t *queries, const rk_page_entry *table,
                       rk_kv_layer layer, uint32_t committed_tokens, uint32_t active_rows,
                       uint32_t row_capacity, const uint32_t *row_masks, float score_scale,
                       int q_fp16, float *out);

/* The same over every lane and kv head of a verify batch laid out like the
 * kernels' buffers (decode/paged_attention.metal:23-60): queries and out are
 * [lane][kv_head][32][group][head_dim]; out is bf16 (rows >= active are 0).
 * Runs OpenMP-parallel over (lane, kv head); this is the timed CPU baseline. */
int rko_attention_verify(uint32_t format, uint32_t kv_heads, uint32_t group, uint32_t head_dim,
                         uint32_t lanes, const uint16_t *queries, const rk_page_entry *const *tables,
                         const rk_verify_params *params, const uint32_t *row_masks,
                         uint16_t *out_bf16, float *out_f32);

/* Fixed-order merge of split partials for one fused row
 * (runtime/metal/kernels/common/paged_attention_tile.h:362-404):
 * partials [splits][D] (stride given in floats), stats [splits]{max,sum}.
 * out_f32[D] receives numerator/denominator before the bf16 rounding. */
void rko_merge_row(const float *partials, uint64_t partial_stride, const float *stats,
                   uint64_t stat_stride, uint32_t written, uint32_t head_dim, float *out_f32);

/* Tree-verify compaction of one lane (decode/paged_attention_store.metal:198-278). */
int rko_tree_compact(uint32_t format, uint32_t kv_heads, uint32_t head_dim,
                     const rk_page_entry *table, const rk_chunk_params *params,
                     const uint32_t *retained_path, uint32_t retained_count);

/* Page copy: every tensor of every layer (runtime/ops/PageStorage.mm:95-114,143-167). */
void rko_copy_page(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                   uint32_t extent_pages, rk_page_entry from, rk_page_entry to);

/* The step before the path (kernels/common/attention_qkv_prepare.h:13-83, kernels/decode/attention_qkv.metal:6-60):
 * per (lane, row) the packed projection row [(q | gate) x query heads, k x KV heads, v x KV heads] becomes the stagings
 * the store and the attention read: per-head RMS norm (sum of squares reduced per 32 dims by an xor butterfly
 * 16,8,4,2,1 — the reference's simd_sum leaves the order open, this fixes one — then the partials in order,
 * 1/sqrt(mean + eps)), times the norm weight, rounded to bf16, rotary on the first 2 x 32 dims (separately rounded
 * products), queries [lane][kv][32][group][D], keys [lane][kv][32][D], values [lane][kv][D][32] (a copy of the bits).
 * `norm_f32` selects fp32 norm weights (the _f32 pipelines). */
int rko_qkv_prepare(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes, uint32_t rows,
                    const uint16_t *packed_qkv, const void *q_norm, const void *k_norm, int norm_f32,
                    const float *rope_cos, const float *rope_sin, float eps, uint16_t *queries, uint16_t *chunk_keys,
                    uint16_t *chunk_values);
/* CRC-32C (Castagnoli, reflected polynomial 0x82F63B78, initial and final inversion) one bit at a time; `crc` continues
 * a running value, 0 to start (runtime/model/Crc32c.hpp:12-29 computes the same function with the CPU's CRC
 * instructions). Known answers: RFC 3720 B.4 and the check value of "123456789". */
uint32_t rko_crc32c(const void *data, uint64_t bytes, uint32_t crc);
int rko_threads(void);

#ifdef __cplusplus
}
#endif
#endif
