/* richkv.h — C ABI of the B200 paged, quantized KV-cache path.
 *
 * Plain pointers and sizes only. Every device pointer argument is a CUDA device
 * address; `stream` is a cudaStream_t passed as void*. Functions return 0 (RK_OK)
 * or a negative status; rk_last_error() gives the text of the calling thread's
 * last failure. Nothing here falls back to the CPU.
 *
 * Each entry point names the reference interface it replaces (paths relative to
 * the reference project root). The reference binds four lanes per dispatch as
 * four table buffers (runtime/ops/PagedAttention.cpp:479-500); here `tables` is a
 * device array of table addresses and `lane_params` a device array of parameter
 * blocks, so any batch width runs in one launch, and the layer placement that the
 * reference writes into every lane's block (PagedAttention.cpp:482,487) travels
 * as the `layer` argument: the lane array is uploaded once per step, not once per
 * layer. A block's own `kv` field is used only where no `layer` is passed.
 */
#ifndef RICHKV_H
#define RICHKV_H

#include "richkv_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

#define RK_OK 0
#define RK_ERR_INVALID (-1)     /* contract violation detected on the host; nothing was launched */
#define RK_ERR_CUDA (-2)        /* a CUDA call failed */
#define RK_ERR_UNSUPPORTED (-3) /* no kernel for this geometry or format */
#define RK_ERR_REFUSED (-4)     /* capacity refusal: budget, driver out of memory, tier limits */
#define RK_ERR_TIMEOUT (-5)     /* a bounded wait inside a kernel ran out */

const char *rk_last_error(void);

/* Layout::extentAlignmentPages (runtime/ops/PagedKv.hpp:175-183). */
uint32_t rk_extent_alignment_pages(uint32_t format, uint32_t kv_heads, uint32_t head_dim);

/* ---- append and quantize ------------------------------------------------------------------ */
/* verify_attention_{q8,int4,bf16,fp8}_store (runtime/metal/kernels/decode/paged_attention_store.metal:3-186,
 * decode/fp8_attention_store.metal:8-70), encoded by PagedAttention::addVerify (PagedAttention.cpp:467-503).
 * chunk_keys [lane][kv_head][32][D], chunk_values [lane][kv_head][D][32] bf16; each lane stores
 * lane_params[lane].chunk_tokens (<= 16, <= max_rows) rows at committed_tokens + row. */
int rk_store_verify(uint32_t format, uint32_t kv_heads, uint32_t head_dim, uint32_t lanes, uint32_t max_rows,
                    const void *chunk_keys, const void *chunk_values, const rk_page_entry *const *tables,
                    const rk_chunk_params *lane_params, rk_kv_layer layer, void *stream);
/* prefill_attention_*_store (runtime/metal/kernels/prefill/paged_attention_store.metal:7-149), encoded by
 * PagedAttention::addPrefillStore (PagedAttention.cpp:424-441). `params` is a HOST pointer (the reference
 * passes the block by value); its kv field places the layer. */
int rk_store_chunk(uint32_t format, uint32_t kv_heads, uint32_t head_dim, const void *chunk_keys,
                   const void *chunk_values, const rk_page_entry *table, const rk_chunk_params *params,
                   void *stream);

/* ---- general attention tile: any row count, tree masks, prefill chunks ----------------------- */
/* verify_attention_*_split / verify_tree_attention_*_split (decode/paged_attention.metal:23-192,
 * decode/fp8_attention.metal:8-62). grid_splits = the plan's split count (max over lanes);
 * row_capacity is 1, 8 or 16 and strides the partial slots; row_masks (tree) may be null. */
int rk_attention_verify_split(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                              uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits, const void *queries,
                              float *partials, float *statistics, const rk_page_entry *const *tables,
                              const uint32_t *row_masks, const rk_verify_params *lane_params, rk_kv_layer layer,
                              void *stream);
/* verify_attention_reduce / verify_tree_attention_reduce (decode/paged_attention.metal:198-263,415-531).
 * output bf16 [lane][kv_head][32][group][D]; output_f32 (optional) receives the value before rounding. */
int rk_attention_verify_reduce(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                               uint32_t row_capacity, const float *partials, const float *statistics,
                               void *output, float *output_f32, const rk_verify_params *lane_params,
                               void *stream);
/* verify_attention_reduce_gate / verify_attention_reduce_gather (decode/paged_attention.metal:273-413), encoded by
 * PagedAttention::addVerify when its gate buffers are bound (PagedAttention.hpp:299-311): the merge that also writes
 * the out-projection's input `hidden` [lane][row][query head][D] bf16 = merged row x sigmoid(gate), the gate read from
 * `packed_qkv` [lane][row][(q | gate) x query heads, k x KV heads, v x KV heads]; with `packed_qkv` null the merged row
 * itself (gather form; `output` may then be null too). Rows per lane = row_capacity. */
int rk_attention_verify_reduce_gate(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                                    uint32_t row_capacity, const float *partials, const float *statistics,
                                    void *output, const void *packed_qkv, void *hidden,
                                    const rk_verify_params *lane_params, void *stream);
/* prefill_attention_*_split and prefill_attention_reduce (prefill/paged_attention.metal:7-206), encoded by
 * PagedAttention::addPrefill (PagedAttention.cpp:443-465). `params` is a HOST pointer. */
int rk_attention_prefill_split(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                               const void *queries, float *partials, float *statistics,
                               const rk_page_entry *table, const rk_prefill_params *params, void *stream);
int rk_attention_prefill_reduce(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, const float *partials,
                                const float *statistics, void *output, float *output_f32,
                                const rk_prefill_params *params, void *stream);

/* ---- the step before the path: packed projection rows -> stagings (and pages) ---------------------- */
/* verify_attention_qkv / verify_attention_qkv_f32 (runtime/metal/kernels/decode/attention_qkv.metal:33-60 over
 * kernels/common/attention_qkv_prepare.h:13-83; encoded by the attention operator before PagedAttention::addVerify):
 * per (lane, row) the packed row [(q | gate) x query heads, k x KV heads, v x KV heads] bf16 becomes
 * queries [lane][kv][32][group][D], keys [lane][kv][32][D], values [lane][kv][D][32]: per-head RMS norm (eps) times
 * the norm weight (bf16, or fp32 with norm_f32), rounded to bf16, rotary on the first 2 x 32 dims with
 * rope_cos / rope_sin [lane][row][32] fp32; values are copied. rows <= 16, the same for every lane. */
int rk_qkv_prepare(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes, uint32_t rows,
                   const void *packed_qkv, const void *q_norm, const void *k_norm, int norm_f32,
                   const float *rope_cos, const float *rope_sin, float eps, void *queries, void *chunk_keys,
                   void *chunk_values, void *stream);
/* The same with the page store merged in (the reference lists this merge as open work, TODO.md:14): the key and
 * value rows are quantised into their page slots instead of being staged. Pages equal rk_qkv_prepare followed by
 * rk_store_verify bit for bit; `lane_params` as for rk_store_verify (chunk_tokens = rows). */
int rk_qkv_prepare_store(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                         uint32_t rows, const void *packed_qkv, const void *q_norm, const void *k_norm, int norm_f32,
                         const float *rope_cos, const float *rope_sin, float eps, void *queries,
                         const rk_page_entry *const *tables, const rk_chunk_params *lane_params, rk_kv_layer layer,
                         void *stream);

/* ---- streaming decode attention (one query row per lane) ---------------------------------------- */
/* The reference has no single-query kernel: a plain decode is its tile with one active row
 * (runtime/metal/kernels/common/paged_attention_tile.h:108-110; tested as history 0, rows 1 in
 * dev/tests/engine/paged_attention_plan_test.mm:1019). This entry replaces split + reduce for
 * active_rows = row_capacity = 1 with the TMA-streamed kernel of the pool's format (int4, int8, fp8 e4m3,
 * bf16; the fp8 kernel contracts fp16-staged queries as decode/fp8_attention.metal does); scratch is sized
 * by the plan. */
typedef struct rk_decode_plan {
  uint32_t lanes, ctas, max_segments, reserved;
  uint64_t partials_bytes, statistics_bytes, descriptor_bytes;
} rk_decode_plan;
int rk_decode_plan_make(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                        uint32_t lanes, uint32_t ctas, rk_decode_plan *plan);
/* The device address window that holds every page of a pool (rk_storage_window): the TMA tensor map. */
void *rk_window_create(uint64_t base, uint64_t bytes);
void rk_window_destroy(void *window);
/* verify_attention_{q8,int4,bf16}_split / verify_tree_attention_*_split (decode/paged_attention.metal:23-192)
 * and verify_attention_fp8_split (decode/fp8_attention.metal) for 1-, 8- or 16-row windows as a tcgen05 contraction: the fused rows are the M side of a 128-row
 * tensor-core tile with accumulators in tensor memory, pages arrive by TMA through the pool's window.
 * Arguments and scratch layout as rk_attention_verify_split; merge with rk_attention_verify_reduce.
 * Any split count the contract allows is valid; about two CTAs' worth of (lane, head, split) per SM
 * is the efficient choice. `status` is one device word the caller zeroes: it turns non-zero when a
 * bounded wait inside a kernel ran out (the step's output is then invalid). RK_ERR_UNSUPPORTED for
 * other geometries or row counts. */
int rk_attention_verify_split_tc(const void *window, uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                 uint32_t head_dim, uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits,
                                 const void *queries, float *partials, float *statistics,
                                 const rk_page_entry *const *tables, const uint32_t *row_masks,
                                 const rk_verify_params *lane_params, rk_kv_layer layer, uint32_t *status,
                                 void *stream);
/* prefill_attention_*_split (prefill/paged_attention.metal:7-67) on the same tcgen05 kernel: one CTA per (KV
 * head, split, 8-row tile of the chunk). Arguments and scratch layout as rk_attention_prefill_split plus the
 * window and the status word; merge with rk_attention_prefill_reduce. `params` is a HOST pointer. */
int rk_attention_prefill_split_tc(const void *window, uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                  uint32_t head_dim, const void *queries, float *partials, float *statistics,
                                  const rk_page_entry *table, const rk_prefill_params *params, uint32_t *status,
                                  void *stream);
/* Test hook of the window kernel's timeout path, no counterpart in the reference: rk_attention_verify_split_tc
 * (chain masks) whose waits give up after `spin_limit` polls (at most 2^20) and whose TMA warp never streams the
 * last `withheld_groups` 64-token groups of each split. `status` turns non-zero, tensor memory is released and
 * the kernel returns; nothing faults and no wait is unbounded. The step's output is invalid by construction. */
int rk_attention_verify_probe_timeout(const void *window, uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                      uint32_t head_dim, uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits,
                                      const void *queries, float *partials, float *statistics,
                                      const rk_page_entry *const *tables, const rk_verify_params *lane_params,
                                      rk_kv_layer layer, uint32_t *status, uint32_t spin_limit,
                                      uint32_t withheld_groups, void *stream);
int rk_attention_decode(const void *window, const rk_decode_plan *plan, uint32_t format, const void *queries,
                        void *output, float *output_f32, float *partials, float *statistics,
                        uint32_t *descriptors, const rk_page_entry *const *tables,
                        const rk_verify_params *lane_params, rk_kv_layer layer, void *stream);
/* Sequence split of one long context over several GPUs (new here; the reference is single-GPU, its
 * split merge paged_attention_tile.h:362-404 is the combine). Each rank attends the pages it holds and
 * leaves {max, sum, un-normalised output} per (lane, query head) in `triples`
 * ([lane][query_head][2 + D] fp32); after an all-gather every rank merges the shards in rank order. */
int rk_attention_decode_shard(const void *window, const rk_decode_plan *plan, uint32_t format, const void *queries,
                              float *triples, float *partials, float *statistics, uint32_t *descriptors,
                              const rk_page_entry *const *tables, const rk_verify_params *lane_params,
                              rk_kv_layer layer, void *stream);
int rk_attention_merge_shards(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                              uint32_t shards, const float *triples, void *output, float *output_f32,
                              void *stream);
/* The same step with the combine inside the library's own kernels instead of a collective library: after the
 * streaming kernel one fused kernel reduces this rank's partials, writes its triple into every rank's exchange
 * buffer with plain peer stores (NVLink), publishes it with system-scope releases, waits (bounded) for every
 * rank's triple in its own buffer and merges them in rank order; `output` ends identical on all ranks.
 * rk_exchange_create allocates this rank's buffer and returns its 64-byte CUDA IPC handle; the caller gathers all
 * ranks' handles (ranks x 64 bytes, in rank order) and passes them to rk_exchange_connect. Every rank calls
 * rk_attention_decode_exchange once per step, in the same order; loopback_rank is -1 (a value >= 0 emulates that
 * rank of a step on ONE GPU over an unconnected exchange: all but the last rank only publish). A wait for a peer
 * that runs out raises the decode status word. The epoch is a launch argument: not for replay from a graph. */
void *rk_exchange_create(uint32_t rank, uint32_t ranks, uint32_t lanes, void *handle_out);
int rk_exchange_connect(void *exchange, const void *handles);
void rk_exchange_destroy(void *exchange);
int rk_attention_decode_exchange(const void *window, const rk_decode_plan *plan, uint32_t format, const void *queries,
                                 void *output, float *output_f32, float *partials, float *statistics,
                                 uint32_t *descriptors, const rk_page_entry *const *tables,
                                 const rk_verify_params *lane_params, rk_kv_layer layer, void *exchange,
                                 int32_t loopback_rank, void *stream);
/* No counterpart in the reference. rk_attention_decode for callers that cannot allocate device
 * memory (the pool owns the whole device, the calling thread may not enter the allocator, or
 * allocation calls are not permitted where it runs): the step's scratch is a fixed array inside
 * the library, about 12 MiB per GPU that loads it, which limits a call to 16 lanes; more are
 * refused with RK_ERR_INVALID. The first call on a device resolves the array's address and should
 * come before any stream capture. Calls share the array: calls that overlap on the GPU race.
 * rk_attention_decode_static_status reports a wait that ran out. */
int rk_attention_decode_static(const void *window, uint32_t format, uint32_t lanes, const void *queries,
                               void *output, float *output_f32, const rk_page_entry *const *tables,
                               const rk_verify_params *lane_params, rk_kv_layer layer, void *stream);
/* The decode kernels' status word (the word after the 2 x lanes descriptors; the caller zeroes `descriptors` once,
 * before its first step) is sticky: a bounded wait that runs out in ANY launch raises it, no launch clears it.
 * This call synchronises `stream`, reports RK_ERR_TIMEOUT if the word was raised since the last read, and clears
 * it. A step whose wait ran out wrote zeros for the affected lanes. The reference's analogue is its command
 * watchdog (runtime/metal/CommandWatchdog.hpp:11-35). */
int rk_attention_decode_status(const rk_decode_plan *plan, uint32_t *descriptors, void *stream);
/* The same for rk_attention_decode_static (its status word lives inside the library's own array). */
int rk_attention_decode_static_status(void *stream);
/* Test hook of the timeout path, no counterpart in the reference: rk_attention_decode whose waits give up after
 * `spin_limit` polls (at most 2^20) and whose producers never stream the last `withheld_pages` pages of each
 * CTA's range. The waiting warps run out of polls, raise the status word, copies in flight land and the kernel
 * returns; nothing faults and no wait is unbounded. The step's output is invalid by construction. With `partials`,
 * `statistics` and `descriptors` all null the probe runs on the library's own array, as rk_attention_decode_static
 * does (plan->lanes <= 16), and rk_attention_decode_static_status reports it. */
int rk_attention_decode_probe_timeout(const void *window, const rk_decode_plan *plan, uint32_t format,
                                      const void *queries, void *output, float *partials, float *statistics,
                                      uint32_t *descriptors, const rk_page_entry *const *tables,
                                      const rk_verify_params *lane_params, rk_kv_layer layer, uint32_t spin_limit,
                                      uint32_t withheld_pages, void *stream);
/* Compact host-style rows <-> the 32-row stagings (row 0): queries [lane][query_head][D],
 * keys / values [lane][kv_head][D]. The reference's QKV projection writes the stagings on the GPU
 * (runtime/metal/kernels/decode/attention_qkv.metal:6-60); these serve callers that hold host rows. */
int rk_stage_decode_rows(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes, const void *q,
                         const void *k, const void *v, void *queries, void *chunk_keys, void *chunk_values,
                         void *stream);
int rk_gather_decode_rows(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                          const void *output, void *out, void *stream);
/* One layer of a decode step with HOST rows, as one call. The reference's host reaches its attention operator with
 * rows the model runtime produced on the GPU (PagedAttention::addVerify, runtime/ops/PagedAttention.cpp:467-545,
 * called per layer from runtime/model/QwenTarget.cpp:799-812); a caller that holds the rows in pinned host memory
 * makes this call instead: q_host [lane][query_head][D], k_host / v_host [lane][kv_head][D] go up, the key / value
 * rows are appended to the pages (rk_store_verify, row capacity 1), the query row attends (rk_attention_decode) and
 * out_host [lane][query_head][D] comes back. Asynchronous: uploads run on the session's copy stream one call ahead
 * of the kernels on `stream`, results leave on a second copy stream behind them; the host buffers must stay
 * unchanged, and out_host is valid, only after rk_session_finish_host(session, stream) and a synchronise of
 * `stream`. `tables`, `chunk_params` (chunk_tokens 1, chunk_stride RK_VERIFY_CHUNK_STRIDE) and `verify_params`
 * (active_rows = row_capacity = 1) are device arrays, one entry per lane, as for the calls it makes. The session owns
 * its device buffers (one allocation at creation, none per call). rk_session_status reads and clears the sticky
 * status word of the session's decode scratch (RK_ERR_TIMEOUT when a bounded wait ran out in any step since the
 * last read). */
void *rk_session_create(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                        const void *window, const rk_kv_layer *layers, uint32_t layer_count, uint32_t ctas);
void rk_session_destroy(void *session);
int rk_session_step_host(void *session, uint32_t layer, const void *q_host, const void *k_host, const void *v_host,
                         void *out_host, const rk_page_entry *const *tables, const rk_chunk_params *chunk_params,
                         const rk_verify_params *verify_params, void *stream);
int rk_session_finish_host(void *session, void *stream);
int rk_session_status(void *session, void *stream);

/* ---- page moves --------------------------------------------------------------------------------- */
/* kv::ExtentStorage::copyPages (runtime/ops/PagedKv.hpp:70-75, PageStorage.mm:95-114) on table entries:
 * every tensor of every layer of from_entries[i] onto to_entries[i]. Also the copy-on-write fork. */
int rk_copy_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t extent_pages,
                  const rk_page_entry *from_entries, const rk_page_entry *to_entries, uint32_t count,
                  void *stream);
/* A page's spans (PageStorage::spans, PageStorage.mm:143-167) packed into / unpacked from contiguous
 * slots of layers * layer-page bytes each: the staging of the host tier. */
int rk_pack_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t extent_pages,
                  const rk_page_entry *from_entries, void *slots, uint32_t count, void *stream);
int rk_unpack_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t extent_pages,
                    const void *slots, const rk_page_entry *to_entries, uint32_t count, void *stream);
/* verify_tree_attention_*_compact (decode/paged_attention_store.metal:198-310), encoded by
 * PagedAttention::addVerifyTreeCompact (PagedAttention.cpp:547-573). retained_path [lane][8]. */
int rk_tree_compact(uint32_t format, uint32_t kv_heads, uint32_t head_dim, uint32_t lanes,
                    const rk_page_entry *const *tables, const rk_chunk_params *lane_params, rk_kv_layer layer,
                    const uint32_t *retained_path, const uint32_t *retained_count, void *stream);

/* ---- extent storage: kv::PageStorage (runtime/ops/PageStorage.hpp:27-102, PageStorage.mm) --------- */
void *rk_storage_create(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                        uint32_t page_count, uint32_t extent_pages);
void rk_storage_destroy(void *storage);
int rk_storage_allocate_extent(void *storage, uint32_t extent); /* 0 granted, RK_ERR_REFUSED, RK_ERR_INVALID */
int rk_storage_release_extent(void *storage, uint32_t extent);
void rk_storage_set_budget(void *storage, uint64_t bytes); /* the admission the reference injects (PageStorage.hpp:31) */
uint32_t rk_storage_page_count(const void *storage);
uint32_t rk_storage_extent_pages(const void *storage);
uint64_t rk_storage_bytes_per_page(const void *storage);
uint64_t rk_storage_extent_bytes(const void *storage);
uint64_t rk_storage_allocated_bytes(const void *storage);
int rk_storage_is_allocated(const void *storage, uint32_t page);
void rk_storage_window(const void *storage, uint64_t *base, uint64_t *bytes);
uint32_t rk_storage_layers(const void *storage, rk_kv_layer *out, uint32_t capacity);
rk_page_entry rk_storage_entry(const void *storage, uint32_t page);
int rk_storage_read_extent(const void *storage, uint32_t extent, uint64_t offset, void *host, uint64_t bytes);
int rk_storage_write_extent(void *storage, uint32_t extent, uint64_t offset, const void *host, uint64_t bytes);
/* PageStorage::writeEntries (PageStorage.mm:127-141) into a device table. */
int rk_storage_write_entries(const void *storage, const uint32_t *pages, uint32_t count, uint32_t first,
                             rk_page_entry *device_table, uint32_t table_capacity, void *stream);
int rk_storage_copy_pages(void *storage, const rk_page_copy *copies, uint32_t count, void *stream);
int rk_storage_pack_pages(void *storage, const uint32_t *pages, uint32_t count, void *device_slots, int unpack,
                          void *stream);
/* Pack + CRC-32C in one pass over each page (what the reference's slot-file IO worker does while it writes a
 * payload, runtime/model/SlotFile.cpp:715-735): slots as rk_storage_pack_pages, `checksums` a device array of
 * `count` words. The host tier's demotions use it. */
int rk_storage_seal_pages(void *storage, const uint32_t *pages, uint32_t count, void *device_slots,
                          uint32_t *checksums, void *stream);

/* ---- checksums of persistent payloads ----------------------------------------------------------------
 * CRC-32C as the reference's slot file keeps it per payload and per record (runtime/model/Crc32c.hpp:12-29,
 * runtime/model/SlotFile.cpp:715-735). rk_crc32c_pages: `count` payloads of `payload_bytes` (whole 512-byte rows,
 * as every packed page is), `stride` bytes apart in DEVICE memory, one word each into out[count] (device);
 * `ctas` = 0 takes one CTA per SM. rk_crc32c_host: a host buffer, continuing from `crc` (0 to start). */
int rk_crc32c_pages(const void *data, uint64_t stride, uint64_t payload_bytes, uint32_t count, uint32_t *out,
                    uint32_t ctas, void *stream);
uint32_t rk_crc32c_host(const void *data, uint64_t bytes, uint32_t crc);

/* ---- pinned-host eviction tier: engine::KvTier (runtime/engine/cache/KvTier.hpp:34-63) with the
 * transfer bounds of KvPageTier (runtime/engine/cache/KvPageTier.cpp:38-132) ------------------------
 * rk_tier_demote / rk_tier_restore accept a transfer and return its id at once; the copies themselves go out in
 * batches of up to 16 of a kind — when a batch is full, at the next rk_tier_poll and at rk_tier_drain — so a caller
 * that waits for a transfer polls, as the reference's cache does (Cache::pollTransfers). A batch of demotions is one
 * kernel (pack + CRC-32C of every page in one pass) and one copy per run of neighbouring host slots; a batch of
 * restores is one kernel that unpacks the pages straight out of the pinned arena. A page stays valid until its
 * demotion has retired; a restored page is valid once its restore has retired. */
void *rk_tier_create(void *storage, uint32_t slots, uint32_t transfer_limit);
void rk_tier_destroy(void *tier);
uint64_t rk_tier_slot_bytes(const void *tier);
int rk_tier_writable(const void *tier);
int rk_tier_can_demote(const void *tier);
int rk_tier_can_restore(const void *tier);
int64_t rk_tier_acquire_slot(void *tier); /* -1 when the quota is full */
void rk_tier_release_slot(void *tier, uint32_t slot);
void rk_tier_fail_next(void *tier, uint32_t count); /* host-side fault injection for tests */
/* CRC-32C of the payload the slot's last landed demotion stored, taken on the device when the page was packed. */
uint32_t rk_tier_slot_checksum(const void *tier, uint32_t slot);
/* model::SlotFile::adopt (runtime/model/SlotFile.hpp:196-200): a free slot takes a payload an earlier process
 * stored; its first restore fails unless the CRC-32C of what reached the device equals `checksum`.
 * Returns the slot id, -1 when the quota is full. */
int64_t rk_tier_adopt_slot(void *tier, const void *payload, uint64_t bytes, uint32_t checksum);
const void *rk_tier_slot_host_pointer(const void *tier, uint32_t slot);
int rk_tier_demote(void *tier, uint32_t page, uint32_t slot, void *after_stream);  /* transfer id or status */
int rk_tier_restore(void *tier, uint32_t slot, uint32_t page, void *after_stream); /* transfer id or status */
int rk_tier_poll(void *tier);
int rk_tier_transfer_ready(const void *tier, uint32_t id);
int rk_tier_transfer_finish(void *tier, uint32_t id); /* 1 success, 0 failure */
int rk_tier_drain(void *tier);

#ifdef __cplusplus
}
#endif
#endif /* RICHKV_H */
