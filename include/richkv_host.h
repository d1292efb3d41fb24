/* richkv_host.h — C handles over the host control plane (C++ classes in richengine_b200/csrc/host):
 * the page allocator, the request/prefix cache with its eviction tier, and the operator plans.
 * They exist so that non-C++ hosts (the Python tests and benchmark here) can drive the same objects;
 * a C++ host uses the classes directly. Reference interfaces mirrored:
 *   engine::KvPool      runtime/engine/cache/KvPool.hpp:75-185
 *   engine::Cache       runtime/engine/cache/Cache.hpp:213-436 (request / page-table / prefix / eviction subset)
 *   ops::PagedAttention runtime/ops/PagedAttention.hpp:199-324 (plans)
 * Status codes are those of richkv.h. */
#ifndef RICHKV_HOST_H
#define RICHKV_HOST_H

#include "richkv.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- pool -------------------------------------------------------------------------------------- */
/* Over a memory-less storage with a page budget (host-only use) or over a device storage handle. */
void *rk_pool_create_budget(uint32_t pages, uint64_t bytes_per_page, uint32_t extent_pages, uint32_t runway_pages,
                            uint64_t budget_pages);
void *rk_pool_create_device(void *storage, uint32_t runway_pages, void *stream);
void rk_pool_destroy(void *pool);
void rk_pool_set_budget(void *pool, uint64_t budget_pages); /* budget storage only */
int rk_pool_acquire(void *pool, uint32_t count, uint32_t *pages_out); /* count, or RK_ERR_REFUSED */
int rk_pool_retain(void *pool, uint32_t page, int prefix_owner);
int rk_pool_release(void *pool, uint32_t page, int prefix_owner);
uint64_t rk_pool_reclaim_empty_extents(void *pool, int keep_runway, uint32_t limit);
/* Destinations of the emptied extent into destinations_out (extent_pages entries); returns its first
 * page, or -1 when nothing moved. */
int64_t rk_pool_compact_extent(void *pool, const uint32_t *fixed, uint32_t fixed_count, uint32_t *destinations_out);
/* out[10] = pagesAllocated, pagesFree, pagesActive, pagesPrefix, allocatedBytes, reclaimableBytes,
 *           extentAllocations, extentReleases, extentCompactions, pagesMoved */
void rk_pool_snapshot(const void *pool, uint64_t *out);
uint64_t rk_pool_page_content(const void *pool, uint32_t page);       /* budget storage: the page's content tag */
void rk_pool_set_page_content(void *pool, uint32_t page, uint64_t tag);

/* ---- cache ------------------------------------------------------------------------------------- */
/* tier_mode 0: no tier; 1: pinned-host tier (device pools) with `slots` slots and `transfers` in flight;
 * 2: a host-only tier whose transfers finish when rk_cache_complete_transfer is called (tests). */
void *rk_cache_create(void *pool, int tier_mode, uint32_t slots, uint32_t transfers);
void rk_cache_destroy(void *cache);
int rk_cache_begin_request(void *cache, uint64_t request);
int rk_cache_end_request(void *cache, uint64_t request);
/* 0 granted, 1 denied, 2 pending (demotions on their way cover the need) */
int rk_cache_ensure_tokens(void *cache, uint64_t request, uint64_t tokens);
/* Copies up to capacity page ids; returns the page count; revision and first_changed as Cache::pageTable. */
int64_t rk_cache_page_table(const void *cache, uint64_t request, uint32_t *pages_out, uint32_t capacity,
                            uint64_t *revision, uint32_t *first_changed);
/* One image in a prompt (ImageSpan, runtime/model/Model.hpp:130-146): the run of placeholder tokens it occupies, its
 * patch grid and a 128-bit digest of its content. Every image has the same placeholder token ids, so the key of a block
 * carries the identity of the images that overlap it (blockImageIdentity, runtime/engine/cache/KvCache.cpp:29-52).
 * Spans are sorted and disjoint; null / 0 = text alone. The same spans go with every call that names the prompt. */
typedef struct rk_image_span {
  uint32_t offset, tokens, grid_height, grid_width;
  uint64_t digest_lo, digest_hi;
} rk_image_span;
/* The identity a block at tokens [block_begin, block_begin + block_tokens) takes from the spans: out[2] = lo, hi (0, 0 for text). */
void rk_block_image_identity(uint64_t block_begin, uint32_t block_tokens, const rk_image_span *images, uint32_t image_count, uint64_t *out);
int rk_cache_publish(void *cache, uint64_t request, const uint32_t *tokens, uint32_t token_count, uint32_t committed,
                     const rk_image_span *images, uint32_t image_count);
/* Matched blocks into blocks_out (capacity entries); returns how many. */
int64_t rk_cache_lookup(void *cache, const uint32_t *prompt, uint32_t prompt_tokens, uint64_t *blocks_out, uint32_t capacity,
                        const rk_image_span *images, uint32_t image_count);
int rk_cache_attach_prefix(void *cache, uint64_t request, const uint64_t *blocks, uint32_t count, uint32_t *resume_tokens);
int rk_cache_restores_pending(const void *cache, uint64_t request);
/* Cache::kvRestoreStatus (Cache.cpp:787-792): 0 nothing to wait for, 1 pending, 2 a read failed (the block matches
 * nothing any more and leaves, with what hangs below it, once its last request has ended: Cache::dropPoisoned). */
int rk_cache_restore_status(const void *cache, uint64_t request);
/* 1: a chain resumes only through a composite state (a hybrid model), so KV no state needs is dropped instead of
 * written to the tier, as Cache::reclaimKvLeaf does (Cache.cpp:629-659). 0 (default): every block is worth its copy. */
void rk_cache_set_state_coupled(void *cache, int coupled);
int rk_cache_fork(void *cache, uint64_t parent, uint64_t child, uint32_t committed_tokens); /* pages copied, or status */
int64_t rk_cache_truncate(void *cache, uint64_t request, uint32_t committed_tokens, uint32_t scratch_tokens);
int rk_cache_reclaim_one(void *cache);
uint32_t rk_cache_reclaim_for_pages(void *cache, uint32_t pages);
void rk_cache_poll_transfers(void *cache);
int rk_cache_compact_extent(void *cache);
int rk_cache_complete_transfer(void *cache, int success); /* tier_mode 2: finishes the oldest transfer; 0 if none */
void rk_cache_fail_next_transfers(void *cache, uint32_t count); /* tier_mode 1: host-side fault injection */
/* tier_mode 2: changes how many transfers the tier takes at a time (0 = none) and whether it takes writes at all */
void rk_cache_manual_tier_set(void *cache, uint32_t transfer_limit, int writable);
/* tier_mode 2: 1 = one bound on demotions and restores together instead of the pinned-host tier's shares */
void rk_cache_manual_tier_plain_limits(void *cache, int plain);
/* out[6] = demotions the tier refused (Cache::demoteKv, Cache.cpp:824-851), tier copies replaced by a full tier
 *          (Cache::freeDiskSpace, Cache.cpp:871-905), restores cancelled before they were submitted (Cache::endRequest),
 *          pages whose demotion is in flight, demotions and restores that landed (rk_cache_snapshot counts the started) */
void rk_cache_tier_counters(const void *cache, uint64_t *out);
/* out[10] = requests, residentBlocks, tierBlocks, transfers, demotions, restores, failedTransfers,
 *           evictedBlocks, forkCopies, truncatedPages */
void rk_cache_snapshot(const void *cache, uint64_t *out);
/* Block state: out[5] = page (0xffffffff = none), has tier copy, transferring, last used, poisoned (a read of it
 * failed: it matches nothing and leaves once nothing hangs on it). -1 if unknown. */
int rk_cache_block_state(const void *cache, uint64_t block, uint64_t *out);

/* ---- KV that survives a restart: slot file + record file --------------------------------------------
 * The reference's persistent slot file (runtime/model/SlotFile.hpp:98-219; records SlotFile.cpp:238-323, open
 * :398-438) in its own byte format: a 4096-byte header area {"SPLASHSF", version 1, label bytes, slot bytes, tag
 * bytes, CRC-32C} + tag, then per slot index a record {0x53524543, payload CRC-32C, payload bytes} + label +
 * CRC-32C, rounded up to 64 bytes. A file written for another tag, slot size or label size is emptied when it
 * opens; a damaged record, or one whose slot lies outside the slot file, is a free slot. Labels are
 * engine::KvBlockLabel (168 bytes: id, parent, lastUsed, images lo/hi, 32 tokens) and engine::StateLabel
 * (runtime/engine/cache/DiskLabels.hpp:22-37). `slot_bytes` is a multiple of 4096. */
void *rk_slot_store_open(const char *slots_path, const char *records_path, const void *tag, uint32_t tag_bytes,
                         uint32_t label_bytes, uint64_t slot_bytes);
void rk_slot_store_close(void *store);
uint32_t rk_slot_store_record_count(const void *store); /* the records found when the file opened */
int rk_slot_store_record(const void *store, uint32_t at, uint32_t *index, uint64_t *payload_bytes, uint32_t *checksum,
                         void *label);
/* Payload from the start of the slot, zeros after it, then the record (SlotFile::write + label). */
int rk_slot_store_write(void *store, uint32_t index, const void *payload, uint64_t payload_bytes, uint32_t checksum,
                        const void *label);
int rk_slot_store_read(const void *store, uint32_t index, void *destination, uint64_t bytes);
int rk_slot_store_free(void *store, uint32_t index); /* clears the record, then returns the blocks */
int rk_slot_store_synchronize(void *store);
uint64_t rk_slot_record_bytes(uint32_t label_bytes);
int rk_slot_record_encode(uint32_t label_bytes, uint64_t payload_bytes, uint32_t checksum, const void *label, void *out);
int64_t rk_slot_records_header(uint64_t slot_bytes, uint32_t label_bytes, const void *tag, uint32_t tag_bytes, void *out,
                               uint32_t capacity);
/* Cache::labelBlock / Cache::adopt (runtime/engine/cache/Cache.cpp:38-140,852-870) over the pinned-host tier:
 * persist seals every landed tier copy (payload, the CRC-32C taken on the GPU when the page was packed, its
 * KvBlockLabel) and returns the slots written; adopt, on an empty cache, takes back every block under an unbroken
 * chain (out[3] = blocks, dropped, bytes) — a payload is checked against its record on the GPU when it is first
 * restored, and a mismatch is a failed restore (a cache miss). */
int64_t rk_cache_persist(void *cache, void *store);
int rk_cache_adopt(void *cache, void *store, uint64_t *out);
/* Restore points, as the reference keeps them for models whose chains resume only through a composite state
 * (Cache::adopt, runtime/engine/cache/Cache.cpp:70-127; StateLabel, DiskLabels.hpp:31-37): each stored state comes back
 * with its whole chain and a block only for a state. state_labels = `count` records of 24 bytes {block u64, lastUsed
 * u64, tokens u32, checkpoint u32}; state_bytes = each state's size. out[4] = blocks, dropped (records and states left
 * behind), bytes, states. rk_cache_state_labels writes the label of every stored state as a clean stop records it
 * (Cache::relabelStates, StateCache.cpp:307-311,619-625) and returns their number, or -1. */
int rk_cache_adopt_restore_points(void *cache, void *store, const void *state_labels, const uint64_t *state_bytes, uint32_t count,
                                  uint64_t *out);
int64_t rk_cache_state_labels(void *cache, void *labels, uint64_t *state_bytes, uint32_t capacity);

/* ---- composite states and the reclaim order they impose (runtime/engine/cache/StateCache.hpp:137-379 as far as the
 * KV path is coupled to it, Cache.hpp:549-556, Cache.cpp:451-628) ------------------------------------------------
 * A state is a byte count published at a complete KV block, disposable (checkpoint) or ordinary, in use while an
 * unfinished request resumes from it, pinned while a restore reads it. rk_cache_evict_one is Cache::evictOne:
 * checkpoints first (not in a page scan), then KV leaves no state needs, then ordinary states and the leaves under
 * them by shared recency, states in use and their KV last and only up_to_in_use; out[4] = made progress, pending,
 * evicted a state, state bytes freed. rk_cache_reclaim_one_state is Cache::reclaimOneState (1 = a state went).
 * rk_cache_state_info out[7] = contains, ordinary, in use, bytes, KV needed by a state, KV needed by a state in use,
 * has a RAM copy;
 * rk_cache_state_summary out[4] = states, resident bytes, evictable states, resume point.
 * rk_cache_lookup_state is the lookup a hybrid model's admission makes (Cache::lookup, Cache.cpp:236-272; CacheLookup,
 * Cache.hpp:20-36): the chain as rk_cache_lookup, out[5] = KV boundary in tokens, the deepest state's block on the
 * chain (0 = none; it comes back pinned, as the reference's lease pins it: rk_cache_state_pin(block, 0) when the
 * restore is done), the boundary the request resumes from, the junction boundary (the matched KV ends at a branch
 * point past the state and another branch holds a state below it: a state materialised there serves both), and
 * whether a matched block past the state once held a reusable state that is gone. `record` != 0 counts the lookup
 * (Cache::recordLookup); rk_cache_lookup_counters out[4] = KV tokens hit, lazy junctions, lost-state misses, pages
 * hashed by scheduling probes.
 * rk_cache_probe_* is the scheduling probe (CacheProbe, Cache.hpp:38-52; Cache::probe / Cache::refresh,
 * Cache.cpp:210-234): what a scheduler keeps per waiting request between admission passes. It pins nothing, touches no
 * recency and counts no hit. While the block graph's generation stands still (no new block, adopted record, poisoning
 * or erase) a refresh hashes nothing; after a change the chain is cut at its first block that no longer matches and
 * only the pages past the cut are hashed. rk_cache_probe_info out[2] = cached tokens (up to the deepest state on the
 * matched chain; looked up again on every refresh), matched blocks. rk_cache_lookup_state given a current probe of the
 * same cache reuses its chain; a stale probe or another cache's is ignored there, and another cache's is refused by
 * rk_cache_probe_refresh (RK_ERR_INVALID). */
int64_t rk_cache_block_at(void *cache, uint64_t request, uint32_t tokens);
int rk_cache_state_publish(void *cache, uint64_t block, uint64_t bytes, int checkpoint);
/* A state whose only copy the model stores elsewhere (StateCache::publishStateToDisk, StateCache.cpp:189-214): it costs
 * no RAM and is no reclaim candidate, and the KV it restores through stays worth a tier copy. Published once per block. */
int rk_cache_state_publish_stored(void *cache, uint64_t block, uint64_t bytes, int checkpoint);
int rk_cache_state_use(void *cache, uint64_t block, int use);
int rk_cache_state_pin(void *cache, uint64_t block, int pin);
int rk_cache_state_info(void *cache, uint64_t block, uint64_t *out);
int rk_cache_state_summary(void *cache, uint64_t *out);
int rk_cache_evict_one(void *cache, int up_to_in_use, int keep_resume_point, int pages_only, uint64_t *out);
/* Cache::reclaimOne with its CacheReclaimMode (Cache.cpp:436-449): memory returns as whole extents. mode 0 (release
 * extents): an empty extent goes as it is, else scattered free pages are gathered until they fill one and that one
 * goes, else one victim is evicted and the extent it emptied goes with it; 1 (keep extents): evict only; 2 (reuse
* pages): evict in a page scan. keep_runway leaves the one empty extent a pass keeps. out[4] = made progress, pending,
 * evicted a state, bytes of the extents returned. rk_cache_evict_all is Cache::evictAll (Cache.cpp:423-434):
 * out[2] = made progress, extent bytes returned. */
int rk_cache_reclaim_step(void *cache, int mode, int up_to_in_use, int keep_resume_point, int keep_runway, uint64_t *out);
int rk_cache_evict_all(void *cache, uint64_t *out);
int rk_cache_reclaim_one_state(void *cache, int checkpoints_only, uint64_t for_block);
int64_t rk_cache_lookup_state(void *cache, const uint32_t *prompt, uint32_t prompt_tokens, uint64_t *blocks_out, uint32_t capacity,
                              uint64_t *out, int record, const void *probe, const rk_image_span *images, uint32_t image_count);
int rk_cache_lookup_counters(void *cache, uint64_t *out);
void *rk_cache_probe_create(void *cache, const uint32_t *prompt, uint32_t prompt_tokens, const rk_image_span *images, uint32_t image_count);
int rk_cache_probe_refresh(void *cache, void *probe, const uint32_t *prompt, uint32_t prompt_tokens, const rk_image_span *images,
                           uint32_t image_count);
int rk_cache_probe_info(const void *probe, uint64_t *out);
void rk_cache_probe_destroy(void *probe);

/* ---- plans -------------------------------------------------------------------------------------- */
/* names: "split\nreduce\nstore"; out[16] = splits, lane splits of the first four lanes, splitGroups xyz,
 * reduceGroups xyz, partialsBytes, statisticsBytes, rowCapacity, streamingDecode, tensorCoreWindow.
 * row_capacity 0 = 8 (chain) / 16 (tree). `ctas` = CTAs the B200 kernels may fill (0 = the current device's
 * SM count; without a device the plan is the reference's: PagedAttention::verifyPlan, PagedAttention.cpp:331-381). */
int rk_plan_verify(uint32_t lanes, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                   uint32_t format, const uint32_t *history, int tree, uint32_t row_capacity, uint32_t ctas,
                   char *names, size_t names_bytes, uint64_t *out);
/* Split count of one lane for the tcgen05 window kernel (new here): (lanes x kv_heads x splits) CTAs fill `ctas`
 * SMs once (0 = the current device's), whole 64-token groups per split. Negative status on error. */
int rk_plan_window_splits(uint32_t lanes, uint32_t kv_heads, uint32_t visible_tokens, uint32_t ctas);
/* out[10] = rows, splits, splitGroups xyz, reduceGroups xyz, partialsBytes, statisticsBytes */
int rk_plan_prefill(uint32_t rows, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                    uint32_t format, char *names, size_t names_bytes, uint64_t *out);
/* out[4] = verify partials, verify statistics, prefill partials, prefill statistics */
int rk_plan_workspaces(uint32_t lanes, uint32_t max_rows, uint32_t query_heads, uint32_t layers, uint32_t kv_heads,
                       uint32_t head_dim, uint32_t format, uint64_t *out);
/* ---- the operator's encoders -------------------------------------------------------------------------
 * ops::PagedAttention::addPrefillStore / addPrefill / addVerify / addVerifyTreeCompact
 * (runtime/ops/PagedAttention.cpp:399-573; declared PagedAttention.hpp:262-324). The reference appends dispatches
 * to a command graph; here a call launches on `stream`. Every check the reference makes before it encodes
 * (PagedAttention.cpp:407-408,448-455,474-478: parameter blocks, plan rows, scratch sizes, aliasing of queries and
 * output, missing tree masks) happens before the FIRST launch and returns RK_ERR_INVALID with the reference's
 * text in rk_last_error(): a refused call has launched nothing (the reference tests that a rejected call never
 * "partially encoded a graph", dev/tests/engine/paged_attention_plan_test.mm:748-761).
 * A plan handle holds PagedAttention::verifyPlan / prefillPlan for one batch shape; rk_op_plan_workspace gives
 * out[6] = partials bytes, statistics bytes, splits, row capacity (verify) or rows (prefill), bit 0 streaming
 * decode | bit 1 tcgen05 window, descriptor bytes of the streaming decode. */
typedef struct rk_verify_buffers {
  void *chunk_keys, *chunk_values, *queries, *output;
  float *partials, *statistics;
  uint32_t *descriptors;                    /* streaming decode only (rk_decode_plan's descriptor bytes, zeroed once) */
  uint32_t *status;                         /* tcgen05 window kernel only: one zeroed device word */
  const rk_page_entry *const *page_tables; /* device array, one table address per lane */
  const uint32_t *tree_masks;
  uint64_t partials_bytes, statistics_bytes; /* sizes of the scratch actually bound */
} rk_verify_buffers;
void *rk_op_verify_plan(uint32_t lanes, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                        uint32_t format, const uint32_t *history, int tree, uint32_t row_capacity, uint32_t ctas);
void *rk_op_prefill_plan(uint32_t rows, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                         uint32_t format);
void rk_op_plan_destroy(void *plan);
int rk_op_plan_workspace(const void *plan, uint64_t *out);
uint32_t rk_op_plan_lane_splits(const void *plan, uint32_t lane);
int rk_op_add_prefill_store(void *stream, rk_kv_layer layer, const void *chunk_keys, const void *chunk_values,
                            const rk_page_entry *table, const rk_chunk_params *params, uint32_t layers,
                            uint32_t kv_heads, uint32_t head_dim, uint32_t format);
int rk_op_add_prefill(void *stream, rk_kv_layer layer, const void *queries, void *output, float *partials,
                      float *statistics, uint64_t partials_bytes, uint64_t statistics_bytes,
                      const rk_page_entry *table, const rk_chunk_params *chunk, const void *plan, const void *window,
                      uint32_t *status);
int rk_op_add_verify(void *stream, rk_kv_layer layer, const rk_verify_buffers *buffers,
                     const rk_chunk_params *device_chunks, const rk_verify_params *device_attention, const void *plan,
                     const void *window);
int rk_op_add_verify_tree_compact(void *stream, rk_kv_layer layer, const rk_page_entry *const *page_tables,
                                  const uint32_t *retained_path, const uint32_t *retained,
                                  const rk_chunk_params *device_chunks, uint32_t lanes, uint32_t layers,
                                  uint32_t kv_heads, uint32_t head_dim, uint32_t format);
/* Empty string when valid, else the reference's tag (PagedAttention.hpp:75-95). */
const char *rk_chunk_validation_error(uint32_t committed, uint32_t tokens, uint32_t stride, uint32_t entries);

#ifdef __cplusplus
}
#endif
#endif /* RICHKV_HOST_H */
