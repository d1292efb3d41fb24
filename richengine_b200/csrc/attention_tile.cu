// attention_tile.cu — the general split-KV paged attention tile and its
// fixed-order reduce, for every row count (1..16 rows per lane), every KV
// format, causal chains and tree masks, verify batches and prefill chunks.
//
// Semantics follow the reference's tile and merge:
//   runtime/metal/kernels/common/paged_attention_tile.h:85-189   (scale fold, admission, online softmax)
//   runtime/metal/kernels/common/paged_attention_tile.h:208-349  (page loop, split partition, partial layout)
//   runtime/metal/kernels/common/paged_attention_tile.h:362-417  (merge in split order)
//   runtime/metal/kernels/decode/paged_attention.metal:23-131,198-263   (verify placement)
//   runtime/metal/kernels/prefill/paged_attention.metal:7-67            (prefill placement)
//   runtime/metal/kernels/common/paged_attention_fp8_tile.h:34-124      (fp16 query staging for fp8)
// This tile keeps probabilities and accumulators in fp32 (the reference rounds
// P*vscale to bf16 before P.V); it is the correctness carrier for shapes the
// specialised kernels (decode_attention.cu, verify_attention.cu) do not take.
#include "common.cuh"

#include <cuda_fp16.h>

namespace rk {
namespace {

constexpr uint32_t kThreads = 256;
constexpr uint32_t kKeyPitch = 260; // floats per dequantized key row (conflict-free float4 reads)

struct TileJob {
  const uint16_t *queries; // [rows][group][D] bf16 of this tile
  const rk_page_entry *table;
  const uint32_t *row_masks; // null = causal chain
  rk_kv_layer layer;
  uint32_t kv_head, committed, active_rows, splits, split;
  uint64_t slot;
  float score_scale;
};

template <uint32_t Format, uint32_t KvHeads, uint32_t Group, uint32_t Rows, uint32_t HeadDim>
__device__ void run_tile(const TileJob &job, float *__restrict__ partials, float *__restrict__ statistics,
                         float *shared) {
  static_assert(HeadDim == 256 && kThreads == HeadDim, "one thread per output dimension");
  using Geometry = PageGeometry<Format, KvHeads, HeadDim>;
  constexpr uint32_t M = Rows * Group, N = kPageTokens, D = HeadDim;
  constexpr uint32_t kRowsPerWarp = (M + 7) / 8;
  // shared: queries[M][D] | keys[N][kKeyPitch] | raw values | P[M][N] | row_max[M] row_sum[M] prev[M] | scales
  float *q_s = shared;
  float *k_s = q_s + M * D;
  uint8_t *v_raw = reinterpret_cast<uint8_t *>(k_s + N * kKeyPitch);
  float *p_s = reinterpret_cast<float *>(v_raw + Geometry::kHeadDataBytes);
  float *row_max = p_s + M * N;
  float *row_sum = row_max + M;
  float *previous = row_sum + M;
  float *vscale_s = previous + M;
  __shared__ int rescale_flag;

  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t visible = job.committed + job.active_rows;
  const uint32_t pages = rk_pages_for(visible);
  const uint32_t per_split = rk_pages_per_split(pages, job.splits);
  const uint32_t page_begin = job.split * per_split;
  if (page_begin >= pages) return; // a split without pages writes nothing
  const uint32_t page_end = min(pages, page_begin + per_split);
  const float score_scale = rk_score_scale(job.score_scale, D);

  for (uint32_t i = tid; i < M * D; i += kThreads) {
    float v = i < job.active_rows * Group * D ? bf16_bits_to_float(job.queries[i]) : 0.0f;
    if (Format == RK_FORMAT_FP8E4M3) v = __half2float(__float2half_rn(v)); // fp16 query staging
    q_s[i] = v;
  }
  for (uint32_t i = tid; i < M; i += kThreads) { row_max[i] = -INFINITY; row_sum[i] = 0.0f; }
  float acc[M];
#pragma unroll
  for (uint32_t m = 0; m < M; ++m) acc[m] = 0.0f;
  __syncthreads();

  for (uint32_t page = page_begin; page < page_end; ++page) {
    const PageSlabs slabs = Geometry::slabs(job.table[page], job.layer, job.kv_head);
    // Dequantized key codes (unscaled) -> shared, raw value slab -> shared.
    for (uint32_t i = tid; i < N * D; i += kThreads)
      k_s[(i / D) * kKeyPitch + (i % D)] = decode_element<Format>(slabs.keys, i);
    {
      const uint4 *source = reinterpret_cast<const uint4 *>(slabs.values);
      uint4 *target = reinterpret_cast<uint4 *>(v_raw);
      for (uint32_t i = tid; i < Geometry::kHeadDataBytes / 16; i += kThreads) target[i] = source[i];
    }
    if (tid < N) vscale_s[tid] = Geometry::kQuantized ? slabs.value_scales[tid] : 1.0f;
    if (tid == 0) rescale_flag = 0;
    __syncthreads();

    // Scores: warp w owns fused rows w, w+8, ...; lane = token of the page.
    float score[kRowsPerWarp];
#pragma unroll
    for (uint32_t r = 0; r < kRowsPerWarp; ++r) score[r] = 0.0f;
    for (uint32_t d = 0; d < D; d += 4) {
      const float4 k = *reinterpret_cast<const float4 *>(&k_s[lane * kKeyPitch + d]);
#pragma unroll
      for (uint32_t r = 0; r < kRowsPerWarp; ++r) {
        const uint32_t m = warp + 8 * r;
        if (m < M) {
          const float4 q = *reinterpret_cast<const float4 *>(&q_s[m * D + d]);
          score[r] = fmaf(q.x, k.x, fmaf(q.y, k.y, fmaf(q.z, k.z, fmaf(q.w, k.w, score[r]))));
        }
      }
    }
    const float key_scale = Geometry::kQuantized ? slabs.key_scales[lane] : 1.0f;
    const uint32_t token = page * N + lane;
#pragma unroll
    for (uint32_t r = 0; r < kRowsPerWarp; ++r) {
      const uint32_t m = warp + 8 * r;
      if (m >= M) continue;
      const uint32_t query_row = m / Group;
      bool admit;
      if (!job.row_masks) {
        const uint32_t causal_end = job.committed + min(query_row, job.active_rows - 1) + 1;
        admit = token < min(visible, causal_end);
      } else {
        admit = token < job.committed ||
                (token < visible && ((job.row_masks[query_row] >> (token - job.committed)) & 1u));
      }
      const float s = admit ? score[r] * key_scale * score_scale : -INFINITY;
      const float tile_max = warp_max(s);
      const float old_max = row_max[m];
      const float new_max = fmaxf(old_max, tile_max);
      const float prob = admit ? expf(s - new_max) : 0.0f;
      const float tile_sum = warp_sum(prob);
      // Masked tokens stay exactly zero whatever their stored scale holds.
      p_s[m * N + lane] = admit ? prob * vscale_s[lane] : 0.0f;
      if (lane == 0) {
        const float scale = (new_max == -INFINITY || new_max == old_max) ? 1.0f : expf(old_max - new_max);
        previous[m] = scale;
        row_sum[m] = row_sum[m] * scale + tile_sum;
        row_max[m] = new_max;
        if (scale != 1.0f) rescale_flag = 1;
      }
    }
    __syncthreads();
    if (rescale_flag) {
#pragma unroll
      for (uint32_t m = 0; m < M; ++m) acc[m] *= previous[m];
    }
    // O += P.V: thread tid owns output dimension tid.
    for (uint32_t t = 0; t < N; ++t) {
      float v;
      if (Format == RK_FORMAT_INT4)
        v = decode_element<Format>(v_raw, t * D + tid); // token-major nibbles
      else
        v = decode_element<Format>(v_raw, tid * N + t); // dimension-major
#pragma unroll
      for (uint32_t m = 0; m < M; ++m) {
        const float p = p_s[m * N + t];
        // 0 * (non-finite stale value) must not poison the sum (bf16 pages).
        acc[m] = p != 0.0f ? fmaf(p, v, acc[m]) : acc[m];
      }
    }
    __syncthreads();
  }

  float *out = partials + job.slot * M * D;
#pragma unroll
  for (uint32_t m = 0; m < M; ++m) out[m * D + tid] = acc[m];
  if (tid < M) {
    statistics[(job.slot * M + tid) * 2] = row_max[tid];
    statistics[(job.slot * M + tid) * 2 + 1] = row_sum[tid];
  }
}

template <uint32_t Format, uint32_t KvHeads, uint32_t Group, uint32_t Rows, uint32_t HeadDim>
constexpr size_t tile_shared_bytes() {
  using Geometry = PageGeometry<Format, KvHeads, HeadDim>;
  constexpr uint32_t M = Rows * Group;
  return sizeof(float) * (M * HeadDim + kPageTokens * kKeyPitch + M * kPageTokens + 3 * M + kPageTokens) +
         Geometry::kHeadDataBytes;
}

// Verify: grid (kv_heads, splits, lanes); queries [lane][kv_head][32][group][D].
template <uint32_t Format, uint32_t KvHeads, uint32_t Group, uint32_t Rows, uint32_t HeadDim>
__global__ void __launch_bounds__(kThreads)
verify_split_kernel(const uint16_t *__restrict__ queries, float *__restrict__ partials,
                    float *__restrict__ statistics, const rk_page_entry *const *__restrict__ tables,
                    const uint32_t *__restrict__ row_masks, const rk_verify_params *__restrict__ lane_params,
                    rk_kv_layer layer) {
  extern __shared__ __align__(16) float shared[];
  const uint32_t kv_head = blockIdx.x, split = blockIdx.y, lane_index = blockIdx.z;
  rk_verify_params p = lane_params[lane_index];
  if (layer.extent_pages) p.kv = layer;
  if (!rk_verify_contract_valid(&p) || p.row_capacity != Rows || split >= p.split_count) return;
  TileJob job;
  job.queries = queries + (uint64_t(lane_index) * KvHeads + kv_head) * (uint64_t(RK_VERIFY_CHUNK_STRIDE) * Group * HeadDim);
  job.table = tables[lane_index];
  job.row_masks = row_masks ? row_masks + uint64_t(lane_index) * p.row_capacity : nullptr;
  job.layer = p.kv;
  job.kv_head = kv_head;
  job.committed = p.committed_tokens;
  job.active_rows = p.active_rows;
  job.splits = p.split_count;
  job.split = split;
  job.slot = (uint64_t(lane_index) * KvHeads + kv_head) * p.slot_splits + split;
  job.score_scale = p.score_scale;
  run_tile<Format, KvHeads, Group, Rows, HeadDim>(job, partials, statistics, shared);
}

// Prefill: grid (kv_heads, tiles, splits); queries [kv_head][stride][group][D], 8-row tiles.
template <uint32_t Format, uint32_t KvHeads, uint32_t Group, uint32_t HeadDim>
__global__ void __launch_bounds__(kThreads)
prefill_split_kernel(const uint16_t *__restrict__ queries, float *__restrict__ partials,
                     float *__restrict__ statistics, const rk_page_entry *__restrict__ table,
                     rk_prefill_params p) {
  extern __shared__ __align__(16) float shared[];
  const uint32_t kv_head = blockIdx.x, tile = blockIdx.y, split = blockIdx.z;
  const uint32_t tile_start = tile * RK_PREFILL_TILE_ROWS;
  if (!rk_prefill_contract_valid(&p) || split >= p.split_count || tile_start >= p.rows) return;
  TileJob job;
  job.queries = queries + (uint64_t(kv_head) * p.chunk_stride + tile_start) * Group * HeadDim;
  job.table = table;
  job.row_masks = nullptr;
  job.layer = p.kv;
  job.kv_head = kv_head;
  job.committed = p.committed_tokens + tile_start;
  job.active_rows = min(RK_PREFILL_TILE_ROWS, p.rows - tile_start);
  job.splits = p.split_count;
  job.split = split;
  job.slot = (uint64_t(tile) * KvHeads + kv_head) * p.split_count + split;
  job.score_scale = p.score_scale;
  run_tile<Format, KvHeads, Group, RK_PREFILL_TILE_ROWS, HeadDim>(job, partials, statistics, shared);
}

// One fused row: merge the written splits in split order and store bf16
// (paged_attention_tile.h:362-417). Block = D threads.
// Returns the bf16 bits of the element this thread reduced (0 for rows past the live rows); a null
// `tile_output` skips the store of the attention rows.
template <uint32_t HeadDim>
__device__ uint16_t reduce_row(const float *__restrict__ partials, const float *__restrict__ statistics,
                           uint16_t *__restrict__ tile_output, float *__restrict__ tile_output_f32,
                           uint32_t committed, uint32_t active_rows, uint32_t group, uint32_t M,
                           uint32_t splits, uint64_t head_slot, uint32_t fused_row) {
  constexpr uint32_t D = HeadDim;
  __shared__ float weights[RK_VERIFY_MAX_SPLITS];
  __shared__ float warp_values[D / 32];
  const uint32_t tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
  if (fused_row / group >= active_rows) { // rows past the live rows are zeros
    if (tile_output) tile_output[fused_row * D + tid] = 0;
    if (tile_output_f32) tile_output_f32[fused_row * D + tid] = 0.0f;
    return 0;
  }
  const uint32_t pages = rk_pages_for(committed + active_rows);
  const uint32_t per_split = rk_pages_per_split(pages, splits);
  const uint32_t written = (pages + per_split - 1) / per_split;
  float maximum = -INFINITY;
  for (uint32_t s = tid; s < written; s += D)
    maximum = fmaxf(maximum, statistics[((head_slot + s) * M + fused_row) * 2]);
  maximum = warp_max(maximum);
  if (lane == 0) warp_values[warp] = maximum;
  __syncthreads();
  float row_maximum = -INFINITY;
  for (uint32_t w = 0; w < D / 32; ++w) row_maximum = fmaxf(row_maximum, warp_values[w]);
  for (uint32_t s = tid; s < written; s += D)
    weights[s] = expf(statistics[((head_slot + s) * M + fused_row) * 2] - row_maximum);
  __syncthreads();
  float numerator = 0.0f, denominator = 0.0f;
  for (uint32_t s = 0; s < written; ++s) { // sequential, in split order
    const float weight = weights[s];
    numerator += weight * partials[((head_slot + s) * M + fused_row) * D + tid];
    denominator += weight * statistics[((head_slot + s) * M + fused_row) * 2 + 1];
  }
  const float value = denominator > 0.0f ? numerator / denominator : 0.0f;
  const uint16_t bits = float_to_bf16_bits(value);
  if (tile_output) tile_output[fused_row * D + tid] = bits;
  if (tile_output_f32) tile_output_f32[fused_row * D + tid] = value;
  return bits;
}

// The logistic sigmoid of the reference's kernels: 1 / (1 + 2^(-log2(e) x)) (kernels/common/activation.h:14-16).
__device__ __forceinline__ float gate_sigmoid(float x) { return 1.0f / (1.0f + exp2f(-1.44269504089f * x)); }

// grid (kv_heads, M, lanes), D threads.
template <uint32_t KvHeads, uint32_t HeadDim>
__global__ void __launch_bounds__(HeadDim)
verify_reduce_kernel(const float *__restrict__ partials, const float *__restrict__ statistics,
                     uint16_t *__restrict__ output, float *__restrict__ output_f32,
                     const rk_verify_params *__restrict__ lane_params, uint32_t group,
                     const uint16_t *__restrict__ packed_qkv, uint16_t *__restrict__ hidden) {
  const uint32_t kv_head = blockIdx.x, fused_row = blockIdx.y, lane_index = blockIdx.z;
  rk_verify_params p = lane_params[lane_index];
  p.kv.extent_pages = 1; // placement plays no part in the merge
  const uint32_t M = p.row_capacity * group;
  if (!rk_verify_contract_valid(&p) || fused_row >= M) return;
  const uint64_t tile = (uint64_t(lane_index) * KvHeads + kv_head) * (uint64_t(RK_VERIFY_CHUNK_STRIDE) * group * HeadDim);
  const uint16_t bits = reduce_row<HeadDim>(partials, statistics, output ? output + tile : nullptr, output_f32 ? output_f32 + tile : nullptr,
                                            p.committed_tokens, p.active_rows, group, M, p.split_count,
                                            (uint64_t(lane_index) * KvHeads + kv_head) * p.slot_splits, fused_row);
  if (hidden) {
    // The epilogue of the out-projection's input (decode/paged_attention.metal:273-413): the row leaves in the
    // [lane][row][query head][dim] layout, scaled by the sigmoid of its gate where the packed QKV rows
    // ([q | gate] per query head, then k and v per KV head) are given, copied otherwise.
    const uint32_t query_heads = KvHeads * group, row = fused_row / group, query_head = kv_head * group + fused_row % group;
    const uint64_t target = ((uint64_t(lane_index) * p.row_capacity + row) * query_heads + query_head) * HeadDim + threadIdx.x;
    if (packed_qkv) {
      const uint64_t packed_stride = 2ull * query_heads * HeadDim + 2ull * KvHeads * HeadDim;
      const float gate = bf16_bits_to_float(packed_qkv[(uint64_t(lane_index) * p.row_capacity + row) * packed_stride +
                                                       uint64_t(query_head) * 2 * HeadDim + HeadDim + threadIdx.x]);
      hidden[target] = float_to_bf16_bits(bf16_bits_to_float(bits) * gate_sigmoid(gate));
    } else {
      hidden[target] = bits;
    }
  }
}

// grid (kv_heads, 8*group, tiles), D threads.
template <uint32_t KvHeads, uint32_t HeadDim>
__global__ void __launch_bounds__(HeadDim)
prefill_reduce_kernel(const float *__restrict__ partials, const float *__restrict__ statistics,
                      uint16_t *__restrict__ output, float *__restrict__ output_f32, rk_prefill_params p,
                      uint32_t group) {
  const uint32_t kv_head = blockIdx.x, fused_row = blockIdx.y, tile = blockIdx.z;
  const uint32_t tile_start = tile * RK_PREFILL_TILE_ROWS, M = RK_PREFILL_TILE_ROWS * group;
  p.kv.extent_pages = 1;
  if (!rk_prefill_contract_valid(&p) || fused_row >= M || tile_start >= p.rows) return;
  const uint32_t active_rows = min(RK_PREFILL_TILE_ROWS, p.rows - tile_start);
  const uint64_t offset = (uint64_t(kv_head) * p.chunk_stride + tile_start) * group * HeadDim;
  reduce_row<HeadDim>(partials, statistics, output + offset, output_f32 ? output_f32 + offset : nullptr,
                      p.committed_tokens + tile_start, active_rows, group, M, p.split_count,
                      (uint64_t(tile) * KvHeads + kv_head) * p.split_count, fused_row);
}

template <typename Kernel> int allow_shared(Kernel kernel, size_t bytes) {
  return cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)),
                     "cudaFuncSetAttribute(shared memory)");
}

template <uint32_t Format, uint32_t Rows>
int launch_verify_split(uint32_t lanes, uint32_t grid_splits, const void *queries, float *partials,
                        float *statistics, const rk_page_entry *const *tables, const uint32_t *row_masks,
                        const rk_verify_params *lane_params, rk_kv_layer layer, cudaStream_t stream) {
  auto kernel = verify_split_kernel<Format, 4, 6, Rows, 256>;
  constexpr size_t bytes = tile_shared_bytes<Format, 4, 6, Rows, 256>();
  if (int status = allow_shared(kernel, bytes)) return status;
  kernel<<<dim3(4, grid_splits, lanes), kThreads, bytes, stream>>>(
      static_cast<const uint16_t *>(queries), partials, statistics, tables, row_masks, lane_params, layer);
  return cuda_status(cudaGetLastError(), "verify split launch");
}

template <uint32_t Format>
int launch_verify_split_rows(uint32_t rows, uint32_t lanes, uint32_t grid_splits, const void *queries,
                             float *partials, float *statistics, const rk_page_entry *const *tables,
                             const uint32_t *row_masks, const rk_verify_params *lane_params,
                             rk_kv_layer layer, cudaStream_t stream) {
  switch (rows) {
  case 1:
    return launch_verify_split<Format, 1>(lanes, grid_splits, queries, partials, statistics, tables, row_masks, lane_params, layer, stream);
  case 8:
    return launch_verify_split<Format, 8>(lanes, grid_splits, queries, partials, statistics, tables, row_masks, lane_params, layer, stream);
  case 16:
    return launch_verify_split<Format, 16>(lanes, grid_splits, queries, partials, statistics, tables, row_masks, lane_params, layer, stream);
  default: return kUnsupported;
  }
}

template <uint32_t Format>
int launch_prefill_split(const void *queries, float *partials, float *statistics, const rk_page_entry *table,
                         const rk_prefill_params &p, cudaStream_t stream) {
  auto kernel = prefill_split_kernel<Format, 4, 6, 256>;
  constexpr size_t bytes = tile_shared_bytes<Format, 4, 6, RK_PREFILL_TILE_ROWS, 256>();
  if (int status = allow_shared(kernel, bytes)) return status;
  const uint32_t tiles = (p.rows + RK_PREFILL_TILE_ROWS - 1) / RK_PREFILL_TILE_ROWS;
  kernel<<<dim3(4, tiles, p.split_count), kThreads, bytes, stream>>>(
      static_cast<const uint16_t *>(queries), partials, statistics, table, p);
  return cuda_status(cudaGetLastError(), "prefill split launch");
}

bool supported_geometry(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim) {
  return kv_heads == 4 && query_heads == 24 && head_dim == 256;
}

} // namespace
} // namespace rk

using namespace rk;

extern "C" int rk_attention_verify_split(uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                         uint32_t head_dim, uint32_t lanes, uint32_t row_capacity,
                                         uint32_t grid_splits, const void *queries, float *partials,
                                         float *statistics, const rk_page_entry *const *tables,
                                         const uint32_t *row_masks, const rk_verify_params *lane_params,
                                         rk_kv_layer layer, void *stream) {
  if (!supported_geometry(kv_heads, query_heads, head_dim)) {
    set_error("rk_attention_verify_split: only 4 KV heads x 24 query heads x 256 is built");
    return kUnsupported;
  }
  if (!lanes || !grid_splits || grid_splits > RK_VERIFY_MAX_SPLITS || !queries || !partials || !statistics ||
      !tables || !lane_params || !layer.extent_pages) {
    set_error("rk_attention_verify_split: invalid arguments");
    return kInvalid;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (format) {
  case RK_FORMAT_INT8:
    return launch_verify_split_rows<RK_FORMAT_INT8>(row_capacity, lanes, grid_splits, queries, partials, statistics, tables, row_masks, lane_params, layer, s);
  case RK_FORMAT_INT4:
    return launch_verify_split_rows<RK_FORMAT_INT4>(row_capacity, lanes, grid_splits, queries, partials, statistics, tables, row_masks, lane_params, layer, s);
  case RK_FORMAT_FP8E4M3:
    return launch_verify_split_rows<RK_FORMAT_FP8E4M3>(row_capacity, lanes, grid_splits, queries, partials, statistics, tables, row_masks, lane_params, layer, s);
  case RK_FORMAT_BF16:
    return launch_verify_split_rows<RK_FORMAT_BF16>(row_capacity, lanes, grid_splits, queries, partials, statistics, tables, row_masks, lane_params, layer, s);
  default: set_error("rk_attention_verify_split: unknown format"); return kInvalid;
  }
}

extern "C" int rk_attention_verify_reduce(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                                          uint32_t lanes, uint32_t row_capacity, const float *partials,
                                          const float *statistics, void *output, float *output_f32,
                                          const rk_verify_params *lane_params, void *stream) {
  if (!supported_geometry(kv_heads, query_heads, head_dim)) return kUnsupported;
  if (!lanes || !row_capacity || row_capacity > RK_TREE_NODES || !partials || !statistics || !output || !lane_params) {
    set_error("rk_attention_verify_reduce: invalid arguments");
    return kInvalid;
  }
  const uint32_t group = query_heads / kv_heads;
  verify_reduce_kernel<4, 256><<<dim3(kv_heads, row_capacity * group, lanes), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partials, statistics, static_cast<uint16_t *>(output), output_f32, lane_params, group, nullptr, nullptr);
  return cuda_status(cudaGetLastError(), "verify reduce launch");
}

// verify_attention_reduce_gate / verify_attention_reduce_gather (decode/paged_attention.metal:273-413; encoded by
// PagedAttention::addVerify when its gate buffers are bound, PagedAttention.hpp:299-311): the split merge that also
// writes the out-projection's input `hidden` [lane][row][query head][D] bf16 — the merged row times the sigmoid of
// its gate, read from `packed_qkv` [lane][row][ (q | gate) x query heads, k x KV heads, v x KV heads ], or the merged
// row itself when `packed_qkv` is null. `output` (the attention staging rows) may be null in the gather form.
extern "C" int rk_attention_verify_reduce_gate(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                                               uint32_t row_capacity, const float *partials, const float *statistics,
                                               void *output, const void *packed_qkv, void *hidden,
                                               const rk_verify_params *lane_params, void *stream) {
  if (!supported_geometry(kv_heads, query_heads, head_dim)) return kUnsupported;
  if (!lanes || !row_capacity || row_capacity > RK_TREE_NODES || !partials || !statistics || !hidden || !lane_params ||
      (packed_qkv && !output)) {
    set_error("rk_attention_verify_reduce_gate: invalid arguments");
    return kInvalid;
  }
  const uint32_t group = query_heads / kv_heads;
  verify_reduce_kernel<4, 256><<<dim3(kv_heads, row_capacity * group, lanes), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partials, statistics, static_cast<uint16_t *>(output), nullptr, lane_params, group,
      static_cast<const uint16_t *>(packed_qkv), static_cast<uint16_t *>(hidden));
  return cuda_status(cudaGetLastError(), "verify reduce-gate launch");
}

extern "C" int rk_attention_prefill_split(uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                          uint32_t head_dim, const void *queries, float *partials,
                                          float *statistics, const rk_page_entry *table,
                                          const rk_prefill_params *params, void *stream) {
  if (!supported_geometry(kv_heads, query_heads, head_dim)) return kUnsupported;
  if (!queries || !partials || !statistics || !table || !params || !rk_prefill_contract_valid(params)) {
    set_error("rk_attention_prefill_split: invalid arguments");
    return kInvalid;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (format) {
  case RK_FORMAT_INT8: return launch_prefill_split<RK_FORMAT_INT8>(queries, partials, statistics, table, *params, s);
  case RK_FORMAT_INT4: return launch_prefill_split<RK_FORMAT_INT4>(queries, partials, statistics, table, *params, s);
  case RK_FORMAT_FP8E4M3: return launch_prefill_split<RK_FORMAT_FP8E4M3>(queries, partials, statistics, table, *params, s);
  case RK_FORMAT_BF16: return launch_prefill_split<RK_FORMAT_BF16>(queries, partials, statistics, table, *params, s);
  default: return kInvalid;
  }
}

extern "C" int rk_attention_prefill_reduce(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                                           const float *partials, const float *statistics, void *output,
                                           float *output_f32, const rk_prefill_params *params, void *stream) {
  if (!supported_geometry(kv_heads, query_heads, head_dim)) return kUnsupported;
  if (!partials || !statistics || !output || !params || !rk_prefill_contract_valid(params)) {
    set_error("rk_attention_prefill_reduce: invalid arguments");
    return kInvalid;
  }
  const uint32_t group = query_heads / kv_heads;
  const uint32_t tiles = (params->rows + RK_PREFILL_TILE_ROWS - 1) / RK_PREFILL_TILE_ROWS;
  prefill_reduce_kernel<4, 256><<<dim3(kv_heads, RK_PREFILL_TILE_ROWS * group, tiles), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partials, statistics, static_cast<uint16_t *>(output), output_f32, *params, group);
  return cuda_status(cudaGetLastError(), "prefill reduce launch");
}
