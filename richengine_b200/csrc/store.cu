// store.cu — append-and-quantize of new K/V rows into their final page slots.
//
// Semantics follow the reference's store kernels:
//   runtime/metal/kernels/common/paged_store_row.h:47-147      (int8, int4, bf16 rows)
//   runtime/metal/kernels/common/paged_store_row_fp8.h:28-78   (fp8 e4m3 rows)
//   runtime/metal/kernels/decode/paged_attention_store.metal:3-45   (verify: many lanes)
//   runtime/metal/kernels/prefill/paged_attention_store.metal:7-27  (prefill: one chunk)
// The launch shape is this library's own: one 256-thread block stores a tile of
// up to 32 consecutive chunk rows of one (lane, KV head); a warp owns a row,
// reduces its absolute maximum with shuffles, quantizes with the reference's
// exact fp32 recipe (x*range, then /amax, round-to-nearest-even, clamp) and
// writes token-major rows as 16-byte stores. Dimension-major value slabs
// (int8, fp8, bf16) are written by one thread per dimension after the row
// maxima are known, packed into 32-bit words wherever four (two for bf16)
// consecutive tokens of one page are present.
#include "common.cuh"

namespace rk {
namespace {

constexpr uint32_t kTileRows = 32;
constexpr uint32_t kThreads = 256;

template <uint32_t Format, uint32_t KvHeads, uint32_t HeadDim>
__global__ void __launch_bounds__(kThreads)
store_rows_kernel(const uint16_t *__restrict__ chunk_keys, const uint16_t *__restrict__ chunk_values,
                  const rk_page_entry *const *__restrict__ tables, const rk_page_entry *single_table,
                  const rk_chunk_params *__restrict__ lane_params, rk_chunk_params single,
                  rk_kv_layer layer, uint64_t lane_stride, uint32_t verify_row_limit) {
  static_assert(HeadDim == 256, "one warp lane owns eight dimensions of a 256-wide row");
  // Launched as a programmatic dependent: wait for the preceding kernel's writes (the stagings may be its output, and
  // the pages may still be read by it), and let the next kernel of the stream be placed early.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  using Geometry = PageGeometry<Format, KvHeads, HeadDim>;
  constexpr bool kTokenMajorValues = Format == RK_FORMAT_INT4;
  constexpr uint32_t kPitch = HeadDim + 8; // halfwords per transposed value row (16-byte pad)
  __shared__ __align__(16) uint16_t value_tile[kTileRows * kPitch];
  __shared__ float value_amax[kTileRows];

  const uint32_t lane_index = blockIdx.z, head = blockIdx.y;
  rk_chunk_params p = lane_params ? lane_params[lane_index] : single;
  if (layer.extent_pages) p.kv = layer;
  // Invalid parameters leave memory untouched (paged_store_row.h:14-29).
  if (!rk_chunk_contract_valid(&p)) return;
  if (verify_row_limit && (p.chunk_tokens > verify_row_limit || p.chunk_stride != RK_VERIFY_CHUNK_STRIDE))
    return;
  const uint32_t row0 = blockIdx.x * kTileRows;
  if (row0 >= p.chunk_tokens) return;
  const uint32_t rows = min(kTileRows, p.chunk_tokens - row0);
  const rk_page_entry *table = tables ? tables[lane_index] : single_table;
  const uint32_t stride = p.chunk_stride;
  const uint16_t *key_rows = chunk_keys + lane_index * lane_stride + (uint64_t(head) * stride + row0) * HeadDim;
  const uint16_t *value_cols = chunk_values + lane_index * lane_stride + uint64_t(head) * HeadDim * stride + row0;

  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;

  // Transpose the tile's value columns [dim][row] into rows [row][dim].
  {
    const uint4 *source = reinterpret_cast<const uint4 *>(value_cols + uint64_t(tid) * stride);
#pragma unroll
    for (uint32_t chunk = 0; chunk < kTileRows / 8; ++chunk) {
      const uint4 v = __ldg(source + chunk);
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (uint32_t i = 0; i < 4; ++i) {
        value_tile[(chunk * 8 + 2 * i) * kPitch + tid] = uint16_t(words[i] & 0xffffu);
        value_tile[(chunk * 8 + 2 * i + 1) * kPitch + tid] = uint16_t(words[i] >> 16);
      }
    }
  }
  __syncthreads();

  for (uint32_t job = warp; job < 2 * rows; job += kThreads / 32) {
    const bool value_tensor = job >= rows;
    const uint32_t row = value_tensor ? job - rows : job;
    const uint4 raw = value_tensor
                          ? *reinterpret_cast<const uint4 *>(&value_tile[row * kPitch + lane * 8])
                          : __ldg(reinterpret_cast<const uint4 *>(key_rows + uint64_t(row) * HeadDim) + lane);
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
    float x[8];
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
      x[2 * i] = bf16_bits_to_float(words[i] & 0xffffu);
      x[2 * i + 1] = bf16_bits_to_float(words[i] >> 16);
    }
    const uint32_t token = p.committed_tokens + row0 + row;
    const PageSlabs slabs = Geometry::slabs(table[token / kPageTokens], p.kv, head);
    const uint32_t page_token = token % kPageTokens;

    if (Format == RK_FORMAT_BF16) {
      if (!value_tensor) // the 16 source bits of every element, untouched
        reinterpret_cast<uint4 *>(slabs.keys + uint64_t(page_token) * Geometry::kRowBytes)[lane] = raw;
      continue; // bf16 values are copied by the per-dimension pass below
    }
    float amax = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
    amax = warp_max(amax);
    if (lane == 0) {
      const float scale = amax == 0.0f ? 0.0f : __fdiv_rn(amax, Quantizer<Format == RK_FORMAT_BF16 ? RK_FORMAT_INT8 : Format>::kRange);
      (value_tensor ? slabs.value_scales : slabs.key_scales)[page_token] = scale;
      if (value_tensor) value_amax[row] = amax;
    }
    if (value_tensor && !kTokenMajorValues) continue;

    uint8_t *destination = (value_tensor ? slabs.values : slabs.keys) + uint64_t(page_token) * Geometry::kRowBytes;
    constexpr uint32_t F = Format == RK_FORMAT_BF16 ? RK_FORMAT_INT8 : Format;
    if (Format == RK_FORMAT_INT4) {
      uint32_t word = 0;
#pragma unroll
      for (uint32_t i = 0; i < 8; ++i) word |= encode<F>(x[i], amax) << (4 * i); // even dim = low nibble
      const uint32_t w1 = __shfl_down_sync(0xffffffffu, word, 1);
      const uint32_t w2 = __shfl_down_sync(0xffffffffu, word, 2);
      const uint32_t w3 = __shfl_down_sync(0xffffffffu, word, 3);
      if ((lane & 3u) == 0) reinterpret_cast<uint4 *>(destination)[lane / 4] = make_uint4(word, w1, w2, w3);
    } else {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (uint32_t i = 0; i < 4; ++i) {
        lo |= encode<F>(x[i], amax) << (8 * i);
        hi |= encode<F>(x[4 + i], amax) << (8 * i);
      }
      const uint32_t lo1 = __shfl_down_sync(0xffffffffu, lo, 1);
      const uint32_t hi1 = __shfl_down_sync(0xffffffffu, hi, 1);
      if ((lane & 1u) == 0) reinterpret_cast<uint4 *>(destination)[lane / 2] = make_uint4(lo, hi, lo1, hi1);
    }
  }

  if (kTokenMajorValues) return;
  __syncthreads();
  // Dimension-major values: thread `tid` owns dimension tid of this head.
  {
    constexpr uint32_t F = Format == RK_FORMAT_BF16 ? RK_FORMAT_INT8 : Format;
    constexpr uint32_t kElementBytes = Format == RK_FORMAT_BF16 ? 2 : 1;
    constexpr uint32_t kGroup = 4 / kElementBytes; // elements per 32-bit store
    uint32_t row = 0;
    while (row < rows) {
      const uint32_t token = p.committed_tokens + row0 + row;
      const uint32_t page_token = token % kPageTokens;
      const uint32_t run = min(rows - row, kPageTokens - page_token); // rows left in this page
      const PageSlabs slabs = Geometry::slabs(table[token / kPageTokens], p.kv, head);
      uint8_t *base = slabs.values + (uint64_t(tid) * kPageTokens + page_token) * kElementBytes;
      uint32_t i = 0;
      while (i < run) {
        const bool aligned = ((page_token + i) % kGroup) == 0 && i + kGroup <= run;
        const uint32_t count = aligned ? kGroup : 1;
        uint32_t packed = 0;
        for (uint32_t j = 0; j < count; ++j) {
          const uint16_t bits = value_tile[(row + i + j) * kPitch + tid];
          const uint32_t code = Format == RK_FORMAT_BF16
                                    ? uint32_t(bits)
                                    : encode<F>(bf16_bits_to_float(bits), value_amax[row + i + j]);
          packed |= code << (8 * kElementBytes * j);
        }
        if (aligned)
          *reinterpret_cast<uint32_t *>(base + i * kElementBytes) = packed;
        else if (kElementBytes == 2)
          *reinterpret_cast<uint16_t *>(base + i * kElementBytes) = uint16_t(packed);
        else
          base[i] = uint8_t(packed);
        i += count;
      }
      row += run;
    }
  }
}

template <uint32_t Format>
int launch_store(uint32_t kv_heads, uint32_t head_dim, uint32_t lanes, uint32_t max_rows,
                 const void *keys, const void *values, const rk_page_entry *const *tables,
                 const rk_page_entry *single_table, const rk_chunk_params *lane_params,
                 rk_chunk_params single, rk_kv_layer layer, uint64_t lane_stride, uint32_t verify_limit,
                 cudaStream_t stream) {
  if (head_dim != 256) return kUnsupported;
  const dim3 grid((max_rows + kTileRows - 1) / kTileRows, kv_heads, lanes);
  auto run = [&](auto kernel) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = dim3(kThreads);
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&config, kernel, static_cast<const uint16_t *>(keys), static_cast<const uint16_t *>(values),
                                          tables, single_table, lane_params, single, layer, lane_stride, verify_limit),
                       "store launch");
  };
  switch (kv_heads) {
  case 4: return run(store_rows_kernel<Format, 4, 256>);
  case 2: return run(store_rows_kernel<Format, 2, 256>);
  default: return kUnsupported;
  }
}

int dispatch_store(uint32_t format, uint32_t kv_heads, uint32_t head_dim, uint32_t lanes, uint32_t max_rows,
                   const void *keys, const void *values, const rk_page_entry *const *tables,
                   const rk_page_entry *single_table, const rk_chunk_params *lane_params,
                   rk_chunk_params single, rk_kv_layer layer, uint64_t lane_stride, uint32_t verify_limit,
                   cudaStream_t stream) {
  switch (format) {
  case RK_FORMAT_INT8:
    return launch_store<RK_FORMAT_INT8>(kv_heads, head_dim, lanes, max_rows, keys, values, tables, single_table,
                                        lane_params, single, layer, lane_stride, verify_limit, stream);
  case RK_FORMAT_INT4:
    return launch_store<RK_FORMAT_INT4>(kv_heads, head_dim, lanes, max_rows, keys, values, tables, single_table,
                                        lane_params, single, layer, lane_stride, verify_limit, stream);
  case RK_FORMAT_FP8E4M3:
    return launch_store<RK_FORMAT_FP8E4M3>(kv_heads, head_dim, lanes, max_rows, keys, values, tables, single_table,
                                           lane_params, single, layer, lane_stride, verify_limit, stream);
  case RK_FORMAT_BF16:
    return launch_store<RK_FORMAT_BF16>(kv_heads, head_dim, lanes, max_rows, keys, values, tables, single_table,
                                        lane_params, single, layer, lane_stride, verify_limit, stream);
  default: return kInvalid;
  }
}

} // namespace
} // namespace rk

using namespace rk;

extern "C" int rk_store_verify(uint32_t format, uint32_t kv_heads, uint32_t head_dim, uint32_t lanes,
                               uint32_t max_rows, const void *chunk_keys, const void *chunk_values,
                               const rk_page_entry *const *tables, const rk_chunk_params *lane_params,
                               rk_kv_layer layer, void *stream) {
  if (!lanes || !max_rows || max_rows > RK_TREE_NODES || !chunk_keys || !chunk_values || !tables ||
      !lane_params || !layer.extent_pages) {
    set_error("rk_store_verify: invalid arguments");
    return kInvalid;
  }
  const uint64_t lane_stride = uint64_t(kv_heads) * RK_VERIFY_CHUNK_STRIDE * head_dim;
  return dispatch_store(format, kv_heads, head_dim, lanes, max_rows, chunk_keys, chunk_values, tables, nullptr,
                        lane_params, rk_chunk_params{}, layer, lane_stride, RK_TREE_NODES,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int rk_store_chunk(uint32_t format, uint32_t kv_heads, uint32_t head_dim, const void *chunk_keys,
                              const void *chunk_values, const rk_page_entry *table,
                              const rk_chunk_params *params, void *stream) {
  if (!chunk_keys || !chunk_values || !table || !params) {
    set_error("rk_store_chunk: invalid arguments");
    return kInvalid;
  }
  // Host-side validation mirrors chunkedPrefillValidationError
  // (runtime/ops/PagedAttention.hpp:75-95): nothing is launched on failure.
  if (!rk_chunk_contract_valid(params)) {
    set_error("rk_store_chunk: chunk parameters violate the store contract");
    return kInvalid;
  }
  return dispatch_store(format, kv_heads, head_dim, 1, params->chunk_tokens, chunk_keys, chunk_values, nullptr,
                        table, nullptr, *params, rk_kv_layer{0, 0}, 0, 0, static_cast<cudaStream_t>(stream));
}
