// qkv_prepare.cu — the step before the paged KV path: the packed projection rows become what the store and the
// attention read.
//
// Semantics: runtime/metal/kernels/common/attention_qkv_prepare.h:13-83 (full_qkv_storage_phase) as instantiated by
// runtime/metal/kernels/decode/attention_qkv.metal:6-60 for 24 query heads x 4 KV heads x 256: per (lane, row, head)
//   q, k: per-head RMS norm (eps 1e-6) times the norm weight (bf16 or fp32), rounded to bf16, then rotary on the
//         first 2 x 32 dims with the row's cos / sin; v: the 16 source bits;
//   queries [lane][kv][32][group][D], keys [lane][kv][32][D], values [lane][kv][D][32] (the stagings of the store).
// One 256-thread block per (row, head), one thread per dim, as there. Every product and sum is rounded on its own
// (_rn intrinsics, no fused multiply-add); the sum of squares is reduced per warp by an xor butterfly 16, 8, 4, 2, 1
// and the eight warp sums are then added in order by every thread: the CPU checker does exactly the same.
//
// The fused form (the reference's own open item: "merge the page store into it") quantises the key and value rows
// straight into their page slots instead of writing the two stagings: one HBM round trip of bf16 rows and one
// launch per layer less. Its pages are bit-identical to prepare + rk_store_verify.
#include "common.cuh"

namespace rk {
namespace {

constexpr uint32_t kD = 256, kRotaryPairs = 32, kStride = RK_VERIFY_CHUNK_STRIDE;

struct PrepareArgs {
  const uint16_t *packed_qkv; // [lane][rows][(q | gate) x Hq, k x Hkv, v x Hkv]
  const void *q_norm, *k_norm;
  const float *rope_cos, *rope_sin; // [lane][rows][32]
  uint16_t *queries, *chunk_keys, *chunk_values;
  float eps;
  uint32_t rows, kv_heads, query_heads;
  // fused form
  const rk_page_entry *const *tables;
  const rk_chunk_params *lane_params;
  rk_kv_layer layer;
};

__device__ __forceinline__ float block_sum_of_squares(float square, float *warp_sums) {
  float v = square;
#pragma unroll
  for (uint32_t offset = 16; offset; offset >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, offset));
  if ((threadIdx.x & 31u) == 0) warp_sums[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (uint32_t w = 0; w < kD / 32; ++w) total = __fadd_rn(total, warp_sums[w]);
  return total;
}

__device__ __forceinline__ float block_max(float value, float *warp_values) {
  value = warp_max(value);
  __syncthreads(); // the caller may still be reading warp_values of an earlier reduction
  if ((threadIdx.x & 31u) == 0) warp_values[threadIdx.x >> 5] = value;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (uint32_t w = 0; w < kD / 32; ++w) total = fmaxf(total, warp_values[w]);
  return total;
}

// One row of one tensor (K or V) of one head into its page slot: the store's recipe and placement
// (kernels/common/paged_store_row.h:47-147, paged_store_row_fp8.h:28-78), one thread per dim.
template <uint32_t Format>
__device__ void store_page_row(uint16_t bits, bool value_tensor, const PageSlabs &slabs, uint32_t page_token, float *scratch) {
  using Geometry = PageGeometry<Format, 4, kD>;
  const uint32_t d = threadIdx.x;
  if (Format == RK_FORMAT_BF16) {
    uint16_t *base = reinterpret_cast<uint16_t *>(value_tensor ? slabs.values : slabs.keys);
    base[value_tensor ? d * kPageTokens + page_token : page_token * kD + d] = bits;
    return;
  }
  constexpr uint32_t F = Format == RK_FORMAT_BF16 ? RK_FORMAT_INT8 : Format;
  const float x = bf16_bits_to_float(bits);
  const float amax = block_max(fabsf(x), scratch);
  if (d == 0) (value_tensor ? slabs.value_scales : slabs.key_scales)[page_token] = amax == 0.0f ? 0.0f : __fdiv_rn(amax, Quantizer<F>::kRange);
  const uint32_t code = encode<F>(x, amax);
  if (Format == RK_FORMAT_INT4) { // token-major for both tensors, even dim in the low nibble
    const uint32_t neighbour = __shfl_down_sync(0xffffffffu, code, 1);
    if ((d & 1u) == 0) (value_tensor ? slabs.values : slabs.keys)[page_token * (kD / 2) + d / 2] = uint8_t(code | (neighbour << 4));
  } else if (value_tensor) {
    slabs.values[d * kPageTokens + page_token] = uint8_t(code);
  } else {
    slabs.keys[page_token * kD + d] = uint8_t(code);
  }
  (void)Geometry::kRowBytes;
}

// grid (rows * (query heads + KV heads), lanes); Format 0 = the unfused form (stagings only).
template <uint32_t Format, bool NormF32>
__global__ void __launch_bounds__(kD)
qkv_prepare_kernel(PrepareArgs a) {
  __shared__ float warp_sums[kD / 32];
  __shared__ float scratch[kD / 32];
  __shared__ uint16_t normalized[kD];
  const uint32_t d = threadIdx.x, lane_index = blockIdx.y;
  const uint32_t tasks_per_row = a.query_heads + a.kv_heads, group = a.query_heads / a.kv_heads;
  const uint32_t row = blockIdx.x / tasks_per_row, task = blockIdx.x % tasks_per_row;
  const bool query = task < a.query_heads;
  const uint32_t head = query ? task : task - a.query_heads;
  const uint64_t packed_stride = uint64_t(a.query_heads) * 2 * kD + 2ull * a.kv_heads * kD;
  const uint16_t *source_row = a.packed_qkv + (uint64_t(lane_index) * a.rows + row) * packed_stride;
  const uint16_t *source = query ? source_row + uint64_t(head) * 2 * kD : source_row + uint64_t(a.query_heads) * 2 * kD + uint64_t(head) * kD;

  rk_chunk_params p{};
  if (Format != 0) { // the fused form keeps the store's contract: an invalid lane writes nothing into the pool
    p = a.lane_params[lane_index];
    p.kv = a.layer;
    if (!query && (!rk_chunk_contract_valid(&p) || p.chunk_tokens > RK_TREE_NODES || p.chunk_stride != kStride || row >= p.chunk_tokens)) return;
  }

  const float x = bf16_bits_to_float(source[d]);
  const float total = block_sum_of_squares(__fmul_rn(x, x), warp_sums);
  const float inverse = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, float(kD)), a.eps)));
  const void *weights = query ? a.q_norm : a.k_norm;
  const float weight = NormF32 ? static_cast<const float *>(weights)[d] : bf16_bits_to_float(static_cast<const uint16_t *>(weights)[d]);
  normalized[d] = float_to_bf16_bits(__fmul_rn(__fmul_rn(x, inverse), weight));
  __syncthreads();
  uint16_t out = normalized[d];
  if (d < 2 * kRotaryPairs) {
    const uint32_t pair = d % kRotaryPairs;
    const float first = bf16_bits_to_float(normalized[pair]), second = bf16_bits_to_float(normalized[pair + kRotaryPairs]);
    const float cosine = a.rope_cos[(uint64_t(lane_index) * a.rows + row) * kRotaryPairs + pair];
    const float sine = a.rope_sin[(uint64_t(lane_index) * a.rows + row) * kRotaryPairs + pair];
    out = d < kRotaryPairs ? float_to_bf16_bits(__fsub_rn(__fmul_rn(first, cosine), __fmul_rn(second, sine)))
                           : float_to_bf16_bits(__fadd_rn(__fmul_rn(second, cosine), __fmul_rn(first, sine)));
  }
  if (query) {
    const uint32_t kv = head / group, local = head % group;
    a.queries[(((uint64_t(lane_index) * a.kv_heads + kv) * kStride + row) * group + local) * kD + d] = out;
    return;
  }
  const uint16_t value_bits = source[uint64_t(a.kv_heads) * kD + d]; // the head's v row follows all k rows
  if (Format == 0) {
    a.chunk_keys[((uint64_t(lane_index) * a.kv_heads + head) * kStride + row) * kD + d] = out;
    a.chunk_values[((uint64_t(lane_index) * a.kv_heads + head) * kD + d) * kStride + row] = value_bits;
  } else {
    constexpr uint32_t F = Format == 0 ? RK_FORMAT_INT8 : Format;
    const uint32_t token = p.committed_tokens + row;
    const PageSlabs slabs = PageGeometry<F, 4, kD>::slabs(a.tables[lane_index][token / kPageTokens], p.kv, head);
    store_page_row<F>(out, false, slabs, token % kPageTokens, scratch);
    store_page_row<F>(value_bits, true, slabs, token % kPageTokens, scratch);
  }
}

template <uint32_t Format>
int launch_prepare(const PrepareArgs &args, uint32_t lanes, int norm_f32, cudaStream_t stream) {
  const dim3 grid(args.rows * (args.query_heads + args.kv_heads), lanes);
  if (norm_f32) qkv_prepare_kernel<Format, true><<<grid, kD, 0, stream>>>(args);
  else qkv_prepare_kernel<Format, false><<<grid, kD, 0, stream>>>(args);
  return cuda_status(cudaGetLastError(), "qkv prepare launch");
}

bool geometry_ok(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t rows) {
  return kv_heads == 4 && query_heads == 24 && head_dim == kD && rows > 0 && rows <= RK_TREE_NODES;
}

} // namespace
} // namespace rk

using namespace rk;

// verify_attention_qkv / verify_attention_qkv_f32 (decode/attention_qkv.metal:33-60): the three stagings.
extern "C" int rk_qkv_prepare(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes, uint32_t rows,
                              const void *packed_qkv, const void *q_norm, const void *k_norm, int norm_f32,
                              const float *rope_cos, const float *rope_sin, float eps, void *queries, void *chunk_keys,
                              void *chunk_values, void *stream) {
  if (!geometry_ok(kv_heads, query_heads, head_dim, rows)) { set_error("rk_qkv_prepare: built for 4 KV heads x 24 query heads x 256, up to 16 rows"); return kUnsupported; }
  if (!lanes || !packed_qkv || !q_norm || !k_norm || !rope_cos || !rope_sin || !queries || !chunk_keys || !chunk_values) {
    set_error("rk_qkv_prepare: invalid arguments");
    return kInvalid;
  }
  PrepareArgs args{static_cast<const uint16_t *>(packed_qkv), q_norm, k_norm, rope_cos, rope_sin, static_cast<uint16_t *>(queries),
                   static_cast<uint16_t *>(chunk_keys), static_cast<uint16_t *>(chunk_values), eps, rows, kv_heads, query_heads,
                   nullptr, nullptr, rk_kv_layer{0, 0}};
  return launch_prepare<0>(args, lanes, norm_f32, static_cast<cudaStream_t>(stream));
}

// The same with the page store merged in: queries staging + K/V rows quantised into their page slots
// (rk_qkv_prepare followed by rk_store_verify, bit for bit, in one launch and without the K/V stagings).
extern "C" int rk_qkv_prepare_store(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                                    uint32_t rows, const void *packed_qkv, const void *q_norm, const void *k_norm, int norm_f32,
                                    const float *rope_cos, const float *rope_sin, float eps, void *queries,
                                    const rk_page_entry *const *tables, const rk_chunk_params *lane_params, rk_kv_layer layer,
                                    void *stream) {
  if (!geometry_ok(kv_heads, query_heads, head_dim, rows) || !rk_format_valid(format)) { set_error("rk_qkv_prepare_store: unsupported geometry or format"); return kUnsupported; }
  if (!lanes || !packed_qkv || !q_norm || !k_norm || !rope_cos || !rope_sin || !queries || !tables || !lane_params || !layer.extent_pages) {
    set_error("rk_qkv_prepare_store: invalid arguments");
    return kInvalid;
  }
  PrepareArgs args{static_cast<const uint16_t *>(packed_qkv), q_norm, k_norm, rope_cos, rope_sin, static_cast<uint16_t *>(queries),
                   nullptr, nullptr, eps, rows, kv_heads, query_heads, tables, lane_params, layer};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (format) {
  case RK_FORMAT_INT4: return launch_prepare<RK_FORMAT_INT4>(args, lanes, norm_f32, s);
  case RK_FORMAT_INT8: return launch_prepare<RK_FORMAT_INT8>(args, lanes, norm_f32, s);
  case RK_FORMAT_FP8E4M3: return launch_prepare<RK_FORMAT_FP8E4M3>(args, lanes, norm_f32, s);
  default: return launch_prepare<RK_FORMAT_BF16>(args, lanes, norm_f32, s);
  }
}
