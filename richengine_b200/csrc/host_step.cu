// host_step.cu — moves one decode step's rows between the compact layout a host
// caller holds and the staging layouts the kernels read.
//
// The reference keeps every lane's current rows in chunk stagings of 32 rows
// per KV head (runtime/metal/kernels/common/paged_store_row.h:31-41 for K/V,
// runtime/metal/kernels/decode/paged_attention.metal:39-41 for queries and
// output), written on the GPU by its QKV projection. A caller that holds host
// buffers sends only the live row of each lane — [lane][query head][D] queries,
// [lane][KV head][D] keys and values — and these kernels scatter it into row 0
// of the stagings (values become dimension-major) and gather row 0 of the
// output back.
#include "common.cuh"

namespace rk {
namespace {

// grid (lanes * kv_heads), 256 threads (one per dimension).
__global__ void __launch_bounds__(256)
stage_rows_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v,
                  uint16_t *__restrict__ queries, uint16_t *__restrict__ chunk_keys,
                  uint16_t *__restrict__ chunk_values, uint32_t group, uint32_t head_dim) {
  const uint64_t tile = blockIdx.x; // lane * kv_heads + kv_head
  const uint32_t d = threadIdx.x;
  if (d >= head_dim) return;
  constexpr uint32_t stride = RK_VERIFY_CHUNK_STRIDE;
  for (uint32_t g = 0; g < group; ++g)
    queries[(tile * stride * group + g) * head_dim + d] = q[(tile * group + g) * head_dim + d];
  chunk_keys[tile * stride * head_dim + d] = k[tile * head_dim + d];
  chunk_values[(tile * head_dim + d) * stride] = v[tile * head_dim + d];
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint16_t *__restrict__ output, uint16_t *__restrict__ out, uint32_t group, uint32_t head_dim) {
  const uint64_t tile = blockIdx.x;
  const uint32_t d = threadIdx.x;
  if (d >= head_dim) return;
  for (uint32_t g = 0; g < group; ++g)
    out[(tile * group + g) * head_dim + d] = output[(tile * RK_VERIFY_CHUNK_STRIDE * group + g) * head_dim + d];
}

} // namespace
} // namespace rk

using namespace rk;

extern "C" int rk_stage_decode_rows(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                                    const void *q, const void *k, const void *v, void *queries, void *chunk_keys,
                                    void *chunk_values, void *stream) {
  if (!lanes || !kv_heads || query_heads % kv_heads || head_dim > 256 || !q || !k || !v || !queries || !chunk_keys || !chunk_values) {
    set_error("rk_stage_decode_rows: invalid arguments");
    return kInvalid;
  }
  stage_rows_kernel<<<lanes * kv_heads, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t *>(q), static_cast<const uint16_t *>(k), static_cast<const uint16_t *>(v),
      static_cast<uint16_t *>(queries), static_cast<uint16_t *>(chunk_keys), static_cast<uint16_t *>(chunk_values),
      query_heads / kv_heads, head_dim);
  return cuda_status(cudaGetLastError(), "stage rows launch");
}

extern "C" int rk_gather_decode_rows(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                                     const void *output, void *out, void *stream) {
  if (!lanes || !kv_heads || query_heads % kv_heads || head_dim > 256 || !output || !out) {
    set_error("rk_gather_decode_rows: invalid arguments");
    return kInvalid;
  }
  gather_rows_kernel<<<lanes * kv_heads, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t *>(output), static_cast<uint16_t *>(out), query_heads / kv_heads, head_dim);
  return cuda_status(cudaGetLastError(), "gather rows launch");
}
