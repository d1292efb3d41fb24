// page_ops.cu — whole-page moves and the tree-verify compaction.
//
//   runtime/ops/PageStorage.mm:95-114,143-167      copyPages / spans: every tensor of every layer
//   runtime/metal/kernels/decode/paged_attention_store.metal:198-278   tree compaction
// The reference copies pages with a host memcpy over unified memory; here a
// page lives in HBM, so the copy is a kernel that moves each (layer, tensor)
// span with 16-byte loads and stores. The same kernel packs a page into one
// contiguous slot (eviction staging) and unpacks it again (restore).
#include "common.cuh"

namespace rk {
namespace {

// One end of a page move: a page reached through its table entry, or a
// contiguous slot holding the page's spans layer by layer in tensor order.
struct PageEnd {
  rk_page_entry entry; // used when slot == nullptr
  uint8_t *slot;
};

struct SpanGeometry {
  uint32_t layers, extent_pages, data_bytes, scale_bytes;
};

__device__ __forceinline__ uint8_t *span_pointer(const PageEnd &end, const SpanGeometry &g, uint32_t layer,
                                                 uint32_t tensor) {
  if (end.slot) {
    const uint64_t per_layer = 2ull * (uint64_t(g.data_bytes) + g.scale_bytes);
    const uint64_t before = uint64_t((tensor + 1) / 2) * g.data_bytes + uint64_t(tensor / 2) * g.scale_bytes;
    return end.slot + layer * per_layer + before;
  }
  return reinterpret_cast<uint8_t *>(rk_entry_extent(end.entry)) +
         rk_extent_offset(g.extent_pages, g.data_bytes, g.scale_bytes, layer, tensor, rk_entry_index(end.entry));
}

// grid (layers * 4, copies); each block moves one span.
__global__ void __launch_bounds__(256)
move_pages_kernel(const rk_page_entry *__restrict__ from_entries, const rk_page_entry *__restrict__ to_entries,
                  uint8_t *from_slots, uint8_t *to_slots, uint64_t slot_bytes, SpanGeometry g) {
  const uint32_t layer = blockIdx.x / 4, tensor = blockIdx.x % 4, copy = blockIdx.y;
  const uint32_t bytes = rk_tensor_page_bytes(g.data_bytes, g.scale_bytes, tensor);
  if (!bytes) return;
  PageEnd from{from_entries ? from_entries[copy] : 0, from_slots ? from_slots + copy * slot_bytes : nullptr};
  PageEnd to{to_entries ? to_entries[copy] : 0, to_slots ? to_slots + copy * slot_bytes : nullptr};
  const uint4 *source = reinterpret_cast<const uint4 *>(span_pointer(from, g, layer, tensor));
  uint4 *target = reinterpret_cast<uint4 *>(span_pointer(to, g, layer, tensor));
  for (uint32_t i = threadIdx.x; i < bytes / 16; i += blockDim.x) target[i] = source[i];
}

// The host tier's restores: packed slots -> the pages named in the batch (entries and slot addresses by value).
// grid (layers * 4, batch.count).
__global__ void __launch_bounds__(256) unpack_batch_kernel(const __grid_constant__ PageBatch batch, SpanGeometry g) {
  const uint32_t layer = blockIdx.x / 4, tensor = blockIdx.x % 4, copy = blockIdx.y;
  const uint32_t bytes = rk_tensor_page_bytes(g.data_bytes, g.scale_bytes, tensor);
  if (!bytes) return;
  const uint4 *source = reinterpret_cast<const uint4 *>(span_pointer(PageEnd{0, batch.slot[copy]}, g, layer, tensor));
  uint4 *target = reinterpret_cast<uint4 *>(span_pointer(PageEnd{batch.entry[copy], nullptr}, g, layer, tensor));
  for (uint32_t i = threadIdx.x; i < bytes / 16; i += blockDim.x) target[i] = source[i];
}

// grid (lanes * kv_heads), HeadDim threads: moves the retained path rows of
// one (lane, head) to their path slots, in path order; every load of a row
// precedes its stores.
template <uint32_t Format, uint32_t KvHeads, uint32_t HeadDim>
__global__ void __launch_bounds__(HeadDim)
tree_compact_kernel(const rk_page_entry *const *__restrict__ tables, const rk_chunk_params *__restrict__ lane_params,
                    rk_kv_layer layer, const uint32_t *__restrict__ retained_path,
                    const uint32_t *__restrict__ retained_count) {
  using Geometry = PageGeometry<Format, KvHeads, HeadDim>;
  constexpr bool kPacked = Format == RK_FORMAT_INT4;
  constexpr uint32_t kElementBytes = Format == RK_FORMAT_BF16 ? 2 : 1;
  constexpr uint32_t kKeyWidth = kPacked ? HeadDim / 2 : HeadDim; // elements (bytes for int4) per key row
  const uint32_t lane_index = blockIdx.x / KvHeads, head = blockIdx.x % KvHeads, tid = threadIdx.x;
  rk_chunk_params p = lane_params[lane_index];
  if (layer.extent_pages) p.kv = layer;
  const uint32_t count = retained_count[lane_index];
  if (!count || count > RK_VERIFY_ROWS || !rk_chunk_contract_valid(&p)) return;
  const rk_page_entry *table = tables[lane_index];
  for (uint32_t i = 0; i < count; ++i) {
    const uint32_t source_row = retained_path[lane_index * RK_VERIFY_ROWS + i];
    if (source_row == i) continue; // uniform across the block
    const uint32_t st = p.committed_tokens + source_row, dt = p.committed_tokens + i;
    if (rk_pages_for(max(st, dt) + 1) > p.page_table_entries) return;
    const PageSlabs s = Geometry::slabs(table[st / kPageTokens], p.kv, head);
    const PageSlabs d = Geometry::slabs(table[dt / kPageTokens], p.kv, head);
    const uint32_t so = st % kPageTokens, dofs = dt % kPageTokens;
    const bool active = tid < kKeyWidth;
    uint16_t key = 0, value = 0;
    float key_scale = 0.0f, value_scale = 0.0f;
    if (Geometry::kQuantized && tid == 0) { key_scale = s.key_scales[so]; value_scale = s.value_scales[so]; }
    if (kPacked) {
      if (active) { key = s.keys[so * kKeyWidth + tid]; value = s.values[so * kKeyWidth + tid]; }
    } else if (kElementBytes == 2) {
      key = reinterpret_cast<const uint16_t *>(s.keys)[so * kKeyWidth + tid];
      value = reinterpret_cast<const uint16_t *>(s.values)[tid * kPageTokens + so];
    } else {
      key = s.keys[so * kKeyWidth + tid];
      value = s.values[tid * kPageTokens + so];
    }
    __syncthreads();
    if (kPacked) {
      if (active) { d.keys[dofs * kKeyWidth + tid] = uint8_t(key); d.values[dofs * kKeyWidth + tid] = uint8_t(value); }
    } else if (kElementBytes == 2) {
      reinterpret_cast<uint16_t *>(d.keys)[dofs * kKeyWidth + tid] = key;
      reinterpret_cast<uint16_t *>(d.values)[tid * kPageTokens + dofs] = value;
    } else {
      d.keys[dofs * kKeyWidth + tid] = uint8_t(key);
      d.values[tid * kPageTokens + dofs] = uint8_t(value);
    }
    if (Geometry::kQuantized && tid == 0) { d.key_scales[dofs] = key_scale; d.value_scales[dofs] = value_scale; }
    __syncthreads();
  }
}

} // namespace

int move_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t extent_pages,
               const rk_page_entry *from_entries, const rk_page_entry *to_entries, uint8_t *from_slots,
               uint8_t *to_slots, uint32_t count, cudaStream_t stream) {
  if (!count) return kOk;
  if (!rk_format_valid(format) || !layers || !extent_pages || (!from_entries == !from_slots) ||
      (!to_entries == !to_slots)) {
    set_error("page move: invalid arguments");
    return kInvalid;
  }
  SpanGeometry g{layers, extent_pages, rk_data_bytes(format, kv_heads, head_dim), rk_scale_bytes(format, kv_heads)};
  const uint64_t slot_bytes = uint64_t(layers) * rk_layer_page_bytes(format, kv_heads, head_dim);
  for (uint32_t done = 0; done < count;) { // grid.y is limited to 65535
    const uint32_t batch = min(count - done, 32768u);
    move_pages_kernel<<<dim3(layers * 4, batch), 256, 0, stream>>>(
        from_entries ? from_entries + done : nullptr, to_entries ? to_entries + done : nullptr,
        from_slots ? from_slots + done * slot_bytes : nullptr, to_slots ? to_slots + done * slot_bytes : nullptr,
        slot_bytes, g);
    if (int status = cuda_status(cudaGetLastError(), "page move launch")) return status;
    done += batch;
  }
  return kOk;
}

int unpack_batch(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t extent_pages,
                 const PageBatch &batch, uint32_t count, cudaStream_t stream) {
  if (!count) return kOk;
  if (!rk_format_valid(format) || !layers || !extent_pages || count > kTierBatch) {
    set_error("page unpack: invalid arguments");
    return kInvalid;
  }
  SpanGeometry g{layers, extent_pages, rk_data_bytes(format, kv_heads, head_dim), rk_scale_bytes(format, kv_heads)};
  unpack_batch_kernel<<<dim3(layers * 4, count), 256, 0, stream>>>(batch, g);
  return cuda_status(cudaGetLastError(), "page unpack launch");
}

} // namespace rk

using namespace rk;

extern "C" int rk_copy_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                             uint32_t extent_pages, const rk_page_entry *from_entries,
                             const rk_page_entry *to_entries, uint32_t count, void *stream) {
  return move_pages(format, layers, kv_heads, head_dim, extent_pages, from_entries, to_entries, nullptr, nullptr,
                    count, static_cast<cudaStream_t>(stream));
}

extern "C" int rk_pack_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                             uint32_t extent_pages, const rk_page_entry *from_entries, void *slots,
                             uint32_t count, void *stream) {
  return move_pages(format, layers, kv_heads, head_dim, extent_pages, from_entries, nullptr, nullptr,
                    static_cast<uint8_t *>(slots), count, static_cast<cudaStream_t>(stream));
}

extern "C" int rk_unpack_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                               uint32_t extent_pages, const void *slots, const rk_page_entry *to_entries,
                               uint32_t count, void *stream) {
  return move_pages(format, layers, kv_heads, head_dim, extent_pages, nullptr, to_entries,
                    static_cast<uint8_t *>(const_cast<void *>(slots)), nullptr, count,
                    static_cast<cudaStream_t>(stream));
}

extern "C" int rk_tree_compact(uint32_t format, uint32_t kv_heads, uint32_t head_dim, uint32_t lanes,
                               const rk_page_entry *const *tables, const rk_chunk_params *lane_params,
                               rk_kv_layer layer, const uint32_t *retained_path,
                               const uint32_t *retained_count, void *stream) {
  if (!lanes || !tables || !lane_params || !retained_path || !retained_count || !layer.extent_pages) {
    set_error("rk_tree_compact: invalid arguments");
    return kInvalid;
  }
  if (format == RK_FORMAT_FP8E4M3) { // PagedAttention.cpp:561-562
    set_error("rk_tree_compact: tree verify has no fp8 kernels");
    return kInvalid;
  }
  if (kv_heads != 4 || head_dim != 256) return kUnsupported;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (format) {
  case RK_FORMAT_INT8:
    tree_compact_kernel<RK_FORMAT_INT8, 4, 256><<<lanes * 4, 256, 0, s>>>(tables, lane_params, layer, retained_path, retained_count);
    break;
  case RK_FORMAT_INT4:
    tree_compact_kernel<RK_FORMAT_INT4, 4, 256><<<lanes * 4, 256, 0, s>>>(tables, lane_params, layer, retained_path, retained_count);
    break;
  case RK_FORMAT_BF16:
    tree_compact_kernel<RK_FORMAT_BF16, 4, 256><<<lanes * 4, 256, 0, s>>>(tables, lane_params, layer, retained_path, retained_count);
    break;
  default: return kInvalid;
  }
  return cuda_status(cudaGetLastError(), "tree compact launch");
}
