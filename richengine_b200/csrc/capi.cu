// capi.cu — error reporting, the CUDA extent storage and the pinned-host tier
// behind the C ABI of include/richkv.h.
//
// Storage mirrors the reference's kv::PageStorage (runtime/ops/PageStorage.hpp:27-102,
// PageStorage.mm:12-167): extents of extentPages pages that only the pool
// allocates and releases, page-table entries = extent address | index, a page's
// spans per layer and tensor. B200-native differences: extents are physical
// allocations mapped at fixed offsets of ONE reserved virtual range (CUDA
// virtual memory management), so every page of the pool lies inside one
// address window that a single TMA tensor map covers; page copies are a
// kernel; the table lives in device memory and is patched by stream-ordered
// copies.
#include "common.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <deque>
#include <vector>

namespace rk {

namespace {
thread_local std::string g_error;
}

void set_error(const char *text) { g_error = text ? text : ""; }

int cuda_status(cudaError_t error, const char *what) {
  if (error == cudaSuccess) return kOk;
  g_error = std::string(what) + ": " + cudaGetErrorString(error);
  return kCudaError;
}

int move_pages(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t extent_pages,
               const rk_page_entry *from_entries, const rk_page_entry *to_entries, uint8_t *from_slots,
               uint8_t *to_slots, uint32_t count, cudaStream_t stream);
int unpack_batch(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t extent_pages,
                 const PageBatch &batch, uint32_t count, cudaStream_t stream);

// ---- driver entry points, resolved at run time (the library links no libcuda) ----
struct DriverApi {
  CUresult (*memAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*memAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long) = nullptr;
  CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t) = nullptr;
  CUresult (*memGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*tensorMapEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill) = nullptr;
  bool ready = false;
};

const DriverApi *driver_api() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    auto load = [](const char *name, auto &slot) {
      void *fn = nullptr;
      cudaDriverEntryPointQueryResult result;
      if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &result) != cudaSuccess ||
          result != cudaDriverEntryPointSuccess || !fn)
        return false;
      slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(fn);
      return true;
    };
    bool ok = true;
    ok &= load("cuMemAddressReserve", api.memAddressReserve);
    ok &= load("cuMemAddressFree", api.memAddressFree);
    ok &= load("cuMemCreate", api.memCreate);
    ok &= load("cuMemRelease", api.memRelease);
    ok &= load("cuMemMap", api.memMap);
    ok &= load("cuMemUnmap", api.memUnmap);
    ok &= load("cuMemSetAccess", api.memSetAccess);
    ok &= load("cuMemGetAllocationGranularity", api.memGetAllocationGranularity);
    ok &= load("cuTensorMapEncodeTiled", api.tensorMapEncodeTiled);
    api.ready = ok;
  });
  return api.ready ? &api : nullptr;
}

int driver_status(CUresult result, const char *what);

// A 2-D view of a device address window as rows of 128 bytes, loaded `box_rows`
// rows at a time with the 128-byte shared-memory swizzle (no multicast).
int encode_window_map(CUtensorMap *map, uint64_t base, uint64_t rows, uint32_t box_rows) {
  const DriverApi *api = driver_api();
  if (!api) {
    set_error("cuTensorMapEncodeTiled is unavailable");
    return kCudaError;
  }
  const cuuint64_t dims[2] = {128, rows};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t element_strides[2] = {1, 1};
  return driver_status(api->tensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void *>(base),
                                                 dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                       "cuTensorMapEncodeTiled");
}

int driver_status(CUresult result, const char *what) {
  if (result == CUDA_SUCCESS) return kOk;
  g_error = std::string(what) + ": CUresult " + std::to_string(int(result));
  return result == CUDA_ERROR_OUT_OF_MEMORY ? kRefused : kCudaError;
}

// ---- extent storage -----------------------------------------------------------
struct Storage {
  uint32_t format = 0, layers = 0, kv_heads = 0, head_dim = 0;
  uint32_t page_count = 0, extent_pages = 0;
  uint32_t data_bytes = 0, scale_bytes = 0;
  uint64_t page_bytes = 0;    // one page over all layers
  uint64_t extent_bytes = 0;  // extent_pages * page_bytes
  uint64_t extent_stride = 0; // extent_bytes rounded up to the mapping granularity
  uint64_t budget_bytes = ~0ull;
  int device = 0;
  CUdeviceptr base = 0;
  uint64_t reserved = 0;
  std::vector<CUmemGenericAllocationHandle> handles;
  std::vector<uint8_t> allocated;
  std::vector<rk_kv_layer> places;

  uint32_t extents() const { return page_count / extent_pages; }
  uint64_t allocated_bytes() const {
    return uint64_t(std::count(allocated.begin(), allocated.end(), uint8_t(1))) * extent_bytes;
  }
  bool page_allocated(uint32_t page) const { return page < page_count && allocated[page / extent_pages]; }
  rk_page_entry entry(uint32_t page) const {
    const uint32_t extent = page / extent_pages;
    return rk_make_entry(uint64_t(base) + extent * extent_stride, page - extent * extent_pages);
  }
};

uint64_t gcd64(uint64_t a, uint64_t b) { while (b) { const uint64_t r = a % b; a = b; b = r; } return a; }

// Pages whose bytes of one tensor fill whole 64 KiB units (PagedKv.hpp:112-119).
uint64_t pages_for_aligned_region(uint64_t bytes) { return bytes ? 65536 / gcd64(65536, bytes) : 0; }

} // namespace rk

using namespace rk;

extern "C" const char *rk_last_error(void) { return g_error.c_str(); }

extern "C" uint32_t rk_extent_alignment_pages(uint32_t format, uint32_t kv_heads, uint32_t head_dim) {
  // Layout::extentAlignmentPages (PagedKv.hpp:175-183)
  const uint64_t data = pages_for_aligned_region(rk_data_bytes(format, kv_heads, head_dim));
  if (format == RK_FORMAT_BF16) return uint32_t(data);
  const uint64_t scale = pages_for_aligned_region(rk_scale_bytes(format, kv_heads));
  return uint32_t(data / gcd64(data, scale) * scale);
}

extern "C" void *rk_storage_create(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                                   uint32_t page_count, uint32_t extent_pages) {
  if (!rk_format_valid(format) || !layers || !kv_heads || !head_dim) {
    set_error("KV page storage layout is invalid");
    return nullptr;
  }
  auto s = std::make_unique<Storage>();
  s->format = format; s->layers = layers; s->kv_heads = kv_heads; s->head_dim = head_dim;
  s->page_count = page_count; s->extent_pages = extent_pages;
  s->data_bytes = rk_data_bytes(format, kv_heads, head_dim);
  s->scale_bytes = rk_scale_bytes(format, kv_heads);
  s->page_bytes = uint64_t(layers) * rk_layer_page_bytes(format, kv_heads, head_dim);
  s->extent_bytes = uint64_t(extent_pages) * s->page_bytes;
  // PageStorage.mm:24-36: whole alignment units, index fits the entry's low
  // bits, a layer offset fits 32 bits, a whole number of extents.
  if (!extent_pages || extent_pages % rk_extent_alignment_pages(format, kv_heads, head_dim) ||
      extent_pages > RK_PAGE_INDEX_MASK || s->extent_bytes > 0xffffffffull) {
    set_error("KV extent geometry is invalid");
    return nullptr;
  }
  if (!page_count || page_count % extent_pages) {
    set_error("KV page pool is not a whole number of extents");
    return nullptr;
  }
  const DriverApi *api = driver_api();
  if (!api) {
    set_error("CUDA driver entry points for virtual memory management are unavailable");
    return nullptr;
  }
  if (cuda_status(cudaGetDevice(&s->device), "cudaGetDevice")) return nullptr;
  if (cuda_status(cudaFree(nullptr), "context creation")) return nullptr;
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = s->device;
  size_t granularity = 0;
  if (driver_status(api->memGetAllocationGranularity(&granularity, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM),
                    "cuMemGetAllocationGranularity"))
    return nullptr;
  s->extent_stride = (s->extent_bytes + granularity - 1) / granularity * granularity;
  s->reserved = s->extent_stride * s->extents();
  if (driver_status(api->memAddressReserve(&s->base, s->reserved, std::max<size_t>(granularity, 1u << 21), 0, 0),
                    "cuMemAddressReserve"))
    return nullptr;
  s->handles.assign(s->extents(), 0);
  s->allocated.assign(s->extents(), 0);
  for (uint32_t layer = 0; layer < layers; ++layer)
    s->places.push_back(rk_make_layer(extent_pages, s->data_bytes, s->scale_bytes, layer));
  return s.release();
}

extern "C" int rk_storage_release_extent(void *storage, uint32_t extent);

extern "C" void rk_storage_destroy(void *storage) {
  auto *s = static_cast<Storage *>(storage);
  if (!s) return;
  cudaDeviceSynchronize();
  for (uint32_t e = 0; e < s->extents(); ++e)
    if (s->allocated[e]) rk_storage_release_extent(s, e);
  if (const DriverApi *api = driver_api()) api->memAddressFree(s->base, s->reserved);
  delete s;
}

// Grants the extent (0), refuses it with the budget or the driver as cause
// (kRefused), or reports misuse: kInvalid for an extent that is already
// allocated or past the pool (PageStorage.mm:61-80).
extern "C" int rk_storage_allocate_extent(void *storage, uint32_t extent) {
  auto *s = static_cast<Storage *>(storage);
  if (!s || extent >= s->extents()) { set_error("invalid KV extent"); return kInvalid; }
  if (s->allocated[extent]) { set_error("KV extent is already allocated"); return kInvalid; }
  if (s->allocated_bytes() + s->extent_bytes > s->budget_bytes) {
    set_error("engine memory budget exceeded");
    return kRefused;
  }
  const DriverApi *api = driver_api();
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = s->device;
  CUmemGenericAllocationHandle handle = 0;
  if (int status = driver_status(api->memCreate(&handle, s->extent_stride, &prop, 0), "cuMemCreate")) return status;
  const CUdeviceptr address = s->base + uint64_t(extent) * s->extent_stride;
  if (int status = driver_status(api->memMap(address, s->extent_stride, 0, handle, 0), "cuMemMap")) {
    api->memRelease(handle);
    return status;
  }
  CUmemAccessDesc access{};
  access.location = prop.location;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (int status = driver_status(api->memSetAccess(address, s->extent_stride, &access, 1), "cuMemSetAccess")) {
    api->memUnmap(address, s->extent_stride);
    api->memRelease(handle);
    return status;
  }
  // A fresh extent reads as zeros: stores write only their own slots, and
  // tests hold every other byte to zero.
  if (int status = cuda_status(cudaMemset(reinterpret_cast<void *>(address), 0, s->extent_stride), "extent clear")) {
    api->memUnmap(address, s->extent_stride);
    api->memRelease(handle);
    return status;
  }
  s->handles[extent] = handle;
  s->allocated[extent] = 1;
  return kOk;
}

// The caller proves no table names a page of the extent and no launched work
// still touches it; the device is drained before the mapping goes
// (the reference refuses while a command is in flight, PageStorage.mm:82-93).
extern "C" int rk_storage_release_extent(void *storage, uint32_t extent) {
  auto *s = static_cast<Storage *>(storage);
  if (!s || extent >= s->extents()) { set_error("invalid KV extent"); return kInvalid; }
  if (!s->allocated[extent]) { set_error("KV extent is not allocated"); return kInvalid; }
  const DriverApi *api = driver_api();
  if (int status = cuda_status(cudaDeviceSynchronize(), "drain before extent release")) return status;
  const CUdeviceptr address = s->base + uint64_t(extent) * s->extent_stride;
  if (int status = driver_status(api->memUnmap(address, s->extent_stride), "cuMemUnmap")) return status;
  api->memRelease(s->handles[extent]);
  s->handles[extent] = 0;
  s->allocated[extent] = 0;
  return kOk;
}

extern "C" void rk_storage_set_budget(void *storage, uint64_t bytes) { static_cast<Storage *>(storage)->budget_bytes = bytes; }
extern "C" uint32_t rk_storage_page_count(const void *storage) { return static_cast<const Storage *>(storage)->page_count; }
extern "C" uint32_t rk_storage_extent_pages(const void *storage) { return static_cast<const Storage *>(storage)->extent_pages; }
extern "C" uint64_t rk_storage_bytes_per_page(const void *storage) { return static_cast<const Storage *>(storage)->page_bytes; }
extern "C" uint64_t rk_storage_extent_bytes(const void *storage) { return static_cast<const Storage *>(storage)->extent_bytes; }
extern "C" uint64_t rk_storage_allocated_bytes(const void *storage) { return static_cast<const Storage *>(storage)->allocated_bytes(); }
extern "C" int rk_storage_is_allocated(const void *storage, uint32_t page) { return static_cast<const Storage *>(storage)->page_allocated(page); }
extern "C" void rk_storage_window(const void *storage, uint64_t *base, uint64_t *bytes) {
  const auto *s = static_cast<const Storage *>(storage);
  *base = uint64_t(s->base);
  *bytes = s->reserved;
}
extern "C" uint32_t rk_storage_layers(const void *storage, rk_kv_layer *out, uint32_t capacity) {
  const auto *s = static_cast<const Storage *>(storage);
  for (uint32_t i = 0; i < s->layers && i < capacity; ++i) out[i] = s->places[i];
  return s->layers;
}
// The table entry of a page; 0 for a page whose extent holds no memory.
extern "C" rk_page_entry rk_storage_entry(const void *storage, uint32_t page) {
  const auto *s = static_cast<const Storage *>(storage);
  return s->page_allocated(page) ? s->entry(page) : 0;
}

// Host <-> extent byte copies for loaders, tests and tools: `offset` and
// `bytes` address the extent's own bytes. Synchronous.
extern "C" int rk_storage_read_extent(const void *storage, uint32_t extent, uint64_t offset, void *host, uint64_t bytes) {
  const auto *s = static_cast<const Storage *>(storage);
  if (!s || extent >= s->extents() || !s->allocated[extent] || offset + bytes > s->extent_bytes) {
    set_error("extent read is out of range or the extent holds no memory");
    return kInvalid;
  }
  return cuda_status(cudaMemcpy(host, reinterpret_cast<const void *>(s->base + extent * s->extent_stride + offset), bytes, cudaMemcpyDeviceToHost), "extent read");
}
extern "C" int rk_storage_write_extent(void *storage, uint32_t extent, uint64_t offset, const void *host, uint64_t bytes) {
  auto *s = static_cast<Storage *>(storage);
  if (!s || extent >= s->extents() || !s->allocated[extent] || offset + bytes > s->extent_bytes) {
    set_error("extent write is out of range or the extent holds no memory");
    return kInvalid;
  }
  return cuda_status(cudaMemcpy(reinterpret_cast<void *>(s->base + extent * s->extent_stride + offset), host, bytes, cudaMemcpyHostToDevice), "extent write");
}

// Writes the entries of pages[first..count) to the device table, leaving the
// entries before `first` as they are (PageStorage.mm:127-141).
extern "C" int rk_storage_write_entries(const void *storage, const uint32_t *pages, uint32_t count, uint32_t first,
                                        rk_page_entry *device_table, uint32_t table_capacity, void *stream) {
  const auto *s = static_cast<const Storage *>(storage);
  if (!s || !device_table || table_capacity < count) {
    set_error("KV page table is too small for its entries");
    return kInvalid;
  }
  if (first > count) {
    set_error("KV page table entries start past the end of its pages");
    return kInvalid;
  }
  if (first == count) return kOk;
  std::vector<rk_page_entry> entries(count - first);
  for (uint32_t i = first; i < count; ++i) {
    if (!s->page_allocated(pages[i])) {
      set_error("KV page is in an extent that is not allocated");
      return kInvalid;
    }
    entries[i - first] = s->entry(pages[i]);
  }
  // Pageable source: the runtime stages it before returning, so `entries`
  // may go out of scope.
  return cuda_status(cudaMemcpyAsync(device_table + first, entries.data(), entries.size() * sizeof(rk_page_entry),
                                     cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)),
                     "page table upload");
}

namespace {
int upload_entries(const Storage *s, const uint32_t *pages, uint32_t count, rk_page_entry **device, cudaStream_t stream) {
  std::vector<rk_page_entry> entries(count);
  for (uint32_t i = 0; i < count; ++i) {
    if (!s->page_allocated(pages[i])) {
      set_error("cannot move a KV page of an extent that is not allocated");
      return kInvalid;
    }
    entries[i] = s->entry(pages[i]);
  }
  if (int status = cuda_status(cudaMallocAsync(reinterpret_cast<void **>(device), count * sizeof(rk_page_entry), stream), "cudaMallocAsync")) return status;
  return cuda_status(cudaMemcpyAsync(*device, entries.data(), count * sizeof(rk_page_entry), cudaMemcpyHostToDevice, stream), "entry upload");
}
} // namespace

// Copies each page's content onto its destination, every tensor of every
// layer, ordered on `stream` (PageStorage.mm:95-114). Nothing is copied when
// any page lies in an unallocated extent.
extern "C" int rk_storage_copy_pages(void *storage, const rk_page_copy *copies, uint32_t count, void *stream) {
  auto *s = static_cast<Storage *>(storage);
  if (!count) return kOk;
  if (!s || !copies) return kInvalid;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  std::vector<uint32_t> ids(2 * size_t(count));
  for (uint32_t i = 0; i < count; ++i) { ids[i] = copies[i].from; ids[count + i] = copies[i].to; }
  rk_page_entry *device = nullptr;
  if (int status = upload_entries(s, ids.data(), 2 * count, &device, st)) return status;
  const int status = move_pages(s->format, s->layers, s->kv_heads, s->head_dim, s->extent_pages, device,
                                device + count, nullptr, nullptr, count, st);
  cudaFreeAsync(device, st);
  return status;
}

namespace rk {
int launch_crc32c(const void *data, uint64_t stride, uint64_t payload_bytes, uint32_t count, uint32_t *out, uint32_t ctas,
                  cudaStream_t stream, const GatherSource *gather);
}

// Seals pages for the host tier or the persistent store: every page's spans are packed into its contiguous device slot
// (as rk_storage_pack_pages does) and the slot's CRC-32C is taken in the same pass, so a page is read once
// (the reference's IO worker checksums a payload while it writes it, runtime/model/SlotFile.cpp:715-735).
// `checksums` is a device array of `count` words.
extern "C" int rk_storage_seal_pages(void *storage, const uint32_t *pages, uint32_t count, void *device_slots, uint32_t *checksums,
                                     void *stream) {
  auto *s = static_cast<Storage *>(storage);
  if (!count) return kOk;
  if (!s || !pages || !device_slots || !checksums) { set_error("rk_storage_seal_pages: invalid arguments"); return kInvalid; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rk_page_entry *device = nullptr;
  if (int status = upload_entries(s, pages, count, &device, st)) return status;
  const GatherSource source{device, s->layers, s->extent_pages, s->data_bytes, s->scale_bytes};
  const int status = launch_crc32c(device_slots, s->page_bytes, s->page_bytes, count, checksums, 0, st, &source);
  cudaFreeAsync(device, st);
  return status;
}

// Packs pages into `count` contiguous device slots of bytes_per_page each
// (spans in layer, tensor order: PageStorage.mm:143-167), or unpacks them.
extern "C" int rk_storage_pack_pages(void *storage, const uint32_t *pages, uint32_t count, void *device_slots, int unpack, void *stream) {
  auto *s = static_cast<Storage *>(storage);
  if (!count) return kOk;
  if (!s || !pages || !device_slots) return kInvalid;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rk_page_entry *device = nullptr;
  if (int status = upload_entries(s, pages, count, &device, st)) return status;
  const int status = unpack ? move_pages(s->format, s->layers, s->kv_heads, s->head_dim, s->extent_pages, nullptr, device,
                                         static_cast<uint8_t *>(device_slots), nullptr, count, st)
                            : move_pages(s->format, s->layers, s->kv_heads, s->head_dim, s->extent_pages, device, nullptr,
                                         nullptr, static_cast<uint8_t *>(device_slots), count, st);
  cudaFreeAsync(device, st);
  return status;
}

// ---- pinned-host tier ------------------------------------------------------------
// The eviction tier the engine drives through engine::KvTier
// (runtime/engine/cache/KvTier.hpp:34-63) with the transfer bounds of
// KvPageTier (runtime/engine/cache/KvPageTier.cpp:38-132): a bounded number of
// transfers in flight, demotions at most half of it, restores at most three
// quarters. The slot store is pinned host memory instead of an SSD file: a
// demotion packs the page's spans into a device staging slot and one DMA takes
// it to the host slot; a restore is the reverse. A page stays valid until its
// demotion reports success.
namespace rk {
namespace {

struct Transfer {
  bool demotion = false;
  bool in_flight = false;
  bool ready = false;
  bool success = false;
  bool forced_failure = false;
  bool verify = false;    // a restore of an adopted slot: its payload must match the record's checksum
  uint32_t expected = 0;
  uint32_t page = 0, slot = 0;
  uint32_t owner = 0;     // the transfer of its batch whose event marks the batch done
  cudaEvent_t done = nullptr;
};

struct HostTier {
  Storage *storage = nullptr;
  uint64_t slot_bytes = 0;
  uint32_t slots = 0, transfer_limit = 0, demotion_limit = 0, restore_limit = 0;
  uint32_t demotions = 0, restores = 0, in_flight = 0, fail_next = 0;
  uint8_t *host = nullptr;    // slots * slot_bytes, pinned
  uint8_t *host_mapped = nullptr; // the same arena as the device addresses it (restores read it in place)
  uint32_t merged_run = 4; // restores of at least this many neighbouring host slots go as one copy
  uint8_t *staging = nullptr; // kStreams * kTierBatch * slot_bytes, device: a batch's packed pages, side by side
  uint32_t *slot_checksums = nullptr;    // pinned: CRC-32C of each slot's payload, taken on the device when it was packed
  uint32_t *arrived_checksums = nullptr; // pinned: CRC-32C of a restored payload after it reached the device, per transfer
  uint32_t *device_checksums = nullptr;  // device: per stream and batch position a seal's accumulator (zero between launches), then per transfer a word for a restore's check
  uint32_t *device_arrivals = nullptr;   // device: per stream and batch position, finished parts of a seal (zero between launches)
  uint32_t *published = nullptr;         // slot_checksums as the device addresses it: a seal stores its checksums there
  // Transfers are started in batches: a demotion or restore the cache asks for is queued, and up to kTierBatch of a
  // kind go out together when the batch is full, at the next poll or at a drain — ONE kernel for the batch (entries,
  // slots and checksum words in its arguments: pack + CRC-32C in one pass for demotions, unpack for restores), one
  // copy per page, one event. Streams are taken in turn: while one batch's bytes cross PCIe the next batch's kernel
  // runs. A stream retires its batches in issue order, so a poll asks only about the oldest one of each.
  static constexpr uint32_t kStreams = 4;
  cudaStream_t streams[kStreams] = {};
  std::deque<uint32_t> order[kStreams];
  uint32_t next_stream = 0;
  std::vector<uint32_t> pending[2];      // [0] demotions, [1] restores: asked for, not issued yet
  cudaStream_t pending_after[2] = {};    // the caller's stream each pending batch must follow
  std::vector<uint8_t> slot_used;
  uint32_t lowest_free = 0;              // no free slot lies below it
  std::vector<uint8_t> slot_verify;      // adopted from an earlier process and not read yet
  std::vector<uint32_t> slot_expected;
  std::vector<Transfer> transfers; // index = transfer id
  bool writable = true;
};

} // namespace
} // namespace rk

extern "C" void *rk_tier_create(void *storage, uint32_t slots, uint32_t transfer_limit) {
  auto *s = static_cast<Storage *>(storage);
  if (!s || !slots || !transfer_limit) { set_error("invalid host tier geometry"); return nullptr; }
  auto t = std::make_unique<HostTier>();
  t->storage = s;
  t->slot_bytes = s->page_bytes;
  t->slots = slots;
  t->transfer_limit = transfer_limit;
  t->demotion_limit = std::max<uint32_t>(1, transfer_limit / 2);
  t->restore_limit = std::max<uint32_t>(1, transfer_limit - transfer_limit / 4);
  t->slot_used.assign(slots, 0);
  t->slot_verify.assign(slots, 0);
  t->slot_expected.assign(slots, 0);
  t->transfers.resize(transfer_limit);
  if (cuda_status(cudaHostAlloc(reinterpret_cast<void **>(&t->host), uint64_t(slots) * t->slot_bytes, cudaHostAllocDefault), "pinned host arena")) return nullptr;
  if (cuda_status(cudaMalloc(reinterpret_cast<void **>(&t->staging), uint64_t(HostTier::kStreams) * kTierBatch * t->slot_bytes), "tier staging")) { cudaFreeHost(t->host); return nullptr; }
  for (cudaStream_t &stream : t->streams)
    if (cuda_status(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "tier stream")) { cudaFree(t->staging); cudaFreeHost(t->host); return nullptr; }
  if (cuda_status(cudaHostAlloc(reinterpret_cast<void **>(&t->slot_checksums), (uint64_t(slots) + transfer_limit) * 4, cudaHostAllocDefault), "tier checksums") ||
      cuda_status(cudaMalloc(reinterpret_cast<void **>(&t->device_checksums), (uint64_t(transfer_limit) + HostTier::kStreams * kTierBatch) * 4), "tier checksums")) {
    cudaFreeHost(t->slot_checksums); for (cudaStream_t stream : t->streams) cudaStreamDestroy(stream); cudaFree(t->staging); cudaFreeHost(t->host);
    return nullptr;
  }
  memset(t->slot_checksums, 0, (uint64_t(slots) + transfer_limit) * 4);
  t->arrived_checksums = t->slot_checksums + slots;
  if (cuda_status(cudaMalloc(reinterpret_cast<void **>(&t->device_arrivals), uint64_t(HostTier::kStreams) * kTierBatch * 4), "tier counters") ||
      cuda_status(cudaMemset(t->device_arrivals, 0, uint64_t(HostTier::kStreams) * kTierBatch * 4), "tier counters") ||
      cuda_status(cudaMemset(t->device_checksums, 0, (uint64_t(transfer_limit) + HostTier::kStreams * kTierBatch) * 4), "tier checksums") ||
      cuda_status(cudaHostGetDevicePointer(reinterpret_cast<void **>(&t->published), t->slot_checksums, 0), "tier checksum words")) {
    cudaFree(t->device_arrivals); cudaFree(t->device_checksums); cudaFreeHost(t->slot_checksums); for (cudaStream_t stream : t->streams) cudaStreamDestroy(stream);
    cudaFree(t->staging); cudaFreeHost(t->host);
    return nullptr;
  }
  for (Transfer &x : t->transfers) cudaEventCreateWithFlags(&x.done, cudaEventDisableTiming);
  if (cuda_status(cudaHostGetDevicePointer(reinterpret_cast<void **>(&t->host_mapped), t->host, 0), "pinned host arena")) {
    rk_tier_destroy(t.release());
    return nullptr;
  }
  return t.release();
}

extern "C" void rk_tier_destroy(void *tier) {
  auto *t = static_cast<HostTier *>(tier);
  if (!t) return;
  for (cudaStream_t stream : t->streams) cudaStreamSynchronize(stream); // every transfer reads or writes its page in place
  for (Transfer &x : t->transfers) cudaEventDestroy(x.done);
  for (cudaStream_t stream : t->streams) cudaStreamDestroy(stream);
  cudaFree(t->staging);
  cudaFree(t->device_checksums);
  cudaFree(t->device_arrivals);
  cudaFreeHost(t->slot_checksums);
  cudaFreeHost(t->host);
  delete t;
}

extern "C" uint64_t rk_tier_slot_bytes(const void *tier) { return static_cast<const HostTier *>(tier)->slot_bytes; }
extern "C" int rk_tier_writable(const void *tier) { return static_cast<const HostTier *>(tier)->writable; }
extern "C" int rk_tier_can_demote(const void *tier) {
  const auto *t = static_cast<const HostTier *>(tier);
  return t->demotions < t->demotion_limit && t->in_flight < t->transfer_limit && t->writable;
}
extern "C" int rk_tier_can_restore(const void *tier) {
  const auto *t = static_cast<const HostTier *>(tier);
  return t->restores < t->restore_limit && t->in_flight < t->transfer_limit;
}
// A free slot id, or -1 when the quota is full.
extern "C" int64_t rk_tier_acquire_slot(void *tier) {
  auto *t = static_cast<HostTier *>(tier);
  // the lowest free slot; every slot below `lowest_free` is in use
  for (uint32_t i = t->lowest_free; i < t->slots; ++i)
    if (!t->slot_used[i]) { t->slot_used[i] = 1; t->lowest_free = i + 1; return i; }
  t->lowest_free = t->slots;
  return -1;
}
extern "C" void rk_tier_release_slot(void *tier, uint32_t slot) {
  auto *t = static_cast<HostTier *>(tier);
  if (slot < t->slots) { t->slot_used[slot] = 0; t->slot_verify[slot] = 0; t->lowest_free = std::min(t->lowest_free, slot); }
}
// CRC-32C of the payload the slot's last completed demotion stored (taken on the device before the copy left).
extern "C" uint32_t rk_tier_slot_checksum(const void *tier, uint32_t slot) {
  const auto *t = static_cast<const HostTier *>(tier);
  return slot < t->slots ? t->slot_checksums[slot] : 0;
}
// Takes a free slot for a payload an earlier process stored (model::SlotFile::adopt,
// runtime/model/SlotFile.hpp:196-200): the first restore of the slot fails unless the payload's CRC-32C,
// taken on the device after the upload, equals `checksum`. Returns the slot id, -1 when the quota is full.
extern "C" int64_t rk_tier_adopt_slot(void *tier, const void *payload, uint64_t bytes, uint32_t checksum) {
  auto *t = static_cast<HostTier *>(tier);
  if (!payload || bytes != t->slot_bytes) { set_error("rk_tier_adopt_slot: the payload is not one slot"); return kInvalid; }
  const int64_t slot = rk_tier_acquire_slot(tier);
  if (slot < 0) return -1;
  memcpy(t->host + uint64_t(slot) * t->slot_bytes, payload, bytes);
  t->slot_checksums[slot] = checksum;
  t->slot_expected[slot] = checksum;
  t->slot_verify[slot] = 1;
  return slot;
}
// Test seam, host side only: the next `count` transfers report failure when
// they retire, as a failed write or read would.
extern "C" void rk_tier_fail_next(void *tier, uint32_t count) { static_cast<HostTier *>(tier)->fail_next = count; }
extern "C" const void *rk_tier_slot_host_pointer(const void *tier, uint32_t slot) {
  const auto *t = static_cast<const HostTier *>(tier);
  return slot < t->slots ? t->host + uint64_t(slot) * t->slot_bytes : nullptr;
}

namespace {
// Issues the pending transfers of one kind as a batch on the next stream.
void flush_pending(HostTier *t, uint32_t kind) {
  std::vector<uint32_t> &members = t->pending[kind];
  if (members.empty()) return;
  const bool demotion = kind == 0;
  // In the order of their host slots, packed side by side in the stream's own staging area: pages whose host slots
  // are neighbours (the usual case: slots are handed out lowest first) cross PCIe in ONE copy. A copy per page
  // costs the copy engine about 5 us between copies, a third of what a 540 KB page takes to transfer.
  std::sort(members.begin(), members.end(), [t](uint32_t a, uint32_t b) { return t->transfers[a].slot < t->transfers[b].slot; });
  const uint32_t lane = t->next_stream, count = uint32_t(members.size()), owner = members.back();
  t->next_stream = (lane + 1) % HostTier::kStreams;
  cudaStream_t stream = t->streams[lane], after = t->pending_after[kind];
  const Storage *s = t->storage;
  int status = kOk;
  if (after) { // order the batch after work already launched on the caller's stream
    status = cuda_status(cudaEventRecord(t->transfers[owner].done, after), "tier order event");
    if (!status) status = cuda_status(cudaStreamWaitEvent(stream, t->transfers[owner].done, 0), "tier order wait");
  }
  // pages from position i on whose host slots follow one another
  auto run_from = [&](uint32_t i) {
    uint32_t n = 1;
    while (i + n < count && t->transfers[members[i + n]].slot == t->transfers[members[i]].slot + n) ++n;
    return n;
  };
  PageBatch batch{};
  for (uint32_t i = 0; i < count; ++i) {
    const Transfer &x = t->transfers[members[i]];
    batch.entry[i] = s->entry(x.page);
    batch.slot[i] = t->staging + (uint64_t(lane) * kTierBatch + i) * t->slot_bytes;
    batch.publish[i] = t->published + x.slot;
  }
  if (demotion) {
    // packed and checksummed in one pass over the pages, before the bytes cross PCIe; the last part of every page
    // stores its checksum to the slot's pinned word
    GatherSource source{nullptr, s->layers, s->extent_pages, s->data_bytes, s->scale_bytes};
    source.batch = &batch;
    source.arrivals = t->device_arrivals + lane * kTierBatch;
    if (!status) status = launch_crc32c(nullptr, t->slot_bytes, t->slot_bytes, count, t->device_checksums + lane * kTierBatch, 0, stream, &source);
    for (uint32_t i = 0; i < count && !status; i += run_from(i))
      status = cuda_status(cudaMemcpyAsync(t->host + uint64_t(t->transfers[members[i]].slot) * t->slot_bytes, batch.slot[i],
                                           run_from(i) * t->slot_bytes, cudaMemcpyDeviceToHost, stream), "demotion copy");
  } else {
    // Pages whose host slots follow one another (a chain that was demoted alone, leaf first, sits in descending slots,
    // so a batch of its restores is one run once sorted) cross PCIe in ONE copy into the staging area, at the copy
    // engine's rate. A short run or a lone page is unpacked straight out of pinned host memory instead: the unpack
    // kernel's own loads cross PCIe (thousands in flight), slower per byte than the copy engine but without its set-up
    // per copy (about 5 us, half of what a 540 KB page takes). A page adopted from an earlier process always goes
    // through the staging area alone: what ARRIVED on the device is checked against its record.
    const uint32_t merged_run = t->merged_run;
    for (uint32_t i = 0; i < count && !status;) {
      const uint32_t id = members[i];
      const Transfer &x = t->transfers[id];
      if (x.verify) {
        status = cuda_status(cudaMemcpyAsync(batch.slot[i], t->host + uint64_t(x.slot) * t->slot_bytes, t->slot_bytes, cudaMemcpyHostToDevice, stream), "restore copy");
        uint32_t *word = t->device_checksums + HostTier::kStreams * kTierBatch + id;
        if (!status) status = launch_crc32c(batch.slot[i], t->slot_bytes, t->slot_bytes, 1, word, 0, stream, nullptr);
        if (!status) status = cuda_status(cudaMemcpyAsync(t->arrived_checksums + id, word, 4, cudaMemcpyDeviceToHost, stream), "restore checksum");
        ++i;
        continue;
      }
      uint32_t run = run_from(i);
      for (uint32_t k = 1; k < run; ++k)
        if (t->transfers[members[i + k]].verify) { run = k; break; }
      if (run >= merged_run) {
        status = cuda_status(cudaMemcpyAsync(batch.slot[i], t->host + uint64_t(x.slot) * t->slot_bytes, uint64_t(run) * t->slot_bytes,
                                             cudaMemcpyHostToDevice, stream), "restore copy");
        i += run;
      } else {
        batch.slot[i] = t->host_mapped + uint64_t(x.slot) * t->slot_bytes;
        ++i;
      }
    }
    if (!status) status = unpack_batch(s->format, s->layers, s->kv_heads, s->head_dim, s->extent_pages, batch, count, stream);
  }
  if (!status) status = cuda_status(cudaEventRecord(t->transfers[owner].done, stream), "tier completion event");
  for (uint32_t id : members) {
    Transfer &x = t->transfers[id];
    x.owner = owner;
    if (status) x.forced_failure = true; // the batch did not go out whole: its transfers retire as failed
    t->order[lane].push_back(id);
  }
  if (status && demotion) t->writable = false; // a failed write closes the tier to demotions
  members.clear();
}

int start_transfer(HostTier *t, bool demotion, uint32_t page, uint32_t slot, cudaStream_t after) {
  if (demotion ? !rk_tier_can_demote(t) : !rk_tier_can_restore(t)) return kRefused;
  if (slot >= t->slots || !t->slot_used[slot] || !t->storage->page_allocated(page)) {
    set_error("host tier transfer names an invalid slot or page");
    return kInvalid;
  }
  uint32_t id = 0;
  while (id < t->transfer_limit && t->transfers[id].in_flight) ++id;
  if (id == t->transfer_limit) return kRefused;
  const uint32_t kind = demotion ? 0 : 1;
  if (!t->pending[kind].empty() && t->pending_after[kind] != after) flush_pending(t, kind);
  Transfer &x = t->transfers[id];
  x.demotion = demotion; x.in_flight = true; x.ready = false; x.success = false;
  x.forced_failure = t->fail_next > 0;
  if (t->fail_next) --t->fail_next;
  x.page = page; x.slot = slot; x.owner = id;
  x.verify = !demotion && t->slot_verify[slot] != 0;
  x.expected = t->slot_expected[slot];
  ++t->in_flight;
  ++(demotion ? t->demotions : t->restores);
  t->pending_after[kind] = after;
  t->pending[kind].push_back(id);
  if (t->pending[kind].size() == kTierBatch) flush_pending(t, kind);
  return int(id);
}
} // namespace

// Start moving `page` to `slot` (demote) or back (restore). Returns the
// transfer id (>= 0), kRefused when the tier takes no more of that kind for
// now, or an error. `after_stream`, when non-null, is a stream whose launched
// work the transfer must follow.
extern "C" int rk_tier_demote(void *tier, uint32_t page, uint32_t slot, void *after_stream) {
  return start_transfer(static_cast<HostTier *>(tier), true, page, slot, static_cast<cudaStream_t>(after_stream));
}
extern "C" int rk_tier_restore(void *tier, uint32_t slot, uint32_t page, void *after_stream) {
  return start_transfer(static_cast<HostTier *>(tier), false, page, slot, static_cast<cudaStream_t>(after_stream));
}
// Retires finished transfers; returns how many retired in this call.
extern "C" int rk_tier_poll(void *tier) {
  auto *t = static_cast<HostTier *>(tier);
  int retired = 0;
  flush_pending(t, 0);
  flush_pending(t, 1);
  for (std::deque<uint32_t> &order : t->order)
  while (!order.empty()) { // a stream's batches finish in issue order: the first one still running ends the scan
    Transfer &x = t->transfers[order.front()];
    const cudaError_t state = cudaEventQuery(t->transfers[x.owner].done);
    if (state == cudaErrorNotReady) break;
    order.pop_front();
    x.ready = true;
    x.success = state == cudaSuccess && !x.forced_failure;
    if (!x.demotion && x.verify) { // a payload that does not match its record is a miss and nothing worse
      const uint32_t id = uint32_t(&x - t->transfers.data());
      if (t->arrived_checksums[id] != x.expected) x.success = false;
      else if (x.success) t->slot_verify[x.slot] = 0; // trusted from now on, as this process's own slots are
    }
    if (x.demotion && !x.success) t->writable = false;
    --t->in_flight;
    --(x.demotion ? t->demotions : t->restores);
    ++retired;
  }
  return retired;
}
extern "C" int rk_tier_transfer_ready(const void *tier, uint32_t id) {
  const auto *t = static_cast<const HostTier *>(tier);
  return id < t->transfer_limit && t->transfers[id].in_flight && t->transfers[id].ready;
}
// Reports the transfer's outcome (1 success, 0 failure) and frees its id.
extern "C" int rk_tier_transfer_finish(void *tier, uint32_t id) {
  auto *t = static_cast<HostTier *>(tier);
  if (id >= t->transfer_limit || !t->transfers[id].in_flight || !t->transfers[id].ready) return kInvalid;
  t->transfers[id].in_flight = false;
  return t->transfers[id].success ? 1 : 0;
}
extern "C" int rk_tier_drain(void *tier) {
  auto *t = static_cast<HostTier *>(tier);
  flush_pending(t, 0);
  flush_pending(t, 1);
  for (cudaStream_t stream : t->streams)
    if (int status = cuda_status(cudaStreamSynchronize(stream), "tier drain")) return status;
  return rk_tier_poll(tier);
}
