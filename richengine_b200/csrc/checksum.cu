// checksum.cu — CRC-32C (Castagnoli) of packed page payloads on the device, and of small host buffers.
//
// The reference keeps a CRC-32C of every persistent slot's payload and record (runtime/model/Crc32c.hpp:12-29,
// computed by the slot file's IO worker while it writes, runtime/model/SlotFile.cpp:715-735,775-795) and checks an
// adopted slot's first read against it. Here a demoted page is packed on the GPU, so its checksum is taken there,
// at memory speed, before the bytes cross PCIe; a restored payload is checked the same way after it arrives.
//
// A CRC is linear over GF(2), which lets a warp read coalesced instead of giving every thread a contiguous run:
//  * a warp walks its chunk in rows of 512 bytes, lane l loading 16 bytes = words 4l..4l+3 of the row; each of
//    the warp's 128 word columns keeps its own remainder and advances it by a whole row per step:
//      acc <- (acc ^ word) * x^4096 mod P        (four table lookups, as slicing-by-4 does for x^32)
//    The lookup tables of that step are replicated 32 times in shared memory, one copy per bank, so the 32 lanes'
//    data-dependent lookups never collide;
//  * the 128 remainders are then a 128-word message of their own: three ordinary steps inside the thread, five
//    shuffle levels across the warp (x^128 .. x^2048), one last step;
//  * chunks combine through crc(A|B) = crc(A) * x^(8 len B) + crc(B): every chunk's multiplier depends only on
//    the payload size, so the host computes them once per launch; contributions are XOR-ed into the result
//    (atomicXor: order-free, so the result is deterministic), and the initial/final inversions are one more term.
#include "common.cuh"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

namespace rk {


namespace {

constexpr uint32_t kPoly = 0x82F63B78u; // reflected Castagnoli polynomial
constexpr uint32_t kRowBytes = 512;     // one warp step: 32 lanes x 16 bytes
constexpr uint32_t kWarps = 32;         // per CTA
constexpr uint32_t kGroupWarps = 8;     // warps that share one payload part; a CTA runs kWarps / kGroupWarps parts at a time
constexpr uint32_t kGroups = kWarps / kGroupWarps;
constexpr uint32_t kMaxParts = 64;      // parts a payload may be cut into

// Polynomials are bit-reversed as in the usual software CRC: bit 31 is x^0.
constexpr uint32_t mul_mod(uint32_t a, uint32_t b) {
  uint32_t product = 0;
  for (uint32_t bit = 0x80000000u; bit; bit >>= 1) {
    if (a & bit) product ^= b;
    b = (b & 1u) ? (b >> 1) ^ kPoly : b >> 1;
  }
  return product;
}
// x^(8 * bytes) mod P
uint32_t x_power_bytes(uint64_t bytes) {
  uint32_t result = 0x80000000u;  // 1
  uint32_t square = 0x00800000u;  // x^8
  for (; bytes; bytes >>= 1) {
    if (bytes & 1u) result = mul_mod(result, square);
    square = mul_mod(square, square);
  }
  return result;
}

// table[k][b] = (b << 8k) * x^(8 * bytes) mod P: advancing a remainder by `bytes` zero bytes, one byte lane at a time
void advance_table(uint64_t bytes, uint32_t *table) {
  const uint32_t power = x_power_bytes(bytes);
  for (uint32_t k = 0; k < 4; ++k)
    for (uint32_t b = 0; b < 256; ++b) table[k * 256 + b] = mul_mod(power, b << (8 * k));
}

constexpr uint32_t kTableWords = 4 * 256;
constexpr uint32_t kLevels = 5;
// [0] row step (512 bytes), [1] word step (4 bytes), [2..6] 16, 32, 64, 128, 256 bytes
constexpr uint32_t kTables = 2 + kLevels;
__device__ uint32_t g_tables[kTables * kTableWords];

const std::vector<uint32_t> &host_tables() {
  static const std::vector<uint32_t> tables = [] {
    std::vector<uint32_t> t(kTables * kTableWords);
    advance_table(kRowBytes, &t[0]);
    advance_table(4, &t[kTableWords]);
    for (uint32_t level = 0; level < kLevels; ++level) advance_table(16ull << level, &t[(2 + level) * kTableWords]);
    return t;
  }();
  return tables;
}

// Seal mode: the payload is not read from `data` but gathered from a page's spans in the pool (layer by layer,
// tensor by tensor: the order of a packed slot) and written to `data` on the way, so a page is read once for both
// its packed copy and its checksum. Every span is a whole number of 512-byte rows.
struct GatherArgs {
  const rk_page_entry *entries; // one per payload; null = the batch below
  uint32_t extent_pages, data_bytes, scale_bytes;
  uint32_t rows_per_layer, data_rows, scale_rows;
  uint32_t *arrivals;           // batch: finished parts per payload (zero between launches)
  PageBatch batch;              // entries, destination slots and checksum words by value
};

struct ChecksumArgs {
  const uint8_t *data;
  uint64_t stride;        // bytes between payloads
  GatherArgs gather;
  uint32_t *out;          // one word per payload, zeroed before the launch
  uint32_t payloads, parts;
  uint32_t rows_low, extra; // chunk g of a payload has rows_low + (g < extra) rows
  uint32_t closing;       // the initial and final inversions as one term
  uint32_t multiplier[kMaxParts * kGroupWarps]; // x^(8 * bytes after chunk g)
};

constexpr uint32_t kReplicaBytes = kTableWords * 32 * 4;                       // the row-step table, one copy per bank
constexpr uint32_t kSharedBytes = kReplicaBytes + (kTables - 1) * kTableWords * 4 + kWarps * 4;

__device__ __forceinline__ uint32_t lookup4(const uint32_t *table, uint32_t x) {
  return table[x & 0xffu] ^ table[256 + ((x >> 8) & 0xffu)] ^ table[512 + ((x >> 16) & 0xffu)] ^ table[768 + (x >> 24)];
}

// Entry (Byte, value of that byte of x) of the lane's copy of the row-step table: one byte permute, one multiply-add
// for the address (the multiply-add pipe is otherwise idle here, the logic pipe is the busy one), one load.
template <uint32_t Byte> __device__ __forceinline__ uint32_t row_lookup(uint32_t x, uint32_t lane_copy) {
  uint32_t address, value;
  asm("mad.lo.u32 %0, %1, 128, %2;" : "=r"(address) : "r"(__byte_perm(x, 0, 0x4440u + Byte)), "r"(lane_copy));
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(value) : "r"(address), "n"(Byte * 256 * 128));
  return value;
}

__device__ __forceinline__ uint32_t mul_mod_device(uint32_t a, uint32_t b) {
  uint32_t product = 0;
#pragma unroll
  for (uint32_t i = 0; i < 32; ++i) {
    product ^= (a & (0x80000000u >> i)) ? b : 0u;
    b = (b >> 1) ^ ((b & 1u) ? kPoly : 0u);
  }
  return product;
}

// Where row `q` of layer `layer` of a page lives in the pool: the spans follow each other as
// [K data][K scales][V data][V scales] inside a packed layer.
__device__ __forceinline__ const uint4 *gathered_row(const GatherArgs &g, rk_page_entry entry, uint32_t layer, uint32_t q) {
  uint32_t tensor = 0, within = q;
  if (q >= g.data_rows) { tensor = 1; within = q - g.data_rows; }
  if (q >= g.data_rows + g.scale_rows) { tensor = 2; within = q - g.data_rows - g.scale_rows; }
  if (q >= 2 * g.data_rows + g.scale_rows) { tensor = 3; within = q - 2 * g.data_rows - g.scale_rows; }
  const uint64_t address = rk_entry_extent(entry) +
                           rk_extent_offset(g.extent_pages, g.data_bytes, g.scale_bytes, layer, tensor, rk_entry_index(entry)) +
                           uint64_t(within) * kRowBytes;
  return reinterpret_cast<const uint4 *>(address);
}

template <bool kGather>
__global__ void __launch_bounds__(kWarps * 32, 1) crc32c_kernel(const __grid_constant__ ChecksumArgs args) {
  extern __shared__ __align__(16) uint32_t shared_words[];
  uint32_t *replica = shared_words;                       // [k][byte][lane]
  uint32_t *tables = shared_words + kTableWords * 32;     // word step, then the five levels
  uint32_t *warp_terms = tables + (kTables - 1) * kTableWords;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  for (uint32_t i = tid; i < kTableWords * 32; i += blockDim.x) replica[i] = g_tables[i >> 5];
  for (uint32_t i = tid; i < (kTables - 1) * kTableWords; i += blockDim.x) tables[i] = g_tables[kTableWords + i];
  __syncthreads();
  // this lane's copy: entry e at byte 128 e behind it
  const uint32_t mine_shared = uint32_t(__cvta_generic_to_shared(replica + lane));
  // Each group of eight warps takes (payload, part) units on its own; long chunks keep the fold of the 128
  // remainders (whose tables are not replicated) a small share of the lookups.
  const uint32_t group = warp / kGroupWarps, member = warp % kGroupWarps;
  const uint32_t units = args.payloads * args.parts;
  for (uint32_t unit = blockIdx.x * kGroups + group; unit < units; unit += gridDim.x * kGroups) {
    const uint32_t payload = unit / args.parts, part = unit - payload * args.parts;
    const uint32_t chunk = part * kGroupWarps + member;
    const uint32_t rows = args.rows_low + (chunk < args.extra ? 1u : 0u);
    const uint64_t first_row = uint64_t(chunk) * args.rows_low + min(chunk, args.extra);
    uint32_t term = 0;
    if (rows) {
      // seal mode: rows come from the page's spans and leave for the packed slot (`source` is then the destination)
      const bool batched = kGather && !args.gather.entries;
      const uint8_t *base = batched ? args.gather.batch.slot[payload] : args.data + uint64_t(payload) * args.stride;
      const uint4 *source = reinterpret_cast<const uint4 *>(base + first_row * kRowBytes) + lane;
      const rk_page_entry entry = !kGather ? 0 : batched ? args.gather.batch.entry[payload] : args.gather.entries[payload];
      uint32_t layer = kGather ? uint32_t(first_row / args.gather.rows_per_layer) : 0;
      uint32_t q = kGather ? uint32_t(first_row - uint64_t(layer) * args.gather.rows_per_layer) : 0;
      auto load_row = [&](uint32_t row) {
        if (!kGather) return __ldcs(source + uint64_t(row) * 32);
        const uint4 v = __ldcs(gathered_row(args.gather, entry, layer, q) + lane);
        __stcs(const_cast<uint4 *>(source) + uint64_t(row) * 32, v);
        if (++q == args.gather.rows_per_layer) { q = 0; ++layer; }
        return v;
      };
      uint32_t acc[4] = {0, 0, 0, 0};
      uint4 next = load_row(0); // one row ahead (a second row in flight measured slower: the kernel sits at 64 registers)
      for (uint32_t row = 0; row + 1 < rows; ++row) {
        const uint4 v = next;
        next = load_row(row + 1);
        const uint32_t x[4] = {acc[0] ^ v.x, acc[1] ^ v.y, acc[2] ^ v.z, acc[3] ^ v.w};
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k)
          acc[k] = row_lookup<0>(x[k], mine_shared) ^ row_lookup<1>(x[k], mine_shared) ^ row_lookup<2>(x[k], mine_shared) ^
                   row_lookup<3>(x[k], mine_shared);
      }
      // the last row enters without the row step: the 128 remainders now form a 128-word message
      uint32_t c = lookup4(tables, acc[0] ^ next.x) ^ acc[1] ^ next.y;
      c = lookup4(tables, c) ^ acc[2] ^ next.z;
      c = lookup4(tables, c) ^ acc[3] ^ next.w;
#pragma unroll
      for (uint32_t level = 0; level < kLevels; ++level) {
        const uint32_t ahead = __shfl_down_sync(0xffffffffu, c, 1u << level);
        c = lookup4(tables + (1 + level) * kTableWords, c) ^ ahead; // meaningful on lanes that are multiples of 2^(level+1)
      }
      if (lane == 0) term = mul_mod_device(lookup4(tables, c), args.multiplier[chunk]);
    }
    if (lane == 0) warp_terms[warp] = term;
    asm volatile("bar.sync %0, %1;" ::"r"(1u + group), "r"(kGroupWarps * 32u) : "memory");
    if (member == 0) {
      uint32_t sum = lane < kGroupWarps ? warp_terms[warp + lane] : 0u;
#pragma unroll
      for (uint32_t o = kGroupWarps / 2; o; o >>= 1) sum ^= __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        atomicXor(args.out + payload, part == 0 ? sum ^ args.closing : sum);
        if (kGather && !args.gather.entries) { // the payload's last part hands the checksum over and leaves the words as it found them
          __threadfence();
          if (atomicAdd(args.gather.arrivals + payload, 1u) + 1u == args.parts) {
            __threadfence();
            *args.gather.batch.publish[payload] = atomicExch(args.out + payload, 0u);
            atomicExch(args.gather.arrivals + payload, 0u);
          }
        }
      }
    }
    asm volatile("bar.sync %0, %1;" ::"r"(1u + group), "r"(kGroupWarps * 32u) : "memory");
  }
}

uint32_t crc32c_bytes(const uint8_t *data, size_t bytes, uint32_t crc) {
  static const std::vector<uint32_t> slices = [] { // slicing-by-8: slices[k][b] = b advanced by k + 1 bytes
    std::vector<uint32_t> t(8 * 256);
    for (uint32_t b = 0; b < 256; ++b) {
      uint32_t r = b;
      for (int i = 0; i < 8; ++i) r = (r & 1u) ? (r >> 1) ^ kPoly : r >> 1;
      t[b] = r;
    }
    for (uint32_t k = 1; k < 8; ++k)
      for (uint32_t b = 0; b < 256; ++b) t[k * 256 + b] = t[t[(k - 1) * 256 + b] & 0xffu] ^ (t[(k - 1) * 256 + b] >> 8);
    return t;
  }();
  const uint32_t *t = slices.data();
  uint32_t state = ~crc;
  for (; bytes >= 8; data += 8, bytes -= 8) {
    uint32_t lo, hi;
    memcpy(&lo, data, 4);
    memcpy(&hi, data + 4, 4);
    lo ^= state;
    state = t[7 * 256 + (lo & 0xffu)] ^ t[6 * 256 + ((lo >> 8) & 0xffu)] ^ t[5 * 256 + ((lo >> 16) & 0xffu)] ^ t[4 * 256 + (lo >> 24)] ^
            t[3 * 256 + (hi & 0xffu)] ^ t[2 * 256 + ((hi >> 8) & 0xffu)] ^ t[1 * 256 + ((hi >> 16) & 0xffu)] ^ t[hi >> 24];
  }
  for (; bytes; ++data, --bytes) state = t[(state ^ *data) & 0xffu] ^ (state >> 8);
  return ~state;
}

} // namespace

// CRC-32C of `count` payloads of `payload_bytes` each, `stride` bytes apart in device memory, into out[count]
// (device). `ctas` = 0 takes one CTA per SM. Payloads are whole 512-byte rows (every packed page is).
int launch_crc32c(const void *data, uint64_t stride, uint64_t payload_bytes, uint32_t count, uint32_t *out, uint32_t ctas,
                  cudaStream_t stream, const GatherSource *gather) {
  const bool batched = gather && !gather->entries;
  if ((!data && !batched) || !out || !count || !payload_bytes || payload_bytes % kRowBytes || stride < payload_bytes || (stride & 15u) ||
      (reinterpret_cast<uintptr_t>(data) & 15u)) {
    set_error("rk_crc32c_pages: payloads must be whole 512-byte rows, 16-byte aligned");
    return kInvalid;
  }
  int device = 0;
  if (int st = cuda_status(cudaGetDevice(&device), "cudaGetDevice")) return st;
  if (device < 0 || device >= 64) { set_error("device index out of range"); return kInvalid; }
  static std::mutex guard;
  static bool configured[64] = {};
  static int multiprocessors[64] = {};
  {
    std::lock_guard<std::mutex> lock(guard);
    if (!configured[device]) {
      const std::vector<uint32_t> &tables = host_tables();
      if (int st = cuda_status(cudaMemcpyToSymbol(g_tables, tables.data(), tables.size() * 4), "checksum tables")) return st;
      if (int st = cuda_status(cudaFuncSetAttribute(crc32c_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSharedBytes)), "checksum shared memory")) return st;
      if (int st = cuda_status(cudaFuncSetAttribute(crc32c_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSharedBytes)), "checksum shared memory")) return st;
      if (int st = cuda_status(cudaDeviceGetAttribute(&multiprocessors[device], cudaDevAttrMultiProcessorCount, device), "SM count")) return st;
      configured[device] = true;
    }
  }
  if (!ctas) ctas = uint32_t(multiprocessors[device]);
  const uint64_t rows = payload_bytes / kRowBytes;
  // enough parts to occupy the grid, never chunks of less than four rows
  const uint32_t parts = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>({uint64_t(kMaxParts), (uint64_t(ctas) * kGroups + count - 1) / count, rows / (4 * kGroupWarps)})));
  // The multipliers depend only on (payload size, parts): the last launch's set is kept.
  static ChecksumArgs cached{};
  static uint64_t cached_bytes = 0;
  ChecksumArgs args;
  {
    std::lock_guard<std::mutex> lock(guard);
    if (cached_bytes != payload_bytes || cached.parts != parts) {
      cached.parts = parts;
      const uint64_t chunks = uint64_t(parts) * kGroupWarps;
      cached.rows_low = uint32_t(rows / chunks);
      cached.extra = uint32_t(rows % chunks);
      // chunks have one of two lengths; walk from the last chunk backwards
      const uint32_t step_low = x_power_bytes(uint64_t(cached.rows_low) * kRowBytes);
      const uint32_t step_high = x_power_bytes((uint64_t(cached.rows_low) + 1) * kRowBytes);
      uint32_t power = 0x80000000u; // x^0: nothing follows the last chunk
      for (uint64_t g = chunks; g-- > 0;) {
        cached.multiplier[g] = power;
        power = mul_mod(power, g < cached.extra ? step_high : step_low);
      }
      // the state ~0 advanced over the payload, and the final inversion
      cached.closing = mul_mod(x_power_bytes(payload_bytes), 0xffffffffu) ^ 0xffffffffu;
      cached_bytes = payload_bytes;
    }
    args = cached;
  }
  args.data = static_cast<const uint8_t *>(data);
  args.stride = stride;
  args.out = out;
  args.payloads = count;
  args.gather = GatherArgs{};
  if (gather) {
    const uint32_t data_bytes = gather->data_bytes, scale_bytes = gather->scale_bytes;
    if ((!gather->entries && (!gather->batch || !gather->arrivals || count > kTierBatch)) ||
        data_bytes % kRowBytes || scale_bytes % kRowBytes || !gather->layers ||
        payload_bytes != uint64_t(gather->layers) * 2 * (uint64_t(data_bytes) + scale_bytes)) {
      set_error("seal: the payload is not a packed page of this pool");
      return kInvalid;
    }
    args.gather = GatherArgs{gather->entries, gather->extent_pages, data_bytes, scale_bytes,
                             2 * (data_bytes + scale_bytes) / kRowBytes, data_bytes / kRowBytes, scale_bytes / kRowBytes,
                             gather->arrivals, gather->entries ? PageBatch{} : *gather->batch};
  }
  // a batched seal finds its accumulators zero: the launch before it left them so
  if (!(gather && !gather->entries))
    if (int st = cuda_status(cudaMemsetAsync(out, 0, uint64_t(count) * 4, stream), "checksum clear")) return st;
  const uint32_t grid = uint32_t(std::min<uint64_t>(ctas, (uint64_t(count) * args.parts + kGroups - 1) / kGroups));
  if (gather) crc32c_kernel<true><<<grid, kWarps * 32, kSharedBytes, stream>>>(args);
  else crc32c_kernel<false><<<grid, kWarps * 32, kSharedBytes, stream>>>(args);
  return cuda_status(cudaGetLastError(), "checksum launch");
}

} // namespace rk

extern "C" int rk_crc32c_pages(const void *data, uint64_t stride, uint64_t payload_bytes, uint32_t count, uint32_t *out,
                               uint32_t ctas, void *stream) {
  return rk::launch_crc32c(data, stride, payload_bytes, count, out, ctas, static_cast<cudaStream_t>(stream), nullptr);
}

// CRC-32C of a host buffer, continuing from `crc` (0 to start): rk_crc32c_host(b, n, rk_crc32c_host(a, m, 0)) is the
// checksum of a followed by b (runtime/model/Crc32c.hpp:12-29).
extern "C" uint32_t rk_crc32c_host(const void *data, uint64_t bytes, uint32_t crc) {
  return rk::crc32c_bytes(static_cast<const uint8_t *>(data), size_t(bytes), crc);
}
