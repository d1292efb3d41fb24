// verify_attention.cu — the speculative-verify window (8 or 16 query rows per lane) over quantized
// pages as a dense tcgen05 contraction with TMEM accumulators.
//
// Semantics: the reference's verify tile
//   runtime/metal/kernels/common/paged_attention_tile.h:85-189   (scale fold, admission, online softmax)
//   runtime/metal/kernels/common/paged_attention_tile.h:208-349  (page loop, split partition, partial layout)
//   runtime/metal/kernels/decode/paged_attention.metal:23-192    (placement; tree masks)
// with partials and statistics in the layout of attention_tile.cu, so the same reduce merges them.
//
// One CTA owns (KV head, split, lane) like the reference grid. The fused rows (rows x 6 query heads,
// 48 or 96) are the M side of a 128-row UMMA tile (padding rows hold zero queries). Per group of 64
// tokens (two pages):
//   1. all eight warps expand the two pages' codes to fp16 — exact: int4/int8 codes and e4m3 values fit
//      fp16 — into K-major shared tiles with the 128-byte swizzle: K[token][dim], V^T[dim][token];
//   2. one thread issues S = Q.K^T: 16 x tcgen05.mma (M128, N64, K16), fp32 accumulators in TMEM;
//   3. warps 0-3 (one thread per row = one TMEM lane) read S, fold key scale and 1/16, apply the row's
//      admission rule, run the online softmax without any shuffle, fold the value scale into the
//      exponent (as decode_attention.cu) and write P as fp16 into its K-major tile; a row whose maximum
//      grew by more than 2^8 rescales its O row in TMEM (rows of a warp move together);
//   4. one thread issues O += P.V: 4 x tcgen05.mma (M128, N256, K16).
// Key codes travel as fp16 bit patterns (u * 2^-24 with u = code + 8, high nibbles x16 with the query
// carrying 1/16), the +8 leaves through 8 * sum(q) per row; value codes are centred exactly.
// Every mbarrier wait is bounded; TMEM is released on every path.
#include "common.cuh"

#include <cuda_fp16.h>

namespace rk {
namespace {

constexpr uint32_t kThreads = 256;
constexpr uint32_t kGroupTokens = 64;
constexpr uint32_t kM = 128, kD = 256, kG = 6, kHeads = 4;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

// shared-memory tiles (bytes); every tile starts 1024-aligned
constexpr uint32_t kQBytes = kM * kD * 2;            // 4 column blocks of [128 rows][64 elements]
constexpr uint32_t kKBytes = kGroupTokens * kD * 2;  // 4 column blocks of [64 rows][64 elements]
constexpr uint32_t kVBytes = kD * kGroupTokens * 2;  // 1 column block of [256 rows][64 elements]
constexpr uint32_t kPBytes = kM * kGroupTokens * 2;  // 1 column block of [128 rows][64 elements]
constexpr uint32_t kTileBytes = kQBytes + kKBytes + kVBytes + kPBytes;

struct Control {
  uint64_t s_done, o_done;
  uint32_t tmem_base;
  uint32_t error;
  float key_scale[kGroupTokens];
  float value_log2[kGroupTokens];
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool barrier_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (barrier_try(bar, parity)) return true;
    if (i > 16) __nanosleep(64);
  }
  return false;
}
// K-major, 128-byte swizzle shared-memory descriptor: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_descriptor(uint32_t address) {
  uint64_t desc = 0;
  desc |= uint64_t((address & 0x3FFFFu) >> 4);   // start address
  desc |= uint64_t(1) << 16;                      // leading byte offset (unused for swizzled K-major)
  desc |= uint64_t(1024 >> 4) << 32;              // stride byte offset
  desc |= uint64_t(1) << 46;                      // descriptor version (sm_100)
  desc |= uint64_t(2) << 61;                      // SWIZZLE_128B
  return desc;
}
// kind::f16 instruction descriptor: fp16 x fp16 -> fp32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_instruction(uint32_t m, uint32_t n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t address, float (&v)[32]) {
  uint32_t r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(address));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_store32(uint32_t address, const float (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(address), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                 "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                 "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                 "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                 "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                 "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                 "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                 "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
               : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float exp2_fast(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float log2_fast(float x) { float r; asm("lg2.approx.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) { const __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t *>(&h); }
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) { uint32_t r; asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r; }
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) { uint32_t r; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r; }

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside one column block.
__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

// Within a 16-byte chunk of 8 dims the element order is (0,4,1,5,2,6,3,7): the order in which an int4
// word yields its nibble pairs; queries and keys use the same order, so the contraction is unchanged.
// Positions 2,3,6,7 of that order (dims 1,5,3,7) carry the 16x of a high nibble for int4 keys.

template <uint32_t Format> struct Expand;

// int4: one 32-bit word = 8 dims of one token.
template <> struct Expand<RK_FORMAT_INT4> {
  // 8 key codes -> one 16-byte chunk of fp16 bit patterns (subnormal u * 2^-24; odd dims x16)
  __device__ static uint4 key_chunk(uint32_t x) {
    const uint32_t y = x >> 8;
    return make_uint4((x & 0x000F000Fu) ^ 0x00080008u, (x & 0x00F000F0u) ^ 0x00800080u,
                      (y & 0x000F000Fu) ^ 0x00080008u, (y & 0x00F000F0u) ^ 0x00800080u);
  }
};

struct VerifyArgs {
  const uint16_t *queries;
  float *partials;
  float *statistics;
  const rk_page_entry *const *tables;
  const uint32_t *row_masks;
  const rk_verify_params *lane_params;
  rk_kv_layer layer;
  uint32_t *status; // one word: non-zero when a bounded wait ran out
};

template <uint32_t Rows>
__global__ void __launch_bounds__(kThreads, 1)
verify_int4_kernel(VerifyArgs args) {
  constexpr uint32_t kRealRows = Rows * kG; // fused rows that exist
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t tiles = (smem_u32(dynamic_shared) + 1023u) & ~1023u;
  uint8_t *tile_ptr = dynamic_shared + (tiles - smem_u32(dynamic_shared));
  Control &ctl = *reinterpret_cast<Control *>(tile_ptr + kTileBytes);
  const uint32_t q_tile = tiles, k_tile = tiles + kQBytes, v_tile = k_tile + kKBytes, p_tile = v_tile + kVBytes;
  uint8_t *q_ptr = tile_ptr, *k_ptr = tile_ptr + kQBytes, *v_ptr = k_ptr + kKBytes, *p_ptr = v_ptr + kVBytes;

  const uint32_t tid = threadIdx.x, warp = tid / 32;
  const uint32_t kv_head = blockIdx.x, split = blockIdx.y, lane_index = blockIdx.z;
  rk_verify_params p = args.lane_params[lane_index];
  p.kv = args.layer;
  if (!rk_verify_contract_valid(&p) || p.row_capacity != Rows || split >= p.split_count) return;
  const uint32_t visible = p.committed_tokens + p.active_rows;
  const uint32_t pages = rk_pages_for(visible);
  const uint32_t per_split = rk_pages_per_split(pages, p.split_count);
  const uint32_t page_begin = split * per_split;
  if (page_begin >= pages) return; // a split without pages writes nothing
  const uint32_t page_end = min(pages, page_begin + per_split);
  const rk_page_entry *table = args.tables[lane_index];
  const uint32_t *row_masks = args.row_masks ? args.row_masks + uint64_t(lane_index) * p.row_capacity : nullptr;

  // ---- setup: barriers, TMEM, query tile ----------------------------------------------------------
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&ctl.s_done)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&ctl.o_done)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    ctl.error = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Query tile: row m = row*6 + g of this (lane, head); fp16, chunk order (0,4,1,5,2,6,3,7), odd dims /16.
  const uint16_t *queries = args.queries + (uint64_t(lane_index) * kHeads + kv_head) * (uint64_t(RK_VERIFY_CHUNK_STRIDE) * kG * kD);
  float q_sum = 0.0f; // of this thread's row (threads 0..127), for the +8 correction
  {
    // thread t handles row t/2 (all 128 rows), half of the 32 chunks each
    const uint32_t row = tid >> 1;
    const bool real = row < p.active_rows * kG;
    for (uint32_t c = (tid & 1u) * 16; c < (tid & 1u) * 16 + 16; ++c) { // chunk c = dims 8c..8c+7
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (real) raw = __ldg(reinterpret_cast<const uint4 *>(queries + uint64_t(row) * kD + 8 * c));
      const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
      float d[8];
#pragma unroll
      for (uint32_t i = 0; i < 4; ++i) { d[2 * i] = bf16_bits_to_float(words[i] & 0xffffu); d[2 * i + 1] = bf16_bits_to_float(words[i] >> 16); }
      const uint4 chunk = make_uint4(pack_half2(d[0], d[4]), pack_half2(d[1] * 0.0625f, d[5] * 0.0625f),
                                     pack_half2(d[2], d[6]), pack_half2(d[3] * 0.0625f, d[7] * 0.0625f));
      *reinterpret_cast<uint4 *>(q_ptr + (c >> 3) * (kM * 128) + swizzled(row, c & 7u)) = chunk;
      const __half2 *h = reinterpret_cast<const __half2 *>(&chunk);
      q_sum += __low2float(h[0]) + __high2float(h[0]) + __low2float(h[2]) + __high2float(h[2]) +
               16.0f * (__low2float(h[1]) + __high2float(h[1]) + __low2float(h[3]) + __high2float(h[3]));
    }
    q_sum += __shfl_xor_sync(0xffffffffu, q_sum, 1); // the two threads of a row
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = ctl.tmem_base;
  const uint32_t tmem_s = tmem, tmem_o = tmem + 64;
  // softmax threads: thread i < 128 owns fused row i = TMEM lane i
  __shared__ float q_sums[kM];
  if ((tid & 1u) == 0) q_sums[tid >> 1] = q_sum;
  __syncthreads();
  const uint32_t my_row = tid; // for tid < 128
  const float score_scale = rk_score_scale(p.score_scale, kD) * kLog2e;
  const float row_factor = ldexpf(score_scale, 24);
  const float row_offset = tid < kM ? -8.0f * q_sums[tid] * score_scale : 0.0f;
  const uint32_t query_row = my_row / kG;
  const uint32_t causal_limit = min(visible, p.committed_tokens + min(query_row, p.active_rows - 1) + 1);
  const uint32_t tree_mask = row_masks && query_row < p.row_capacity ? row_masks[query_row] : 0u;

  float row_max = -1.0e30f, row_sum = 0.0f;
  const uint32_t idesc_qk = umma_instruction(kM, kGroupTokens), idesc_pv = umma_instruction(kM, kD);
  const uint32_t data_bytes = kPageTokens * kHeads * kD / 2, scale_bytes = kPageTokens * kHeads * 4;
  uint32_t phase = 0;
  bool failed = false;

  for (uint32_t group_page = page_begin; group_page < page_end; group_page += 2, phase ^= 1u) {
    const uint32_t group_pages = min(2u, page_end - group_page);
    // ---- 1. expand the group's pages into the K and V^T tiles ---------------------------------------
    const uint8_t *keys[2] = {nullptr, nullptr}, *values[2] = {nullptr, nullptr};
#pragma unroll
    for (uint32_t local = 0; local < 2; ++local) {
      if (local >= group_pages) continue;
      const rk_page_entry entry = table[group_page + local];
      const uint32_t index = rk_entry_index(entry);
      const uint8_t *region = reinterpret_cast<const uint8_t *>(rk_entry_extent(entry)) + args.layer.offset;
      const uint64_t extent_pages = args.layer.extent_pages;
      keys[local] = region + uint64_t(index) * data_bytes + kv_head * 4096u;
      values[local] = region + extent_pages * (uint64_t(data_bytes) + scale_bytes) + uint64_t(index) * data_bytes + kv_head * 4096u;
      if (tid < kPageTokens) {
        const float *key_scales = reinterpret_cast<const float *>(region + extent_pages * data_bytes + uint64_t(index) * scale_bytes) + kv_head * kPageTokens;
        const float *value_scales = reinterpret_cast<const float *>(region + extent_pages * (2ull * data_bytes + scale_bytes) + uint64_t(index) * scale_bytes) + kv_head * kPageTokens;
        ctl.key_scale[local * kPageTokens + tid] = key_scales[tid];
        ctl.value_log2[local * kPageTokens + tid] = log2_fast(value_scales[tid]);
      }
    }
    // keys: a thread takes word w (8 dims) of a token; a warp reads whole 128-byte rows and writes whole
    // swizzled rows. An absent second page leaves finite codes behind (its tokens are never admitted).
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
      const uint32_t local = i >> 2, word = tid + (i & 3u) * kThreads, token = word >> 5, w = word & 31u;
      const uint32_t x = keys[local] ? __ldg(reinterpret_cast<const uint32_t *>(keys[local]) + word) : 0u;
      *reinterpret_cast<uint4 *>(k_ptr + (w >> 3) * (kGroupTokens * 128) + swizzled(local * kPageTokens + token, w & 7u)) =
          Expand<RK_FORMAT_INT4>::key_chunk(x);
    }
    // values: thread = (8 tokens, word w of 8 dims); an 8x8 transpose in registers turns the token-major
    // nibbles into 16-byte runs of 8 tokens for the dim-major tile. The eight lanes of a store phase
    // differ in their token run, so they fill one 128-byte row: no bank conflict.
    {
      const uint32_t run = tid & 7u, w = tid >> 3, local = run >> 2; // run = 16-byte chunk along the 64 tokens
      const uint8_t *source = local ? values[1] : values[0];
      uint32_t x[8];
#pragma unroll
      for (uint32_t t = 0; t < 8; ++t)
        x[t] = source ? __ldg(reinterpret_cast<const uint32_t *>(source) + ((run & 3u) * 8 + t) * 32 + w) : 0u;
#pragma unroll
      for (uint32_t b = 0; b < 4; ++b) { // byte b of each word = dims 8w+2b (low nibble), 8w+2b+1 (high nibble)
        uint32_t lo[4], hi[4];
        const uint32_t selector = b | (b << 4) | ((4 + b) << 8) | ((4 + b) << 12);
#pragma unroll
        for (uint32_t pair = 0; pair < 4; ++pair) {
          const uint32_t joined = __byte_perm(x[2 * pair], x[2 * pair + 1], selector);
          lo[pair] = sub_f16x2((joined & 0x000F000Fu) ^ 0x64086408u, 0x64086408u);                                  // 1024+u - 1032
          hi[pair] = fma_f16x2((joined & 0x00F000F0u) ^ 0x64806480u, 0x2C002C00u /* 1/16 */, 0xD480D480u /* -72 */); // (1024+16u)/16 - 72
        }
        const uint32_t dim = 8 * w + 2 * b;
        *reinterpret_cast<uint4 *>(v_ptr + swizzled(dim, run)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint4 *>(v_ptr + swizzled(dim + 1, run)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();

    // ---- 2. S = Q.K^T ---------------------------------------------------------------------------------
    if (tid == 128) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (uint32_t j = 0; j < 16; ++j) {
        const uint64_t a = umma_descriptor(q_tile + (j >> 2) * (kM * 128) + (j & 3u) * 32);
        const uint64_t b = umma_descriptor(k_tile + (j >> 2) * (kGroupTokens * 128) + (j & 3u) * 32);
        umma_f16(tmem_s, a, b, idesc_qk, j ? 1u : 0u);
      }
      umma_commit(smem_u32(&ctl.s_done));
    }

    // ---- 3. softmax: one thread per row ---------------------------------------------------------------
    if (warp < 4) {
      if (!failed && !barrier_wait(smem_u32(&ctl.s_done), phase)) { failed = true; ctl.error = 1; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_address = (warp * 32u) << 16;
      const uint32_t token_base = group_page * kPageTokens;
      const uint32_t group_tokens = group_pages * kPageTokens; // a split may end inside the group
      float scores[kGroupTokens];
      float group_max = -INFINITY;
#pragma unroll
      for (uint32_t half = 0; half < 2; ++half) {
        float raw[32];
        tmem_load32(tmem_s + lane_address + half * 32, raw);
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i) {
          const uint32_t t = half * 32 + i, token = token_base + t;
          const bool admitted = t < group_tokens &&
                                (!row_masks ? token < causal_limit
                                            : (token < p.committed_tokens || (token < visible && ((tree_mask >> (token - p.committed_tokens)) & 1u))));
          const float s = fmaf(raw[i], row_factor, row_offset) * ctl.key_scale[t];
          scores[t] = admitted ? s : -INFINITY;
          group_max = fmaxf(group_max, admitted ? s + fmaxf(ctl.value_log2[t], -40.0f) : -INFINITY);
        }
      }
      // Lazy rescale: the reference value only moves when the maximum grew by more than 2^8, so the
      // fp16 probabilities stay below 2^(8+6); rows of a warp move together (collective TMEM access).
      const bool grow = group_max > row_max + 8.0f;
      float scale = 1.0f;
      if (grow) {
        scale = exp2_fast(row_max - group_max);
        row_max = group_max;
        row_sum *= scale;
      }
      if (__any_sync(0xffffffffu, grow) && group_page != page_begin) {
#pragma unroll 1
        for (uint32_t c = 0; c < kD / 32; ++c) {
          float o[32];
          tmem_load32(tmem_o + lane_address + c * 32, o);
#pragma unroll
          for (uint32_t i = 0; i < 32; ++i) o[i] *= scale;
          tmem_store32(tmem_o + lane_address + c * 32, o);
        }
      }
#pragma unroll
      for (uint32_t c = 0; c < kGroupTokens / 8; ++c) {
        uint32_t packed[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
          float w[2];
#pragma unroll
          for (uint32_t e = 0; e < 2; ++e) {
            const uint32_t t = c * 8 + 2 * i + e;
            const float s = scores[t];
            const bool live = s != -INFINITY;
            w[e] = live ? exp2_fast(s + ctl.value_log2[t] - row_max + 6.0f) : 0.0f;
            row_sum += live ? exp2_fast(s - row_max) : 0.0f;
          }
          packed[i] = pack_half2(w[0], w[1]);
        }
        *reinterpret_cast<uint4 *>(p_ptr + swizzled(my_row, c)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();

    // ---- 4. O += P.V -------------------------------------------------------------------------------------
    if (tid == 128) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j)
        umma_f16(tmem_o, umma_descriptor(p_tile + j * 32), umma_descriptor(v_tile + j * 32), idesc_pv,
                 (group_page != page_begin || j) ? 1u : 0u);
      umma_commit(smem_u32(&ctl.o_done));
    }
    // every thread waits: the tiles are rewritten by the next group
    if (!failed && !barrier_wait(smem_u32(&ctl.o_done), phase)) { failed = true; ctl.error = 3; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    if (ctl.error) failed = true;
  }

  // ---- partial output: row i of O, un-normalised; statistics {reference exponent, sum} -------------------
  if (warp < 4) {
    const uint64_t slot = (uint64_t(lane_index) * kHeads + kv_head) * p.slot_splits + split;
    const uint32_t lane_address = (warp * 32u) << 16;
    float *out = args.partials + (slot * kRealRows + my_row) * kD;
#pragma unroll 1
    for (uint32_t c = 0; c < kD / 32; ++c) {
      float o[32];
      tmem_load32(tmem_o + lane_address + c * 32, o);
      if (my_row < kRealRows) {
#pragma unroll
        for (uint32_t i = 0; i < 32; i += 4)
          *reinterpret_cast<float4 *>(out + c * 32 + i) = make_float4(o[i] * 0.015625f, o[i + 1] * 0.015625f, o[i + 2] * 0.015625f, o[i + 3] * 0.015625f);
      }
    }
    if (my_row < kRealRows) {
      float *stats = args.statistics + (slot * kRealRows + my_row) * 2;
      stats[0] = failed ? -INFINITY : row_max * kLn2;
      stats[1] = failed ? 0.0f : row_sum;
    }
  }
  if (failed && tid == 0) atomicExch(args.status, 1u);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

} // namespace
} // namespace rk

using namespace rk;

// verify_attention_int4_split / verify_tree_attention_int4_split for 8 or 16 rows as a tcgen05
// contraction (decode/paged_attention.metal:23-192). Same arguments and scratch layout as
// rk_attention_verify_split; `status` (one device word, may be null-initialised by the caller) turns
// non-zero when a bounded wait ran out. Merge with rk_attention_verify_reduce.
extern "C" int rk_attention_verify_split_tc(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                                            uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits, const void *queries,
                                            float *partials, float *statistics, const rk_page_entry *const *tables,
                                            const uint32_t *row_masks, const rk_verify_params *lane_params,
                                            rk_kv_layer layer, uint32_t *status, void *stream) {
  if (kv_heads != kHeads || query_heads != kHeads * kG || head_dim != kD || format != RK_FORMAT_INT4 ||
      (row_capacity != 8 && row_capacity != 16)) {
    set_error("rk_attention_verify_split_tc: built for int4, 4 KV heads x 24 query heads x 256, 8 or 16 rows");
    return kUnsupported;
  }
  if (!lanes || !grid_splits || grid_splits > RK_VERIFY_MAX_SPLITS || !queries || !partials || !statistics || !tables ||
      !lane_params || !layer.extent_pages || !status) {
    set_error("rk_attention_verify_split_tc: invalid arguments");
    return kInvalid;
  }
  constexpr size_t shared_bytes = 1024 + kTileBytes + sizeof(Control);
  VerifyArgs args{static_cast<const uint16_t *>(queries), partials, statistics, tables, row_masks, lane_params, layer, status};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(kHeads, grid_splits, lanes);
  if (row_capacity == 8) {
    if (int st = cuda_status(cudaFuncSetAttribute(verify_int4_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(shared_bytes)), "verify shared memory")) return st;
    verify_int4_kernel<8><<<grid, kThreads, shared_bytes, s>>>(args);
  } else {
    if (int st = cuda_status(cudaFuncSetAttribute(verify_int4_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(shared_bytes)), "verify shared memory")) return st;
    verify_int4_kernel<16><<<grid, kThreads, shared_bytes, s>>>(args);
  }
  return cuda_status(cudaGetLastError(), "verify tcgen05 launch");
}
