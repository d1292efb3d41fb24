// verify_attention.cu — the speculative-verify window (8 or 16 query rows per lane) over int4 pages as
// a dense tcgen05 contraction with TMEM accumulators, warp-specialised and pipelined.
//
// Semantics: the reference's verify tile
//   runtime/metal/kernels/common/paged_attention_tile.h:85-189   (scale fold, admission, online softmax)
//   runtime/metal/kernels/common/paged_attention_tile.h:208-349  (page loop, split partition, partial layout)
//   runtime/metal/kernels/decode/paged_attention.metal:23-192    (placement; tree masks)
// with partials and statistics in the layout of attention_tile.cu, so the same reduce merges them.
//
// One CTA owns (KV head, split, lane) like the reference grid. The fused rows (rows x 6 query heads,
// 48 or 96) are the M side of a 128-row UMMA tile (padding rows hold zero queries). The pages of the
// split are taken in groups of 64 tokens (two pages). Tensor memory holds O (256 columns), S twice
// (2 x 64, the fp16 probabilities overwrite the first half of their S) and the query tile itself (128):
// both contractions take their A operand from tensor memory, shared memory only carries the page data.
// Roles:
//   warp 24 (one thread)  TMA: the two pages' K and V slabs of this head (32-row boxes of the window
//                         map, 128-byte swizzle) and their scales into a ring of four raw stages.
//   warps 16-23           two teams of four warps, team t takes the groups g = t (mod 2): expand the raw
//                         nibbles to fp16 — exact — into stage t of the K-major swizzled operand tiles
//                         K[position][dim] and V^T[dim][position] (an 8x8 transpose in registers), and
//                         prepare the per-token scale triples.
//   warp 25               tcgen05.mma S(g) = Q.K^T (16 x M128 N64 K16) into S buffer g&1;
//   warp 26               tcgen05.mma O += P.V (4 x M128 N256 K16). Both walk their loop as a whole warp
//                         and one elected lane issues, which keeps descriptors on the uniform datapath.
//                         P(g) overwrites the first half of S(g); QK(g+2) waits for PV(g) to land.
//   warps 0-15            softmax, four threads per row (= TMEM lane), 16 tokens each: read S, fold key
//                         scale and 1/16, admit, online maximum (one exchange through shared memory),
//                         value scale folded into the exponent, P as fp16 back into tensor memory; a row
//                         whose maximum grew by more than 2^8 rescales its O row (rows of a warp move
//                         together).
// Key codes travel as fp16 bit patterns (u * 2^-24 with u = code + 8, high nibbles x16 with the query
// carrying 1/16), the +8 leaves through 8 * sum(q) per row; value codes are centred exactly. Inside a
// group both contractions index the tokens through one fixed permutation (position 8r+j holds token
// 8j+r), which makes every shared-memory access of the two expansions conflict-free.
// Every mbarrier wait is bounded and gives up at once after any wait failed; TMEM is released on
// every path.
#include "common.cuh"
#include "window.cuh"

#include <cuda_bf16.h>
#include <type_traits>
#include <cuda_fp16.h>

namespace rk {
namespace {

constexpr uint32_t kRowThreads = 4;                      // softmax threads per fused row (one per warp of the row's quarter)
constexpr uint32_t kSoftmaxWarps = 4 * kRowThreads;
constexpr uint32_t kRowTokens = 64 / kRowThreads;         // contraction positions of a group per softmax thread
constexpr uint32_t kExpandWarps = 8;   // kTileStages teams: team t expands the groups g = t (mod kTileStages) into operand stage t
constexpr uint32_t kSoftmaxThreads = kSoftmaxWarps * 32;
constexpr uint32_t kThreads = (kSoftmaxWarps + kExpandWarps + 3) * 32;
constexpr uint32_t kTmaWarp = kSoftmaxWarps + kExpandWarps, kScoreWarp = kTmaWarp + 1, kValueWarp = kTmaWarp + 2;
constexpr uint32_t kScaleStages = 4;
constexpr uint32_t kGroupTokens = 64;
constexpr uint32_t kM = 128, kD = 256, kG = 6, kHeads = 4;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

// shared-memory tiles (bytes); every tile starts 1024-aligned
constexpr uint32_t kKBytes = kGroupTokens * kD * 2;  // 4 column blocks of [64 rows][64 elements]
constexpr uint32_t kVBytes = kD * kGroupTokens * 2;  // 1 column block of [256 rows][64 elements]
constexpr uint32_t kMaxRawStages = 4;

// What differs between the stored formats: the size of one head's K (or V) slab of a page, whether
// scales exist, how codes become 16-bit tensor-core operands, and the depth of the raw ring that fits.
//   int4      fp16 operands; key codes as u * 2^-24 with u = code + 8 (the +8 leaves through sum(q)),
//             odd dims x16 against queries / 16, dims of every 8 in the order (0,4,1,5,2,6,3,7).
//   int8      fp16 operands; key codes as u * 2^-24 with u = code + 128; values exact (1024 + u - 1152).
//   fp8 e4m3  fp16 operands, exact (cvt); queries staged as fp16 like the reference's fp8 tile
//             (paged_attention_fp8_tile.h:34-60).
//   bf16      bf16 operands (bits as stored). Both operands of a contraction are of one kind, so the
//             probabilities are bf16 too: a high and a low part, contracted one after the other (16 bits).
template <uint32_t Format> struct Traits;
template <> struct Traits<RK_FORMAT_INT4> {
  static constexpr uint32_t kSlab = 4096, kRawStages = 4, kTileStages = 2;
  static constexpr bool kScales = true, kBf16 = false;
  static constexpr float kKeyOffset = 8.0f;
  static constexpr int kKeyShift = 24;
};
template <> struct Traits<RK_FORMAT_INT8> {
  static constexpr uint32_t kSlab = 8192, kRawStages = 2, kTileStages = 2;
  static constexpr bool kScales = true, kBf16 = false;
  static constexpr float kKeyOffset = 128.0f;
  static constexpr int kKeyShift = 24;
};
template <> struct Traits<RK_FORMAT_FP8E4M3> {
  static constexpr uint32_t kSlab = 8192, kRawStages = 2, kTileStages = 2;
  static constexpr bool kScales = true, kBf16 = false;
  static constexpr float kKeyOffset = 0.0f;
  static constexpr int kKeyShift = 0;
};
template <> struct Traits<RK_FORMAT_BF16> {
  static constexpr uint32_t kSlab = 16384, kRawStages = 2, kTileStages = 1; // the slabs are large: one operand stage, two raw stages
  static constexpr bool kScales = false, kBf16 = true;
  static constexpr float kKeyOffset = 0.0f;
  static constexpr int kKeyShift = 0;
};
// raw stage: K0 | K1 | V0 | V1 | ks0 ks1 vs0 vs1 (128 B each) | pad to 1 KiB
template <uint32_t Format> __host__ __device__ constexpr uint32_t raw_stage_bytes() { return 4 * Traits<Format>::kSlab + 1024; }
template <uint32_t Format> __host__ __device__ constexpr uint32_t tile_bytes() {
  return Traits<Format>::kTileStages * (kKBytes + kVBytes) + Traits<Format>::kRawStages * raw_stage_bytes<Format>();
}
// tensor-memory columns
constexpr uint32_t kTmemO = 0, kTmemS = 256, kTmemQ = 384; // S twice (64 columns each); P(g) overwrites the first half of S(g)

struct Control {
  uint64_t raw_full[kMaxRawStages], raw_free[kMaxRawStages];
  uint64_t k_full[2], k_free[2], v_full[2], v_free[2], s_full[2], p_full[2], p_free[2], scale_free[kScaleStages];
  uint64_t drained[2]; // one per issue warp: every contraction it issued has completed
  uint32_t tmem_base;
  uint32_t error;
  uint32_t spin_limit; // directly after `error`: barrier_wait reads it through the error pointer
  float q_sums[kM];
  float exchange[2][kM][kRowThreads]; // the part-row maxima of a group (and, at the end, the part-row sums)
  float4 scales[kScaleStages][kGroupTokens]; // {key scale, log2 value scale, 2^-6 / value scale, -}
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void barrier_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void barrier_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void barrier_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool barrier_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Waits for completion number `count` (0-based) of a barrier. Bounded: gives up after the launch's poll limit,
// or at once when another wait of this CTA already gave up; either way `error` ends non-zero.
// `error` points at Control::error; the word after it holds the poll limit of this launch.
__device__ __forceinline__ void barrier_wait(uint64_t *barrier, uint32_t count, volatile uint32_t *error) {
  const uint32_t bar = smem_u32(barrier), parity = count & 1u, limit = error[1];
  for (uint32_t i = 0; i < limit; ++i) {
    if (barrier_try(bar, parity)) return; // try_wait itself suspends the thread for a while
    if ((i & 63u) == 63u) {
      if (*error) return;
      if (i > 4096) __nanosleep(256);
    }
  }
  *error = 1;
}
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap *map, int32_t row, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(0), "r"(row), "r"(bar) : "memory");
}
// Asks L2 for `bytes` of global memory (16-byte granular) without a destination: the later copy of the same
// bytes into shared memory then pays the L2 latency, not the HBM one.
__device__ __forceinline__ void prefetch_l2(uint64_t address, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(address), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
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
// kind::f16 instruction descriptor: 16-bit operands (0 = fp16, 1 = bf16) -> fp32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_instruction(uint32_t m, uint32_t n, uint32_t a_format = 0, uint32_t b_format = 0) {
  return (1u << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// True in exactly one lane of a converged warp; unlike a test of the lane index it keeps the surrounding
// control flow warp-uniform, so descriptors and addresses stay on the uniform datapath.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
  return pred != 0;
}
// A operand from tensor memory: lane = row, each 32-bit column two consecutive K elements.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *barrier) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(barrier)) : "memory");
}
__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void async_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
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
__device__ __forceinline__ void tmem_load16(uint32_t address, float (&v)[16]) {
  uint32_t r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(address));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_store8(uint32_t address, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_load_scores(uint32_t address, float (&v)[16]) { tmem_load16(address, v); }
__device__ __forceinline__ void tmem_store_packed(uint32_t address, const uint32_t (&v)[8]) { tmem_store8(address, v); }
__device__ __forceinline__ float exp2_fast(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float log2_fast(float x) { float r; asm("lg2.approx.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) { const __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t *>(&h); }
__device__ __forceinline__ uint32_t pack_bfloat2(float lo, float hi) { const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<const uint32_t *>(&h); }
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) { uint32_t r; asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r; }
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) { uint32_t r; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r; }
// (a & mask) ^ flip in one logic instruction; both constants sit in registers.
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t mask, uint32_t flip) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(mask), "r"(flip));
  return r;
}
__device__ __forceinline__ uint32_t register_constant(uint32_t value) {
  uint32_t r;
  asm volatile("mov.b32 %0, %1;" : "=r"(r) : "r"(value));
  return r;
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside one 128-byte-swizzled block.
__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

// Within a 16-byte operand chunk of 8 dims the element order is (0,4,1,5,2,6,3,7): the order in which
// an int4 word yields its nibble pairs; queries and keys use the same order, so the contraction is
// unchanged. Dims 1,5,3,7 of each 8 carry the 16x of a high nibble on the key side, 1/16 on the query.

struct VerifyArgs {
  const uint16_t *queries;
  float *partials;
  float *statistics;
  const rk_page_entry *const *tables;
  const uint32_t *row_masks;
  const rk_verify_params *lane_params;
  rk_kv_layer layer;
  uint64_t window_base;
  uint32_t *status; // one word: non-zero when a bounded wait ran out
  uint32_t spin_limit;      // polls a wait may take (kSpinLimit in production; the timeout probe passes a few thousand)
  uint32_t withheld_groups; // timeout probe only: the TMA warp never streams the last groups of a split
  // prefill launches (grid z = 8-row tile of the chunk): the sequence's table and parameters instead of per-lane ones
  const rk_page_entry *prefill_table;
  rk_prefill_params prefill;
};


// ---- raw codes -> 16-bit operand tiles, one team of `Team` threads (e = 0..Team-1) per 64-token group ---------
// K tile: four column blocks of [64 positions][64 dims], 128-byte rows, 128-byte swizzle. V^T tile: one block
// of [256 dims][64 positions]. `raw` = K0 | K1 | V0 | V1 slabs as TMA left them (128-byte rows, swizzled).
// `valid` = positions of the group whose tokens exist; formats whose stale bytes can decode to NaN or
// infinity (fp8, bf16) get zeros at value positions past it, so a zero probability meets a finite value.

template <uint32_t Format> struct Expand;

__device__ __forceinline__ uint32_t mask_pair(uint32_t value, uint32_t position, uint32_t valid) {
  return value & ((position < valid ? 0x0000FFFFu : 0u) | (position + 1 < valid ? 0xFFFF0000u : 0u));
}

template <> struct Expand<RK_FORMAT_INT4> {
  // position 8r+j holds token 8j+r: every access of both transposes is conflict-free
  __device__ static uint32_t token_of(uint32_t position) { return 8 * (position & 7u) + (position >> 3); }
  template <uint32_t Team> __device__ static void keys(const uint8_t *raw, uint8_t *k_stage, uint32_t e) {
    const uint32_t low_mask = register_constant(0x000F000Fu), high_mask = register_constant(0x00F000F0u);
    const uint32_t key_low = register_constant(0x00080008u), key_high = register_constant(0x00800080u);
    // a thread takes a raw 16-byte chunk (32 dims of one token) = four operand chunks. The eight lanes of an
    // access phase take tokens 8k + t and chunks c0 ^ k.
#pragma unroll
    for (uint32_t i = 0; i < (512 + Team - 1) / Team; ++i) {
      const uint32_t item = e + i * Team;
      if (512 % Team && item >= 512) break;
      const uint32_t k8 = item & 7u, c = ((item >> 3) & 7u) ^ k8, t = item >> 6;
      const uint32_t token = 8 * k8 + t, position = 8 * t + k8;
      const uint4 x = *reinterpret_cast<const uint4 *>(raw + (token >> 5) * 4096 + swizzled(token & 31u, c));
      const uint32_t words[4] = {x.x, x.y, x.z, x.w};
      uint8_t *block = k_stage + (c >> 1) * (kGroupTokens * 128);
#pragma unroll
      for (uint32_t w = 0; w < 4; ++w) {
        const uint32_t y = words[w] >> 8;
        *reinterpret_cast<uint4 *>(block + swizzled(position, ((c & 1u) << 2) + w)) =
            make_uint4(and_xor(words[w], low_mask, key_low), and_xor(words[w], high_mask, key_high),
                       and_xor(y, low_mask, key_low), and_xor(y, high_mask, key_high));
      }
    }
  }
  template <uint32_t Team> __device__ static void values(const uint8_t *raw, uint8_t *v_stage, uint32_t e, uint32_t) {
    const uint32_t low_mask = register_constant(0x000F000Fu), high_mask = register_constant(0x00F000F0u);
    const uint32_t value_low = register_constant(0x64086408u), value_high = register_constant(0x64806480u);
    // thread = (r8, word w of 8 dims) takes tokens 8j + r8, j = 0..7, and transposes 8x8 in registers: each
    // dim gets a 16-byte run of eight tokens at contraction positions 8*r8 + j.
#pragma unroll
    for (uint32_t half = 0; half < (256 + Team - 1) / Team; ++half) {
      const uint32_t unit = e + half * Team, r8 = unit & 7u, w = unit >> 3;
      if ((256 % Team || Team > 256) && unit >= 256) break;
      uint32_t x[8];
#pragma unroll
      for (uint32_t j = 0; j < 8; ++j)
        x[j] = *reinterpret_cast<const uint32_t *>(raw + (2 + (j >> 2)) * 4096 + swizzled(8 * (j & 3u) + r8, w >> 2) + (w & 3u) * 4);
#pragma unroll
      for (uint32_t byte = 0; byte < 4; ++byte) { // byte of each word = dims 8w+2*byte (low nibble), +1 (high nibble)
        uint32_t lo[4], hi[4];
        const uint32_t selector = byte | (byte << 4) | ((4 + byte) << 8) | ((4 + byte) << 12);
#pragma unroll
        for (uint32_t pair = 0; pair < 4; ++pair) {
          const uint32_t joined = __byte_perm(x[2 * pair], x[2 * pair + 1], selector);
          lo[pair] = sub_f16x2(and_xor(joined, low_mask, value_low), value_low);                                   // 1024+u - 1032
          hi[pair] = fma_f16x2(and_xor(joined, high_mask, value_high), 0x2C002C00u /* 1/16 */, 0xD480D480u /* -72 */); // (1024+16u)/16 - 72
        }
        const uint32_t dim = 8 * w + 2 * byte;
        *reinterpret_cast<uint4 *>(v_stage + swizzled(dim, r8)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint4 *>(v_stage + swizzled(dim + 1, r8)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      }
    }
  }
};

// One-byte codes (int8, fp8): K rows are 256 bytes = two 128-byte TMA rows; V rows (one dim) are 32 bytes, four
// dims to a TMA row. Positions are the tokens in order.
template <bool kFloat8> struct ExpandBytes {
  __device__ static uint32_t token_of(uint32_t position) { return position; }
  // four codes -> two registers of two 16-bit operands
  __device__ static void key_pairs(uint32_t word, uint32_t &first, uint32_t &second) {
    if (kFloat8) {
      asm("{\n.reg .b16 lo, hi;\nmov.b32 {lo, hi}, %2;\ncvt.rn.f16x2.e4m3x2 %0, lo;\ncvt.rn.f16x2.e4m3x2 %1, hi;\n}" : "=r"(first), "=r"(second) : "r"(word));
    } else { // u = code + 128 as fp16 bits: u * 2^-24
      const uint32_t flipped = word ^ 0x80808080u;
      first = __byte_perm(flipped, 0, 0x4140);
      second = __byte_perm(flipped, 0, 0x4342);
    }
  }
  __device__ static void value_pairs(uint32_t word, uint32_t &first, uint32_t &second) {
    if (kFloat8) {
      key_pairs(word, first, second);
    } else { // 1024 + u, minus 1152: the code itself
      const uint32_t flipped = word ^ 0x80808080u;
      first = sub_f16x2(__byte_perm(flipped, 0x64646464u, 0x4140), 0x64806480u);
      second = sub_f16x2(__byte_perm(flipped, 0x64646464u, 0x4342), 0x64806480u);
    }
  }
  template <uint32_t Team> __device__ static void keys(const uint8_t *raw, uint8_t *k_stage, uint32_t e) {
    // item = (token, 16-byte chunk c of its 256-byte row): 16 dims -> two operand chunks. The eight lanes of a
    // shared-memory phase take chunks c..c+3 of token t and chunks c+4..c+7 of token t ^ 1: their raw rows differ by 2
    // and their chunk sets by bit 2 (eight distinct chunks to read), and their operand rows differ in bit 0 (eight
    // distinct chunks to write).
#pragma unroll
    for (uint32_t i = 0; i < (1024 + Team - 1) / Team; ++i) {
      const uint32_t item = e + i * Team, c = item & 15u, token = (item >> 4) ^ ((item >> 2) & 1u);
      if (1024 % Team && item >= 1024) break;
      const uint32_t row = 2 * (token & 31u) + (c >> 3);
      const uint4 x = *reinterpret_cast<const uint4 *>(raw + (token >> 5) * 8192 + swizzled(row, c & 7u));
      uint32_t out[8];
      key_pairs(x.x, out[0], out[1]); key_pairs(x.y, out[2], out[3]);
      key_pairs(x.z, out[4], out[5]); key_pairs(x.w, out[6], out[7]);
      uint8_t *block = k_stage + (c >> 2) * (kGroupTokens * 128);
      *reinterpret_cast<uint4 *>(block + swizzled(token, 2 * (c & 3u))) = make_uint4(out[0], out[1], out[2], out[3]);
      *reinterpret_cast<uint4 *>(block + swizzled(token, 2 * (c & 3u) + 1)) = make_uint4(out[4], out[5], out[6], out[7]);
    }
  }
  template <uint32_t Team> __device__ static void values(const uint8_t *raw, uint8_t *v_stage, uint32_t e, uint32_t valid) {
    // item = (page, dim, half h of its 32 tokens): 16 tokens -> two operand chunks of the dim's row. The eight lanes
    // of a shared-memory phase take eight consecutive dims of one half: two raw rows whose chunk sets have opposite
    // parity (eight distinct chunks to read), eight operand rows whose swizzles differ (eight distinct chunks to write).
#pragma unroll
    for (uint32_t i = 0; i < (1024 + Team - 1) / Team; ++i) {
      const uint32_t item = e + i * Team, h = (item >> 3) & 1u, dim = (item & 7u) | ((item >> 1) & 248u), page = item >> 9;
      if (1024 % Team && item >= 1024) break;
      const uint4 x = *reinterpret_cast<const uint4 *>(raw + (2 + page) * 8192 + swizzled(dim >> 2, 2 * (dim & 3u) + h));
      uint32_t out[8];
      value_pairs(x.x, out[0], out[1]); value_pairs(x.y, out[2], out[3]);
      value_pairs(x.z, out[4], out[5]); value_pairs(x.w, out[6], out[7]);
      const uint32_t position = 32 * page + 16 * h;
      if (kFloat8 && position + 16 > valid) {
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) out[r] = mask_pair(out[r], position + 2 * r, valid);
      }
      *reinterpret_cast<uint4 *>(v_stage + swizzled(dim, 4 * page + 2 * h)) = make_uint4(out[0], out[1], out[2], out[3]);
      *reinterpret_cast<uint4 *>(v_stage + swizzled(dim, 4 * page + 2 * h + 1)) = make_uint4(out[4], out[5], out[6], out[7]);
    }
  }
};
template <> struct Expand<RK_FORMAT_INT8> : ExpandBytes<false> {};
template <> struct Expand<RK_FORMAT_FP8E4M3> : ExpandBytes<true> {};

// bf16: the stored bits are the operands; the expansion is a re-tiling copy. K rows are 512 bytes = four TMA
// rows (= the four column blocks); V rows (one dim) are 64 bytes, two dims to a TMA row.
template <> struct Expand<RK_FORMAT_BF16> {
  __device__ static uint32_t token_of(uint32_t position) { return position; }
  template <uint32_t Team> __device__ static void keys(const uint8_t *raw, uint8_t *k_stage, uint32_t e) {
#pragma unroll
    for (uint32_t i = 0; i < (2048 + Team - 1) / Team; ++i) {
      const uint32_t item = e + i * Team, c = item & 31u, token = item >> 5;
      if (2048 % Team && item >= 2048) break;
      const uint32_t row = 4 * (token & 31u) + (c >> 3);
      const uint4 x = *reinterpret_cast<const uint4 *>(raw + (token >> 5) * 16384 + swizzled(row, c & 7u));
      *reinterpret_cast<uint4 *>(k_stage + (c >> 3) * (kGroupTokens * 128) + swizzled(token, c & 7u)) = x;
    }
  }
  template <uint32_t Team> __device__ static void values(const uint8_t *raw, uint8_t *v_stage, uint32_t e, uint32_t valid) {
#pragma unroll
    for (uint32_t i = 0; i < (2048 + Team - 1) / Team; ++i) {
      // the eight lanes of a shared-memory phase take the four 16-byte pieces of dim d and of dim d ^ 5: raw rows two
      // apart with the other half of the row (eight distinct chunks to read), operand rows whose swizzles differ in
      // bit 2 (eight distinct chunks to write)
      const uint32_t item = e + i * Team, q = item & 3u, page = item >> 10;
      const uint32_t dim = ((item >> 2) & 255u) ^ (item & 4u); // odd dims trade places with the odd dim four further
      if (2048 % Team && item >= 2048) break;
      uint4 x = *reinterpret_cast<const uint4 *>(raw + (2 + page) * 16384 + swizzled(dim >> 1, 4 * (dim & 1u) + q));
      const uint32_t position = 32 * page + 8 * q;
      if (position + 8 > valid) {
        x.x = mask_pair(x.x, position, valid); x.y = mask_pair(x.y, position + 2, valid);
        x.z = mask_pair(x.z, position + 4, valid); x.w = mask_pair(x.w, position + 6, valid);
      }
      *reinterpret_cast<uint4 *>(v_stage + swizzled(dim, 4 * page + q)) = x;
    }
  }
};

// kPrefill: the CTA's window is `Rows` consecutive rows of a prefill chunk (prefill/paged_attention.metal:7-67), starting
// at row Rows*blockIdx.z: one 8-row tile, or, for unsplit plans, two tiles at once (a 16-row causal window is exactly
// two consecutive tiles). Queries [kv_head][stride][group][D]; each tile keeps its own partial slot
// (tile*heads + head)*splits + split of 48 fused rows.
template <uint32_t Format, uint32_t Rows, bool kTree, bool kPrefill = false>
__global__ void __launch_bounds__(kThreads, 1)
window_attention_kernel(const __grid_constant__ CUtensorMap head_map, VerifyArgs args) {
  using Kind = Traits<Format>;
  constexpr uint32_t kRealRows = Rows * kG;                       // fused rows that exist
  constexpr uint32_t kQuarters = (kRealRows + 31) / 32;           // 32-row quarters of the tile that hold real rows
  constexpr uint32_t kActiveSoftmax = kQuarters * kRowThreads * 32; // softmax threads that take part
  constexpr uint32_t kSlab = Kind::kSlab, kRawStages = Kind::kRawStages, kRawStageBytes = raw_stage_bytes<Format>();
  constexpr uint32_t kRawScaleOffset = 4 * kSlab;
  // int8 and fp8 keep only two raw stages (66 KB) in flight per SM, short of what HBM latency asks for: they also
  // request the groups behind the ring from HBM into L2. The other formats measured slower with it.
  constexpr bool kPrefetch = Kind::kSlab == 8192;
  constexpr uint32_t kPrefetchGroups = kRawStages + 4; // groups between the shared-memory copy and the L2 request
  // Softmax warps of quarters without a real row (12 of 16 for one row, 8 for eight rows, 4 for sixteen) expand too.
  constexpr uint32_t kIdleWarps = (4 - kQuarters) * kRowThreads;
  constexpr uint32_t kTileStages = Kind::kTileStages, kExpandThreads = (kExpandWarps + kIdleWarps) * 32 / kTileStages; // threads of one team
  static_assert(kRawStages % kTileStages == 0, "a raw stage belongs to one expander team: its barrier is never waited on two completions behind");
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t tiles = (smem_u32(dynamic_shared) + 1023u) & ~1023u;
  uint8_t *tile_ptr = dynamic_shared + (tiles - smem_u32(dynamic_shared));
  Control &ctl = *reinterpret_cast<Control *>(tile_ptr + tile_bytes<Format>());
  volatile uint32_t *error = &ctl.error;
  const uint32_t k_tile = tiles, v_tile = k_tile + kTileStages * kKBytes, raw_tile = v_tile + kTileStages * kVBytes; // K stages | V stages | raw ring
  uint8_t *k_ptr = tile_ptr, *v_ptr = k_ptr + kTileStages * kKBytes;
  const uint8_t *raw_ptr = v_ptr + kTileStages * kVBytes;

  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t kv_head = blockIdx.x, split = blockIdx.y, lane_index = blockIdx.z;
  rk_verify_params p;
  if (kPrefill) {
    const rk_prefill_params &chunk = args.prefill;
    const uint32_t tile_start = lane_index * Rows;
    if (!rk_prefill_contract_valid(&chunk) || tile_start >= chunk.rows || (Rows != RK_PREFILL_TILE_ROWS && chunk.split_count != 1)) return;
    p.committed_tokens = chunk.committed_tokens + tile_start;
    p.page_table_entries = chunk.page_table_entries;
    p.split_count = p.slot_splits = chunk.split_count;
    p.active_rows = min(Rows, chunk.rows - tile_start);
    p.row_capacity = Rows;
    p.score_scale = chunk.score_scale;
  } else {
    p = args.lane_params[lane_index];
  }
  p.kv = args.layer;
  if (!rk_verify_contract_valid(&p) || p.row_capacity != Rows || split >= p.split_count) return;
  const uint32_t visible = p.committed_tokens + p.active_rows;
  const uint32_t pages = rk_pages_for(visible);
  const uint32_t per_split = rk_pages_per_split(pages, p.split_count);
  const uint32_t page_begin = split * per_split;
  if (page_begin >= pages) return; // a split without pages writes nothing
  const uint32_t page_end = min(pages, page_begin + per_split);
  const uint32_t groups = (page_end - page_begin + 1) / 2;
  const rk_page_entry *table = kPrefill ? args.prefill_table : args.tables[lane_index];
  const uint32_t *row_masks = kTree ? args.row_masks + uint64_t(lane_index) * p.row_capacity : nullptr;

  // ---- setup: barriers, TMEM, query tile ----------------------------------------------------------
  if (tid == 0) {
    for (uint32_t r = 0; r < kRawStages; ++r) {
      barrier_init(smem_u32(&ctl.raw_full[r]), 1);
      barrier_init(smem_u32(&ctl.raw_free[r]), kExpandThreads);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      barrier_init(smem_u32(&ctl.k_full[b]), kExpandThreads);
      barrier_init(smem_u32(&ctl.v_full[b]), kExpandThreads);
      barrier_init(smem_u32(&ctl.k_free[b]), 1);
      barrier_init(smem_u32(&ctl.v_free[b]), 1);
      barrier_init(smem_u32(&ctl.s_full[b]), 1);
      barrier_init(smem_u32(&ctl.p_free[b]), 1);
      barrier_init(smem_u32(&ctl.p_full[b]), kActiveSoftmax);
    }
    for (uint32_t b = 0; b < kScaleStages; ++b) barrier_init(smem_u32(&ctl.scale_free[b]), kActiveSoftmax);
    barrier_init(smem_u32(&ctl.drained[0]), 1);
    barrier_init(smem_u32(&ctl.drained[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    ctl.error = 0;
    ctl.spin_limit = args.spin_limit;
  }
  if (warp == kTmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  const uint32_t tmem_o = tmem + kTmemO, tmem_s = tmem + kTmemS, tmem_q = tmem + kTmemQ;
  const uint32_t data_bytes = kHeads * kSlab, scale_bytes = Kind::kScales ? kPageTokens * kHeads * 4 : 0;

  // Query tile into tensor memory: the row's threads convert 128/kRowThreads columns each. int4: fp16, element
  // order (0,4,1,5,2,6,3,7) inside every 8 dims, dims 1,5,3,7 divided by 16; int8, fp8: fp16 in order; bf16: the bits.
  if (warp < kSoftmaxWarps) {
    const uint32_t quarter = warp & 3u, part = warp >> 2, row = quarter * 32 + lane;
    const uint16_t *queries = kPrefill ? args.queries + (uint64_t(kv_head) * args.prefill.chunk_stride + lane_index * Rows) * (kG * kD)
                                       : args.queries + (uint64_t(lane_index) * kHeads + kv_head) * (uint64_t(RK_VERIFY_CHUNK_STRIDE) * kG * kD);
    const bool real = row < p.active_rows * kG;
    float q_sum = 0.0f; // over the values the tensor core will see, for the key-offset correction
#pragma unroll 1
    for (uint32_t piece = 0; piece < 4 / kRowThreads; ++piece) { // 32 columns = 8 chunks of 8 dims
      const uint32_t column = part * (128 / kRowThreads) + piece * 32;
      float columns[32];
#pragma unroll
      for (uint32_t c = 0; c < 8; ++c) {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (real) raw = __ldg(reinterpret_cast<const uint4 *>(queries + uint64_t(row) * kD + 2 * column + 8 * c));
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t chunk[4];
        if (Kind::kBf16) {
#pragma unroll
          for (uint32_t i = 0; i < 4; ++i) chunk[i] = words[i];
        } else {
          float d[8];
#pragma unroll
          for (uint32_t i = 0; i < 4; ++i) { d[2 * i] = bf16_bits_to_float(words[i] & 0xffffu); d[2 * i + 1] = bf16_bits_to_float(words[i] >> 16); }
          if (Format == RK_FORMAT_INT4) {
            chunk[0] = pack_half2(d[0], d[4]); chunk[1] = pack_half2(d[1] * 0.0625f, d[5] * 0.0625f);
            chunk[2] = pack_half2(d[2], d[6]); chunk[3] = pack_half2(d[3] * 0.0625f, d[7] * 0.0625f);
          } else {
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) chunk[i] = pack_half2(d[2 * i], d[2 * i + 1]);
          }
#pragma unroll
          for (uint32_t i = 0; i < 4; ++i) {
            const __half2 h = *reinterpret_cast<const __half2 *>(&chunk[i]);
            q_sum += ((Format == RK_FORMAT_INT4 && (i & 1u)) ? 16.0f : 1.0f) * (__low2float(h) + __high2float(h));
          }
        }
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) columns[c * 4 + i] = __uint_as_float(chunk[i]);
      }
      tmem_store32(tmem_q + ((quarter * 32u) << 16) + column, columns);
    }
    ctl.exchange[0][row][part] = q_sum;
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  if (tid < kM) {
    float total = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < kRowThreads; ++i) total += ctl.exchange[0][tid][i];
    ctl.q_sums[tid] = total;
  }
  __syncthreads();

  if (warp == kTmaWarp) {
    // ---- TMA producer: lanes 0-7 issue one copy each (page, {K, V, key scales, value scales}) of the group, lanes
    // 8-15 the matching L2 requests of a later group; one thread alone spent ~1 000 cycles per group on them ----
    const uint32_t local = (lane >> 2) & 1u, kind = lane & 3u; // page of the group; {K, V, key scales, value scales}
    const bool copier = lane < 8 && (kind < 2 || Kind::kScales), prefetcher = kPrefetch && lane >= 8 && lane < 16;
    // this lane's tensor inside a layer region ([K data][K scales][V data][V scales], each x extent pages) and head
    const uint64_t extent_pages = args.layer.extent_pages;
    const uint64_t tensor_base = args.layer.offset +
                                 extent_pages * (kind == 0 ? 0ull : kind == 2 ? uint64_t(data_bytes)
                                                  : kind == 1 ? uint64_t(data_bytes) + scale_bytes : 2ull * data_bytes + scale_bytes) +
                                 kv_head * (kind < 2 ? kSlab : 128u);
    const uint32_t page_stride = kind < 2 ? data_bytes : scale_bytes, copy_bytes = kind < 2 ? kSlab : 128u;
    auto source = [&](rk_page_entry entry) { return rk_entry_extent(entry) + tensor_base + uint64_t(rk_entry_index(entry)) * page_stride; };
    // table entries travel one group ahead of their use (copies) and of their L2 request (prefetch)
    rk_page_entry next = lane < 8 && page_begin + local < page_end ? table[page_begin + local] : 0;
    rk_page_entry next_ahead = prefetcher && page_begin + 2 * kPrefetchGroups + local < page_end ? table[page_begin + 2 * kPrefetchGroups + local] : 0;
    const uint32_t issued = groups - min(groups, args.withheld_groups); // all of them, except under the timeout probe
    for (uint32_t g = 0; g < issued; ++g) {
      const uint32_t r = g % kRawStages;
      const uint32_t first = page_begin + 2 * g, group_pages = min(2u, page_end - first);
      const rk_page_entry entry = next, entry_ahead = next_ahead;
      const uint32_t ahead = first + 2 * kPrefetchGroups + local;
      if (lane < 8 && first + 2 + local < page_end) next = table[first + 2 + local];
      if (prefetcher && ahead + 2 < page_end) next_ahead = table[ahead + 2];
      if (g >= kRawStages) barrier_wait(&ctl.raw_free[r], g / kRawStages - 1, error); // the stage's last readers
      const uint32_t full = smem_u32(&ctl.raw_full[r]), stage = raw_tile + r * kRawStageBytes;
      if (lane == 0) barrier_expect(full, group_pages * (2 * kSlab + (Kind::kScales ? 256 : 0)));
      __syncwarp();
      if (copier && local < group_pages) {
        const uint64_t address = source(entry);
        if (kind < 2) tma_load_rows(stage + (2 * kind + local) * kSlab, &head_map, int32_t((address - args.window_base) >> 7), full);
        else bulk_load(stage + kRawScaleOffset + (2 * (kind - 2) + local) * 128, reinterpret_cast<const void *>(address), 128, full);
      }
      // The raw ring holds at most kRawStages groups; the groups behind it are already requested from HBM into L2,
      // kPrefetchGroups ahead, so the ring is refilled at L2 latency.
      if (prefetcher && ahead < page_end && (kind < 2 || Kind::kScales)) prefetch_l2(source(entry_ahead), copy_bytes);
    }
    // Every copy this warp started has landed before the CTA may leave (also after a failed wait).
    if (lane == 0)
      for (uint32_t g = issued > kRawStages ? issued - kRawStages : 0; g < issued; ++g) {
        const uint32_t bar = smem_u32(&ctl.raw_full[g % kRawStages]), parity = (g / kRawStages) & 1u;
        for (uint32_t i = 0; i < kSpinLimit && !barrier_try(bar, parity); ++i) __nanosleep(64);
      }
  } else if (warp == kScoreWarp) {
    // ---- tensor-core issue, S = Q.K^T: S buffer g&1 is free once PV(g-2), which read P(g-2) from it, has landed (p_free) ----
    // The whole warp walks the loop (uniform control flow); one elected lane issues.
    const uint32_t idesc_qk = umma_instruction(kM, kGroupTokens, Kind::kBf16, Kind::kBf16);
    // a descriptor advances by (bytes >> 4) in its low word; nothing here carries out of the 14-bit field
    const uint64_t k_desc0 = umma_descriptor(k_tile), k_desc1 = umma_descriptor(k_tile + kKBytes);
    for (uint32_t g = 0; g < groups; ++g) {
      const uint32_t b = g & 1u, t = g % kTileStages; // S buffer, operand stage
      barrier_wait(&ctl.k_full[t], g / kTileStages, error);
      if (g >= 2) barrier_wait(&ctl.p_free[b], (g >> 1) - 1, error);
      tmem_fence_after();
      const uint64_t desc = t ? k_desc1 : k_desc0;
      const uint32_t target = tmem_s + b * 64;
      if (elect_one()) {
#pragma unroll
        for (uint32_t j = 0; j < 16; ++j)
          umma_f16_ts(target, tmem_q + 8 * j, desc + (((j >> 2) * (kGroupTokens * 128) + (j & 3u) * 32) >> 4), idesc_qk, j ? 1u : 0u);
        umma_commit(&ctl.s_full[b]);
        umma_commit(&ctl.k_free[t]);
      }
      __syncwarp();
    }
    // Tensor memory is released at the end of the kernel: every contraction this warp issued has completed by then,
    // also when a wait gave up and nobody else waits for them any more.
    if (elect_one()) umma_commit(&ctl.drained[0]);
    __syncwarp();
    for (uint32_t i = 0; i < kSpinLimit && !barrier_try(smem_u32(&ctl.drained[0]), 0); ++i) __nanosleep(64);
  } else if (warp == kValueWarp) {
    // ---- tensor-core issue, O += P.V ------------------------------------------------------------------------------
    const uint32_t idesc_pv = umma_instruction(kM, kD, Kind::kBf16, Kind::kBf16); // both operands of one kind: bf16 values take bf16 probabilities
    const uint64_t v_desc0 = umma_descriptor(v_tile), v_desc1 = umma_descriptor(v_tile + kVBytes);
    for (uint32_t g = 0; g < groups; ++g) {
      const uint32_t b = g & 1u, t = g % kTileStages;
      barrier_wait(&ctl.v_full[t], g / kTileStages, error);
      barrier_wait(&ctl.p_full[b], g >> 1, error);
      tmem_fence_after();
      const uint64_t desc = t ? v_desc1 : v_desc0;
      const uint32_t source = tmem_s + b * 64;
      if (elect_one()) {
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
          umma_f16_ts(tmem_o, source + 8 * j, desc + ((j * 32) >> 4), idesc_pv, (g || j) ? 1u : 0u);
          if (Kind::kBf16) umma_f16_ts(tmem_o, source + 32 + 8 * j, desc + ((j * 32) >> 4), idesc_pv, 1u); // the low parts
        }
        umma_commit(&ctl.v_free[t]);
        umma_commit(&ctl.p_free[b]);
      }
      __syncwarp();
    }
    if (elect_one()) umma_commit(&ctl.drained[1]);
    __syncwarp();
    for (uint32_t i = 0; i < kSpinLimit && !barrier_try(smem_u32(&ctl.drained[1]), 0); ++i) __nanosleep(64);
  } else if (warp >= kSoftmaxWarps || (warp & 3u) >= kQuarters) {
    // ---- expanders: raw codes -> 16-bit operand tiles --------------------------------------------------------------
    const uint32_t index = warp >= kSoftmaxWarps ? tid - kSoftmaxThreads
                                                  : kExpandWarps * 32 + ((warp >> 2) * (4 - kQuarters) + (warp & 3u) - kQuarters) * 32 + lane;
    const uint32_t team = index / kExpandThreads, e = index - team * kExpandThreads;
    for (uint32_t g = team; g < groups; g += kTileStages) {
      const uint32_t r = g % kRawStages, slot = r, b = team, round = g / kTileStages;
      const uint32_t first = page_begin + 2 * g;
      // positions of the group whose tokens exist: the split may end inside the group, the lane inside the page
      const uint32_t valid = min(min(2u, page_end - first) * kPageTokens, visible - first * kPageTokens);
      const uint8_t *raw = raw_ptr + r * kRawStageBytes;
      barrier_wait(&ctl.raw_full[slot], g / kRawStages, error);
      // per-position scale triples {key scale, log2 value scale, 2^-6 / value scale}; zeros past the valid tokens
      // (stale scale bytes never reach the arithmetic)
      if (e < kGroupTokens) {
        if (g >= kScaleStages) barrier_wait(&ctl.scale_free[g % kScaleStages], g / kScaleStages - 1, error);
        const uint32_t token = Expand<Format>::token_of(e);
        float4 triple = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (token < valid) {
          if (Kind::kScales) {
            const float ks = reinterpret_cast<const float *>(raw + kRawScaleOffset)[token];
            const float vs = fmaxf(reinterpret_cast<const float *>(raw + kRawScaleOffset)[64 + token], 9.094947e-13f); // 2^-40
            triple = make_float4(ks, log2_fast(vs), __fdividef(0.015625f, vs), 0.0f);
          } else {
            triple = make_float4(1.0f, 0.0f, 0.015625f, 0.0f);
          }
        }
        ctl.scales[g % kScaleStages][e] = triple;
      }
      if (round) barrier_wait(&ctl.k_free[b], round - 1, error);
      Expand<Format>::template keys<kExpandThreads>(raw, k_ptr + b * kKBytes, e);
      async_proxy_fence();
      barrier_arrive(smem_u32(&ctl.k_full[b]));
      if (round) barrier_wait(&ctl.v_free[b], round - 1, error);
      Expand<Format>::template values<kExpandThreads>(raw, v_ptr + b * kVBytes, e, valid);
      async_proxy_fence();
      barrier_arrive(smem_u32(&ctl.v_full[b]));
      barrier_arrive(smem_u32(&ctl.raw_free[slot]));
    }
  } else {
    // ---- softmax: kRowThreads threads per fused row (= TMEM lane), kRowTokens contraction positions each;
    // the warps of quarters without a real row work as expanders instead ----
    const uint32_t quarter = warp & 3u, part = warp >> 2;
    const uint32_t my_row = quarter * 32 + lane;
    const float score_scale = rk_score_scale(p.score_scale, kD) * kLog2e;
    const float row_factor = ldexpf(score_scale, Kind::kKeyShift);
    const float row_offset = -Kind::kKeyOffset * ctl.q_sums[my_row] * score_scale;
    const uint32_t query_row = my_row / kG;
    const uint32_t causal_limit = min(visible, p.committed_tokens + min(query_row, p.active_rows - 1) + 1);
    const uint32_t tree_mask = kTree && query_row < p.row_capacity ? row_masks[query_row] : 0u;
    const uint32_t lane_address = (quarter * 32u) << 16;
    constexpr uint32_t kOutColumns = kD / kRowThreads; // columns of O this thread rescales and writes out
    float row_max = -1.0e30f, row_sum = 0.0f;          // row_sum: this thread's tokens only

    for (uint32_t g = 0; g < groups; ++g) {
      const uint32_t first = page_begin + 2 * g, b = g & 1u;
      const uint32_t token_base = first * kPageTokens;
      // tokens of the group that exist (a split may end inside it) and, on a chain, pass the causal rule.
      // int4: position kRowTokens*part + i holds token 8*(i%8) + i/8 + (kRowTokens/8)*part; else token = position
      const uint32_t present = min(2u, page_end - first) * kPageTokens;
      const uint32_t limit = kTree ? present : min(present, causal_limit > token_base ? causal_limit - token_base : 0u);
      constexpr bool kPermuted = Format == RK_FORMAT_INT4;
      const uint32_t part_token = kPermuted ? (kRowTokens / 8) * part : kRowTokens * part;
      const int32_t bound = int32_t(limit) - int32_t(part_token);
      const float4 *triples = ctl.scales[g % kScaleStages] + part * kRowTokens;
      barrier_wait(&ctl.s_full[b], g >> 1, error);
      tmem_fence_after();
      float scores[kRowTokens];
      tmem_load_scores(tmem_s + b * 64 + lane_address + part * kRowTokens, scores);

      float group_max = -INFINITY;
      if (!kTree && limit >= kGroupTokens) { // every token of the group is admitted (all but the last groups of a lane)
#pragma unroll
        for (uint32_t i = 0; i < kRowTokens; ++i) {
          const float4 triple = triples[i];
          scores[i] = fmaf(scores[i], row_factor, row_offset) * triple.x + triple.y; // score + log2(value scale)
          group_max = fmaxf(group_max, scores[i]);
        }
      } else {
#pragma unroll
        for (uint32_t i = 0; i < kRowTokens; ++i) {
          const int32_t local = kPermuted ? int32_t(8 * (i & 7u) + (i >> 3)) : int32_t(i);
          bool admitted = local < bound;
          if (kTree) {
            const uint32_t token = token_base + uint32_t(local) + part_token;
            admitted = admitted && (token < p.committed_tokens || (token < visible && ((tree_mask >> (token - p.committed_tokens)) & 1u)));
          }
          const float4 triple = triples[i];
          const float s = fmaf(scores[i], row_factor, row_offset) * triple.x + triple.y;
          scores[i] = admitted ? s : -INFINITY;
          group_max = fmaxf(group_max, scores[i]);
        }
      }
      // the row's other parts; past this barrier every part holds its scores in registers, so the
      // probabilities may overwrite the first 32 columns of the buffer
      ctl.exchange[b][my_row][part] = group_max;
      tmem_fence_before();
      asm volatile("bar.sync %0, %1;" ::"r"(1u + quarter), "n"(32 * kRowThreads) : "memory");
      tmem_fence_after();
#pragma unroll
      for (uint32_t i = 0; i < kRowThreads; ++i) group_max = fmaxf(group_max, ctl.exchange[b][my_row][i]);
      // Lazy rescale: the reference exponent only moves when the maximum grew by more than 2^8, so the
      // fp16 probabilities stay below 2^(8+6); rows of a warp move together (collective TMEM access).
      const bool grow = group_max > row_max + 8.0f;
      float scale = 1.0f;
      if (grow) {
        scale = exp2_fast(row_max - group_max);
        row_max = group_max;
        row_sum *= scale;
      }
      const float exponent_base = row_max - 6.0f;
      // bf16 probabilities alone carry 8 bits: they travel as a high and a low bf16 part (two contractions), which
      // restores 16 bits; the low parts take the second half of the S buffer
      uint32_t packed[kRowTokens / 2], packed_low[Kind::kBf16 ? kRowTokens / 2 : 1];
#pragma unroll
      for (uint32_t c = 0; c < kRowTokens / 2; ++c) {
        float w[2];
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) {
          w[h] = exp2_fast(scores[2 * c + h] - exponent_base);     // 0 for a masked token
          row_sum = fmaf(w[h], triples[2 * c + h].z, row_sum);     // 2^(score - row_max)
        }
        if (Kind::kBf16) {
          packed[c] = pack_bfloat2(w[0], w[1]);
          packed_low[c] = pack_bfloat2(w[0] - __uint_as_float(packed[c] << 16), w[1] - __uint_as_float(packed[c] & 0xffff0000u));
        } else {
          packed[c] = pack_half2(w[0], w[1]);
        }
      }
      if (g && __any_sync(0xffffffffu, grow)) { // this part rescales its columns of O once P.V(g-1) has landed
        barrier_wait(&ctl.v_free[(g - 1) % kTileStages], (g - 1) / kTileStages, error);
        tmem_fence_after();
#pragma unroll 1
        for (uint32_t c = 0; c < kOutColumns / 32; ++c) {
          float o[32];
          tmem_load32(tmem_o + lane_address + part * kOutColumns + c * 32, o);
#pragma unroll
          for (uint32_t i = 0; i < 32; ++i) o[i] *= scale;
          tmem_store32(tmem_o + lane_address + part * kOutColumns + c * 32, o);
        }
      }
      tmem_store_packed(tmem_s + b * 64 + lane_address + part * (kRowTokens / 2), packed);
      if constexpr (Kind::kBf16) tmem_store_packed(tmem_s + b * 64 + 32 + lane_address + part * (kRowTokens / 2), packed_low);
      tmem_fence_before();
      barrier_arrive(smem_u32(&ctl.p_full[b]));
      barrier_arrive(smem_u32(&ctl.scale_free[g % kScaleStages]));
    }

    // ---- partial output: row i of O, un-normalised; statistics {reference exponent, sum} -------------------
    barrier_wait(&ctl.v_free[(groups - 1) % kTileStages], (groups - 1) / kTileStages, error);
    tmem_fence_after();
    const bool failed = *error != 0;
    // verify: one slot of kRealRows fused rows per (lane, head, split); prefill: one slot of 48 fused rows per tile
    constexpr uint32_t kSlotRows = kPrefill ? RK_PREFILL_TILE_ROWS * kG : kRealRows;
    const uint32_t sub_tile = kPrefill ? my_row / kSlotRows : 0, slot_row = my_row - sub_tile * kSlotRows;
    const uint64_t slot_owner = kPrefill ? uint64_t(lane_index) * (Rows / RK_PREFILL_TILE_ROWS) + sub_tile : lane_index;
    const uint64_t slot = (slot_owner * kHeads + kv_head) * p.slot_splits + split;
    // a chunk with an odd number of tiles has no second tile in its last pair: nothing is written for it
    const bool row_exists = my_row < kRealRows && (!kPrefill || sub_tile * RK_PREFILL_TILE_ROWS < p.active_rows);
    float *out = args.partials + (slot * kSlotRows + slot_row) * kD + part * kOutColumns;
#pragma unroll 1
    for (uint32_t c = 0; c < kOutColumns / 32; ++c) {
      float o[32];
      tmem_load32(tmem_o + lane_address + part * kOutColumns + c * 32, o);
      if (row_exists) {
#pragma unroll
        for (uint32_t i = 0; i < 32; i += 4)
          *reinterpret_cast<float4 *>(out + c * 32 + i) = make_float4(o[i] * 0.015625f, o[i + 1] * 0.015625f, o[i + 2] * 0.015625f, o[i + 3] * 0.015625f);
      }
    }
    ctl.exchange[groups & 1u][my_row][part] = row_sum;
    asm volatile("bar.sync %0, %1;" ::"r"(1u + quarter), "n"(32 * kRowThreads) : "memory");
    if (part == 0 && row_exists) {
      float total = 0.0f;
#pragma unroll
      for (uint32_t i = 0; i < kRowThreads; ++i) total += ctl.exchange[groups & 1u][my_row][i];
      float *stats = args.statistics + (slot * kSlotRows + slot_row) * 2;
      stats[0] = failed ? -INFINITY : row_max * kLn2;
      stats[1] = failed ? 0.0f : total;
    }
  }
  tmem_fence_before();
  __syncthreads();
  if (tid == 0 && ctl.error) atomicExch(args.status, 1u);
  if (warp == kTmaWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

} // namespace
} // namespace rk

using namespace rk;

// verify_attention_{int4,q8,fp8,bf16}_split and the tree variants (decode/paged_attention.metal:23-192,
// decode/fp8_attention.metal:8-62) as a tcgen05 contraction for row capacity 1 (plain decode), 8 or 16.
// Arguments and scratch layout as rk_attention_verify_split plus the pool's window (rk_window_create);
// `status` is one device word the caller zeroes, non-zero after a bounded wait ran out. Merge with
// rk_attention_verify_reduce.
namespace {
template <uint32_t Format>
int launch_window(const Window *w, uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits, const VerifyArgs &args, cudaStream_t s) {
  constexpr size_t shared_bytes = 1024 + tile_bytes<Format>() + sizeof(Control);
  const CUtensorMap &map = Format == RK_FORMAT_INT4 ? w->int4_head_map : Format == RK_FORMAT_BF16 ? w->int4_map : w->byte_head_map;
  const dim3 grid(kHeads, grid_splits, lanes);
  auto launch = [&](auto kernel) -> int {
    if (int st = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(shared_bytes)), "window kernel shared memory")) return st;
    kernel<<<grid, kThreads, shared_bytes, s>>>(map, args);
    return kOk;
  };
  const bool tree = args.row_masks != nullptr;
  if (row_capacity == 1) return launch(window_attention_kernel<Format, 1, false>);
  if (row_capacity == 8) return tree ? launch(window_attention_kernel<Format, 8, true>) : launch(window_attention_kernel<Format, 8, false>);
  return tree ? launch(window_attention_kernel<Format, 16, true>) : launch(window_attention_kernel<Format, 16, false>);
}
} // namespace

static int verify_split_tc(const void *window, uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                           uint32_t head_dim, uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits,
                           const void *queries, float *partials, float *statistics,
                           const rk_page_entry *const *tables, const uint32_t *row_masks,
                           const rk_verify_params *lane_params, rk_kv_layer layer, uint32_t *status,
                           uint32_t spin_limit, uint32_t withheld_groups, void *stream) {
  if (kv_heads != kHeads || query_heads != kHeads * kG || head_dim != kD || !rk_format_valid(format) ||
      (row_capacity != 1 && row_capacity != 8 && row_capacity != 16) || (row_capacity == 1 && row_masks) ||
      (format == RK_FORMAT_FP8E4M3 && row_masks)) {
    set_error("rk_attention_verify_split_tc: built for 4 KV heads x 24 query heads x 256, row capacity 1, 8 or 16 (tree: 8 or 16, not fp8)");
    return kUnsupported;
  }
  const auto *w = static_cast<const Window *>(window);
  if (!w || !lanes || !grid_splits || grid_splits > RK_VERIFY_MAX_SPLITS || !queries || !partials || !statistics || !tables ||
      !lane_params || !layer.extent_pages || !status) {
    set_error("rk_attention_verify_split_tc: invalid arguments");
    return kInvalid;
  }
  VerifyArgs args{static_cast<const uint16_t *>(queries), partials, statistics, tables, row_masks, lane_params, layer, w->base, status,
                  spin_limit, withheld_groups, nullptr, {}};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int st = kUnsupported;
  switch (format) {
  case RK_FORMAT_INT4: st = launch_window<RK_FORMAT_INT4>(w, lanes, row_capacity, grid_splits, args, s); break;
  case RK_FORMAT_INT8: st = launch_window<RK_FORMAT_INT8>(w, lanes, row_capacity, grid_splits, args, s); break;
  case RK_FORMAT_FP8E4M3: st = launch_window<RK_FORMAT_FP8E4M3>(w, lanes, row_capacity, grid_splits, args, s); break;
  case RK_FORMAT_BF16: st = launch_window<RK_FORMAT_BF16>(w, lanes, row_capacity, grid_splits, args, s); break;
  }
  if (st) return st;
  return cuda_status(cudaGetLastError(), "window kernel launch");
}

extern "C" int rk_attention_verify_split_tc(const void *window, uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                            uint32_t head_dim, uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits,
                                            const void *queries, float *partials, float *statistics,
                                            const rk_page_entry *const *tables, const uint32_t *row_masks,
                                            const rk_verify_params *lane_params, rk_kv_layer layer, uint32_t *status,
                                            void *stream) {
  return verify_split_tc(window, format, kv_heads, query_heads, head_dim, lanes, row_capacity, grid_splits, queries, partials,
                         statistics, tables, row_masks, lane_params, layer, status, kSpinLimit, 0, stream);
}

// Test hook of the window kernel's timeout path: the same launch with waits that give up after `spin_limit` polls
// and a TMA warp that never streams the last `withheld_groups` 64-token groups of each split. The waiting warps run
// out of polls, every other wait of the CTA then gives up at once, tensor memory is released, `status` turns
// non-zero and the kernel returns; nothing faults and no wait is unbounded. The step's output is invalid.
extern "C" int rk_attention_verify_probe_timeout(const void *window, uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                                 uint32_t head_dim, uint32_t lanes, uint32_t row_capacity, uint32_t grid_splits,
                                                 const void *queries, float *partials, float *statistics,
                                                 const rk_page_entry *const *tables, const rk_verify_params *lane_params,
                                                 rk_kv_layer layer, uint32_t *status, uint32_t spin_limit,
                                                 uint32_t withheld_groups, void *stream) {
  if (!spin_limit || spin_limit > kSpinLimit) { set_error("rk_attention_verify_probe_timeout: spin limit out of range"); return kInvalid; }
  return verify_split_tc(window, format, kv_heads, query_heads, head_dim, lanes, row_capacity, grid_splits, queries, partials,
                         statistics, tables, nullptr, lane_params, layer, status, spin_limit, withheld_groups, stream);
}

// prefill_attention_*_split (prefill/paged_attention.metal:7-67) on the tcgen05 kernel: one CTA per (KV head, split,
// 8-row tile). Arguments and scratch layout as rk_attention_prefill_split plus the pool's window and the status
// word; merge with rk_attention_prefill_reduce. `params` is a HOST pointer.
extern "C" int rk_attention_prefill_split_tc(const void *window, uint32_t format, uint32_t kv_heads, uint32_t query_heads,
                                             uint32_t head_dim, const void *queries, float *partials, float *statistics,
                                             const rk_page_entry *table, const rk_prefill_params *params, uint32_t *status,
                                             void *stream) {
  if (kv_heads != kHeads || query_heads != kHeads * kG || head_dim != kD || !rk_format_valid(format)) {
    set_error("rk_attention_prefill_split_tc: built for 4 KV heads x 24 query heads x 256");
    return kUnsupported;
  }
  const auto *w = static_cast<const Window *>(window);
  if (!w || !queries || !partials || !statistics || !table || !params || !status || !rk_prefill_contract_valid(params)) {
    set_error("rk_attention_prefill_split_tc: invalid arguments");
    return kInvalid;
  }
  VerifyArgs args{static_cast<const uint16_t *>(queries), partials, statistics, nullptr, nullptr, nullptr, params->kv, w->base, status,
                  kSpinLimit, 0, table, *params};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t tiles = (params->rows + RK_PREFILL_TILE_ROWS - 1) / RK_PREFILL_TILE_ROWS;
  const bool pairs = params->split_count == 1 && tiles > 1; // two tiles per CTA fill 96 of the 128 tensor-core rows
  const dim3 grid(kHeads, params->split_count, pairs ? (tiles + 1) / 2 : tiles);
  auto launch = [&](auto kernel, size_t shared_bytes, const CUtensorMap &map) -> int {
    if (int st = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(shared_bytes)), "window kernel shared memory")) return st;
    kernel<<<grid, kThreads, shared_bytes, s>>>(map, args);
    return cuda_status(cudaGetLastError(), "prefill window kernel launch");
  };
  auto launch_format = [&](auto format_tag, const CUtensorMap &map) -> int {
    constexpr uint32_t F = decltype(format_tag)::value;
    constexpr size_t shared_bytes = 1024 + tile_bytes<F>() + sizeof(Control);
    return pairs ? launch(window_attention_kernel<F, 16, false, true>, shared_bytes, map)
                 : launch(window_attention_kernel<F, 8, false, true>, shared_bytes, map);
  };
  switch (format) {
  case RK_FORMAT_INT4: return launch_format(std::integral_constant<uint32_t, RK_FORMAT_INT4>{}, w->int4_head_map);
  case RK_FORMAT_INT8: return launch_format(std::integral_constant<uint32_t, RK_FORMAT_INT8>{}, w->byte_head_map);
  case RK_FORMAT_FP8E4M3: return launch_format(std::integral_constant<uint32_t, RK_FORMAT_FP8E4M3>{}, w->byte_head_map);
  default: return launch_format(std::integral_constant<uint32_t, RK_FORMAT_BF16>{}, w->int4_map);
  }
}
