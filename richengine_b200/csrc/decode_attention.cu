// decode_attention.cu — paged GQA decode attention (one query row per lane)
// streaming pages at HBM speed: the int4 kernel described here, and its
// int8 / fp8 and bf16 siblings further down.
//
// Semantics: the reference's tile with active_rows = 1
//   runtime/metal/kernels/common/paged_attention_tile.h:85-189,208-349  (scores, scale fold, online softmax, P.V)
//   runtime/metal/kernels/common/paged_attention_tile.h:362-404         (fixed-order merge)
//   runtime/metal/kernels/decode/paged_attention.metal:23-60            (query / output placement)
// The execution design is B200-native, not the reference's:
//  * Work is every lane's pages laid end to end and cut into one contiguous range per CTA (one CTA per SM) in a
//    coordinate stretched at lane boundaries (struct Cut); a range that crosses lanes yields one partial per lane
//    piece. Every CTA derives the same cut from the lane parameters, so no plan is uploaded and the result is the
//    same bits for a given grid.
//  * One producer thread streams whole pages — all four heads' keys (16 KiB), all four heads' values (16 KiB) and the
//    two 512-byte scale rows — into a ring of six shared-memory stages with TMA (128-byte swizzle, no multicast, L2
//    evict-first), completion on mbarriers. Consumer warps wait with bounded polls and give a stage back lane by
//    lane, behind a generic-to-async proxy fence.
//  * Twelve consumer warps = 4 KV heads x 3 page residues; each runs an independent online softmax over its pages.
//    Group-of-6 query heads against 4-bit codes is 12 multiply-adds per KV byte — above what the fp32 pipes sustain
//    at HBM speed — so the contractions run on the warp-level tensor path (mma.sync m16n8k16, fp16 operands, fp32
//    accumulate) with the codes expanded in registers:
//      S^T[token, head] = K[token, dim] . Q^T[dim, head]   (tokens are the M rows)
//      O^T[dim, head]  += V^T[dim, token] . P^T[token, head]
//    Key and value nibbles become fp16 bit patterns directly (u * 2^-24, u = code + 8); the keys' +8 is removed
//    exactly through 8 * sum(q), the values' through 8 * the sum of the rounded weights. Codes, queries (bf16 ->
//    fp16, exact in range) and products are exact; accumulation is fp32.
//  * The token scale folds into the softmax as in the reference, and the value
//    scale folds into the exponent: w = 2^(s + log2 vscale - m), so the fp16
//    probabilities stay in (0, 2^14] whatever the value magnitudes are.
//  * A CTA's last segment is folded in the (then idle) ring to one partial per KV head before it leaves the SM; the
//    merge kernel that follows (a programmatic dependent launch) combines a lane's partials in segment order.
#include "common.cuh"
#include "window.cuh"

#include <cuda.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstring>

namespace rk {

struct DriverApi;
const DriverApi *driver_api();

namespace {

constexpr uint32_t kKvHeads = 4, kGroup = 6, kHeadDim = 256;
constexpr uint32_t kPageWarps = 3;                          // warps per KV head, each takes every third page
constexpr uint32_t kConsumerWarps = kKvHeads * kPageWarps;
// Sixteen warps = four warp groups: three of consumers and one that holds the producer warp and three idle warps.
// A CTA of thirteen warps would put four warps on one of the SM's four schedulers, which caps every thread at 128
// registers and spills the consumers' accumulators; with whole warp groups the producer's group hands its registers
// back (setmaxnreg.dec) and the consumer groups take them (setmaxnreg.inc): 152 registers, no spill.
constexpr uint32_t kProducerGroupWarps = 4;
constexpr uint32_t kThreads = (kConsumerWarps + kProducerGroupWarps) * 32;
constexpr uint32_t kStages = 6;
constexpr uint32_t kSlabBytes = 4096;                       // one head's K (or V) of a page, int4
constexpr uint32_t kTensorBytes = kKvHeads * kSlabBytes;    // all heads' K (or V) of a page
constexpr uint32_t kScaleBytes = kKvHeads * kPageTokens * 4;
constexpr uint32_t kStageBytes = 2 * kTensorBytes + 2 * kScaleBytes; // K | V | key scales | value scales
constexpr uint32_t kMaxLanes = 1024;
#ifndef RK_SWITCH_PAGES
#define RK_SWITCH_PAGES 10
#endif
// what a lane boundary inside a CTA's range costs, in pages of each kernel's format (a page of bytes takes twice,
// a bf16 page four times as long to stream as an int4 page)
constexpr uint32_t kSwitchPages = RK_SWITCH_PAGES, kByteSwitchPages = (RK_SWITCH_PAGES + 1) / 2, kWideSwitchPages = (RK_SWITCH_PAGES + 3) / 4;
constexpr uint32_t kSpinLimit = 1u << 20; // polls of ~100 ns: a wait gives up after roughly 0.1-0.2 s
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
static_assert(kStageBytes % 1024 == 0, "stages keep the 1 KiB swizzle alignment");

struct DecodeArgs {
  const uint16_t *queries;
  float *partials;
  float *statistics;
  uint32_t *descriptors; // [lanes]{first segment, segments | last segment holds three slots << 31}, then the status word
  const rk_page_entry *const *tables;
  const rk_verify_params *lane_params;
  rk_kv_layer layer;
  uint64_t window_base;
  uint32_t lanes;
  uint32_t *status;     // sticky device status word: set when a bounded wait ran out, cleared by the status readers
  uint32_t spin_limit;  // polls a wait may take (kSpinLimit in production; the timeout probe passes a few thousand)
  uint32_t withheld;    // timeout probe only: the producer never streams the last `withheld` pages of its range
};

__device__ __forceinline__ uint32_t smem_address(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void barrier_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void barrier_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Register hand-over between warp groups; every warp of a group executes its instruction.
__device__ __forceinline__ void release_registers() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }
__device__ __forceinline__ void take_registers() { asm volatile("setmaxnreg.inc.sync.aligned.u32 152;"); }
// A consumer lane is done with a stage that TMA will refill: its generic-proxy reads are ordered before later
// async-proxy writes (fence.proxy.async), then it arrives on the stage's "empty" barrier.
__device__ __forceinline__ void release_stage(uint32_t bar) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool barrier_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait: false when the limit ran out (the caller records the error and leaves).
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (barrier_try(bar, parity)) return true;
    if (i > 32) __nanosleep(32);
  }
  return false;
}
// Pages are read once per step: they are marked first to leave L2, so that what is read again (queries, tables,
// parameters, the partials on their way to the merge) stays.
__device__ __forceinline__ uint64_t stream_policy() {
  uint64_t policy;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap *map, int32_t row, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
               ::"r"(dst), "l"(map), "r"(0), "r"(row), "r"(bar), "l"(stream_policy()) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(stream_policy()) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t transpose_8x8(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// (a & mask) ^ flip in ONE logic instruction: both constants must sit in
// registers (an immediate pair would split it in two half-rate ALU operations).
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t mask, uint32_t flip) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(mask), "r"(flip));
  return r;
}
// A constant the compiler must keep in a register.
__device__ __forceinline__ uint32_t register_constant(uint32_t value) {
  uint32_t r;
  asm volatile("mov.b32 %0, %1;" : "=r"(r) : "r"(value));
  return r;
}
__device__ __forceinline__ float exp2_fast(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float log2_fast(float x) {
  float r;
  asm("lg2.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t load_shared_32(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address) : "memory");
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 load_shared_16(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address) : "memory");
  return v;
}
__device__ __forceinline__ float load_shared_f32(uint32_t address) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(address) : "memory");
  return v;
}

// How the flattened pages of all lanes are cut into one range per CTA. A lane boundary inside a range costs its CTA
// about as much as streaming `pad` pages (the partial of the lane that ends is flushed and the next lane's queries are
// fetched and laid out while the ring stands still), and a CTA that ends late holds the whole grid back. So the cut is
// made in a stretched coordinate in which `pad` empty positions follow every lane but the last: page x of lane i
// sits at x + pad * i, and the stretched line is cut into `ctas` equal ranges [b * length / ctas, (b + 1) * length /
// ctas). A range that spans a boundary then holds `pad` pages fewer. The cut depends only on the lanes' page counts
// and the grid, so a step is repeatable bit for bit.
struct Cut {
  uint64_t length; // stretched positions
  uint32_t ctas, pad;
  __device__ __forceinline__ static Cut make(uint64_t total_pages, uint32_t ctas, uint32_t lanes, uint32_t switch_pages) {
    Cut cut;
    cut.ctas = ctas;
    // never more than a quarter of a range: short ranges keep their pages
    cut.pad = lanes > 1 ? uint32_t(min(uint64_t(switch_pages), total_pages / ctas / 4)) : 0;
    cut.length = total_pages + uint64_t(cut.pad) * (lanes - (lanes ? 1 : 0));
    return cut;
  }
  // the CTA that owns flattened page `x`, a page of lane `lane`
  __device__ __forceinline__ uint32_t cta_of(uint64_t x, uint32_t lane) const {
    return uint32_t(((x + uint64_t(pad) * lane + 1) * ctas - 1) / length);
  }
  // the first flattened page of range `range` (the page count for range == ctas); `lane_start[0..lanes]` are the lanes' prefix sums
  __device__ __forceinline__ uint32_t first_page(uint32_t range, const uint32_t *lane_start, uint32_t lanes) const {
    const uint64_t position = uint64_t(range) * length / ctas;
    uint32_t lo = 0, hi = lanes; // largest lane whose stretched start is <= position
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) / 2;
      if (lane_start[mid] + uint64_t(pad) * mid <= position) lo = mid; else hi = mid;
    }
    const uint64_t within = position - (lane_start[lo] + uint64_t(pad) * lo);
    return lane_start[lo] + uint32_t(min(within, uint64_t(lane_start[lo + 1] - lane_start[lo])));
  }
};

struct Shared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t warp_full[kConsumerWarps];   // bf16 kernel: one barrier per consumer warp
  uint2 query[kKvHeads][16][32];        // per KV head: B fragments of Q^T for the 16 k-steps
  float head_factor[kKvHeads][8];       // per query head of the group: score factor ...
  float head_offset[kKvHeads][8];       // ... and the -8*sum(q) correction
  uint32_t lane_start[kMaxLanes + 1];   // pages before each lane
  uint32_t segment_base[kMaxLanes + 1]; // partial segments before each lane
  uint32_t scan[kThreads / 32 + 1];
  float unit_scales[kScaleBytes / 4 + kPageTokens]; // ones: the scale rows of a format without scales
  Cut cut;                                          // how the grid's ranges were cut
  uint32_t range_begin, range_end, first_lane;      // this CTA's flattened pages and the first lane with pages among them
  volatile uint32_t error;
};

// Block-wide exclusive prefix sum of values[0..n) in place (values[n] = total).
__device__ void exclusive_scan(uint32_t *values, uint32_t n, uint32_t *scratch) {
  const uint32_t tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
  uint32_t carry = 0;
  for (uint32_t base = 0; base < n; base += kThreads) {
    const uint32_t i = base + tid;
    const uint32_t v = i < n ? values[i] : 0;
    uint32_t inclusive = v;
#pragma unroll
    for (uint32_t o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, inclusive, o);
      if (lane >= o) inclusive += up;
    }
    if (lane == 31) scratch[warp] = inclusive;
    __syncthreads();
    uint32_t before = 0;
    for (uint32_t w = 0; w < warp; ++w) before += scratch[w];
    uint32_t total = 0;
    for (uint32_t w = 0; w < kThreads / 32; ++w) total += scratch[w];
    if (i < n) values[i] = carry + before + inclusive - v;
    carry += total;
    __syncthreads();
  }
  if (tid == 0) values[n] = carry;
  __syncthreads();
}

// Online softmax of one page for this lane's 4 tokens x 2 query heads, and the fp16 probability
// fragments (B operand of O^T += V^T.P^T). Masked = the page holds tokens past the visible ones.
template <bool Masked, bool Wide = false, bool Ride = false>
__device__ __forceinline__ void page_softmax(const float (&sacc)[2][2][4], const float (&hfac)[2],
                                             const float (&negoff)[2], uint32_t scales, uint32_t r3g,
                                             uint32_t valid, float (&m)[2], float (&l_sum)[2], float (&o)[16][4],
                                             uint32_t (&pb_frag)[2][2], uint32_t (*pb_low)[2] = nullptr, float *psum = nullptr) {
  float s2[2][2][2], lv[2][2];
  float local_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (uint32_t mt = 0; mt < 2; ++mt)
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {
      const uint32_t token = 16 * mt + 8 * half + r3g;
      const float ks = load_shared_f32(scales + token * 4);
      const float vs = load_shared_f32(scales + kScaleBytes + token * 4);
      const bool live = !Masked || token < valid;
      lv[mt][half] = live ? log2_fast(vs) : -INFINITY; // a zero value row weighs nothing
      const float floor_lv = live ? fmaxf(lv[mt][half], -40.0f) : -INFINITY;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        const float acc = sacc[mt][0][half * 2 + j] + sacc[mt][1][half * 2 + j];
        const float score = live ? fmaf(acc, hfac[j], negoff[j]) * ks : -INFINITY;
        s2[mt][half][j] = score;
        local_max[j] = fmaxf(local_max[j], score + floor_lv);
      }
    }
  if (__any_sync(0xffffffffu, local_max[0] > m[0] || local_max[1] > m[1])) {
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      float v = local_max[j];
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
      const float next = fmaxf(m[j], v);
      const float scale = exp2_fast(m[j] - next);
      m[j] = next;
      l_sum[j] *= scale;
      if (Ride) psum[j] *= scale;
#pragma unroll
      for (uint32_t t = 0; t < 16; ++t) { o[t][j] *= scale; o[t][2 + j] *= scale; }
    }
  }
#pragma unroll
  for (uint32_t mt = 0; mt < 2; ++mt) {
    float w[2][2];
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half)
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        const float score = s2[mt][half][j];
        const bool live = !Masked || score != -INFINITY;
        // probabilities carry 2^14 so the smallest weights keep fp16 precision
        w[half][j] = live ? exp2_fast(score + lv[mt][half] - m[j] + 14.0f) : 0.0f;
        l_sum[j] += live ? exp2_fast(score - m[j]) : 0.0f;
      }
    if (Wide) {
      // bf16 values need bf16 probabilities: each weight travels as a truncated high part and the rest
#pragma unroll
      for (uint32_t half = 0; half < 2; ++half) {
        const uint32_t hi0 = __float_as_uint(w[half][0]) & 0xffff0000u, hi1 = __float_as_uint(w[half][1]) & 0xffff0000u;
        pb_frag[mt][half] = transpose_8x8((hi0 >> 16) | hi1);
        pb_low[mt][half] = transpose_8x8(pack_bf16x2(w[half][0] - __uint_as_float(hi0), w[half][1] - __uint_as_float(hi1)));
      }
    } else if (Ride) {
      // the value codes ride their +8 through the accumulation: keep the sum of the ROUNDED weights to take it out
#pragma unroll
      for (uint32_t half = 0; half < 2; ++half) {
        const __half2 h = __floats2half2_rn(w[half][0], w[half][1]);
        psum[0] += __low2float(h);
        psum[1] += __high2float(h);
        pb_frag[mt][half] = transpose_8x8(*reinterpret_cast<const uint32_t *>(&h));
      }
    } else {
      pb_frag[mt][0] = transpose_8x8(pack_half2(w[0][0], w[0][1]));
      pb_frag[mt][1] = transpose_8x8(pack_half2(w[1][0], w[1][1]));
    }
  }
}

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may be scheduled while
// its predecessor drains; it must not touch memory before the predecessor's writes are visible (wait), and it lets
// its own successor be scheduled early (launch_dependents). Both are no-ops in an ordinary launch.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The prologue of the three decode kernels: pages per lane -> prefix, the cut, segments per lane -> prefix, this CTA's
// range. A function of its own (not inlined) so that the kernels' streaming loops are compiled the same whatever
// changes here: the int4 loop runs at the edge of what the SM issues, and its schedule moved by 2 % with unrelated
// edits of a prologue compiled into the same body. Every thread of the CTA calls it; an empty range comes back as
// range_begin == range_end.
__device__ __noinline__ void cut_ranges(Shared &sh, const DecodeArgs &args, uint32_t switch_pages) {
  const uint32_t tid = threadIdx.x, lanes = args.lanes, cta = blockIdx.x;
  for (uint32_t i = tid; i < lanes; i += kThreads) {
    rk_verify_params p = args.lane_params[i];
    p.kv = args.layer;
    const bool valid = rk_verify_contract_valid(&p) && p.active_rows == 1 && p.row_capacity == 1;
    sh.lane_start[i] = valid ? rk_pages_for(p.committed_tokens + 1) : 0;
  }
  if (tid == 0) { sh.error = 0; sh.range_begin = sh.range_end = sh.first_lane = 0; }
  __syncthreads();
  exclusive_scan(sh.lane_start, lanes, sh.scan);
  const uint64_t total_pages = sh.lane_start[lanes];
  // Never more ranges than pages, so every range between a lane's first and last is non-empty.
  const uint32_t ctas = uint32_t(min(uint64_t(gridDim.x), total_pages));
  if (cta >= ctas) return; // the whole CTA: its range stays empty (it never needed its predecessor's results)
  const Cut cut = Cut::make(total_pages, ctas, lanes, switch_pages);
  for (uint32_t i = tid; i < lanes; i += kThreads) {
    const uint32_t begin = sh.lane_start[i], end = sh.lane_start[i + 1];
    sh.segment_base[i] = end > begin ? cut.cta_of(end - 1, i) - cut.cta_of(begin, i) + 1 : 0;
  }
  __syncthreads();
  exclusive_scan(sh.segment_base, lanes, sh.scan);
  // Up to here the kernel has read only the lanes' parameter blocks, which no kernel of this library writes: when it
  // was launched early (programmatic dependent launch behind this library's store, prepare or merge kernel) the
  // partition above ran beside its predecessor's tail. Pages, queries and the scratch the predecessor's merge still
  // reads are touched only from here on. (A predecessor that is not one of these kernels never lets a dependent start
  // early, so a caller's own kernel that writes the parameter blocks is complete before this grid begins.)
  dependency_wait();
  if (cta == 0)
    for (uint32_t i = tid; i < lanes; i += kThreads) {
      // a lane with pages gets its descriptor from the CTA that flushes its last segment; a lane without has no segment
      if (sh.segment_base[i + 1] == sh.segment_base[i]) {
        args.descriptors[2 * i] = sh.segment_base[i];
        args.descriptors[2 * i + 1] = 0;
      }
    }
  if (tid == 0) {
    const uint32_t range_begin = cut.first_page(cta, sh.lane_start, lanes);
    uint32_t lo = 0, hi = lanes; // first lane whose pages reach into the range: the largest i with lane_start[i] <= range_begin
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) / 2;
      if (sh.lane_start[mid] <= range_begin) lo = mid; else hi = mid;
    }
    sh.cut = cut;
    sh.range_begin = range_begin;
    sh.range_end = cut.first_page(cta + 1, sh.lane_start, lanes);
    sh.first_lane = lo;
  }
  __syncthreads();
}

// ---- the fold of a CTA's last segment ---------------------------------------------------------------------------
// When a CTA flushes the last segment of its range no page of it is in flight any more and the ring is free. The
// twelve consumer warps leave their partials there (the flush's own stores, aimed at the ring) and the three warps
// of a KV head fold their three page residues into ONE partial: a third of the bytes leave the SM, and the merge reads a third. Every segment of a lane but its
// last is the last of its CTA (the lane goes on in the next CTA), so a lane's partials are one slot per segment, and
// three for its last segment when that segment's CTA goes on into the next lane (then the ring is busy); the decode
// kernel says which in bit 31 of the lane's descriptor.
constexpr uint32_t kFoldRow = kHeadDim + 4; // a row's floats in the ring: the pad spreads the lanes' stores over all banks
struct FoldScratch {
  float rows[kConsumerWarps][kGroup * kFoldRow];
  float stats[kConsumerWarps][kGroup * 2];
};
constexpr uint32_t kConsumersBarrier = 5; // named barriers 1..4 belong to the KV heads' warp triples
// The three warps of `head` (96 threads, `member` = 32 * residue + lane) fold their rows and store the one partial.
__device__ __forceinline__ void fold_and_store(const FoldScratch &fold, uint32_t head, uint32_t member, float *out, float *stats) {
#pragma unroll
  for (uint32_t i = 0; i < kGroup * (kHeadDim / 4) / (kPageWarps * 32); ++i) {
    const uint32_t item = member + kPageWarps * 32 * i, query_head = item >> 6, quad = item & 63u;
    float2 stat[kPageWarps];
    float maximum = -INFINITY;
#pragma unroll
    for (uint32_t r = 0; r < kPageWarps; ++r) {
      stat[r] = *reinterpret_cast<const float2 *>(&fold.stats[r * kKvHeads + head][query_head * 2]);
      maximum = fmaxf(maximum, stat[r].x);
    }
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float denominator = 0.0f;
#pragma unroll
    for (uint32_t r = 0; r < kPageWarps; ++r) { // residues in rising order: the same bits every time
      const float weight = stat[r].x == -INFINITY ? 0.0f : expf(stat[r].x - maximum);
      const float4 v = *reinterpret_cast<const float4 *>(&fold.rows[r * kKvHeads + head][query_head * kFoldRow + 4 * quad]);
      sum.x += weight * v.x; sum.y += weight * v.y; sum.z += weight * v.z; sum.w += weight * v.w;
      denominator += weight * stat[r].y;
    }
    *reinterpret_cast<float4 *>(out + query_head * kHeadDim + 4 * quad) = sum;
    if (quad == 0) { // a failed step left (-inf, 0) in every residue: it stays so
      stats[query_head * 2] = maximum;
      stats[query_head * 2 + 1] = denominator;
    }
  }
}
// A lane's descriptor {first segment, segments | last segment holds three slots << 31} -> its partial slots in order.
struct LaneSlots {
  uint32_t first, single, slots; // segments [first, first + single) hold one slot each; then up to three of segment first + single
  __device__ __forceinline__ explicit LaneSlots(uint2 descriptor) {
    const uint32_t segments = descriptor.y & 0x7fffffffu, triple = descriptor.y >> 31;
    first = descriptor.x;
    single = segments - (segments ? triple : 0u);
    slots = single + (segments - single) * kPageWarps;
  }
  __device__ __forceinline__ uint64_t slot(uint32_t t, uint32_t head) const {
    return t < single ? (uint64_t(first + t) * kKvHeads + head) * kPageWarps
                      : (uint64_t(first + single) * kKvHeads + head) * kPageWarps + (t - single);
  }
};

__device__ __forceinline__ void group_barrier(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
decode_int4_kernel(const __grid_constant__ CUtensorMap window_map, DecodeArgs args) {
  extern __shared__ uint8_t dynamic_shared[];
  // Stages need 1024-byte alignment for the 128-byte swizzle pattern.
  const uint32_t ring = (smem_address(dynamic_shared) + 1023u) & ~1023u;
  Shared &sh = *reinterpret_cast<Shared *>(dynamic_shared + (ring - smem_address(dynamic_shared)) + kStages * kStageBytes);
  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t lanes = args.lanes, cta = blockIdx.x;
  uint32_t *error_word = args.status;
  const uint32_t spin_limit = args.spin_limit;
  dependents_may_launch(); // the merge kernel's blocks may take their places; they wait for this grid to finish

  // ---- barriers, then the partition (the function's barriers publish both) --------------------
  if (tid == 0) {
    for (uint32_t s = 0; s < kStages; ++s) {
      barrier_init(smem_address(&sh.full[s]), 1);
      barrier_init(smem_address(&sh.empty[s]), kKvHeads * 32); // every lane of the page's four warps (one per head) releases it
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  cut_ranges(sh, args, kSwitchPages);
  const uint32_t range_begin = sh.range_begin, range_end = sh.range_end, first_lane = sh.first_lane;
  if (range_begin >= range_end) return;
  const Cut cut = sh.cut;

  if (warp >= kConsumerWarps) {
    // ================= producer: one thread streams whole pages =============================
    release_registers();
    if (warp != kConsumerWarps || lane != 0) return;
    uint32_t unit = 0; // pages issued by this CTA
    bool ok = true;
    // the timeout probe withholds the last pages of the range: their consumers must give up, not hang
    const uint32_t issue_limit = (range_end - range_begin) - min(args.withheld, range_end - range_begin);
    // The table pointer and the first entry of the lane after this one are fetched while this lane streams: under a
    // saturated memory system each of the two dependent loads takes microseconds, more than the ring holds.
    const rk_page_entry *upcoming_table = nullptr;
    rk_page_entry upcoming_first = 0;
    bool upcoming = false;
    for (uint32_t l = first_lane; ok && unit < issue_limit && l < lanes && sh.lane_start[l] < range_end; ++l) {
      const uint32_t lane_begin = sh.lane_start[l], lane_end = sh.lane_start[l + 1];
      const uint32_t pa = max(range_begin, lane_begin) - lane_begin;
      const uint32_t pb = min(range_end, lane_end) - lane_begin;
      if (pb <= pa || lane_end <= range_begin) continue;
      const rk_page_entry *table = upcoming ? upcoming_table : args.tables[l];
      rk_page_entry next_entry = upcoming ? upcoming_first : table[pa];
      // the next lane with pages in this range starts at its page 0
      uint32_t after = l + 1;
      while (after < lanes && sh.lane_start[after + 1] == sh.lane_start[after]) ++after;
      upcoming = after < lanes && sh.lane_start[after] < range_end;
      if (upcoming) upcoming_table = args.tables[after];
      const uint32_t fetch_at = pa + min(8u, pb - pa - 1);
      for (uint32_t page = pa; ok && unit < issue_limit && page < pb; ++page, ++unit) {
        const rk_page_entry entry = next_entry;
        if (page + 1 < pb) next_entry = table[page + 1]; // in flight while this page's copies are issued
        if (upcoming && page == fetch_at) upcoming_first = upcoming_table[0];
        const uint32_t index = rk_entry_index(entry);
        const uint64_t region = rk_entry_extent(entry) + args.layer.offset;
        const uint64_t pages = args.layer.extent_pages;
        const uint64_t keys = region + uint64_t(index) * kTensorBytes;
        const uint64_t key_scales = region + pages * kTensorBytes + uint64_t(index) * kScaleBytes;
        const uint64_t values = region + pages * (uint64_t(kTensorBytes) + kScaleBytes) + uint64_t(index) * kTensorBytes;
        const uint64_t value_scales = region + pages * (2ull * kTensorBytes + kScaleBytes) + uint64_t(index) * kScaleBytes;
        const uint32_t slot = unit % kStages, round = unit / kStages;
        const uint32_t full = smem_address(&sh.full[slot]), stage = ring + slot * kStageBytes;
        if (sh.error || !barrier_wait(smem_address(&sh.empty[slot]), (round & 1u) ^ 1u, spin_limit)) { ok = false; break; }
        barrier_expect(full, kStageBytes);
        tma_load_rows(stage, &window_map, int32_t((keys - args.window_base) >> 7), full);
        tma_load_rows(stage + kTensorBytes, &window_map, int32_t((values - args.window_base) >> 7), full);
        bulk_load(stage + 2 * kTensorBytes, reinterpret_cast<const void *>(key_scales), kScaleBytes, full);
        bulk_load(stage + 2 * kTensorBytes + kScaleBytes, reinterpret_cast<const void *>(value_scales), kScaleBytes, full);
      }
    }
    if (!ok) {
      atomicExch(error_word, 1u);
      sh.error = 1;
    }
    // Copies already issued must land before the block's shared memory goes: consumers that gave up no longer wait
    // for them. The last fill of each stage is the barrier's latest phase, so this returns at once when all went well.
    const uint32_t armed = min(unit, kStages);
    for (uint32_t back = 0; back < armed; ++back) {
      const uint32_t u = unit - 1 - back;
      barrier_wait(smem_address(&sh.full[u % kStages]), (u / kStages) & 1u, spin_limit);
    }
    return;
  }

  // ================= consumers: warp = (KV head, page residue) ===============================
  take_registers();
  const uint32_t head = warp & 3u, residue = warp >> 2;
  const uint32_t g = lane >> 2, c = lane & 3u;
  const uint32_t r3g = ((g & 1u) << 2) | (g >> 1); // row-in-8 swizzle partner: phase mates differ in bit 2
  const uint32_t kLowNibbles = register_constant(0x000F000Fu), kHighNibbles = register_constant(0x00F000F0u);
  const uint32_t kFlipLow = register_constant(0x00080008u), kFlipHigh = register_constant(0x00800080u);
  const uint32_t query_shared = smem_address(&sh.query[head][0][lane]);

  uint32_t units_before = 0; // pages of this CTA in earlier segments
  for (uint32_t l = first_lane; l < lanes && sh.lane_start[l] < range_end; ++l) {
    const uint32_t lane_begin = sh.lane_start[l], lane_end = sh.lane_start[l + 1];
    const uint32_t pa = max(range_begin, lane_begin) - lane_begin;
    const uint32_t pb = min(range_end, lane_end) - lane_begin;
    if (pb <= pa || lane_end <= range_begin) continue;
    const rk_verify_params p = args.lane_params[l];
    const uint32_t visible = p.committed_tokens + 1;
    const uint32_t lane_pages = lane_end - lane_begin;

    // ---- the head's query fragments (B operand of S^T = K.Q^T), shared by its three warps ----
    group_barrier(1 + head, kPageWarps * 32); // every warp of the head is done with the previous lane
    if (residue == 0) {
      const uint16_t *q = args.queries + ((uint64_t(l) * kKvHeads + head) * RK_VERIFY_CHUNK_STRIDE) * kGroup * kHeadDim +
                          uint64_t(g) * kHeadDim;
      float raw[2][4][8];
      float amax = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j)
#pragma unroll
        for (uint32_t w = 0; w < 4; ++w) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (g < kGroup) v = __ldg(reinterpret_cast<const uint4 *>(q + 32 * (c + 4 * j) + 8 * w));
          const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (uint32_t i = 0; i < 4; ++i) {
            raw[j][w][2 * i] = bf16_bits_to_float(words[i] & 0xffffu);
            raw[j][w][2 * i + 1] = bf16_bits_to_float(words[i] >> 16);
            amax = fmaxf(amax, fmaxf(fabsf(raw[j][w][2 * i]), fabsf(raw[j][w][2 * i + 1])));
          }
        }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      // Power-of-two prescale keeps every query inside fp16's range (exact).
      int exponent = 0;
      if (amax >= 8192.0f) exponent = ilogbf(amax) - 12;
      const float down = ldexpf(1.0f, -exponent);
      float qsum = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j)
#pragma unroll
        for (uint32_t w = 0; w < 4; ++w)
#pragma unroll
          for (uint32_t hs = 0; hs < 2; ++hs) {
            const uint32_t s = (j * 4 + w) * 2 + hs;
            const float e0 = raw[j][w][2 * hs] * down, e1 = raw[j][w][2 * hs + 4] * down;
            const float o0 = raw[j][w][2 * hs + 1] * down * 0.0625f, o1 = raw[j][w][2 * hs + 5] * down * 0.0625f;
            const __half2 even = __floats2half2_rn(e0, e1), odd = __floats2half2_rn(o0, o1);
            sh.query[head][s][lane] = make_uint2(*reinterpret_cast<const uint32_t *>(&even),
                                                 *reinterpret_cast<const uint32_t *>(&odd));
            qsum += __low2float(even) + __high2float(even) + 16.0f * (__low2float(odd) + __high2float(odd));
          }
      qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
      qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
      // scores (log2 domain) = fma(acc, factor, offset) * key_scale
      const float ss = rk_score_scale(p.score_scale, kHeadDim) * kLog2e;
      if (c == 0) {
        sh.head_factor[head][g] = ldexpf(ss, 24 + exponent);
        sh.head_offset[head][g] = -8.0f * qsum * ldexpf(ss, exponent);
      }
    }
    group_barrier(1 + head, kPageWarps * 32); // fragments visible to the head's warps
    float hfac[2], negoff[2];
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) { // C fragment columns are query heads 2c, 2c+1 of the group
      hfac[j] = sh.head_factor[head][2 * c + j];
      negoff[j] = sh.head_offset[head][2 * c + j];
    }

    float m[2] = {-1.0e30f, -1.0e30f}, l_sum[2] = {0.0f, 0.0f};
    float psum[2] = {0.0f, 0.0f}; // this lane's share of the sum of the rounded weights since the last correction
    uint32_t ridden = 0;          // pages since the last correction
    float o[16][4];
#pragma unroll
    for (uint32_t t = 0; t < 16; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f; }

    for (uint32_t page = pa + residue; page < pb && !sh.error; page += kPageWarps) {
      const uint32_t unit = units_before + (page - pa);
      const uint32_t slot = unit % kStages, round = unit / kStages;
      if (!barrier_wait(smem_address(&sh.full[slot]), round & 1u, spin_limit)) {
        atomicExch(error_word, 2u);
        sh.error = 2;
        break;
      }
      const uint32_t stage = ring + slot * kStageBytes;
      const uint32_t keys = stage + head * kSlabBytes;
      const uint32_t values = stage + kTensorBytes + head * kSlabBytes;
      const uint32_t scales = stage + 2 * kTensorBytes + head * (kPageTokens * 4);
      const uint32_t valid = page + 1 == lane_pages ? visible - page * kPageTokens : kPageTokens;

      // ---- S^T = K.Q^T : two 16-token tiles, 16 k-steps each --------------------------
      float sacc[2][2][4];
#pragma unroll
      for (uint32_t mt = 0; mt < 2; ++mt)
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) sacc[mt][h][0] = sacc[mt][h][1] = sacc[mt][h][2] = sacc[mt][h][3] = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        const uint32_t chunk = ((c + 4 * j) ^ r3g) * 16;
        uint4 kr[2][2];
#pragma unroll
        for (uint32_t mt = 0; mt < 2; ++mt) {
          kr[mt][0] = load_shared_16(keys + (16 * mt + r3g) * 128 + chunk);
          kr[mt][1] = load_shared_16(keys + (16 * mt + 8 + r3g) * 128 + chunk);
        }
#pragma unroll
        for (uint32_t w = 0; w < 4; ++w) {
          const uint32_t s = (j * 4 + w) * 2;
          uint2 q0, q1;
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(q0.x), "=r"(q0.y) : "r"(query_shared + s * 256) : "memory");
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(q1.x), "=r"(q1.y) : "r"(query_shared + (s + 1) * 256) : "memory");
#pragma unroll
          for (uint32_t mt = 0; mt < 2; ++mt) {
            const uint32_t xa = w == 0 ? kr[mt][0].x : w == 1 ? kr[mt][0].y : w == 2 ? kr[mt][0].z : kr[mt][0].w;
            const uint32_t xb = w == 0 ? kr[mt][1].x : w == 1 ? kr[mt][1].y : w == 2 ? kr[mt][1].z : kr[mt][1].w;
            const uint32_t ya = xa >> 8, yb = xb >> 8;
            mma_f16(sacc[mt][0], and_xor(xa, kLowNibbles, kFlipLow), and_xor(xb, kLowNibbles, kFlipLow),
                    and_xor(xa, kHighNibbles, kFlipHigh), and_xor(xb, kHighNibbles, kFlipHigh), q0.x, q0.y);
            mma_f16(sacc[mt][1], and_xor(ya, kLowNibbles, kFlipLow), and_xor(yb, kLowNibbles, kFlipLow),
                    and_xor(ya, kHighNibbles, kFlipHigh), and_xor(yb, kHighNibbles, kFlipHigh), q1.x, q1.y);
          }
        }
      }

      // ---- online softmax over the page's 32 tokens -------------------------------------
      uint32_t pb_frag[2][2];
      if (valid == kPageTokens)
        page_softmax<false, false, true>(sacc, hfac, negoff, scales, r3g, valid, m, l_sum, o, pb_frag, nullptr, psum);
      else
        page_softmax<true, false, true>(sacc, hfac, negoff, scales, r3g, valid, m, l_sum, o, pb_frag, nullptr, psum);

      // ---- O^T += V^T.P^T : 16 tiles of 16 dims, 2 k-steps of 16 tokens -----------------
#pragma unroll
      for (uint32_t s = 0; s < 2; ++s) {
        const uint32_t ta = 16 * s + c;
        const uint32_t chunk_a = (r3g ^ c) * 16, chunk_b = (r3g ^ (c + 4)) * 16;
        const uint4 va = load_shared_16(values + ta * 128 + chunk_a);
        const uint4 vb = load_shared_16(values + (ta + 4) * 128 + chunk_b);
        const uint4 vc = load_shared_16(values + (ta + 8) * 128 + chunk_a);
        const uint4 vd = load_shared_16(values + (ta + 12) * 128 + chunk_b);
        const uint32_t xa[4] = {va.x, va.y, va.z, va.w}, xb[4] = {vb.x, vb.y, vb.z, vb.w};
        const uint32_t xc[4] = {vc.x, vc.y, vc.z, vc.w}, xd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
        for (uint32_t w = 0; w < 4; ++w)
#pragma unroll
          for (uint32_t b = 0; b < 4; ++b) {
            const uint32_t selector = b | (b << 4) | ((4 + b) << 8) | ((4 + b) << 12);
            const uint32_t ab = __byte_perm(xa[w], xb[w], selector), cd = __byte_perm(xc[w], xd[w], selector);
            // low nibble: 1024 + (n ^ 8), minus 1032 = code; high nibble: 1024 + 16 (n ^ 8), minus 1152 = 16 code
            // codes travel as u * 2^-24 (u = code + 8; high nibbles x16), exact fp16 subnormals like the keys
            mma_f16(o[4 * w + b], and_xor(ab, kLowNibbles, kFlipLow), and_xor(ab, kHighNibbles, kFlipHigh),
                    and_xor(cd, kLowNibbles, kFlipLow), and_xor(cd, kHighNibbles, kFlipHigh), pb_frag[s][0], pb_frag[s][1]);
          }
      }
      // Every lane gives the stage back itself, behind a generic-to-async proxy fence: the stage was read through the
      // generic proxy (ld.shared) and is refilled through the async proxy (TMA), and an mbarrier arrive / wait pair alone
      // orders generic-proxy accesses only. Without the fence the refill of the next page in this stage was seen to
      // land under the last value rows the slowest warp was still reading.
      release_stage(smem_address(&sh.empty[slot]));
      if (++ridden == 64) { // the +8 never rides more than 64 pages of a warp's accumulation
        ridden = 0;
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j) {
          float total = psum[j];
          total += __shfl_xor_sync(0xffffffffu, total, 4);
          total += __shfl_xor_sync(0xffffffffu, total, 8);
          total += __shfl_xor_sync(0xffffffffu, total, 16);
          psum[j] = 0.0f;
#pragma unroll
          for (uint32_t t = 0; t < 16; ++t) { o[t][j] = fmaf(total, -4.76837158203125e-07f, o[t][j]); o[t][2 + j] = fmaf(total, -7.62939453125e-06f, o[t][2 + j]); }
        }
      }
    }
    units_before += pb - pa;

    // ---- flush this warp's partial of (lane l, head, page residue) --------------------------
    {
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 4);
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 8);
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 16);
      }
      const uint32_t segment = sh.segment_base[l] + (cta - cut.cta_of(lane_begin, l));
      const uint64_t slot_index = (uint64_t(segment) * kKvHeads + head) * kPageWarps + residue;
      // the CTA's last segment goes to the ring, to be folded there; any other straight to its slot
      const bool fold_here = range_end <= lane_end;
      FoldScratch &fold = *reinterpret_cast<FoldScratch *>(dynamic_shared + (ring - smem_address(dynamic_shared)));
      if (fold_here) group_barrier(kConsumersBarrier, kConsumerWarps * 32); // every consumer warp has read its last page
      if (warp == 0 && lane == 0 && pb == lane_pages) { // the lane's last segment: its descriptor, with how this segment is stored
        args.descriptors[2 * l] = sh.segment_base[l];
        args.descriptors[2 * l + 1] = (sh.segment_base[l + 1] - sh.segment_base[l]) | (fold_here ? 0u : 0x80000000u);
      }
      float *out = fold_here ? fold.rows[warp] : args.partials + slot_index * kGroup * kHeadDim;
      float *stats = fold_here ? fold.stats[warp] : args.statistics + slot_index * kGroup * 2;
      const uint32_t row_floats = fold_here ? kFoldRow : kHeadDim;
      const bool failed = sh.error != 0;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        psum[j] += __shfl_xor_sync(0xffffffffu, psum[j], 4);
        psum[j] += __shfl_xor_sync(0xffffffffu, psum[j], 8);
        psum[j] += __shfl_xor_sync(0xffffffffu, psum[j], 16);
      }
      // A lane holds 32 consecutive dimensions (one 128-byte line) of each of its two query heads. Lanes g and g ^ 2
      // hold neighbouring lines: they swap halves so that every store instruction writes whole 32-byte sectors (a
      // lane's own 16-byte pieces would leave every sector half written, and the path to L2 counts sectors).
      const bool upper = (g & 2u) != 0;
      float *line_low = out + 32 * (r3g & ~1u) + 4 * (upper ? 1u : 0u); // both lanes: the lower line, then the upper one
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        const uint32_t query_head = 2 * c + j;
        // accumulators hold 2^-24 * sum(u * w) (x16 for the odd dims), weights carry 2^14: take the +8 out, then 2^24 * 2^-14
        const float offset = psum[j] * 4.76837158203125e-07f; // 8 * 2^-24 * sum of weights
#pragma unroll
        for (uint32_t pair = 0; pair < 4; ++pair) { // 16-byte pieces 2 * pair and 2 * pair + 1 of the lane's line
          float piece[2][4];
#pragma unroll
          for (uint32_t h = 0; h < 2; ++h)
#pragma unroll
            for (uint32_t e = 0; e < 2; ++e) {
              const uint32_t t = 4 * pair + 2 * h + e;
              piece[h][2 * e] = (o[t][j] - offset) * 1024.0f;
              piece[h][2 * e + 1] = (o[t][2 + j] - 16.0f * offset) * 64.0f;
            }
          float theirs[4]; // the lower lane gives its odd piece away, the upper lane its even piece
#pragma unroll
          for (uint32_t e = 0; e < 4; ++e) theirs[e] = __shfl_xor_sync(0xffffffffu, upper ? piece[0][e] : piece[1][e], 8);
          if (query_head < kGroup) {
            float *target = line_low + query_head * row_floats + 8 * pair;
            *reinterpret_cast<float4 *>(target) = upper ? make_float4(theirs[0], theirs[1], theirs[2], theirs[3])
                                                        : make_float4(piece[0][0], piece[0][1], piece[0][2], piece[0][3]);
            *reinterpret_cast<float4 *>(target + 32) = upper ? make_float4(piece[1][0], piece[1][1], piece[1][2], piece[1][3])
                                                             : make_float4(theirs[0], theirs[1], theirs[2], theirs[3]);
          }
        }
        if (query_head >= kGroup) continue;
        if (g == 0) {
          stats[query_head * 2] = failed ? -INFINITY : m[j] * kLn2;
          stats[query_head * 2 + 1] = failed ? 0.0f : l_sum[j];
        }
      }
      if (fold_here) {
        group_barrier(1 + head, kPageWarps * 32);
        const uint64_t slot = (uint64_t(segment) * kKvHeads + head) * kPageWarps;
        fold_and_store(fold, head, residue * 32 + lane, args.partials + slot * kGroup * kHeadDim, args.statistics + slot * kGroup * 2);
      }
    }
  }
}

// ---- one-byte formats (int8, fp8 e4m3): the same streaming kernel with 8 KiB slabs and three stages -----------------
constexpr uint32_t kByteStages = 3;
constexpr uint32_t kByteSlabBytes = 8192;                          // one head's K (or V) of a page
constexpr uint32_t kByteTensorBytes = kKvHeads * kByteSlabBytes;   // all heads' K (or V) of a page: two 128-row TMA boxes
constexpr uint32_t kByteStageBytes = 2 * kByteTensorBytes + 2 * kScaleBytes;
static_assert(kByteStageBytes % 1024 == 0, "stages keep the 1 KiB swizzle alignment");

// Four key codes of one token row (dims d..d+3) -> the fragment halves (d, d+1) and (d+2, d+3).
// int8: u = code + 128 as fp16 bits, u * 2^-24 (exact subnormals; the +128 leaves through sum(q)); fp8: cvt, exact.
template <bool kFloat8> __device__ __forceinline__ void key_pairs(uint32_t word, uint32_t &first, uint32_t &second) {
  if (kFloat8) {
    asm("{\n.reg .b16 lo, hi;\nmov.b32 {lo, hi}, %2;\ncvt.rn.f16x2.e4m3x2 %0, lo;\ncvt.rn.f16x2.e4m3x2 %1, hi;\n}" : "=r"(first), "=r"(second) : "r"(word));
  } else {
    const uint32_t flipped = word ^ 0x80808080u;
    first = __byte_perm(flipped, 0, 0x4140);
    second = __byte_perm(flipped, 0, 0x4342);
  }
}
// Two value codes of one dim (bytes c0 and c0 + 2 of a word of four tokens) -> one fragment register, exact:
// int8 through 1024 + u minus 1152, fp8 through cvt.
template <bool kFloat8> __device__ __forceinline__ uint32_t value_pair(uint32_t word, uint32_t selector) {
  if (kFloat8) {
    uint32_t result;
    const uint32_t gathered = __byte_perm(word, 0, selector);
    asm("{\n.reg .b16 lo, hi;\nmov.b32 {lo, hi}, %1;\ncvt.rn.f16x2.e4m3x2 %0, lo;\n}" : "=r"(result) : "r"(gathered));
    return result;
  }
  return sub_f16x2(__byte_perm(word ^ 0x80808080u, 0x64646464u, selector), 0x64806480u);
}

template <bool kFloat8>
__global__ void __launch_bounds__(kThreads, 1)
decode_bytes_kernel(const __grid_constant__ CUtensorMap window_map, DecodeArgs args) {
  extern __shared__ uint8_t dynamic_shared[];
  // Stages need 1024-byte alignment for the 128-byte swizzle pattern.
  const uint32_t ring = (smem_address(dynamic_shared) + 1023u) & ~1023u;
  Shared &sh = *reinterpret_cast<Shared *>(dynamic_shared + (ring - smem_address(dynamic_shared)) + kByteStages * kByteStageBytes);
  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t lanes = args.lanes, cta = blockIdx.x;
  uint32_t *error_word = args.status;
  const uint32_t spin_limit = args.spin_limit;
  dependents_may_launch(); // the merge kernel's blocks may take their places; they wait for this grid to finish

  // ---- barriers, then the partition (the function's barriers publish both) --------------------
  if (tid == 0) {
    for (uint32_t s = 0; s < kByteStages; ++s) {
      barrier_init(smem_address(&sh.full[s]), 1);
      barrier_init(smem_address(&sh.empty[s]), kKvHeads * 32); // every lane of the page's four warps (one per head) releases it
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  cut_ranges(sh, args, kByteSwitchPages);
  const uint32_t range_begin = sh.range_begin, range_end = sh.range_end, first_lane = sh.first_lane;
  if (range_begin >= range_end) return;
  const Cut cut = sh.cut;

  if (warp >= kConsumerWarps) {
    // ================= producer: one thread streams whole pages =============================
    release_registers();
    if (warp != kConsumerWarps || lane != 0) return;
    uint32_t unit = 0; // pages issued by this CTA
    bool ok = true;
    // the timeout probe withholds the last pages of the range: their consumers must give up, not hang
    const uint32_t issue_limit = (range_end - range_begin) - min(args.withheld, range_end - range_begin);
    for (uint32_t l = first_lane; ok && unit < issue_limit && l < lanes && sh.lane_start[l] < range_end; ++l) {
      const uint32_t lane_begin = sh.lane_start[l], lane_end = sh.lane_start[l + 1];
      const uint32_t pa = max(range_begin, lane_begin) - lane_begin;
      const uint32_t pb = min(range_end, lane_end) - lane_begin;
      if (pb <= pa || lane_end <= range_begin) continue;
      const rk_page_entry *table = args.tables[l];
      rk_page_entry next_entry = table[pa];
      for (uint32_t page = pa; ok && unit < issue_limit && page < pb; ++page, ++unit) {
        const rk_page_entry entry = next_entry;
        if (page + 1 < pb) next_entry = table[page + 1]; // in flight while this page's copies are issued
        const uint32_t index = rk_entry_index(entry);
        const uint64_t region = rk_entry_extent(entry) + args.layer.offset;
        const uint64_t pages = args.layer.extent_pages;
        const uint64_t keys = region + uint64_t(index) * kByteTensorBytes;
        const uint64_t key_scales = region + pages * kByteTensorBytes + uint64_t(index) * kScaleBytes;
        const uint64_t values = region + pages * (uint64_t(kByteTensorBytes) + kScaleBytes) + uint64_t(index) * kByteTensorBytes;
        const uint64_t value_scales = region + pages * (2ull * kByteTensorBytes + kScaleBytes) + uint64_t(index) * kScaleBytes;
        const uint32_t slot = unit % kByteStages, round = unit / kByteStages;
        const uint32_t full = smem_address(&sh.full[slot]), stage = ring + slot * kByteStageBytes;
        if (sh.error || !barrier_wait(smem_address(&sh.empty[slot]), (round & 1u) ^ 1u, spin_limit)) { ok = false; break; }
        barrier_expect(full, kByteStageBytes);
        const int32_t key_row = int32_t((keys - args.window_base) >> 7), value_row = int32_t((values - args.window_base) >> 7);
        tma_load_rows(stage, &window_map, key_row, full);                                   // heads 0-1 (128 rows of 128 bytes)
        tma_load_rows(stage + kByteTensorBytes / 2, &window_map, key_row + 128, full);      // heads 2-3
        tma_load_rows(stage + kByteTensorBytes, &window_map, value_row, full);
        tma_load_rows(stage + kByteTensorBytes + kByteTensorBytes / 2, &window_map, value_row + 128, full);
        bulk_load(stage + 2 * kByteTensorBytes, reinterpret_cast<const void *>(key_scales), kScaleBytes, full);
        bulk_load(stage + 2 * kByteTensorBytes + kScaleBytes, reinterpret_cast<const void *>(value_scales), kScaleBytes, full);
      }
    }
    if (!ok) {
      atomicExch(error_word, 1u);
      sh.error = 1;
    }
    // Copies already issued must land before the block's shared memory goes: consumers that gave up no longer wait
    // for them. The last fill of each stage is the barrier's latest phase, so this returns at once when all went well.
    const uint32_t armed = min(unit, kByteStages);
    for (uint32_t back = 0; back < armed; ++back) {
      const uint32_t u = unit - 1 - back;
      barrier_wait(smem_address(&sh.full[u % kByteStages]), (u / kByteStages) & 1u, spin_limit);
    }
    return;
  }

  // ================= consumers: warp = (KV head, page residue) ===============================
  take_registers();
  const uint32_t head = warp & 3u, residue = warp >> 2;
  const uint32_t g = lane >> 2, c = lane & 3u;
  // MMA row g (and g+8) of a 16-token tile is token r3g (and 8 + r3g) of its 16: bits 0 and 1 of g swapped. A token
  // row is two 128-byte swizzle rows here, so the two rows a shared-memory phase reads (g, g^1) must differ by 2.
  const uint32_t r3g = (g & 4u) | ((g & 1u) << 1) | ((g >> 1) & 1u);
  const uint32_t c0 = c & 1u, c1 = c >> 1;
  // value bytes of this lane inside a 32-bit word of four tokens: bytes c0 and c0 + 2
  const uint32_t value_selector = kFloat8 ? (c0 | ((c0 + 2) << 4) | 0x4400u) : (c0 | (4u << 4) | ((c0 + 2) << 8) | (4u << 12));
  const uint32_t query_shared = smem_address(&sh.query[head][0][lane]);

  uint32_t units_before = 0; // pages of this CTA in earlier segments
  for (uint32_t l = first_lane; l < lanes && sh.lane_start[l] < range_end; ++l) {
    const uint32_t lane_begin = sh.lane_start[l], lane_end = sh.lane_start[l + 1];
    const uint32_t pa = max(range_begin, lane_begin) - lane_begin;
    const uint32_t pb = min(range_end, lane_end) - lane_begin;
    if (pb <= pa || lane_end <= range_begin) continue;
    const rk_verify_params p = args.lane_params[l];
    const uint32_t visible = p.committed_tokens + 1;
    const uint32_t lane_pages = lane_end - lane_begin;

    // ---- the head's query fragments (B operand of S^T = K.Q^T), shared by its three warps ----
    group_barrier(1 + head, kPageWarps * 32); // every warp of the head is done with the previous lane
    if (residue == 0) {
      const uint16_t *q = args.queries + ((uint64_t(l) * kKvHeads + head) * RK_VERIFY_CHUNK_STRIDE) * kGroup * kHeadDim +
                          uint64_t(g) * kHeadDim;
      // k-step s = 4j + w covers, for lane column c, dims 16(c + 4j) + 4w .. +3: b0 = the first two, b1 = the last two
      float raw[4][4][4];
      float amax = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) {
        uint4 v[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        if (g < kGroup) {
          v[0] = __ldg(reinterpret_cast<const uint4 *>(q + 16 * (c + 4 * j)));
          v[1] = __ldg(reinterpret_cast<const uint4 *>(q + 16 * (c + 4 * j) + 8));
        }
        const uint32_t words[8] = {v[0].x, v[0].y, v[0].z, v[0].w, v[1].x, v[1].y, v[1].z, v[1].w};
#pragma unroll
        for (uint32_t w = 0; w < 4; ++w)
#pragma unroll
          for (uint32_t i = 0; i < 2; ++i) {
            raw[j][w][2 * i] = bf16_bits_to_float(words[2 * w + i] & 0xffffu);
            raw[j][w][2 * i + 1] = bf16_bits_to_float(words[2 * w + i] >> 16);
            amax = fmaxf(amax, fmaxf(fabsf(raw[j][w][2 * i]), fabsf(raw[j][w][2 * i + 1])));
          }
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      // Power-of-two prescale keeps every query inside fp16's range (exact).
      int exponent = 0;
      if (amax >= 8192.0f) exponent = ilogbf(amax) - 12;
      const float down = ldexpf(1.0f, -exponent);
      float qsum = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j)
#pragma unroll
        for (uint32_t w = 0; w < 4; ++w) {
          const __half2 first = __floats2half2_rn(raw[j][w][0] * down, raw[j][w][1] * down);
          const __half2 second = __floats2half2_rn(raw[j][w][2] * down, raw[j][w][3] * down);
          sh.query[head][4 * j + w][lane] = make_uint2(*reinterpret_cast<const uint32_t *>(&first), *reinterpret_cast<const uint32_t *>(&second));
          qsum += __low2float(first) + __high2float(first) + __low2float(second) + __high2float(second);
        }
      qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
      qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
      // scores (log2 domain) = fma(acc, factor, offset) * key_scale
      const float ss = rk_score_scale(p.score_scale, kHeadDim) * kLog2e;
      if (c == 0) {
        // int8 keys travel as u * 2^-24 with u = code + 128; fp8 keys as their value
        sh.head_factor[head][g] = ldexpf(ss, (kFloat8 ? 0 : 24) + exponent);
        sh.head_offset[head][g] = kFloat8 ? 0.0f : -128.0f * qsum * ldexpf(ss, exponent);
      }
    }
    group_barrier(1 + head, kPageWarps * 32); // fragments visible to the head's warps
    float hfac[2], negoff[2];
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) { // C fragment columns are query heads 2c, 2c+1 of the group
      hfac[j] = sh.head_factor[head][2 * c + j];
      negoff[j] = sh.head_offset[head][2 * c + j];
    }

    float m[2] = {-1.0e30f, -1.0e30f}, l_sum[2] = {0.0f, 0.0f};
    float o[16][4];
#pragma unroll
    for (uint32_t t = 0; t < 16; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f; }

    for (uint32_t page = pa + residue; page < pb && !sh.error; page += kPageWarps) {
      const uint32_t unit = units_before + (page - pa);
      const uint32_t slot = unit % kByteStages, round = unit / kByteStages;
      if (!barrier_wait(smem_address(&sh.full[slot]), round & 1u, spin_limit)) {
        atomicExch(error_word, 2u);
        sh.error = 2;
        break;
      }
      const uint32_t stage = ring + slot * kByteStageBytes;
      const uint32_t keys = stage + head * kByteSlabBytes;
      const uint32_t values = stage + kByteTensorBytes + head * kByteSlabBytes;
      const uint32_t scales = stage + 2 * kByteTensorBytes + head * (kPageTokens * 4);
      const uint32_t valid = page + 1 == lane_pages ? visible - page * kPageTokens : kPageTokens;

      // ---- S^T = K.Q^T : two 16-token tiles, 16 k-steps each --------------------------
      float sacc[2][2][4];
#pragma unroll
      for (uint32_t mt = 0; mt < 2; ++mt)
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) sacc[mt][h][0] = sacc[mt][h][1] = sacc[mt][h][2] = sacc[mt][h][3] = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) { // 16-byte chunk c + 4j of each token row: 16 dims = four k-steps
        const uint32_t half_row = j >> 1, chunk = c + 4 * (j & 1u);
        uint4 kr[2][2];
#pragma unroll
        for (uint32_t mt = 0; mt < 2; ++mt) {
          const uint32_t row_a = 2 * (16 * mt + r3g) + half_row, row_b = 2 * (16 * mt + 8 + r3g) + half_row;
          kr[mt][0] = load_shared_16(keys + row_a * 128 + ((chunk ^ (row_a & 7u)) << 4));
          kr[mt][1] = load_shared_16(keys + row_b * 128 + ((chunk ^ (row_b & 7u)) << 4));
        }
#pragma unroll
        for (uint32_t w = 0; w < 4; ++w) {
          const uint32_t s = j * 4 + w;
          uint2 q;
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(q.x), "=r"(q.y) : "r"(query_shared + s * 256) : "memory");
#pragma unroll
          for (uint32_t mt = 0; mt < 2; ++mt) {
            const uint32_t xa = w == 0 ? kr[mt][0].x : w == 1 ? kr[mt][0].y : w == 2 ? kr[mt][0].z : kr[mt][0].w;
            const uint32_t xb = w == 0 ? kr[mt][1].x : w == 1 ? kr[mt][1].y : w == 2 ? kr[mt][1].z : kr[mt][1].w;
            uint32_t a0, a1, a2, a3;
            key_pairs<kFloat8>(xa, a0, a2);
            key_pairs<kFloat8>(xb, a1, a3);
            mma_f16(sacc[mt][w & 1u], a0, a1, a2, a3, q.x, q.y);
          }
        }
      }

      // ---- online softmax over the page's 32 tokens -------------------------------------
      uint32_t pb_frag[2][2];
      if (valid == kPageTokens)
        page_softmax<false>(sacc, hfac, negoff, scales, r3g, valid, m, l_sum, o, pb_frag);
      else
        page_softmax<true>(sacc, hfac, negoff, scales, r3g, valid, m, l_sum, o, pb_frag);

      if (kFloat8 && valid != kPageTokens) {
        // A lane's last page: stale bytes past the visible tokens may decode to NaN, and a zero weight must meet a
        // finite value. The head's value slab belongs to this warp alone, so the stale bytes are zeroed in place,
        // once, and the contraction below carries no mask. Word i of the slab: swizzle row i / 32, physical chunk
        // (i % 32) / 4 = logical chunk ^ (row % 8), whose low bit is the half of the page; tokens rise with the bytes.
        for (uint32_t i = lane; i < kByteSlabBytes / 4; i += 32) {
          const uint32_t row = i >> 5, half = (((i >> 2) & 7u) ^ row) & 1u;
          const uint32_t first_token = 16 * half + 4 * (i & 3u);
          if (first_token + 4 <= valid) continue;
          const uint32_t keep = first_token >= valid ? 0u : (1u << (8 * (valid - first_token))) - 1u;
          const uint32_t word = load_shared_32(values + 4 * i) & keep;
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(values + 4 * i), "r"(word) : "memory");
        }
        __syncwarp();
      }
      // ---- O^T += V^T.P^T : 16 tiles of 16 dims (rows g and g+8 of a tile = dims 16t+g, 16t+8+g), 2 k-steps of 16 tokens
#pragma unroll
      for (uint32_t s = 0; s < 2; ++s) {
#pragma unroll
        for (uint32_t t = 0; t < 16; ++t) {
          // a dim's 32 token bytes are a quarter of a 128-byte swizzle row; this k-step reads its half s (16 bytes)
          const uint32_t dim_a = 16 * t + g, dim_b = dim_a + 8;
          const uint32_t row_a = dim_a >> 2, row_b = dim_b >> 2;
          const uint4 va = load_shared_16(values + row_a * 128 + ((((dim_a & 3u) * 2 + s) ^ (row_a & 7u)) << 4));
          const uint4 vb = load_shared_16(values + row_b * 128 + ((((dim_b & 3u) * 2 + s) ^ (row_b & 7u)) << 4));
          // this lane's tokens of the 16: 4 c1 + c0 (+2) in word c1, 8 + the same in word c1 + 2
          uint32_t a0 = value_pair<kFloat8>(c1 ? va.y : va.x, value_selector), a2 = value_pair<kFloat8>(c1 ? va.w : va.z, value_selector);
          uint32_t a1 = value_pair<kFloat8>(c1 ? vb.y : vb.x, value_selector), a3 = value_pair<kFloat8>(c1 ? vb.w : vb.z, value_selector);
          mma_f16(o[t], a0, a1, a2, a3, pb_frag[s][0], pb_frag[s][1]);
        }
      }
      // Every lane gives the stage back itself, behind a generic-to-async proxy fence: the stage was read through the
      // generic proxy (ld.shared) and is refilled through the async proxy (TMA), and an mbarrier arrive / wait pair alone
      // orders generic-proxy accesses only. Without the fence the refill of the next page in this stage was seen to
      // land under the last value rows the slowest warp was still reading.
      release_stage(smem_address(&sh.empty[slot]));
    }
    units_before += pb - pa;

    // ---- flush this warp's partial of (lane l, head, page residue) --------------------------
    {
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 4);
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 8);
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 16);
      }
      const uint32_t segment = sh.segment_base[l] + (cta - cut.cta_of(lane_begin, l));
      const uint64_t slot_index = (uint64_t(segment) * kKvHeads + head) * kPageWarps + residue;
      // the CTA's last segment goes to the ring, to be folded there; any other straight to its slot
      const bool fold_here = range_end <= lane_end;
      FoldScratch &fold = *reinterpret_cast<FoldScratch *>(dynamic_shared + (ring - smem_address(dynamic_shared)));
      if (fold_here) group_barrier(kConsumersBarrier, kConsumerWarps * 32); // every consumer warp has read its last page
      if (warp == 0 && lane == 0 && pb == lane_pages) { // the lane's last segment: its descriptor, with how this segment is stored
        args.descriptors[2 * l] = sh.segment_base[l];
        args.descriptors[2 * l + 1] = (sh.segment_base[l + 1] - sh.segment_base[l]) | (fold_here ? 0u : 0x80000000u);
      }
      float *out = fold_here ? fold.rows[warp] : args.partials + slot_index * kGroup * kHeadDim;
      float *stats = fold_here ? fold.stats[warp] : args.statistics + slot_index * kGroup * 2;
      const uint32_t row_floats = fold_here ? kFoldRow : kHeadDim;
      const float unscale = 6.103515625e-05f; // 2^-14
      const bool failed = sh.error != 0;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        const uint32_t query_head = 2 * c + j;
        if (query_head >= kGroup) continue;
#pragma unroll
        for (uint32_t t = 0; t < 16; ++t) {
          out[query_head * row_floats + 16 * t + g] = o[t][j] * unscale;
          out[query_head * row_floats + 16 * t + 8 + g] = o[t][2 + j] * unscale;
        }
        if (g == 0) {
          stats[query_head * 2] = failed ? -INFINITY : m[j] * kLn2;
          stats[query_head * 2 + 1] = failed ? 0.0f : l_sum[j];
        }
      }
      if (fold_here) {
        group_barrier(1 + head, kPageWarps * 32);
        const uint64_t slot = (uint64_t(segment) * kKvHeads + head) * kPageWarps;
        fold_and_store(fold, head, residue * 32 + lane, args.partials + slot * kGroup * kHeadDim, args.statistics + slot * kGroup * 2);
      }
    }
  }
}

// ---- bf16 pools: (page, KV head) units of 16 KiB keys + 16 KiB values, six stages, no scales --------------------------
// Keys, values and queries stay bf16 (mma.sync bf16 operands, fp32 accumulate); a probability travels as two bf16
// parts so its precision matches the fp16 probabilities of the other formats.
constexpr uint32_t kWideStages = 6;
constexpr uint32_t kWideSlabBytes = 16384; // one head's K (or V) of a page: one 128-row TMA box
constexpr uint32_t kWideStageBytes = 2 * kWideSlabBytes;
static_assert(kWideStages <= kStages, "the barrier arrays hold the stages");

__global__ void __launch_bounds__(kThreads, 1)
decode_bf16_kernel(const __grid_constant__ CUtensorMap window_map, DecodeArgs args) {
  extern __shared__ uint8_t dynamic_shared[];
  // Stages need 1024-byte alignment for the 128-byte swizzle pattern.
  const uint32_t ring = (smem_address(dynamic_shared) + 1023u) & ~1023u;
  Shared &sh = *reinterpret_cast<Shared *>(dynamic_shared + (ring - smem_address(dynamic_shared)) + kWideStages * kWideStageBytes);
  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t lanes = args.lanes, cta = blockIdx.x;
  uint32_t *error_word = args.status;
  const uint32_t spin_limit = args.spin_limit;
  dependents_may_launch(); // the merge kernel's blocks may take their places; they wait for this grid to finish

  // ---- barriers, then the partition (the function's barriers publish both) --------------------
  if (tid == 0) {
    // A unit is one head's slabs of one page and has one consumer warp. Each warp waits on its own "full" barrier,
    // so it sees every completion of the barrier it waits on (a parity wait cannot tell completions two apart);
    // the stages themselves are released through per-stage "empty" barriers that only the producer waits on.
    for (uint32_t s = 0; s < kWideStages; ++s) barrier_init(smem_address(&sh.empty[s]), 32); // every lane of the unit's warp
    for (uint32_t w = 0; w < kConsumerWarps; ++w) barrier_init(smem_address(&sh.warp_full[w]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (uint32_t i = tid; i < sizeof(sh.unit_scales) / sizeof(float); i += kThreads) sh.unit_scales[i] = 1.0f;
  cut_ranges(sh, args, kWideSwitchPages);
  const uint32_t range_begin = sh.range_begin, range_end = sh.range_end, first_lane = sh.first_lane;
  if (range_begin >= range_end) return;
  const Cut cut = sh.cut;

  if (warp >= kConsumerWarps) {
    // ================= producer: one thread streams (page, KV head) units of 32 KiB =============
    release_registers();
    if (warp != kConsumerWarps || lane != 0) return;
    uint32_t unit = 0, ordinal = 0; // units issued by this CTA; pages of this CTA before the current one
    bool ok = true;
    // the timeout probe withholds the last pages of the range: their consumers must give up, not hang
    const uint32_t issue_limit = (range_end - range_begin) - min(args.withheld, range_end - range_begin);
    for (uint32_t l = first_lane; ok && ordinal < issue_limit && l < lanes && sh.lane_start[l] < range_end; ++l) {
      const uint32_t lane_begin = sh.lane_start[l], lane_end = sh.lane_start[l + 1];
      const uint32_t pa = max(range_begin, lane_begin) - lane_begin;
      const uint32_t pb = min(range_end, lane_end) - lane_begin;
      if (pb <= pa || lane_end <= range_begin) continue;
      const rk_page_entry *table = args.tables[l];
      rk_page_entry next_entry = table[pa];
      for (uint32_t page = pa; ok && ordinal < issue_limit && page < pb; ++page, ++ordinal) {
        const rk_page_entry entry = next_entry;
        if (page + 1 < pb) next_entry = table[page + 1]; // in flight while this page's copies are issued
        const uint32_t index = rk_entry_index(entry);
        const uint64_t region = rk_entry_extent(entry) + args.layer.offset;
        const uint64_t keys = region + uint64_t(index) * (kKvHeads * kWideSlabBytes);
        const uint64_t values = keys + args.layer.extent_pages * uint64_t(kKvHeads * kWideSlabBytes);
        const int32_t key_row = int32_t((keys - args.window_base) >> 7), value_row = int32_t((values - args.window_base) >> 7);
        for (uint32_t head = 0; head < kKvHeads; ++head, ++unit) {
          // page ordinal n of this CTA belongs to the warps of residue n % 3; a warp's units are 12 apart in issue
          // order and the ring holds 6, so a warp's barrier never has two fills in flight
          const uint32_t slot = unit % kWideStages, round = unit / kWideStages;
          const uint32_t full = smem_address(&sh.warp_full[head + kKvHeads * (ordinal % kPageWarps)]), stage = ring + slot * kWideStageBytes;
          if (sh.error || !barrier_wait(smem_address(&sh.empty[slot]), (round & 1u) ^ 1u, spin_limit)) { ok = false; break; }
          barrier_expect(full, kWideStageBytes);
          tma_load_rows(stage, &window_map, key_row + int32_t(head * (kWideSlabBytes / 128)), full); // 128 rows of 128 bytes
          tma_load_rows(stage + kWideSlabBytes, &window_map, value_row + int32_t(head * (kWideSlabBytes / 128)), full);
        }
      }
    }
    if (!ok) {
      atomicExch(error_word, 1u);
      sh.error = 1;
    }
    // Copies already issued must land before the block's shared memory goes: consumers that gave up no longer wait
    // for them. The last six units are the latest fills of six different warp barriers.
    const uint32_t armed = min(unit, kWideStages);
    for (uint32_t back = 0; back < armed; ++back) {
      const uint32_t u = unit - 1 - back, n = u / kKvHeads;
      barrier_wait(smem_address(&sh.warp_full[u % kKvHeads + kKvHeads * (n % kPageWarps)]), (n / kPageWarps) & 1u, spin_limit);
    }
    return;
  }

  // ================= consumers: warp = (KV head, page residue) ===============================
  take_registers();
  const uint32_t head = warp & 3u, residue = warp >> 2;
  const uint32_t g = lane >> 2, c = lane & 3u;
  // A token row is four 128-byte swizzle rows, so neighbouring tokens already differ in bit 2 of the row:
  // MMA row g (and g+8) of a 16-token tile is simply token g (and 8 + g).
  const uint32_t r3g = g;
  const uint32_t query_shared = smem_address(&sh.query[head][0][lane]);
  const uint32_t scales = smem_address(&sh.unit_scales[0]);

  uint32_t units_before = 0; // pages of this CTA in earlier segments
  for (uint32_t l = first_lane; l < lanes && sh.lane_start[l] < range_end; ++l) {
    const uint32_t lane_begin = sh.lane_start[l], lane_end = sh.lane_start[l + 1];
    const uint32_t pa = max(range_begin, lane_begin) - lane_begin;
    const uint32_t pb = min(range_end, lane_end) - lane_begin;
    if (pb <= pa || lane_end <= range_begin) continue;
    const rk_verify_params p = args.lane_params[l];
    const uint32_t visible = p.committed_tokens + 1;
    const uint32_t lane_pages = lane_end - lane_begin;

    // ---- the head's query fragments (B operand of S^T = K.Q^T), shared by its three warps ----
    group_barrier(1 + head, kPageWarps * 32); // every warp of the head is done with the previous lane
    if (residue == 0) {
      const uint16_t *q = args.queries + ((uint64_t(l) * kKvHeads + head) * RK_VERIFY_CHUNK_STRIDE) * kGroup * kHeadDim +
                          uint64_t(g) * kHeadDim;
      // k-step s = 2j + w covers, for lane column c, dims 8(c + 4j) + 4w .. +3: b0 = the first two, b1 = the last two.
      // Queries and keys are both bf16: nothing is converted.
#pragma unroll
      for (uint32_t j = 0; j < 8; ++j) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < kGroup) v = __ldg(reinterpret_cast<const uint4 *>(q + 8 * (c + 4 * j)));
        sh.query[head][2 * j][lane] = make_uint2(v.x, v.y);
        sh.query[head][2 * j + 1][lane] = make_uint2(v.z, v.w);
      }
      if (c == 0) {
        sh.head_factor[head][g] = rk_score_scale(p.score_scale, kHeadDim) * kLog2e; // scores in the log2 domain
        sh.head_offset[head][g] = 0.0f;
      }
    }
    group_barrier(1 + head, kPageWarps * 32); // fragments visible to the head's warps
    float hfac[2], negoff[2];
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) { // C fragment columns are query heads 2c, 2c+1 of the group
      hfac[j] = sh.head_factor[head][2 * c + j];
      negoff[j] = sh.head_offset[head][2 * c + j];
    }

    float m[2] = {-1.0e30f, -1.0e30f}, l_sum[2] = {0.0f, 0.0f};
    float o[16][4];
#pragma unroll
    for (uint32_t t = 0; t < 16; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f; }

    // this warp takes the pages whose ordinal inside the CTA's range is its residue modulo 3
    for (uint32_t page = pa + (residue + kPageWarps - units_before % kPageWarps) % kPageWarps; page < pb && !sh.error; page += kPageWarps) {
      const uint32_t ordinal = units_before + (page - pa);
      const uint32_t slot = (ordinal * kKvHeads + head) % kWideStages;
      if (!barrier_wait(smem_address(&sh.warp_full[warp]), (ordinal / kPageWarps) & 1u, spin_limit)) {
        atomicExch(error_word, 2u);
        sh.error = 2;
        break;
      }
      const uint32_t keys = ring + slot * kWideStageBytes;
      const uint32_t values = keys + kWideSlabBytes;
      const uint32_t valid = page + 1 == lane_pages ? visible - page * kPageTokens : kPageTokens;

      // ---- S^T = K.Q^T : two 16-token tiles, 16 k-steps each --------------------------
      float sacc[2][2][4];
#pragma unroll
      for (uint32_t mt = 0; mt < 2; ++mt)
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) sacc[mt][h][0] = sacc[mt][h][1] = sacc[mt][h][2] = sacc[mt][h][3] = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < 8; ++j) { // 16-byte chunk c + 4j of each 512-byte token row: 8 dims = two k-steps
        const uint32_t quarter = j >> 1, chunk = c + 4 * (j & 1u);
        uint4 kr[2][2];
#pragma unroll
        for (uint32_t mt = 0; mt < 2; ++mt) {
          const uint32_t row_a = 4 * (16 * mt + g) + quarter, row_b = 4 * (16 * mt + 8 + g) + quarter;
          kr[mt][0] = load_shared_16(keys + row_a * 128 + ((chunk ^ (row_a & 7u)) << 4));
          kr[mt][1] = load_shared_16(keys + row_b * 128 + ((chunk ^ (row_b & 7u)) << 4));
        }
#pragma unroll
        for (uint32_t w = 0; w < 2; ++w) {
          uint2 q;
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(q.x), "=r"(q.y) : "r"(query_shared + (2 * j + w) * 256) : "memory");
#pragma unroll
          for (uint32_t mt = 0; mt < 2; ++mt)
            mma_bf16(sacc[mt][w], w ? kr[mt][0].z : kr[mt][0].x, w ? kr[mt][1].z : kr[mt][1].x,
                     w ? kr[mt][0].w : kr[mt][0].y, w ? kr[mt][1].w : kr[mt][1].y, q.x, q.y);
        }
      }

      // ---- online softmax over the page's 32 tokens -------------------------------------
      uint32_t pb_frag[2][2], pb_low[2][2];
      if (valid == kPageTokens)
        page_softmax<false, true>(sacc, hfac, negoff, scales, r3g, valid, m, l_sum, o, pb_frag, pb_low);
      else
        page_softmax<true, true>(sacc, hfac, negoff, scales, r3g, valid, m, l_sum, o, pb_frag, pb_low);

      // ---- O^T += V^T.P^T : 16 tiles of 16 dims (rows g and g+8 of a tile = dims 16t+g, 16t+8+g), 2 k-steps of 16 tokens
#pragma unroll
      for (uint32_t s = 0; s < 2; ++s) {
        // this lane's tokens of the 16: 2c, 2c+1 (one word) and 8 + the same
        uint32_t low = 0xffffffffu, high = 0xffffffffu;
        if (valid != kPageTokens) { // stale bits past the visible tokens may be NaN: a zero weight must meet a finite value
          const uint32_t token = 16 * s + 2 * c;
          low = (token < valid ? 0x0000ffffu : 0u) | (token + 1 < valid ? 0xffff0000u : 0u);
          high = (token + 8 < valid ? 0x0000ffffu : 0u) | (token + 9 < valid ? 0xffff0000u : 0u);
        }
#pragma unroll
        for (uint32_t t = 0; t < 16; ++t) {
          // a dim's 32 tokens are half of a 128-byte swizzle row; this k-step reads two 16-byte chunks of it
          const uint32_t dim_a = 16 * t + g, dim_b = dim_a + 8;
          const uint32_t row_a = dim_a >> 1, row_b = dim_b >> 1;
          const uint32_t chunk_a = (dim_a & 1u) * 4 + 2 * s, chunk_b = (dim_b & 1u) * 4 + 2 * s;
          const uint32_t a0 = load_shared_32(values + row_a * 128 + ((chunk_a ^ (row_a & 7u)) << 4) + 4 * c) & low;
          const uint32_t a2 = load_shared_32(values + row_a * 128 + (((chunk_a + 1) ^ (row_a & 7u)) << 4) + 4 * c) & high;
          const uint32_t a1 = load_shared_32(values + row_b * 128 + ((chunk_b ^ (row_b & 7u)) << 4) + 4 * c) & low;
          const uint32_t a3 = load_shared_32(values + row_b * 128 + (((chunk_b + 1) ^ (row_b & 7u)) << 4) + 4 * c) & high;
          mma_bf16(o[t], a0, a1, a2, a3, pb_frag[s][0], pb_frag[s][1]);
          mma_bf16(o[t], a0, a1, a2, a3, pb_low[s][0], pb_low[s][1]);
        }
      }
      // Every lane gives the stage back itself, behind a generic-to-async proxy fence: the stage was read through the
      // generic proxy (ld.shared) and is refilled through the async proxy (TMA), and an mbarrier arrive / wait pair alone
      // orders generic-proxy accesses only. Without the fence the refill of the next page in this stage was seen to
      // land under the last value rows the slowest warp was still reading.
      release_stage(smem_address(&sh.empty[slot]));
    }
    units_before += pb - pa;

    // ---- flush this warp's partial of (lane l, head, page residue) --------------------------
    {
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 4);
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 8);
        l_sum[j] += __shfl_xor_sync(0xffffffffu, l_sum[j], 16);
      }
      const uint32_t segment = sh.segment_base[l] + (cta - cut.cta_of(lane_begin, l));
      const uint64_t slot_index = (uint64_t(segment) * kKvHeads + head) * kPageWarps + residue;
      // the CTA's last segment goes to the ring, to be folded there; any other straight to its slot
      const bool fold_here = range_end <= lane_end;
      FoldScratch &fold = *reinterpret_cast<FoldScratch *>(dynamic_shared + (ring - smem_address(dynamic_shared)));
      if (fold_here) group_barrier(kConsumersBarrier, kConsumerWarps * 32); // every consumer warp has read its last page
      if (warp == 0 && lane == 0 && pb == lane_pages) { // the lane's last segment: its descriptor, with how this segment is stored
        args.descriptors[2 * l] = sh.segment_base[l];
        args.descriptors[2 * l + 1] = (sh.segment_base[l + 1] - sh.segment_base[l]) | (fold_here ? 0u : 0x80000000u);
      }
      float *out = fold_here ? fold.rows[warp] : args.partials + slot_index * kGroup * kHeadDim;
      float *stats = fold_here ? fold.stats[warp] : args.statistics + slot_index * kGroup * 2;
      const uint32_t row_floats = fold_here ? kFoldRow : kHeadDim;
      const float unscale = 6.103515625e-05f; // 2^-14
      const bool failed = sh.error != 0;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        const uint32_t query_head = 2 * c + j;
        if (query_head >= kGroup) continue;
#pragma unroll
        for (uint32_t t = 0; t < 16; ++t) {
          out[query_head * row_floats + 16 * t + g] = o[t][j] * unscale;
          out[query_head * row_floats + 16 * t + 8 + g] = o[t][2 + j] * unscale;
        }
        if (g == 0) {
          stats[query_head * 2] = failed ? -INFINITY : m[j] * kLn2;
          stats[query_head * 2 + 1] = failed ? 0.0f : l_sum[j];
        }
      }
      if (fold_here) {
        group_barrier(1 + head, kPageWarps * 32);
        const uint64_t slot = (uint64_t(segment) * kKvHeads + head) * kPageWarps;
        fold_and_store(fold, head, residue * 32 + lane, args.partials + slot * kGroup * kHeadDim, args.statistics + slot * kGroup * 2);
      }
    }
  }
}

// ---- merge of one (lane, KV head, query head): its partial slots -> {maximum, denominator, numerator} -------------
// The slots of a (lane, head) are one per segment, in segment order, and the three page residues of the lane's last
// segment when its CTA did not fold them (LaneSlots). The combination is a fixed function of the slot count
// (same grid, same bits): slot s belongs to slot group s mod G; a group folds its slots in rising order with a
// running maximum (an online merge: statistics and partial rows of a batch of slots are loaded together, one round
// trip to L2 per batch instead of one for the statistics and another for the rows); the G group results are then
// merged in group order against their common maximum.
template <uint32_t kGroups> struct ReduceShared {
  float4 sums[kGroups][kHeadDim / 4];
  float group_maximum[kGroups], group_denominator[kGroups];
  float maximum, denominator;
};

// Threads = 64 * kGroups: thread = (slot group, four consecutive dims). Returns the numerator's four dims in the
// threads of group 0 (tid < 64); maximum and denominator in shared memory.
template <uint32_t kGroups>
__device__ __forceinline__ float4 reduce_slots(const float *__restrict__ partials, const float *__restrict__ statistics,
                                               uint2 descriptor, uint32_t head, uint32_t query_head,
                                               ReduceShared<kGroups> &sh) {
  constexpr uint32_t kBatch = 8; // slots a thread has in flight at a time
  const uint32_t tid = threadIdx.x, group = tid >> 6, quad = tid & 63u;
  const LaneSlots lane_slots(descriptor);
  const uint32_t slots = lane_slots.slots;
  auto slot_of = [&](uint32_t t) { return lane_slots.slot(t, head); };
  float running = -INFINITY, denominator = 0.0f;
  float4 numerator = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (uint32_t t = group; t < slots; t += kGroups * kBatch) {
    float2 stat[kBatch];
    float4 part[kBatch];
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) { // every load of the batch is in flight before the first fold
      const uint32_t at = t + k * kGroups;
      const bool live = at < slots;
      const uint64_t slot = live ? slot_of(at) : 0;
      stat[k] = live ? __ldcg(reinterpret_cast<const float2 *>(statistics + (slot * kGroup + query_head) * 2)) : make_float2(-INFINITY, 0.0f);
      part[k] = live ? __ldcg(reinterpret_cast<const float4 *>(partials + (slot * kGroup + query_head) * kHeadDim) + quad)
                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) {
      if (stat[k].x == -INFINITY) continue; // an empty partial (or past the last slot) weighs nothing
      if (stat[k].x > running) {
        const float scale = expf(running - stat[k].x); // 0 for the first slot
        numerator.x *= scale; numerator.y *= scale; numerator.z *= scale; numerator.w *= scale;
        denominator *= scale;
        running = stat[k].x;
      }
      const float weight = expf(stat[k].x - running);
      numerator.x += weight * part[k].x; numerator.y += weight * part[k].y;
      numerator.z += weight * part[k].z; numerator.w += weight * part[k].w;
      denominator += weight * stat[k].y;
    }
  }
  sh.sums[group][quad] = numerator;
  if (quad == 0) { sh.group_maximum[group] = running; sh.group_denominator[group] = denominator; }
  __syncthreads();
  float maximum = sh.group_maximum[0];
#pragma unroll
  for (uint32_t g = 1; g < kGroups; ++g) maximum = fmaxf(maximum, sh.group_maximum[g]);
  float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float total_denominator = 0.0f;
  if (tid < 64) {
#pragma unroll
    for (uint32_t g = 0; g < kGroups; ++g) {
      const float own = sh.group_maximum[g];
      const float weight = own == -INFINITY ? 0.0f : expf(own - maximum);
      const float4 other = sh.sums[g][quad];
      total.x += weight * other.x; total.y += weight * other.y; total.z += weight * other.z; total.w += weight * other.w;
      total_denominator += weight * sh.group_denominator[g];
    }
    if (tid == 0) { sh.maximum = maximum; sh.denominator = total_denominator; }
  }
  __syncthreads();
  return total;
}

__device__ __forceinline__ void store_output_quad(uint16_t *output, float *output_f32, uint64_t at, float4 value) {
  const uint32_t low = uint32_t(float_to_bf16_bits(value.x)) | (uint32_t(float_to_bf16_bits(value.y)) << 16);
  const uint32_t high = uint32_t(float_to_bf16_bits(value.z)) | (uint32_t(float_to_bf16_bits(value.w)) << 16);
  *reinterpret_cast<uint2 *>(output + at) = make_uint2(low, high);
  if (output_f32) *reinterpret_cast<float4 *>(output_f32 + at) = value;
}

// Merge one query head's partials and store bf16 (and optionally fp32), or leave the shard triple of a sequence
// split. grid (group, kv_heads, lanes), 64 * kGroups threads.
template <uint32_t kGroups>
__global__ void __launch_bounds__(64 * kGroups)
decode_reduce_kernel(const float *__restrict__ partials, const float *__restrict__ statistics,
                     const uint32_t *__restrict__ descriptors, uint16_t *__restrict__ output,
                     float *__restrict__ output_f32, const rk_verify_params *__restrict__ lane_params,
                     rk_kv_layer layer, float *__restrict__ shard_out) {
  __shared__ ReduceShared<kGroups> sh;
  const uint32_t query_head = blockIdx.x, head = blockIdx.y, l = blockIdx.z, tid = threadIdx.x;
  dependents_may_launch(); // the next kernel of the stream may take its place; it waits for this grid's writes
  dependency_wait();       // partials, statistics and descriptors come from the decode kernel launched just before
  const uint2 descriptor = __ldcg(reinterpret_cast<const uint2 *>(descriptors + 2 * l)); // in flight beside the parameters
  rk_verify_params p = lane_params[l];
  p.kv = layer;
  if (!rk_verify_contract_valid(&p) || p.active_rows != 1 || p.row_capacity != 1) return;
  const float4 numerator = reduce_slots<kGroups>(partials, statistics, descriptor, head, query_head, sh);
  const float denominator = sh.denominator;
  if (shard_out) { // this rank's piece of a sequence split: {max, sum, un-normalised output} per query head
    float *triple = shard_out + ((uint64_t(l) * kKvHeads + head) * kGroup + query_head) * (kHeadDim + 2);
    if (tid == 0) { triple[0] = sh.maximum; triple[1] = denominator; }
    if (tid < 64) { // triples are 8-byte aligned (258 floats each): two 8-byte stores
      *reinterpret_cast<float2 *>(triple + 2 + 4 * tid) = make_float2(numerator.x, numerator.y);
      *reinterpret_cast<float2 *>(triple + 4 + 4 * tid) = make_float2(numerator.z, numerator.w);
    }
    return;
  }
  if (tid < 64) {
    const uint64_t tile = ((uint64_t(l) * kKvHeads + head) * RK_VERIFY_CHUNK_STRIDE) * kGroup * kHeadDim;
    const float4 value = denominator > 0.0f ? make_float4(numerator.x / denominator, numerator.y / denominator,
                                                          numerator.z / denominator, numerator.w / denominator)
                                            : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    store_output_quad(output, output_f32, tile + query_head * kHeadDim + 4 * tid, value);
  }
}

// The merge for batches of many lanes: one block per (lane, KV head), 384 threads = (query head of the group, four
// consecutive dims). A thread folds every slot of its (lane, head, query head) in rising order with a running maximum,
// statistics and partial rows of a batch of slots in flight together: two round trips to L2 for a lane that spans
// up to four CTAs, no shared memory, no barrier, and few enough blocks (4 x lanes) to run in one wave.
constexpr uint32_t kRowMergeThreads = kGroup * (kHeadDim / 4);
__global__ void __launch_bounds__(kRowMergeThreads)
decode_reduce_rows_kernel(const float *__restrict__ partials, const float *__restrict__ statistics,
                          const uint32_t *__restrict__ descriptors, uint16_t *__restrict__ output,
                          float *__restrict__ output_f32, const rk_verify_params *__restrict__ lane_params, rk_kv_layer layer) {
  constexpr uint32_t kBatch = 12; // four CTAs' worth of slots in one round trip
  const uint32_t head = blockIdx.x, l = blockIdx.y, tid = threadIdx.x, query_head = tid >> 6, quad = tid & 63u;
  dependents_may_launch(); // the next kernel of the stream may take its place; it waits for this grid's writes
  dependency_wait();       // partials, statistics and descriptors come from the decode kernel launched just before
  const uint2 descriptor = __ldcg(reinterpret_cast<const uint2 *>(descriptors + 2 * l)); // in flight beside the parameters
  rk_verify_params p = lane_params[l];
  p.kv = layer;
  if (!rk_verify_contract_valid(&p) || p.active_rows != 1 || p.row_capacity != 1) return;
  const LaneSlots lane_slots(descriptor);
  const uint32_t slots = lane_slots.slots;
  auto slot_of = [&](uint32_t t) { return lane_slots.slot(t, head); };
  float running = -INFINITY, denominator = 0.0f;
  float4 numerator = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (uint32_t t = 0; t < slots; t += kBatch) {
    float2 stat[kBatch];
    float4 part[kBatch];
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) { // every load of the batch is in flight before the first fold
      const bool live = t + k < slots;
      const uint64_t slot = live ? slot_of(t + k) : 0;
      stat[k] = live ? __ldcg(reinterpret_cast<const float2 *>(statistics + (slot * kGroup + query_head) * 2)) : make_float2(-INFINITY, 0.0f);
      part[k] = live ? __ldcg(reinterpret_cast<const float4 *>(partials + (slot * kGroup + query_head) * kHeadDim) + quad)
                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) {
      if (stat[k].x == -INFINITY) continue; // an empty partial (or past the last slot) weighs nothing
      if (stat[k].x > running) {
        const float scale = expf(running - stat[k].x); // 0 for the first slot
        numerator.x *= scale; numerator.y *= scale; numerator.z *= scale; numerator.w *= scale;
        denominator *= scale;
        running = stat[k].x;
      }
      const float weight = expf(stat[k].x - running);
      numerator.x += weight * part[k].x; numerator.y += weight * part[k].y;
      numerator.z += weight * part[k].z; numerator.w += weight * part[k].w;
      denominator += weight * stat[k].y;
    }
  }
  const float4 value = denominator > 0.0f ? make_float4(numerator.x / denominator, numerator.y / denominator,
                                                        numerator.z / denominator, numerator.w / denominator)
                                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  const uint64_t tile = ((uint64_t(l) * kKvHeads + head) * RK_VERIFY_CHUNK_STRIDE) * kGroup * kHeadDim;
  store_output_quad(output, output_f32, tile + query_head * kHeadDim + 4 * quad, value);
}

// ---- sequence split without a library collective: reduce -> peer stores -> flags -> rank-order merge, one kernel ----
// Every rank owns one exchange buffer that its peers can address (CUDA IPC mappings): slots
// [parity][source rank][lane][query head]{max, sum, D numerators} and flags [parity][source rank][lane][query head].
// A block (query head, KV head, lane) reduces its own partials, writes its triple into slot [parity][my rank] of
// EVERY rank's buffer with plain stores (NVLink for the peers), publishes it with one system-scope release per rank,
// then waits (bounded) until every source rank's flag in ITS OWN buffer carries this step's epoch and merges the
// sources in rank order (paged_attention_tile.h:362-404 with "split" = rank), so all ranks end with identical bits.
// Parity = epoch & 1: a rank can only reach step k+2 after every rank published step k+1, which each rank does
// after its own merge of step k, so a slot is never overwritten while someone still reads it. Only this kernel
// touches peer memory; no TMA and no multicast is involved.
constexpr uint32_t kMaxRanks = 8;
constexpr uint32_t kTripleFloats = kHeadDim + 2;
struct ExchangeArgs {
  float *slots[kMaxRanks];    // every rank's slot area (own entry = local memory)
  uint32_t *flags[kMaxRanks]; // every rank's flag area
  uint32_t rank, ranks, lanes, epoch, spin_limit;
  uint32_t post_only;         // single-GPU emulation of the earlier ranks: publish, do not wait or merge
  uint32_t *status;
};

__device__ __forceinline__ void store_release_system(uint32_t *address, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t *address) {
  uint32_t value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}

template <uint32_t kGroups>
__global__ void __launch_bounds__(64 * kGroups)
shard_exchange_kernel(const float *__restrict__ partials, const float *__restrict__ statistics,
                      const uint32_t *__restrict__ descriptors, uint16_t *__restrict__ output,
                      float *__restrict__ output_f32, const rk_verify_params *__restrict__ lane_params,
                      rk_kv_layer layer, ExchangeArgs ex) {
  __shared__ ReduceShared<kGroups> sh;
  __shared__ uint32_t arrived;
  const uint32_t query_head = blockIdx.x, head = blockIdx.y, l = blockIdx.z, tid = threadIdx.x;
  dependents_may_launch();
  dependency_wait();
  const uint2 descriptor = __ldcg(reinterpret_cast<const uint2 *>(descriptors + 2 * l)); // in flight beside the parameters
  rk_verify_params p = lane_params[l];
  p.kv = layer;
  // a lane this rank holds no pages of (an empty shard, or an invalid lane) still publishes an empty triple
  const bool valid = rk_verify_contract_valid(&p) && p.active_rows == 1 && p.row_capacity == 1;
  float4 numerator = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float maximum = -INFINITY, denominator = 0.0f;
  if (valid) {
    numerator = reduce_slots<kGroups>(partials, statistics, descriptor, head, query_head, sh);
    maximum = sh.maximum;
    denominator = sh.denominator;
  }
  const uint32_t parity = ex.epoch & 1u, fused_head = head * kGroup + query_head;
  const uint64_t cell = uint64_t(l) * (kKvHeads * kGroup) + fused_head;                     // (lane, query head)
  const uint64_t cells = uint64_t(ex.lanes) * (kKvHeads * kGroup);
  const uint64_t mine = (uint64_t(parity) * ex.ranks + ex.rank) * cells + cell;               // where my triple goes, in every buffer
  for (uint32_t r = 0; r < ex.ranks; ++r) {
    float *triple = ex.slots[r] + mine * kTripleFloats;
    if (tid == 0) *reinterpret_cast<float2 *>(triple) = make_float2(maximum, denominator);
    if (tid < 64) {
      *reinterpret_cast<float2 *>(triple + 2 + 4 * tid) = make_float2(numerator.x, numerator.y);
      *reinterpret_cast<float2 *>(triple + 4 + 4 * tid) = make_float2(numerator.z, numerator.w);
    }
  }
  __syncthreads(); // every thread's stores are ordered before the fences and releases below
  if (tid < ex.ranks) {
    __threadfence_system();
    store_release_system(ex.flags[tid] + mine, ex.epoch);
  }
  if (ex.post_only) return;
  // wait for every source rank's triple of this step in my own buffer
  if (tid == 0) arrived = 1;
  __syncthreads();
  if (tid < ex.ranks) {
    const uint32_t *flag = ex.flags[ex.rank] + (uint64_t(parity) * ex.ranks + tid) * cells + cell;
    bool seen = false;
    for (uint32_t i = 0; i < ex.spin_limit; ++i) {
      if (load_acquire_system(flag) == ex.epoch) { seen = true; break; }
      if (i > 64) __nanosleep(64);
    }
    if (!seen) { arrived = 0; atomicExch(ex.status, 3u); }
  }
  __syncthreads();
  if (tid >= 64) return;
  float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float total_denominator = 0.0f;
  if (arrived) {
    const float *local = ex.slots[ex.rank] + (uint64_t(parity) * ex.ranks * cells + cell) * kTripleFloats;
    const uint64_t stride = cells * kTripleFloats;
    float all_maximum = -INFINITY;
    for (uint32_t r = 0; r < ex.ranks; ++r) all_maximum = fmaxf(all_maximum, __ldcg(local + r * stride));
    for (uint32_t r = 0; r < ex.ranks; ++r) {
      const float2 stat = __ldcg(reinterpret_cast<const float2 *>(local + r * stride));
      const float weight = stat.x == -INFINITY ? 0.0f : expf(stat.x - all_maximum);
      const float2 a = __ldcg(reinterpret_cast<const float2 *>(local + r * stride + 2 + 4 * tid));
      const float2 b = __ldcg(reinterpret_cast<const float2 *>(local + r * stride + 4 + 4 * tid));
      total.x += weight * a.x; total.y += weight * a.y; total.z += weight * b.x; total.w += weight * b.y;
      total_denominator += weight * stat.y;
    }
  }
  const float4 value = total_denominator > 0.0f ? make_float4(total.x / total_denominator, total.y / total_denominator,
                                                              total.z / total_denominator, total.w / total_denominator)
                                                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  const uint64_t tile = ((uint64_t(l) * kKvHeads + head) * RK_VERIFY_CHUNK_STRIDE) * kGroup * kHeadDim;
  store_output_quad(output, output_f32, tile + query_head * kHeadDim + 4 * tid, value);
}

// Combine the shards of a sequence split: shard r holds {max, sum, un-normalised output} per
// (lane, query head); the merge of the split kernel (paged_attention_tile.h:362-404) with
// "split" = rank, in rank order, so every rank computes identical bits.
// grid (query_heads, lanes), 256 threads.
__global__ void __launch_bounds__(256)
merge_shards_kernel(const float *__restrict__ triples, uint32_t shards, uint32_t lanes, uint16_t *__restrict__ output,
                    float *__restrict__ output_f32) {
  const uint32_t query_head = blockIdx.x, l = blockIdx.y, tid = threadIdx.x;
  constexpr uint32_t kQueryHeads = kKvHeads * kGroup, kTriple = kHeadDim + 2;
  const uint64_t stride = uint64_t(lanes) * kQueryHeads * kTriple;
  const float *mine = triples + (uint64_t(l) * kQueryHeads + query_head) * kTriple;
  float maximum = -INFINITY;
  for (uint32_t r = 0; r < shards; ++r) maximum = fmaxf(maximum, mine[r * stride]);
  float numerator = 0.0f, denominator = 0.0f;
  for (uint32_t r = 0; r < shards; ++r) {
    const float own = mine[r * stride];
    const float weight = own == -INFINITY ? 0.0f : expf(own - maximum);
    numerator += weight * mine[r * stride + 2 + tid];
    denominator += weight * mine[r * stride + 1];
  }
  const float value = denominator > 0.0f ? numerator / denominator : 0.0f;
  const uint32_t head = query_head / kGroup, g = query_head % kGroup;
  const uint64_t at = ((uint64_t(l) * kKvHeads + head) * RK_VERIFY_CHUNK_STRIDE) * kGroup * kHeadDim + g * kHeadDim + tid;
  output[at] = float_to_bf16_bits(value);
  if (output_f32) output_f32[at] = value;
}

constexpr size_t kDecodeSharedBytes = 1024 + kStages * kStageBytes + sizeof(Shared);
constexpr size_t kByteDecodeSharedBytes = 1024 + kByteStages * kByteStageBytes + sizeof(Shared);
constexpr size_t kWideDecodeSharedBytes = 1024 + kWideStages * kWideStageBytes + sizeof(Shared);
static_assert(kByteDecodeSharedBytes <= 227 * 1024, "the byte-format ring fits one SM");
static_assert(kWideDecodeSharedBytes <= 227 * 1024, "the bf16 ring fits one SM");

// The kernel's dynamic shared-memory limit is a per-device function attribute.
int configure_decode_kernel() {
  static std::atomic<bool> configured[64] = {}; // setting the attribute twice is harmless: two threads may race here
  int device = 0;
  if (int st = cuda_status(cudaGetDevice(&device), "cudaGetDevice")) return st;
  if (device < 0 || device >= 64) { set_error("device index out of range"); return kInvalid; }
  if (!configured[device].load(std::memory_order_acquire)) {
    if (int st = cuda_status(cudaFuncSetAttribute(decode_int4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kDecodeSharedBytes)), "decode shared memory")) return st;
    if (int st = cuda_status(cudaFuncSetAttribute(decode_bytes_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kByteDecodeSharedBytes)), "decode shared memory")) return st;
    if (int st = cuda_status(cudaFuncSetAttribute(decode_bytes_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kByteDecodeSharedBytes)), "decode shared memory")) return st;
    if (int st = cuda_status(cudaFuncSetAttribute(decode_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kWideDecodeSharedBytes)), "decode shared memory")) return st;
    configured[device].store(true, std::memory_order_release);
  }
  return kOk;
}

} // namespace
} // namespace rk

using namespace rk;

// The merge follows its decode kernel as a programmatic dependent launch: its blocks are placed while the decode
// grid drains and start the moment that grid's writes are visible.
// The merge of few lanes runs in ONE wave: a block per (lane, query head) with sixteen slot groups (1 024 threads,
// one block per SM) while the blocks do not outnumber the SMs, eight groups (512 threads, two blocks per SM) up to
// twice that; beyond, the row merge (or four groups for the shards of a sequence split).
static uint32_t merge_groups(uint32_t lanes) {
  const uint32_t blocks = lanes * kKvHeads * kGroup;
  return blocks <= 148 ? 16 : blocks <= 2 * 148 ? 8 : 4;
}

template <typename Kernel, typename... Args>
static int launch_dependent(Kernel kernel, dim3 grid, uint32_t threads, cudaStream_t stream, const char *what, Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = dim3(threads);
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&config, kernel, args...), what);
}

static int launch_merge(uint32_t lanes, cudaStream_t stream, const float *partials, const float *statistics,
                        const uint32_t *descriptors, uint16_t *output, float *output_f32,
                        const rk_verify_params *lane_params, rk_kv_layer layer, float *triples) {
  const dim3 grid(kGroup, kKvHeads, lanes);
  const uint32_t groups = merge_groups(lanes);
  if (groups == 16)
    return launch_dependent(decode_reduce_kernel<16>, grid, 1024, stream, "decode reduce launch", partials, statistics, descriptors,
                            output, output_f32, lane_params, layer, triples);
  if (groups == 8)
    return launch_dependent(decode_reduce_kernel<8>, grid, 512, stream, "decode reduce launch", partials, statistics, descriptors,
                            output, output_f32, lane_params, layer, triples);
  if (!triples)
    return launch_dependent(decode_reduce_rows_kernel, dim3(kKvHeads, lanes), kRowMergeThreads, stream, "decode reduce launch", partials,
                            statistics, descriptors, output, output_f32, lane_params, layer);
  return launch_dependent(decode_reduce_kernel<4>, grid, 256, stream, "decode reduce launch", partials, statistics, descriptors,
                          output, output_f32, lane_params, layer, triples);
}

static int launch_exchange(uint32_t lanes, cudaStream_t stream, const float *partials, const float *statistics,
                           const uint32_t *descriptors, uint16_t *output, float *output_f32,
                           const rk_verify_params *lane_params, rk_kv_layer layer, const ExchangeArgs &exchange) {
  const dim3 grid(kGroup, kKvHeads, lanes);
  const uint32_t groups = merge_groups(lanes);
  if (groups == 16)
    return launch_dependent(shard_exchange_kernel<16>, grid, 1024, stream, "shard exchange launch", partials, statistics, descriptors,
                            output, output_f32, lane_params, layer, exchange);
  if (groups == 8)
    return launch_dependent(shard_exchange_kernel<8>, grid, 512, stream, "shard exchange launch", partials, statistics, descriptors,
                            output, output_f32, lane_params, layer, exchange);
  return launch_dependent(shard_exchange_kernel<4>, grid, 256, stream, "shard exchange launch", partials, statistics, descriptors,
                          output, output_f32, lane_params, layer, exchange);
}

// The streaming kernel of a format on `ctas` CTAs.
// Launched as a programmatic dependent of whatever precedes it on the stream: its CTAs may be placed while that
// kernel drains (the kernel waits for its predecessor's writes before it reads anything).
static int launch_decode(uint32_t format, uint32_t ctas, cudaStream_t s, const Window *w, const DecodeArgs &args) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(ctas);
  config.blockDim = dim3(kThreads);
  config.stream = s;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  cudaError_t error;
  if (format == RK_FORMAT_INT4) { config.dynamicSmemBytes = kDecodeSharedBytes; error = cudaLaunchKernelEx(&config, decode_int4_kernel, w->int4_map, args); }
  else if (format == RK_FORMAT_INT8) { config.dynamicSmemBytes = kByteDecodeSharedBytes; error = cudaLaunchKernelEx(&config, decode_bytes_kernel<false>, w->int4_map, args); }
  else if (format == RK_FORMAT_FP8E4M3) { config.dynamicSmemBytes = kByteDecodeSharedBytes; error = cudaLaunchKernelEx(&config, decode_bytes_kernel<true>, w->int4_map, args); }
  else { config.dynamicSmemBytes = kWideDecodeSharedBytes; error = cudaLaunchKernelEx(&config, decode_bf16_kernel, w->int4_map, args); }
  return cuda_status(error, "decode launch");
}

extern "C" {

// Sizes the scratch of a decode step: `ctas` = 0 takes one CTA per SM of the current device.
int rk_decode_plan_make(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                        uint32_t lanes, uint32_t ctas, rk_decode_plan *plan) {
  if (!plan || !lanes || lanes > kMaxLanes) { set_error("rk_decode_plan_make: lanes out of range"); return kInvalid; }
  if (format < RK_FORMAT_INT8 || format > RK_FORMAT_FP8E4M3 || kv_heads != kKvHeads ||
      query_heads != kKvHeads * kGroup || head_dim != kHeadDim) {
    set_error("rk_decode_plan_make: the streaming decode kernels are built for 4 KV heads x 24 query heads x 256");
    return kUnsupported;
  }
  if (!ctas) {
    int device = 0, sms = 0;
    if (int s = cuda_status(cudaGetDevice(&device), "cudaGetDevice")) return s;
    if (int s = cuda_status(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "SM count")) return s;
    ctas = uint32_t(sms);
  }
  plan->lanes = lanes;
  plan->ctas = ctas;
  plan->max_segments = lanes + ctas;
  plan->reserved = 0;
  const uint64_t slots = uint64_t(plan->max_segments) * kKvHeads * kPageWarps;
  plan->partials_bytes = slots * kGroup * kHeadDim * sizeof(float);
  plan->statistics_bytes = slots * kGroup * 2 * sizeof(float);
  plan->descriptor_bytes = (2ull * lanes + 4) * sizeof(uint32_t);
  return kOk;
}

// The device address window every page of a pool lies in (rk_storage_window).
void *rk_window_create(uint64_t base, uint64_t bytes) {
  if (!base || (base & 1023u) || !bytes || (bytes >> 7) > 0x7fffffffull) {
    set_error("rk_window_create: the window must be 1 KiB-aligned and span less than 256 GiB");
    return nullptr;
  }
  auto *w = new Window;
  w->base = base;
  w->bytes = bytes;
  if (encode_window_map(&w->int4_map, base, bytes >> 7, kTensorBytes / 128) ||
      encode_window_map(&w->int4_head_map, base, bytes >> 7, kSlabBytes / 128) ||
      encode_window_map(&w->byte_head_map, base, bytes >> 7, 2 * kSlabBytes / 128)) {
    delete w;
    return nullptr;
  }
  return w;
}
void rk_window_destroy(void *window) { delete static_cast<Window *>(window); }

int rk_attention_decode(const void *window, const rk_decode_plan *plan, uint32_t format, const void *queries,
                        void *output, float *output_f32, float *partials, float *statistics, uint32_t *descriptors,
                        const rk_page_entry *const *tables, const rk_verify_params *lane_params, rk_kv_layer layer,
                        void *stream) {
  const auto *w = static_cast<const Window *>(window);
  if (!w || !plan || !queries || !output || !partials || !statistics || !descriptors || !tables || !lane_params ||
      !layer.extent_pages || format < RK_FORMAT_INT8 || format > RK_FORMAT_FP8E4M3) {
    set_error("rk_attention_decode: invalid arguments");
    return kInvalid;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int st = configure_decode_kernel()) return st;
  DecodeArgs args{static_cast<const uint16_t *>(queries), partials, statistics, descriptors, tables, lane_params, layer, w->base, plan->lanes,
                  descriptors + 2 * plan->lanes, kSpinLimit, 0};
  if (int st = launch_decode(format, plan->ctas, s, w, args)) return st;
  return launch_merge(plan->lanes, s, partials, statistics, descriptors, static_cast<uint16_t *>(output), output_f32, lane_params, layer, nullptr);
}

// One rank's part of a sequence-split decode: attention over the pages this rank holds, left as
// {max, sum, un-normalised output} per (lane, query head) in `triples`
// ([lane][query_head][2 + D] fp32, 24 768 bytes per lane at 24 x 256) for an all-gather.
int rk_attention_decode_shard(const void *window, const rk_decode_plan *plan, uint32_t format, const void *queries,
                              float *triples, float *partials, float *statistics, uint32_t *descriptors,
                              const rk_page_entry *const *tables, const rk_verify_params *lane_params,
                              rk_kv_layer layer, void *stream) {
  const auto *w = static_cast<const Window *>(window);
  if (!w || !plan || !queries || !triples || !partials || !statistics || !descriptors || !tables || !lane_params ||
      !layer.extent_pages || format < RK_FORMAT_INT8 || format > RK_FORMAT_FP8E4M3) {
    set_error("rk_attention_decode_shard: invalid arguments");
    return kInvalid;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int st = configure_decode_kernel()) return st;
  DecodeArgs args{static_cast<const uint16_t *>(queries), partials, statistics, descriptors, tables, lane_params, layer, w->base, plan->lanes,
                  descriptors + 2 * plan->lanes, kSpinLimit, 0};
  if (int st = launch_decode(format, plan->ctas, s, w, args)) return st;
  return launch_merge(plan->lanes, s, partials, statistics, descriptors, nullptr, nullptr, lane_params, layer, triples);
}

// Merges `shards` gathered triples ([shard][lane][query_head][2 + D]) in shard order into the bf16
// output [lane][kv_head][32][group][D] (row 0) and optionally the fp32 value before rounding.
int rk_attention_merge_shards(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes, uint32_t shards,
                              const float *triples, void *output, float *output_f32, void *stream) {
  if (kv_heads != kKvHeads || query_heads != kKvHeads * kGroup || head_dim != kHeadDim) return kUnsupported;
  if (!lanes || !shards || !triples || !output) { set_error("rk_attention_merge_shards: invalid arguments"); return kInvalid; }
  merge_shards_kernel<<<dim3(query_heads, lanes), 256, 0, static_cast<cudaStream_t>(stream)>>>(triples, shards, lanes, static_cast<uint16_t *>(output), output_f32);
  return cuda_status(cudaGetLastError(), "merge shards launch");
}

// ---- sequence split over peer memory ------------------------------------------------------------------------------
// One rank's exchange buffer and its view of the peers' buffers (see shard_exchange_kernel).
struct Exchange {
  uint32_t rank = 0, ranks = 1, lanes = 1, epoch = 0;
  unsigned char *local = nullptr;
  size_t slot_bytes = 0, flag_bytes = 0;
  unsigned char *mapped[kMaxRanks] = {}; // peers' buffers as this process sees them (own entry = local)
  bool opened[kMaxRanks] = {};
};

void *rk_exchange_create(uint32_t rank, uint32_t ranks, uint32_t lanes, void *handle_out) {
  if (!ranks || ranks > kMaxRanks || rank >= ranks || !lanes || lanes > kMaxLanes) {
    set_error("rk_exchange_create: ranks 1..8, rank < ranks, lanes 1..1024");
    return nullptr;
  }
  auto *ex = new Exchange;
  ex->rank = rank; ex->ranks = ranks; ex->lanes = lanes;
  const size_t cells = size_t(2) * ranks * lanes * kKvHeads * kGroup;
  ex->slot_bytes = (cells * kTripleFloats * sizeof(float) + 255) / 256 * 256;
  ex->flag_bytes = (cells * sizeof(uint32_t) + 255) / 256 * 256;
  void *memory = nullptr;
  if (cuda_status(cudaMalloc(&memory, ex->slot_bytes + ex->flag_bytes), "exchange buffer") ||
      cuda_status(cudaMemset(memory, 0, ex->slot_bytes + ex->flag_bytes), "exchange buffer clear")) {
    if (memory) cudaFree(memory);
    delete ex;
    return nullptr;
  }
  ex->local = static_cast<unsigned char *>(memory);
  for (uint32_t r = 0; r < ranks; ++r) ex->mapped[r] = ex->local; // until connected: every "peer" is this buffer
  if (handle_out) {
    cudaIpcMemHandle_t handle;
    if (cuda_status(cudaIpcGetMemHandle(&handle, memory), "cudaIpcGetMemHandle")) {
      cudaFree(memory);
      delete ex;
      return nullptr;
    }
    static_assert(sizeof(handle) == 64, "the handle travels as 64 bytes");
    memcpy(handle_out, &handle, sizeof(handle));
  }
  return ex;
}

// `handles`: ranks x 64 bytes, rank r's from its rk_exchange_create (gathered by the caller, e.g. over
// torch.distributed). Maps every peer's buffer into this process.
int rk_exchange_connect(void *exchange, const void *handles) {
  auto *ex = static_cast<Exchange *>(exchange);
  if (!ex || !handles) { set_error("rk_exchange_connect: invalid arguments"); return kInvalid; }
  for (uint32_t r = 0; r < ex->ranks; ++r) {
    if (r == ex->rank || ex->opened[r]) continue;
    cudaIpcMemHandle_t handle;
    memcpy(&handle, static_cast<const unsigned char *>(handles) + size_t(r) * sizeof(handle), sizeof(handle));
    void *peer = nullptr;
    if (int st = cuda_status(cudaIpcOpenMemHandle(&peer, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return st;
    ex->mapped[r] = static_cast<unsigned char *>(peer);
    ex->opened[r] = true;
  }
  return kOk;
}

void rk_exchange_destroy(void *exchange) {
  auto *ex = static_cast<Exchange *>(exchange);
  if (!ex) return;
  for (uint32_t r = 0; r < ex->ranks; ++r)
    if (ex->opened[r]) cudaIpcCloseMemHandle(ex->mapped[r]);
  if (ex->local) cudaFree(ex->local);
  delete ex;
}

// One rank's whole sequence-split decode step in two launches: the streaming decode kernel over the pages this
// rank holds, then shard_exchange_kernel (reduce -> peer stores -> flags -> rank-order merge). Every rank calls it
// once per step, in the same order; `output` ends identical on all ranks. loopback_rank < 0 in production. With
// loopback_rank >= 0 (an unconnected exchange on ONE GPU) the call acts as that rank of an emulated step: ranks
// 0 .. ranks-2 only publish, the call for the last rank waits (its flags are already there) and merges.
// A wait for a peer that runs out raises the decode status word (rk_attention_decode_status) and writes zeros.
// The step's epoch is a launch argument: do not replay these launches from a captured graph.
int rk_attention_decode_exchange(const void *window, const rk_decode_plan *plan, uint32_t format, const void *queries,
                                 void *output, float *output_f32, float *partials, float *statistics, uint32_t *descriptors,
                                 const rk_page_entry *const *tables, const rk_verify_params *lane_params, rk_kv_layer layer,
                                 void *exchange, int32_t loopback_rank, void *stream) {
  const auto *w = static_cast<const Window *>(window);
  auto *ex = static_cast<Exchange *>(exchange);
  if (!w || !plan || !ex || !queries || !output || !partials || !statistics || !descriptors || !tables || !lane_params ||
      !layer.extent_pages || format < RK_FORMAT_INT8 || format > RK_FORMAT_FP8E4M3 || plan->lanes != ex->lanes ||
      loopback_rank >= int32_t(ex->ranks)) {
    set_error("rk_attention_decode_exchange: invalid arguments");
    return kInvalid;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int st = configure_decode_kernel()) return st;
  DecodeArgs args{static_cast<const uint16_t *>(queries), partials, statistics, descriptors, tables, lane_params, layer, w->base, plan->lanes,
                  descriptors + 2 * plan->lanes, kSpinLimit, 0};
  if (int st = launch_decode(format, plan->ctas, s, w, args)) return st;
  ExchangeArgs e{};
  for (uint32_t r = 0; r < ex->ranks; ++r) {
    e.slots[r] = reinterpret_cast<float *>(ex->mapped[r]);
    e.flags[r] = reinterpret_cast<uint32_t *>(ex->mapped[r] + ex->slot_bytes);
  }
  e.rank = loopback_rank >= 0 ? uint32_t(loopback_rank) : ex->rank;
  if (loopback_rank <= 0) ++ex->epoch; // a new step (in an emulated step: when its rank 0 runs)
  e.ranks = ex->ranks;
  e.lanes = ex->lanes;
  e.epoch = ex->epoch;
  e.spin_limit = 1u << 22; // polls of ~0.1-0.3 us: a peer may lag by about a second before the wait gives up
  e.post_only = loopback_rank >= 0 && uint32_t(loopback_rank) + 1 != ex->ranks;
  e.status = descriptors + 2 * plan->lanes;
  return launch_exchange(plan->lanes, s, partials, statistics, descriptors, static_cast<uint16_t *>(output), output_f32, lane_params, layer, e);
}

// ---- decode attention without any allocation -----------------------------------------------------
// Scratch of the no-allocation entry point: partial outputs, their statistics and the lane
// descriptors of one step of at most kStaticLanes lanes on a kStaticCtas-wide grid. The array is
// part of the library image, so every GPU that loads the library holds these bytes until exit.
constexpr uint32_t kStaticLanes = 16, kStaticCtas = 148;
constexpr size_t kStaticSlots = size_t(kStaticLanes + kStaticCtas) * kKvHeads * kPageWarps;
constexpr size_t kStaticPartialBytes = kStaticSlots * kGroup * kHeadDim * sizeof(float);
constexpr size_t kStaticStatisticBytes = (kStaticSlots * kGroup * 2 * sizeof(float) + 255) / 256 * 256;
constexpr size_t kStaticDescriptorBytes = ((2 * kStaticLanes + 4) * sizeof(uint32_t) + 255) / 256 * 256;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticPartialBytes + kStaticStatisticBytes + kStaticDescriptorBytes];

// The device address of g_decode_scratch on the current device. In host code the array's name is only a handle
// for the runtime, never an address a kernel may use: the address comes from cudaGetSymbolAddress, once per device,
// with that device current. Two host threads may both do the first lookup; both get the same address.
static int static_scratch(unsigned char **base) {
  static std::atomic<unsigned char *> scratch_address[64] = {};
  int device = 0;
  if (int st = cuda_status(cudaGetDevice(&device), "cudaGetDevice")) return st;
  if (device < 0 || device >= 64) { set_error("device index out of range"); return kInvalid; }
  unsigned char *known = scratch_address[device].load(std::memory_order_acquire);
  if (!known) {
    void *address = nullptr;
    if (int st = cuda_status(cudaGetSymbolAddress(&address, g_decode_scratch), "cudaGetSymbolAddress(decode scratch)")) return st;
    if (int st = configure_decode_kernel()) return st;
    known = static_cast<unsigned char *>(address);
    scratch_address[device].store(known, std::memory_order_release);
  }
  *base = known;
  return kOk;
}
static uint32_t *static_descriptors(unsigned char *base) {
  return reinterpret_cast<uint32_t *>(base + kStaticPartialBytes + kStaticStatisticBytes);
}

// rk_attention_decode for callers that must not allocate device memory: an engine that gave the
// whole device to its KV pool and has no allocator left to ask, a serving thread that may not
// enter cudaMalloc because it can stall on a device-wide lock, a caller inside a region where
// allocation calls are simply not permitted. The caller still passes queries, tables, lane
// parameters and the output; the step's scratch lives in g_decode_scratch (about 12 MiB) and
// that caps the step at kStaticLanes (16) lanes — more lanes are refused with an error text.
//
// The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
// device current) and sets the kernel's shared-memory attribute; make that first call before any
// stream capture begins. No call allocates or frees anything, on the device or through a library.
// Every call on a device uses the same array: every partial the merge reads is rewritten by the
// same call, the status word (fixed place, after the descriptors of 16 lanes) is sticky until
// rk_attention_decode_static_status reads it, and two calls that overlap on the GPU (different
// streams, no ordering between them) race on the array.
int rk_attention_decode_static(const void *window, uint32_t format, uint32_t lanes, const void *queries, void *output,
                               float *output_f32, const rk_page_entry *const *tables,
                               const rk_verify_params *lane_params, rk_kv_layer layer, void *stream) {
  const auto *w = static_cast<const Window *>(window);
  if (!w || !queries || !output || !tables || !lane_params || !layer.extent_pages || format < RK_FORMAT_INT8 ||
      format > RK_FORMAT_FP8E4M3 || !lanes) {
    set_error("rk_attention_decode_static: invalid arguments");
    return kInvalid;
  }
  if (lanes > kStaticLanes) {
    set_error("rk_attention_decode_static: at most 16 lanes fit the built-in scratch; use rk_attention_decode with caller scratch");
    return kInvalid;
  }
  unsigned char *base = nullptr;
  if (int st = static_scratch(&base)) return st;
  float *partials = reinterpret_cast<float *>(base);
  float *statistics = reinterpret_cast<float *>(base + kStaticPartialBytes);
  uint32_t *descriptors = static_descriptors(base);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DecodeArgs args{static_cast<const uint16_t *>(queries), partials, statistics, descriptors, tables, lane_params, layer, w->base, lanes,
                  descriptors + 2 * kStaticLanes, kSpinLimit, 0};
  if (int st = launch_decode(format, kStaticCtas, s, w, args)) return st;
  return launch_merge(lanes, s, partials, statistics, descriptors, static_cast<uint16_t *>(output), output_f32, lane_params, layer, nullptr);
}

// Reads AND clears a sticky status word on `stream` (synchronises it): kTimeout when a bounded wait inside a decode
// kernel ran out in any step launched since the last read.
static int read_status_word(uint32_t *word_address, cudaStream_t s) {
  uint32_t word = 0;
  if (int st = cuda_status(cudaMemcpyAsync(&word, word_address, sizeof(word), cudaMemcpyDeviceToHost, s), "decode status read")) return st;
  if (int st = cuda_status(cudaStreamSynchronize(s), "decode status sync")) return st;
  if (!word) return kOk;
  if (int st = cuda_status(cudaMemsetAsync(word_address, 0, sizeof(word), s), "decode status clear")) return st;
  if (int st = cuda_status(cudaStreamSynchronize(s), "decode status sync")) return st;
  set_error(word == 1 ? "a bounded wait in the decode kernel ran out (the producer waiting for a free stage)"
                      : "a bounded wait in the decode kernel ran out (a consumer waiting for a page)");
  return kTimeout;
}

int rk_attention_decode_status(const rk_decode_plan *plan, uint32_t *descriptors, void *stream) {
  if (!plan || !descriptors) { set_error("rk_attention_decode_status: invalid arguments"); return kInvalid; }
  return read_status_word(descriptors + 2 * plan->lanes, static_cast<cudaStream_t>(stream));
}

// The same for rk_attention_decode_static, whose status word lives in the library's own array.
int rk_attention_decode_static_status(void *stream) {
  unsigned char *base = nullptr;
  if (int st = static_scratch(&base)) return st;
  return read_status_word(static_descriptors(base) + 2 * kStaticLanes, static_cast<cudaStream_t>(stream));
}

// Test hook of the timeout path: rk_attention_decode whose waits give up after `spin_limit` polls and whose
// producers never stream the last `withheld_pages` pages of their CTA's range. The consumers of those pages run
// out of polls, the kernel raises its status word, lets copies in flight land and returns; nothing faults and
// nothing waits without a bound. The step's output is invalid by construction.
int rk_attention_decode_probe_timeout(const void *window, const rk_decode_plan *plan, uint32_t format, const void *queries,
                                      void *output, float *partials, float *statistics, uint32_t *descriptors,
                                      const rk_page_entry *const *tables, const rk_verify_params *lane_params,
                                      rk_kv_layer layer, uint32_t spin_limit, uint32_t withheld_pages, void *stream) {
  const auto *w = static_cast<const Window *>(window);
  const bool own_scratch = !partials && !statistics && !descriptors; // probe the no-allocation entry's path
  if (!w || !plan || !queries || !output || (!own_scratch && (!partials || !statistics || !descriptors)) || !tables || !lane_params ||
      !layer.extent_pages || format < RK_FORMAT_INT8 || format > RK_FORMAT_FP8E4M3 || !spin_limit || spin_limit > kSpinLimit ||
      (own_scratch && plan->lanes > kStaticLanes)) {
    set_error("rk_attention_decode_probe_timeout: invalid arguments");
    return kInvalid;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int st = configure_decode_kernel()) return st;
  uint32_t *status = own_scratch ? nullptr : descriptors + 2 * plan->lanes;
  uint32_t ctas = plan->ctas;
  if (own_scratch) {
    unsigned char *base = nullptr;
    if (int st = static_scratch(&base)) return st;
    partials = reinterpret_cast<float *>(base);
    statistics = reinterpret_cast<float *>(base + kStaticPartialBytes);
    descriptors = static_descriptors(base);
    status = descriptors + 2 * kStaticLanes;
    ctas = min(ctas, kStaticCtas);
  }
  DecodeArgs args{static_cast<const uint16_t *>(queries), partials, statistics, descriptors, tables, lane_params, layer, w->base, plan->lanes,
                  status, spin_limit, withheld_pages};
  if (int st = launch_decode(format, ctas, s, w, args)) return st;
  return launch_merge(plan->lanes, s, partials, statistics, descriptors, static_cast<uint16_t *>(output), nullptr, lane_params, layer, nullptr);
}

} // extern "C"
