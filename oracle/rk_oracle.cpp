// rk_oracle.cpp — CPU restatement of the reference's paged-KV algorithms.
//
// TEST INFRASTRUCTURE ONLY: the checker for the CUDA path (parity tests, the
// smoke test, the benchmark's cpu_baseline leg). The product library never
// links or calls it. Parity pinned: the int8 and fp8 quantizers, the bf16 and
// e4m3 conversions and the page layout are checked against the reference's own
// CPU headers compiled in place (oracle/ref_shim.cpp); the int8 / int4 / bf16
// stores, the tree compaction, the attention tile and the merge are checked
// against the reference's own Metal kernel source compiled as C++ and run on
// host threads (oracle/ref_metal_kernels.cpp, tests/test_reference_kernels.py),
// and against the closed-form fixtures of the reference's tests
// (tests/test_oracle_pins.py).
//
// Build: g++ -std=c++20 -O3 -march=native -fopenmp -shared -fPIC (oracle/Makefile).
// -ffast-math must stay off: quantized codes are bit-exact by contract.
#include "rk_oracle.h"

#include <algorithm>
#include <bit>
#include <cmath>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

struct Geometry {
  uint32_t format, kv_heads, head_dim, data_bytes, scale_bytes;
  Geometry(uint32_t f, uint32_t h, uint32_t d)
      : format(f), kv_heads(h), head_dim(d), data_bytes(rk_data_bytes(f, h, d)),
        scale_bytes(rk_scale_bytes(f, h)) {}
  bool quantized() const { return rk_format_quantized(format); }
};

// Pointers to one page's four tensors in one layer (all kv heads).
struct PagePointers {
  uint8_t *keys, *values;
  float *key_scales, *value_scales;
};

PagePointers page_pointers(const Geometry &g, rk_page_entry entry, rk_kv_layer layer) {
  PagePointers p{};
  p.keys = reinterpret_cast<uint8_t *>(rk_tensor_address(entry, layer, g.data_bytes, g.scale_bytes, RK_TENSOR_KEYS));
  p.values = reinterpret_cast<uint8_t *>(rk_tensor_address(entry, layer, g.data_bytes, g.scale_bytes, RK_TENSOR_VALUES));
  if (g.quantized()) {
    p.key_scales = reinterpret_cast<float *>(rk_tensor_address(entry, layer, g.data_bytes, g.scale_bytes, RK_TENSOR_KEY_SCALES));
    p.value_scales = reinterpret_cast<float *>(rk_tensor_address(entry, layer, g.data_bytes, g.scale_bytes, RK_TENSOR_VALUE_SCALES));
  }
  return p;
}

inline int int4_code(uint8_t byte, uint32_t nibble) {
  const int code = (byte >> (nibble * 4)) & 0xF;
  return code - ((code & 0x8) ? 16 : 0);
}

// The stored code (not yet scaled) of one key element as a float.
inline float key_code(const Geometry &g, const PagePointers &p, uint32_t head, uint32_t token, uint32_t d) {
  const uint64_t e = rk_key_element(head, token, d, g.head_dim);
  switch (g.format) {
  case RK_FORMAT_INT8: return float(reinterpret_cast<const int8_t *>(p.keys)[e]);
  case RK_FORMAT_INT4: return float(int4_code(p.keys[e / 2], uint32_t(e & 1)));
  case RK_FORMAT_FP8E4M3: return rko_e4m3_to_f32(p.keys[e]);
  default: return rko_bf16_to_f32(reinterpret_cast<const uint16_t *>(p.keys)[e]);
  }
}

// INT4 values are token-major like the keys (paged_store_row.h:95-103);
// every other format keeps values dimension-major (KvExtent.h:52-58).
inline float value_code(const Geometry &g, const PagePointers &p, uint32_t head, uint32_t token, uint32_t d) {
  if (g.format == RK_FORMAT_INT4) {
    const uint64_t e = rk_key_element(head, token, d, g.head_dim);
    return float(int4_code(p.values[e / 2], uint32_t(e & 1)));
  }
  const uint64_t e = rk_value_element(head, token, d, g.head_dim);
  switch (g.format) {
  case RK_FORMAT_INT8: return float(reinterpret_cast<const int8_t *>(p.values)[e]);
  case RK_FORMAT_FP8E4M3: return rko_e4m3_to_f32(p.values[e]);
  default: return rko_bf16_to_f32(reinterpret_cast<const uint16_t *>(p.values)[e]);
  }
}

// paged_store_row.h:67-146 and paged_store_row_fp8.h:48-77 for one row of one
// tensor: `x` holds the row's head_dim source elements as bf16 bits.
void store_row(const Geometry &g, const PagePointers &p, bool value_tensor, uint32_t head,
               uint32_t page_token, const uint16_t *x, uint64_t x_stride) {
  const uint32_t D = g.head_dim;
  uint8_t *data = value_tensor ? p.values : p.keys;
  if (g.format == RK_FORMAT_BF16) {
    auto *out = reinterpret_cast<uint16_t *>(data);
    for (uint32_t d = 0; d < D; ++d) {
      const uint64_t e = value_tensor ? rk_value_element(head, page_token, d, D)
                                      : rk_key_element(head, page_token, d, D);
      out[e] = x[d * x_stride]; // the 16 source bits, untouched
    }
    return;
  }
  float maximum = 0.0f;
  for (uint32_t d = 0; d < D; ++d)
    maximum = std::max(maximum, std::fabs(rko_bf16_to_f32(x[d * x_stride])));
  const float range = g.format == RK_FORMAT_INT8 ? 127.0f : (g.format == RK_FORMAT_INT4 ? 7.0f : 448.0f);
  const float scale = maximum == 0.0f ? 0.0f : maximum / range;
  (value_tensor ? p.value_scales : p.key_scales)[rk_scale_element(head, page_token)] = scale;
  for (uint32_t d = 0; d < D; ++d) {
    const float v = rko_bf16_to_f32(x[d * x_stride]);
    // (v * range) / maximum, both IEEE round-to-nearest, then ties-to-even.
    const float scaled = maximum == 0.0f ? 0.0f : (v * range) / maximum;
    if (g.format == RK_FORMAT_FP8E4M3) {
      const uint64_t e = value_tensor ? rk_value_element(head, page_token, d, D)
                                      : rk_key_element(head, page_token, d, D);
      data[e] = maximum == 0.0f ? uint8_t(0) : rko_f32_to_e4m3(scaled);
      continue;
    }
    const int limit = int(range);
    const int q = maximum == 0.0f ? 0 : std::clamp(int(std::nearbyintf(scaled)), -limit, limit);
    if (g.format == RK_FORMAT_INT8) {
      const uint64_t e = value_tensor ? rk_value_element(head, page_token, d, D)
                                      : rk_key_element(head, page_token, d, D);
      reinterpret_cast<int8_t *>(data)[e] = int8_t(q);
    } else { // INT4: both tensors token-major, even dim in the low nibble
      const uint64_t e = rk_key_element(head, page_token, d, D);
      uint8_t &byte = data[e / 2];
      byte = (e & 1) ? uint8_t((byte & 0x0F) | ((q & 0xF) << 4)) : uint8_t((byte & 0xF0) | (q & 0xF));
    }
  }
}

float resolved_scale(float requested, uint32_t head_dim) { return rk_score_scale(requested, head_dim); }

// Whether query row `row` attends logical token `t`
// (paged_attention_tile.h:103-143).
inline bool admitted(uint32_t t, uint32_t row, uint32_t committed, uint32_t active_rows,
                     const uint32_t *row_masks) {
  const uint32_t visible = committed + active_rows;
  if (!row_masks) {
    const uint32_t causal_end = committed + std::min(row, active_rows - 1) + 1;
    return t < std::min(visible, causal_end);
  }
  return t < committed || (t < visible && ((row_masks[row] >> (t - committed)) & 1u));
}

} // namespace

extern "C" {

uint16_t rko_f32_to_bf16(float value) {
  uint32_t bits = std::bit_cast<uint32_t>(value);
  if ((bits & 0x7f800000u) == 0x7f800000u) {
    uint16_t upper = uint16_t(bits >> 16);
    if ((bits & 0x007fffffu) && !(upper & 0x007fu)) upper |= 1;
    return upper;
  }
  const uint32_t bias = 0x7fffu + ((bits >> 16) & 1u);
  return uint16_t((bits + bias) >> 16);
}

float rko_bf16_to_f32(uint16_t bits) { return std::bit_cast<float>(uint32_t(bits) << 16); }

uint8_t rko_f32_to_e4m3(float value) {
  const uint8_t sign = std::signbit(value) ? 0x80 : 0x00;
  const float a = std::fabs(value);
  if (!std::isfinite(a)) return uint8_t(sign | 0x7F);
  if (a >= 512.0f) return uint8_t(sign | 0x7E);
  if (a < 0x1p-6f) { // subnormal grid of 2^-9; 8 steps reach the first normal
    const long steps = std::lrintf(a * 512.0f);
    return uint8_t(sign | uint8_t(std::min<long>(steps, 8)));
  }
  int exponent = std::ilogb(a);
  long mantissa = std::lrintf(std::ldexp(a, 3 - exponent)); // 8..16
  if (mantissa == 16) { ++exponent; mantissa = 8; }
  if (exponent > 8 || (exponent == 8 && mantissa - 8 > 6)) return uint8_t(sign | 0x7E);
  return uint8_t(sign | uint8_t(((exponent + 7) << 3) | (mantissa - 8)));
}

float rko_e4m3_to_f32(uint8_t code) {
  const float sign = (code & 0x80) ? -1.0f : 1.0f;
  const int exponent = (code >> 3) & 0xF, mantissa = code & 0x7;
  if (exponent == 0) return sign * std::ldexp(float(mantissa), -9);
  if (exponent == 15 && mantissa == 7) return std::numeric_limits<float>::quiet_NaN();
  return sign * std::ldexp(1.0f + float(mantissa) / 8.0f, exponent - 7);
}

float rko_query_stage_f16(float value) { return float(_Float16(value)); }

int rko_store_chunk(uint32_t format, uint32_t kv_heads, uint32_t head_dim, const uint16_t *chunk_keys,
                    const uint16_t *chunk_values, const rk_page_entry *table,
                    const rk_chunk_params *params) {
  if (!rk_format_valid(format) || !rk_chunk_contract_valid(params)) return -1;
  const Geometry g(format, kv_heads, head_dim);
  const uint32_t stride = params->chunk_stride;
  for (uint32_t row = 0; row < params->chunk_tokens; ++row) {
    const uint32_t t = params->committed_tokens + row;
    const PagePointers p = page_pointers(g, table[t / RK_PAGE_TOKENS], params->kv);
    for (uint32_t head = 0; head < kv_heads; ++head) {
      // staging: K [head][stride][D], V [head][D][stride] (paged_store_row.h:31-41)
      store_row(g, p, false, head, t % RK_PAGE_TOKENS,
                chunk_keys + (uint64_t(head) * stride + row) * head_dim, 1);
      store_row(g, p, true, head, t % RK_PAGE_TOKENS,
                chunk_values + uint64_t(head) * head_dim * stride + row, stride);
    }
  }
  return 0;
}

int rko_store_verify(uint32_t format, uint32_t kv_heads, uint32_t head_dim, uint32_t lanes,
                     const uint16_t *chunk_keys, const uint16_t *chunk_values,
                     const rk_page_entry *const *tables, const rk_chunk_params *params) {
  const uint64_t lane_stride = uint64_t(kv_heads) * RK_VERIFY_CHUNK_STRIDE * head_dim;
  int status = 0;
  for (uint32_t lane = 0; lane < lanes; ++lane) {
    // decode/paged_attention_store.metal:23-27 (row bound widened from 15 to
    // the tile's 16 rows for the 16-token verify window).
    if (params[lane].chunk_tokens > RK_TREE_NODES || params[lane].chunk_stride != RK_VERIFY_CHUNK_STRIDE) {
      status = -1;
      continue;
    }
    if (rko_store_chunk(format, kv_heads, head_dim, chunk_keys + lane * lane_stride,
                        chunk_values + lane * lane_stride, tables[lane], &params[lane]) != 0)
      status = -1;
  }
  return status;
}

int rko_attention_tile(uint32_t format, uint32_t kv_heads, uint32_t group, uint32_t head_dim,
                       uint32_t kv_head, const uint16_t *queries, const rk_page_entry *table,
                       rk_kv_layer layer, uint32_t committed, uint32_t active_rows,
                       uint32_t row_capacity, const uint32_t *row_masks, float score_scale,
                       int q_fp16, float *out) {
  if (!rk_format_valid(format) || !active_rows || active_rows > row_capacity || kv_head >= kv_heads)
    return -1;
  const Geometry g(format, kv_heads, head_dim);
  const uint32_t D = head_dim, M = row_capacity * group;
  const uint32_t visible = committed + active_rows;
  const double scale = resolved_scale(score_scale, D);
  std::fill(out, out + uint64_t(M) * D, 0.0f);
  std::vector<double> q(D), scores(visible), acc(D);
  for (uint32_t m = 0; m < active_rows * group; ++m) {
    const uint32_t row = m / group;
    for (uint32_t d = 0; d < D; ++d) {
      float v = rko_bf16_to_f32(queries[uint64_t(m) * D + d]);
      q[d] = q_fp16 ? rko_query_stage_f16(v) : v;
    }
    double maximum = -std::numeric_limits<double>::infinity();
    for (uint32_t t = 0; t < visible; ++t) {
      if (!admitted(t, row, committed, active_rows, row_masks)) {
        scores[t] = -std::numeric_limits<double>::infinity();
        continue;
      }
      const PagePointers p = page_pointers(g, table[t / RK_PAGE_TOKENS], layer);
      const uint32_t pt = t % RK_PAGE_TOKENS;
      double dot = 0.0;
      for (uint32_t d = 0; d < D; ++d) dot += q[d] * double(key_code(g, p, kv_head, pt, d));
      if (g.quantized()) dot *= double(p.key_scales[rk_scale_element(kv_head, pt)]);
      scores[t] = dot * scale;
      maximum = std::max(maximum, scores[t]);
    }
    std::fill(acc.begin(), acc.end(), 0.0);
    double denominator = 0.0;
    for (uint32_t t = 0; t < visible; ++t) {
      if (scores[t] == -std::numeric_limits<double>::infinity()) continue;
      const double w = std::exp(scores[t] - maximum);
      denominator += w;
      const PagePointers p = page_pointers(g, table[t / RK_PAGE_TOKENS], layer);
      const uint32_t pt = t % RK_PAGE_TOKENS;
      const double vs = g.quantized() ? double(p.value_scales[rk_scale_element(kv_head, pt)]) : 1.0;
      if (vs == 0.0) continue; // a zero row contributes nothing whatever its codes hold
      for (uint32_t d = 0; d < D; ++d) acc[d] += w * vs * double(value_code(g, p, kv_head, pt, d));
    }
    for (uint32_t d = 0; d < D; ++d)
      out[uint64_t(m) * D + d] = denominator > 0.0 ? float(acc[d] / denominator) : 0.0f;
  }
  return 0;
}

// Float two-pass evaluation of one (lane, kv head) tile, page by page; the
// arithmetic the timed CPU baseline runs. Agrees with rko_attention_tile to
// fp32 rounding (checked in tests/test_oracle_pins.py).
static void attention_tile_fast(const Geometry &g, uint32_t group, uint32_t kv_head,
                                const uint16_t *queries, const rk_page_entry *table,
                                rk_kv_layer layer, uint32_t committed, uint32_t active_rows,
                                const uint32_t *row_masks, float score_scale, bool q_fp16,
                                float *out /* [active_rows*group][D] */) {
  const uint32_t D = g.head_dim, rows = active_rows * group;
  const uint32_t visible = committed + active_rows, pages = rk_pages_for(visible);
  const float scale = resolved_scale(score_scale, D);
  std::vector<float> q(uint64_t(rows) * D), s(uint64_t(rows) * pages * RK_PAGE_TOKENS);
  std::vector<float> krow(D), vpage(uint64_t(RK_PAGE_TOKENS) * D);
  for (uint64_t i = 0; i < q.size(); ++i) {
    const float v = rko_bf16_to_f32(queries[i]);
    q[i] = q_fp16 ? rko_query_stage_f16(v) : v;
  }
  const float ninf = -std::numeric_limits<float>::infinity();
  for (uint32_t page = 0; page < pages; ++page) {
    const PagePointers p = page_pointers(g, table[page], layer);
    for (uint32_t pt = 0; pt < RK_PAGE_TOKENS; ++pt) {
      const uint32_t t = page * RK_PAGE_TOKENS + pt;
      if (t >= visible) {
        for (uint32_t m = 0; m < rows; ++m) s[(uint64_t(m) * pages + page) * RK_PAGE_TOKENS + pt] = ninf;
        continue;
      }
      for (uint32_t d = 0; d < D; ++d) krow[d] = key_code(g, p, kv_head, pt, d);
      const float ks = g.quantized() ? p.key_scales[rk_scale_element(kv_head, pt)] : 1.0f;
      for (uint32_t m = 0; m < rows; ++m) {
        float dot = 0.0f;
        const float *qm = &q[uint64_t(m) * D];
        for (uint32_t d = 0; d < D; ++d) dot += qm[d] * krow[d];
        s[(uint64_t(m) * pages + page) * RK_PAGE_TOKENS + pt] =
            admitted(t, m / group, committed, active_rows, row_masks) ? dot * ks * scale : ninf;
      }
    }
  }
  std::vector<float> denominators(rows);
  for (uint32_t m = 0; m < rows; ++m) {
    float *sm = &s[uint64_t(m) * pages * RK_PAGE_TOKENS];
    float maximum = ninf;
    for (uint64_t i = 0; i < uint64_t(pages) * RK_PAGE_TOKENS; ++i) maximum = std::max(maximum, sm[i]);
    double sum = 0.0;
    for (uint64_t i = 0; i < uint64_t(pages) * RK_PAGE_TOKENS; ++i) {
      sm[i] = sm[i] == ninf ? 0.0f : std::exp(sm[i] - maximum);
      sum += sm[i];
    }
    denominators[m] = float(sum);
  }
  std::fill(out, out + uint64_t(rows) * D, 0.0f);
  for (uint32_t page = 0; page < pages; ++page) {
    const PagePointers p = page_pointers(g, table[page], layer);
    const uint32_t live = std::min<uint32_t>(RK_PAGE_TOKENS, visible - page * RK_PAGE_TOKENS);
    for (uint32_t pt = 0; pt < live; ++pt) {
      const float vs = g.quantized() ? p.value_scales[rk_scale_element(kv_head, pt)] : 1.0f;
      float *row = &vpage[uint64_t(pt) * D];
      if (vs == 0.0f) { std::fill(row, row + D, 0.0f); continue; }
      for (uint32_t d = 0; d < D; ++d) row[d] = vs * value_code(g, p, kv_head, pt, d);
    }
    for (uint32_t m = 0; m < rows; ++m) {
      const float *pm = &s[(uint64_t(m) * pages + page) * RK_PAGE_TOKENS];
      float *om = out + uint64_t(m) * D;
      for (uint32_t pt = 0; pt < live; ++pt) {
        const float w = pm[pt];
        if (w == 0.0f) continue;
        const float *row = &vpage[uint64_t(pt) * D];
        for (uint32_t d = 0; d < D; ++d) om[d] += w * row[d];
      }
    }
  }
  for (uint32_t m = 0; m < rows; ++m) {
    const float inv = denominators[m] > 0.0f ? 1.0f / denominators[m] : 0.0f;
    for (uint32_t d = 0; d < D; ++d) out[uint64_t(m) * D + d] *= inv;
  }
}

int rko_attention_verify(uint32_t format, uint32_t kv_heads, uint32_t group, uint32_t head_dim,
                         uint32_t lanes, const uint16_t *queries, const rk_page_entry *const *tables,
                         const rk_verify_params *params, const uint32_t *row_masks,
                         uint16_t *out_bf16, float *out_f32) {
  if (!rk_format_valid(format)) return -1;
  const Geometry g(format, kv_heads, head_dim);
  const uint64_t tile = uint64_t(RK_VERIFY_CHUNK_STRIDE) * group * head_dim;
  int status = 0;
  const int64_t tiles = int64_t(lanes) * kv_heads;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t index = 0; index < tiles; ++index) {
    const uint32_t lane = uint32_t(index / kv_heads), head = uint32_t(index % kv_heads);
    const rk_verify_params &p = params[lane];
    if (!rk_verify_contract_valid(&p)) {
#pragma omp atomic write
      status = -1;
      continue;
    }
    const uint32_t rows = p.active_rows * group;
    std::vector<float> result(uint64_t(rows) * head_dim);
    attention_tile_fast(g, group, head, queries + uint64_t(index) * tile, tables[lane], p.kv,
                        p.committed_tokens, p.active_rows,
                        row_masks ? row_masks + uint64_t(lane) * p.row_capacity : nullptr,
                        p.score_scale, format == RK_FORMAT_FP8E4M3, result.data());
    for (uint32_t m = 0; m < p.row_capacity * group; ++m)
      for (uint32_t d = 0; d < head_dim; ++d) {
        const float v = m < rows ? result[uint64_t(m) * head_dim + d] : 0.0f;
        const uint64_t at = uint64_t(index) * tile + uint64_t(m) * head_dim + d;
        if (out_bf16) out_bf16[at] = rko_f32_to_bf16(v);
        if (out_f32) out_f32[at] = v;
      }
  }
  return status;
}

void rko_merge_row(const float *partials, uint64_t partial_stride, const float *stats,
                   uint64_t stat_stride, uint32_t written, uint32_t head_dim, float *out_f32) {
  float maximum = -std::numeric_limits<float>::infinity();
  for (uint32_t s = 0; s < written; ++s) maximum = std::max(maximum, stats[s * stat_stride]);
  for (uint32_t d = 0; d < head_dim; ++d) {
    float numerator = 0.0f, denominator = 0.0f;
    for (uint32_t s = 0; s < written; ++s) { // split order, sequentially
      const float weight = std::exp(stats[s * stat_stride] - maximum);
      numerator += weight * partials[s * partial_stride + d];
      denominator += weight * stats[s * stat_stride + 1];
    }
    out_f32[d] = denominator > 0.0f ? numerator / denominator : 0.0f;
  }
}

int rko_tree_compact(uint32_t format, uint32_t kv_heads, uint32_t head_dim, const rk_page_entry *table,
                     const rk_chunk_params *params, const uint32_t *retained_path,
                     uint32_t retained_count) {
  if (!rk_format_valid(format) || format == RK_FORMAT_FP8E4M3) return -1;
  const Geometry g(format, kv_heads, head_dim);
  const uint32_t D = head_dim;
  const uint32_t element_bytes = format == RK_FORMAT_BF16 ? 2 : 1;
  for (uint32_t head = 0; head < kv_heads; ++head) {
    for (uint32_t i = 0; i < retained_count; ++i) {
      const uint32_t source_row = retained_path[i];
      if (source_row == i) continue;
      const uint32_t st = params->committed_tokens + source_row, dt = params->committed_tokens + i;
      const PagePointers s = page_pointers(g, table[st / RK_PAGE_TOKENS], params->kv);
      const PagePointers d = page_pointers(g, table[dt / RK_PAGE_TOKENS], params->kv);
      const uint32_t so = st % RK_PAGE_TOKENS, dofs = dt % RK_PAGE_TOKENS;
      if (format == RK_FORMAT_INT4) { // both tensors token-major rows of D/2 bytes
        const uint64_t sb = rk_key_element(head, so, 0, D) / 2, db = rk_key_element(head, dofs, 0, D) / 2;
        std::memmove(d.keys + db, s.keys + sb, D / 2);
        std::memmove(d.values + db, s.values + sb, D / 2);
      } else {
        std::memmove(d.keys + rk_key_element(head, dofs, 0, D) * element_bytes,
                     s.keys + rk_key_element(head, so, 0, D) * element_bytes, uint64_t(D) * element_bytes);
        for (uint32_t dim = 0; dim < D; ++dim)
          std::memcpy(d.values + rk_value_element(head, dofs, dim, D) * element_bytes,
                      s.values + rk_value_element(head, so, dim, D) * element_bytes, element_bytes);
      }
      if (g.quantized()) {
        d.key_scales[rk_scale_element(head, dofs)] = s.key_scales[rk_scale_element(head, so)];
        d.value_scales[rk_scale_element(head, dofs)] = s.value_scales[rk_scale_element(head, so)];
      }
    }
  }
  return 0;
}

void rko_copy_page(uint32_t format, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                   uint32_t extent_pages, rk_page_entry from, rk_page_entry to) {
  const Geometry g(format, kv_heads, head_dim);
  for (uint32_t layer = 0; layer < layers; ++layer)
    for (uint32_t tensor = RK_TENSOR_KEYS; tensor <= RK_TENSOR_VALUE_SCALES; ++tensor) {
      const uint32_t bytes = rk_tensor_page_bytes(g.data_bytes, g.scale_bytes, tensor);
      if (!bytes) continue;
      const auto *src = reinterpret_cast<const uint8_t *>(
          rk_entry_extent(from) + rk_extent_offset(extent_pages, g.data_bytes, g.scale_bytes, layer, tensor, rk_entry_index(from)));
      auto *dst = reinterpret_cast<uint8_t *>(
          rk_entry_extent(to) + rk_extent_offset(extent_pages, g.data_bytes, g.scale_bytes, layer, tensor, rk_entry_index(to)));
      std::memcpy(dst, src, bytes);
    }
}

// No fused multiply-add anywhere in this function: every product and sum is rounded on its own, as the CUDA
// kernel does with its _rn intrinsics.
__attribute__((optimize("fp-contract=off")))
int rko_qkv_prepare(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes, uint32_t rows,
                    const uint16_t *packed_qkv, const void *q_norm, const void *k_norm, int norm_f32,
                    const float *rope_cos, const float *rope_sin, float eps, uint16_t *queries, uint16_t *chunk_keys,
                    uint16_t *chunk_values) {
  constexpr uint32_t kRotaryPairs = 32, kStride = RK_VERIFY_CHUNK_STRIDE;
  if (!kv_heads || query_heads % kv_heads || head_dim % 32 || head_dim < 2 * kRotaryPairs || !rows || rows > kStride) return -1;
  const uint32_t D = head_dim, group = query_heads / kv_heads;
  const uint64_t packed_stride = uint64_t(query_heads) * 2 * D + 2ull * kv_heads * D;
  auto weight = [&](const void *w, uint32_t d) {
    return norm_f32 ? static_cast<const float *>(w)[d] : rko_bf16_to_f32(static_cast<const uint16_t *>(w)[d]);
  };
  std::vector<float> x(D), sq(D);
  std::vector<uint16_t> normalized(D);
  for (uint32_t lane = 0; lane < lanes; ++lane)
    for (uint32_t row = 0; row < rows; ++row) {
      const uint16_t *source_row = packed_qkv + (uint64_t(lane) * rows + row) * packed_stride;
      const float *cosine = rope_cos + (uint64_t(lane) * rows + row) * kRotaryPairs;
      const float *sine = rope_sin + (uint64_t(lane) * rows + row) * kRotaryPairs;
      for (uint32_t task = 0; task < query_heads + kv_heads; ++task) {
        const bool query = task < query_heads;
        const uint32_t head = query ? task : task - query_heads;
        const uint16_t *source = query ? source_row + uint64_t(head) * 2 * D : source_row + uint64_t(query_heads) * 2 * D + uint64_t(head) * D;
        for (uint32_t d = 0; d < D; ++d) { x[d] = rko_bf16_to_f32(source[d]); sq[d] = x[d] * x[d]; }
        float total = 0.0f;
        for (uint32_t base = 0; base < D; base += 32) { // per 32 dims: xor butterfly, every lane ends with the same sum
          float v[32];
          for (uint32_t i = 0; i < 32; ++i) v[i] = sq[base + i];
          for (uint32_t offset = 16; offset; offset >>= 1) {
            float next[32];
            for (uint32_t i = 0; i < 32; ++i) next[i] = v[i] + v[i ^ offset];
            for (uint32_t i = 0; i < 32; ++i) v[i] = next[i];
          }
          total += v[0];
        }
        const float inverse = 1.0f / std::sqrt(total / float(D) + eps);
        const void *w = query ? q_norm : k_norm;
        for (uint32_t d = 0; d < D; ++d) normalized[d] = rko_f32_to_bf16((x[d] * inverse) * weight(w, d));
        uint16_t *destination;
        if (query) {
          const uint32_t kv = head / group, local = head % group;
          destination = queries + (((uint64_t(lane) * kv_heads + kv) * kStride + row) * group + local) * D;
        } else {
          destination = chunk_keys + ((uint64_t(lane) * kv_heads + head) * kStride + row) * D;
          const uint16_t *value_source = source + uint64_t(kv_heads) * D; // the head's v row follows all k rows
          for (uint32_t d = 0; d < D; ++d)
            chunk_values[((uint64_t(lane) * kv_heads + head) * D + d) * kStride + row] = value_source[d];
        }
        for (uint32_t i = 0; i < kRotaryPairs; ++i) {
          const float first = rko_bf16_to_f32(normalized[i]), second = rko_bf16_to_f32(normalized[i + kRotaryPairs]);
          const float a = first * cosine[i], b = second * sine[i], c = second * cosine[i], e = first * sine[i];
          destination[i] = rko_f32_to_bf16(a - b);
          destination[i + kRotaryPairs] = rko_f32_to_bf16(c + e);
        }
        for (uint32_t d = 2 * kRotaryPairs; d < D; ++d) destination[d] = normalized[d];
      }
    }
  return 0;
}

uint32_t rko_crc32c(const void *data, uint64_t bytes, uint32_t crc) {
  const uint8_t *p = static_cast<const uint8_t *>(data);
  uint32_t state = ~crc;
  for (uint64_t i = 0; i < bytes; ++i) {
    state ^= p[i];
    for (int bit = 0; bit < 8; ++bit) state = (state & 1u) ? (state >> 1) ^ 0x82F63B78u : state >> 1;
  }
  return ~state;
}

int rko_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

} // extern "C"
