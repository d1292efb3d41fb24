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

#include <memory>
#include <vector>

namespace rk {
namespace {

// grid (lanes * kv_heads), 256 threads (one per dimension).
__global__ void __launch_bounds__(256)
stage_rows_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v,
                  uint16_t *__restrict__ queries, uint16_t *__restrict__ chunk_keys,
                  uint16_t *__restrict__ chunk_values, uint32_t group, uint32_t head_dim) {
  const uint64_t tile = blockIdx.x; // lane * kv_heads + kv_head
  const uint32_t d = threadIdx.x;
  // the store and attention kernels behind this one may take their places and run their prologues; this kernel
  // overwrites stagings the attention kernel before it read, so it waits for that one first
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
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
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory"); // the merge that writes `output` runs just before
  if (d >= head_dim) return;
  for (uint32_t g = 0; g < group; ++g)
    out[(tile * group + g) * head_dim + d] = output[(tile * RK_VERIFY_CHUNK_STRIDE * group + g) * head_dim + d];
}

// A launch that may begin before the kernel ahead of it in the stream has drained (programmatic dependent launch);
// both kernels wait for it themselves before they touch its results.
template <typename Kernel, typename... Args>
int launch_chained(Kernel kernel, uint32_t blocks, cudaStream_t stream, const char *what, Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(blocks);
  config.blockDim = dim3(256);
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&config, kernel, args...), what);
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
  return launch_chained(stage_rows_kernel, lanes * kv_heads, static_cast<cudaStream_t>(stream), "stage rows launch",
                        static_cast<const uint16_t *>(q), static_cast<const uint16_t *>(k), static_cast<const uint16_t *>(v),
                        static_cast<uint16_t *>(queries), static_cast<uint16_t *>(chunk_keys), static_cast<uint16_t *>(chunk_values),
                        query_heads / kv_heads, head_dim);
}

extern "C" int rk_gather_decode_rows(uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim, uint32_t lanes,
                                     const void *output, void *out, void *stream) {
  if (!lanes || !kv_heads || query_heads % kv_heads || head_dim > 256 || !output || !out) {
    set_error("rk_gather_decode_rows: invalid arguments");
    return kInvalid;
  }
  return launch_chained(gather_rows_kernel, lanes * kv_heads, static_cast<cudaStream_t>(stream), "gather rows launch",
                        static_cast<const uint16_t *>(output), static_cast<uint16_t *>(out), query_heads / kv_heads, head_dim);
}

// ---- one decode step with HOST rows, as a C entry -------------------------------------------------------------------
// What a host-side caller of the reference's attention operator does per layer with rows it holds in host memory
// (runtime/ops/PagedAttention.cpp:467-545 encodes store -> split -> reduce; the rows reach the stagings through the
// model runtime's uploads): rk_session_step_host sends the lanes' query / key / value rows from pinned host memory,
// appends the key / value rows to the pages, attends and brings the output rows back to pinned host memory. Calls
// pipeline: the rows of a call are uploaded on a copy stream while the previous call's kernels run, and a call's
// output leaves on a second copy stream while the next call computes (two sets of row buffers, events between the
// streams); rk_session_finish_host orders the caller's stream after every result copy.
namespace rk {
namespace {
struct HostSession {
  uint32_t format = 0, kv_heads = 0, query_heads = 0, head_dim = 0, lanes = 0;
  const void *window = nullptr;
  std::vector<rk_kv_layer> layers;
  rk_decode_plan plan{};
  uint8_t *arena = nullptr; // every device buffer of the session, one allocation
  uint16_t *queries = nullptr, *output = nullptr, *chunk_keys = nullptr, *chunk_values = nullptr;
  uint16_t *q_rows[2] = {}, *k_rows[2] = {}, *v_rows[2] = {}, *out_rows[2] = {};
  float *partials = nullptr, *statistics = nullptr;
  uint32_t *descriptors = nullptr;
  cudaStream_t upload = nullptr, download = nullptr;
  cudaEvent_t uploaded[2] = {}, consumed[2] = {}, gathered[2] = {}, downloaded[2] = {};
  uint64_t calls = 0;
  ~HostSession() {
    for (cudaEvent_t *set : {uploaded, consumed, gathered, downloaded})
      for (int i = 0; i < 2; ++i)
        if (set[i]) cudaEventDestroy(set[i]);
    if (upload) cudaStreamDestroy(upload);
    if (download) cudaStreamDestroy(download);
    if (arena) cudaFree(arena);
  }
};
} // namespace
} // namespace rk

extern "C" void *rk_session_create(uint32_t format, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                                   uint32_t lanes, const void *window, const rk_kv_layer *layers, uint32_t layer_count,
                                   uint32_t ctas) {
  if (!window || !layers || !layer_count || !lanes) { set_error("rk_session_create: invalid arguments"); return nullptr; }
  auto session = std::make_unique<HostSession>();
  HostSession &s = *session;
  s.format = format; s.kv_heads = kv_heads; s.query_heads = query_heads; s.head_dim = head_dim; s.lanes = lanes;
  s.window = window;
  s.layers.assign(layers, layers + layer_count);
  if (rk_decode_plan_make(format, kv_heads, query_heads, head_dim, lanes, ctas, &s.plan) != kOk) return nullptr;
  const uint64_t stride = RK_VERIFY_CHUNK_STRIDE;
  const uint64_t query_tile = uint64_t(lanes) * query_heads * stride * head_dim * 2; // [lane][kv head][32][group][D]
  const uint64_t kv_tile = uint64_t(lanes) * kv_heads * stride * head_dim * 2;
  const uint64_t query_rows = uint64_t(lanes) * query_heads * head_dim * 2, kv_rows = uint64_t(lanes) * kv_heads * head_dim * 2;
  auto rounded = [](uint64_t bytes) { return (bytes + 255) & ~uint64_t(255); };
  const uint64_t sizes[] = {query_tile, query_tile, kv_tile, kv_tile, query_rows, query_rows, kv_rows, kv_rows, kv_rows, kv_rows,
                            query_rows, query_rows, s.plan.partials_bytes, s.plan.statistics_bytes, s.plan.descriptor_bytes};
  uint64_t total = 0;
  for (uint64_t bytes : sizes) total += rounded(bytes);
  if (cuda_status(cudaMalloc(reinterpret_cast<void **>(&s.arena), total), "session buffers") ||
      cuda_status(cudaMemset(s.arena, 0, total), "session buffers"))
    return nullptr;
  uint8_t *at = s.arena;
  auto take = [&](uint64_t bytes) { uint8_t *p = at; at += rounded(bytes); return p; };
  s.queries = reinterpret_cast<uint16_t *>(take(query_tile));
  s.output = reinterpret_cast<uint16_t *>(take(query_tile));
  s.chunk_keys = reinterpret_cast<uint16_t *>(take(kv_tile));
  s.chunk_values = reinterpret_cast<uint16_t *>(take(kv_tile));
  for (int i = 0; i < 2; ++i) s.q_rows[i] = reinterpret_cast<uint16_t *>(take(query_rows));
  for (int i = 0; i < 2; ++i) s.k_rows[i] = reinterpret_cast<uint16_t *>(take(kv_rows));
  for (int i = 0; i < 2; ++i) s.v_rows[i] = reinterpret_cast<uint16_t *>(take(kv_rows));
  for (int i = 0; i < 2; ++i) s.out_rows[i] = reinterpret_cast<uint16_t *>(take(query_rows));
  s.partials = reinterpret_cast<float *>(take(s.plan.partials_bytes));
  s.statistics = reinterpret_cast<float *>(take(s.plan.statistics_bytes));
  s.descriptors = reinterpret_cast<uint32_t *>(take(s.plan.descriptor_bytes));
  if (cuda_status(cudaStreamCreateWithFlags(&s.upload, cudaStreamNonBlocking), "session stream") ||
      cuda_status(cudaStreamCreateWithFlags(&s.download, cudaStreamNonBlocking), "session stream"))
    return nullptr;
  for (cudaEvent_t *set : {s.uploaded, s.consumed, s.gathered, s.downloaded})
    for (int i = 0; i < 2; ++i)
      if (cuda_status(cudaEventCreateWithFlags(&set[i], cudaEventDisableTiming), "session event")) return nullptr;
  return session.release();
}

extern "C" void rk_session_destroy(void *session) {
  auto *s = static_cast<HostSession *>(session);
  if (!s) return;
  cudaStreamSynchronize(s->upload);
  cudaStreamSynchronize(s->download);
  delete s;
}

extern "C" int rk_session_step_host(void *session, uint32_t layer, const void *q_host, const void *k_host,
                                    const void *v_host, void *out_host, const rk_page_entry *const *tables,
                                    const rk_chunk_params *chunk_params, const rk_verify_params *verify_params,
                                    void *stream) {
  auto *s = static_cast<HostSession *>(session);
  if (!s || layer >= s->layers.size() || !q_host || !k_host || !v_host || !out_host || !tables || !chunk_params || !verify_params) {
    set_error("rk_session_step_host: invalid arguments");
    return kInvalid;
  }
  cudaStream_t compute = static_cast<cudaStream_t>(stream);
  const uint32_t slot = uint32_t(s->calls++ & 1u);
  const uint64_t query_rows = uint64_t(s->lanes) * s->query_heads * s->head_dim * 2, kv_rows = uint64_t(s->lanes) * s->kv_heads * s->head_dim * 2;
  // upload: after the call before last has read this set of row buffers
  if (int st = cuda_status(cudaStreamWaitEvent(s->upload, s->consumed[slot], 0), "session upload order")) return st;
  if (int st = cuda_status(cudaMemcpyAsync(s->q_rows[slot], q_host, query_rows, cudaMemcpyHostToDevice, s->upload), "session upload")) return st;
  if (int st = cuda_status(cudaMemcpyAsync(s->k_rows[slot], k_host, kv_rows, cudaMemcpyHostToDevice, s->upload), "session upload")) return st;
  if (int st = cuda_status(cudaMemcpyAsync(s->v_rows[slot], v_host, kv_rows, cudaMemcpyHostToDevice, s->upload), "session upload")) return st;
  if (int st = cuda_status(cudaEventRecord(s->uploaded[slot], s->upload), "session upload event")) return st;
  if (int st = cuda_status(cudaStreamWaitEvent(compute, s->uploaded[slot], 0), "session compute order")) return st;
  // the output rows of the call before last must have left their buffer; waited for here, ahead of the kernels, so
  // that the five kernels of the call follow one another without a host-side wait between them
  if (int st = cuda_status(cudaStreamWaitEvent(compute, s->downloaded[slot], 0), "session download order")) return st;
  if (int st = rk_stage_decode_rows(s->kv_heads, s->query_heads, s->head_dim, s->lanes, s->q_rows[slot], s->k_rows[slot],
                                    s->v_rows[slot], s->queries, s->chunk_keys, s->chunk_values, compute)) return st;
  if (int st = cuda_status(cudaEventRecord(s->consumed[slot], compute), "session consumed event")) return st;
  const rk_kv_layer place = s->layers[layer];
  if (int st = rk_store_verify(s->format, s->kv_heads, s->head_dim, s->lanes, 1, s->chunk_keys, s->chunk_values, tables,
                               chunk_params, place, compute)) return st;
  if (int st = rk_attention_decode(s->window, &s->plan, s->format, s->queries, s->output, nullptr, s->partials,
                                   s->statistics, s->descriptors, tables, verify_params, place, compute)) return st;
  if (int st = rk_gather_decode_rows(s->kv_heads, s->query_heads, s->head_dim, s->lanes, s->output, s->out_rows[slot], compute)) return st;
  if (int st = cuda_status(cudaEventRecord(s->gathered[slot], compute), "session gathered event")) return st;
  if (int st = cuda_status(cudaStreamWaitEvent(s->download, s->gathered[slot], 0), "session download order")) return st;
  if (int st = cuda_status(cudaMemcpyAsync(out_host, s->out_rows[slot], query_rows, cudaMemcpyDeviceToHost, s->download), "session download")) return st;
  return cuda_status(cudaEventRecord(s->downloaded[slot], s->download), "session download event");
}

extern "C" int rk_session_finish_host(void *session, void *stream) {
  auto *s = static_cast<HostSession *>(session);
  if (!s) { set_error("rk_session_finish_host: invalid arguments"); return kInvalid; }
  for (int i = 0; i < 2; ++i)
    if (int st = cuda_status(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), s->downloaded[i], 0), "session finish")) return st;
  return kOk;
}

extern "C" int rk_session_status(void *session, void *stream) {
  auto *s = static_cast<HostSession *>(session);
  if (!s) { set_error("rk_session_status: invalid arguments"); return kInvalid; }
  return rk_attention_decode_status(&s->plan, s->descriptors, stream);
}
