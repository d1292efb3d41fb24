// Stands in for Metal Performance Primitives' tensor operations when the reference's attention tile
// (runtime/metal/kernels/common/paged_attention_tile.h) is compiled as C++ for the test-only checker: tensor views over
// plain memory (bf16, fp16, int8, fp32, e4m3 bytes, and 4-bit two's-complement pairs with the even element in the low
// nibble), a
// matmul2d whose destination is a cooperative tensor spread evenly over the 256 threads of the threadgroup, products
// widened to fp32 and summed in index order. Only what that header uses exists. TEST INFRASTRUCTURE ONLY.
#pragma once
#include <metal_stdlib>
#include <vector>

namespace metal {
struct int4b_format {};
struct tensor_inline {};
template <typename Index, size_t Rank> struct dextents {
  Index e0, e1;
  constexpr dextents(Index a, Index b) : e0(a), e1(b) {}
};

namespace rk_detail {
inline float widen(float v) { return v; }
inline float widen(bfloat v) { return float(v); }
inline float widen(int8_t v) { return float(v); }
inline float widen(half v) { return float(v); }
inline void narrow(float &to, float v) { to = v; }
inline void narrow(half &to, float v) { to = half(v); }
inline void narrow(bfloat &to, float v) { to = bfloat(v); }
} // namespace rk_detail

// A two-dimensional view: element (i0, i1) lives at data[i0 * s0 + i1 * s1].
template <typename Element, typename Extents = dextents<int, 2>, typename Tag = tensor_inline> struct tensor {
  Element *data;
  int e0, e1, s0, s1;
  tensor(Element *pointer, Extents extents, array<int, 2> strides) : data(pointer), e0(extents.e0), e1(extents.e1), s0(strides[0]), s1(strides[1]) {}
  template <int A, int B> tensor slice(int i0, int i1) const {
    tensor view = *this;
    view.data = data + long(i0) * s0 + long(i1) * s1;
    view.e0 = A; view.e1 = B;
    return view;
  }
  float load(int i0, int i1) const { return rk_detail::widen(data[long(i0) * s0 + long(i1) * s1]); }
  void store(int i0, int i1, float value) const { rk_detail::narrow(data[long(i0) * s0 + long(i1) * s1], value); }
};
// 4-bit operands: element index i0 * s0 + i1 * s1 counts nibbles from the slab's first byte.
template <typename Extents, typename Tag> struct tensor<int4b_format, Extents, Tag> {
  const uchar *data;
  long first;
  int e0, e1, s0, s1;
  tensor(const uchar *pointer, Extents extents, array<int, 2> strides) : data(pointer), first(0), e0(extents.e0), e1(extents.e1), s0(strides[0]), s1(strides[1]) {}
  template <int A, int B> tensor slice(int i0, int i1) const {
    tensor view = *this;
    view.first = first + long(i0) * s0 + long(i1) * s1;
    view.e0 = A; view.e1 = B;
    return view;
  }
  float load(int i0, int i1) const {
    const long at = first + long(i0) * s0 + long(i1) * s1;
    const uint nibble = (data[at >> 1] >> ((at & 1) * 4)) & 0xFu;
    return float(int(nibble ^ 8u) - 8);
  }
};
// e4m3 operands: one byte per element, decoded by the reference's own conversion.
template <typename Extents, typename Tag> struct tensor<metal_fp8_e4m3_format, Extents, Tag> {
  const uchar *data;
  int e0, e1, s0, s1;
  tensor(const uchar *pointer, Extents extents, array<int, 2> strides) : data(pointer), e0(extents.e0), e1(extents.e1), s0(strides[0]), s1(strides[1]) {}
  template <int A, int B> tensor slice(int i0, int i1) const {
    tensor view = *this;
    view.data = data + long(i0) * s0 + long(i1) * s1;
    view.e0 = A; view.e1 = B;
    return view;
  }
  float load(int i0, int i1) const { return ref_e4m3_to_f32(data[long(i0) * s0 + long(i1) * s1]); }
};
template <typename Element, typename Extents> tensor(Element *, Extents, array<int, 2>) -> tensor<Element, Extents, tensor_inline>;
} // namespace metal

namespace mpp {
namespace tensor_ops {
struct matmul2d_descriptor {
  enum class mode { multiply, multiply_accumulate };
  int m, n, k;
  bool transpose_left, transpose_right, relaxed_precision;
  mode reduction;
  constexpr matmul2d_descriptor(int m_, int n_, int k_, bool left, bool right, bool relaxed, mode reduction_)
      : m(m_), n(n_), k(k_), transpose_left(left), transpose_right(right), relaxed_precision(relaxed), reduction(reduction_) {}
};
template <int Groups> struct execution_simdgroups { static constexpr int threads = Groups * 32; };

// The destination of a matmul2d: extents {n, m}, dealt to the threads in runs of `capacity` consecutive elements.
template <typename Value> struct cooperative_tensor {
  int n = 0, m = 0, threads = 256, capacity = 0;
  std::vector<Value> values;
  cooperative_tensor(int n_, int m_, int threads_) : n(n_), m(m_), threads(threads_), capacity((n_ * m_ + threads_ - 1) / threads_), values(size_t(capacity), Value(0)) {}
  int linear(int index) const { return int(rk_metal_thread_index) * capacity + index; }
  int get_capacity() const { return capacity; }
  bool is_valid_element(int index) const { return linear(index) < n * m; }
  metal::array<int, 2> get_multidimensional_index(int index) const { return {linear(index) % n, linear(index) / n}; }
  Value &operator[](int index) { return values[size_t(index)]; }
  template <typename Destination> void store(Destination destination) const {
    for (int index = 0; index < capacity; ++index)
      if (is_valid_element(index)) destination.store(linear(index) % n, linear(index) / n, values[size_t(index)]);
  }
};

// destination(j, i) (+)= sum over k of left(k, i) * right, where the right operand is (j, k) as it stands and (k, j)
// transposed: the shapes paged_attention_tile.h gives its operands (left {K, M}; right {N, K} or {K, N}; result {N, M}).
template <matmul2d_descriptor Descriptor, typename Execution> struct matmul2d {
  template <typename Left, typename Right, typename Value> cooperative_tensor<Value> get_destination_cooperative_tensor() const {
    return cooperative_tensor<Value>(Descriptor.n, Descriptor.m, Execution::threads);
  }
  template <typename Left, typename Right, typename Destination> void run(Left left, Right right, Destination &destination) const {
    static_assert(!Descriptor.transpose_left, "the tile never transposes its left operand");
    for (int index = 0; index < destination.get_capacity(); ++index) {
      if (!destination.is_valid_element(index)) continue;
      const auto at = destination.get_multidimensional_index(index);
      float sum = 0.0f;
      for (int k = 0; k < Descriptor.k; ++k)
        sum += left.load(k, at[1]) * (Descriptor.transpose_right ? right.load(k, at[0]) : right.load(at[0], k));
      if (Descriptor.reduction == matmul2d_descriptor::mode::multiply) destination[index] = sum;
      else destination[index] += sum;
    }
  }
};
} // namespace tensor_ops
} // namespace mpp
