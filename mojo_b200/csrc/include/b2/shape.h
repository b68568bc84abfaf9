// Fixed-rank shapes, strides and coordinates for kernel parameters.
//
// The role of the reference's `IndexList` / `Index` / `product` (stdlib/src/utils/index.mojo:169-840, 842-1076,
// 1077-1113): a small integer tuple passed by value, usable on host and device, with the arithmetic every indexed
// kernel needs (element count, row-major strides, coordinate <-> linear offset). Plain aggregates, no heap, no
// virtuals: they sit in `__grid_constant__` parameter structs as they are.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define B2_HD __host__ __device__ __forceinline__
#define B2_UNROLL _Pragma("unroll")
#else
#define B2_HD inline
#define B2_UNROLL
#endif

namespace b2 {

template <int N>
struct Shape {
  int64_t d[N];

  B2_HD int64_t& operator[](int i) { return d[i]; }
  B2_HD const int64_t& operator[](int i) const { return d[i]; }
  static constexpr int rank() { return N; }

  // number of elements (the product of the extents; 1 for an empty product is never needed: N >= 1)
  B2_HD int64_t numel() const {
    int64_t n = 1;
B2_UNROLL
    for (int i = 0; i < N; ++i) n *= d[i];
    return n;
  }
  B2_HD bool operator==(const Shape& o) const {
    bool eq = true;
B2_UNROLL
    for (int i = 0; i < N; ++i) eq = eq && d[i] == o.d[i];
    return eq;
  }
};

template <int N>
using Coord = Shape<N>;

template <int N>
struct Stride {
  int64_t s[N];

  B2_HD int64_t& operator[](int i) { return s[i]; }
  B2_HD const int64_t& operator[](int i) const { return s[i]; }

  // element offset of a coordinate
  B2_HD int64_t offset(const Coord<N>& c) const {
    int64_t o = 0;
B2_UNROLL
    for (int i = 0; i < N; ++i) o += c.d[i] * s[i];
    return o;
  }
};

// Strides of a densely packed row-major tensor of this shape (last extent contiguous).
template <int N>
B2_HD Stride<N> row_major(const Shape<N>& shape) {
  Stride<N> st{};
  int64_t run = 1;
B2_UNROLL
  for (int i = N - 1; i >= 0; --i) {
    st.s[i] = run;
    run *= shape.d[i];
  }
  return st;
}

// Coordinate of the linear index `i` of a row-major walk over `shape` (inverse of row_major(shape).offset).
template <int N>
B2_HD Coord<N> delinearize(int64_t i, const Shape<N>& shape) {
  Coord<N> c{};
B2_UNROLL
  for (int k = N - 1; k >= 0; --k) {
    c.d[k] = i % shape.d[k];
    i /= shape.d[k];
  }
  return c;
}

// True when every coordinate lies inside the shape: the check a kernel makes before it trusts run-time metadata.
template <int N>
B2_HD bool in_bounds(const Coord<N>& c, const Shape<N>& shape) {
  bool ok = true;
B2_UNROLL
  for (int i = 0; i < N; ++i) ok = ok && c.d[i] >= 0 && c.d[i] < shape.d[i];
  return ok;
}

template <typename... T>
B2_HD Shape<static_cast<int>(sizeof...(T))> make_shape(T... v) {
  return Shape<static_cast<int>(sizeof...(T))>{{static_cast<int64_t>(v)...}};
}

}  // namespace b2
