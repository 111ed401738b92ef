// Minimal stand-in for the two xtensor facilities the reference CPU GEMM uses:
// xt::no_ownership() and xt::adapt(ptr, size, no_ownership, shape) returning a
// row-major N-d view with operator()(i, j, ...).  Test infrastructure only: it
// lets the reference's src/reference/GEMM.cpp compile unmodified where xtensor
// itself is not installed.  Indexing only; no arithmetic lives here.
#ifndef ORACLE_REF_SHIM_XADAPT_HPP_
#define ORACLE_REF_SHIM_XADAPT_HPP_
#include <array>
#include <cstddef>

namespace xt {
struct no_ownership {};

template <typename T, std::size_t N> class row_major_view {
public:
  row_major_view(T *data, const std::array<std::size_t, N> &shape)
      : data_(data) {
    std::size_t stride = 1;
    for (std::size_t d = N; d-- > 0;) {
      strides_[d] = stride;
      stride *= shape[d];
    }
  }
  template <typename... Idx> T &operator()(Idx... idx) const {
    static_assert(sizeof...(Idx) == N, "index rank mismatch");
    const std::size_t ids[N] = {static_cast<std::size_t>(idx)...};
    std::size_t offset = 0;
    for (std::size_t d = 0; d < N; ++d) {
      offset += ids[d] * strides_[d];
    }
    return data_[offset];
  }

private:
  T *data_;
  std::size_t strides_[N];
};

template <typename T, std::size_t N>
row_major_view<T, N> adapt(T *data, std::size_t /*size*/, no_ownership,
                           const std::array<std::size_t, N> &shape) {
  return row_major_view<T, N>(data, shape);
}
} // namespace xt
#endif
