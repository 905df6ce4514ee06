// culib::range and the strided device ranges the reference's drivers and kernels iterate with
// (lib/range.hpp:204-264): `for (int i : culib::range(0, n))`, `range(a, b).step(s)`,
// `grid_stride_range`, `block_stride_range`, `warp_stride_range`.  A small re-implementation:
// one iterator type that walks an arithmetic progression and compares "not yet past the end".
#pragma once
#include <cstddef>
#include <initializer_list>
#include <type_traits>

#if defined(__CUDACC__)
#define ET_RANGE_FN __host__ __device__
#else
#define ET_RANGE_FN
#endif

namespace culib {

template <typename T> class range_proxy {
  public:
    class iter {
        T at_, step_, end_;

      public:
        ET_RANGE_FN iter(T at, T step, T end) : at_(at), step_(step), end_(end) {}
        ET_RANGE_FN T operator*() const { return at_; }
        ET_RANGE_FN iter& operator++() {
            at_ += step_;
            return *this;
        }
        // compared against the end sentinel only: true while the walk has not passed the end
        ET_RANGE_FN bool operator!=(const iter&) const {
            return step_ > T(0) ? at_ < end_ : at_ > end_;
        }
    };
    class step_range_proxy {
        T begin_, end_, step_;

      public:
        ET_RANGE_FN step_range_proxy(T b, T e, T s) : begin_(b), end_(e), step_(s) {}
        ET_RANGE_FN iter begin() const { return iter(begin_, step_, end_); }
        ET_RANGE_FN iter end() const { return iter(end_, step_, end_); }
    };

    ET_RANGE_FN range_proxy(T b, T e) : begin_(b), end_(e) {}
    ET_RANGE_FN step_range_proxy step(T s) const { return step_range_proxy(begin_, end_, s); }
    ET_RANGE_FN iter begin() const { return iter(begin_, T(1), end_); }
    ET_RANGE_FN iter end() const { return iter(end_, T(1), end_); }

  private:
    T begin_, end_;
};

template <typename T> ET_RANGE_FN range_proxy<T> range(T begin, T end) { return {begin, end}; }

template <typename C> auto indices(const C& cont) -> range_proxy<decltype(cont.size())> {
    return {0, cont.size()};
}
template <typename T, std::size_t N> ET_RANGE_FN range_proxy<std::size_t> indices(T (&)[N]) {
    return {0, N};
}

template <typename T> using step_range = typename range_proxy<T>::step_range_proxy;

#if defined(__CUDACC__)
template <typename T> __device__ step_range<T> grid_stride_range(T begin, T end) {
    begin += blockDim.x * blockIdx.x + threadIdx.x;
    return range(begin, end).step(static_cast<T>(gridDim.x * blockDim.x));
}
template <typename T> __device__ step_range<T> block_stride_range(T begin, T end) {
    begin += threadIdx.x;
    return range(begin, end).step(static_cast<T>(blockDim.x));
}
template <typename T> __device__ step_range<T> warp_stride_range(T begin, T end) {
    begin += threadIdx.x % 32;
    return range(begin, end).step(T(32));
}
#endif

}  // namespace culib
