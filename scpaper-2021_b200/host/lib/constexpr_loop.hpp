// make_loop<F, T, N>(): calls the functors F<0, T>() ... F<N-1, T>() in ascending order, the
// compile-time loop the reference's sweep drivers use to walk a list of weight formats
// (lib/constexpr_loop.hpp, e.g. Linear/test/benchmark.cu:39-48).  With T = void, run() just
// calls them; otherwise run(op) folds their results from the left: op(op(f0, f1), f2) ...
#pragma once
#include <cstddef>
#include <utility>

namespace et_host {
template <template <std::size_t, typename> class F, typename T, std::size_t N> class unrolled_loop {
    template <typename Op, std::size_t... I> T fold(const Op& op, std::index_sequence<I...>) {
        T acc = F<0, T>()();
        ((I == 0 ? void() : void(acc = op(acc, F<I, T>()()))), ...);
        return acc;
    }

  public:
    template <typename Op> T run(const Op& op) { return fold(op, std::make_index_sequence<N>{}); }
};
template <template <std::size_t, typename> class F, std::size_t N> class unrolled_loop<F, void, N> {
    template <std::size_t... I> void each(std::index_sequence<I...>) { (F<I, void>()(), ...); }

  public:
    void run() { each(std::make_index_sequence<N>{}); }
};
}  // namespace et_host

template <template <std::size_t, typename> class F, typename T, int N> constexpr auto make_loop() {
    static_assert(N > 0);
    return et_host::unrolled_loop<F, T, static_cast<std::size_t>(N)>();
}
