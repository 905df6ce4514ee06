// Wall-clock timers with the reference's names and call forms (lib/wtime.h:4-35).
//   wtime(times, action, prep):     prep() runs untimed before every repetition, action() is
//                                   timed on its own; nothing synchronises the device unless
//                                   the caller's action does.
//   wtime_new(times, action, end):  `times` back-to-back action() calls, then end() once (the
//                                   reference's drivers pass a device synchronisation there),
//                                   all inside one timed region.
// Both return microseconds per repetition.
#pragma once
#include <chrono>

#include "range.hpp"

template <typename _Action, typename _Prep>
double wtime(const int times, _Action action, _Prep prep) {
    using clk = std::chrono::steady_clock;
    double total = 0.0;
    for (int i = 0; i < times; ++i) {
        prep();
        const auto t0 = clk::now();
        action();
        total += std::chrono::duration<double, std::micro>(clk::now() - t0).count();
    }
    return total / times;
}

template <typename _Action, typename _End>
double wtime_new(const int times, _Action action, _End end) {
    using clk = std::chrono::steady_clock;
    const auto t0 = clk::now();
    for (int i = 0; i < times; ++i) action();
    end();
    return std::chrono::duration<double, std::micro>(clk::now() - t0).count() / times;
}
