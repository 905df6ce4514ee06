// Wall-clock timers with the reference's names (lib/wtime.h:4-35): wtime synchronises the
// device after every repetition, wtime_new once at the end.  Both return microseconds per
// repetition.
#pragma once
#include <cuda_runtime.h>

#include <chrono>

template <typename F, typename... Args> double wtime(const int reps, F&& f, Args&&... args) {
    using clk = std::chrono::steady_clock;
    double total = 0;
    for (int i = 0; i < reps; ++i) {
        auto t0 = clk::now();
        f(args...);
        cudaDeviceSynchronize();
        total += std::chrono::duration<double, std::micro>(clk::now() - t0).count();
    }
    return total / reps;
}

template <typename F, typename... Args> double wtime_new(const int reps, F&& f, Args&&... args) {
    using clk = std::chrono::steady_clock;
    auto t0 = clk::now();
    for (int i = 0; i < reps; ++i) f(args...);
    cudaDeviceSynchronize();
    return std::chrono::duration<double, std::micro>(clk::now() - t0).count() / reps;
}
