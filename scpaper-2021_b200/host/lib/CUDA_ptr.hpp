// culib::CUDA_ptr<T>: owning device buffer with the reference's constructors and members
// (lib/CUDA_ptr.hpp:10-69): size ctor zero-fills, pointer ctor copies from host OR device
// memory, vector ctor uploads, (size, value) ctor fills, copy ctor deep-copies on the
// device, move ctor steals.  Filling is done with a host staging copy instead of the
// reference's <<<256,1024>>> kernel: it only runs at set-up time.
#pragma once
#include <cstddef>
#include <utility>
#include <vector>

#include "utils.h"

namespace culib {

template <typename T> class CUDA_ptr {
    T* ptr = nullptr;

  public:
    std::size_t size = 0;

    CUDA_ptr() = delete;
    // An empty buffer still owns one element's worth of memory (so get() is never null), but
    // copies, fills and clears move exactly `size` elements: nothing is read from an empty source.
    explicit CUDA_ptr(const std::size_t n) : size(n) {
        cudaChk(cudaMalloc(reinterpret_cast<void**>(&ptr), alloc_bytes()));
        cudaChk(cudaMemset(ptr, 0, alloc_bytes()));
    }
    CUDA_ptr(const T* src, const std::size_t n) : size(n) {
        cudaChk(cudaMalloc(reinterpret_cast<void**>(&ptr), alloc_bytes()));
        if (n) cudaChk(cudaMemcpy(ptr, src, bytes(), cudaMemcpyDefault));
    }
    CUDA_ptr(const std::vector<T>& v) : size(v.size()) {
        cudaChk(cudaMalloc(reinterpret_cast<void**>(&ptr), alloc_bytes()));
        if (size) cudaChk(cudaMemcpy(ptr, v.data(), bytes(), cudaMemcpyHostToDevice));
    }
    CUDA_ptr(const std::size_t n, const T val) : size(n) {
        cudaChk(cudaMalloc(reinterpret_cast<void**>(&ptr), alloc_bytes()));
        set(val);
    }
    CUDA_ptr(const CUDA_ptr<T>& o) : size(o.size) {
        cudaChk(cudaMalloc(reinterpret_cast<void**>(&ptr), alloc_bytes()));
        if (size) cudaChk(cudaMemcpy(ptr, o.ptr, bytes(), cudaMemcpyDeviceToDevice));
    }
    CUDA_ptr(CUDA_ptr<T>&& o) noexcept : ptr(o.ptr), size(o.size) { o.ptr = nullptr; }
    CUDA_ptr& operator=(const CUDA_ptr&) = delete;
    CUDA_ptr& operator=(CUDA_ptr&& o) noexcept {
        if (this != &o) {
            util::cuda_free_safe(ptr);
            ptr = o.ptr;
            size = o.size;
            o.ptr = nullptr;
        }
        return *this;
    }
    ~CUDA_ptr() { util::cuda_free_safe(ptr); }

    void clear() { cudaChk(cudaMemset(ptr, 0, alloc_bytes())); }
    T* get() { return ptr; }
    T* get() const { return ptr; }
    void dump(T* dst) const {
        if (size) cudaChk(cudaMemcpy(dst, ptr, bytes(), cudaMemcpyDeviceToHost));
    }
    std::vector<T> to_host() const {
        std::vector<T> h(size);
        if (size) dump(h.data());
        return h;
    }
    void set(const T val) {
        if (size == 0) return;
        std::vector<T> h(size, val);
        cudaChk(cudaMemcpy(ptr, h.data(), bytes(), cudaMemcpyHostToDevice));
    }

  private:
    std::size_t bytes() const { return sizeof(T) * size; }
    std::size_t alloc_bytes() const { return sizeof(T) * (size ? size : 1); }
};

}  // namespace culib
