// Error macro, fp16 constants and small helpers with the names the reference drivers use
// (lib/utils.h:32-33, lib/utils.cu:28-35).  Unlike the reference, a failing CUDA call or a
// failing library status throws std::runtime_error instead of calling exit(1), so a host
// application (or a test) can observe it.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <limits>
#include <stdexcept>
#include <string>

// the C ABI header: beside this tree in the repository layout, else on the include path
#if __has_include("../../../include/et_b200.h")
#include "../../../include/et_b200.h"
#else
#include <et_b200.h>
#endif

namespace culib {
namespace util {

inline void cuda_check(cudaError_t e, const char* file, int line) {
    if (e != cudaSuccess)
        throw std::runtime_error(std::string(file) + ":" + std::to_string(line) + ": " +
                                 cudaGetErrorString(e));
}

inline void et_check(int status, const char* what) {
    if (status != ET_OK)
        throw std::runtime_error(std::string(what) + ": " + et_status_string(status));
}

template <typename T> void cuda_free_safe(T*& p) {
    if (p != nullptr) cudaFree(p);
    p = nullptr;
}

inline void sync_streams(cudaStream_t* streams, int n) {
    for (int i = 0; i < n; ++i) cuda_check(cudaStreamSynchronize(streams[i]), __FILE__, __LINE__);
}

template <bool C, typename A, typename B> struct type_if { using type = A; };
template <typename A, typename B> struct type_if<false, A, B> { using type = B; };

// fp32 -> fp16 conversion of a host array into a device buffer
inline void to_half_devptr(half* dst, const float* src_host, size_t n) {
    std::string tmp(n * sizeof(half), '\0');
    half* h = reinterpret_cast<half*>(&tmp[0]);
    for (size_t i = 0; i < n; ++i) h[i] = __float2half_rn(src_host[i]);
    cuda_check(cudaMemcpy(dst, h, n * sizeof(half), cudaMemcpyHostToDevice), __FILE__, __LINE__);
}

}  // namespace util
}  // namespace culib

#define cudaChk(call) ::culib::util::cuda_check((call), __FILE__, __LINE__)
#define etChk(call) ::culib::util::et_check((call), #call)

#define half_zero __float2half_rn(0.0f)
#define half_one __float2half_rn(1.0f)
#define half_ninf __float2half_rn(-std::numeric_limits<float>::infinity())

inline et_half* et_ptr(half* p) { return reinterpret_cast<et_half*>(p); }
inline const et_half* et_ptr(const half* p) { return reinterpret_cast<const et_half*>(p); }
