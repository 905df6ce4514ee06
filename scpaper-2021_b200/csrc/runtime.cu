// Host-side runtime of the library: status strings, the per-device error word, the
// tensor-map encoder (driver entry point fetched at run time, so the library does not
// link against libcuda) and the host validators of the pruned-weight index arrays.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace et {

namespace {

constexpr int kMaxDevices = 64;

// Written by kernels whose bounded waits ran out (first code wins until it is read).
__device__ int g_device_error_word = 0;

struct PerDevice {
    int* err_word = nullptr;
    int sm_count = 0;
    std::atomic<bool> ready{false};  // published with release order after the fields above
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mutex;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::atomic<EncodeTiledFn> g_encode{nullptr};

PerDevice* current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    PerDevice* pd = &g_dev[dev];
    if (pd->ready.load(std::memory_order_acquire)) return pd;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (pd->ready.load(std::memory_order_relaxed)) return pd;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_error_word) != cudaSuccess) return nullptr;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return nullptr;
    pd->err_word = static_cast<int*>(p);
    pd->sm_count = sms;
    pd->ready.store(true, std::memory_order_release);
    return pd;
}

}  // namespace

namespace {
std::atomic<long long> g_launches{0};
bool g_pdl = true;
}
bool pdl_enabled() { return g_pdl; }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
void set_pdl_enabled(bool on) { g_pdl = on; }

int* device_error_word() {
    PerDevice* pd = current_device();
    return pd ? pd->err_word : nullptr;
}

int sm_count() {
    PerDevice* pd = current_device();
    return pd ? pd->sm_count : 0;
}

namespace {
int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle);
}

int make_tensor_map_f16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box,
                        CUtensorMapSwizzle swizzle) {
    return make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base, rank, dims, strides_bytes,
                           box, swizzle);
}

int make_tensor_map_f32(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box,
                        CUtensorMapSwizzle swizzle) {
    return make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes,
                           box, swizzle);
}

namespace {
int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle) {
    EncodeTiledFn encode = g_encode.load(std::memory_order_acquire);
    if (!encode) {
        std::lock_guard<std::mutex> lock(g_mutex);
        encode = g_encode.load(std::memory_order_relaxed);
        if (!encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) !=
                    cudaSuccess ||
                qres != cudaDriverEntryPointSuccess || fn == nullptr)
                return ET_ERR_CUDA;
            encode = reinterpret_cast<EncodeTiledFn>(fn);
            g_encode.store(encode, std::memory_order_release);
        }
    }
    if (rank < 2 || rank > 3) return ET_ERR_INVALID_ARG;
    if (!aligned16(base)) return ET_ERR_ALIGNMENT;
    cuuint64_t gdims[3];
    cuuint64_t gstrides[2];
    cuuint32_t gbox[3];
    cuuint32_t estr[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
    }
    for (int i = 0; i + 1 < rank; ++i) {
        if (strides_bytes[i] % 16 != 0) return ET_ERR_ALIGNMENT;
        gstrides[i] = strides_bytes[i];
    }
    CUresult r = encode(map, dtype, static_cast<cuuint32_t>(rank),
                          const_cast<void*>(base), gdims, gstrides, gbox, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ET_OK : ET_ERR_CUDA;
}
}  // namespace

}  // namespace et

extern "C" {

const char* et_status_string(int status) {
    switch (status) {
        case ET_OK: return "ok";
        case ET_ERR_INVALID_ARG: return "invalid argument";
        case ET_ERR_ALIGNMENT: return "pointer or leading dimension not 16-byte aligned";
        case ET_ERR_SHAPE: return "unsupported shape";
        case ET_ERR_INDEX: return "corrupt index array";
        case ET_ERR_CUDA: return "CUDA call failed";
        case ET_ERR_WORKSPACE: return "scratch buffer missing or too small";
        case ET_ERR_DEVICE_TIMEOUT: return "a kernel gave up on a bounded wait";
        case ET_ERR_NO_DEVICE: return "no usable sm_100 device is current";
        default: return "unknown status";
    }
}

#ifdef ET_TEST_HOOKS
// Test hook: 0 = plain launches, 1 = programmatic dependent launches (default).
void et_debug_set_pdl(int on) { et::set_pdl_enabled(on != 0); }
#endif  // ET_TEST_HOOKS

long long et_launch_count(void) { return et::g_launches.load(std::memory_order_relaxed); }

int et_version(void) { return 100; }
int et_built_for_sm(void) { return 100; }

int et_device_error(int* code) {
    if (!code) return ET_ERR_INVALID_ARG;
    int* word = et::device_error_word();
    if (!word) return ET_ERR_NO_DEVICE;
    if (cudaDeviceSynchronize() != cudaSuccess) return ET_ERR_CUDA;
    int v = 0;
    if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return ET_ERR_CUDA;
    if (v != 0) {
        int zero = 0;
        if (cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess)
            return ET_ERR_CUDA;
    }
    *code = v;
    return ET_OK;
}

// ---- host validators of index arrays ----------------------------------------------------

int et_validate_tile_mat(const int32_t* row_ptr, const int32_t* row_off, int nnz_tiles, int in,
                         int out) {
    if (!row_ptr || (nnz_tiles > 0 && !row_off) || in <= 0 || out <= 0 || nnz_tiles < 0)
        return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16) return ET_ERR_SHAPE;
    const int nbr = out / 16, nbc = in / 16;
    if (row_ptr[0] != 0 || row_ptr[nbr] != nnz_tiles) return ET_ERR_INDEX;
    for (int br = 0; br < nbr; ++br) {
        // monotone and inside the stored range BEFORE any row_off entry is read
        if (row_ptr[br + 1] < row_ptr[br] || row_ptr[br + 1] > nnz_tiles) return ET_ERR_INDEX;
        for (int i = row_ptr[br]; i < row_ptr[br + 1]; ++i) {
            if (row_off[i] < 0 || row_off[i] >= nbc) return ET_ERR_INDEX;
            if (i > row_ptr[br] && row_off[i] <= row_off[i - 1]) return ET_ERR_INDEX;
        }
    }
    return ET_OK;
}

int et_validate_id_list(const int32_t* ids, int n, int limit, int require_sorted) {
    if (n < 0 || limit <= 0 || (n > 0 && !ids)) return ET_ERR_INVALID_ARG;
    for (int i = 0; i < n; ++i) {
        if (ids[i] < 0 || ids[i] >= limit) return ET_ERR_INDEX;
        if (require_sorted && i > 0 && ids[i] <= ids[i - 1]) return ET_ERR_INDEX;
    }
    return ET_OK;
}

int et_validate_1x16(const int32_t* tile_idx, const int32_t* row_idx, int nvec, int in, int out) {
    if (!tile_idx || (nvec > 0 && !row_idx) || in <= 0 || out <= 0 || nvec < 0)
        return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16) return ET_ERR_SHAPE;
    const int nset = out / 16, npart = in / 16;
    int prev_end = 0;
    for (int r = 0; r < nset; ++r) {
        const int32_t* t = tile_idx + (size_t)r * (npart + 1);
        if (t[0] != prev_end) return ET_ERR_INDEX;
        for (int p = 0; p < npart; ++p) {
            if (t[p + 1] < t[p] || t[p + 1] - t[p] > 16) return ET_ERR_INDEX;
            for (int i = t[p]; i < t[p + 1]; ++i) {
                if (i >= nvec) return ET_ERR_INDEX;
                if (row_idx[i] / 16 != r || row_idx[i] < 0) return ET_ERR_INDEX;
                if (i > t[p] && row_idx[i] <= row_idx[i - 1]) return ET_ERR_INDEX;
            }
        }
        prev_end = t[npart];
    }
    return prev_end == nvec ? ET_OK : ET_ERR_INDEX;
}

int et_validate_csr(const int32_t* indptr, const int32_t* indices, int nnz, int in, int out) {
    if (!indptr || (nnz > 0 && !indices) || in <= 0 || out <= 0 || nnz < 0)
        return ET_ERR_INVALID_ARG;
    if (indptr[0] != 0 || indptr[out] != nnz) return ET_ERR_INDEX;
    for (int o = 0; o < out; ++o) {
        if (indptr[o + 1] < indptr[o] || indptr[o + 1] > nnz) return ET_ERR_INDEX;
        for (int i = indptr[o]; i < indptr[o + 1]; ++i) {
            if (indices[i] < 0 || indices[i] >= in) return ET_ERR_INDEX;
            if (i > indptr[o] && indices[i] <= indices[i - 1]) return ET_ERR_INDEX;
        }
    }
    return ET_OK;
}

}  // extern "C"
