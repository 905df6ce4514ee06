// Instruction-rate probes (test hooks; compiled only with -DET_TEST_HOOKS).
//
// The plan-time choices of the tile-pruned Linear rest on two machine figures: how long one
// tcgen05.mma of a narrow shape (M x N x 16 with N as small as 16, the width of one weight
// tile) occupies the tensor pipe, and what the warp-level mma.sync.m16n8k16 path sustains
// per SM.  These kernels measure both with the SM's cycle counter; operands hold small
// constants, results are discarded.
#ifdef ET_TEST_HOOKS
#include "common.cuh"

namespace et {
namespace {

// ---- tcgen05: cycles per product --------------------------------------------------------
// One CTA.  Thread 0 issues `count` products D[M x N] (+)= A[M x 16] . B[N x 16]^T with A
// and B in shared memory, rotating over `nacc` accumulators (column offset i * N), then
// commits and waits (bounded).  a_step != 0 walks A over the four 16-column slabs of a
// 128-byte-swizzled 64-column block, as a kernel that picks the activation slab by
// descriptor address would.
__global__ void __launch_bounds__(128, 1)
tc_probe_kernel(int M, int N, int nacc, int count, int a_step, long long* cycles, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sA = smem;              // 128 rows x 128 bytes (64 fp16), 128-byte swizzle
    uint8_t* sB = smem + 16384;      // up to 256 rows x 32 bytes, 32-byte swizzle
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 16384 + 8192);
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot + 1);
    for (int i = threadIdx.x; i < (16384 + 8192) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(smem)[i] = 0x2C002C00u;  // 0.0625 in both halves
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async_smem();
    if (threadIdx.x < 32) {
        tmem_alloc(slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = make_idesc_f16(M, N, 0, 0);
        const uint64_t a_desc = make_smem_desc(smem_u32(sA), 16, 1024, SWZ_128B);
        const uint64_t b_desc = make_smem_desc(smem_u32(sB), 16, 256, SWZ_32B);
        const long long t0 = clock64();
        int acc = 0;
        for (int i = 0; i < count; ++i) {
            const uint64_t ad = a_step ? a_desc + static_cast<uint64_t>((i & 3) * 2) : a_desc;
            mma_f16_ss(tmem_base + acc * N, ad, b_desc, idesc, i >= nacc ? 1u : 0u);
            if (++acc == nacc) acc = 0;
        }
        mma_commit(bar);
        const bool ok = mbar_wait_bounded(bar, 0, abort_flag);
        const long long t1 = clock64();
        *cycles = t1 - t0;
        *status = ok ? 0 : 1;
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tmem_base, 512);
}

// ---- mma.sync: multiply-accumulates per clock per SM -------------------------------------
// Every warp runs `iters` rounds of 16 products against 16 independent accumulators (one
// 16 x 16 weight tile applied to 128 tokens).  MODE 0: both operands stay in registers.
// MODE 1: the token operand of every product comes from shared memory through ldmatrix
// (a 128 x 64 fp16 slab in the 128-byte-swizzled layout a tiled bulk copy produces), the
// slab column rotating per round; the weight operand is re-read from global memory per round.
template <int MODE>
__global__ void __launch_bounds__(512)
mma_sync_probe_kernel(int iters, const uint32_t* __restrict__ wtiles, long long* cycles,
                      float* sink) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int lane = threadIdx.x & 31;
    if (MODE == 1) {
        for (int i = threadIdx.x; i < 3 * 16384 / 4; i += blockDim.x)
            reinterpret_cast<uint32_t*>(smem)[i] = 0x2C002C00u;
        __syncthreads();
    }
    float c[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) c[j][k] = 0.f;
    uint32_t a[4] = {0x2C002C00u, 0x2C002C00u, 0x2C002C00u, 0x2C002C00u};
    uint32_t b0 = 0x2C002C00u + lane, b1 = 0x2C002C00u;
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        if (MODE == 1) {
            // weight tile: 16 x 16 fp16 row-major, fragment read straight from global memory
            const uint32_t* wt = wtiles + ((it + (threadIdx.x >> 5)) & 63) * 128;
            a[0] = __ldg(wt + (lane >> 2) * 8 + (lane & 3));
            a[1] = __ldg(wt + ((lane >> 2) + 8) * 8 + (lane & 3));
            a[2] = __ldg(wt + (lane >> 2) * 8 + 4 + (lane & 3));
            a[3] = __ldg(wt + ((lane >> 2) + 8) * 8 + 4 + (lane & 3));
            const int slab = it % 12;  // (stage, 16-column slab) of three staged 64-column blocks
            const uint32_t base = smem_u32(smem) + (slab >> 2) * 16384;
            const int kb = slab & 3;
            // lane -> (token row within 16, which 8-column half)
            const int row_in = (lane & 7) + ((lane >> 4) << 3);
            const int chunk = kb * 2 + ((lane >> 3) & 1);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int row = j * 16 + row_in;
                uint32_t r[4];
                ldmatrix_x4(r, base + row * 128 + ((chunk ^ (row & 7)) << 4));
                mma_m16n8k16(c[2 * j], a, r[0], r[1]);
                mma_m16n8k16(c[2 * j + 1], a, r[2], r[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) mma_m16n8k16(c[j], a, b0, b1);
        }
    }
    const long long t1 = clock64();
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) s += c[j][0] + c[j][1] + c[j][2] + c[j][3];
    if (s == 123.456f) sink[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
}

// ---- both paths at once -------------------------------------------------------------------
// One CTA per SM.  Thread 0 of each of the first `issuers` warps issues `count` tcgen05
// products (128 x 16 x 16, own accumulator columns); the following `sync_warps` warps run
// `iters` rounds of 16 register-operand mma.sync products.  Reports the cycles the slowest
// issuer and the slowest mma.sync warp took, so that the rates with and without the other
// path can be compared.
__global__ void __launch_bounds__(512, 1)
mixed_probe_kernel(int issuers, int count, int sync_warps, int iters, int commit_every,
                   long long* cycles, int* status, float* sink) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sA = smem;
    uint8_t* sB = smem + 16384;
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 16384 + 8192);  // one per issuer (<= 8)
    uint64_t* side_bar = bar + 8;  // receives the periodic commits; nobody waits on it
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot + 1);
    long long* s_cycles = reinterpret_cast<long long*>(smem + 16384 + 8192 + 128);  // [16]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < (16384 + 8192) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(smem)[i] = 0x2C002C00u;
    if (threadIdx.x < 16) s_cycles[threadIdx.x] = 0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) mbar_init(&bar[i], 1);
        mbar_init(side_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        tmem_alloc(slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *slot;
    bool ok = true;
    if (warp < issuers) {
        if (lane == 0 && count > 0) {
            const uint32_t idesc = make_idesc_f16(128, 16, 0, 0);
            const uint64_t a_desc = make_smem_desc(smem_u32(sA), 16, 1024, SWZ_128B);
            const uint64_t b_desc = make_smem_desc(smem_u32(sB), 16, 256, SWZ_32B);
            const long long t0 = clock64();
            // groups of `commit_every` products, each followed by one commit (no division in the
            // loop: a single thread's dependent integer chain would dominate the timing)
            const int group = commit_every > 0 ? commit_every : count;
            for (int i = 0; i < count; i += group) {
                const int end = i + group < count ? i + group : count;
                for (int j = i; j < end; ++j)
                    mma_f16_ss(tmem_base + warp * 64 + (j & 3) * 16,
                               a_desc + static_cast<uint64_t>((j & 3) * 2), b_desc, idesc,
                               j >= 4 ? 1u : 0u);
                if (commit_every > 0) mma_commit(side_bar);
            }
            mma_commit(&bar[warp]);
            ok = mbar_wait_bounded(&bar[warp], 0, abort_flag);
            s_cycles[warp] = clock64() - t0;
        }
    } else if (warp < issuers + sync_warps && iters > 0) {
        float c[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) c[j][k] = 0.f;
        const uint32_t a[4] = {0x2C002C00u, 0x2C002C00u, 0x2C002C00u, 0x2C002C00u};
        const uint32_t b0 = 0x2C002C00u + lane, b1 = 0x2C002C00u;
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int j = 0; j < 16; ++j) mma_m16n8k16(c[j], a, b0, b1);
        }
        const long long t1 = clock64();
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum += c[j][0] + c[j][1] + c[j][2] + c[j][3];
        if (sum == 123.456f) sink[threadIdx.x] = sum;
        if (lane == 0) s_cycles[8 + ((warp - issuers) & 7)] = t1 - t0;
    }
    if (!ok) *status = 1;
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        long long tc = 0, ms = 0;
        for (int i = 0; i < 8; ++i) {
            tc = s_cycles[i] > tc ? s_cycles[i] : tc;
            ms = s_cycles[8 + i] > ms ? s_cycles[8 + i] : ms;
        }
        cycles[0] = tc;
        cycles[1] = ms;
    }
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace
}  // namespace et

extern "C" {

// Cycles one tcgen05.mma (kind::f16, cta_group::1) of shape m x n x 16 occupies the tensor
// pipe when `count` of them are issued back to back over `nacc` accumulators.
int et_debug_probe_tcgen05(int m, int n, int nacc, int count, int a_step, double* cycles_per_product) {
    if (!cycles_per_product || (m != 64 && m != 128) || n < 16 || n > 256 || (n & 15) || nacc < 1 ||
        nacc * n > 512 || count < nacc || count > (1 << 20))
        return ET_ERR_INVALID_ARG;
    long long* d_cycles = nullptr;
    int* d_status = nullptr;
    if (cudaMalloc(&d_cycles, sizeof(long long)) != cudaSuccess) return ET_ERR_CUDA;
    if (cudaMalloc(&d_status, sizeof(int)) != cudaSuccess) {
        cudaFree(d_cycles);
        return ET_ERR_CUDA;
    }
    const int smem = 16384 + 8192 + 64 + 1024;
    int rc = ET_OK;
    et::tc_probe_kernel<<<1, 128, smem>>>(m, n, nacc, count, a_step, d_cycles, d_status);
    long long cyc = 0;
    int st = 0;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(&cyc, d_cycles, sizeof(cyc), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(&st, d_status, sizeof(st), cudaMemcpyDeviceToHost) != cudaSuccess)
        rc = ET_ERR_CUDA;
    else if (st != 0)
        rc = ET_ERR_DEVICE_TIMEOUT;
    else
        *cycles_per_product = static_cast<double>(cyc) / count;
    cudaFree(d_cycles);
    cudaFree(d_status);
    return rc;
}

// Multiply-accumulates per clock per SM sustained by mma.sync.m16n8k16 (fp16 in, fp32
// accumulate) with `warps` warps per CTA and `ctas_per_sm` CTAs per SM on every SM.
// mode 0: operands in registers; mode 1: token operand through ldmatrix from shared memory.
int et_debug_probe_mma_sync(int warps, int ctas_per_sm, int iters, int mode,
                            double* mac_per_clk_per_sm) {
    if (!mac_per_clk_per_sm || warps < 1 || warps > 16 || ctas_per_sm < 1 || warps * ctas_per_sm > 16 ||
        iters < 1 || iters > (1 << 20) || mode < 0 || mode > 1)
        return ET_ERR_INVALID_ARG;
    const int sms = et::sm_count();
    if (sms <= 0) return ET_ERR_NO_DEVICE;
    const int grid = sms * ctas_per_sm;
    long long* d_cycles = nullptr;
    float* d_sink = nullptr;
    uint32_t* d_w = nullptr;
    if (cudaMalloc(&d_cycles, grid * sizeof(long long)) != cudaSuccess) return ET_ERR_CUDA;
    if (cudaMalloc(&d_sink, 512 * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&d_w, 64 * 512) != cudaSuccess) {
        cudaFree(d_cycles);
        cudaFree(d_sink);
        return ET_ERR_CUDA;
    }
    cudaMemset(d_w, 0x2C, 64 * 512);
    const int smem = mode == 1 ? 3 * 16384 + 1024 : 0;
    int rc = ET_OK;
    if (mode == 1) {
        if (cudaFuncSetAttribute(et::mma_sync_probe_kernel<1>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            rc = ET_ERR_CUDA;
        else
            et::mma_sync_probe_kernel<1><<<grid, warps * 32, smem>>>(iters, d_w, d_cycles, d_sink);
    } else {
        et::mma_sync_probe_kernel<0><<<grid, warps * 32, 0>>>(iters, d_w, d_cycles, d_sink);
    }
    if (rc == ET_OK) {
        long long* h = new long long[grid];
        if (cudaDeviceSynchronize() != cudaSuccess ||
            cudaMemcpy(h, d_cycles, grid * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess) {
            rc = ET_ERR_CUDA;
        } else {
            double sum = 0;
            for (int i = 0; i < grid; ++i) sum += static_cast<double>(h[i]);
            const double mean_cycles = sum / grid;
            const double macs_per_sm = static_cast<double>(warps) * ctas_per_sm * iters * 16.0 * 2048.0;
            *mac_per_clk_per_sm = macs_per_sm / mean_cycles;
        }
        delete[] h;
    }
    cudaFree(d_cycles);
    cudaFree(d_sink);
    cudaFree(d_w);
    return rc;
}

// tcgen05 (128 x 16 x 16 products from `issuers` threads) and mma.sync (`sync_warps` warps)
// in the same CTAs at the same time, one CTA per SM.  Outputs: cycles per tcgen05 product
// (all issuers together) and multiply-accumulates per clock per SM of the mma.sync warps;
// either side may be switched off with count = 0 / iters = 0 for the solo figures.
// commit_every > 0: every issuer also issues a tcgen05.commit after that many products (what a
// pipelined kernel does to release an operand stage).
int et_debug_probe_mixed(int issuers, int count, int sync_warps, int iters, int commit_every,
                         double* cycles_per_product, double* mac_per_clk_per_sm) {
    if (!cycles_per_product || !mac_per_clk_per_sm || issuers < 1 || issuers > 8 || sync_warps < 0 ||
        sync_warps > 8 || count < 0 || count > (1 << 20) || iters < 0 || iters > (1 << 20))
        return ET_ERR_INVALID_ARG;
    const int sms = et::sm_count();
    if (sms <= 0) return ET_ERR_NO_DEVICE;
    long long* d_cycles = nullptr;
    int* d_status = nullptr;
    float* d_sink = nullptr;
    if (cudaMalloc(&d_cycles, 2 * sizeof(long long)) != cudaSuccess) return ET_ERR_CUDA;
    if (cudaMalloc(&d_status, sizeof(int)) != cudaSuccess || cudaMalloc(&d_sink, 512 * 4) != cudaSuccess) {
        cudaFree(d_cycles);
        cudaFree(d_status);
        return ET_ERR_CUDA;
    }
    cudaMemset(d_status, 0, sizeof(int));
    const int smem = 16384 + 8192 + 128 + 128 + 1024;
    et::mixed_probe_kernel<<<sms, (issuers + sync_warps) * 32, smem>>>(issuers, count, sync_warps, iters,
                                                                      commit_every, d_cycles, d_status,
                                                                      d_sink);
    long long cyc[2] = {0, 0};
    int st = 0, rc = ET_OK;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(cyc, d_cycles, sizeof(cyc), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(&st, d_status, sizeof(st), cudaMemcpyDeviceToHost) != cudaSuccess)
        rc = ET_ERR_CUDA;
    else if (st != 0)
        rc = ET_ERR_DEVICE_TIMEOUT;
    else {
        *cycles_per_product = count > 0 ? static_cast<double>(cyc[0]) / (static_cast<double>(count) * issuers) : 0.0;
        *mac_per_clk_per_sm =
            iters > 0 && cyc[1] > 0 ? static_cast<double>(sync_warps) * iters * 16.0 * 2048.0 / cyc[1] : 0.0;
    }
    cudaFree(d_cycles);
    cudaFree(d_status);
    cudaFree(d_sink);
    return rc;
}

}  // extern "C"
#endif  // ET_TEST_HOOKS
