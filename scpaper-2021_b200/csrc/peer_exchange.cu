// Head-parallel layer: the sum of the ranks' partial attention outputs, the residual add and
// the first LayerNorm as kernels over PEER MEMORY instead of a library all-reduce.
//
// Every rank owns T / world token rows; a rank's partial [T, hidden] (fp16) is written by its
// output projection straight into its exchange buffer, which every other rank has mapped.
// Three kernels per layer and rank, all on the caller's stream:
//   1. signal:  one thread publishes the layer's epoch in every peer's flag word for this rank
//               (release, system scope) once the kernels before it - the projection - are done
//               (a separate small kernel, or the first thing kernel 2 does: `publish_ready`);
//   2. reduce:  the owner waits (bounded) until all ranks' flags show the epoch, PULLS its rows
//               of every rank's partial through the peer mappings (NVLink reads, 16 bytes per
//               lane), sums them in fp32, adds bias and residual, normalises (eps 1e-5, fp32
//               statistics) and writes the fp16 rows into EVERY rank's copy of y (the all-gather,
//               by peer stores); the last CTA publishes the epoch in the second flag set;
//   3. wait:    one small kernel that returns once all ranks' second flags show the epoch; the
//               feed-forward kernels behind it on the stream then read y locally.
// Token-sharded form (`gather` = 0 in kernel 2): the feed-forward block and the second LayerNorm
// act on tokens independently, so a rank may run them on ITS rows only (1 / world of the work)
// and pass the finished rows on: kernel 2 then keeps y local, the rank's feed-forward kernels
// write its rows of the layer output into its own out[slot], hp_allgather_rows_kernel stores them
// into every other rank's out[slot] and publishes the second flag set, kernel 3 waits for it.
// The bytes moved are those of one all-reduce (a reduce-scatter after the output projection, an
// all-gather after the layer); two out buffers alternate from layer to layer, so a rank that is
// already writing layer l + 1's rows never touches rows a slower rank still reads as layer l's.
// Kernels of different ranks wait on one another only across GPUs (one rank per GPU).  For a
// single-GPU emulation of several ranks the caller runs every rank's kernel 1, then every kernel
// 2, then the waits, so that no wait ever has to spin.  Buffer reuse across layers is safe
// without double buffering: a rank overwrites its partial for layer l + 1 only after its own
// feed-forward of layer l, which needed every owner's kernel 2 of layer l, i.e. every read of
// that partial.  Every wait is bounded: when it runs out the kernel records a code in the device
// error word and returns (the output is then garbage and the host sees the code).
#include "common.cuh"
#include "kernels.h"

namespace et {
namespace {

constexpr int PEER_MAX_WORLD = 16;
constexpr uint32_t PEER_POLL_LIMIT = 1u << 21;  // x ~0.5 us per poll: about a second

struct PeerPtrs {
    uint8_t* p[PEER_MAX_WORLD];
};

struct PeerLayout {
    int rows_r;          // token rows owned by a rank
    size_t y_off;        // y [T, hidden] fp16 (the rank's partial [T, hidden] fp16 sits at 0)
    size_t out_off[2];   // two layer-output buffers [T, hidden] fp16 (token-sharded form)
    size_t flags_off;    // int partial_ready[16], rows_ready[16], counters[4]
    size_t total;
};

__host__ __device__ inline PeerLayout peer_layout(int world, int T, int hidden) {
    PeerLayout l;
    l.rows_r = (T + world - 1) / world;
    l.y_off = (static_cast<size_t>(T) * hidden * 2 + 255) & ~static_cast<size_t>(255);
    l.out_off[0] = 2 * l.y_off;
    l.out_off[1] = 3 * l.y_off;
    l.flags_off = 4 * l.y_off;
    l.total = l.flags_off + 256;
    return l;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Last-CTA-done: the CTA's stores are ordered before thread 0's system-scope fence by the CTA
// barrier (one fence per CTA: a system-scope fence costs microseconds, so launches that end with
// this use about one CTA per SM); returns true in thread 0 of the CTA that arrives last (and
// resets the counter for the next launch).
__device__ __forceinline__ bool last_cta_done(int* counter) {
    __syncthreads();
    if (threadIdx.x != 0 || threadIdx.y != 0) return false;
    __threadfence_system();
    const int before = atomicAdd(counter, 1);
    if (before != static_cast<int>(gridDim.x) - 1) return false;
    atomicExch(counter, 0);
    __threadfence_system();
    return true;
}

// Bounded wait until flags[0 .. world) >= epoch; thread i < world polls flag i.
__device__ __forceinline__ bool wait_flags(const int* flags, int world, int epoch, int* s_ok) {
    if (threadIdx.x == 0) *s_ok = 1;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world) {
        bool seen = false;
        for (uint32_t it = 0; it < PEER_POLL_LIMIT; ++it) {
            if (ld_acquire_sys(flags + threadIdx.x) - epoch >= 0) {
                seen = true;
                break;
            }
            __nanosleep(200);
        }
        if (!seen) *s_ok = 0;
    }
    __syncthreads();
    return *s_ok != 0;
}

__global__ void hp_signal_kernel(PeerPtrs peers, int rank, int world, size_t flags_off, int epoch) {
    pdl_launch_dependents();
    pdl_wait();  // the partial is complete: every kernel before this one on the stream has ended
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int d = 0; d < world; ++d)
            st_release_sys(reinterpret_cast<int*>(peers.p[d] + flags_off) + rank, epoch);
    }
}

// One thread per 16-byte vector of an owned row: blockDim = (threads per row: hidden / 8 rounded up
// to a warp multiple, rows per CTA).  Every thread has `world` remote loads in flight at once and
// all rows of the launch are resident together, which is what hides the NVLink round trip.
__global__ void __launch_bounds__(512)
hp_reduce_ln_kernel(PeerPtrs peers, const __half* __restrict__ x, const __half* __restrict__ bias,
                    const __half* __restrict__ gamma, const __half* __restrict__ beta, int rank, int world,
                    int T, int hidden, int epoch, float eps, int publish_ready, int gather, int* err_word) {
    __shared__ int s_ok;
    __shared__ float2 s_part[16][16];  // [row of the CTA][warp of the row]
    const PeerLayout l = peer_layout(world, T, hidden);
    uint8_t* mine = peers.p[rank];
    const int tid = threadIdx.y * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    // publish_ready: this kernel also tells the peers that this rank's partial is complete (the
    // kernels before it on the stream have ended), which saves the separate signal launch
    if (publish_ready && blockIdx.x == 0 && tid == 0) {
        __threadfence_system();
        for (int d = 0; d < world; ++d)
            st_release_sys(reinterpret_cast<int*>(peers.p[d] + l.flags_off) + rank, epoch);
    }
    // bounded wait until every rank's partial is ready: thread i < world polls flag i
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < world) {
        const int* flags = reinterpret_cast<const int*>(mine + l.flags_off);
        bool seen = false;
        for (uint32_t it = 0; it < PEER_POLL_LIMIT; ++it) {
            if (ld_acquire_sys(flags + tid) - epoch >= 0) {
                seen = true;
                break;
            }
            __nanosleep(200);
        }
        if (!seen) s_ok = 0;
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    if (!ok && tid == 0 && err_word) atomicCAS(err_word, 0, DEV_TIMEOUT_PEER);

    const int row0 = rank * l.rows_r;
    const int nrows = (T - row0) < l.rows_r ? (T - row0 > 0 ? T - row0 : 0) : l.rows_r;
    const int vec_per_row = hidden >> 3;
    const int c = threadIdx.x, ty = threadIdx.y;
    const int lane = threadIdx.x & 31, wrow = threadIdx.x >> 5, nwrow = blockDim.x >> 5;
    const float inv_n = 1.0f / static_cast<float>(hidden);
    if (ok)
        for (int base = blockIdx.x * blockDim.y; base < nrows; base += gridDim.x * blockDim.y) {
            const int lrow = base + ty;
            const bool live = lrow < nrows && c < vec_per_row;
            const int row = row0 + lrow;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
            float sum = 0.f, sq = 0.f;
            if (live) {
                const size_t off = static_cast<size_t>(row) * vec_per_row + c;
                for (int s0 = 0; s0 < world; s0 += 4) {  // four ranks' loads in flight together
                    uint4 q[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        q[k] = s0 + k < world ? __ldcg(reinterpret_cast<const uint4*>(peers.p[s0 + k]) + off)
                                              : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const __half2* h = reinterpret_cast<const __half2*>(&q[k]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __half22float2(h[j]);
                            v[2 * j] += f.x;
                            v[2 * j + 1] += f.y;
                        }
                    }
                }
                const uint4 qx = __ldcg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * hidden) + c);
                const __half2* hx = reinterpret_cast<const __half2*>(&qx);
                uint4 qb = make_uint4(0u, 0u, 0u, 0u);
                if (bias != nullptr) qb = __ldg(reinterpret_cast<const uint4*>(bias) + c);
                const __half2* hb = reinterpret_cast<const __half2*>(&qb);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 fx = __half22float2(hx[j]), fb = __half22float2(hb[j]);
                    v[2 * j] += fx.x + fb.x;
                    v[2 * j + 1] += fx.y + fb.y;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    sum += v[j];
                    sq = fmaf(v[j], v[j], sq);
                }
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, d);
                sq += __shfl_xor_sync(0xffffffffu, sq, d);
            }
            if (lane == 0) s_part[ty][wrow] = make_float2(sum, sq);
            __syncthreads();
            float tsum = 0.f, tsq = 0.f;
            for (int k = 0; k < nwrow; ++k) {
                tsum += s_part[ty][k].x;
                tsq += s_part[ty][k].y;
            }
            __syncthreads();  // s_part is rewritten by the next pass
            if (live) {
                const float mean = tsum * inv_n;
                const float rstd = rsqrtf(fmaxf(tsq * inv_n - mean * mean, 0.f) + eps);
                const uint4 qg = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
                const uint4 qt = __ldg(reinterpret_cast<const uint4*>(beta) + c);
                const __half2* hg = reinterpret_cast<const __half2*>(&qg);
                const __half2* ht = reinterpret_cast<const __half2*>(&qt);
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 fg = __half22float2(hg[j]), ft = __half22float2(ht[j]);
                    o[j] = pack_half2(fmaf((v[2 * j] - mean) * rstd, fg.x, ft.x),
                                      fmaf((v[2 * j + 1] - mean) * rstd, fg.y, ft.y));
                }
                const uint4 q = make_uint4(o[0], o[1], o[2], o[3]);
                const size_t off = static_cast<size_t>(row) * vec_per_row + c;
                if (gather) {
                    for (int d = 0; d < world; ++d) *(reinterpret_cast<uint4*>(peers.p[d] + l.y_off) + off) = q;
                } else {
                    *(reinterpret_cast<uint4*>(mine + l.y_off) + off) = q;
                }
            }
        }
    int* counters = reinterpret_cast<int*>(mine + l.flags_off) + 32;
    if (gather) {
        if (last_cta_done(counters + 1)) {
            // published even after a give-up: the peers' waits then end at once and the code in
            // the error word tells the host that this layer's output is not valid
            for (int d = 0; d < world; ++d)
                st_release_sys(reinterpret_cast<int*>(peers.p[d] + l.flags_off) + 16 + rank, epoch);
        }
    }
}

// Token-sharded form: this rank's rows of the layer output (in its own out[slot]) go into every
// other rank's out[slot]; the last CTA publishes the epoch in the second flag set.
__global__ void __launch_bounds__(512)
hp_allgather_rows_kernel(PeerPtrs peers, int rank, int world, int T, int hidden, int epoch, int slot) {
    const PeerLayout l = peer_layout(world, T, hidden);
    const int vec_per_row = hidden >> 3;
    const int row0 = rank * l.rows_r;
    const int nrows = (T - row0) < l.rows_r ? (T - row0 > 0 ? T - row0 : 0) : l.rows_r;
    const size_t total = static_cast<size_t>(nrows) * vec_per_row;
    const size_t base = static_cast<size_t>(row0) * vec_per_row;
    const uint4* src = reinterpret_cast<const uint4*>(peers.p[rank] + l.out_off[slot]) + base;
    pdl_launch_dependents();
    pdl_wait();  // the rows belong to the kernels before this one
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < total;
         v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint4 q = __ldcg(src + v);
        for (int d = 0; d < world; ++d)
            if (d != rank) *(reinterpret_cast<uint4*>(peers.p[d] + l.out_off[slot]) + base + v) = q;
    }
    int* counters = reinterpret_cast<int*>(peers.p[rank] + l.flags_off) + 32;
    if (last_cta_done(counters + 2)) {
        for (int d = 0; d < world; ++d)
            st_release_sys(reinterpret_cast<int*>(peers.p[d] + l.flags_off) + 16 + rank, epoch);
    }
}

__global__ void hp_wait_kernel(const int* flags, int world, int epoch, int* err_word) {
    __shared__ int s_ok;
    pdl_launch_dependents();
    pdl_wait();
    const bool ok = wait_flags(flags, world, epoch, &s_ok);
    if (!ok && threadIdx.x == 0 && err_word) atomicCAS(err_word, 0, DEV_TIMEOUT_PEER);
}

int check_args(void* const* peer_buffers, int rank, int world, int T, int hidden) {
    if (!peer_buffers || world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world || T <= 0)
        return ET_ERR_INVALID_ARG;
    if (hidden <= 0 || hidden % 8 || hidden > 2048) return ET_ERR_SHAPE;
    for (int d = 0; d < world; ++d) {
        if (!peer_buffers[d]) return ET_ERR_INVALID_ARG;
        if (reinterpret_cast<uintptr_t>(peer_buffers[d]) & 255u) return ET_ERR_ALIGNMENT;
    }
    return ET_OK;
}

PeerPtrs pack(void* const* peer_buffers, int world) {
    PeerPtrs p;
    for (int d = 0; d < PEER_MAX_WORLD; ++d) p.p[d] = d < world ? static_cast<uint8_t*>(peer_buffers[d]) : nullptr;
    return p;
}

}  // namespace
}  // namespace et

extern "C" {

int et_peer_buffer_bytes(int world, int T, int hidden, size_t* bytes) {
    if (!bytes || world < 1 || world > et::PEER_MAX_WORLD || T <= 0 || hidden <= 0) return ET_ERR_INVALID_ARG;
    *bytes = et::peer_layout(world, T, hidden).total;
    return ET_OK;
}

int et_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!ptr || !handle || bytes == 0) return ET_ERR_INVALID_ARG;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return ET_ERR_CUDA;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(p);
        return ET_ERR_CUDA;
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return ET_ERR_CUDA;
    }
    memcpy(handle, &h, 64);
    *ptr = p;
    return ET_OK;
}

int et_peer_buffer_open(const unsigned char handle[64], void** ptr) {
    if (!handle || !ptr) return ET_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return ET_ERR_CUDA;
    }
    *ptr = p;
    return ET_OK;
}

int et_peer_buffer_close(void* ptr) {
    if (!ptr) return ET_ERR_INVALID_ARG;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

int et_peer_buffer_destroy(void* ptr) {
    if (!ptr) return ET_ERR_INVALID_ARG;
    return cudaFree(ptr) == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

int et_peer_buffer_y(void* own_buffer, int world, int T, int hidden, et_half** y) {
    if (!own_buffer || !y || world < 1 || world > et::PEER_MAX_WORLD || T <= 0 || hidden <= 0)
        return ET_ERR_INVALID_ARG;
    *y = reinterpret_cast<et_half*>(static_cast<uint8_t*>(own_buffer) + et::peer_layout(world, T, hidden).y_off);
    return ET_OK;
}

int et_peer_buffer_partial(void* own_buffer, et_half** partial) {
    if (!own_buffer || !partial) return ET_ERR_INVALID_ARG;
    *partial = static_cast<et_half*>(own_buffer);
    return ET_OK;
}

int et_hp_signal_partial_fwd(void* const* peer_buffers, int rank, int world, int T, int hidden, int epoch,
                             et_stream stream) {
    int st = et::check_args(peer_buffers, rank, world, T, hidden);
    if (st != ET_OK) return st;
    return et::launch_kernel(et::hp_signal_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                             et::pack(peer_buffers, world), rank, world,
                             et::peer_layout(world, T, hidden).flags_off, epoch) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

int et_peer_buffer_out(void* own_buffer, int world, int T, int hidden, int slot, et_half** out) {
    if (!own_buffer || !out || world < 1 || world > et::PEER_MAX_WORLD || T <= 0 || hidden <= 0 || slot < 0 ||
        slot > 1)
        return ET_ERR_INVALID_ARG;
    *out = reinterpret_cast<et_half*>(static_cast<uint8_t*>(own_buffer) +
                                      et::peer_layout(world, T, hidden).out_off[slot]);
    return ET_OK;
}

int et_hp_allgather_rows_fwd(void* const* peer_buffers, int rank, int world, int T, int hidden, int epoch,
                             int slot, et_stream stream) {
    int st = et::check_args(peer_buffers, rank, world, T, hidden);
    if (st != ET_OK) return st;
    if (slot < 0 || slot > 1) return ET_ERR_INVALID_ARG;
    const int rows_r = (T + world - 1) / world;
    const size_t vecs = static_cast<size_t>(rows_r) * (hidden / 8);
    const int sms = et::sm_count() > 0 ? et::sm_count() : 148;
    const size_t want = (vecs + 511) / 512;
    const int blocks = static_cast<int>(want < 1 ? 1 : (want < static_cast<size_t>(sms) ? want : sms));
    return et::launch_kernel(et::hp_allgather_rows_kernel, dim3(blocks), dim3(512), 0,
                             static_cast<cudaStream_t>(stream), et::pack(peer_buffers, world), rank, world, T,
                             hidden, epoch, slot) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

int et_hp_reduce_layernorm_fwd(void* const* peer_buffers, const et_half* x, const et_half* bias,
                               const et_half* gamma, const et_half* beta, int rank, int world, int T,
                               int hidden, int epoch, int publish_ready, int gather, et_stream stream) {
    int st = et::check_args(peer_buffers, rank, world, T, hidden);
    if (st != ET_OK) return st;
    if (!x || !gamma || !beta) return ET_ERR_INVALID_ARG;
    if (!et::aligned16(x) || !et::aligned16(gamma) || !et::aligned16(beta) || (bias && !et::aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    int* err = et::device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;
    const int rows_r = (T + world - 1) / world;
    const int sms = et::sm_count() > 0 ? et::sm_count() : 148;
    const int tpr = ((hidden / 8 + 31) / 32) * 32;  // threads per row (<= 256)
    int rpb = 384 / tpr;                             // rows per CTA
    rpb = rpb < 1 ? 1 : (rpb > 16 ? 16 : rpb);
    int blocks = (rows_r + rpb - 1) / rpb;
    blocks = blocks < 1 ? 1 : (blocks > 2 * sms ? 2 * sms : blocks);
    const cudaError_t e = et::launch_kernel(
        et::hp_reduce_ln_kernel, dim3(blocks), dim3(tpr, rpb), 0, static_cast<cudaStream_t>(stream),
        et::pack(peer_buffers, world), reinterpret_cast<const __half*>(x), reinterpret_cast<const __half*>(bias),
        reinterpret_cast<const __half*>(gamma), reinterpret_cast<const __half*>(beta), rank, world, T, hidden, epoch,
        1e-5f, publish_ready, gather, err);
    return e == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

int et_hp_wait_fwd(void* own_buffer, int world, int T, int hidden, int epoch, et_stream stream) {
    if (!own_buffer || world < 1 || world > et::PEER_MAX_WORLD || T <= 0 || hidden <= 0)
        return ET_ERR_INVALID_ARG;
    int* err = et::device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;
    const int* flags =
        reinterpret_cast<const int*>(static_cast<uint8_t*>(own_buffer) + et::peer_layout(world, T, hidden).flags_off) + 16;
    return et::launch_kernel(et::hp_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), flags,
                             world, epoch, err) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

}  // extern "C"
