// Tile-pruned Linear straight from the tile-CSR arrays (row_ptr, row_off, tiles), warp-level
// tensor path.
//
// A stored 16 x 16 weight tile applied to a block of tokens is a handful of small products.
// Through tcgen05 that is one instruction with N = 16, which holds the tensor pipe about 60
// cycles whatever its arithmetic (measured with the instruction-rate probes of this library: a
// tcgen05.mma costs max(~40-60, N / 2) cycles) and needs one thread to issue, commit and
// synchronise every product.  The same arithmetic as mma.sync.m16n8k16 products sustains 800-1000
// multiply-accumulates per clock per SM with every warp issuing for itself and no per-product
// synchronisation, so random tile sparsity is served by the warp-level path here; activations
// still arrive by tiled bulk copies (TMA) signalled on mbarriers, results leave by tiled bulk
// stores.
//
// One CTA of 16 warps per SM walks work items of 128 tokens x 16 output block rows (256 output
// features), each in steps of 192 input features:
//   * a step's activation block (128 tokens x 192 features: three slabs of 128 x 64, 128-byte
//     swizzle) is fetched with ONE 3-D tiled bulk copy into one of two buffers.  There is no
//     producer warp: the warp that finishes a buffer LAST (a counter in shared memory) issues
//     the copy that refills it, two steps ahead;
//   * every warp owns one block row: 128 tokens x 16 outputs of fp32 accumulators in registers.
//     Its tiles are consumed exactly in the order the format stores them - item after item - so
//     the warp streams them through its own ring of six 512-byte slots with cp.async (16 bytes
//     per lane and tile, six tiles ahead, across item boundaries: the L2 latency is covered
//     without any inter-warp hand-shake).  At the start of an item the warp turns its row's
//     column list (fetched one item ahead) into one presence mask per step.  Per tile: one
//     ldmatrix for the tile fragment, eight for the activation fragments (conflict-free under
//     the swizzle), sixteen products;
//   * bias, activation and conversion follow from registers; the warp's 128 x 16 output block
//     goes through its staging tile and leaves with one tiled bulk store that overlaps the next
//     item.  A block row without any tile yields act(bias) with no special case.
// Warps never wait for one another inside a step.  Every wait is bounded; a wait that runs out
// records a code and the CTA drains and returns.
//
// Standing (measured on B200, BERT shapes, 80-95 % of the tiles pruned): the kernel is correct
// and its products run at the warp-level rate while a warp has tiles, but an item's 196 KB of
// activations pass through a 96 KB window two steps ahead, and bias / conversion / staging of
// 128 x 256 outputs are not overlapped with products of the same warp; end to end it ties with
// the tcgen05 kernels of linear_tile.cu at 95 % and loses to them at 80 % (768 -> 3072, 8192
// tokens: 48 / 37 / 31 us at 80 / 90 / 95 % against 38 / 32 / 29 us).  It therefore runs only
// when the test hook selects it; the tcgen05 kernels stay the default.
#include "common.cuh"
#include "kernels.h"

namespace et {
namespace {

// Optional per-CTA timestamps for bring-up builds (-DET_TIMELINE); compiled out otherwise.
#ifdef ET_TIMELINE
__device__ long long et_rtile_timeline[1024];
#define RT_TL(slot) \
    if (blockIdx.x == 0 && (slot) < 1024) et_rtile_timeline[(slot)] = clock64()
#else
#define RT_TL(slot) ((void)0)
#endif

constexpr int R_BM = 128;            // tokens per item
constexpr int R_WARPS = 16;
constexpr int R_THREADS = 32 * R_WARPS;
constexpr int R_ROWS = R_WARPS;      // block rows per item (one per warp)
constexpr int R_SEG_SLABS = 3;       // 64-feature slabs per step (192 features, 12 block columns)
constexpr int R_SEG_COLS = R_SEG_SLABS * 4;
constexpr int R_SLAB_BYTES = R_BM * 64 * 2;
constexpr int R_XBUF_BYTES = R_SEG_SLABS * R_SLAB_BYTES;  // 48 KB
constexpr int R_DEPTH = 6;                                // tiles in flight per warp
constexpr int R_RING_BYTES = R_WARPS * R_DEPTH * 512;     // 48 KB
constexpr int R_STAGING_BYTES = R_WARPS * 4096;           // per warp 128 tokens x 16 outputs, fp16
constexpr int R_MAX_SEGS = 64;                            // in <= 12288
constexpr int R_MASK_BYTES = R_WARPS * R_MAX_SEGS * 4;
constexpr int R_MISC_BYTES = 256;
constexpr int R_SMEM_BYTES =
    2 * R_XBUF_BYTES + R_RING_BYTES + R_STAGING_BYTES + R_MASK_BYTES + R_MISC_BYTES + 1024;
static_assert(R_SMEM_BYTES <= 227 * 1024, "shared memory");

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int ACT>
__global__ void __launch_bounds__(R_THREADS, 1)
linear_tile_rows_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                        const int* __restrict__ row_ptr, const int* __restrict__ row_off,
                        const __half* __restrict__ tiles, const __half* __restrict__ bias, int T, int in,
                        int out, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* ring_all = smem + 2 * R_XBUF_BYTES;
    uint8_t* staging = ring_all + R_RING_BYTES;
    uint32_t* masks_all = reinterpret_cast<uint32_t*>(staging + R_STAGING_BYTES);
    uint8_t* misc = reinterpret_cast<uint8_t*>(masks_all) + R_MASK_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);  // [2]
    int* done_cnt = reinterpret_cast<int*>(full_bar + 2);    // [2] warps that finished the buffer
    int* last_issued = done_cnt + 2;                         // highest step whose copy was issued
    volatile int* abort_flag = reinterpret_cast<volatile int*>(done_cnt + 3);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nbr = out >> 4;
    const int nslab = in >> 6;  // in % 64 == 0
    const int nseg = (nslab + R_SEG_SLABS - 1) / R_SEG_SLABS;
    const int seg_slabs = nslab < R_SEG_SLABS ? nslab : R_SEG_SLABS;  // the copy's box depth
    const uint32_t seg_bytes = static_cast<uint32_t>(seg_slabs) * R_SLAB_BYTES;
    const int items_n = (nbr + R_ROWS - 1) / R_ROWS;
    const int items_m = (T + R_BM - 1) / R_BM;
    const int total_items = items_n * items_m;
    const int my_items =
        static_cast<int>(blockIdx.x) < total_items ? (total_items - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int total_steps = my_items * nseg;  // step q = (item of this CTA, segment)

    // the copy that fills a buffer for step q
    auto issue_step = [&](int q) {
        const int it = q / nseg, seg = q - it * nseg;
        const int t = blockIdx.x + it * gridDim.x;
        const int m0 = (t / items_n) * R_BM;
        const int b = q & 1;
        atomicMax(last_issued, q);
        mbar_arrive_expect_tx(&full_bar[b], seg_bytes);
        tma_load_3d(smem + b * R_XBUF_BYTES, &tmX, &full_bar[b], 0, m0, seg * R_SEG_SLABS);
    };

    if (threadIdx.x == 0) RT_TL(0);
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmY);
        mbar_init(&full_bar[0], 1);
        mbar_init(&full_bar[1], 1);
        done_cnt[0] = done_cnt[1] = 0;
        *last_issued = -1;
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();  // activations and Y belong to the kernels before / after this one
    if (threadIdx.x == 0) {
        if (total_steps > 0) issue_step(0);
        if (total_steps > 1) issue_step(1);
    }

    // ldmatrix lane addresses.  Activation fragment (16 tokens x 16 features of a slab: 128-byte
    // rows, 16-byte unit u of a row stored at u ^ (token & 7)): matrices = (tokens 0-7,
    // features 0-7), (8-15, 0-7), (0-7, 8-15), (8-15, 8-15).
    const uint32_t a_lane = ((lane & 7) + (((lane >> 3) & 1) << 3)) * 128;
    const uint32_t a_hi = lane >> 4, a_x = lane & 7;
    // Tile fragment (16 outputs x 16 features, row-major, 32-byte rows): matrices = (outputs
    // 0-7, features 0-7), (0-7, 8-15), (8-15, 0-7), (8-15, 8-15).
    const uint32_t b_lane = ((lane & 7) + ((lane >> 4) << 3)) * 32 + (((lane >> 3) & 1) << 4);
    const int g4 = lane >> 2, t4 = lane & 3;
    const uint32_t xbase = smem_u32(smem);
    const uint32_t ring = smem_u32(ring_all) + warp * (R_DEPTH * 512);
    uint8_t* stg = staging + warp * 4096;
    uint32_t* masks = masks_all + warp * R_MAX_SEGS;  // [step]
    const uint8_t* tile_bytes = reinterpret_cast<const uint8_t*>(tiles) + lane * 16;
    const int max_row_tiles = nslab * 4;  // a row holds at most this many tiles

    // tile range of this warp's block row of item `it` (empty past the matrix / past the items)
    auto row_range = [&](int it, int& c, int& e) {
        c = e = 0;
        if (it >= my_items) return;
        const int t = blockIdx.x + it * gridDim.x;
        const int br = (t % items_n) * R_ROWS + warp;
        if (br < nbr) {
            c = __ldg(row_ptr + br);
            e = __ldg(row_ptr + br + 1);
        }
    };

    // ---- the request stream: this warp's tiles of all its items, in the order they are stored
    // and consumed; it runs R_DEPTH tiles ahead of the products, across item boundaries ----
    int rq_it = 0, rq_idx, rq_end;
    row_range(0, rq_idx, rq_end);
    int slot_w = 0, slot_r = 0;
    auto request_next = [&]() {
        while (rq_idx >= rq_end && rq_it < my_items) {
            ++rq_it;
            row_range(rq_it, rq_idx, rq_end);
        }
        if (rq_idx < rq_end) {
            cp_async_16(ring + slot_w * 512 + lane * 16, tile_bytes + static_cast<size_t>(rq_idx) * 512);
            ++rq_idx;
        }
        cp_async_commit();  // (an empty group past the end keeps the group count in step)
        slot_w = slot_w + 1 == R_DEPTH ? 0 : slot_w + 1;
    };
#pragma unroll 1
    for (int i = 0; i < R_DEPTH; ++i) request_next();

    bool ok = true, store_open = false;
    int q = 0;
    // the NEXT item's range and (for rows of up to 64 tiles) its column list, fetched while the
    // current item runs
    int nbeg, nend, ncol0 = -1, ncol1 = -1;
    auto prefetch_cols = [&]() {
        ncol0 = nbeg + lane < nend ? __ldg(row_off + nbeg + lane) : -1;
        ncol1 = nbeg + 32 + lane < nend ? __ldg(row_off + nbeg + 32 + lane) : -1;
    };
    row_range(0, nbeg, nend);
    prefetch_cols();
    for (int it = 0; it < my_items && ok; ++it) {
        const int t = blockIdx.x + it * gridDim.x;
        const int m0 = (t / items_n) * R_BM;
        const int br = (t % items_n) * R_ROWS + warp;  // this warp's block row
        const int beg = nbeg, end = nend;
        if ((warp == 0 || warp == 15) && lane == 0 && it < 8) RT_TL(10 + it + (warp ? 40 : 0));

        // ---- presence mask per step from the row's column list ----
        for (int i = lane; i < nseg; i += 32) masks[i] = 0u;
        __syncwarp();
        {
            auto mark = [&](int col) {
                if (col >= 0 && col < max_row_tiles)  // (a validated matrix never fails the bound)
                    atomicOr(&masks[col / R_SEG_COLS], 1u << (col % R_SEG_COLS));
            };
            mark(ncol0);
            mark(ncol1);
            for (int i = beg + 64 + lane; i < end; i += 32) mark(__ldg(row_off + i));
        }
        row_range(it + 1, nbeg, nend);
        prefetch_cols();
        // (kept as loaded: converting here would wait for the loads before the products)
        uint32_t braw[2] = {0u, 0u};
        if (bias != nullptr && br < nbr) {
#pragma unroll
            for (int nh = 0; nh < 2; ++nh)
                braw[nh] = __ldg(reinterpret_cast<const unsigned int*>(bias + br * 16 + nh * 8 + 2 * t4));
        }
        __syncwarp();

        float acc[8][2][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;

        for (int seg = 0; seg < nseg && ok; ++seg, ++q) {
            const int b = q & 1;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full_bar[b], (q >> 1) & 1, abort_flag))) {
                if (lane == 0) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                ok = false;
                break;
            }
            if ((warp == 0 || warp == 15) && lane == 0 && it < 8 && seg == 0) RT_TL(20 + it + (warp ? 40 : 0));
            const uint32_t xb = xbase + b * R_XBUF_BYTES + a_lane;
            uint32_t m = masks[seg];
            while (m) {
                const int cs = __ffs(m) - 1;  // block column inside the step
                m &= m - 1;
                cp_async_wait<R_DEPTH - 1>();  // the oldest tile in flight has landed
                __syncwarp();
                uint32_t bf[4];
                ldmatrix_x4(bf, ring + slot_r * 512 + b_lane);
                const uint32_t aoff = xb + (cs >> 2) * R_SLAB_BYTES + ((((cs & 3) * 2 + a_hi) ^ a_x) << 4);
                // the activation fragments of four 16-token groups are in flight while the products
                // of the four before them issue
                uint32_t a[8][4];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) ldmatrix_x4(a[mt], aoff + mt * 2048);
                __syncwarp();  // every lane has read the slot: it may be refilled
                request_next();
                slot_r = slot_r + 1 == R_DEPTH ? 0 : slot_r + 1;
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    mma_m16n8k16(acc[mt][0], a[mt], bf[0], bf[1]);
                    mma_m16n8k16(acc[mt][1], a[mt], bf[2], bf[3]);
                    ldmatrix_x4(a[mt + 4], aoff + (mt + 4) * 2048);
                }
#pragma unroll
                for (int mt = 4; mt < 8; ++mt) {
                    mma_m16n8k16(acc[mt][0], a[mt], bf[0], bf[1]);
                    mma_m16n8k16(acc[mt][1], a[mt], bf[2], bf[3]);
                }
            }
            // this warp is done with the buffer; the last of the 16 refills it for step q + 2
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                const int before = atomicAdd(&done_cnt[b], 1);
                if (before == R_WARPS - 1) {
                    atomicExch(&done_cnt[b], 0);
                    __threadfence_block();
                    fence_proxy_async_smem();
                    if (q + 2 < total_steps) issue_step(q + 2);
                }
            }
        }
        if (!ok) break;
        if ((warp == 0 || warp == 15) && lane == 0 && it < 8) RT_TL(30 + it + (warp ? 40 : 0));

        // ---- epilogue from registers: thread (g4, t4) holds tokens mt * 16 + g4 (+ 8), outputs
        // 2 * t4 (+ 1) and 8 + 2 * t4 (+ 1) of the block row.  A 4 x 4 exchange inside the quad
        // gives every lane 16 contiguous bytes (lane 0 / 1 the two halves of token g4, lane 2 / 3
        // of token g4 + 8); the 128 x 16 block is staged token-major and leaves with one tiled
        // bulk store.
        if (br < nbr) {
            float bv[2][2];
#pragma unroll
            for (int nh = 0; nh < 2; ++nh) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&braw[nh]));
                bv[nh][0] = f.x;
                bv[nh][1] = f.y;
            }
            if (store_open) {
                if (lane == 0) tma_store_wait_read();  // the previous item's store has read the tile
                __syncwarp();
            }
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t v[4];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int nh = 0; nh < 2; ++nh)
                        v[hh * 2 + nh] = pack_half2(apply_act(acc[mt][nh][hh * 2] + bv[nh][0], ACT),
                                                    apply_act(acc[mt][nh][hh * 2 + 1] + bv[nh][1], ACT));
                {
                    const bool odd = t4 & 1;
                    const uint32_t s0 = odd ? v[0] : v[1], s1 = odd ? v[2] : v[3];
                    const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 1);
                    const uint32_t r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
                    if (odd) {
                        v[0] = r0;
                        v[2] = r1;
                    } else {
                        v[1] = r0;
                        v[3] = r1;
                    }
                }
                {
                    const bool up = t4 & 2;
                    const uint32_t s0 = up ? v[0] : v[2], s1 = up ? v[1] : v[3];
                    const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 2);
                    const uint32_t r1 = __shfl_xor_sync(0xffffffffu, s1, 2);
                    if (up) {
                        v[0] = r0;
                        v[1] = r1;
                    } else {
                        v[2] = r0;
                        v[3] = r1;
                    }
                }
                // now v[j] is lane j's word t4: lane t4 = (token half t4 / 2, output half t4 % 2)
                uint4 o;
                o.x = v[0];
                o.y = v[1];
                o.z = v[2];
                o.w = v[3];
                *reinterpret_cast<uint4*>(stg + (mt * 16 + g4 + ((t4 >> 1) << 3)) * 32 + (t4 & 1) * 16) = o;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(&tmY, stg, br * 16, m0);  // tokens past T are clipped
                tma_store_commit();
            }
            store_open = true;
        }
        if ((warp == 0 || warp == 15) && lane == 0 && it < 8) RT_TL(40 + it + (warp ? 40 : 0));
    }
    cp_async_wait<0>();
    if (store_open && lane == 0) tma_store_wait_read();

    // copies in flight must land before the CTA's shared memory is released: after a give-up the
    // last two steps' copies may still be outstanding
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const int last = *last_issued;
        for (int qq = last; qq >= 0 && qq > last - 2; --qq)
            for (uint32_t k = 0; k < ET_SPIN_LIMIT; ++k)
                if (mbar_try_wait(&full_bar[qq & 1], (qq >> 1) & 1)) break;
    }
}

}  // namespace

bool linear_tile_rows_supported(int in, int out) {
    return in > 0 && out > 0 && in % 64 == 0 && out % 16 == 0 && in <= R_MAX_SEGS * R_SEG_SLABS * 64;
}

int launch_linear_tile_rows(const int* row_ptr, const int* row_off, const __half* tiles, int nnz_tiles,
                            const __half* bias, const __half* X, __half* Y, int T, int in, int out,
                            int act, cudaStream_t stream) {
    if (!row_ptr || !row_off || !tiles || !X || !Y || T <= 0 || nnz_tiles <= 0) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (!linear_tile_rows_supported(in, out)) return ET_ERR_SHAPE;
    if (!aligned16(X) || !aligned16(Y) || !aligned16(tiles) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;
    const int nslab = in / 64;
    CUtensorMap tmX, tmY;
    {
        // {feature inside a slab, token, slab}: one box = 128 tokens of up to three slabs, stored
        // slab by slab (128 rows of 128 bytes each)
        const uint64_t dims[3] = {64, static_cast<uint64_t>(T), static_cast<uint64_t>(nslab)};
        const uint64_t strides[2] = {static_cast<uint64_t>(in) * 2, 128};
        const uint32_t box[3] = {64, R_BM, static_cast<uint32_t>(nslab < R_SEG_SLABS ? nslab : R_SEG_SLABS)};
        int st = make_tensor_map_f16(&tmX, X, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    {
        // one box = a warp's block row (16 outputs) of 128 tokens, as the warp stages it
        const uint64_t dims[2] = {static_cast<uint64_t>(out), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(out) * 2};
        const uint32_t box[2] = {16, R_BM};
        int st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (st != ET_OK) return st;
    }
    const int nbr = out / 16;
    const int items = ((nbr + R_ROWS - 1) / R_ROWS) * ((T + R_BM - 1) / R_BM);
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const dim3 grid(items < sms ? items : sms);
    int dev = 0;
    cudaGetDevice(&dev);
    auto go = [&](auto kern, int slot) -> cudaError_t {
        static std::atomic<bool> attr_set[3][64] = {};
        if (dev >= 0 && dev < 64 && !attr_set[slot][dev]) {
            const cudaError_t ea =
                cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, R_SMEM_BYTES);
            if (ea != cudaSuccess) return ea;
            attr_set[slot][dev] = true;
        }
        return launch_kernel(kern, grid, dim3(R_THREADS), R_SMEM_BYTES, stream, tmX, tmY, row_ptr, row_off,
                             tiles, bias, T, in, out, err);
    };
    const cudaError_t e = act == ET_ACT_GELU   ? go(linear_tile_rows_kernel<ET_ACT_GELU>, 0)
                          : act == ET_ACT_RELU ? go(linear_tile_rows_kernel<ET_ACT_RELU>, 1)
                                               : go(linear_tile_rows_kernel<ET_ACT_NONE>, 2);
    return e == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

}  // namespace et
