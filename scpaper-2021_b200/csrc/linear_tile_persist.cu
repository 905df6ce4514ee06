// Tile-pruned Linear on re-packed weights, persistent form.
//
// One CTA per SM walks a list of work items (128 tokens x 2 panels of 8 output block rows =
// 256 output features).  What a 16 x 16 weight tile costs on this tensor core is set by the
// instruction, not by its arithmetic.  Measured on B200 (instruction-rate probes of this
// library): a 128 x 16 x 16 tcgen05.mma occupies the pipe 39 cycles at best (several issuing
// threads, operands that stay put), about 60 in this kernel, where every product re-reads its
// 4 KB activation slab from shared memory while bulk copies write the next stages; a thread
// that issues them needs 60-90 cycles per product and about 110 per tcgen05.commit, and a
// bulk-copy instruction costs its thread about 100.  So the kernel is organised to keep many
// threads issuing and to spend as few per-stage instructions as it can:
//   * a ring stage holds TWO 64-feature chunks of the item: two 128 x 64 activation slabs
//     (tiled bulk copies, 128-byte swizzle) fetched by warp 0 and the two chunks' tiles of
//     both panels fetched by warp 1 with ONE untiled bulk copy (the packed order keeps them
//     adjacent); chunks without a tile of the item are skipped by every role.  Inside a
//     producer warp the lane that loaded a stage's masks and offsets issues its copy itself;
//   * warps 2-9: one thread each issues the products of block row (warp - 2) of both panels
//     for a stage and commits them to the stage's barrier, so eight threads feed the pipe in
//     parallel.  Per item each of these warps first turns the item's masks into a small
//     table in shared memory (all lanes), then lane 0 alone walks it: one 8-byte read per
//     stage, no exchange between lanes inside the loop;
//   * warps 10-17 drain the PREVIOUS item's accumulators (tensor memory holds two items'
//     worth, 2 x 256 columns) - bias, activation, fp16, swizzled staging tile, bulk store -
//     while the current item's products run; item boundaries cost no pipeline drain.
// Every wait is bounded; a wait that runs out records a code and the CTA drains and returns.
#include "common.cuh"
#include "kernels.h"

namespace et {
namespace {

// Optional per-CTA timestamps for bring-up builds (-DET_TIMELINE); compiled out otherwise.
#ifdef ET_TIMELINE
__device__ long long et_ptile_timeline[1024];
#define PT_TL(slot) \
    if (blockIdx.x == 0 && (slot) < 1024) et_ptile_timeline[(slot)] = clock64()
#else
#define PT_TL(slot) ((void)0)
#endif

constexpr int P_TBM = 128;          // tokens per item
constexpr int P_ROWS = 8;           // block rows per panel
constexpr int P_PANELS = 2;         // panels per item
constexpr int P_TBN = P_ROWS * 16;  // output features per panel
constexpr int P_CHUNK = 64;         // input features per chunk (the packed format's unit)
constexpr int P_SLAB_BYTES = P_TBM * P_CHUNK * 2;
constexpr int P_X_BYTES = 2 * P_SLAB_BYTES;  // a stage's two activation slabs
constexpr int P_RING_BYTES = 144 * 1024;
constexpr int P_MAX_STAGES = 5;
constexpr int P_ISSUERS = 8;
constexpr int P_EPI_WARPS = 8;
constexpr int P_THREADS = 32 * (2 + P_ISSUERS + P_EPI_WARPS);
constexpr int P_STAGING_BYTES = P_EPI_WARPS * 2 * 4096;  // two 32 x 64 fp16 tiles per warp
constexpr int P_MAX_STEPS = 64;                          // stages per item: in <= 8192
// barriers and flags (256 bytes), the epilogue warps' bias lines (8 warps x 2 panels x 64
// floats), the issuing warps' per-item tables (8 warps x 64 stages x 2 words)
constexpr int P_BIAS_BYTES = P_EPI_WARPS * P_PANELS * 64 * 4;
constexpr int P_TAB_BYTES = P_ISSUERS * P_MAX_STEPS * 8;
constexpr int P_MISC_BYTES = 256 + P_BIAS_BYTES + P_TAB_BYTES;
constexpr int P_SMEM_BYTES = P_RING_BYTES + P_STAGING_BYTES + P_MISC_BYTES + 1024;
static_assert(P_SMEM_BYTES <= 227 * 1024, "shared memory");

struct TileItem {
    int m0;      // first token
    int panel0;  // first of the two panels
};

template <int ACT>
__global__ void __launch_bounds__(P_THREADS, 1)
linear_tile_persist_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                           const uint32_t* __restrict__ pk_mask, const int* __restrict__ pk_off,
                           const __half* __restrict__ pk_tiles, const __half* __restrict__ bias, int T,
                           int in, int out, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* ring = smem;
    uint8_t* staging = smem + P_RING_BYTES;
    uint8_t* misc = staging + P_STAGING_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);  // [P_MAX_STAGES]
    uint64_t* empty_bar = full_bar + P_MAX_STAGES;           // [P_MAX_STAGES]
    uint64_t* acc_full = empty_bar + P_MAX_STAGES;           // [2]
    uint64_t* acc_empty = acc_full + 2;                      // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* max_cnt = reinterpret_cast<int*>(tmem_slot + 2);
    float* s_bias = reinterpret_cast<float*>(misc + 256);                      // [8][2][64]
    uint32_t* s_tab = reinterpret_cast<uint32_t*>(misc + 256 + P_BIAS_BYTES);  // [8][64][2]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nchunk = (in + P_CHUNK - 1) / P_CHUNK;
    const int nstep = (nchunk + 1) >> 1;       // stages per item (two chunks each)
    const int ngroup = (2 * nstep + 31) >> 5;  // groups of 32 chunks (one warp-wide load each)
    const int npanel = (out + P_TBN - 1) / P_TBN;
    const int items_n = (npanel + P_PANELS - 1) / P_PANELS;
    const int items_m = (T + P_TBM - 1) / P_TBM;
    const int total_items = items_n * items_m;
    // consecutive items share a token block: CTAs that run side by side read the same
    // activation rows from L2
    auto item_of = [&](int t) {
        TileItem it;
        it.m0 = (t / items_n) * P_TBM;
        it.panel0 = (t % items_n) * P_PANELS;
        return it;
    };

    // ---- set-up (weights only: may overlap the previous kernel's tail) ----
    if (threadIdx.x == 0) PT_TL(0);
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmY);
        for (int s = 0; s < P_MAX_STAGES; ++s) {
            mbar_init(&full_bar[s], 2);  // the slabs' and the tiles' producers
            mbar_init(&empty_bar[s], P_ISSUERS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], P_ISSUERS);
            mbar_init(&acc_empty[b], P_EPI_WARPS);
        }
        *abort_flag = 0;
        *max_cnt = 1;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    __syncthreads();
    {
        // the ring's stage size follows the fullest (panel pair, stage) of the whole weight
        int mc = 0;
        for (int i = threadIdx.x; i < items_n * nstep; i += P_THREADS) {
            const int pp = i / nstep, d = i - pp * nstep;
            int cnt = 0;
            for (int k = 0; k < P_PANELS; ++k)
                for (int j = 0; j < 2; ++j)
                    if (2 * pp + k < npanel && 2 * d + j < nchunk)
                        cnt += __popc(__ldg(pk_mask + static_cast<size_t>(2 * pp + k) * nchunk + 2 * d + j));
            mc = cnt > mc ? cnt : mc;
        }
        for (int d = 16; d > 0; d >>= 1) {
            const int o = __shfl_xor_sync(0xffffffffu, mc, d);
            mc = o > mc ? o : mc;
        }
        if (lane == 0 && mc > 1) atomicMax(max_cnt, mc);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int nslot = (*max_cnt + 3) & ~3;  // tile slots per stage (both chunks, both panels, dense)
    const int stage_bytes = P_X_BYTES + nslot * 512;
    int nstages = P_RING_BYTES / stage_bytes;
    nstages = nstages < 1 ? 1 : (nstages > P_MAX_STAGES ? P_MAX_STAGES : nstages);
    if (threadIdx.x == 0) PT_TL(1);
    pdl_launch_dependents();
    pdl_wait();  // activations and Y belong to the kernels before / after this one

    // the masks of 32 chunks (chunk = group * 32 + lane) of the item's two panels
    auto load_masks = [&](const TileItem& it, int g, uint32_t& m0, uint32_t& m1) {
        const int c = g * 32 + lane;
        m0 = m1 = 0u;
        if (c < nchunk) {
            if (it.panel0 < npanel) m0 = __ldg(pk_mask + static_cast<size_t>(it.panel0) * nchunk + c);
            if (it.panel0 + 1 < npanel)
                m1 = __ldg(pk_mask + static_cast<size_t>(it.panel0 + 1) * nchunk + c);
        }
    };

    if (warp < 2) {
        // ---------------- producers: warp 0 the activation slabs, warp 1 the tiles ----------------
        // The even lane 2j of a group owns stage j of the group (chunks 2j, 2j + 1): it takes
        // the odd lane's masks and offsets once per group and issues the stage's copies itself.
        int s = 0, issued = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
            const TileItem it = item_of(t);
            for (int g = 0; g < ngroup && ok; ++g) {
                uint32_t m0, m1;
                load_masks(it, g, m0, m1);
                const int c = g * 32 + lane;
                int o0 = 0, o1 = 0;
                if (warp == 1) {
                    if (m0) o0 = __ldg(pk_off + static_cast<size_t>(it.panel0) * nchunk + c);
                    if (m1) o1 = __ldg(pk_off + static_cast<size_t>(it.panel0 + 1) * nchunk + c);
                }
                // the odd neighbour's values, for the even lane
                const uint32_t m0b = __shfl_down_sync(0xffffffffu, m0, 1);
                const uint32_t m1b = __shfl_down_sync(0xffffffffu, m1, 1);
                const int o0b = __shfl_down_sync(0xffffffffu, o0, 1);
                const int o1b = __shfl_down_sync(0xffffffffu, o1, 1);
                const bool any_a = (m0 | m1) != 0u, any_b = (m0b | m1b) != 0u;
                uint32_t live = __ballot_sync(0xffffffffu, (lane & 1) == 0 && (any_a || any_b));
                while (live) {
                    const int cc = __ffs(live) - 1;
                    live &= live - 1;
                    if (lane == cc) {
                        uint8_t* stage = ring + s * stage_bytes;
                        if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) {
                            report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_PRODUCER);
                        } else if (warp == 0) {
                            if (issued < 60) PT_TL(100 + 2 * issued);
                            mbar_arrive_expect_tx(&full_bar[s],
                                                  (any_a ? P_SLAB_BYTES : 0) + (any_b ? P_SLAB_BYTES : 0));
                            if (any_a) tma_load_2d(stage, &tmX, &full_bar[s], c * P_CHUNK, it.m0);
                            if (any_b)
                                tma_load_2d(stage + P_SLAB_BYTES, &tmX, &full_bar[s], (c + 1) * P_CHUNK,
                                            it.m0);
                            if (issued < 60) PT_TL(101 + 2 * issued);
                        } else {
                            // runs in packed order: (panel 0, chunk a), (panel 1, chunk a), (panel 0,
                            // chunk b), (panel 1, chunk b); adjacent runs merge into one copy
                            const int ro[4] = {o0, o1, o0b, o1b};
                            const int rn[4] = {__popc(m0), __popc(m1), __popc(m0b), __popc(m1b)};
                            mbar_arrive_expect_tx(&full_bar[s], 512u * (rn[0] + rn[1] + rn[2] + rn[3]));
                            uint8_t* dst = stage + P_X_BYTES;
                            int start = 0, cnt = 0;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (rn[i] == 0) continue;
                                if (cnt > 0 && ro[i] != start + cnt) {
                                    bulk_load(dst, pk_tiles + static_cast<size_t>(start) * 256, 512u * cnt,
                                              &full_bar[s]);
                                    dst += cnt * 512;
                                    cnt = 0;
                                }
                                if (cnt == 0) start = ro[i];
                                cnt += rn[i];
                            }
                            if (cnt > 0)
                                bulk_load(dst, pk_tiles + static_cast<size_t>(start) * 256, 512u * cnt,
                                          &full_bar[s]);
                        }
                    }
                    __syncwarp();
                    if (*abort_flag) {
                        ok = false;
                        break;
                    }
                    ++issued;
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
        if (*abort_flag && lane == 0) {
            // let copies in flight land: the last min(issued, nstages) stages
            int ss = s;
            uint32_t pp = ph;
            const int pending = issued < nstages ? issued : nstages;
            for (int i = 0; i < pending; ++i) {
                if (--ss < 0) {
                    ss = nstages - 1;
                    pp ^= 1u;
                }
                for (uint32_t k = 0; k < ET_SPIN_LIMIT; ++k)
                    if (mbar_try_wait(&full_bar[ss], pp)) break;
            }
        }
    } else if (warp < 2 + P_ISSUERS) {
        // ---------------- product issue: block row e of both panels ----------------
        const int e = warp - 2;
        constexpr uint32_t idesc = make_idesc_f16(P_TBM, 16, 0, 0);
        const uint32_t ring_addr = smem_u32(ring);
        // descriptors differ between stages, slabs and tiles only in the start-address field
        // (16-byte units)
        const uint64_t a_desc0 = make_smem_desc(ring_addr, 16, 1024, SWZ_128B);
        const uint64_t b_desc0 = make_smem_desc(ring_addr + P_X_BYTES, 16, 256, SWZ_32B);
        const uint32_t stage_units = static_cast<uint32_t>(stage_bytes) >> 4;
        const uint32_t below = (1u << (4 * e)) - 1u;
        uint32_t* tab = s_tab + e * (P_MAX_STEPS * 2);  // [stage][chunk a, chunk b]
        int s = 0, item_it = 0, seen = 0;
        uint32_t ph = 0;
        for (int t = blockIdx.x; t < total_items; t += gridDim.x, ++item_it) {
            const TileItem it = item_of(t);
            const int buf = item_it & 1;
            // The item's table, one word per chunk: bits 0-3 this row's tiles of panel 0 among the
            // chunk's 4 block columns, bits 4-11 their first slot among the stage's tiles, bits
            // 12-15 / 16-23 the same for panel 1, bit 31 = the chunk holds a tile of the item.
            for (int g = 0; g < ngroup; ++g) {
                uint32_t m0, m1;
                load_masks(it, g, m0, m1);
                const uint32_t n = __popc(m0) + __popc(m1);
                const uint32_t before = __shfl_up_sync(0xffffffffu, n, 1);  // the even neighbour's tiles
                const uint32_t base = (lane & 1) ? before : 0u;
                const uint32_t word = ((m0 >> (4 * e)) & 0xFu) | ((base + __popc(m0 & below)) << 4) |
                                      (((m1 >> (4 * e)) & 0xFu) << 12) |
                                      ((base + __popc(m0) + __popc(m1 & below)) << 16) |
                                      ((m0 | m1) != 0u ? 0x80000000u : 0u);
                if (g * 32 + lane < 2 * nstep) tab[g * 32 + lane] = word;
            }
            __syncwarp();
            if (lane == 0) {
                bool ok = true;
                if (item_it < 8 && e == 0) PT_TL(10 + item_it);
                if (item_it >= 2) {
                    // the epilogue must have drained what the item two back left in this buffer
                    ok = mbar_wait_bounded(&acc_empty[buf], ((item_it >> 1) - 1) & 1, abort_flag);
                    if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                    tc_fence_after_sync();
                }
                const uint32_t d_tmem = tmem_base + buf * (P_PANELS * P_TBN) + e * 16;
                uint32_t started = 0u;  // bit j: this row of panel j has received a product
                for (int d = 0; d < nstep && ok; ++d) {
                    const uint2 w = *reinterpret_cast<const uint2*>(tab + 2 * d);
                    if (((w.x | w.y) & 0x80000000u) == 0u) continue;
                    // a row without a tile in this stage still waits: its arrival must not run
                    // ahead into the stage's next use
                    ok = mbar_wait_bounded(&full_bar[s], ph, abort_flag);
                    if (e == 0 && seen < 60) PT_TL(300 + 2 * seen);
                    if (!ok) {
                        report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                        break;
                    }
                    if ((w.x | w.y) & 0xF00Fu) {
                        tc_fence_after_sync();
                        const uint64_t a_stage = a_desc0 + static_cast<uint64_t>(s) * stage_units;
                        const uint64_t b_stage = b_desc0 + static_cast<uint64_t>(s) * stage_units;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {  // the stage's two chunks
                            const uint32_t word = h == 0 ? w.x : w.y;
                            const uint64_t a_base = a_stage + static_cast<uint64_t>(h) * (P_SLAB_BYTES >> 4);
#pragma unroll
                            for (int j = 0; j < P_PANELS; ++j) {
                                uint32_t nib = (word >> (12 * j)) & 0xFu;
                                uint64_t bd = b_stage + ((word >> (4 + 12 * j)) & 0xFFu) * 32u;
                                while (nib) {
                                    const int kb = __ffs(nib) - 1;
                                    nib &= nib - 1;
                                    mma_f16_ss(d_tmem + j * P_TBN, a_base + static_cast<uint64_t>(kb * 2), bd,
                                               idesc, (started >> j) & 1u);
                                    started |= 1u << j;
                                    bd += 32;  // next 512-byte slot
                                }
                            }
                        }
                        mma_commit(&empty_bar[s]);
                    } else {
                        mbar_arrive(&empty_bar[s]);
                    }
                    if (e == 0 && seen < 60) PT_TL(301 + 2 * seen);
                    ++seen;
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok) mma_commit(&acc_full[buf]);  // arrives once this row's products are done
            }
            // lanes 1-31 do not track the ring position: only lane 0 uses it
            __syncwarp();
            if (*abort_flag) break;
        }
    } else {
        // ---------------- epilogue: bias, activation, fp16, store ----------------
        const int w = warp - (2 + P_ISSUERS);  // 0 .. 7
        const int q = warp & 3;                // tensor-memory lane quadrant this warp may read
        const int half = w >> 2;               // which 64 output columns of each panel
        float* wb = s_bias + w * (P_PANELS * 64);
        bool ok = true;
        int groups_open = 0;  // bulk store groups of lane 0 that may still read a staging tile
        int item_it = 0;
        for (int t = blockIdx.x; t < total_items; t += gridDim.x, ++item_it) {
            const TileItem it = item_of(t);
            const int buf = item_it & 1;
            if (w == 0 && lane == 0 && item_it < 8) PT_TL(500 + 4 * item_it);
            // while the item's products run: which block rows of the two panels hold any tile at
            // all (rows without one were never written by the tensor core and carry the bias
            // alone), and this warp's bias values
            uint32_t any0 = 0u, any1 = 0u;
            for (int g = 0; g < ngroup; ++g) {
                uint32_t m0, m1;
                load_masks(it, g, m0, m1);
                any0 |= m0;
                any1 |= m1;
            }
            for (int d = 16; d > 0; d >>= 1) {
                any0 |= __shfl_xor_sync(0xffffffffu, any0, d);
                any1 |= __shfl_xor_sync(0xffffffffu, any1, d);
            }
#pragma unroll
            for (int k = 0; k < P_PANELS; ++k)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int n = (it.panel0 + k) * P_TBN + half * 64 + lane + 32 * i;
                    wb[k * 64 + lane + 32 * i] =
                        (bias != nullptr && n < out) ? __half2float(__ldg(bias + n)) : 0.f;
                }
            __syncwarp();
            if (ok) {
                ok = mbar_wait_bounded_relaxed(&acc_full[buf], (item_it >> 1) & 1, abort_flag);
                if (!ok && lane == 0) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_EPILOGUE);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) continue;
            tc_fence_after_sync();
            if (w == 0 && lane == 0 && item_it < 8) PT_TL(501 + 4 * item_it);
#pragma unroll
            for (int k = 0; k < P_PANELS; ++k) {
                const int n0 = (it.panel0 + k) * P_TBN + half * 64;
                if (n0 >= out) continue;
                const uint32_t anyk = k == 0 ? any0 : any1;
                uint8_t* tile = staging + (w * 2 + k) * 4096;
                uint8_t* srow = tile + lane * 128;
                const uint32_t lane_addr = tmem_base + buf * (P_PANELS * P_TBN) + k * P_TBN + half * 64 +
                                           (static_cast<uint32_t>(q * 32) << 16);
                uint32_t v0[32], v1[32];
                tmem_ld32(lane_addr, v0);
                tmem_ld32(lane_addr + 32, v1);
                // the store that last used this staging tile must have read it; the two tiles
                // alternate, so the one younger group may still be in flight
                if (lane == 0 && groups_open >= 2) tma_store_wait_read_pending<1>();
                __syncwarp();
                tmem_ld_wait_regs(v0);  // ties the wait to the destination registers
                tmem_ld_wait_regs(v1);
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    // 32 columns = block rows 2 * (half * 2 + cc) and the next of the panel
                    const int br = (half * 2 + cc) * 2;
                    const bool has0 = ((anyk >> (4 * br)) & 0xFu) != 0u;
                    const bool has1 = ((anyk >> (4 * (br + 1))) & 0xFu) != 0u;
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) {
                        float f[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t raw = cc == 0 ? v0[gq * 8 + j] : v1[gq * 8 + j];
                            const bool has = gq < 2 ? has0 : has1;
                            f[j] = apply_act((has ? __uint_as_float(raw) : 0.f) +
                                                 wb[k * 64 + cc * 32 + gq * 8 + j],
                                             ACT);
                        }
                        uint4 o;
                        o.x = pack_half2(f[0], f[1]);
                        o.y = pack_half2(f[2], f[3]);
                        o.z = pack_half2(f[4], f[5]);
                        o.w = pack_half2(f[6], f[7]);
                        *reinterpret_cast<uint4*>(srow + ((((cc << 2) + gq) ^ (lane & 7)) * 16)) = o;
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    // a group is committed even when the rows lie outside the matrix and nothing
                    // is stored: tiles and groups stay in step
                    if (it.m0 + q * 32 < T) tma_store_2d(&tmY, tile, n0, it.m0 + q * 32);
                    tma_store_commit();
                    ++groups_open;
                }
            }
            // A panel that was skipped (it lies outside the matrix) breaks the alternation of the
            // two staging tiles: drain before the next item then.
            if ((it.panel0 + 1) * P_TBN + half * 64 >= out) {
                if (lane == 0) {
                    tma_store_wait_read();
                    groups_open = 0;
                }
            }
            // the accumulators of this buffer have been read: the item after next may overwrite them
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (w == 0 && lane == 0 && item_it < 8) PT_TL(502 + 4 * item_it);
        }
        if (lane == 0) tma_store_wait_read();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

int g_tile_packed_mode = -1;  // test hook, see tile_packed_mode()

int tile_packed_mode() { return g_tile_packed_mode; }

int launch_linear_tile_persist(const int* row_ptr, const uint32_t* pk_mask, const int* pk_off,
                               const __half* pk_tiles, int nnz_tiles, const __half* bias,
                               const __half* X, __half* Y, int T, int in, int out, int act,
                               cudaStream_t stream) {
    if (!row_ptr || !pk_mask || !pk_off || !pk_tiles || !X || !Y || T <= 0 || in <= 0 || out <= 0 ||
        nnz_tiles <= 0)
        return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16 || in > 8192) return ET_ERR_SHAPE;
    if (!aligned16(X) || !aligned16(Y) || !aligned16(pk_tiles) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;
    CUtensorMap tmX, tmY;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(in), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(in) * 2};
        const uint32_t box[2] = {P_CHUNK, P_TBM};
        int st = make_tensor_map_f16(&tmX, X, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(out), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(out) * 2};
        const uint32_t box[2] = {64, 32};
        int st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    const int npanel = (out + P_TBN - 1) / P_TBN;
    const int items = ((npanel + P_PANELS - 1) / P_PANELS) * ((T + P_TBM - 1) / P_TBM);
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const dim3 grid(items < sms ? items : sms);
    int dev = 0;
    cudaGetDevice(&dev);
    auto go = [&](auto kern, int slot) -> cudaError_t {
        static std::atomic<bool> attr_set[3][64] = {};
        if (dev >= 0 && dev < 64 && !attr_set[slot][dev]) {
            const cudaError_t ea =
                cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
            if (ea != cudaSuccess) return ea;
            attr_set[slot][dev] = true;
        }
        return launch_kernel(kern, grid, dim3(P_THREADS), P_SMEM_BYTES, stream, tmX, tmY, pk_mask,
                             pk_off, pk_tiles, bias, T, in, out, err);
    };
    const cudaError_t e = act == ET_ACT_GELU   ? go(linear_tile_persist_kernel<ET_ACT_GELU>, 0)
                          : act == ET_ACT_RELU ? go(linear_tile_persist_kernel<ET_ACT_RELU>, 1)
                                               : go(linear_tile_persist_kernel<ET_ACT_NONE>, 2);
    return e == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

}  // namespace et

#ifdef ET_TEST_HOOKS
extern "C" {
// Test hook: kernel for packed weights: 1 = persistent, anything else = one item per CTA
// (default).
void et_debug_set_tile_persist(int mode) { et::g_tile_packed_mode = mode; }
}
#endif
