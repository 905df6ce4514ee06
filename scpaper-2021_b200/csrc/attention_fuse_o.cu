// Self-attention and the tile-pruned output projection in ONE kernel launch.
//
// Stands in for the cooperative kernel of Attention/kernel_fuseO.cu:138-243, which runs every
// head's attention, a grid-wide barrier and then the tile SpMM over Z.  Here the grid-wide
// barrier is replaced by one counter per (sequence, 128-query block) and work is handed out by
// ticket (one global counter):
//
//   tickets 0 .. n_att - 1   the (sequence, query block, head) attention units (attention_cta,
//            the body of the stand-alone attention kernel).  After a unit - once its rows of Z
//            are complete in global memory - the CTA adds one to the counter of the unit's
//            (sequence, query block);
//   tickets n_att ..         the (128-token block, panel of 128 output features) items of the
//            projection (linear_tile_cta, the body of the stand-alone tile Linear).  An item
//            builds its index tables, then one thread waits until the counters of the query
//            blocks that overlap the token block have reached the number of heads, then the
//            item runs with Z as its input.
//
// A projection item therefore starts as soon as ITS rows of Z exist, while other CTAs are
// still busy with other sequences' heads.  Forward progress needs no co-residency guarantee:
// a CTA takes a ticket only while it runs, attention units never wait, and an item waits only
// for attention units, all of which have lower tickets - i.e. have already been taken by
// running CTAs - by the time any item ticket is handed out.  (A cooperative launch is not
// used: the driver admits one CTA per SM to a cooperative launch of any kernel that allocates
// tensor memory - cudaOccupancyMaxActiveBlocksPerMultiprocessor returns 1 whatever the
// registers and shared memory - and both bodies are built for two co-resident CTAs per SM that
// overlap each other's phases; a first, cooperative form of this kernel took twice the time.)
// The wait is bounded: when it runs out the kernel reports DEV_TIMEOUT_FUSE_O and abandons
// the remaining work.  The last CTA to leave zeroes the counters, so a launch needs no memset.
//
// Z travels through global memory (L2) between the two kinds of work, written and read by TMA:
// the writer waits for its bulk stores to complete, fences the async proxy and releases at GPU
// scope; the reader acquires at GPU scope and fences the async proxy before its loads.
//
// Standing (measured on B200, 80 % of W_O's tiles pruned, 12 heads of 64, calls replayed back to
// back from a CUDA graph; one kernel / the two stand-alone kernels chained by programmatic
// dependent launch): 1 x 128 tokens 17.2 / 13.7 us, 16 x 128 20.1 / 15.6, 64 x 128 43.1 / 39.3,
// 4 x 512 causal 27.5 / 23.8, 32 x 512 103.3 / 99.1, 1 x 4096 121.2 / 120.4.  Inside the kernel
// the two kinds of work take what the stand-alone kernels take; what is left is the ticket and
// counter traffic (a global atomic before each piece of work, bulk-store completion, fence and
// atomic after each attention unit) and the counter clean-up at the end, none of which a
// dependent launch pays.  et_attention_fuse_o_fwd therefore runs the two kernels; this kernel
// is et_attention_fuse_o_single_launch_fwd.
#include <atomic>

#include "attention_body.cuh"
#include "linear_tile_body.cuh"

namespace et {

namespace {

using namespace attn;
using namespace tile;

static_assert(ATT_THREADS == TILE_THREADS, "both bodies run on the same CTA shape");

constexpr uint32_t FUSE_POLL_LIMIT = 1u << 23;  // x >= 100 ns per poll: about a second

struct FuseOArgs {
    const int* row_ptr;
    const int* row_off;
    const __half* tiles;
    const __half* bias;
    int T, in, out;
    int* done;    // [batch][nqb] counters, zero at launch; the last CTA to finish zeroes them
    int* exited;  // CTAs that have finished, zero at launch
    int* ticket;  // next piece of work to hand out, zero at launch
    unsigned long long* trace;  // test hook: [ticket][4] = start ns, end ns, SM, CTA (null: no trace)
    int n_done;   // batch * nqb
    int nqb;      // 128-query blocks per sequence
    int n_att;    // batch * nqb * nhead attention units
    int npanel;   // panels of 128 output features
    int n_items;  // npanel * ceil(T / 128) projection items
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Waits until *p >= target; gives up when the poll limit runs out or an error was recorded.
__device__ __forceinline__ bool wait_count(const int* p, int target, volatile int* abort_flag,
                                           const int* err_word) {
    for (uint32_t it = 0; it < FUSE_POLL_LIMIT; ++it) {
        if (ld_acquire_gpu(p) >= target) return true;
        if (*abort_flag || *reinterpret_cast<const volatile int*>(err_word) != 0) return false;
        __nanosleep(100);
    }
    return false;
}

template <int MASK>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_fuse_o_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmZ,
                        const AttnArgs a, const __grid_constant__ CUtensorMap tmX,
                        const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmY,
                        const FuseOArgs f) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ int s_last;
    __shared__ int s_ticket;
    __shared__ unsigned long long s_t0;
    volatile int* abort_flag = &s_abort;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) s_abort = 0;
    if (warp == 1) {
        tmem_alloc(&s_tmem, a.tmem_cols);  // >= the 128 columns the projection needs
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    // Work is handed out by ticket: attention units first (heads of one query block next to
    // each other), then projection items in the order their inputs become ready.  The two kinds
    // of work have loops of their own (in one loop the compiler spills registers in both bodies),
    // and nothing but the ticket, in shared memory, lives across a piece of work.
    const volatile int* ticket = &s_ticket;
    auto take_ticket = [&]() {
        if (threadIdx.x == 0) {
            s_ticket = atomicAdd(f.ticket, 1);
            if (f.trace) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(s_t0));
        }
        __syncthreads();
    };
    auto trace_done = [&]() {
        if (f.trace && threadIdx.x == 0) {
            unsigned long long t_end;
            unsigned smid;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            unsigned long long* rec = f.trace + 4 * static_cast<size_t>(*ticket);
            rec[0] = s_t0;
            rec[1] = t_end;
            rec[2] = smid;
            rec[3] = blockIdx.x;
        }
    };

    pdl_launch_dependents();
    // Q, K, V come from earlier kernels, Z and out may still be read by them - and an earlier
    // launch that uses the same counters must have left them at zero before a ticket is taken
    // (kernels launched as dependents start before their predecessors finish).
    pdl_wait();
    take_ticket();
    while (*ticket < f.n_att && !*abort_flag) {
        {
            const int t = *ticket;
            const int h = t % a.nhead;
            const int rest = t / a.nhead;
            int qb = rest % f.nqb;
            // causal: a sequence's last query blocks have the most key blocks and go first
            if (MASK == ET_MASK_CAUSAL) qb = f.nqb - 1 - qb;
            attention_cta<MASK, true>(tmQ, tmK, tmV, tmZ, a, smem, qb * BQ, h, rest / f.nqb, s_tmem,
                                      abort_flag);
        }
        // (the body ends with a CTA-wide barrier after its stores to Z have completed)
        if (threadIdx.x == 0 && !*abort_flag) {
            const int rest = *ticket / a.nhead;
            int qb = rest % f.nqb;
            if (MASK == ET_MASK_CAUSAL) qb = f.nqb - 1 - qb;
            __threadfence();
            atomicAdd(f.done + (rest / f.nqb) * f.nqb + qb, 1);
        }
        trace_done();
        take_ticket();
    }
    // the ticket in hand is the CTA's first projection item (or past the end)
    while (*ticket < f.n_att + f.n_items && !*abort_flag) {
        const int i = *ticket - f.n_att;
        const int m0 = (i / f.npanel) * TBM;
        // called inside the item once its index tables are built: one thread waits for the
        // query blocks the token block overlaps, then every thread passes the barrier
        auto wait_inputs = [&]() {
            if (threadIdx.x == 0) {
                const int t1 = m0 + TBM < f.T ? m0 + TBM : f.T;
                bool ok = true;
                for (int b = m0 / a.seq; ok && b <= (t1 - 1) / a.seq; ++b) {
                    const int lo = m0 - b * a.seq > 0 ? m0 - b * a.seq : 0;
                    const int hi = t1 - b * a.seq < a.seq ? t1 - b * a.seq : a.seq;
                    for (int qb = lo / BQ; ok && qb <= (hi - 1) / BQ; ++qb)
                        ok = wait_count(f.done + b * f.nqb + qb, a.nhead, abort_flag, a.err_word);
                }
                if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_FUSE_O);
                fence_proxy_async_global();
            }
            __syncthreads();
        };
        linear_tile_cta<false, ET_ACT_NONE, 1, true>(tmX, tmW, tmY, f.row_ptr, f.row_off, nullptr,
                                                    nullptr, f.tiles, f.bias, f.T, f.in, f.out,
                                                    a.err_word, smem, i % f.npanel, m0, s_tmem,
                                                    abort_flag, wait_inputs);
        trace_done();
        take_ticket();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(s_tmem, a.tmem_cols);

    // The last CTA to get here leaves the counters as it found them (every other CTA is past
    // its last wait), also when the run was abandoned after an error.
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(f.exited, 1) == static_cast<int>(gridDim.x) - 1 ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        for (int i = threadIdx.x; i < f.n_done; i += ATT_THREADS) f.done[i] = 0;
        if (threadIdx.x == 0) {
            *f.exited = 0;
            *f.ticket = 0;
        }
    }
}

// ---- completion counters -----------------------------------------------------------------
// Part of the library image (no allocation at call time), zero when the library is loaded and
// zero again at the end of every launch.  Calls take the slots in turn, so up to FUSE_SLOTS
// calls may be in flight on one GPU (in different streams) at once.
constexpr int FUSE_SLOTS = 16;
constexpr int FUSE_SLOT_INTS = 4096;  // batch * ceil(seq / 128) + 2 may not exceed this
static __device__ int g_fuse_o_done[FUSE_SLOTS * FUSE_SLOT_INTS];

int* fuse_o_counters() {
    static std::atomic<int*> cached[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* known = cached[dev].load(std::memory_order_acquire);
    if (known != nullptr) return known;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_fuse_o_done) != cudaSuccess || p == nullptr) return nullptr;
    cached[dev].store(static_cast<int*>(p), std::memory_order_release);
    return static_cast<int*>(p);
}

std::atomic<unsigned> g_next_slot{0};
unsigned long long* g_fuse_o_trace = nullptr;  // test hook

}  // namespace

int launch_attention_fuse_o(const __half* Q, const __half* K, const __half* V, const __half* mask,
                            __half* Z, const int* o_row_ptr, const int* o_row_off,
                            const __half* o_tiles, int o_nnz, const __half* o_bias, __half* out,
                            int batch, int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk,
                            int ldv, int emdim, int mask_kind, const int* valid_len, float scale,
                            bool single_launch, cudaStream_t stream) {
    if (!Z || !out) return ET_ERR_INVALID_ARG;
    const long vdim_l = static_cast<long>(nhead) * dh_v;
    const long nqb_l = (static_cast<long>(seq) + BQ - 1) / BQ;
    // Without a stored tile there is no projection to fuse; beyond the counter array the two
    // stand-alone kernels do the work.
    const bool fused = single_launch && o_nnz > 0 && batch > 0 && seq > 0 && nhead > 0 &&
                       dh_v > 0 && dh_v % 16 == 0 && batch * nqb_l < FUSE_SLOT_INTS - 1 &&
                       vdim_l <= MAX_IN;
    if (!fused) {
        int st = launch_attention(Q, K, V, Z, batch, seq, nhead, dh_qk, dh_v, ldq, ldk, ldv,
                                  static_cast<int>(vdim_l), mask_kind, mask, valid_len, scale, stream);
        if (st != ET_OK) return st;
        return launch_linear_tile(o_row_ptr, o_row_off, o_tiles, o_nnz, o_bias, Z, out, batch * seq,
                                  static_cast<int>(vdim_l), emdim, ET_ACT_NONE, stream);
    }
    const int vdim = static_cast<int>(vdim_l), nqb = static_cast<int>(nqb_l), ldz = vdim;
    const int T = batch * seq;
    // ---- the checks of both stand-alone launchers ----
    if (!Q || !K || !V || dh_qk <= 0 || emdim <= 0 || !o_row_ptr || !o_row_off || !o_tiles)
        return ET_ERR_INVALID_ARG;
    if (mask_kind < ET_MASK_NONE || mask_kind > ET_MASK_ADDITIVE) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_ADDITIVE && !mask) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_PADDING && !valid_len) return ET_ERR_INVALID_ARG;
    if (!(scale > 0.f)) return ET_ERR_INVALID_ARG;
    if (dh_qk % 16 || dh_qk > 128 || dh_v > 128) return ET_ERR_SHAPE;
    if (ldq % 8 || ldk % 8 || ldv % 8 || vdim % 16 || emdim % 16) return ET_ERR_SHAPE;
    if (ldq < nhead * dh_qk || ldk < nhead * dh_qk || ldv < vdim) return ET_ERR_SHAPE;
    if (batch > 65535 || nhead > 65535) return ET_ERR_SHAPE;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(Z) || !aligned16(out) ||
        !aligned16(o_tiles) || (o_bias && !aligned16(o_bias)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    int* counters = fuse_o_counters();
    if (!err || !counters) return ET_ERR_NO_DEVICE;

    CUtensorMap tmQ, tmK, tmV, tmZ, tmX, tmW, tmY;
    auto make3 = [&](CUtensorMap* m, const __half* p, int ld, int width, uint32_t box_rows) {
        const uint64_t dims[3] = {static_cast<uint64_t>(width), static_cast<uint64_t>(seq),
                                  static_cast<uint64_t>(batch)};
        const uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2,
                                     static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(seq)};
        const uint32_t box[3] = {64, box_rows, 1};
        return make_tensor_map_f16(m, p, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    };
    auto make2 = [&](CUtensorMap* m, const __half* p, uint64_t width, uint64_t rows, uint32_t bx,
                     uint32_t by, CUtensorMapSwizzle sw) {
        const uint64_t dims[2] = {width, rows};
        const uint64_t strides[1] = {width * 2};
        const uint32_t box[2] = {bx, by};
        return make_tensor_map_f16(m, p, 2, dims, strides, box, sw);
    };
    int st;
    if ((st = make3(&tmQ, Q, ldq, nhead * dh_qk, 128)) != ET_OK) return st;
    if ((st = make3(&tmK, K, ldk, nhead * dh_qk, 128)) != ET_OK) return st;
    if ((st = make3(&tmV, V, ldv, vdim, 128)) != ET_OK) return st;
    const bool tma_out = dh_v % 64 == 0;
    tmZ = tmQ;
    if (tma_out && (st = make3(&tmZ, Z, ldz, vdim, 32)) != ET_OK) return st;
    if ((st = make2(&tmX, Z, vdim, T, CHUNK, TBM, CU_TENSOR_MAP_SWIZZLE_128B)) != ET_OK) return st;
    // the tile array seen as a [nnz * 16, 16] matrix: one box = one stored tile
    if ((st = make2(&tmW, o_tiles, 16, static_cast<uint64_t>(o_nnz) * 16, 16, 16,
                    CU_TENSOR_MAP_SWIZZLE_32B)) != ET_OK)
        return st;
    if ((st = make2(&tmY, out, emdim, T, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)) != ET_OK) return st;

    AttnArgs a;
    a.Z = Z;
    a.mask = mask;
    a.valid_len = valid_len;
    a.ldz = ldz;
    a.batch = batch;
    a.seq = seq;
    a.nhead = nhead;
    a.dh_qk = dh_qk;
    a.dh_v = dh_v;
    a.mask_kind = mask_kind;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.err_word = err;
    a.col_id = nullptr;
    a.head_ptr = nullptr;
    const int nqa = (dh_qk + 63) / 64, nva = (dh_v + 63) / 64;
    a.nva_max = nva;
    a.tmem_cols = TMEM_COLS_ATT;
    a.tma_out = tma_out ? 1 : 0;
    a.n_units = 0;
    for (int u = 0; u < ATT_MAX_UNITS; ++u) {
        a.unit_head[u] = 0;
        a.unit_first[u] = 0;
    }

    const int nbc = vdim / 16, nchunk = (vdim + CHUNK - 1) / CHUNK, nchunk_p = (nchunk + 3) & ~3;
    FuseOArgs f;
    f.row_ptr = o_row_ptr;
    f.row_off = o_row_off;
    f.tiles = o_tiles;
    f.bias = o_bias;
    f.T = T;
    f.in = vdim;
    f.out = emdim;
    f.nqb = nqb;
    f.n_att = batch * nqb * nhead;
    f.npanel = (emdim + TBN - 1) / TBN;
    f.n_items = f.npanel * ((T + TBM - 1) / TBM);
    f.done = counters + (g_next_slot.fetch_add(1, std::memory_order_relaxed) % FUSE_SLOTS) * FUSE_SLOT_INTS;
    f.exited = f.done + FUSE_SLOT_INTS - 1;
    f.ticket = f.done + FUSE_SLOT_INTS - 2;
    f.trace = g_fuse_o_trace;
    f.n_done = batch * nqb;

    const int att_bytes = (2 * nqa + nva + 2) * ATOM_BYTES + EXTRA_BYTES;
    const int tile_bytes = RING_BYTES + 256 + TBN * 4 + nchunk_p * 4 + PANEL_ROWS * nbc * 4 +
                           PANEL_ROWS * nchunk_p * 2;
    const int smem_bytes = (att_bytes > tile_bytes ? att_bytes : tile_bytes) + 1024;

    int dev = 0;
    cudaGetDevice(&dev);
    auto go = [&](auto kern, int slot) -> int {
        static std::atomic<int> attr_bytes[4][64] = {};
        if (dev >= 0 && dev < 64 && attr_bytes[slot][dev] < smem_bytes) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     smem_bytes) != cudaSuccess)
                return ET_ERR_CUDA;
            attr_bytes[slot][dev] = smem_bytes;
        }
        // two CTAs fit an SM (registers, shared memory, 256 of the 512 tensor-memory columns
        // each); more CTAs than that would only queue behind them
        const int sms = sm_count() > 0 ? sm_count() : 148;
        const long want = static_cast<long>(f.n_att) + f.n_items;
        const long cap = 2L * sms;
        return launch_kernel(kern, dim3(static_cast<unsigned>(want < cap ? want : cap)),
                             dim3(ATT_THREADS), smem_bytes, stream, tmQ, tmK, tmV, tmZ, a, tmX, tmW,
                             tmY, f) == cudaSuccess
                   ? ET_OK
                   : ET_ERR_CUDA;
    };
    switch (mask_kind) {
        case ET_MASK_CAUSAL: return go(attention_fuse_o_kernel<ET_MASK_CAUSAL>, 1);
        case ET_MASK_PADDING: return go(attention_fuse_o_kernel<ET_MASK_PADDING>, 2);
        case ET_MASK_ADDITIVE: return go(attention_fuse_o_kernel<ET_MASK_ADDITIVE>, 3);
        default: return go(attention_fuse_o_kernel<ET_MASK_NONE>, 0);
    }
}

}  // namespace et

extern "C" {

#ifdef ET_TEST_HOOKS
// Test hook: device array of 4 x (work items) 64-bit words that receives each item's start and
// end time (ns), SM and CTA; null switches the trace off.
void et_debug_set_fuse_o_trace(void* p) { et::g_fuse_o_trace = static_cast<unsigned long long*>(p); }
#endif  // ET_TEST_HOOKS

int et_attention_fuse_o_fwd(const et_half* Q, const et_half* K, const et_half* V,
                            const et_half* mask, et_half* Z, const int32_t* o_row_ptr,
                            const int32_t* o_row_off, const et_half* o_tiles, int o_nnz,
                            const et_half* o_bias, et_half* out, int batch, int seq, int nhead,
                            int dh_qk, int dh_v, int ldq, int ldk, int ldv, int emdim,
                            int mask_kind, const int32_t* valid_len, float scale,
                            et_stream stream) {
    return et::launch_attention_fuse_o(
        reinterpret_cast<const __half*>(Q), reinterpret_cast<const __half*>(K),
        reinterpret_cast<const __half*>(V), reinterpret_cast<const __half*>(mask),
        reinterpret_cast<__half*>(Z), o_row_ptr, o_row_off, reinterpret_cast<const __half*>(o_tiles),
        o_nnz, reinterpret_cast<const __half*>(o_bias), reinterpret_cast<__half*>(out), batch, seq,
        nhead, dh_qk, dh_v, ldq, ldk, ldv, emdim, mask_kind, valid_len, scale, false,
        static_cast<cudaStream_t>(stream));
}

int et_attention_fuse_o_single_launch_fwd(const et_half* Q, const et_half* K, const et_half* V,
                                          const et_half* mask, et_half* Z, const int32_t* o_row_ptr,
                                          const int32_t* o_row_off, const et_half* o_tiles, int o_nnz,
                                          const et_half* o_bias, et_half* out, int batch, int seq,
                                          int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv,
                                          int emdim, int mask_kind, const int32_t* valid_len,
                                          float scale, et_stream stream) {
    return et::launch_attention_fuse_o(
        reinterpret_cast<const __half*>(Q), reinterpret_cast<const __half*>(K),
        reinterpret_cast<const __half*>(V), reinterpret_cast<const __half*>(mask),
        reinterpret_cast<__half*>(Z), o_row_ptr, o_row_off, reinterpret_cast<const __half*>(o_tiles),
        o_nnz, reinterpret_cast<const __half*>(o_bias), reinterpret_cast<__half*>(out), batch, seq,
        nhead, dh_qk, dh_v, ldq, ldk, ldv, emdim, mask_kind, valid_len, scale, true,
        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
