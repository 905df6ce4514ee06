// Tile-pruned Linear (16x16 tile-CSR, block rows = output features) on tcgen05.
//
// One CTA owns 128 tokens and a panel of 8 output block rows (128 output features,
// 8 x 16 fp32 accumulator columns in tensor memory).  The input is walked in chunks of
// 64 features (4 block columns).  In the prologue the CTA builds, in shared memory, a
// table tile_at[row][block column] of the panel's stored tiles and one 32-bit presence
// mask per chunk (bit = row * 4 + column inside the chunk).  Chunks without any stored
// tile are skipped by every role, so only non-zero tiles and the activations they need are
// loaded.  For a chunk, warp 0 fetches the 128x64 activation slab (TMA, 128-byte swizzle)
// and each stored tile (TMA, 32-byte swizzle: a 16x16 fp16 tile is 16 rows of 32 bytes) into
// densely packed 512-byte slots (16 per stage when no chunk of the panel holds more, else
// 32; the ring gets as many stages as fit); one thread of warp 1 issues one tcgen05.mma
// (M=128, N=16, K=16) per stored tile, choosing the activation slab by descriptor address
// and the accumulator columns by block row; warps 2-9 run the bias / activation / fp16
// epilogue through a swizzled staging tile and TMA stores, writing bias alone for block
// rows that hold no tile.
//
// Packed form.  Issuing one TMA per 512-byte tile makes the producer the bottleneck at high
// sparsity, so the operator can re-pack its (static) weights once: tiles are reordered into
// (pair of panels, chunk, panel, row, column) order - the order in which the kernels consume them - and
// stored pre-swizzled, with one presence mask and one tile offset per (panel, chunk).  A
// chunk's tiles are then one contiguous run fetched by a single bulk copy, and the prologue
// reads ready-made masks instead of building them.  The re-packing is a pure permutation of
// the tile-CSR arrays (et_tile_pack_plan on the host indices, et_tile_pack_tiles on the GPU).
#include <vector>

#include "linear_tile_body.cuh"

namespace et {

using namespace tile;

namespace {

// PACKED, ACT, NP: see linear_tile_cta.  One CTA per (panel or pair of panels, 128-token block).
template <bool PACKED, int ACT, int NP>
__global__ void __launch_bounds__(TILE_THREADS, 2)
linear_tile_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ CUtensorMap tmY, const int* __restrict__ row_ptr,
                   const int* __restrict__ row_off, const uint32_t* __restrict__ pk_mask,
                   const int* __restrict__ pk_off, const __half* __restrict__ pk_tiles,
                   const __half* __restrict__ bias, int T, int in, int out, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    linear_tile_cta<PACKED, ACT, NP, false>(tmX, tmW, tmY, row_ptr, row_off, pk_mask, pk_off, pk_tiles,
                                            bias, T, in, out, err_word, smem, blockIdx.x * NP,
                                            blockIdx.y * TBM, 0u, nullptr);
}

__global__ void tile_fill_bias_kernel(__half* __restrict__ Y, const __half* __restrict__ bias,
                                      size_t rows, int cols, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t total = rows * cols;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float b = bias ? __half2float(__ldg(bias + (i % cols))) : 0.f;
        Y[i] = __float2half_rn(apply_act(b, act));
    }
}

}  // namespace

// One CTA per block row: dense[br * 16 + i][off * 16 + j] = tile[i][j] for every stored tile.
__global__ void densify_tiles_kernel(const int* __restrict__ row_ptr, const int* __restrict__ row_off,
                                     const __half* __restrict__ tiles, int nbc, int in,
                                     __half* __restrict__ dense) {
    const int br = blockIdx.x;
    const int i = threadIdx.x >> 4, j = threadIdx.x & 15;
    for (int t = __ldg(row_ptr + br); t < __ldg(row_ptr + br + 1); ++t) {
        const int off = __ldg(row_off + t);
        if (off < 0 || off >= nbc) continue;
        dense[(static_cast<size_t>(br) * 16 + i) * in + off * 16 + j] =
            tiles[static_cast<size_t>(t) * 256 + threadIdx.x];
    }
}

// dst[i] = tile perm[i] of src, stored with the 32-byte swizzle the tensor core expects
// (16-byte half j of row r lands at half j ^ ((r >> 2) & 1)).
__global__ void pack_tiles_kernel(const uint4* __restrict__ src, const int* __restrict__ perm,
                                  uint4* __restrict__ dst, int nnz) {
    const size_t total = static_cast<size_t>(nnz) * 32;  // 32 x 16 bytes per tile
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = i >> 5;
        const int c = static_cast<int>(i & 31);  // 16-byte unit inside the tile: row = c / 2
        const int row = c >> 1, hf = c & 1;
        const int dc = (row << 1) | (hf ^ ((row >> 2) & 1));
        dst[t * 32 + dc] = __ldg(src + static_cast<size_t>(__ldg(perm + t)) * 32 + c);
    }
}

int g_tile_wide = -1;  // test hook: -1 = automatic, 0 = one panel per CTA, 1 = two panels per CTA

namespace {
int launch_tile_common(bool packed, const int* row_ptr, const int* row_off, const uint32_t* pk_mask,
                       const int* pk_off, const __half* tiles, int nnz_tiles, const __half* bias,
                       const __half* X, __half* Y, int T, int in, int out, int act,
                       cudaStream_t stream) {
    if (!row_ptr || !X || !Y || T <= 0 || in <= 0 || out <= 0 || nnz_tiles < 0)
        return ET_ERR_INVALID_ARG;
    if (nnz_tiles > 0 && !tiles) return ET_ERR_INVALID_ARG;
    if (nnz_tiles > 0 && (packed ? (!pk_mask || !pk_off) : !row_off)) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16 || in > MAX_IN) return ET_ERR_SHAPE;
    if (!aligned16(X) || !aligned16(Y) || (tiles && !aligned16(tiles)) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;

    if (nnz_tiles == 0) {
        const size_t total = static_cast<size_t>(T) * out;
        const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        return launch_kernel(tile_fill_bias_kernel, dim3(blocks), dim3(256), 0, stream, Y, bias,
                             static_cast<size_t>(T), out, act) == cudaSuccess
                   ? ET_OK
                   : ET_ERR_CUDA;
    }

    CUtensorMap tmX, tmW, tmY;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(in), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(in) * 2};
        const uint32_t box[2] = {CHUNK, TBM};
        int st = make_tensor_map_f16(&tmX, X, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    {
        // the tile array seen as a [nnz * 16, 16] matrix: one box = one stored tile
        const uint64_t dims[2] = {16, static_cast<uint64_t>(nnz_tiles) * 16};
        const uint64_t strides[1] = {32};
        const uint32_t box[2] = {16, 16};
        int st = make_tensor_map_f16(&tmW, tiles, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B);
        if (st != ET_OK) return st;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(out), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(out) * 2};
        const uint32_t box[2] = {64, 32};
        int st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    const int nbc = in / 16, nchunk = (in + CHUNK - 1) / CHUNK, nchunk_p = (nchunk + 3) & ~3;
    const int npanel = (out + TBN - 1) / TBN;
    // two panels per CTA when that grid still holds more CTAs than fit at once (measured on
    // B200: 768 -> 3072 at 2048 tokens gains 20 %, 768 -> 2304 with 144 wide CTAs loses 25 %):
    // the panels share every activation slab
    const long wide_ctas = static_cast<long>((npanel + 1) / 2) * ((T + TBM - 1) / TBM);
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const bool wide =
        packed && g_tile_wide != 0 && (g_tile_wide > 0 || (npanel >= 2 && wide_ctas * 4 >= sms * 5L));
    const int np = wide ? 2 : 1;
    const int smem_bytes = RING_BYTES + 256 + np * TBN * 4 + np * nchunk_p * 4 +
                           (packed ? np * nchunk_p * 4 : PANEL_ROWS * nbc * 4) +
                           np * PANEL_ROWS * nchunk_p * 2 + 1024;
    int dev = 0;
    cudaGetDevice(&dev);
    dim3 grid((npanel + np - 1) / np, (T + TBM - 1) / TBM);
    auto go = [&](auto kern, int slot) -> cudaError_t {
        static std::atomic<int> attr_bytes[9][64] = {};
        if (dev >= 0 && dev < 64 && attr_bytes[slot][dev] < smem_bytes) {
            const cudaError_t ea =
                cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
            if (ea != cudaSuccess) return ea;
            attr_bytes[slot][dev] = smem_bytes;
        }
        return launch_kernel(kern, grid, dim3(TILE_THREADS), smem_bytes, stream, tmX, tmW, tmY,
                             row_ptr, row_off, pk_mask, pk_off, tiles, bias, T, in, out, err);
    };
    cudaError_t e;
    if (wide) {
        e = act == ET_ACT_GELU   ? go(linear_tile_kernel<true, ET_ACT_GELU, 2>, 6)
            : act == ET_ACT_RELU ? go(linear_tile_kernel<true, ET_ACT_RELU, 2>, 7)
                                 : go(linear_tile_kernel<true, ET_ACT_NONE, 2>, 8);
    } else if (packed) {
        e = act == ET_ACT_GELU   ? go(linear_tile_kernel<true, ET_ACT_GELU, 1>, 0)
            : act == ET_ACT_RELU ? go(linear_tile_kernel<true, ET_ACT_RELU, 1>, 1)
                                 : go(linear_tile_kernel<true, ET_ACT_NONE, 1>, 2);
    } else {
        e = act == ET_ACT_GELU   ? go(linear_tile_kernel<false, ET_ACT_GELU, 1>, 3)
            : act == ET_ACT_RELU ? go(linear_tile_kernel<false, ET_ACT_RELU, 1>, 4)
                                 : go(linear_tile_kernel<false, ET_ACT_NONE, 1>, 5);
    }
    return e == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}
}  // namespace

int g_tile_rows = 0;  // test hook: 1 = tile-CSR arrays run on the warp-level kernel (linear_tile_rows.cu)

int launch_linear_tile(const int* row_ptr, const int* row_off, const __half* tiles, int nnz_tiles,
                       const __half* bias, const __half* X, __half* Y, int T, int in, int out,
                       int act, cudaStream_t stream) {
    if (g_tile_rows != 0 && nnz_tiles > 0 && linear_tile_rows_supported(in, out))
        return launch_linear_tile_rows(row_ptr, row_off, tiles, nnz_tiles, bias, X, Y, T, in, out, act,
                                       stream);
    return launch_tile_common(false, row_ptr, row_off, nullptr, nullptr, tiles, nnz_tiles, bias, X, Y,
                              T, in, out, act, stream);
}

int launch_linear_tile_packed(const int* row_ptr, const uint32_t* pk_mask, const int* pk_off,
                              const __half* pk_tiles, int nnz_tiles, const __half* bias,
                              const __half* X, __half* Y, int T, int in, int out, int act,
                              cudaStream_t stream) {
    // Measured on B200 (768 / 3072-wide BERT shapes, 2048 and 8192 tokens, 80-95 % of the tiles
    // pruned): the one-item-per-CTA kernel - one panel per CTA while the grid is small, two panels
    // once two-panel items cover the SMs 1.25 times - is never slower than the persistent kernel
    // by more than 2 % and up to 30 % faster on small grids (3072 -> 768 at 2048 tokens: 20.5 us
    // against 27.2), so the persistent form runs only when the test hook selects it.
    if (nnz_tiles > 0 && tile_packed_mode() == 1)
        return launch_linear_tile_persist(row_ptr, pk_mask, pk_off, pk_tiles, nnz_tiles, bias, X, Y, T, in,
                                          out, act, stream);
    return launch_tile_common(true, row_ptr, nullptr, pk_mask, pk_off, pk_tiles, nnz_tiles, bias, X, Y,
                              T, in, out, act, stream);
}

}  // namespace et

extern "C" {

#ifdef ET_TEST_HOOKS
// Test hook: -1 = automatic, 0 = one panel per CTA, 1 = two panels per CTA (packed weights).
void et_debug_set_tile_wide(int mode) { et::g_tile_wide = mode; }
// Test hook: 1 = tile-CSR arrays run on the warp-level kernel, 0 = on the tcgen05 one (default).
void et_debug_set_tile_rows(int on) { et::g_tile_rows = on; }
#endif  // ET_TEST_HOOKS

int et_linear_tile_fwd(const int32_t* row_ptr, const int32_t* row_off, const et_half* tiles,
                       int nnz_tiles, const et_half* bias, const et_half* X, et_half* Y, int T,
                       int in, int out, int act, et_stream stream) {
    return et::launch_linear_tile(row_ptr, row_off, reinterpret_cast<const __half*>(tiles),
                                  nnz_tiles, reinterpret_cast<const __half*>(bias),
                                  reinterpret_cast<const __half*>(X), reinterpret_cast<__half*>(Y),
                                  T, in, out, act, static_cast<cudaStream_t>(stream));
}

// ---- re-packing of tile-CSR weights for the packed forward ---------------------------------
// Sizes: the packed layout has ceil(out / 128) panels x ceil(in / 64) chunks.
int et_tile_pack_dims(int in, int out, int* npanel, int* nchunk) {
    if (in <= 0 || out <= 0 || !npanel || !nchunk) return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16) return ET_ERR_SHAPE;
    *npanel = (out + et::TBN - 1) / et::TBN;
    *nchunk = (in + et::CHUNK - 1) / et::CHUNK;
    return ET_OK;
}

// Host side (index arrays in host memory): computes, for every (panel, chunk), the presence
// mask (bit = row_in_panel * 4 + column_in_chunk) and the first packed tile, and the
// permutation perm[i] = tile-CSR index of the i-th packed tile.
int et_tile_pack_plan(const int32_t* row_ptr, const int32_t* row_off, int nnz_tiles, int in, int out,
                      uint32_t* pk_mask, int32_t* pk_off, int32_t* perm) {
    int st = et_validate_tile_mat(row_ptr, row_off, nnz_tiles, in, out);
    if (st != ET_OK) return st;
    if (!pk_mask || !pk_off || (nnz_tiles > 0 && !perm)) return ET_ERR_INVALID_ARG;
    const int npanel = (out + et::TBN - 1) / et::TBN, nchunk = (in + et::CHUNK - 1) / et::CHUNK;
    const int nbr = out / 16;
    int next = 0;
    // Packed order: (pair of panels, chunk, panel of the pair, row, column).  The tiles of one
    // (panel, chunk) stay one contiguous run, which is all the one-item kernels rely on, and the
    // two panels of a pair follow each other inside a chunk, so the persistent kernel fetches a
    // pair's tiles of a chunk with one bulk copy.
    for (int p0 = 0; p0 < npanel; p0 += 2) {
        // cursor per block row of the pair (columns ascend inside a row)
        int cur[2 * et::PANEL_ROWS], end[2 * et::PANEL_ROWS];
        for (int r = 0; r < 2 * et::PANEL_ROWS; ++r) {
            const int br = p0 * et::PANEL_ROWS + r;
            cur[r] = br < nbr ? row_ptr[br] : 0;
            end[r] = br < nbr ? row_ptr[br + 1] : 0;
        }
        for (int c = 0; c < nchunk; ++c) {
            for (int k = 0; k < 2 && p0 + k < npanel; ++k) {
                uint32_t mask = 0;
                pk_off[(p0 + k) * nchunk + c] = next;
                for (int r = 0; r < et::PANEL_ROWS; ++r) {
                    int& cu = cur[k * et::PANEL_ROWS + r];
                    const int en = end[k * et::PANEL_ROWS + r];
                    while (cu < en && row_off[cu] < (c + 1) * 4) {
                        mask |= 1u << (r * 4 + (row_off[cu] & 3));
                        perm[next++] = cu++;
                    }
                }
                pk_mask[(p0 + k) * nchunk + c] = mask;
            }
        }
    }
    return next == nnz_tiles ? ET_OK : ET_ERR_INDEX;
}

// Device side: packed_tiles[i] = tiles[perm[i]], pre-swizzled.  perm is a device array.
int et_tile_pack_tiles(const et_half* tiles, const int32_t* perm, int nnz_tiles,
                       et_half* packed_tiles, et_stream stream) {
    if (nnz_tiles < 0 || (nnz_tiles > 0 && (!tiles || !perm || !packed_tiles)))
        return ET_ERR_INVALID_ARG;
    if (nnz_tiles == 0) return ET_OK;
    if (!et::aligned16(tiles) || !et::aligned16(packed_tiles)) return ET_ERR_ALIGNMENT;
    const size_t total = static_cast<size_t>(nnz_tiles) * 32;
    const int blocks = static_cast<int>((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
    et::count_launch();
    et::pack_tiles_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4*>(tiles), perm, reinterpret_cast<uint4*>(packed_tiles),
        nnz_tiles);
    return cudaGetLastError() == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

int et_linear_tile_packed_fwd(const int32_t* row_ptr, const uint32_t* pk_mask, const int32_t* pk_off,
                              const et_half* pk_tiles, int nnz_tiles, const et_half* bias,
                              const et_half* X, et_half* Y, int T, int in, int out, int act,
                              et_stream stream) {
    return et::launch_linear_tile_packed(row_ptr, pk_mask, pk_off,
                                         reinterpret_cast<const __half*>(pk_tiles), nnz_tiles,
                                         reinterpret_cast<const __half*>(bias),
                                         reinterpret_cast<const __half*>(X),
                                         reinterpret_cast<__half*>(Y), T, in, out, act,
                                         static_cast<cudaStream_t>(stream));
}

// ---- plan-time choice between the tile kernel and dense math -------------------------------
// A 128 x 16 x 16 tensor-core product occupies the tensor pipe for about 45 cycles on B200
// whatever its operands' source, against 8 cycles of arithmetic, and every panel of the tile
// kernel streams the whole activation matrix.  Measured at 2048 tokens on BERT-base shapes
// (packed tile kernel time / dense GEMM time): 768 -> 3072 with two panels per CTA 1.21 at
// 80 % sparsity, 0.98 at 90 %, 0.88 at 95 %; 768 -> 2304 0.97 / 0.87 / 0.83; 768 -> 768 and
// 3072 -> 768 never below 1.0 up to 97 %.  So weights are expanded once and served by the dense
// GEMM unless they are both wide and sparse enough.
int et_tile_prefer_dense(int in, int out, int nnz_tiles) {
    if (in <= 0 || out <= 0 || (in & 15) || (out & 15)) return 0;
    const double total = static_cast<double>(in >> 4) * (out >> 4);
    const double keep = out >= 3072 ? 0.10 : (out >= 2048 ? 0.15 : 0.02);
    return nnz_tiles > keep * total ? 1 : 0;
}

int et_tile_densify(const int32_t* row_ptr, const int32_t* row_off, const et_half* tiles,
                    int nnz_tiles, int in, int out, et_half* dense, et_stream stream) {
    if (!row_ptr || !dense || in <= 0 || out <= 0 || nnz_tiles < 0) return ET_ERR_INVALID_ARG;
    if ((in & 15) || (out & 15)) return ET_ERR_SHAPE;
    if (nnz_tiles > 0 && (!row_off || !tiles)) return ET_ERR_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(dense, 0, static_cast<size_t>(in) * out * sizeof(__half), s) != cudaSuccess)
        return ET_ERR_CUDA;
    if (nnz_tiles > 0) {
        et::count_launch();
        et::densify_tiles_kernel<<<out >> 4, 256, 0, s>>>(row_ptr, row_off,
                                                           reinterpret_cast<const __half*>(tiles),
                                                           in >> 4, in,
                                                           reinterpret_cast<__half*>(dense));
        if (cudaGetLastError() != cudaSuccess) return ET_ERR_CUDA;
    }
    return ET_OK;
}

}  // extern "C"
