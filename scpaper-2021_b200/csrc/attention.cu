// On-the-fly fused self-attention on tcgen05 tensor cores: scores never leave the SM.
//
// One CTA owns 128 queries of one (sequence, head).  Warp 0 streams Q once and then K / V
// blocks of 128 keys with TMA (3-D tensor maps {feature, position, sequence}, so positions
// past the end of a sequence are zero-filled and never read the next sequence).  One
// thread of warp 1 issues S = Q.K^T (M=128, N=128) into tensor memory.  Eight softmax warps
// share the 128 x 128 score block: two per tensor-memory lane quadrant, each thread owning
// 64 keys of one query row, which it reads from tensor memory ONCE and keeps in registers.
// The two halves of a row exchange their maxima through shared memory, then each thread
// computes exp2 (with log2(e)/sqrt(dh) folded into one FMA), keeps a running max / partial
// sum (online softmax across key blocks), writes its fp16 probabilities into the
// 128-byte-swizzled shared-memory tile that is the A operand of the second product and
// rescales its share of the output accumulator when the running max was raised (only when a
// block exceeds it by more than 2^8, so a few times per row).  The MMA thread issues the next
// block's Q.K^T ahead of O += P.V (V consumed directly in its row-major, MN-major layout), so
// the scores of block j+1 are ready when the softmax warps finish block j.  After
// the last block the row sums are combined, each thread scales its share of the output
// columns and the tile leaves through a swizzled staging buffer and TMA stores.
// All waits are bounded.
#include "attention_body.cuh"

namespace et {

namespace {

using namespace attn;

// One CTA per (128-query block, head or work unit, sequence).
template <int MASK>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmZ,
                 const AttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // causal: the last query blocks have the most key blocks; they are launched first so that
    // the short ones fill the tail of the grid
    const int qb_first = a.n_units > 0 ? a.unit_first[blockIdx.y] : 0;
    const int q0 =
        (qb_first + (MASK == ET_MASK_CAUSAL ? gridDim.x - 1 - blockIdx.x : blockIdx.x)) * BQ;
    const int h = a.n_units > 0 ? a.unit_head[blockIdx.y] : blockIdx.y;
    attention_cta<MASK, false>(tmQ, tmK, tmV, tmZ, a, smem, q0, h, blockIdx.z, 0u, nullptr);
}

int launch_attention_impl(const __half* Q, const __half* K, const __half* V, __half* Z, int batch,
                          int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv,
                          int ldz, int mask_kind, const __half* mask, const int* valid_len,
                          float scale, const int* col_id, const int* head_ptr, int nnz_col,
                          cudaStream_t stream, const int* unit_head = nullptr,
                          const int* unit_first = nullptr, int n_units = 0, int blocks_per_unit = 0) {
    if (n_units < 0 || n_units > ATT_MAX_UNITS) return ET_ERR_SHAPE;
    if (n_units > 0) {
        if (!unit_head || !unit_first || blocks_per_unit <= 0) return ET_ERR_INVALID_ARG;
        for (int u = 0; u < n_units; ++u)
            if (unit_head[u] < 0 || unit_head[u] >= nhead || unit_head[u] > 255 || unit_first[u] < 0 ||
                (unit_first[u] + blocks_per_unit - 1) * BQ >= seq || unit_first[u] > 65535)
                return ET_ERR_INDEX;
    }
    if (!Q || !K || !V || !Z || batch <= 0 || seq <= 0 || nhead <= 0 || dh_qk <= 0 || dh_v <= 0)
        return ET_ERR_INVALID_ARG;
    if (mask_kind < ET_MASK_NONE || mask_kind > ET_MASK_ADDITIVE) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_ADDITIVE && !mask) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_PADDING && !valid_len) return ET_ERR_INVALID_ARG;
    if (!(scale > 0.f)) return ET_ERR_INVALID_ARG;
    if (dh_qk % 16 || dh_v % 16 || dh_qk > 128 || dh_v > 128) return ET_ERR_SHAPE;
    if (ldq % 8 || ldk % 8 || ldv % 8 || ldz % 8) return ET_ERR_SHAPE;
    const bool pruned = head_ptr != nullptr;
    if (pruned && (!col_id || nnz_col <= 0)) return ET_ERR_INVALID_ARG;
    if (ldq < nhead * dh_qk || ldk < nhead * dh_qk || ldz < nhead * dh_v) return ET_ERR_SHAPE;
    if (ldv < (pruned ? nnz_col : nhead * dh_v)) return ET_ERR_SHAPE;
    if (batch > 65535 || nhead > 65535) return ET_ERR_SHAPE;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(Z)) return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;

    CUtensorMap tmQ, tmK, tmV, tmZ;
    auto make = [&](CUtensorMap* m, const __half* p, int ld, int width, uint32_t box_rows) {
        const uint64_t dims[3] = {static_cast<uint64_t>(width), static_cast<uint64_t>(seq),
                                  static_cast<uint64_t>(batch)};
        const uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2,
                                     static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(seq)};
        const uint32_t box[3] = {64, box_rows, 1};
        return make_tensor_map_f16(m, p, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    };
    int st;
    if ((st = make(&tmQ, Q, ldq, nhead * dh_qk, 128)) != ET_OK) return st;
    if ((st = make(&tmK, K, ldk, nhead * dh_qk, 128)) != ET_OK) return st;
    if ((st = make(&tmV, V, ldv, pruned ? nnz_col : nhead * dh_v, 128)) != ET_OK) return st;
    // the output leaves through 64-column x 32-row TMA boxes when heads are whole atoms wide
    const bool tma_out = !pruned && (dh_v % 64 == 0);
    tmZ = tmQ;
    if (tma_out && (st = make(&tmZ, Z, ldz, nhead * dh_v, 32)) != ET_OK) return st;

    // a compressed V window may start up to 7 features before the head's first kept feature
    const int v_n_max = pruned ? ((7 + dh_v + 15) & ~15) : dh_v;
    const int nqa = (dh_qk + 63) / 64, nva = (v_n_max + 63) / 64;
    const int smem_bytes = (2 * nqa + nva + 2) * ATOM_BYTES + EXTRA_BYTES + 1024;
    int dev = 0;
    cudaGetDevice(&dev);
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
    a.col_id = col_id;
    a.head_ptr = head_ptr;
    a.nva_max = nva;
    a.tmem_cols = (128 + v_n_max > 256) ? 512 : TMEM_COLS_ATT;
    a.tma_out = tma_out ? 1 : 0;
    a.n_units = n_units;
    for (int u = 0; u < ATT_MAX_UNITS; ++u) {
        a.unit_head[u] = static_cast<unsigned char>(u < n_units ? unit_head[u] : 0);
        a.unit_first[u] = static_cast<unsigned short>(u < n_units ? unit_first[u] : 0);
    }
    const dim3 grid = n_units > 0 ? dim3(blocks_per_unit, n_units, batch)
                                  : dim3((seq + BQ - 1) / BQ, nhead, batch);
    auto go = [&](auto kern, int slot) -> int {
        static std::atomic<bool> attr_set[4][64] = {};
        if (dev >= 0 && dev < 64 && !attr_set[slot][dev]) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (2 * 2 + 3 + 2) * ATOM_BYTES + EXTRA_BYTES + 1024) !=
                cudaSuccess)
                return ET_ERR_CUDA;
            attr_set[slot][dev] = true;
        }
        return launch_kernel(kern, grid, dim3(ATT_THREADS), smem_bytes, stream, tmQ, tmK, tmV, tmZ,
                             a) == cudaSuccess
                   ? ET_OK
                   : ET_ERR_CUDA;
    };
    switch (mask_kind) {
        case ET_MASK_CAUSAL: return go(attention_kernel<ET_MASK_CAUSAL>, 1);
        case ET_MASK_PADDING: return go(attention_kernel<ET_MASK_PADDING>, 2);
        case ET_MASK_ADDITIVE: return go(attention_kernel<ET_MASK_ADDITIVE>, 3);
        default: return go(attention_kernel<ET_MASK_NONE>, 0);
    }
}
}  // namespace

int launch_attention(const __half* Q, const __half* K, const __half* V, __half* Z, int batch,
                     int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv, int ldz,
                     int mask_kind, const __half* mask, const int* valid_len, float scale,
                     cudaStream_t stream) {
    return launch_attention_impl(Q, K, V, Z, batch, seq, nhead, dh_qk, dh_v, ldq, ldk, ldv, ldz,
                                 mask_kind, mask, valid_len, scale, nullptr, nullptr, 0, stream);
}

int launch_attention_units(const __half* Q, const __half* K, const __half* V, __half* Z, int batch,
                           int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv,
                           int ldz, int mask_kind, const __half* mask, const int* valid_len,
                           float scale, const int* unit_head, const int* unit_first, int n_units,
                           int blocks_per_unit, cudaStream_t stream) {
    if (n_units <= 0) return ET_ERR_INVALID_ARG;
    return launch_attention_impl(Q, K, V, Z, batch, seq, nhead, dh_qk, dh_v, ldq, ldk, ldv, ldz,
                                 mask_kind, mask, valid_len, scale, nullptr, nullptr, 0, stream,
                                 unit_head, unit_first, n_units, blocks_per_unit);
}

}  // namespace et

extern "C" {

int et_attention_units_fwd(const et_half* Q, const et_half* K, const et_half* V, et_half* Z, int batch,
                           int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv,
                           int ldz, int mask_kind, const et_half* mask, const int32_t* valid_len,
                           float scale, const int32_t* unit_head, const int32_t* unit_first_block,
                           int n_units, int blocks_per_unit, et_stream stream) {
    return et::launch_attention_units(
        reinterpret_cast<const __half*>(Q), reinterpret_cast<const __half*>(K),
        reinterpret_cast<const __half*>(V), reinterpret_cast<__half*>(Z), batch, seq, nhead, dh_qk,
        dh_v, ldq, ldk, ldv, ldz, mask_kind, reinterpret_cast<const __half*>(mask), valid_len,
        scale, unit_head, unit_first_block, n_units, blocks_per_unit,
        static_cast<cudaStream_t>(stream));
}

int et_attention_fwd(const et_half* Q, const et_half* K, const et_half* V, et_half* Z, int batch,
                     int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv, int ldz,
                     int mask_kind, const et_half* mask, const int32_t* valid_len, float scale,
                     et_stream stream) {
    return et::launch_attention(
        reinterpret_cast<const __half*>(Q), reinterpret_cast<const __half*>(K),
        reinterpret_cast<const __half*>(V), reinterpret_cast<__half*>(Z), batch, seq, nhead, dh_qk,
        dh_v, ldq, ldk, ldv, ldz, mask_kind, reinterpret_cast<const __half*>(mask), valid_len,
        scale, static_cast<cudaStream_t>(stream));
}

int et_attention_pruned_v_fwd(const et_half* Q, const et_half* K, const et_half* Vc,
                              const int32_t* col_id, const int32_t* head_ptr, int nnz_col,
                              et_half* Z, int batch, int seq, int nhead, int dh_qk, int dh_v,
                              int ldq, int ldk, int ldz, int mask_kind, const et_half* mask,
                              const int32_t* valid_len, float scale, et_stream stream) {
    if (!col_id || !head_ptr || nnz_col <= 0) return ET_ERR_INVALID_ARG;
    if (nnz_col % 8) return ET_ERR_SHAPE;  // row pitch of the compressed V must be 16-byte aligned
    return et::launch_attention_impl(
        reinterpret_cast<const __half*>(Q), reinterpret_cast<const __half*>(K),
        reinterpret_cast<const __half*>(Vc), reinterpret_cast<__half*>(Z), batch, seq, nhead, dh_qk,
        dh_v, ldq, ldk, nnz_col, ldz, mask_kind, reinterpret_cast<const __half*>(mask), valid_len,
        scale, col_id, head_ptr, nnz_col, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
