// Internal launch functions shared between the C-ABI translation units.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace et {

// Y[M, N] = act(X[M, K] . W[N, K]^T + bias).  col_map == nullptr: plain store to Y[m, n]
// (N % 8 == 0, ldy % 8 == 0).  col_map != nullptr: the bias is taken at col_map[n] and the
// value stored at column col_map[n] (scatter != 0) or n (scatter == 0).
int launch_gemm_f16(const __half* X, int ldx, const __half* W, int ldw, const __half* bias,
                    __half* Y, int ldy, const int* col_map, int scatter, int M, int N, int K,
                    int act, cudaStream_t stream);

// The same product on CTA pairs (256 x bn tiles, bn = 128 or 256); see gemm_pair.cu.
int launch_gemm_pair_f16(const __half* X, int ldx, const __half* W, int ldw, const __half* bias,
                         __half* Y, int ldy, int M, int N, int K, int act, int bn,
                         cudaStream_t stream);

// The same product on 256 x bn single-CTA tiles (two accumulators share one weight tile);
// see gemm_tall.cu.
int launch_gemm_tall_f16(const __half* X, int ldx, const __half* W, int ldw, const __half* bias,
                         __half* Y, int ldy, int M, int N, int K, int act, int bn,
                         cudaStream_t stream);

// Fused Q/K/V projection + attention for seq <= 128 and 64-wide heads; see qkv_attention.cu.
bool qkv_attention_applies(int seq, int nhead, int kdim, int vdim);
int launch_qkv_attention(const __half* X, const __half* Wqkv, const __half* bqkv, __half* Z,
                         int batch, int seq, int hidden, int nhead, int kdim, int vdim, int ldz,
                         int mask_kind, const __half* mask, const int* valid_len, float scale,
                         cudaStream_t stream);

// fp32 split-K partial sums on 256 x 256 pair tiles; see gemm_pair.cu.
int launch_gemm_pair_splitk(const __half* X, int ldx, const __half* W, int ldw, float* P, int M,
                            int N, int K, int splits, cudaStream_t stream);

// Grouped GEMM over weights stored [groups][K, N] (N contiguous); see gemm_dense.cu.
int launch_gemm_f16_grouped_kn(const __half* X, int ldx, const __half* W, const __half* bias,
                               __half* Y, int M, int N, int K, int groups, int grp_rows,
                               cudaStream_t stream);

// Split-K fp32 partial sums P[splits][M, N] (no bias) and the LayerNorm that consumes them:
// out = LN(sum_p P[p] + bias + skip) * gamma + beta.  size <= 2048.
int launch_gemm_f16_splitk(const __half* X, int ldx, const __half* W, int ldw, float* P, int M,
                           int N, int K, int splits, cudaStream_t stream);
int launch_skip_layernorm_partials(const float* partials, int nsplit, size_t split_stride,
                                   const __half* bias, const __half* skip, const __half* gamma,
                                   const __half* beta, __half* out, int rows, int size,
                                   cudaStream_t stream);

// Tile-CSR Linear (see linear_tile.cu).
int launch_linear_tile(const int* row_ptr, const int* row_off, const __half* tiles, int nnz_tiles,
                       const __half* bias, const __half* X, __half* Y, int T, int in, int out,
                       int act, cudaStream_t stream);

int launch_linear_tile_packed(const int* row_ptr, const uint32_t* pk_mask, const int* pk_off,
                              const __half* pk_tiles, int nnz_tiles, const __half* bias,
                              const __half* X, __half* Y, int T, int in, int out, int act,
                              cudaStream_t stream);

// The packed tile-CSR Linear as a persistent kernel (one CTA per SM walks work items of 128
// tokens x 256 output features, two items' accumulators in tensor memory); see
// linear_tile_persist.cu.  nnz_tiles > 0.
// Which kernel serves packed weights: 1 = persistent, anything else = one item per CTA (the
// default).
int tile_packed_mode();
int launch_linear_tile_persist(const int* row_ptr, const uint32_t* pk_mask, const int* pk_off,
                               const __half* pk_tiles, int nnz_tiles, const __half* bias,
                               const __half* X, __half* Y, int T, int in, int out, int act,
                               cudaStream_t stream);

// The tile-CSR Linear straight from the format's arrays on the warp-level tensor path (every warp
// walks its block rows' tiles); see linear_tile_rows.cu.  Needs in % 64 == 0; nnz_tiles > 0.
bool linear_tile_rows_supported(int in, int out);
int launch_linear_tile_rows(const int* row_ptr, const int* row_off, const __half* tiles, int nnz_tiles,
                            const __half* bias, const __half* X, __half* Y, int T, int in, int out,
                            int act, cudaStream_t stream);

// Fused attention (see attention.cu).  Vc_col_id / head_ptr are null for an uncompressed V.
int launch_attention(const __half* Q, const __half* K, const __half* V, __half* Z, int batch,
                     int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv, int ldz,
                     int mask_kind, const __half* mask, const int* valid_len, float scale,
                     cudaStream_t stream);

// The same kernel over a list of work units (head, first 128-query block), each covering
// blocks_per_unit query blocks; query rows outside the units are not written.  unit_head and
// unit_first are HOST arrays of n_units <= 16 entries.
int launch_attention_units(const __half* Q, const __half* K, const __half* V, __half* Z, int batch,
                           int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv,
                           int ldz, int mask_kind, const __half* mask, const int* valid_len,
                           float scale, const int* unit_head, const int* unit_first, int n_units,
                           int blocks_per_unit, cudaStream_t stream);

// Attention over every head, then out = Z W_O^T + bias with tile-CSR W_O (attention_fuse_o.cu);
// Z [batch * seq, nhead * dh_v] receives the heads' outputs.  single_launch: one kernel with
// work tickets and per-block completion counters instead of the two stand-alone kernels.
int launch_attention_fuse_o(const __half* Q, const __half* K, const __half* V, const __half* mask,
                            __half* Z, const int* o_row_ptr, const int* o_row_off,
                            const __half* o_tiles, int o_nnz, const __half* o_bias, __half* out,
                            int batch, int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk,
                            int ldv, int emdim, int mask_kind, const int* valid_len, float scale,
                            bool single_launch, cudaStream_t stream);

// out = LN(X W^T + bias + resid) * gamma + beta in one kernel (gemm_ln.cu); N = 256 .. 1024 in
// steps of 128.
bool gemm_ln_applies(int M, int N, int K);
int gemm_ln_resident_clusters(int N);  // clusters of N / 128 CTAs the device holds at once
int launch_gemm_ln(const __half* X, int ldx, const __half* W, int ldw, const __half* bias,
                   const __half* resid, int ldr, const __half* gamma, const __half* beta,
                   __half* out, int ldo, int M, int N, int K, cudaStream_t stream);

// out = LN(src + skip) * gamma + beta (skip may be null).
int launch_skip_layernorm(const __half* src, const __half* skip, const __half* gamma,
                          const __half* beta, __half* out, int rows, int size,
                          cudaStream_t stream);

}  // namespace et
