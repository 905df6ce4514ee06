/*
 * et_b200 — C ABI of the B200 (sm_100a) encoder-layer hot path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA
 * stream, returns an int status (0 = ok, negative = error, see et_status_string), never
 * throws, never synchronises the device and never allocates: scratch memory is passed
 * in by the caller.  One host thread per GPU may call into the library concurrently; the
 * per-device state the library caches on a first call (error word address, kernel attributes,
 * occupancy answers) is published with atomic stores, so first calls may overlap too.
 *
 * Layout conventions (all from the reference, cctry/SCpaper-2021):
 *   - activations: row-major fp16 [tokens, features], tokens = batch * seq, heads are
 *     contiguous feature ranges (Attention/OTFkernel_full.h:34,49,116);
 *   - dense weight: W[out, in] row-major, y = x W^T + b (Linear/Linear.h:11-15);
 *   - index arrays: int32.
 *
 * The reference has no C ABI (it is a C++17 template library); each function below
 * names the reference member function or kernel launch it stands in for.
 */
#ifndef ET_B200_H
#define ET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* fp16 values cross the ABI as raw 16-bit words (IEEE binary16). */
typedef uint16_t et_half;
/* cudaStream_t crosses the ABI as an opaque pointer. */
typedef void* et_stream;

/* ---- status codes --------------------------------------------------------------- */
#define ET_OK 0
#define ET_ERR_INVALID_ARG (-1)   /* null pointer, non-positive size, bad enum        */
#define ET_ERR_ALIGNMENT (-2)     /* pointer or leading dimension not 16-byte aligned  */
#define ET_ERR_SHAPE (-3)         /* a size the kernels do not support (see each call) */
#define ET_ERR_INDEX (-4)         /* corrupt index array found by a validator          */
#define ET_ERR_CUDA (-5)          /* a CUDA runtime / driver call failed               */
#define ET_ERR_WORKSPACE (-6)     /* scratch buffer missing or too small               */
#define ET_ERR_DEVICE_TIMEOUT (-7)/* a kernel gave up on a bounded wait                */
#define ET_ERR_NO_DEVICE (-8)     /* no sm_100 device is current                       */

const char* et_status_string(int status);

/* Library version, and the compute capability the kernels were built for (100). */
int et_version(void);
int et_built_for_sm(void);

/* Reads (and clears) the device-side error word of the current device.  Kernels never
 * trap: a bounded wait that runs out records a code there and the kernel returns.
 * This call synchronises the device.  *code = 0 when no kernel reported a problem.
 * Replaces the reference's cudaChk/assert/exit(1) convention (lib/utils.cu:28-35). */
int et_device_error(int* code);

/* Kernels launched by this library so far in this process (host-side count; a CUDA graph
 * replays what was counted while it was captured).  Diagnostic only: lets a caller state how
 * many kernels one call issued.  The reference has no counterpart (it counts nothing). */
long long et_launch_count(void);

/* ---- activation / epilogue selectors ------------------------------------------- */
#define ET_ACT_NONE 0
#define ET_ACT_RELU 1 /* Encoder/Encoder.h:29-32                                       */
#define ET_ACT_GELU 2 /* tanh form, constants of Encoder/Encoder.cu:25-39              */

/* ---- attention mask selectors --------------------------------------------------- */
#define ET_MASK_NONE 0     /* all keys visible                                        */
#define ET_MASK_CAUSAL 1   /* key j <= query i: the mask Attention.h:97-104 builds     */
#define ET_MASK_PADDING 2  /* keys >= valid_len[b] dropped                             */
#define ET_MASK_ADDITIVE 3 /* fp16 [seq, seq] added to the scaled scores (0 / -inf)    */

/* =================================================================================
 * Linear layers:  Y[T, out] = act( X[T, in] . W^T + bias )
 * bias may be NULL (treated as zero).  X, Y and weight pointers must be 16-byte
 * aligned; in % 16 == 0 and out % 16 == 0 (the reference's own precondition).
 * ================================================================================= */

/* Dense weights W[out, in].
 * Stands in for Linear<base_mat>::forward (Linear/Linear.h:53-64: cuBLAS GEMM followed
 * by a separate bias pass) and, with act != NONE, for the act<> pass of
 * Encoder/Encoder.h:27-37. */
int et_linear_dense_fwd(const et_half* X, const et_half* W, const et_half* bias, et_half* Y,
                        int T, int in, int out, int act, et_stream stream);

/* Dense Linear fused with the skip-LayerNorm that follows it:
 *   out = LayerNorm(X . W^T + bias + resid) * gamma + beta        (eps 1e-5, fp32 statistics)
 * in one kernel; the pre-normalisation activations never reach memory.  out: 256 .. 1024 in
 * steps of 128 (ET_ERR_SHAPE otherwise: use et_linear_dense_fwd + et_skip_layernorm_fwd);
 * bias and resid may be NULL; `result` must not alias X or resid.  Replaces the pair
 * Linear<base_mat>::forward + SkipLayerNorm::forward of the encoder layer (Encoder/Encoder.h:
 * the O projection and FFN2, each followed by SkipLayerNorm/SkipLayerNorm.cu:73-82). */
int et_linear_skip_layernorm_fwd(const et_half* X, const et_half* W, const et_half* bias,
                                 const et_half* resid, const et_half* gamma, const et_half* beta,
                                 et_half* result, int T, int in, int out, et_stream stream);
/* Plan-time query for the call above: 1 when it is expected to beat et_linear_dense_fwd followed
 * by et_skip_layernorm_fwd on the current device, i.e. when the width is supported and every
 * thread-block cluster of the launch (one per 128 rows) is resident at once; else 0. */
int et_linear_skip_layernorm_pays(int T, int in, int out);

/* 16x16 tile-CSR weights: row_ptr[out/16 + 1], row_off[nnz] (input block column,
 * ascending inside a block row), tiles[nnz][16][16] row-major [out_local][in_local].
 * Only stored tiles are loaded.  Stands in for Linear<tile_mat>::forward
 * (Linear/SPMM_tile.cu:312-324 launching the kernel at :250-310). */
int et_linear_tile_fwd(const int32_t* row_ptr, const int32_t* row_off, const et_half* tiles,
                       int nnz_tiles, const et_half* bias, const et_half* X, et_half* Y, int T,
                       int in, int out, int act, et_stream stream);

/* The same tile-pruned Linear on RE-PACKED weights.  Weights are static, so the operator
 * may reorder its tiles once into the order the kernels consume them - (pair of panels of 8
 * block rows, chunk of 4 block columns, panel of the pair, row, column) - with one presence
 * mask and one tile offset per (panel, chunk); the tiles a panel pair needs for a chunk then
 * arrive with a single bulk copy.  The re-packing is a pure permutation of the tile-CSR arrays:
 *   et_tile_pack_dims   sizes of the mask / offset arrays (npanel * nchunk entries each);
 *   et_tile_pack_plan   HOST index arrays in, masks / offsets / permutation out (host);
 *   et_tile_pack_tiles  packed_tiles[i] = tiles[perm[i]] on the GPU (perm: device array);
 *   et_linear_tile_packed_fwd  the forward pass; row_ptr as in et_linear_tile_fwd.  One CTA per
 *     work item of 128 tokens x one or two panels of 128 output features (two once such items
 *     cover the SMs 1.25 times: the panels then share every activation slab).
 * Stands in for the same reference call as et_linear_tile_fwd (Linear/SPMM_tile.cu:312-324);
 * the reference keeps its tiles in file order. */
int et_tile_pack_dims(int in, int out, int* npanel, int* nchunk);
int et_tile_pack_plan(const int32_t* row_ptr, const int32_t* row_off, int nnz_tiles, int in, int out,
                      uint32_t* pk_mask, int32_t* pk_off, int32_t* perm);
int et_tile_pack_tiles(const et_half* tiles, const int32_t* perm, int nnz_tiles,
                       et_half* packed_tiles, et_stream stream);
int et_linear_tile_packed_fwd(const int32_t* row_ptr, const uint32_t* pk_mask, const int32_t* pk_off,
                              const et_half* pk_tiles, int nnz_tiles, const et_half* bias,
                              const et_half* X, et_half* Y, int T, int in, int out, int act,
                              et_stream stream);

/* Plan-time choice for a tile-pruned weight.  On B200 one 128 x 16 x 16 tensor-core product
 * occupies the tensor pipe about as long as a product eight times wider, so the tile kernel
 * only pays for very sparse weights.  et_tile_prefer_dense returns 1 when the dense GEMM on
 * the expanded weight is expected to be faster (more than 10 % of the tiles stored for
 * out >= 3072, 15 % for out >= 2048, 2 % otherwise: measured crossovers at 2048 tokens);
 * et_tile_densify expands tile-CSR (device arrays) into dense[out, in], pruned tiles zero, for
 * et_linear_dense_fwd.  The result equals et_linear_tile_fwd's up to fp32 summation order.
 * Like every weight, `dense` must be complete (stream synchronised) before the first Linear
 * call that uses it: the Linear kernels fetch weights before they wait for their predecessors
 * on the stream.  The same holds for the output of et_tile_pack_tiles.
 * Same reference call as et_linear_tile_fwd (Linear/SPMM_tile.cu:312-324). */
int et_tile_prefer_dense(int in, int out, int nnz_tiles);
int et_tile_densify(const int32_t* row_ptr, const int32_t* row_off, const et_half* tiles,
                    int nnz_tiles, int in, int out, et_half* dense, et_stream stream);

/* Row-pruned weights: rows[nn_row, in] are the weights of output features
 * row_id[0..nn_row) (ascending); every other output column receives the bias alone.
 * Stands in for Linear<row_mat>::forward(half*, half*) (Linear/SPMM_row.cu:62-75:
 * cuBLAS on the kept rows, scatter kernel :14-30, bias pass).  Y needs no pre-zeroing. */
int et_linear_row_fwd(const int32_t* row_id, const et_half* rows, int nn_row,
                      const et_half* bias, const et_half* X, et_half* Y, int T, int in, int out,
                      int act, et_stream stream);

/* Row-pruned weights with COMPRESSED output Yc[T, nn_row] (column k = feature row_id[k]),
 * bias of the kept features added.  Stands in for Linear<row_mat>::forward(col_mat*, ...)
 * (Linear/SPMM_row.cu:78-95), which feeds the pruned-V attention. */
int et_linear_row_compressed_fwd(const int32_t* row_id, const et_half* rows, int nn_row,
                                 const et_half* bias, const et_half* X, et_half* Yc, int T,
                                 int in, et_stream stream);

/* Column-pruned weights: cols[out, nn_col] multiply the input features col_id[0..nn_col).
 * scratch must hold T * nn_col fp16 values (the gathered activations).
 * Stands in for Linear<col_mat>::forward (Linear/SPMM_col.cu:57-69: gather kernel :8-23
 * into the operator's workspace, cuBLAS, bias pass). */
int et_linear_col_fwd(const int32_t* col_id, const et_half* cols, int nn_col,
                      const et_half* bias, const et_half* X, et_half* Y, int T, int in, int out,
                      int act, et_half* scratch, size_t scratch_bytes, et_stream stream);

/* The same column-pruned Linear for callers that have no way to hand over scratch memory:
 * code that runs where device allocation is off limits, for example a plugin that is only
 * given its input and output tensors by a host framework that owns every allocation, or a
 * latency-critical serving loop that must not touch the allocator once it is running.  The
 * gathered activations go to a fixed 8 MiB array inside the library image (held by every
 * GPU that loads the library until the process exits), so T * nn_col may not exceed
 * 4 194 304 values; larger problems return ET_ERR_WORKSPACE and must use
 * et_linear_col_fwd.  No cudaMalloc / cudaFree or allocating routine is called.
 * The first call on a device looks up the array's device address; make that call before
 * starting any stream capture.  All calls share the one array: it keeps whatever the last
 * call gathered (nothing in it has to start at zero, each call overwrites the part it
 * reads), and two calls that overlap in time on the GPU race on it - issue them on one
 * stream or order them yourself.
 * This entry point has no counterpart in the reference, whose Linear<col_mat> always owns
 * a cudaMalloc'ed workspace. */
int et_linear_col_noalloc_fwd(const int32_t* col_id, const et_half* cols, int nn_col,
                              const et_half* bias, const et_half* X, et_half* Y, int T, int in,
                              int out, int act, et_stream stream);

/* 1x16-vector weights: tile_idx[(out/16) * (in/16 + 1)], row_idx[nvec], data[nvec][16]
 * (mat_type/mat1x16/mat1x16.h:9-15).  Stands in for Linear<mat1x16>::forward
 * (Linear/SPMM1x16.cu:89-115, whose body the reference leaves empty; the intended
 * product of :56-83 is computed). */
int et_linear_1x16_fwd(const int32_t* tile_idx, const int32_t* row_idx, const et_half* data,
                       int nvec, const et_half* bias, const et_half* X, et_half* Y, int T, int in,
                       int out, int act, et_stream stream);

/* CSR weights W[out, in].  Stands in for Linear<csr_mat>::forward (Linear/cusp.cu:23-50:
 * cuSPARSE SpMM + bias pass). */
int et_linear_csr_fwd(const int32_t* indptr, const int32_t* indices, const et_half* data,
                      int nnz, const et_half* bias, const et_half* X, et_half* Y, int T, int in,
                      int out, int act, et_stream stream);

/* 1x16-vector weights on the tensor cores.  A tensor-core product cannot skip single vectors
 * inside a 16 x 16 tile, and at 90 % vector sparsity four tiles in five still hold a vector,
 * so the fast path for this format is the dense GEMM on the expanded weight:
 * et_1x16_prefer_dense returns 1 when that is expected to beat et_linear_1x16_fwd (unless
 * fewer than 1 % of the vectors are stored), et_1x16_densify expands the device arrays into
 * dense[out, in] (pruned vectors zero) for et_linear_dense_fwd.  `dense` must be complete
 * (stream synchronised) before the first Linear call that uses it.  Same reference call as
 * et_linear_1x16_fwd (Linear/SPMM1x16.cu:35-124). */
int et_1x16_prefer_dense(int in, int out, int nvec);
int et_1x16_densify(const int32_t* tile_idx, const int32_t* row_idx, const et_half* data, int nvec,
                    int in, int out, et_half* dense, et_stream stream);

/* Host-side validators for index arrays that live in HOST memory (call before upload).
 * Return ET_OK or ET_ERR_INDEX; they never touch the GPU. */
int et_validate_tile_mat(const int32_t* row_ptr, const int32_t* row_off, int nnz_tiles, int in,
                         int out);
int et_validate_id_list(const int32_t* ids, int n, int limit, int require_sorted);
int et_validate_1x16(const int32_t* tile_idx, const int32_t* row_idx, int nvec, int in, int out);
int et_validate_csr(const int32_t* indptr, const int32_t* indices, int nnz, int in, int out);

/* =================================================================================
 * Normalisation and element-wise passes
 * ================================================================================= */

/* out = LayerNorm(src + skip) * gamma + beta, eps 1e-5, statistics in fp32.
 * Stands in for SkipLayerNorm::forward (SkipLayerNorm/SkipLayerNorm.cu:73-82). */
int et_skip_layernorm_fwd(const et_half* src, const et_half* skip, const et_half* gamma,
                          const et_half* beta, et_half* out, int rows, int size, et_stream stream);

/* out = LayerNorm(src) * gamma + beta.  Stands in for LayerNorm::forward
 * (LayerNorm/LayerNorm.cu:51-57), without its per-call device synchronisation. */
int et_layernorm_fwd(const et_half* src, const et_half* gamma, const et_half* beta, et_half* out,
                     int rows, int size, et_stream stream);

/* In-place capable activation pass over n values.  Stands in for act<RELU_OP|GELU_OP>
 * (Encoder/Encoder.h:27-37) and GELU::computeGelu (Encoder/Encoder.cu:41-68). */
int et_act_fwd(const et_half* in, et_half* out, size_t n, int act, et_stream stream);

/* data[r, c] += bias[c]; the reference's bias map (Linear/Linear.h:57-63). */
int et_bias_add_fwd(et_half* data, const et_half* bias, int rows, int cols, et_stream stream);

/* =================================================================================
 * Attention
 * ================================================================================= */

/* Z[b*seq+i, h*dh_v ..] = softmax_j( scale * Q_i.K_j + mask_ij ) V_j  for every
 * sequence b and head h, scores never written to memory.
 * Q/K/V/Z are [batch*seq, ld*] with head h at feature offset h*dh; the three inputs
 * may alias one fused [Q | K | V] projection buffer (ldq = ldk = ldv = 2*kdim + vdim).
 * dh_qk, dh_v: multiples of 16, at most 128.  ld*: multiples of 8.
 * mask: fp16 [seq, seq] for ET_MASK_ADDITIVE, else NULL; valid_len: int32[batch] for
 * ET_MASK_PADDING, else NULL.  A query whose keys are all dropped yields zeros.
 * Stands in for Multihead_atttion<OTF_attn_full> (Attention/Attention.cu:80-95 launching
 * Attention/OTFkernel_full.h:17-125) and the fused-QKV launch of
 * Attention/Attention.h:246-265 (Attention/Attention_single.cu:10-108). */
int et_attention_fwd(const et_half* Q, const et_half* K, const et_half* V, et_half* Z, int batch,
                     int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv, int ldz,
                     int mask_kind, const et_half* mask, const int32_t* valid_len, float scale,
                     et_stream stream);

/* Fused Q/K/V projection + self-attention for short sequences: Z[b, :, head h] =
 * softmax(Q_h K_h^T * scale + mask) V_h with [Q | K | V] = X Wqkv^T + bqkv computed inside the
 * same kernel (one CTA per sequence and head; the projected activations never reach memory).
 * Wqkv: [2 * kdim + vdim, hidden] with output features ordered Q | K | V, bqkv may be null, Z:
 * [batch * seq, vdim].  Requires seq <= 128 and kdim = vdim = 64 * nhead (ET_ERR_SHAPE
 * otherwise: use et_linear_dense_fwd + et_attention_fwd).  Masks as et_attention_fwd.
 * Replaces the fused-QKV Linear + attention launch of Attention<cfg, single>::forward
 * (Attention/Attention.h:204-266). */
int et_qkv_attention_fwd(const et_half* X, const et_half* Wqkv, const et_half* bqkv, et_half* Z,
                         int batch, int seq, int hidden, int nhead, int kdim, int vdim,
                         int mask_kind, const et_half* mask, const int32_t* valid_len, float scale,
                         et_stream stream);

/* Attention whose V is column-compressed: Vc[T, nnz_col] holds the value features
 * col_id[0..nnz_col) (ascending); head_ptr[h]..head_ptr[h+1] delimits head h's entries
 * (mat_type/col_mat/col_mat.cu:34-58).  Z[T, nhead*dh_v] is written in full: pruned
 * features are zero.  Stands in for Multihead_atttion<Prune_attn>
 * (Attention/Attention.cu:55-78, kernel Attention/kernels.cu:363-460). */
int et_attention_pruned_v_fwd(const et_half* Q, const et_half* K, const et_half* Vc,
                              const int32_t* col_id, const int32_t* head_ptr, int nnz_col,
                              et_half* Z, int batch, int seq, int nhead, int dh_qk, int dh_v,
                              int ldq, int ldk, int ldz, int mask_kind, const et_half* mask,
                              const int32_t* valid_len, float scale, et_stream stream);

/* Attention followed by a tile-CSR output projection in one call:
 * out = tileLinear_O( attention(Q, K, V) ) + bias_o.  Z[T, nhead*dh_v] receives the heads'
 * outputs (the reference's Z argument).  Stands in for Multihead_atttion_fuseO
 * (Attention/kernel_fuseO.cu:254-290).  Runs the attention kernel and the tile Linear as two
 * launches chained by programmatic dependent launch: on B200 that is the faster of the two
 * forms (see et_attention_fuse_o_single_launch_fwd). */
int et_attention_fuse_o_fwd(const et_half* Q, const et_half* K, const et_half* V,
                            const et_half* mask, et_half* Z, const int32_t* o_row_ptr,
                            const int32_t* o_row_off, const et_half* o_tiles, int o_nnz,
                            const et_half* o_bias, et_half* out, int batch, int seq, int nhead,
                            int dh_qk, int dh_v, int ldq, int ldk, int ldv, int emdim,
                            int mask_kind, const int32_t* valid_len, float scale,
                            et_stream stream);

/* The same operator as ONE kernel launch, the form of the reference's
 * __kernel_multi_head_full_fuseO (Attention/kernel_fuseO.cu:138-243) with its grid-wide barrier
 * replaced by one completion counter per (sequence, 128-query block).  CTAs take work by
 * ticket: first the (sequence, query block, head) attention units, then the (128-token block,
 * 128 output features) projection items, each of which starts as soon as the query blocks it
 * reads are complete.  An item only ever waits for work with a lower ticket, which a running
 * CTA already holds, so the launch needs no co-residency guarantee.  Same arguments and
 * bit-identical results.  The counters live in the library image: at most 16 such calls may be
 * in flight on one GPU at once, and batch * ceil(seq / 128) must stay below 4094 (beyond that,
 * or when W_O stores no tile, the call runs the two-launch form).  A counter wait is bounded
 * (about a second); when it runs out et_device_error reports 304.  Measured on B200 it is 1 %
 * (one 4096-token sequence) to 30 % (16 x 128 tokens) slower than the two-launch form: the
 * ticket and counter traffic is not hidden the way a dependent launch hides a launch. */
int et_attention_fuse_o_single_launch_fwd(const et_half* Q, const et_half* K, const et_half* V,
                                          const et_half* mask, et_half* Z, const int32_t* o_row_ptr,
                                          const int32_t* o_row_off, const et_half* o_tiles, int o_nnz,
                                          const et_half* o_bias, et_half* out, int batch, int seq,
                                          int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv,
                                          int emdim, int mask_kind, const int32_t* valid_len,
                                          float scale, et_stream stream);

/* Pre-multiplied V.O attention: out[t, :] = sum_h P_h[t, :] . VO_h + bias_o with
 * VO given as [batch][nhead][seq][emdim] (Fused_attention/Linear_VO.h:38-58).
 * Heads are reduced in a fixed order (the reference uses half2 atomics).
 * Stands in for Fused_Multihead_attention<OTF_fused_attn>
 * (Fused_attention/Fused_attention.cu:231-253, kernel :10-116). */
int et_fused_vo_attention_fwd(const et_half* Q, const et_half* K, const et_half* VO,
                              const et_half* bias_o, et_half* out, int batch, int seq, int nhead,
                              int dh_qk, int emdim, int ldq, int ldk, int mask_kind,
                              const et_half* mask, const int32_t* valid_len, float scale,
                              et_stream stream);

/* VO[b][h] = X_b . W_VO[h] + bias[h] for W_VO [nhead][emdim(in)][emdim(out)].
 * Stands in for Linear_VO::forward (Fused_attention/Linear_VO.h:38-58 + Linear_VO.cu:32-45). */
int et_linear_vo_fwd(const et_half* X, const et_half* Wvo_t, const et_half* bias, et_half* VO,
                     int batch, int seq, int nhead, int emdim, et_stream stream);

/* Column-pruned V.O: the pre-multiplied weight keeps only the output features
 * col_id[0 .. nnz_col) (ascending, nnz_col % 16 == 0).
 *   et_linear_vo_pruned_fwd: VOc[b][h] = X_b . Wvo_c[h] + bias[h] with Wvo_c
 *     [nhead][emdim][nnz_col], bias [nhead][nnz_col] or null, VOc [batch][nhead][seq][nnz_col]
 *     (Linear_VO_prune::forward, Fused_attention/Linear_VO.h:60-96).
 *   et_fused_vo_attention_pruned_fwd: the attention at width nnz_col into scratch
 *     [batch * seq, nnz_col], then out[t, col_id[k]] = scratch[t, k] + bias_o[col_id[k]] and
 *     out[t, c] = bias_o[c] for pruned c (bias_o [emdim] or null)
 *     (Fused_prune_Multihead_attention, Fused_attention/Fused_attention.cu:273-309). */
int et_linear_vo_pruned_fwd(const et_half* X, const et_half* Wvo_c, const et_half* bias,
                            et_half* VOc, int batch, int seq, int nhead, int emdim, int nnz_col,
                            et_stream stream);
int et_fused_vo_attention_pruned_fwd(const et_half* Q, const et_half* K, const et_half* VOc,
                                     const int32_t* col_id, int nnz_col, const et_half* bias_o,
                                     et_half* scratch, et_half* out, int batch, int seq, int nhead,
                                     int dh_qk, int emdim, int ldq, int ldk, int mask_kind,
                                     const et_half* mask, const int32_t* valid_len, float scale,
                                     et_stream stream);

/* =================================================================================
 * Whole encoder layer (post-LN), the call Encoder<config>::forward makes
 * (Encoder/Encoder.h:81-96):
 *   a = O(attention(QKV(x)));  y = LN1(a + x);  out = LN2(W2 act(W1 y + b1) + b2 + y)
 * With dense weights the layer runs as four kernels where the shapes allow it: Q/K/V
 * projection + attention (et_qkv_attention_fwd), O projection + residual + LN1
 * (et_linear_skip_layernorm_fwd), FFN1 + activation, FFN2 + residual + LN2; the separate
 * calls otherwise.  A row-pruned FFN1 followed by a column-pruned FFN2 over the SAME id list
 * (ffn1.row_ptr == ffn2.row_ptr, the pruned hidden units of the feed-forward block) runs as
 * two dense products of the kept width: the pruned units are never materialised.
 * ================================================================================= */
#define ET_FMT_DENSE 0
#define ET_FMT_TILE 1        /* tile-CSR as the reference stores it                        */
#define ET_FMT_TILE_PACKED 2 /* re-packed tile-CSR (et_tile_pack_plan / et_tile_pack_tiles) */
#define ET_FMT_1X16 3        /* 1x16 vectors (mat1x16)                                     */
#define ET_FMT_ROW 4         /* kept output rows (row_mat)                                 */
#define ET_FMT_COL 5         /* kept input columns (col_mat)                               */
#define ET_FMT_CSR 6         /* CSR                                                        */

/* One Linear layer of the encoder in any of the reference's weight formats.  The index and
 * count fields are shared between formats:
 *   format            weight                 row_ptr          row_off        nnz_tiles
 *   DENSE             W[out, in]             -                -              -
 *   TILE              tiles[nnz][256]        row_ptr          row_off        stored tiles
 *   TILE_PACKED       packed tiles           row_ptr          -              stored tiles
 *   1X16              data[nvec][16]         tile_idx         row_idx        nvec
 *   ROW               rows[nn_row, in]       row_id[nn_row]   -              nn_row
 *   COL               cols[out, nn_col]      col_id[nn_col]   -              nn_col
 *   CSR               data[nnz]              indptr[out + 1]  indices[nnz]   nnz
 * (argument meaning as in the et_linear_*_fwd call of each format). */
typedef struct {
    int format;             /* one of ET_FMT_*                                          */
    int in, out;
    const et_half* weight;
    const int32_t* row_ptr; /* first index array of the format                          */
    const int32_t* row_off; /* second index array of the format                         */
    int nnz_tiles;          /* stored units of the format                               */
    const et_half* bias;    /* [out] or NULL                                            */
    const uint32_t* pk_mask; /* ET_FMT_TILE_PACKED only                                 */
    const int32_t* pk_off;   /* ET_FMT_TILE_PACKED only                                 */
} et_linear_t;

typedef struct {
    et_linear_t qkv;  /* hidden -> 2*kdim + vdim, output features ordered Q | K | V     */
    et_linear_t o;    /* vdim -> hidden                                                 */
    et_linear_t ffn1; /* hidden -> ff                                                   */
    et_linear_t ffn2; /* ff -> hidden                                                   */
    const et_half *ln1_gamma, *ln1_beta, *ln2_gamma, *ln2_beta; /* [hidden]              */
    int hidden, nhead, kdim, vdim, ff;
    int act;          /* ET_ACT_RELU or ET_ACT_GELU                                     */
} et_encoder_layer_t;

size_t et_encoder_layer_workspace_bytes(const et_encoder_layer_t* layer, int batch, int seq);

int et_encoder_layer_fwd(const et_encoder_layer_t* layer, const et_half* x, et_half* out,
                         int batch, int seq, int mask_kind, const et_half* mask,
                         const int32_t* valid_len, void* workspace, size_t workspace_bytes,
                         et_stream stream);

/* =================================================================================
 * Head-parallel form of the layer, for ONE long sequence spread over several GPUs (the
 * reference is single-GPU; this is the tensor-parallel reading of Attention/Attention.h:
 * 58-142 where each GPU owns some heads' rows of W_Q, W_K, W_V and columns of W_O).  The
 * attention block is cut into work units (head, range of 128-query blocks); a rank runs its
 * units and multiplies by its heads' columns of W_O, which gives a partial [T, hidden] sum;
 * the caller adds the ranks' partial sums with ONE all-reduce and hands the total to the
 * second call, which every rank runs in full (LayerNorm and the feed-forward block are
 * replicated).
 *
 * et_attention_units_fwd: et_attention_fwd over n_units <= 16 work units given as HOST arrays
 *   unit_head[u], unit_first_block[u]; each unit covers blocks_per_unit blocks of 128 queries
 *   against all keys of its head.  Rows of Z outside the units are left untouched.
 * et_encoder_attention_units_fwd: `layer` describes THIS RANK'S slice: qkv = the rows of the
 *   fused projection of its heads ([Q | K | V] order, dense), o = the matching columns of W_O
 *   (in = vdim = local heads * head width), nhead / kdim / vdim local, hidden the model width.
 *   Writes partial[T, hidden] = attention(units) . o^T as fp16 (+ o.bias if given: pass it on
 *   one rank only) or, with partial_is_f32, as fp32 without bias.
 * et_encoder_after_attention_fwd: out = LN2(FFN(y) + y), y = LN1(attn_sum + x) with attn_sum
 *   the all-reduced total: fp16 (bias already inside), or fp32 (layer->o.bias is added here).
 *   `layer` is the full layer; only its o.bias, LayerNorm and ffn fields are read.
 * Both take the workspace of et_encoder_layer_workspace_bytes(layer, batch, seq).
 * ================================================================================= */
int et_attention_units_fwd(const et_half* Q, const et_half* K, const et_half* V, et_half* Z, int batch,
                           int seq, int nhead, int dh_qk, int dh_v, int ldq, int ldk, int ldv,
                           int ldz, int mask_kind, const et_half* mask, const int32_t* valid_len,
                           float scale, const int32_t* unit_head, const int32_t* unit_first_block,
                           int n_units, int blocks_per_unit, et_stream stream);
int et_encoder_attention_units_fwd(const et_encoder_layer_t* layer, const et_half* x, void* partial,
                                   int partial_is_f32, int batch, int seq, int mask_kind,
                                   const et_half* mask, const int32_t* valid_len,
                                   const int32_t* unit_head, const int32_t* unit_first_block,
                                   int n_units, int blocks_per_unit, void* workspace,
                                   size_t workspace_bytes, et_stream stream);
int et_encoder_after_attention_fwd(const et_encoder_layer_t* layer, const void* attn_sum,
                                   int sum_is_f32, const et_half* x, et_half* out, int batch,
                                   int seq, void* workspace, size_t workspace_bytes,
                                   et_stream stream);

/* out = LN2(FFN(y) + y): the feed-forward half of the layer on an LN1 output the caller already
 * holds (the head-parallel exchange below leaves it in the rank's peer buffer). */
int et_encoder_ffn_fwd(const et_encoder_layer_t* layer, const et_half* y, et_half* out, int batch,
                       int seq, void* workspace, size_t workspace_bytes, et_stream stream);

/* Head-parallel exchange over PEER MEMORY (instead of a library all-reduce): the ranks' partial
 * attention outputs are summed, the residual added and LN1 applied by this library's own
 * kernels writing through peer mappings (NVLink), one rank per GPU.  Every rank owns
 * ceil(T / world) token rows.
 *   et_peer_buffer_bytes / _create / _open / _close / _destroy: one exchange buffer per rank
 *     (cudaMalloc + a 64-byte CUDA IPC handle the caller passes to the other ranks by its own
 *     means; _open maps a peer's buffer and enables peer access).  Created zeroed.
 *   peer_buffers[world]: every rank's buffer as seen from THIS rank (own pointer at [rank]).
 *   epoch: a counter the caller raises by one per layer call, the same on every rank.
 *   et_peer_buffer_partial      where this rank's partial [T, hidden] (fp16) must be written
 *                               (pass it as `partial` to et_encoder_attention_units_fwd);
 *   et_hp_signal_partial_fwd    tells every rank that this rank's partial is complete (not
 *                               needed when et_hp_reduce_layernorm_fwd is called with
 *                               publish_ready = 1, which does the same as its first step; the
 *                               separate call exists for callers that run several ranks' kernels
 *                               one after the other on one GPU);
 *   et_hp_reduce_layernorm_fwd  y[rows of this rank] = LN(sum over ranks of their partials' rows
 *                               (pulled through the peer mappings) + bias + x) * gamma + beta,
 *                               written into EVERY rank's y (gather = 1);
 *   et_hp_wait_fwd              returns (on the stream) once every rank's rows of y have landed
 *                               here; et_peer_buffer_y gives the rank's y [T, hidden].
 * A rank calls the three in this order on one stream, then et_encoder_ffn_fwd on y.  Waits are
 * bounded (about a second): when one runs out, et_device_error reports 501 and the layer's
 * output is not valid.  hidden % 8 == 0, hidden <= 2048, world <= 16. */
int et_peer_buffer_bytes(int world, int T, int hidden, size_t* bytes);
int et_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]);
int et_peer_buffer_open(const unsigned char handle[64], void** ptr);
int et_peer_buffer_close(void* ptr);
int et_peer_buffer_destroy(void* ptr);
int et_peer_buffer_y(void* own_buffer, int world, int T, int hidden, et_half** y);
int et_peer_buffer_partial(void* own_buffer, et_half** partial);
int et_hp_signal_partial_fwd(void* const* peer_buffers, int rank, int world, int T, int hidden, int epoch,
                             et_stream stream);
int et_hp_reduce_layernorm_fwd(void* const* peer_buffers, const et_half* x, const et_half* bias,
                               const et_half* gamma, const et_half* beta, int rank, int world, int T,
                               int hidden, int epoch, int publish_ready, int gather, et_stream stream);
/* Token-sharded form: with gather = 0 et_hp_reduce_layernorm_fwd keeps y local (only this rank's
 * rows are valid); the rank runs et_encoder_ffn_fwd on those rows alone, writing into its rows
 * of et_peer_buffer_out(own, ..., slot), and et_hp_allgather_rows_fwd stores them into every
 * rank's out[slot]; after et_hp_wait_fwd out[slot] holds the whole layer output on every rank.
 * The caller alternates slot = 0, 1 from layer to layer. */
int et_peer_buffer_out(void* own_buffer, int world, int T, int hidden, int slot, et_half** out);
int et_hp_allgather_rows_fwd(void* const* peer_buffers, int rank, int world, int T, int hidden, int epoch,
                             int slot, et_stream stream);
int et_hp_wait_fwd(void* own_buffer, int world, int T, int hidden, int epoch, et_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* ET_B200_H */
