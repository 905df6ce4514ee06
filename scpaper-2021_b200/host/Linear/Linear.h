// Linear operator over the reference's weight containers: y = x A^T + b with x a batch of
// row vectors and A[out, in] (Linear/Linear.h:11-15).  Same class template, constructor
// signatures (in_size, out_size, weight, bias, size) and forward(out, in, stream) as the
// reference (Linear/Linear.h:16-167); `size` is the number of token rows of every call.
// Each forward is one call into the C ABI (include/et_b200.h): GEMM, bias and scatter /
// gather are fused there, so no cuBLAS / cuSPARSE handle is held.
#pragma once
#include <memory>
#include <vector>

#include "../lib/CUDA_ptr.hpp"
#include "../mat_type/mat_type.h"

using base_mat = culib::CUDA_ptr<half>;

template <typename _MAT_T> class Linear;

template <> class Linear<base_mat> {
  public:
    const int in_size;
    const int out_size;
    base_mat weight;
    culib::CUDA_ptr<half> bias;
    int size;

    Linear(int _in_size, int _out_size, const base_mat& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), weight(w), bias(b, _out_size), size(_size) {}
    Linear(int _in_size, int _out_size, base_mat&& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), weight(std::move(w)), bias(b, _out_size),
          size(_size) {}
    void forward(half* output, half* input, cudaStream_t stream = 0) const {
        forward_act(output, input, ET_ACT_NONE, stream);
    }
    // forward with the activation folded into the GEMM epilogue
    void forward_act(half* output, const half* input, int act, cudaStream_t stream = 0) const {
        etChk(et_linear_dense_fwd(et_ptr(input), et_ptr(weight.get()), et_ptr(bias.get()),
                                  et_ptr(output), size, in_size, out_size, act, stream));
    }
};

// The transposed matrix is column pruned: only the output features in weight.row_id exist.
template <> class Linear<row_mat> {
  public:
    const uint32_t in_size;
    const uint32_t out_size;
    row_mat weight;
    culib::CUDA_ptr<half> bias;
    int size;

    Linear(int _in_size, int _out_size, const row_mat& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), weight(w), bias(b, _out_size), size(_size) {}
    Linear(int _in_size, int _out_size, row_mat&& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), weight(std::move(w)), bias(b, _out_size),
          size(_size) {}
    void forward(half* output, half* input, cudaStream_t stream = 0) const {
        forward_act(output, input, ET_ACT_NONE, stream);
    }
    void forward_act(half* output, const half* input, int act, cudaStream_t stream = 0) const {
        etChk(et_linear_row_fwd(weight.row_id->get(), et_ptr(weight.rows->get()),
                                (int)weight.row_id->size, et_ptr(bias.get()), et_ptr(input),
                                et_ptr(output), size, (int)in_size, (int)out_size, act, stream));
    }
    // compressed output [size, nn_row] into a col_mat activation (feeds Prune_attn)
    void forward(col_mat* output, half* input, cudaStream_t stream = 0) const {
        etChk(et_linear_row_compressed_fwd(weight.row_id->get(), et_ptr(weight.rows->get()),
                                           (int)weight.row_id->size, et_ptr(bias.get()),
                                           et_ptr(input), et_ptr(output->cols->get()), size,
                                           (int)in_size, stream));
    }
};

template <> class Linear<csr_mat> {
  public:
    const uint32_t in_size;
    const uint32_t out_size;
    const int size;
    culib::CUDA_ptr<int>* indptr;
    culib::CUDA_ptr<int>* indices;
    culib::CUDA_ptr<half>* data;
    culib::CUDA_ptr<half> bias;

    Linear(int _in_size, int _out_size, const csr_mat& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), size(_size), bias(b, _out_size) {
        etChk(et_validate_csr(w.indptr.data(), w.indices.data(), w.nnz, _in_size, _out_size));
        std::vector<half> h(w.data.size());
        for (size_t i = 0; i < h.size(); ++i) h[i] = __float2half_rn(w.data[i]);
        indptr = new culib::CUDA_ptr<int>(w.indptr);
        indices = new culib::CUDA_ptr<int>(w.indices);
        data = new culib::CUDA_ptr<half>(h);
    }
    Linear(Linear<csr_mat>&& o)
        : in_size(o.in_size), out_size(o.out_size), size(o.size), indptr(o.indptr),
          indices(o.indices), data(o.data), bias(std::move(o.bias)) {
        o.indptr = o.indices = nullptr;
        o.data = nullptr;
    }
    ~Linear() {
        delete indptr;
        delete indices;
        delete data;
    }
    void forward(half* output, half* input, cudaStream_t stream = 0) {
        etChk(et_linear_csr_fwd(indptr->get(), indices->get(), et_ptr(data->get()),
                                (int)indices->size, et_ptr(bias.get()), et_ptr(input),
                                et_ptr(output), size, (int)in_size, (int)out_size, ET_ACT_NONE,
                                stream));
    }
};

// The transposed matrix is row pruned: only the input features in weight.col_id are used.
template <> class Linear<col_mat> {
  public:
    const uint32_t in_size;
    const uint32_t out_size;
    col_mat weight;
    culib::CUDA_ptr<half> bias;
    int size;
    culib::CUDA_ptr<half> workspace;  // gathered activations [size, nnz_col]

    Linear(int _in_size, int _out_size, const col_mat& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), weight(w), bias(b, _out_size), size(_size),
          workspace((size_t)_size * w.col_id->size) {}
    Linear(int _in_size, int _out_size, col_mat&& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), weight(std::move(w)), bias(b, _out_size),
          size(_size), workspace((size_t)_size * weight.col_id->size) {}
    void forward(half* output, half* input, cudaStream_t stream = 0) const {
        forward_act(output, input, ET_ACT_NONE, stream);
    }
    void forward_act(half* output, const half* input, int act, cudaStream_t stream = 0) const {
        etChk(et_linear_col_fwd(weight.col_id->get(), et_ptr(weight.cols->get()),
                                (int)weight.col_id->size, et_ptr(bias.get()), et_ptr(input),
                                et_ptr(output), size, (int)in_size, (int)out_size, act,
                                et_ptr(workspace.get()), workspace.size * sizeof(half), stream));
    }
};

// Tile-pruned Linear.  At construction the weight is prepared once for the kernel that will
// serve it (the choice et_tile_prefer_dense makes): expanded to a dense matrix for the GEMM, or
// re-packed (tiles of a panel and chunk contiguous, pre-swizzled) for the tile kernel.  The
// reference's arrays stay available in `weight`.
template <> class Linear<tile_mat> {
  public:
    const uint32_t in_size;
    const uint32_t out_size;
    const int size;
    tile_mat weight;
    culib::CUDA_ptr<half> bias;

    Linear(int _in_size, int _out_size, const tile_mat& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), size(_size), weight(w), bias(b, _out_size) {
        prepare();
    }
    Linear(int _in_size, int _out_size, const tile_mat& w, culib::CUDA_ptr<half>& b, int _size)
        : in_size(_in_size), out_size(_out_size), size(_size), weight(w), bias(b) {
        prepare();
    }
    Linear(int _in_size, int _out_size, tile_mat&& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), size(_size), weight(std::move(w)),
          bias(b, _out_size) {
        prepare();
    }
    Linear(Linear<tile_mat>&& o)
        : in_size(o.in_size), out_size(o.out_size), size(o.size), weight(std::move(o.weight)),
          bias(std::move(o.bias)), dense(std::move(o.dense)), pk_mask(std::move(o.pk_mask)),
          pk_off(std::move(o.pk_off)), pk_tiles(std::move(o.pk_tiles)) {}
    void forward(half* output, const half* const input, cudaStream_t stream = 0) {
        forward_act(output, input, ET_ACT_NONE, stream);
    }
    void forward_act(half* output, const half* input, int act, cudaStream_t stream = 0) {
        if (dense) {
            etChk(et_linear_dense_fwd(et_ptr(input), et_ptr(dense->get()), et_ptr(bias.get()),
                                      et_ptr(output), size, (int)in_size, (int)out_size, act,
                                      stream));
        } else if (pk_tiles) {
            etChk(et_linear_tile_packed_fwd(
                weight.row_ptr.get(), reinterpret_cast<const uint32_t*>(pk_mask->get()),
                pk_off->get(), et_ptr(pk_tiles->get()), weight.num_blk, et_ptr(bias.get()),
                et_ptr(input), et_ptr(output), size, (int)in_size, (int)out_size, act, stream));
        } else {
            etChk(et_linear_tile_fwd(weight.row_ptr.get(), weight.row_offset.get(),
                                     et_ptr(weight.data.get()), weight.num_blk, et_ptr(bias.get()),
                                     et_ptr(input), et_ptr(output), size, (int)in_size,
                                     (int)out_size, act, stream));
        }
    }

  private:
    std::unique_ptr<culib::CUDA_ptr<half>> dense;     // expanded weight [out, in]
    std::unique_ptr<culib::CUDA_ptr<int>> pk_mask;    // per (panel, chunk) presence bits
    std::unique_ptr<culib::CUDA_ptr<int>> pk_off;     // per (panel, chunk) first tile
    std::unique_ptr<culib::CUDA_ptr<half>> pk_tiles;  // tiles in packed order

    void prepare() {
        if (weight.num_blk <= 0) return;
        if (et_tile_prefer_dense((int)in_size, (int)out_size, weight.num_blk)) {
            dense = std::make_unique<culib::CUDA_ptr<half>>((size_t)in_size * out_size);
            etChk(et_tile_densify(weight.row_ptr.get(), weight.row_offset.get(),
                                  et_ptr(weight.data.get()), weight.num_blk, (int)in_size,
                                  (int)out_size, et_ptr(dense->get()), 0));
            cudaChk(cudaStreamSynchronize(0));
            return;
        }
        int npanel = 0, nchunk = 0;
        etChk(et_tile_pack_dims((int)in_size, (int)out_size, &npanel, &nchunk));
        const std::vector<int> rp = weight.row_ptr.to_host(), ro = weight.row_offset.to_host();
        std::vector<uint32_t> mask((size_t)npanel * nchunk);
        std::vector<int> off((size_t)npanel * nchunk), perm((size_t)weight.num_blk);
        etChk(et_tile_pack_plan(rp.data(), ro.data(), weight.num_blk, (int)in_size, (int)out_size,
                                mask.data(), off.data(), perm.data()));
        pk_mask = std::make_unique<culib::CUDA_ptr<int>>(reinterpret_cast<const int*>(mask.data()),
                                                         mask.size());
        pk_off = std::make_unique<culib::CUDA_ptr<int>>(off.data(), off.size());
        culib::CUDA_ptr<int> dperm(perm.data(), perm.size());
        pk_tiles = std::make_unique<culib::CUDA_ptr<half>>((size_t)weight.num_blk * 256);
        etChk(et_tile_pack_tiles(et_ptr(weight.data.get()), dperm.get(), weight.num_blk,
                                 et_ptr(pk_tiles->get()), 0));
        cudaChk(cudaStreamSynchronize(0));
    }
};

// 1x16-vector weights.  A tensor-core product cannot skip single vectors inside a 16 x 16
// tile, so at construction the weight is expanded once to a dense matrix when the library
// expects the dense GEMM to win (et_1x16_prefer_dense: unless almost nothing is stored); the
// vector kernel serves the rest.  The reference's arrays stay available in `weight`.
template <> class Linear<mat1x16> {
  public:
    const uint32_t in_size;
    const uint32_t out_size;
    const int size;
    mat1x16 weight;
    culib::CUDA_ptr<half> bias;

    Linear(int _in_size, int _out_size, const mat1x16& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), size(_size), weight(w), bias(b, _out_size) {
        prepare();
    }
    Linear(int _in_size, int _out_size, mat1x16&& w, const half* b, int _size)
        : in_size(_in_size), out_size(_out_size), size(_size), weight(std::move(w)),
          bias(b, _out_size) {
        prepare();
    }
    void forward(half* output, half* input, cudaStream_t stream = 0) {
        forward_act(output, input, ET_ACT_NONE, stream);
    }
    void forward_act(half* output, const half* input, int act, cudaStream_t stream = 0) {
        if (dense) {
            etChk(et_linear_dense_fwd(et_ptr(input), et_ptr(dense->get()), et_ptr(bias.get()),
                                      et_ptr(output), size, (int)in_size, (int)out_size, act,
                                      stream));
            return;
        }
        etChk(et_linear_1x16_fwd(weight.tile_idx.get(), weight.row_idx.get(),
                                 et_ptr(weight.data.get()), weight.ntile, et_ptr(bias.get()),
                                 et_ptr(input), et_ptr(output), size, (int)in_size, (int)out_size,
                                 act, stream));
    }

  private:
    std::unique_ptr<culib::CUDA_ptr<half>> dense;  // expanded weight [out, in]

    void prepare() {
        if (weight.ntile <= 0 || !et_1x16_prefer_dense((int)in_size, (int)out_size, weight.ntile))
            return;
        dense = std::make_unique<culib::CUDA_ptr<half>>((size_t)in_size * out_size);
        etChk(et_1x16_densify(weight.tile_idx.get(), weight.row_idx.get(), et_ptr(weight.data.get()),
                              weight.ntile, (int)in_size, (int)out_size, et_ptr(dense->get()), 0));
        cudaChk(cudaStreamSynchronize(0));
    }
};

// ---- factories (Linear/gen_linear.hpp:1-28): nrow = out features, ncol = in features,
// constant weights 1.0, bias 0.5 ----------------------------------------------------------
template <typename T> std::unique_ptr<Linear<T>> gen_dense_linear(int nrow, int ncol, int size) {
    auto W = T::gen_dense_mat(nrow, ncol);
    std::vector<half> bias(nrow, __float2half_rn(0.5f));
    return std::make_unique<Linear<T>>(ncol, nrow, std::move(W), bias.data(), size);
}
template <>
inline std::unique_ptr<Linear<base_mat>> gen_dense_linear<base_mat>(int nrow, int ncol, int size) {
    base_mat W((size_t)nrow * ncol, __float2half_rn(1.0f));
    std::vector<half> bias(nrow, __float2half_rn(0.5f));
    return std::make_unique<Linear<base_mat>>(ncol, nrow, std::move(W), bias.data(), size);
}
template <typename T>
std::unique_ptr<Linear<T>> gen_sparse_linear(int nrow, int ncol, int size, float sparsity) {
    auto W = T::gen_sparse_mat(nrow, ncol, sparsity);
    std::vector<half> bias(nrow, __float2half_rn(0.5f));
    return std::make_unique<Linear<T>>(ncol, nrow, std::move(W), bias.data(), size);
}
template <>
inline std::unique_ptr<Linear<base_mat>> gen_sparse_linear<base_mat>(int nrow, int ncol, int size,
                                                                     float) {
    return gen_dense_linear<base_mat>(nrow, ncol, size);
}
