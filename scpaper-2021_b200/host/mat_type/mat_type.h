// The five pruned-weight containers of the reference, with the same class names, public
// members, constructors and static generators:
//   tile_mat  mat_type/tile_mat/tile_mat.h:3-58     16x16 tile-CSR, block rows = output features
//   mat1x16   mat_type/mat1x16/mat1x16.h:5-22       1x16 vectors grouped by (row set, column part)
//   row_mat   mat_type/row_mat/row_mat.hpp:9-56     kept output rows
//   col_mat   mat_type/col_mat/col_mat.hpp:10-73    kept input columns (also a compressed activation)
//   csr_mat   mat_type/csr_mat/csr_mat.h:11-42      host-side CSR
// Generators produce constant weights 1.0 like the reference's (tile_mat.cu:13), so its
// closed-form smoke values carry over; which units survive is decided by a SEEDED
// Fisher-Yates shuffle (the reference shuffles unseeded), keeping exactly
// floor(units * (1 - sparsity)) of them, ids sorted ascending and padded down to x16.
#pragma once
#include <algorithm>
#include <cstdint>
#include <fstream>
#include <memory>
#include <numeric>
#include <string>
#include <vector>

#include "../lib/CUDA_ptr.hpp"

namespace et_host {

inline uint64_t splitmix64(uint64_t& s) {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// ids[0..keep) = a seeded sample without replacement of range(n), in shuffle order
inline std::vector<int> sample_ids(int n, int keep, uint64_t seed) {
    std::vector<int> ids(n);
    std::iota(ids.begin(), ids.end(), 0);
    uint64_t s = seed;
    for (int i = n - 1; i > 0; --i) std::swap(ids[i], ids[splitmix64(s) % (uint64_t)(i + 1)]);
    ids.resize(keep);
    return ids;
}

inline int kept_units(int n, float sparsity) { return (int)((double)n * (1.0 - (double)sparsity) + 1e-9); }

template <typename T> std::vector<T> read_vec(std::ifstream& f, size_t n) {
    std::vector<T> v(n);
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)(n * sizeof(T)));
    if (!f) throw std::runtime_error("short read in weight file");
    return v;
}

inline uint64_t& generator_seed() {
    static uint64_t seed = 2021;
    return seed;
}

}  // namespace et_host

// Seed used by every gen_sparse_mat call that follows (default 2021).
inline void et_set_generator_seed(uint64_t seed) { et_host::generator_seed() = seed; }

class tile_mat {
  public:
    static constexpr int tile_m = 16, tile_n = 16, tile_k = 16;
    static constexpr int tile_size = tile_m * tile_k;
    int blk_row_num;  // out / 16
    int blk_col_num;  // in / 16
    int num_blk;      // stored tiles
    culib::CUDA_ptr<int> row_ptr;
    culib::CUDA_ptr<int> row_offset;
    culib::CUDA_ptr<half> data;

    tile_mat(const int _blk_row_num, const int _blk_col_num, const int _num_blk, const int* _row_ptr,
             const int* _row_offset, const half* _data)
        : blk_row_num(_blk_row_num), blk_col_num(_blk_col_num), num_blk(_num_blk),
          row_ptr(_row_ptr, _blk_row_num + 1), row_offset(_row_offset, _num_blk),
          data(_data, (size_t)_num_blk * tile_size) {}
    tile_mat(const culib::CUDA_ptr<int>& _row_ptr, const culib::CUDA_ptr<int>& _row_offset,
             const culib::CUDA_ptr<half>& _data, int _blk_col_num)
        : blk_row_num((int)_row_ptr.size - 1), blk_col_num(_blk_col_num),
          num_blk((int)(_data.size / tile_size)), row_ptr(_row_ptr), row_offset(_row_offset),
          data(_data) {}
    tile_mat(const std::vector<int>& _row_ptr, const std::vector<int>& _row_offset,
             const std::vector<half>& _data, int _blk_col_num)
        : blk_row_num((int)_row_ptr.size() - 1), blk_col_num(_blk_col_num),
          num_blk((int)(_data.size() / tile_size)), row_ptr(_row_ptr), row_offset(_row_offset),
          data(_data) {}
    tile_mat(culib::CUDA_ptr<int>&& _row_ptr, culib::CUDA_ptr<int>&& _row_offset,
             culib::CUDA_ptr<half>&& _data, int _blk_col_num)
        : blk_row_num((int)_row_ptr.size - 1), blk_col_num(_blk_col_num),
          num_blk((int)(_data.size / tile_size)), row_ptr(std::move(_row_ptr)),
          row_offset(std::move(_row_offset)), data(std::move(_data)) {}

    // nrow = output features, ncol = input features (both multiples of 16)
    static tile_mat gen_sparse_mat(int nrow, int ncol, float sparsity) {
        const int nbr = nrow / 16, nbc = ncol / 16;
        const int keep = et_host::kept_units(nbr * nbc, sparsity);
        std::vector<int> ids = et_host::sample_ids(nbr * nbc, keep, et_host::generator_seed());
        std::sort(ids.begin(), ids.end());  // block-row major, ascending column inside a row
        std::vector<int> rp(nbr + 1, 0), ro(keep);
        for (int i = 0; i < keep; ++i) {
            rp[ids[i] / nbc + 1]++;
            ro[i] = ids[i] % nbc;
        }
        for (int r = 0; r < nbr; ++r) rp[r + 1] += rp[r];
        std::vector<half> d((size_t)keep * tile_size, __float2half_rn(1.0f));
        return tile_mat(rp, ro, d, nbc);
    }
    static tile_mat gen_dense_mat(int nrow, int ncol) { return gen_sparse_mat(nrow, ncol, 0.f); }
};

class mat1x16 {
    template <typename T> using weight_ptr = culib::CUDA_ptr<T>;

  public:
    const int npart;
    const int nrow;
    const int ncol;
    const int ntile;           // stored 1x16 vectors
    weight_ptr<int> tile_idx;  // (nrow / 16) * (npart + 1)
    weight_ptr<int> row_idx;   // ntile, global output row of each vector
    weight_ptr<half> data;     // ntile * 16
    mat1x16(int _nrow, int _ncol, const std::vector<int>& _tile_idx, const std::vector<int>& _row_idx,
            const std::vector<half>& _data)
        : npart(_ncol / 16), nrow(_nrow), ncol(_ncol), ntile((int)_row_idx.size()),
          tile_idx(_tile_idx), row_idx(_row_idx), data(_data) {}

    static mat1x16 gen_sparse_mat(int nrow, int ncol, float sparsity) {
        const int nset = nrow / 16, npart = ncol / 16;
        const int total = nrow * npart;
        const int keep = et_host::kept_units(total, sparsity);
        // unit id = (set, part, q) in storage order, so sorting yields the stored order
        std::vector<int> ids = et_host::sample_ids(total, keep, et_host::generator_seed());
        std::sort(ids.begin(), ids.end());
        std::vector<int> tidx((size_t)nset * (npart + 1), 0), ridx(keep);
        std::vector<int> count((size_t)nset * npart, 0);
        for (int i = 0; i < keep; ++i) {
            const int q = ids[i] % 16, sp = ids[i] / 16;  // sp = set * npart + part
            count[sp]++;
            ridx[i] = (sp / npart) * 16 + q;
        }
        int run = 0;
        for (int s = 0; s < nset; ++s) {
            for (int p = 0; p < npart; ++p) {
                tidx[(size_t)s * (npart + 1) + p] = run;
                run += count[(size_t)s * npart + p];
            }
            tidx[(size_t)s * (npart + 1) + npart] = run;
        }
        std::vector<half> d((size_t)keep * 16, __float2half_rn(1.0f));
        return mat1x16(nrow, ncol, tidx, ridx, d);
    }
    static mat1x16 gen_dense_mat(int nrow, int ncol) { return gen_sparse_mat(nrow, ncol, 0.f); }
};

class row_mat {
  public:
    int nrow;  // output features of the full matrix
    int ncol;  // input features
    std::unique_ptr<culib::CUDA_ptr<int>> row_id;  // kept output rows, ascending
    std::unique_ptr<culib::CUDA_ptr<half>> rows;   // [len, ncol]

    // file: uint32 nrow, ncol, len; uint32 ids[len]; float32 rows[len * ncol]
    // (row_mat.hpp:15-29, written by mat_type/row_mat/gen_mat.py:24-29)
    explicit row_mat(const std::string& filename) {
        std::ifstream f(filename, std::ios::binary);
        if (!f) throw std::runtime_error("cannot open " + filename);
        auto meta = et_host::read_vec<int>(f, 3);
        nrow = meta[0];
        ncol = meta[1];
        const int len = meta[2];
        row_id = std::make_unique<culib::CUDA_ptr<int>>(et_host::read_vec<int>(f, len));
        auto rf = et_host::read_vec<float>(f, (size_t)ncol * len);
        rows = std::make_unique<culib::CUDA_ptr<half>>((size_t)ncol * len);
        culib::util::to_half_devptr(rows->get(), rf.data(), rf.size());
    }
    row_mat(const culib::CUDA_ptr<int>& _row_id, const culib::CUDA_ptr<half>& _rows, const int _nrow,
            const int _ncol)
        : nrow(_nrow), ncol(_ncol), row_id(std::make_unique<culib::CUDA_ptr<int>>(_row_id)),
          rows(std::make_unique<culib::CUDA_ptr<half>>(_rows)) {}
    row_mat(culib::CUDA_ptr<int>&& _row_id, culib::CUDA_ptr<half>&& _rows, const int _nrow,
            const int _ncol)
        : nrow(_nrow), ncol(_ncol),
          row_id(std::make_unique<culib::CUDA_ptr<int>>(std::move(_row_id))),
          rows(std::make_unique<culib::CUDA_ptr<half>>(std::move(_rows))) {}
    row_mat(const row_mat& m)
        : nrow(m.nrow), ncol(m.ncol), row_id(std::make_unique<culib::CUDA_ptr<int>>(*m.row_id)),
          rows(std::make_unique<culib::CUDA_ptr<half>>(*m.rows)) {}
    row_mat(row_mat&& m) noexcept
        : nrow(m.nrow), ncol(m.ncol), row_id(std::move(m.row_id)), rows(std::move(m.rows)) {}

    static row_mat gen_sparse_mat(int nrow, int ncol, float sparsity) {
        const int keep = et_host::kept_units(nrow, sparsity) / 16 * 16;
        std::vector<int> ids = et_host::sample_ids(nrow, keep, et_host::generator_seed());
        std::sort(ids.begin(), ids.end());
        return row_mat(culib::CUDA_ptr<int>(ids),
                       culib::CUDA_ptr<half>((size_t)keep * ncol, __float2half_rn(1.0f)), nrow, ncol);
    }
    static row_mat gen_dense_mat(int nrow, int ncol) { return gen_sparse_mat(nrow, ncol, 0.f); }
};

// cols is row-major [nrow, nnz_col]
class col_mat {
  public:
    int nrow;
    int ncol;
    int nnz_col;
    int ldm;
    std::unique_ptr<culib::CUDA_ptr<int>> head_ptr;
    std::unique_ptr<culib::CUDA_ptr<int>> col_id;
    std::unique_ptr<culib::CUDA_ptr<half>> cols;

    // head_ptr[h] .. head_ptr[h+1]: entries of the (ascending) id list that fall in head h of a
    // full_dim-wide value tensor (mat_type/col_mat/col_mat.cu:34-58).
    void set_metadata(const culib::CUDA_ptr<int>& _col_id, int _nnz_col, int nhead, int full_dim) {
        std::vector<int> ids = _col_id.to_host();
        ids.resize(_nnz_col);
        const int dh = full_dim / nhead;
        std::vector<int> hp(nhead + 1, 0);
        for (int h = 0; h <= nhead; ++h)
            hp[h] = (int)(std::lower_bound(ids.begin(), ids.end(), h * dh) - ids.begin());
        head_ptr = std::make_unique<culib::CUDA_ptr<int>>(hp);
        col_id = std::make_unique<culib::CUDA_ptr<int>>(ids);
        nnz_col = _nnz_col;
    }
    // file: same header as row_mat with float32 cols[nrow * len] (col_mat.hpp:22-36)
    explicit col_mat(const std::string& filename) {
        std::ifstream f(filename, std::ios::binary);
        if (!f) throw std::runtime_error("cannot open " + filename);
        auto meta = et_host::read_vec<int>(f, 3);
        nrow = meta[0];
        ncol = meta[1];
        nnz_col = meta[2];
        col_id = std::make_unique<culib::CUDA_ptr<int>>(et_host::read_vec<int>(f, nnz_col));
        auto cf = et_host::read_vec<float>(f, (size_t)nrow * nnz_col);
        cols = std::make_unique<culib::CUDA_ptr<half>>((size_t)nrow * nnz_col);
        culib::util::to_half_devptr(cols->get(), cf.data(), cf.size());
        ldm = nnz_col;
    }
    col_mat(const culib::CUDA_ptr<int>& _col_id, const culib::CUDA_ptr<half>& _cols, int _nrow,
            int _ncol, int _nnz_col)
        : nrow(_nrow), ncol(_ncol), nnz_col(_nnz_col),
          col_id(std::make_unique<culib::CUDA_ptr<int>>(_col_id)),
          cols(std::make_unique<culib::CUDA_ptr<half>>(_cols)) {
        ldm = (int)(cols->size / nrow);
    }
    col_mat(culib::CUDA_ptr<int>&& _col_id, culib::CUDA_ptr<half>&& _cols, const int _nrow,
            const int _ncol, int _nnz_col)
        : nrow(_nrow), ncol(_ncol), nnz_col(_nnz_col),
          col_id(std::make_unique<culib::CUDA_ptr<int>>(std::move(_col_id))),
          cols(std::make_unique<culib::CUDA_ptr<half>>(std::move(_cols))) {
        ldm = (int)(cols->size / nrow);
    }
    col_mat(const col_mat& m)
        : nrow(m.nrow), ncol(m.ncol), nnz_col(m.nnz_col), ldm(m.ldm),
          col_id(std::make_unique<culib::CUDA_ptr<int>>(*m.col_id)),
          cols(std::make_unique<culib::CUDA_ptr<half>>(*m.cols)) {
        if (m.head_ptr) head_ptr = std::make_unique<culib::CUDA_ptr<int>>(*m.head_ptr);
    }
    col_mat(col_mat&& m) noexcept
        : nrow(m.nrow), ncol(m.ncol), nnz_col(m.nnz_col), ldm(m.ldm), head_ptr(std::move(m.head_ptr)),
          col_id(std::move(m.col_id)), cols(std::move(m.cols)) {}
    // an empty compressed activation [nrow, nn_col] of a ncol-wide tensor
    col_mat(int _nrow, int _ncol, int _nn_col) : nrow(_nrow), ncol(_ncol), nnz_col(_nn_col) {
        col_id = std::make_unique<culib::CUDA_ptr<int>>((size_t)_nn_col);
        cols = std::make_unique<culib::CUDA_ptr<half>>((size_t)_nrow * _nn_col);
        ldm = _nn_col;
    }
    col_mat* get() { return this; }

    static col_mat gen_sparse_mat(int nrow, int ncol, float sparsity) {
        const int keep = et_host::kept_units(ncol, sparsity) / 16 * 16;
        std::vector<int> ids = et_host::sample_ids(ncol, keep, et_host::generator_seed());
        std::sort(ids.begin(), ids.end());
        return col_mat(culib::CUDA_ptr<int>(ids),
                       culib::CUDA_ptr<half>((size_t)nrow * keep, __float2half_rn(1.0f)), nrow, ncol,
                       keep);
    }
    static col_mat gen_dense_mat(int nrow, int ncol) { return gen_sparse_mat(nrow, ncol, 0.f); }
};

struct csr_mat {
    std::vector<int> indptr;
    std::vector<int> indices;
    std::vector<float> data;
    int nrow;
    int ncol;
    int nnz;
    csr_mat() = delete;
    // file: uint32 nrow, ncol, nnz; int32 indptr[nrow + 1]; int32 indices[nnz]; float32 data[nnz]
    // (csr_mat.h:19-35; fixture mat_type/csr_mat/dense_4_3.csr)
    explicit csr_mat(const std::string& path) {
        std::ifstream fs(path, std::ios::binary);
        if (!fs) throw std::runtime_error("cannot open " + path);
        auto header = et_host::read_vec<uint32_t>(fs, 3);
        nrow = (int)header[0];
        ncol = (int)header[1];
        nnz = (int)header[2];
        indptr = et_host::read_vec<int>(fs, (size_t)nrow + 1);
        indices = et_host::read_vec<int>(fs, (size_t)nnz);
        data = et_host::read_vec<float>(fs, (size_t)nnz);
    }
    csr_mat(std::vector<int> _indptr, std::vector<int> _indices, std::vector<float> _data, int _nrow,
            int _ncol, int _nnz)
        : indptr(std::move(_indptr)), indices(std::move(_indices)), data(std::move(_data)),
          nrow(_nrow), ncol(_ncol), nnz(_nnz) {}

    static csr_mat gen_sparse_mat(int nrow, int ncol, float sparsity) {
        const int total = nrow * ncol;
        const int keep = et_host::kept_units(total, sparsity);
        std::vector<int> ids = et_host::sample_ids(total, keep, et_host::generator_seed());
        std::sort(ids.begin(), ids.end());
        std::vector<int> ip(nrow + 1, 0), ix(keep);
        for (int i = 0; i < keep; ++i) {
            ip[ids[i] / ncol + 1]++;
            ix[i] = ids[i] % ncol;
        }
        for (int r = 0; r < nrow; ++r) ip[r + 1] += ip[r];
        return csr_mat(ip, ix, std::vector<float>(keep, 1.0f), nrow, ncol, keep);
    }
    static csr_mat gen_dense_mat(int nrow, int ncol) { return gen_sparse_mat(nrow, ncol, 0.f); }
};
