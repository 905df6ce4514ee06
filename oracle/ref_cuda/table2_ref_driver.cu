// Times the REFERENCE's own CUDA implementation (its kernels, cuBLAS calls and host classes,
// compiled unmodified from the reference checkout) on its paper-table workload: BERT-base
// shapes, batch 1, seq 128, fp16, N encoder layers built by its constant-weight generators,
// through test_uniform<tile_mat> / test_uniform<base_mat> of its test/Table2/template.hpp.
// Prints one JSON line with microseconds per stack forward.  The reference prints a marker on
// every Encoder::forward; run this program with stdout of the child redirected, or read the
// last line only.  Its OUTPUTS are not a parity target (the shipped kernels have known
// numerical defects); only the time is reported.
#include "template.hpp"

int main(int argc, char** argv) {
    const int nlayer = argc > 1 ? std::atoi(argv[1]) : 12;
    const float sparsity = argc > 2 ? (float)std::atof(argv[2]) : 0.8f;
    auto para = std::make_shared<Model_t>(Model_t{768, 768, 128, 12, 3072, 768});
    std::srand(2021);  // the generators shuffle with std::random_shuffle
    std::streambuf* saved = std::cout.rdbuf(nullptr);  // drop the per-forward marker
    const double t_tile = test_uniform<tile_mat>(para, sparsity, nlayer);
    const double t_dense = test_uniform<base_mat>(para, 0.0f, nlayer);
    std::cout.rdbuf(saved);
    const cudaError_t err = cudaDeviceSynchronize();
    std::printf("{\"reference_cuda\": true, \"layers\": %d, \"batch\": 1, \"seq_len\": 128, "
                "\"tile_sparsity\": %.2f, \"tile_us\": %.1f, \"dense_us\": %.1f, \"cuda_error\": \"%s\"}\n",
                nlayer, sparsity, t_tile, t_dense, cudaGetErrorString(err));
    return err == cudaSuccess ? 0 : 1;
}
