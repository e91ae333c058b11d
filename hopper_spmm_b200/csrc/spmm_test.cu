// spmm_test <matrix_file> <feature_dim> [fp16|tf32] [rw8] [gpus=N]
//
// The command-line run of the reference's main (src/fp16.cu:283-319) on top of the C ABI: load a
// MatrixMarket file, convert it to the condensed format, fill B with rand() / RAND_MAX as the
// reference does, time the SpMM with its protocol (3 warm-up launches, 5 timed ones) and print
// the matrix summary and the timing block.  Unlike the reference, whose "result check" is an
// empty comment, it then checks a sample of C's rows against a plain CSR product on the host.
// With "rw8" the matrix is first converted with the reference's own 8-row windows (ROW_WINDOW,
// src/common.h:17) and that format is re-windowed to the 16 rows the kernels consume - the route a
// format built by the reference's converter takes.  With "gpus=N" the product is also run row-sharded
// over N GPUs through the sharded operator (host B in, host C out) and compared with the one-GPU result.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/b200_spmm.h"

namespace {

int fail(const char *what, int st) {
    std::fprintf(stderr, "%s: %s %s\n", what, b200spmm_status_string(st), st == B200SPMM_ERR_CUDA ? b200spmm_last_cuda_error() : "");
    return 1;
}

float element(const void *values, bool f16, uint64_t i) {
    return f16 ? __half2float(static_cast<const __half *>(values)[i]) : static_cast<const float *>(values)[i];
}

}  // namespace

int main(int argc, char *argv[]) {
    if (argc < 3 || argc > 6) {
        std::printf("Usage: %s <matrix_file> <feature_dim> [fp16|tf32] [rw8] [gpus=N]\n", argv[0]);
        return 1;
    }
    const char *matrix_file = argv[1];
    const int64_t n = std::atoll(argv[2]);
    bool f16 = true, via_rw8 = false;
    int gpus = 1;
    for (int i = 3; i < argc; ++i) {
        if (std::strcmp(argv[i], "tf32") == 0) f16 = false;
        else if (std::strcmp(argv[i], "rw8") == 0) via_rw8 = true;
        else if (std::strncmp(argv[i], "gpus=", 5) == 0 && std::atoi(argv[i] + 5) >= 1) gpus = std::atoi(argv[i] + 5);
        else if (std::strcmp(argv[i], "fp16") != 0) {
            std::fprintf(stderr, "unknown option %s\n", argv[i]);
            return 1;
        }
    }
    const int dtype = f16 ? B200SPMM_F16 : B200SPMM_TF32;
    if (n <= 0 || n % 8) {
        std::fprintf(stderr, "feature_dim must be a positive multiple of 8\n");
        return 1;
    }

    b200spmm_csr_t *csr = nullptr;
    int st = b200spmm_load_matrix(matrix_file, dtype, &csr);
    if (st) return fail("load_matrix", st);
    uint64_t rows, cols, nnz, declared;
    b200spmm_csr_info(csr, &rows, &cols, &nnz, &declared);
    if (nnz != declared) std::printf("warning: %llu entries read, %llu promised\n", (unsigned long long)nnz, (unsigned long long)declared);
    const uint32_t *row_ptr = b200spmm_csr_row_ptr(csr), *col_idx = b200spmm_csr_col_idx(csr);
    const void *values = b200spmm_csr_values(csr);

    b200spmm_btcf_t *btcf = nullptr;
    st = b200spmm_csr2btcf_nobitmap(rows, cols, nnz, row_ptr, col_idx, values, dtype, via_rw8 ? 8 : 16, 0, 0, &btcf);
    if (st) return fail("CSR2BTCFNOBITMAP", st);
    b200spmm_btcf_info_t info;
    b200spmm_btcf_info(btcf, &info);
    if (via_rw8) {  // the 8-row format, as the reference builds it, brought to 16-row windows
        std::printf("8-row format: %llu non-empty row windows, %llu tiles\n", (unsigned long long)info.eff_row_windows,
                    (unsigned long long)info.total_tiles);
        b200spmm_btcf_t *wide = nullptr;
        st = b200spmm_btcf_rewindow(&info, b200spmm_btcf_rowOffset(btcf), b200spmm_btcf_tcA2B(btcf), b200spmm_btcf_data(btcf),
                                    b200spmm_btcf_rowIdx(btcf), 16, 0, &wide);
        if (st) return fail("btcf_rewindow", st);
        b200spmm_btcf_destroy(btcf);
        btcf = wide;
        b200spmm_btcf_info(btcf, &info);
    }
    std::printf("=== BTCF matrix ===\n");
    std::printf("rows: %llu\n", (unsigned long long)info.rows);
    std::printf("cols: %llu\n", (unsigned long long)info.cols);
    std::printf("nonzeros: %llu\n", (unsigned long long)info.nnzs);
    std::printf("row windows: %llu\n", (unsigned long long)info.total_row_windows);
    std::printf("non-empty row windows: %llu\n", (unsigned long long)info.eff_row_windows);
    std::printf("tiles (%dx%d): %llu\n", info.row_window, info.col_window, (unsigned long long)info.total_tiles);

    // B: rand() / RAND_MAX, element after element (src/fp16.cu:304-306)
    const size_t esz = f16 ? 2 : 4;
    std::vector<uint8_t> hB((size_t)cols * n * esz);
    for (size_t i = 0; i < (size_t)cols * n; ++i) {
        const float v = static_cast<float>(std::rand()) / RAND_MAX;
        if (f16) reinterpret_cast<__half *>(hB.data())[i] = __float2half(v);
        else reinterpret_cast<float *>(hB.data())[i] = v;
    }

    b200spmm_plan_t *plan = nullptr;
    st = b200spmm_plan_create(btcf, 0, 0, &plan);
    if (st) return fail("plan_create", st);
    void *dB = nullptr, *dC = nullptr;
    if (cudaMalloc(&dB, hB.size()) != cudaSuccess || cudaMalloc(&dC, (size_t)rows * n * sizeof(float)) != cudaSuccess ||
        cudaMemcpy(dB, hB.data(), hB.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
        std::fprintf(stderr, "device buffers: %s\n", cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    float total_ms = 0.f;
    const int warmup = 3, runs = 5;  // WARMUP_RUNS, RUNS (src/common.h:47-48)
    st = b200spmm_bench(plan, dB, n, n, dC, n, B200SPMM_C_F32, warmup, runs, nullptr, &total_ms);
    if (st) return fail("spmm", st);
    std::printf("SPMM total time: %.3f ms\n", total_ms);  // PERF_RESULT::print (src/common.h:54-58)
    std::printf("SPMM runs: %d\n", runs);
    std::printf("SPMM mean time: %.3f ms\n", total_ms / runs);
    if (nnz) std::printf("SPMM rate: %.1f GFLOP/s (2*nnz*N)\n", 2.0 * nnz * n / (total_ms / runs * 1e-3) / 1e9);

    // check up to 64 rows spread over the matrix against a CSR product in double precision
    std::vector<float> hC((size_t)rows * n);
    if (cudaMemcpy(hC.data(), dC, hC.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
    const uint64_t step = rows > 64 ? rows / 64 : 1;
    double worst = 0.0;
    for (uint64_t r = 0; r < rows; r += step) {
        for (int64_t j = 0; j < n; ++j) {
            double sum = 0.0, mag = 0.0;
            for (uint32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
                const double a = element(values, f16, p), b = element(hB.data(), f16, (uint64_t)col_idx[p] * n + j);
                sum += a * b;
                mag += std::fabs(a * b);
            }
            const double err = std::fabs(hC[r * n + j] - sum) / (mag > 0 ? mag : 1.0);
            if (err > worst) worst = err;
        }
    }
    const double tol = f16 ? 1e-2 : 5e-3;
    std::printf("check: largest error relative to the magnitude sum %.3e (%s, tolerance %.0e)\n", worst,
                worst <= tol ? "ok" : "FAILED", tol);

    if (gpus > 1) {  // the same product row-sharded over several GPUs, host buffers in and out
        std::vector<int> devices(gpus);
        for (int d = 0; d < gpus; ++d) devices[d] = d;
        b200spmm_sharded_t *sh = nullptr;
        st = b200spmm_sharded_create(rows, cols, nnz, row_ptr, col_idx, values, dtype, devices.data(), gpus, 6, &sh);
        if (st) return fail("sharded_create", st);
        std::vector<uint64_t> cuts(gpus + 1);
        b200spmm_sharded_info(sh, nullptr, cuts.data());
        std::vector<float> hC2((size_t)rows * n);
        st = b200spmm_spmm_sharded_host(sh, hB.data(), n, hC2.data(), B200SPMM_C_F32);
        if (st) return fail("spmm_sharded_host", st);
        double diff = 0.0;
        for (size_t i = 0; i < hC.size(); ++i) diff = std::fmax(diff, std::fabs((double)hC[i] - hC2[i]));
        std::printf("sharded over %d GPUs (row cuts:", gpus);
        for (uint64_t c : cuts) std::printf(" %llu", (unsigned long long)c);
        std::printf("): largest difference to the one-GPU result %.3e\n", diff);
        b200spmm_sharded_destroy(sh);
        if (diff > 1e-3) worst = 1.0;
    }

    cudaFree(dB);
    cudaFree(dC);
    b200spmm_plan_destroy(plan);
    b200spmm_btcf_destroy(btcf);
    b200spmm_csr_destroy(csr);
    return worst <= tol ? 0 : 2;
}
