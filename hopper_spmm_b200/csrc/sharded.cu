// Row-sharded SpMM over several GPUs of one process, behind the C ABI (include/b200_spmm.h).
//
// The reference's operator is one blocking host call on one GPU (fp16_spmm, src/fp16.cu:221-281);
// its only decomposition is row windows over CTAs (src/fp16.cu:86,138).  Row windows are just as
// independent across GPUs: device p converts and multiplies the contiguous row range the
// time-balanced cuts give it, B is replicated, C is row-sharded, and no data moves between GPUs
// while they compute.  NCCL (over NVLink / NVSwitch) is used for exactly two things: bringing a
// host-resident B onto every GPU with one trip over the host link per byte (every GPU uploads 1/N,
// then an all-gather), and the optional all-gather of C.  Every buffer handed to NCCL or to a
// kernel is the owning GPU's own memory; no kernel reads a peer's memory.
//
// NCCL is loaded with dlopen on first use, so the library itself has no link-time dependency on it
// and loads on machines without it; a missing NCCL surfaces as B200SPMM_ERR_UNSUPPORTED from the
// calls that need a collective (a single-device handle never needs one).
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/b200_spmm.h"
#include "common.hpp"
#include "format.hpp"

namespace b200spmm {
namespace {

struct Nccl {
    void *handle = nullptr;
    bool tried = false;
    decltype(&ncclCommInitAll) CommInitAll = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclSend) Send = nullptr;
    decltype(&ncclRecv) Recv = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    bool ok() const { return handle != nullptr; }
};

Nccl &nccl() {
    static Nccl n;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    if (n.tried) return n;
    n.tried = true;
    void *h = nullptr;
    for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
        h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
        if (h) break;
    }
    if (!h) return n;
    auto sym = [&](const char *s) { return dlsym(h, s); };
    n.CommInitAll = reinterpret_cast<decltype(n.CommInitAll)>(sym("ncclCommInitAll"));
    n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
    n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
    n.GroupStart = reinterpret_cast<decltype(n.GroupStart)>(sym("ncclGroupStart"));
    n.GroupEnd = reinterpret_cast<decltype(n.GroupEnd)>(sym("ncclGroupEnd"));
    n.Send = reinterpret_cast<decltype(n.Send)>(sym("ncclSend"));
    n.Recv = reinterpret_cast<decltype(n.Recv)>(sym("ncclRecv"));
    n.AllGather = reinterpret_cast<decltype(n.AllGather)>(sym("ncclAllGather"));
    if (n.CommInitAll && n.CommDestroy && n.GetErrorString && n.GroupStart && n.GroupEnd && n.Send && n.Recv && n.AllGather)
        n.handle = h;
    return n;
}

}  // namespace
}  // namespace b200spmm

using namespace b200spmm;

struct b200spmm_sharded {
    int n_dev = 0;
    uint64_t rows = 0, cols = 0, nnz = 0;
    int dtype = 0, elt_size = 2;
    std::vector<int> devices;
    std::vector<uint64_t> row_begin;  // [n_dev + 1]
    std::vector<b200spmm_dbtcf_t *> formats;
    std::vector<b200spmm_plan_t *> plans;
    std::vector<cudaStream_t> streams;
    std::vector<ncclComm_t> comms;  // empty until a collective is needed
    // buffers of the host-buffer call, per device, grown on demand
    std::vector<void *> d_B, d_C;
    std::vector<size_t> d_B_bytes, d_C_bytes;
};

namespace {

#define B200_NCCL_TRY(expr)                                                                   \
    do {                                                                                      \
        ncclResult_t r__ = (expr);                                                            \
        if (r__ != ncclSuccess) {                                                             \
            set_last_error_static(nccl().GetErrorString ? nccl().GetErrorString(r__) : #expr); \
            return B200SPMM_ERR_CUDA;                                                         \
        }                                                                                     \
    } while (0)

int ensure_comms(b200spmm_sharded *s) {
    if (s->n_dev == 1 || !s->comms.empty()) return B200SPMM_OK;
    if (!nccl().ok()) {
        set_last_error_static("NCCL (libnccl.so.2) could not be loaded: collectives over several GPUs are unavailable");
        return B200SPMM_ERR_UNSUPPORTED;
    }
    s->comms.assign((size_t)s->n_dev, nullptr);
    ncclResult_t r = nccl().CommInitAll(s->comms.data(), s->n_dev, s->devices.data());
    if (r != ncclSuccess) {
        s->comms.clear();
        set_last_error_static(nccl().GetErrorString(r));
        return B200SPMM_ERR_CUDA;
    }
    return B200SPMM_OK;
}

// Every device holds all of `full[d]` except that only its own byte range [cut[d], cut[d+1]) is valid;
// on return (stream order) every device holds every range.  The ranges may differ in length - the rows are
// cut for equal work, so the device with the lightest rows holds several times the average - and a direct
// exchange is as slow as that device's outgoing link (eight GPUs: 31.6 ms for 8.6 GB).  So it runs in two
// steps: (1) one grouped send/receive moves every byte that lies outside its holder's EVEN part (part q =
// bytes [q total / N, (q + 1) total / N), rounded to 512) to the device whose even part it falls into - each
// such byte crosses one link once; (2) the library's in-place all-gather of the even parts, which loads all
// links alike.  The few bytes past N whole parts go to everybody in step 1.  Where the busiest device would send
// hardly less that way than by sending its range to everybody (two devices), step 1 alone does it all.
int exchange_ranges(b200spmm_sharded *s, void *const *full, const std::vector<uint64_t> &cut) {
    if (s->n_dev == 1) return B200SPMM_OK;
    int st = ensure_comms(s);
    if (st != B200SPMM_OK) return st;
    const Nccl &n = nccl();
    const int N = s->n_dev;
    bool equal = true;
    for (int d = 0; d < N; ++d) equal = equal && (cut[d + 1] - cut[d] == cut[1] - cut[0]);
    const uint64_t part = exchange_even_part(cut.data(), N);
    auto fail = [&](ncclResult_t r) {
        n.GroupEnd();
        set_last_error_static(n.GetErrorString(r));
        return B200SPMM_ERR_CUDA;
    };
    if (!equal) {
        B200_NCCL_TRY(n.GroupStart());
        for (int d = 0; d < N; ++d) {
            char *base = static_cast<char *>(full[d]);
            for (int step = 1; step < N; ++step) {
                int to = 0, from = 0;
                uint64_t pc[8];
                exchange_pieces(cut.data(), N, part, d, step, &to, &from, pc);
                ncclResult_t r = ncclSuccess;
                // sends and receives of a pair of devices in the same order: even part, then tail
                if (pc[1] > pc[0]) r = n.Send(base + pc[0], pc[1] - pc[0], ncclChar, to, s->comms[d], s->streams[d]);
                if (r == ncclSuccess && pc[3] > pc[2]) r = n.Send(base + pc[2], pc[3] - pc[2], ncclChar, to, s->comms[d], s->streams[d]);
                if (r == ncclSuccess && pc[5] > pc[4]) r = n.Recv(base + pc[4], pc[5] - pc[4], ncclChar, from, s->comms[d], s->streams[d]);
                if (r == ncclSuccess && pc[7] > pc[6]) r = n.Recv(base + pc[6], pc[7] - pc[6], ncclChar, from, s->comms[d], s->streams[d]);
                if (r != ncclSuccess) return fail(r);
            }
        }
        B200_NCCL_TRY(n.GroupEnd());
    }
    if (part) {
        B200_NCCL_TRY(n.GroupStart());
        for (int d = 0; d < N; ++d) {  // the library's all-gather, in place
            char *base = static_cast<char *>(full[d]);
            ncclResult_t r = n.AllGather(base + part * (uint64_t)d, base, part, ncclChar, s->comms[d], s->streams[d]);
            if (r != ncclSuccess) return fail(r);
        }
        B200_NCCL_TRY(n.GroupEnd());
    }
    return B200SPMM_OK;
}

int grow(void **buf, size_t *have, size_t need) {
    if (need <= *have) return B200SPMM_OK;
    cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    B200_CUDA_TRY(cudaMalloc(buf, need));
    *have = need;
    return B200SPMM_OK;
}

}  // namespace

extern "C" {

void b200spmm_sharded_destroy(b200spmm_sharded_t *s) {
    if (!s) return;
    for (int d = 0; d < (int)s->devices.size(); ++d) {
        cudaSetDevice(s->devices[d]);
        if (d < (int)s->streams.size() && s->streams[d]) cudaStreamSynchronize(s->streams[d]);
    }
    if (!s->comms.empty() && nccl().ok())
        for (ncclComm_t c : s->comms)
            if (c) nccl().CommDestroy(c);
    for (int d = 0; d < (int)s->devices.size(); ++d) {
        cudaSetDevice(s->devices[d]);
        if (d < (int)s->plans.size()) b200spmm_plan_destroy(s->plans[d]);
        if (d < (int)s->formats.size()) b200spmm_dbtcf_destroy(s->formats[d]);
        if (d < (int)s->d_B.size()) cudaFree(s->d_B[d]);
        if (d < (int)s->d_C.size()) cudaFree(s->d_C[d]);
        if (d < (int)s->streams.size() && s->streams[d]) cudaStreamDestroy(s->streams[d]);
    }
    delete s;
}

int b200spmm_sharded_create(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx,
                            const void *values, int dtype, const int *devices, int n_devices, uint64_t row_charge,
                            b200spmm_sharded_t **out) {
    if (!out) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    if (!devices || n_devices < 1 || n_devices > 64 || !row_ptr || (nnz && (!col_idx || !values))) return B200SPMM_ERR_INVALID_ARG;
    if (dtype != B200SPMM_F16 && dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    for (int a = 0; a < n_devices; ++a)
        for (int b = a + 1; b < n_devices; ++b)
            if (devices[a] == devices[b]) return B200SPMM_ERR_INVALID_ARG;
    int st = validate_csr(rows, cols, nnz, row_ptr, col_idx);
    if (st != B200SPMM_OK) return st;
    int n_dev_present = 0;
    if (cudaGetDeviceCount(&n_dev_present) != cudaSuccess) {
        cudaGetLastError();
        return B200SPMM_ERR_NO_DEVICE;
    }
    for (int d = 0; d < n_devices; ++d)
        if (devices[d] < 0 || devices[d] >= n_dev_present) return B200SPMM_ERR_NO_DEVICE;

    b200spmm_sharded *s = new (std::nothrow) b200spmm_sharded();
    if (!s) return B200SPMM_ERR_NO_MEMORY;
    struct Guard {
        b200spmm_sharded *s;
        ~Guard() { if (s) b200spmm_sharded_destroy(s); }
    } guard{s};
    s->n_dev = n_devices;
    s->rows = rows;
    s->cols = cols;
    s->nnz = nnz;
    s->dtype = dtype;
    s->elt_size = dtype == B200SPMM_F16 ? 2 : 4;
    s->devices.assign(devices, devices + n_devices);
    s->row_begin.assign((size_t)n_devices + 1, 0);
    st = shard_rows(rows, row_ptr, 16, n_devices, row_charge, s->row_begin.data());
    if (st != B200SPMM_OK) return st;
    s->formats.assign((size_t)n_devices, nullptr);
    s->plans.assign((size_t)n_devices, nullptr);
    s->streams.assign((size_t)n_devices, nullptr);
    s->d_B.assign((size_t)n_devices, nullptr);
    s->d_C.assign((size_t)n_devices, nullptr);
    s->d_B_bytes.assign((size_t)n_devices, 0);
    s->d_C_bytes.assign((size_t)n_devices, 0);

    // Every device gets its rows of the CSR (row_ptr rebased to zero), converts them on the device and
    // plans them; the CSR copies are dropped as soon as the format exists.
    std::vector<uint32_t> rp_local;
    for (int d = 0; d < n_devices; ++d) {
        const uint64_t r0 = s->row_begin[d], r1 = s->row_begin[d + 1];
        const uint64_t lo = row_ptr[r0], hi = row_ptr[r1], part_nnz = hi - lo;
        B200_CUDA_TRY(cudaSetDevice(devices[d]));
        B200_CUDA_TRY(cudaStreamCreateWithFlags(&s->streams[d], cudaStreamNonBlocking));
        rp_local.resize(r1 - r0 + 1);
        for (uint64_t r = r0; r <= r1; ++r) rp_local[r - r0] = (uint32_t)(row_ptr[r] - lo);
        uint32_t *d_rp = nullptr, *d_ci = nullptr;
        void *d_v = nullptr;
        auto drop = [&]() { cudaFree(d_rp); cudaFree(d_ci); cudaFree(d_v); };
        cudaError_t e = cudaMalloc(&d_rp, rp_local.size() * 4);
        if (e == cudaSuccess) e = cudaMalloc(&d_ci, std::max<uint64_t>(part_nnz * 4, 16));
        if (e == cudaSuccess) e = cudaMalloc(&d_v, std::max<uint64_t>(part_nnz * s->elt_size, 16));
        if (e == cudaSuccess) e = cudaMemcpy(d_rp, rp_local.data(), rp_local.size() * 4, cudaMemcpyHostToDevice);
        if (e == cudaSuccess && part_nnz) e = cudaMemcpy(d_ci, col_idx + lo, part_nnz * 4, cudaMemcpyHostToDevice);
        if (e == cudaSuccess && part_nnz)
            e = cudaMemcpy(d_v, static_cast<const char *>(values) + lo * s->elt_size, part_nnz * s->elt_size, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            drop();
            record_cuda_error(e, "uploading a shard's CSR");
            return B200SPMM_ERR_CUDA;
        }
        st = b200spmm_csr2btcf_nobitmap_device(r1 - r0, cols, part_nnz, d_rp, d_ci, d_v, dtype, 16, 0, devices[d], s->streams[d],
                                               &s->formats[d]);
        drop();
        if (st != B200SPMM_OK) return st;
        b200spmm_btcf_info_t info;
        b200spmm_dbtcf_info(s->formats[d], &info);
        st = b200spmm_plan_create_device(&info, b200spmm_dbtcf_rowOffset(s->formats[d]), b200spmm_dbtcf_tcA2B(s->formats[d]),
                                         b200spmm_dbtcf_data(s->formats[d]), b200spmm_dbtcf_rowIdx(s->formats[d]), devices[d], 0,
                                         &s->plans[d]);
        if (st != B200SPMM_OK) return st;
    }
    guard.s = nullptr;
    *out = s;
    return B200SPMM_OK;
}

int b200spmm_sharded_info(const b200spmm_sharded_t *s, int *n_devices, uint64_t *row_begin) {
    if (!s) return B200SPMM_ERR_INVALID_ARG;
    if (n_devices) *n_devices = s->n_dev;
    if (row_begin) std::memcpy(row_begin, s->row_begin.data(), s->row_begin.size() * sizeof(uint64_t));
    return B200SPMM_OK;
}

void *b200spmm_sharded_stream(const b200spmm_sharded_t *s, int shard) {
    return (s && shard >= 0 && shard < s->n_dev) ? s->streams[shard] : nullptr;
}

int b200spmm_spmm_sharded(b200spmm_sharded_t *s, const void *const *d_B, int64_t ldb, int64_t n, void *const *d_C, int64_t ldc,
                          int c_dtype) {
    if (!s || !d_B || !d_C) return B200SPMM_ERR_INVALID_ARG;
    for (int d = 0; d < s->n_dev; ++d) {
        if (s->row_begin[d + 1] == s->row_begin[d]) continue;  // a shard without rows
        int st = b200spmm_spmm(s->plans[d], d_B[d], ldb, n, d_C[d], ldc, c_dtype, s->streams[d]);
        if (st != B200SPMM_OK) return st;
    }
    return B200SPMM_OK;
}

int b200spmm_sharded_sync(b200spmm_sharded_t *s) {
    if (!s) return B200SPMM_ERR_INVALID_ARG;
    int worst = B200SPMM_OK;
    for (int d = 0; d < s->n_dev; ++d) {
        int st = b200spmm_plan_sync(s->plans[d], s->streams[d]);
        if (st != B200SPMM_OK && worst == B200SPMM_OK) worst = st;
    }
    return worst;
}

int b200spmm_allgather_c(b200spmm_sharded_t *s, void *const *d_C_full, int64_t n, int c_dtype) {
    if (!s || !d_C_full || n <= 0) return B200SPMM_ERR_INVALID_ARG;
    if (c_dtype != B200SPMM_C_F32 && c_dtype != B200SPMM_C_F16) return B200SPMM_ERR_INVALID_ARG;
    const uint64_t row_bytes = (uint64_t)n * (c_dtype == B200SPMM_C_F32 ? 4 : 2);
    std::vector<uint64_t> cut(s->row_begin);
    for (auto &c : cut) c *= row_bytes;
    return exchange_ranges(s, d_C_full, cut);
}

int b200spmm_spmm_sharded_host(b200spmm_sharded_t *s, const void *h_B, int64_t n, void *h_C, int c_dtype) {
    if (!s || !h_B || !h_C || n <= 0) return B200SPMM_ERR_INVALID_ARG;
    if (c_dtype != B200SPMM_C_F32 && c_dtype != B200SPMM_C_F16) return B200SPMM_ERR_INVALID_ARG;
    const uint64_t b_row = (uint64_t)n * s->elt_size, c_row = (uint64_t)n * (c_dtype == B200SPMM_C_F32 ? 4 : 2);
    const size_t b_bytes = s->cols * b_row;
    // B: device d uploads rows [cols d / N, cols (d+1) / N) of it, then the parts are exchanged GPU to GPU
    std::vector<uint64_t> cut((size_t)s->n_dev + 1);
    for (int d = 0; d <= s->n_dev; ++d) cut[d] = s->cols * (uint64_t)d / (uint64_t)s->n_dev * b_row;
    for (int d = 0; d < s->n_dev; ++d) {
        B200_CUDA_TRY(cudaSetDevice(s->devices[d]));
        int st = grow(&s->d_B[d], &s->d_B_bytes[d], b_bytes);
        if (st == B200SPMM_OK) st = grow(&s->d_C[d], &s->d_C_bytes[d], std::max<uint64_t>((s->row_begin[d + 1] - s->row_begin[d]) * c_row, 16));
        if (st != B200SPMM_OK) return st;
        if (cut[d + 1] > cut[d])
            B200_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(s->d_B[d]) + cut[d], static_cast<const char *>(h_B) + cut[d],
                                          cut[d + 1] - cut[d], cudaMemcpyHostToDevice, s->streams[d]));
    }
    int st = exchange_ranges(s, s->d_B.data(), cut);
    if (st != B200SPMM_OK) return st;
    st = b200spmm_spmm_sharded(s, s->d_B.data(), n, n, s->d_C.data(), n, c_dtype);
    if (st != B200SPMM_OK) return st;
    for (int d = 0; d < s->n_dev; ++d) {
        const uint64_t r0 = s->row_begin[d], r1 = s->row_begin[d + 1];
        if (r1 == r0) continue;
        B200_CUDA_TRY(cudaSetDevice(s->devices[d]));
        B200_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(h_C) + r0 * c_row, s->d_C[d], (r1 - r0) * c_row, cudaMemcpyDeviceToHost,
                                      s->streams[d]));
    }
    return b200spmm_sharded_sync(s);
}

}  // extern "C"
