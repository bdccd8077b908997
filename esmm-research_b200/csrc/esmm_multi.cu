// Several GPUs of one machine from one process: N-column shards of B and C, A replicated.
//
//   C[:, n0:n1] = A * B[:, n0:n1]
//
// needs no exchange between the GPUs: every device holds all of A (and runs the A preprocessor on its own
// replica), a contiguous K x N/G block of B's columns with that block's cached patterns, and the matching
// M x N/G block of C.  One host thread per device launches that device's work; a step's time is taken on each
// device with CUDA events and the whole-box time is the slowest device's.  The reference has no multi-GPU code;
// this is the launcher its command line gets through `--gpus` (driver.cu of this repository).
//
// A collective appears only when all of C must land on one device: an NCCL all-gather of the shards into a
// staging buffer on every device, then the interleave kernel on the first device.  NCCL is looked up at run time
// (dlopen) the first time a gather is asked for, so the library loads and the sharded compute runs without it.
// Before NCCL is entered every device thread has reported, through host memory, that its buffers exist and its
// last step succeeded: a device that failed never enters a collective the others would wait in.
// No kernel here reads another GPU's memory.
#include <dlfcn.h>

#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "esmm_common.cuh"

namespace esmm {

// ---- the few NCCL entry points used, resolved with dlopen ----------------------------------------------------
typedef struct ncclComm *ncclComm_t;
typedef int ncclResult_t;  // 0 = ncclSuccess
struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};
constexpr int kNcclFloat = 7;  // ncclFloat32 in nccl.h's ncclDataType_t

static NcclApi &nccl_api()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) return;
        auto sym = [&](const char *n) { return dlsym(api.handle, n); };
        api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.ok = api.CommInitAll && api.CommDestroy && api.AllGather && api.GroupStart && api.GroupEnd;
    });
    return api;
}

struct Rank {
    int device = 0;
    int n0 = 0, n1 = 0;          // this rank's columns of B and C
    float *d_A = nullptr;        // M x K replica
    float *d_B = nullptr;        // K x width, contiguous
    float *d_C = nullptr;        // M x width
    uint8_t *d_bpat = nullptr;   // cached B patterns of the shard
    void *d_ws = nullptr;        // A patterns + packed A
    float *d_staging = nullptr;  // [G][M][width], allocated at the first gather
    float *d_full = nullptr;     // M x N on rank 0, allocated at the first gather
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int status = ESMM_OK;
    char error[256] = "";
};

}  // namespace esmm

struct esmm_multi {
    int M = 0, N = 0, K = 0, G = 0, width = 0;
    bool have_a = false, have_b = false, have_c = false;
    std::vector<esmm::Rank> ranks;
    std::vector<esmm::ncclComm_t> comms;  // empty until the first gather
};

namespace esmm {

// Runs fn(rank index) on one host thread per device, that device current, and returns the first failing status.
// A rank's failure text is kept in its record and copied to the calling thread's error string.
static int for_each_rank(esmm_multi *m, const std::function<int(int)> &fn)
{
    std::vector<std::thread> pool;
    for (int g = 0; g < m->G; ++g)
        pool.emplace_back([m, g, &fn] {
            Rank &r = m->ranks[g];
            cudaError_t e = cudaSetDevice(r.device);
            if (e != cudaSuccess) {
                r.status = ESMM_ERR_CUDA;
                snprintf(r.error, sizeof r.error, "cudaSetDevice(%d): %s", r.device, cudaGetErrorString(e));
                return;
            }
            r.status = fn(g);
            if (r.status != ESMM_OK) snprintf(r.error, sizeof r.error, "GPU %d: %s %s", r.device, esmm_strerror(r.status),
                                              esmm_last_cuda_error());
        });
    for (auto &t : pool) t.join();
    for (int g = 0; g < m->G; ++g)
        if (m->ranks[g].status != ESMM_OK) {
            record_cuda_error_text(m->ranks[g].error);
            return m->ranks[g].status;
        }
    return ESMM_OK;
}

static int cuda_fail(cudaError_t e, const char *what) { return e == cudaSuccess ? ESMM_OK : record_cuda_error(e, what); }

}  // namespace esmm

extern "C" {

int esmm_multi_shard_columns(int N, int num_gpus, int rank, int *n0, int *n1)
{
    if (num_gpus <= 0 || rank < 0 || rank >= num_gpus || N <= 0) return ESMM_ERR_SHAPE;
    if (N % (num_gpus * 128)) return ESMM_ERR_SHAPE;  // whole GEMM tiles and pattern blocks per shard
    const int w = N / num_gpus;
    if (n0) *n0 = rank * w;
    if (n1) *n1 = (rank + 1) * w;
    return ESMM_OK;
}

int esmm_multi_create(int M, int N, int K, int num_gpus, const int *devices, esmm_multi **out)
{
    if (!out) return ESMM_ERR_NULL;
    *out = nullptr;
    if (M <= 0 || N <= 0 || K <= 0 || (K & 3)) return ESMM_ERR_SHAPE;
    if (esmm_multi_shard_columns(N, num_gpus, 0, nullptr, nullptr) != ESMM_OK) return ESMM_ERR_SHAPE;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return esmm::record_cuda_error_text("no CUDA device");
    }
    for (int g = 0; g < num_gpus; ++g) {
        const int dev = devices ? devices[g] : g;
        if (dev < 0 || dev >= count) {
            char buf[96];
            snprintf(buf, sizeof buf, "rank %d wants device %d but the machine has %d", g, dev, count);
            esmm::record_cuda_error_text(buf);
            return ESMM_ERR_UNSUPPORTED;
        }
    }
    esmm_multi *m = new esmm_multi;
    m->M = M;
    m->N = N;
    m->K = K;
    m->G = num_gpus;
    m->width = N / num_gpus;
    m->ranks.resize(num_gpus);
    for (int g = 0; g < num_gpus; ++g) {
        m->ranks[g].device = devices ? devices[g] : g;
        esmm_multi_shard_columns(N, num_gpus, g, &m->ranks[g].n0, &m->ranks[g].n1);
    }
    int prev = 0;
    cudaGetDevice(&prev);
    const int st = esmm::for_each_rank(m, [m](int g) {
        esmm::Rank &r = m->ranks[g];
        const size_t w = (size_t)m->width;
        ESMM_CUDA_TRY(cudaStreamCreateWithFlags(&r.stream, cudaStreamNonBlocking));
        ESMM_CUDA_TRY(cudaEventCreate(&r.ev0));
        ESMM_CUDA_TRY(cudaEventCreate(&r.ev1));
        ESMM_CUDA_TRY(cudaMalloc(&r.d_A, (size_t)m->M * m->K * sizeof(float)));
        ESMM_CUDA_TRY(cudaMalloc(&r.d_B, (size_t)m->K * w * sizeof(float)));
        ESMM_CUDA_TRY(cudaMalloc(&r.d_C, (size_t)m->M * w * sizeof(float)));
        ESMM_CUDA_TRY(cudaMalloc(&r.d_bpat, esmm_b_pattern_bytes(m->K, m->width)));
        ESMM_CUDA_TRY(cudaMalloc(&r.d_ws, esmm_sgemm_joint_workspace_bytes(m->M, m->K)));
        return (int)ESMM_OK;
    });
    cudaSetDevice(prev);
    if (st != ESMM_OK) {
        esmm_multi_destroy(m);
        return st;
    }
    *out = m;
    return ESMM_OK;
}

int esmm_multi_num_gpus(const esmm_multi *m) { return m ? m->G : 0; }

int esmm_multi_upload(esmm_multi *m, const float *h_A, const float *h_B)
{
    if (!m) return ESMM_ERR_NULL;
    if (!h_A && !h_B) return ESMM_ERR_NULL;
    const int st = esmm::for_each_rank(m, [m, h_A, h_B](int g) {
        esmm::Rank &r = m->ranks[g];
        if (h_A)
            ESMM_CUDA_TRY(cudaMemcpyAsync(r.d_A, h_A, (size_t)m->M * m->K * sizeof(float), cudaMemcpyHostToDevice, r.stream));
        if (h_B) {
            // the rank's columns of the row-major K x N host matrix become a contiguous K x width matrix
            ESMM_CUDA_TRY(cudaMemcpy2DAsync(r.d_B, (size_t)m->width * sizeof(float), h_B + r.n0, (size_t)m->N * sizeof(float),
                                            (size_t)m->width * sizeof(float), (size_t)m->K, cudaMemcpyHostToDevice, r.stream));
            const int s = esmm_preprocess_b(r.d_B, m->K, m->width, r.d_bpat, r.stream);   // offline: once per B
            if (s != ESMM_OK) return s;
        }
        ESMM_CUDA_TRY(cudaStreamSynchronize(r.stream));
        return (int)ESMM_OK;
    });
    if (st == ESMM_OK) {
        m->have_a = m->have_a || h_A != nullptr;
        m->have_b = m->have_b || h_B != nullptr;
    }
    return st;
}

int esmm_multi_fill(esmm_multi *m, uint64_t seed, int mode, uint8_t pattern_a, uint8_t pattern_b, float p_a, float p_b, int gran)
{
    if (!m) return ESMM_ERR_NULL;
    const int st = esmm::for_each_rank(m, [=](int g) {
        esmm::Rank &r = m->ranks[g];
        // the same A on every device; B's shard is generated as its own K x width matrix (seed + 1 + rank)
        int s = esmm_fill_normal(r.d_A, m->M, m->K, 0, seed, 0.f, 1.f, 0, mode, pattern_a, p_a, gran, seed * 7919u + 1, r.stream);
        if (s == ESMM_OK)
            s = esmm_fill_normal(r.d_B, m->K, m->width, 1, seed + 1 + (uint64_t)g, 0.f, 1.f, 0, mode, pattern_b, p_b, gran,
                                 seed * 7919u + 2 + (uint64_t)g, r.stream);
        if (s == ESMM_OK) s = esmm_preprocess_b(r.d_B, m->K, m->width, r.d_bpat, r.stream);
        if (s != ESMM_OK) return s;
        ESMM_CUDA_TRY(cudaStreamSynchronize(r.stream));
        return (int)ESMM_OK;
    });
    if (st == ESMM_OK) m->have_a = m->have_b = true;
    return st;
}

int esmm_multi_run(esmm_multi *m, int runs, float *ms_max, float *ms_per_gpu)
{
    if (!m) return ESMM_ERR_NULL;
    if (runs <= 0) return ESMM_ERR_SHAPE;
    if (!m->have_a || !m->have_b) {
        esmm::record_cuda_error_text("esmm_multi_run before A and B were uploaded");
        return ESMM_ERR_NULL;
    }
    // host barrier: the devices' timed loops start together
    std::mutex mu;
    std::condition_variable cv;
    int arrived = 0, warmed = 0;
    bool warm_failed = false;
    std::vector<float> ms(m->G, 0.f);
    const int st = esmm::for_each_rank(m, [&](int g) {
        esmm::Rank &r = m->ranks[g];
        {
            std::unique_lock<std::mutex> lk(mu);
            if (++arrived == m->G) cv.notify_all();
            else cv.wait(lk, [&] { return arrived == m->G; });
        }
        // one untimed call first: the first launch on a device pays for the loading of the library's device code
        // (a device that fails here still reaches the host barrier below, so that the others are not left waiting,
        // and every device leaves before the timed loop)
        int warm = esmm_sgemm_joint(m->M, m->width, m->K, r.d_A, r.d_B, r.d_C, r.d_bpat, r.d_ws, r.stream);
        if (warm == ESMM_OK) warm = esmm::cuda_fail(cudaStreamSynchronize(r.stream), "warm-up run");
        {
            std::unique_lock<std::mutex> lk(mu);
            if (warm != ESMM_OK) warm_failed = true;
            if (++warmed == m->G) cv.notify_all();
            else cv.wait(lk, [&] { return warmed == m->G; });
        }
        if (warm != ESMM_OK) return warm;
        if (warm_failed) return (int)ESMM_OK;   // another device failed: nothing more is launched here
        ESMM_CUDA_TRY(cudaEventRecord(r.ev0, r.stream));
        for (int i = 0; i < runs; ++i) {
            const int s = esmm_sgemm_joint(m->M, m->width, m->K, r.d_A, r.d_B, r.d_C, r.d_bpat, r.d_ws, r.stream);
            if (s != ESMM_OK) return s;
        }
        ESMM_CUDA_TRY(cudaEventRecord(r.ev1, r.stream));
        const int s = esmm_device_status(r.stream);   // synchronises the stream; ESMM_ERR_TIMEOUT if a wait gave up
        if (s != ESMM_OK) return s;
        float t = 0.f;
        ESMM_CUDA_TRY(cudaEventElapsedTime(&t, r.ev0, r.ev1));
        ms[g] = t / runs;
        return (int)ESMM_OK;
    });
    if (st != ESMM_OK) return st;
    m->have_c = true;
    float worst = 0.f;
    for (int g = 0; g < m->G; ++g) {
        if (ms_per_gpu) ms_per_gpu[g] = ms[g];
        worst = ms[g] > worst ? ms[g] : worst;
    }
    if (ms_max) *ms_max = worst;
    return ESMM_OK;
}

int esmm_multi_download(esmm_multi *m, float *h_C)
{
    if (!m || !h_C) return ESMM_ERR_NULL;
    if (!m->have_c) {
        esmm::record_cuda_error_text("esmm_multi_download before esmm_multi_run");
        return ESMM_ERR_NULL;
    }
    return esmm::for_each_rank(m, [m, h_C](int g) {
        esmm::Rank &r = m->ranks[g];
        ESMM_CUDA_TRY(cudaMemcpy2DAsync(h_C + r.n0, (size_t)m->N * sizeof(float), r.d_C, (size_t)m->width * sizeof(float),
                                        (size_t)m->width * sizeof(float), (size_t)m->M, cudaMemcpyDeviceToHost, r.stream));
        ESMM_CUDA_TRY(cudaStreamSynchronize(r.stream));
        return (int)ESMM_OK;
    });
}

int esmm_multi_gather(esmm_multi *m, float *h_C, float *ms)
{
    if (!m) return ESMM_ERR_NULL;
    if (ms) *ms = 0.f;
    if (!m->have_c) {
        esmm::record_cuda_error_text("esmm_multi_gather before esmm_multi_run");
        return ESMM_ERR_NULL;
    }
    // Pre-flight on the host, before anything of NCCL: distinct devices, NCCL present, every rank's buffers.
    for (int a = 0; a < m->G; ++a)
        for (int b = a + 1; b < m->G; ++b)
            if (m->ranks[a].device == m->ranks[b].device) {
                esmm::record_cuda_error_text("gather needs one rank per device (NCCL refuses a device used twice)");
                return ESMM_ERR_UNSUPPORTED;
            }
    esmm::NcclApi &nc = esmm::nccl_api();
    if (!nc.ok) {
        esmm::record_cuda_error_text("NCCL (libnccl.so.2) not found: use esmm_multi_download instead");
        return ESMM_ERR_UNSUPPORTED;
    }
    int st = esmm::for_each_rank(m, [m](int g) {
        esmm::Rank &r = m->ranks[g];
        if (!r.d_staging) ESMM_CUDA_TRY(cudaMalloc(&r.d_staging, (size_t)m->M * m->N * sizeof(float)));
        if (g == 0 && !r.d_full) ESMM_CUDA_TRY(cudaMalloc(&r.d_full, (size_t)m->M * m->N * sizeof(float)));
        ESMM_CUDA_TRY(cudaStreamSynchronize(r.stream));
        return (int)ESMM_OK;
    });
    if (st != ESMM_OK) return st;   // some rank is not ready: NCCL is never entered
    const bool fresh_comms = m->comms.empty();
    if (fresh_comms) {
        std::vector<int> devs(m->G);
        for (int g = 0; g < m->G; ++g) devs[g] = m->ranks[g].device;
        m->comms.assign(m->G, nullptr);
        const esmm::ncclResult_t r = nc.CommInitAll(m->comms.data(), m->G, devs.data());
        if (r != 0) {
            char buf[160];
            snprintf(buf, sizeof buf, "ncclCommInitAll: %s", nc.GetErrorString ? nc.GetErrorString(r) : "error");
            m->comms.clear();
            return esmm::record_cuda_error_text(buf);
        }
    }
    int prev = 0;
    cudaGetDevice(&prev);
    const size_t count = (size_t)m->M * m->width;
    if (fresh_comms) {
        // a first, small all-gather (untimed) makes NCCL set up its connections
        esmm::ncclResult_t wr = nc.GroupStart();
        for (int g = 0; g < m->G && wr == 0; ++g)
            wr = nc.AllGather(m->ranks[g].d_C, m->ranks[g].d_staging, count < 1024 ? count : 1024, esmm::kNcclFloat, m->comms[g],
                              m->ranks[g].stream);
        const esmm::ncclResult_t we = nc.GroupEnd();
        for (int g = 0; g < m->G; ++g) {
            cudaSetDevice(m->ranks[g].device);
            cudaStreamSynchronize(m->ranks[g].stream);
        }
        if (wr != 0 || we != 0) {
            cudaSetDevice(prev);
            return esmm::record_cuda_error_text("ncclAllGather (connection set-up) failed");
        }
    }
    for (int g = 0; g < m->G; ++g) {
        cudaSetDevice(m->ranks[g].device);
        cudaEventRecord(m->ranks[g].ev0, m->ranks[g].stream);
    }
    // one thread issues the whole group (the single-process form NCCL documents)
    esmm::ncclResult_t nr = nc.GroupStart();
    for (int g = 0; g < m->G && nr == 0; ++g)
        nr = nc.AllGather(m->ranks[g].d_C, m->ranks[g].d_staging, count, esmm::kNcclFloat, m->comms[g], m->ranks[g].stream);
    const esmm::ncclResult_t ne = nc.GroupEnd();
    if (nr == 0) nr = ne;
    if (nr != 0) {
        char buf[160];
        snprintf(buf, sizeof buf, "ncclAllGather: %s", nc.GetErrorString ? nc.GetErrorString(nr) : "error");
        cudaSetDevice(prev);
        return esmm::record_cuda_error_text(buf);
    }
    esmm::Rank &r0 = m->ranks[0];
    cudaSetDevice(r0.device);
    st = esmm_interleave_shards(r0.d_staging, r0.d_full, m->M, m->N, m->G, r0.stream);
    float worst = 0.f;
    for (int g = 0; g < m->G && st == ESMM_OK; ++g) {
        esmm::Rank &r = m->ranks[g];
        cudaSetDevice(r.device);
        st = esmm::cuda_fail(cudaEventRecord(r.ev1, r.stream), "cudaEventRecord");
        if (st == ESMM_OK) st = esmm::cuda_fail(cudaStreamSynchronize(r.stream), "gather");
        float t = 0.f;
        if (st == ESMM_OK) st = esmm::cuda_fail(cudaEventElapsedTime(&t, r.ev0, r.ev1), "cudaEventElapsedTime");
        worst = t > worst ? t : worst;
    }
    if (st == ESMM_OK && h_C) {
        cudaSetDevice(r0.device);
        st = esmm::cuda_fail(cudaMemcpy(h_C, r0.d_full, (size_t)m->M * m->N * sizeof(float), cudaMemcpyDeviceToHost), "copy of C");
    }
    cudaSetDevice(prev);
    if (ms) *ms = worst;
    return st;
}

const float *esmm_multi_gathered_c(const esmm_multi *m) { return m ? m->ranks[0].d_full : nullptr; }

int esmm_multi_destroy(esmm_multi *m)
{
    if (!m) return ESMM_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    esmm::NcclApi &nc = esmm::nccl_api();
    for (int g = 0; g < m->G; ++g) {
        esmm::Rank &r = m->ranks[g];
        if (cudaSetDevice(r.device) != cudaSuccess) continue;
        if (r.stream) cudaStreamSynchronize(r.stream);
        if (g < (int)m->comms.size() && m->comms[g] && nc.ok) nc.CommDestroy(m->comms[g]);
        cudaFree(r.d_A);
        cudaFree(r.d_B);
        cudaFree(r.d_C);
        cudaFree(r.d_bpat);
        cudaFree(r.d_ws);
        cudaFree(r.d_staging);
        cudaFree(r.d_full);
        if (r.ev0) cudaEventDestroy(r.ev0);
        if (r.ev1) cudaEventDestroy(r.ev1);
        if (r.stream) cudaStreamDestroy(r.stream);
    }
    cudaSetDevice(prev);
    cudaGetLastError();
    delete m;
    return ESMM_OK;
}

}  // extern "C"
