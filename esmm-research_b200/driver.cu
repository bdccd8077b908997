// exec_b200 - the research harness CLI on top of libesmm_b200.
//
// Same command line as the reference driver (driver.cu:142-487, usage text include/utils.cuh:66-101):
//
//   exec_b200 [kernels] [runs] [--verbose|-v] [--no-check|-n] [--random|-r] [--blockwise|-b]
//             [--size|-s N] [--pattern|-p P] [--pattern-a|-pa P] [--pattern-b|-pb P]
//             [--load-a file] [--load-b file] [--dims M K N] [--skip-stats] [--help|-h]
//
// kernels: "29", "29,15", "14-17", "all"; data modes, seeds (12345 / 12346), messages, the cuBLAS
// verification reference with absolute tolerance 1e-2 and the exit code (0 iff every selected
// kernel passed) follow the reference.  Difference: the default kernel is 29 (the reference's
// default is 17).  The single-operand ids 14, 16, 17 run as degenerate cases of the joint kernel.
//
// Additive flags for the inputs the reference CLI cannot express:
//   --uniform            N(0,1) values, the pattern applied to A's K columns AND B's K rows of every
//                        8-slice (joint density = pattern density), generated on the device
//   --tile-random pA pB  N(0,1) values, independent per-tile patterns at 64-row / 64-column granularity
//   --tile-gran G        rows of A / columns of B per tile of --tile-random (default 64; a multiple of 32)
//   --shape M K N        generated data on a non-cubic problem (the reference's --size is cubic only)
//   --seed S             seed of the two modes above (A uses S, B uses S + 1)
//   --cpu-check          also compare C with the driver's CPU SGEMM (matrixMultiplyCPU, all host
//                        threads, relative inf-norm tolerance 1e-4)
//   --cache-b            keep B's pattern bytes in "<load-b file>.bpat" (or the file given with
//                        --cache-b-file): loaded when present and matching, else computed once
//                        and saved; the timed loop then preprocesses A only ("B offline")
//   --gpus G [--gather]  kernel 29 with B, its patterns and C sharded by columns over G GPUs of this machine, A
//                        replicated; one process, one host thread per GPU; whole-box time = slowest GPU's device
//                        time.  --gather collects C on GPU 0 with an NCCL all-gather (timed separately),
//                        otherwise the shards are copied back device by device
//   --json               one machine-readable line per kernel
#include <algorithm>
#include <cctype>
#include <cstring>
#include <thread>

#include "include/utils.cuh"
#include "include/runners.cuh"

namespace {

// The reference's usage text plus the flags and the kernel id added here.
void usage(const char *prog)
{
    std::cout.flush();
    esmm_print_usage(prog, 1);
}

bool pattern_ok(const std::string &p)
{
    return p.size() == 8 && std::all_of(p.begin(), p.end(), [](char c) { return c == '0' || c == '1'; });
}

bool load_bin(const std::string &path, float *buf, size_t n)
{
    if (path.empty()) return true;
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) {
        printf("Error: cannot open %s\n", path.c_str());
        return false;
    }
    const size_t got = fread(buf, sizeof(float), n, f);
    fclose(f);
    if (got != n) {
        printf("Error: expected %zu floats, got %zu from %s\n", n, got, path.c_str());
        return false;
    }
    return true;
}

void cpu_sgemm_threaded(const float *A, const float *B, float *C, int M, int N, int K)
{
    const unsigned nt = std::max(1u, std::thread::hardware_concurrency());
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < nt; ++t)
        pool.emplace_back([=] {
            const int r0 = (int)((long)M * t / nt), r1 = (int)((long)M * (t + 1) / nt);
            if (r1 > r0) matrixMultiplyCPU(A + (size_t)r0 * K, B, C + (size_t)r0 * N, r1 - r0, N, K);
        });
    for (auto &th : pool) th.join();
}

struct Options {
    int rows = 4096, cols = 4096, inners = 4096;
    std::string pattern = "11000000", pattern_a, pattern_b;
    std::vector<int> kernels = {29};
    int runs = 1;
    bool verbose = false, check = true, random_mode = false, blockwise = false, skip_stats = false;
    bool uniform = false, tile_random = false, cpu_check = false, json = false, cache_b = false;
    std::string cache_b_file;
    float p_a = 0.5f, p_b = 0.5f;
    int tile_gran = 64;
    int gpus = 0;          // 0 = the single-GPU path
    bool gather = false;
    int shape_M = 0, shape_K = 0, shape_N = 0;
    unsigned seed = 12345;
    float random_sparsity = 37.5f;
    std::string load_a, load_b;
    int load_M = 0, load_K = 0, load_N = 0;
};

// Returns -1 to continue, otherwise the process exit code.
int parse_args(int argc, char **argv, Options &o)
{
    using std::cout;
    using std::endl;
    auto need = [&](int i, int n, const char *msg) {
        if (i + n >= argc) {
            cout << "Error: " << msg << endl;
            return false;
        }
        return true;
    };
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--help" || a == "-h") {
            usage(argv[0]);
            return 0;
        } else if (a == "--verbose" || a == "-v") o.verbose = true;
        else if (a == "--no-check" || a == "-n") o.check = false;
        else if (a == "--random" || a == "-r") o.random_mode = true;
        else if (a == "--blockwise" || a == "-b") o.blockwise = true;
        else if (a == "--skip-stats") o.skip_stats = true;
        else if (a == "--uniform") o.uniform = true;
        else if (a == "--cpu-check") o.cpu_check = true;
        else if (a == "--json") o.json = true;
        else if (a == "--cache-b") o.cache_b = true;
        else if (a == "--cache-b-file") {
            if (!need(i, 1, "--cache-b-file requires a path")) return 1;
            o.cache_b = true;
            o.cache_b_file = argv[++i];
        }
        else if (a == "--size" || a == "-s") {
            if (!need(i, 1, "--size requires an argument")) {
                usage(argv[0]);
                return 1;
            }
            const int s = atoi(argv[++i]);
            if (s <= 0) {
                cout << "Error: Size must be positive" << endl;
                return 1;
            }
            o.rows = o.cols = o.inners = s;
        } else if (a == "--pattern" || a == "-p" || a == "--pattern-a" || a == "-pa" || a == "--pattern-b" ||
                   a == "-pb") {
            const std::string flag = (a == "-p") ? "--pattern" : (a == "-pa") ? "--pattern-a" : (a == "-pb") ? "--pattern-b" : a;
            if (!need(i, 1, (flag + " requires an argument").c_str())) {
                usage(argv[0]);
                return 1;
            }
            const std::string p = argv[++i];
            if (p.size() != 8) {
                cout << "Error: Pattern must be exactly 8 characters (e.g., '11000000')" << endl;
                return 1;
            }
            if (!pattern_ok(p)) {
                cout << "Error: Pattern must contain only '0' and '1' characters" << endl;
                return 1;
            }
            (flag == "--pattern" ? o.pattern : flag == "--pattern-a" ? o.pattern_a : o.pattern_b) = p;
        } else if (a == "--load-a" || a == "--load-b") {
            if (!need(i, 1, (a + " requires a path").c_str())) return 1;
            (a == "--load-a" ? o.load_a : o.load_b) = argv[++i];
        } else if (a == "--dims") {
            if (!need(i, 3, "--dims requires M K N")) return 1;
            o.load_M = atoi(argv[++i]);
            o.load_K = atoi(argv[++i]);
            o.load_N = atoi(argv[++i]);
        } else if (a == "--tile-random") {
            if (!need(i, 2, "--tile-random requires pA pB")) return 1;
            o.tile_random = true;
            o.p_a = (float)atof(argv[++i]);
            o.p_b = (float)atof(argv[++i]);
        } else if (a == "--gpus") {
            if (!need(i, 1, "--gpus requires an argument")) return 1;
            o.gpus = atoi(argv[++i]);
            if (o.gpus <= 0) {
                cout << "Error: --gpus must be positive" << endl;
                return 1;
            }
        } else if (a == "--gather") {
            o.gather = true;
        } else if (a == "--tile-gran") {
            if (!need(i, 1, "--tile-gran requires an argument")) return 1;
            o.tile_gran = atoi(argv[++i]);
            if (o.tile_gran <= 0 || o.tile_gran % 32) {
                cout << "Error: --tile-gran must be a positive multiple of 32" << endl;
                return 1;
            }
        } else if (a == "--shape") {
            if (!need(i, 3, "--shape requires M K N")) return 1;
            o.shape_M = atoi(argv[++i]);
            o.shape_K = atoi(argv[++i]);
            o.shape_N = atoi(argv[++i]);
            if (o.shape_M <= 0 || o.shape_K <= 0 || o.shape_N <= 0) {
                cout << "Error: --shape needs three positive sizes" << endl;
                return 1;
            }
        } else if (a == "--tune") {
            // additive: one of the library's launch heuristics, by name (esmm_tuning_set)
            if (!need(i, 1, "--tune requires NAME=VALUE")) return 1;
            const std::string nv = argv[++i];
            const size_t eq = nv.find('=');
            if (eq == std::string::npos || eq == 0 || eq + 1 >= nv.size() ||
                esmm_tuning_set(nv.substr(0, eq).c_str(), atoi(nv.c_str() + eq + 1)) != ESMM_OK) {
                cout << "Error: --tune wants NAME=VALUE with a name the library knows, got '" << nv << "'" << endl;
                return 1;
            }
        } else if (a == "--seed") {
            if (!need(i, 1, "--seed requires an argument")) return 1;
            o.seed = (unsigned)strtoul(argv[++i], nullptr, 10);
        } else if (i == 1) {
            if (isdigit((unsigned char)a[0]) || a == "all" || a.find(',') != std::string::npos ||
                a.find('-') != std::string::npos) {
                o.kernels = parse_kernel_selection(a);
                if (o.kernels.empty()) {
                    cout << "Error: Invalid kernel selection '" << a << "'" << endl;
                    usage(argv[0]);
                    return 1;
                }
            }
        } else if (i == 2 && isdigit((unsigned char)a[0])) {
            o.runs = atoi(argv[i]);
            if (o.runs <= 0) {
                cout << "Error: Number of runs must be positive" << endl;
                return 1;
            }
        }
    }
    return -1;
}

}  // namespace

int main(int argc, char **argv)
{
    using std::cout;
    using std::endl;
    Options o;
    const int early = parse_args(argc, argv, o);
    if (early >= 0) return early;

    for (int k : o.kernels)
        if (!esmm_kernel_id_valid(k)) {
            cout << "Error: Kernel " << k
                 << " is not a valid kernel. Valid kernels are: 14, 15, 16, 17, 20, 21, 25, 26, 27, 28, 29, 30, 129." << endl;
            cout << "Run '" << argv[0] << " --help' to see available kernels." << endl;
            return 1;
        }
    if (o.pattern_a.empty()) o.pattern_a = o.pattern;
    if (o.pattern_b.empty()) o.pattern_b = o.pattern;

    const bool load_mode = !o.load_a.empty() || !o.load_b.empty();
    if (load_mode) {
        if (o.load_M <= 0 || o.load_K <= 0 || o.load_N <= 0) {
            cout << "Error: --dims M K N required with --load-a / --load-b" << endl;
            return 1;
        }
        o.rows = o.load_M;
        o.inners = o.load_K;
        o.cols = o.load_N;
    }
    if (!load_mode && o.shape_M > 0) {  // generated data on a non-cubic problem (the reference's --size is cubic only)
        o.rows = o.shape_M;
        o.inners = o.shape_K;
        o.cols = o.shape_N;
    }
    const int M = o.rows, N = o.cols, K = o.inners;
    if (o.gpus > 0) {
        // host-side pre-flight, before any device is touched
        if (esmm_multi_shard_columns(N, o.gpus, 0, nullptr, nullptr) != ESMM_OK) {
            cout << "Error: N = " << N << " does not split into " << o.gpus << " column shards of a multiple of 128" << endl;
            return 1;
        }
        for (int k : o.kernels)
            if (k != 29) {
                cout << "Error: --gpus runs kernel 29 only (got " << k << ")" << endl;
                return 1;
            }
    } else if (o.gather) {
        cout << "Error: --gather needs --gpus" << endl;
        return 1;
    }

    if (o.verbose) {
        cout << "Matrix dimensions: " << M << "x" << K << " * " << K << "x" << N << endl;
        cout << "Number of runs per kernel: " << o.runs << endl;
        cout << "Result checking: " << (o.check ? "ENABLED" : "DISABLED") << endl;
        const char *mode = load_mode ? "LOADED (raw float32 files)"
                           : o.uniform ? "UNIFORM (pattern on A's K columns and B's K rows, N(0,1))"
                           : o.tile_random ? "TILE-RANDOM (independent 64-wide tile patterns, N(0,1))"
                           : o.blockwise ? "BLOCK-LEVEL (warp-uniform patterns)"
                           : o.random_mode ? "RANDOM (unstructured)" : "PATTERN-BASED (column-wise)";
        cout << "Sparsity mode: " << mode << endl;
        cout << "  A-matrix pattern: " << o.pattern_a << "  B-matrix pattern: " << o.pattern_b << endl;
        cout << "Kernels to run: ";
        for (size_t i = 0; i < o.kernels.size(); ++i) cout << o.kernels[i] << (i + 1 < o.kernels.size() ? ", " : "");
        cout << endl << endl;
    }

    const size_t nA = (size_t)M * K, nB = (size_t)K * N, nC = (size_t)M * N;
    float *h_A = (float *)malloc(nA * sizeof(float));
    float *h_B = (float *)malloc(nB * sizeof(float));
    float *h_C = (float *)malloc(nC * sizeof(float));
    float *h_C_ref = (float *)malloc(nC * sizeof(float));
    if (!h_A || !h_B || !h_C || !h_C_ref) {
        cout << "Error: host allocation failed" << endl;
        return 1;
    }
    float *d_A, *d_B, *d_C;
    cudaCheckError(cudaMalloc(&d_A, nA * sizeof(float)));
    cudaCheckError(cudaMalloc(&d_B, nB * sizeof(float)));
    cudaCheckError(cudaMalloc(&d_C, nC * sizeof(float)));

    const bool device_generated = !load_mode && (o.uniform || o.tile_random);
    if (device_generated) {
        const int mode = o.uniform ? 1 : 2;
        const int pa = esmm_pattern_from_string(o.pattern_a.c_str()), pb = esmm_pattern_from_string(o.pattern_b.c_str());
        int st = esmm_fill_normal(d_A, M, K, 0, o.seed, 0.f, 1.f, 0, mode, (uint8_t)pa, o.p_a, o.tile_gran, o.seed * 7919u + 1, nullptr);
        if (st == ESMM_OK)
            st = esmm_fill_normal(d_B, K, N, 1, o.seed + 1, 0.f, 1.f, 0, mode, (uint8_t)pb, o.p_b, o.tile_gran, o.seed * 7919u + 2, nullptr);
        if (st != ESMM_OK) {
            cout << "Error: generator failed: " << esmm_strerror(st) << " " << esmm_last_cuda_error() << endl;
            return 1;
        }
        cudaCheckError(cudaMemcpy(h_A, d_A, nA * sizeof(float), cudaMemcpyDeviceToHost));
        cudaCheckError(cudaMemcpy(h_B, d_B, nB * sizeof(float), cudaMemcpyDeviceToHost));
    } else {
        if (load_mode) {
            if (!load_bin(o.load_a, h_A, nA) || !load_bin(o.load_b, h_B, nB)) return 1;
            if (o.load_a.empty()) {  // dense random A in [-1, 1] (driver.cu:356-360)
                srand(o.seed);
                for (size_t i = 0; i < nA; ++i) h_A[i] = ((float)rand() / RAND_MAX) * 2.0f - 1.0f;
            }
            if (o.load_b.empty()) {
                srand(o.seed + 1);
                for (size_t i = 0; i < nB; ++i) h_B[i] = ((float)rand() / RAND_MAX) * 2.0f - 1.0f;
            }
        } else if (o.blockwise) {
            auto sparsity_of = [](const std::string &p) {
                return 100.0f - ((float)std::count(p.begin(), p.end(), '1') / 8.0f) * 100.0f;
            };
            // A is regenerated once per selected id, 8-row tiles for id 21 and 32-row tiles otherwise, so the
            // last id decides (driver.cu:379-387); the generators are the reference's own, by name
            for (int k : o.kernels) {
                if (k == 21) randomize_matrix_A<8, 8>(h_A, M, K, sparsity_of(o.pattern_a), o.seed);
                else randomize_matrix_A_blocklevel<8, 32>(h_A, M, K, sparsity_of(o.pattern_a), o.seed);
            }
            randomize_matrix_B_blocklevel_fixed<8, 32>(h_B, K, N, sparsity_of(o.pattern_b), o.seed + 1);
        } else if (o.random_mode) {
            randomize_matrix_unstructured(h_A, M, K, o.random_sparsity, o.seed);
            randomize_matrix_unstructured(h_B, K, N, o.random_sparsity, o.seed + 1);
        } else {
            randomize_matrix_with_pattern(h_A, M, K, o.pattern_a);
            randomize_matrix_with_pattern(h_B, K, N, o.pattern_b);
        }
        cudaCheckError(cudaMemcpy(d_A, h_A, nA * sizeof(float), cudaMemcpyHostToDevice));
        cudaCheckError(cudaMemcpy(d_B, h_B, nB * sizeof(float), cudaMemcpyHostToDevice));
    }
    memset(h_C, 0, nC * sizeof(float));

    if (o.check) {
        if (o.verbose) cout << "Generating GPU reference solution using cuBLAS..." << endl;
        const int st = esmm_cublas_sgemm(M, N, K, d_A, d_B, d_C, nullptr);
        if (st != ESMM_OK || cudaDeviceSynchronize() != cudaSuccess) {
            cout << "Error generating reference with cuBLAS: " << esmm_strerror(st) << endl;
            return 1;
        }
        cudaCheckError(cudaMemcpy(h_C_ref, d_C, nC * sizeof(float), cudaMemcpyDeviceToHost));
        if (o.verbose) cout << "GPU reference generated successfully." << endl;
    } else if (o.verbose) {
        cout << "Skipping reference solution (no-check mode)..." << endl;
    }

    // B pattern cache: the patterns of a static B are computed once and reused.
    uint8_t *d_b_cached = nullptr;
    if (o.cache_b) {
        std::string path = o.cache_b_file;
        if (path.empty() && !o.load_b.empty()) path = o.load_b + ".bpat";
        if (path.empty()) {
            cout << "Error: --cache-b needs --load-b or --cache-b-file" << endl;
            return 1;
        }
        const size_t nb = esmm_b_pattern_bytes(K, N);
        std::vector<uint8_t> h_bpat(nb);
        cudaCheckError(cudaMalloc(&d_b_cached, nb));
        int st = esmm_bpat_load(path.c_str(), h_bpat.data(), K, N);
        if (st == ESMM_OK) {
            cudaCheckError(cudaMemcpy(d_b_cached, h_bpat.data(), nb, cudaMemcpyHostToDevice));
            cout << "B patterns: loaded from " << path << endl;
        } else {
            if (st == ESMM_ERR_MISMATCH) cout << "B patterns: " << path << " was written for another shape, recomputing" << endl;
            st = esmm_preprocess_b(d_B, K, N, d_b_cached, nullptr);
            if (st != ESMM_OK || cudaDeviceSynchronize() != cudaSuccess) {
                cout << "Error: B preprocessing failed: " << esmm_strerror(st) << endl;
                return 1;
            }
            cudaCheckError(cudaMemcpy(h_bpat.data(), d_b_cached, nb, cudaMemcpyDeviceToHost));
            st = esmm_bpat_save(path.c_str(), h_bpat.data(), K, N);
            cout << "B patterns: computed" << (st == ESMM_OK ? " and saved to " : "; could not write ") << path << endl;
        }
    }

    std::vector<float> h_cpu;
    if (o.cpu_check) {
        h_cpu.resize(nC);
        if (o.verbose) cout << "Computing CPU SGEMM on " << std::thread::hardware_concurrency() << " host threads..." << endl;
        cpu_sgemm_threaded(h_A, h_B, h_cpu.data(), M, N, K);
    }

    int passed = 0;
    if (o.gpus > 0) {
        // Kernel 29 on column shards: one process, one host thread per device, A replicated, no exchange in
        // the compute; the blocks of C come back device by device, or through an NCCL all-gather with --gather.
        esmm_multi *mg = nullptr;
        int st = esmm_multi_create(M, N, K, o.gpus, nullptr, &mg);
        if (st == ESMM_OK) st = esmm_multi_upload(mg, h_A, h_B);
        std::vector<float> ms_gpu((size_t)o.gpus, 0.f);
        float ms_max = 0.f, ms_gather = 0.f;
        if (st == ESMM_OK) st = esmm_multi_run(mg, o.runs, &ms_max, ms_gpu.data());
        if (st == ESMM_OK) st = o.gather ? esmm_multi_gather(mg, h_C, &ms_gather) : esmm_multi_download(mg, h_C);
        esmm_multi_destroy(mg);
        if (st != ESMM_OK) {
            cout << "Error: multi-GPU run failed: " << esmm_strerror(st) << " " << esmm_last_cuda_error() << endl;
            return 1;
        }
        printf("Kernel time: %.3f ms (avg: %.3f ms)\n", ms_max * o.runs, ms_max);
        printf("  %d GPUs, column shards of %d; per-GPU avg ms:", o.gpus, N / o.gpus);
        for (float t : ms_gpu) printf(" %.3f", t);
        printf("; whole-box dense-equivalent %.1f TFLOP/s\n", 2.0 * M * N * K / (ms_max * 1e-3) / 1e12);
        if (o.gather) printf("  gather of C to GPU 0 (NCCL all-gather + interleave): %.3f ms\n", ms_gather);
        bool res = true;
        if (o.check) res = verifyResults(h_C, h_C_ref, (int)nC);
        double cpu_rel = -1.0;
        if (o.cpu_check) {
            double num = 0.0, den = 0.0;
            for (size_t i = 0; i < nC; ++i) {
                num = std::max(num, (double)std::fabs(h_C[i] - h_cpu[i]));
                den = std::max(den, (double)std::fabs(h_cpu[i]));
            }
            cpu_rel = den > 0 ? num / den : num;
            cout << "CPU SGEMM check: rel-inf error " << cpu_rel << (cpu_rel <= 1e-4 ? " (ok)" : " (FAILED)") << endl;
            if (cpu_rel > 1e-4) res = false;
        }
        if (res) ++passed;
        cout << "Kernel 29 (" << get_kernel_name(29) << "): "
             << ((o.check || o.cpu_check) ? (res ? "PASSED" : "FAILED") : "COMPLETED (no verification)") << endl;
        if (o.json) {
            printf("{\"kernel\": 29, \"gpus\": %d, \"M\": %d, \"N\": %d, \"K\": %d, \"runs\": %d, \"avg_ms\": %.6f, "
                   "\"dense_equiv_tflops\": %.3f, \"gather_ms\": %.6f, \"passed\": %s, \"cpu_rel_inf\": %g, \"ms_per_gpu\": [",
                   o.gpus, M, N, K, o.runs, ms_max, 2.0 * M * N * K / (ms_max * 1e-3) / 1e12, ms_gather, res ? "true" : "false",
                   cpu_rel);
            for (int g = 0; g < o.gpus; ++g) printf("%s%.6f", g ? ", " : "", ms_gpu[g]);
            printf("]}\n");
        }
        o.kernels.assign(1, 29);
    }
    for (int id : o.kernels) {
        if (o.gpus > 0) break;
        cudaCheckError(cudaMemset(d_C, 0, nC * sizeof(float)));
        if (o.verbose) cout << "Running kernel " << id << ": " << get_kernel_name(id) << (o.check ? "" : " (Performance-only mode)") << endl;
        int ok_flag = 0;
        float avg_ms = 0.f;
        const bool need_c = o.check || o.cpu_check;
        int st = esmm_run_kernel_pattern(id, M, N, K, d_A, d_B, d_C, need_c ? h_C : nullptr, o.check ? h_C_ref : nullptr,
                                         o.runs, o.check && id != 15 ? 1 : 0, o.skip_stats ? 1 : 0, d_b_cached,
                                         o.pattern.c_str(), &ok_flag, &avg_ms);
        bool res = (st == ESMM_OK) && ok_flag;
        if (st == ESMM_ERR_UNSUPPORTED) cout << "Kernel " << id << " is not provided by this library" << endl;
        double cpu_rel = -1.0;
        if (o.cpu_check && st == ESMM_OK) {
            if (!o.check) cudaCheckError(cudaMemcpy(h_C, d_C, nC * sizeof(float), cudaMemcpyDeviceToHost));
            double num = 0.0, den = 0.0;
            for (size_t i = 0; i < nC; ++i) {
                num = std::max(num, (double)std::fabs(h_C[i] - h_cpu[i]));
                den = std::max(den, (double)std::fabs(h_cpu[i]));
            }
            cpu_rel = den > 0 ? num / den : num;
            cout << "CPU SGEMM check: rel-inf error " << cpu_rel << (cpu_rel <= 1e-4 ? " (ok)" : " (FAILED)") << endl;
            if (cpu_rel > 1e-4) res = false;
        }
        if (res || (!o.check && !o.cpu_check && st == ESMM_OK)) ++passed;
        if (o.verbose) {
            cout << "  Status: " << (o.check ? (res ? "PASSED" : "FAILED") : "COMPLETED (no verification)") << endl;
            if (id != o.kernels.back()) cout << endl;
        } else {
            cout << "Kernel " << id << " (" << get_kernel_name(id) << "): "
                 << (o.check ? (res ? "PASSED" : "FAILED") : (st == ESMM_OK ? "COMPLETED (no verification)" : "FAILED")) << endl;
        }
        if (o.json)
            printf("{\"kernel\": %d, \"M\": %d, \"N\": %d, \"K\": %d, \"runs\": %d, \"avg_ms\": %.6f, \"dense_equiv_tflops\": %.3f, "
                   "\"status\": %d, \"passed\": %s, \"cpu_rel_inf\": %g}\n",
                   id, M, N, K, o.runs, avg_ms, avg_ms > 0 ? 2.0 * M * N * K / (avg_ms * 1e-3) / 1e12 : 0.0, st,
                   res ? "true" : "false", cpu_rel);
    }

    const int total = (int)o.kernels.size();
    cout << endl << "Summary: " << passed << "/" << total << " kernels " << (o.check ? "passed" : "completed (no verification)") << endl;
    free(h_A);
    free(h_B);
    free(h_C);
    free(h_C_ref);
    cudaFree(d_A);
    cudaFree(d_B);
    cudaFree(d_C);
    if (d_b_cached) cudaFree(d_b_cached);
    return passed == total ? 0 : 1;
}
