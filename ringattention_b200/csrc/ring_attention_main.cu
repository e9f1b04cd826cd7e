// Driver executable: the reference's main() (csrc/ring_attention.cu:750-790) over this library.
//
// Same experiment: dim 64, 8192 rows per rank, deterministic fill h[i][j] = i/130 + j/110 + i*j/600 for Q, K and V
// (fillWithNum, :731-741), 50 warm-up calls and 50 timed calls of ring_attention(...) between two CUDA events
// (:767-783), then "mype: N success" per rank, the top-left 8x8 of rank 0's output and the time per call (:784-789).
// Differences: one process per GPU is started by any launcher that sets RING_RANK / RING_WORLD (default 0 / 1;
// the reference uses nvshmrun -n 2, makefile:2), the NCCL id travels through the file named by RING_ID_FILE,
// and K / V are plain cudaMalloc memory (the reference needs nvshmem_malloc, :760-761).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/attention_api.cuh"

using FPC = __half;  // the reference's element type alias (csrc/ring_attention.cu:18)

static void printDeviceFloat(const float* out, int m, int n) {  // csrc/ring_attention.cu:723-729
    (void)m;
    std::vector<float> h(8 * static_cast<size_t>(n));
    CUDA_ERROR_CHECK(cudaMemcpy(h.data(), out, h.size() * sizeof(float), cudaMemcpyDeviceToHost));
    for (int i = 0; i < 8; ++i) {
        for (int j = 0; j < 8; ++j) std::printf("%10.4f ", h[static_cast<size_t>(i) * n + j]);
        std::printf("\n");
    }
}

static void fillWithNum(FPC* mat, int m, int n) {  // csrc/ring_attention.cu:731-741
    std::vector<FPC> h(static_cast<size_t>(m) * n);
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j)
            h[static_cast<size_t>(i) * n + j] = __float2half(static_cast<float>(i / 130.0 + j / 110.0 + i * j / 600.0));
    CUDA_ERROR_CHECK(cudaMemcpy(mat, h.data(), h.size() * sizeof(FPC), cudaMemcpyHostToDevice));
}

static void initQKV(FPC* q, FPC* k, FPC* v, int m, int n) {  // csrc/ring_attention.cu:743-748
    fillWithNum(q, m, n);
    fillWithNum(k, m, n);
    fillWithNum(v, m, n);
    CUDA_ERROR_CHECK(cudaDeviceSynchronize());
}

static int env_int(const char* name, int fallback) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : fallback;
}

static bool share_id(unsigned char* id, int mype) {
    const char* path = std::getenv("RING_ID_FILE");
    if (!path) return false;
    if (mype == 0) {
        std::string tmp = std::string(path) + ".tmp";
        FILE* f = std::fopen(tmp.c_str(), "wb");
        if (!f) return false;
        std::fwrite(id, 1, RING_UNIQUE_ID_BYTES, f);
        std::fclose(f);
        return std::rename(tmp.c_str(), path) == 0;
    }
    for (int tries = 0; tries < 600; ++tries) {  // up to a minute
        FILE* f = std::fopen(path, "rb");
        if (f) {
            const size_t n = std::fread(id, 1, RING_UNIQUE_ID_BYTES, f);
            std::fclose(f);
            if (n == RING_UNIQUE_ID_BYTES) return true;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    return false;
}

int main() {
    const int dim = env_int("RING_DIM", 64);
    const int max_seq = env_int("RING_SEQ", 8192);
    const int mype = env_int("RING_RANK", 0);
    const int npes = env_int("RING_WORLD", 1);
    const int warmup = env_int("RING_WARMUP", 50), test_loop = env_int("RING_LOOPS", 50);
    std::vector<int> seqlen(npes, max_seq);
    CUDA_ERROR_CHECK(cudaSetDevice(env_int("RING_DEVICE", mype)));

    RingCtx* ctx = nullptr;
    unsigned char id[RING_UNIQUE_ID_BYTES] = {0};
    if (npes > 1) {
        if (mype == 0 && ring_get_unique_id(id) != RING_OK) { std::printf("%s\n", ring_last_error_string()); return 1; }
        if (!share_id(id, mype)) { std::printf("could not share the communicator id (set RING_ID_FILE)\n"); return 1; }
    }
    if (ring_ctx_create(&ctx, mype, npes, npes > 1 ? id : nullptr) != RING_OK) { std::printf("%s\n", ring_last_error_string()); return 1; }
    ring_set_default_ctx(ctx);

    FPC *q, *k, *v;
    float* out;
    const size_t elems = static_cast<size_t>(seqlen[mype]) * dim;
    CUDA_ERROR_CHECK(cudaMalloc(&q, elems * sizeof(FPC)));
    CUDA_ERROR_CHECK(cudaMalloc(&k, elems * sizeof(FPC)));
    CUDA_ERROR_CHECK(cudaMalloc(&v, elems * sizeof(FPC)));
    CUDA_ERROR_CHECK(cudaMalloc(&out, elems * sizeof(float)));
    initQKV(q, k, v, seqlen[mype], dim);

    for (int i = 0; i < warmup; ++i)
        if (ring_attention(q, k, v, out, npes, mype, seqlen.data(), dim, max_seq) != RING_OK) {
            std::printf("ring_attention failed: %s\n", ring_last_error_string());
            return 1;
        }
    cudaEvent_t start, stop;
    float elapsedTime = 0.f;
    cudaEventCreate(&start);
    cudaEventCreate(&stop);
    cudaEventRecord(start, 0);
    for (int i = 0; i < test_loop; ++i) ring_attention(q, k, v, out, npes, mype, seqlen.data(), dim, max_seq);
    cudaEventRecord(stop, 0);
    cudaEventSynchronize(stop);
    cudaEventElapsedTime(&elapsedTime, start, stop);
    std::printf("mype: %d success\n", mype);
    if (!mype) printDeviceFloat(out, seqlen[mype], dim);
    if (!mype) std::printf("elapsedtime=%f\n", elapsedTime / test_loop);
    ring_ctx_destroy(ctx);
    return 0;
}
