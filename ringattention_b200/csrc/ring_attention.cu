// Host side of the B200 ring-attention forward: launchers, the ring driver loop, the K/V exchange
// and the C ABI.
//
// Keeps the reference's three host entry points by name and role:
//   set_params_fprop  (csrc/ring_attention.cu:361-395)  fill Ring_fwd_params
//   run_ring_fwd<Kernel_traits>  (csrc/ring_attention.cu:669-704)  derive grid / shared memory and launch
//   ring_attention  (csrc/ring_attention.cu:706-722)  the call users make
// with these differences: nothing is allocated per call (the reference allocates d_seqlen, k_buffer and
// v_buffer on every call and never frees them, :384,391,393); run_ring_fwd is the ring loop itself
// (one block-kernel launch per ring step instead of one kernel looping over PEs, :456) and honours its
// stream argument (the reference launches on stream 0, :700); the exchange runs on a side stream into two
// alternating receive buffers instead of an in-kernel NVSHMEM get into a single buffer (:611-619), either as
// copy-engine pushes into the peers' IPC-shared buffers (the default when the ranks can map each other's
// memory) or as NCCL send/recv; errors are returned, not printed-and-exit (csrc/utils.h:1-11).
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cuda.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include "../../include/ring_attention_b200.h"
#include "block_attention.cuh"
#include "block_attention_pair.cuh"
#include "kernel_traits.h"
#include "lse_merge.cuh"
#include "ring.h"

namespace {

// ------------------------------------------------------------------------------------------ errors
thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define RING_CUDA(call)                                                                              \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ != cudaSuccess)                                                                       \
            return fail(RING_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, \
                        __LINE__);                                                                   \
    } while (0)

std::atomic<int64_t> g_launches{0};
#ifdef RING_TRACE
long long* g_trace = nullptr;  // debug builds only: device buffer for clock stamps of one CTA
#endif

// ------------------------------------------------------------------------------------------ NCCL (loaded lazily)
// The library is usable on one GPU without NCCL being present; multi-rank contexts load it on demand.
// Inside a process that already loaded a libnccl.so.2 (for example through torch) the same copy is used.
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    bool ok = false;
};

NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) return;
#define LOAD(field, sym)                                                     \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, sym)); \
    if (!api.field) return;
        LOAD(GetUniqueId, "ncclGetUniqueId");
        LOAD(CommInitRank, "ncclCommInitRank");
        LOAD(CommInitRankConfig, "ncclCommInitRankConfig");
        LOAD(CommDestroy, "ncclCommDestroy");
        LOAD(CommAbort, "ncclCommAbort");
        LOAD(Send, "ncclSend");
        LOAD(Recv, "ncclRecv");
        LOAD(AllGather, "ncclAllGather");
        LOAD(GroupStart, "ncclGroupStart");
        LOAD(GroupEnd, "ncclGroupEnd");
        LOAD(GetErrorString, "ncclGetErrorString");
        LOAD(CommGetAsyncError, "ncclCommGetAsyncError");
#undef LOAD
        api.ok = true;
    });
    return api;
}

#define RING_NCCL(call)                                                                                \
    do {                                                                                               \
        ncclResult_t r_ = (call);                                                                      \
        if (r_ != ncclSuccess)                                                                         \
            return fail(RING_ERR_NCCL, "%s failed: %s (%s:%d)", #call, nccl().GetErrorString(r_), __FILE__, \
                        __LINE__);                                                                     \
    } while (0)

// ------------------------------------------------------------------------------------------ per-device state
struct DeviceState {
    int* d_status = nullptr;  // device status word written by kernels whose bounded waits ran out
    int sm_count = 0;
    bool attr_set[12] = {};  // [one-CTA | pair | pair with two threads per row][dim == 128][bf16]: shared-memory attribute set
};

std::mutex g_dev_mutex;
DeviceState g_dev[64];

int device_state(DeviceState** out) {
    int dev = 0;
    RING_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(RING_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState& st = g_dev[dev];
    if (!st.d_status) {
        RING_CUDA(cudaMalloc(&st.d_status, sizeof(int)));
        RING_CUDA(cudaMemset(st.d_status, 0, sizeof(int)));
        RING_CUDA(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
    }
    *out = &st;
    return RING_OK;
}

// ------------------------------------------------------------------------------------------ tensor maps
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_fn(EncodeTiledFn* out) {
    static EncodeTiledFn fn = nullptr;
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        RING_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !p)
            return fail(RING_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    *out = fn;
    return RING_OK;
}

// [batch, heads, rows, dim] 16-bit tensor -> 4-D map, box = 64 x 128 x 1 x 1 elements, 128-byte swizzle.
// Out-of-range rows read as zero, which gives tail predication for free (the reference has none and
// needs seqlen % 64 == 0, csrc/ring_attention.cu:131,143-145).
int make_tensor_map(CUtensorMap* tm, const void* base, int batch, int heads, int rows, int dim, bool bf16,
                    int64_t rows_total = 0, int box_rows = 128) {
    if (rows_total <= 0) rows_total = rows;  // rows_total > rows: `base` points at a row range inside longer (b, h) slabs
    EncodeTiledFn enc = nullptr;
    int rc = encode_fn(&enc);
    if (rc) return rc;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(dim), static_cast<cuuint64_t>(rows),
                                static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(dim) * 2, static_cast<cuuint64_t>(rows_total) * dim * 2,
                                   static_cast<cuuint64_t>(heads) * rows_total * dim * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RING_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return RING_OK;
}

// ------------------------------------------------------------------------------------------ stream memory operations
// cuStreamWriteValue32 / cuStreamWaitValue32: a 32-bit store / a ">= value" wait executed by the stream's
// front end, in stream order, without a kernel.  The peer-copy exchange uses them as cross-process flags.
using StreamValueFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
struct StreamMemOps {
    StreamValueFn write = nullptr;
    StreamValueFn wait = nullptr;
};

int stream_mem_ops(StreamMemOps* out) {
    static StreamMemOps ops;
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
    if (!ops.write) {
        void *pw = nullptr, *pq = nullptr;
        cudaDriverEntryPointQueryResult q1, q2;
        RING_CUDA(cudaGetDriverEntryPoint("cuStreamWriteValue32", &pw, cudaEnableDefault, &q1));
        RING_CUDA(cudaGetDriverEntryPoint("cuStreamWaitValue32", &pq, cudaEnableDefault, &q2));
        if (q1 != cudaDriverEntryPointSuccess || q2 != cudaDriverEntryPointSuccess || !pw || !pq)
            return fail(RING_ERR_UNSUPPORTED, "stream memory operations are not available from this driver");
        ops.write = reinterpret_cast<StreamValueFn>(pw);
        ops.wait = reinterpret_cast<StreamValueFn>(pq);
    }
    *out = ops;
    return RING_OK;
}

#define RING_CU(call)                                                                                     \
    do {                                                                                                  \
        CUresult r_ = (call);                                                                             \
        if (r_ != CUDA_SUCCESS)                                                                           \
            return fail(RING_ERR_CUDA, "%s failed with CUresult %d (%s:%d)", #call, (int)r_, __FILE__, __LINE__); \
    } while (0)

// ------------------------------------------------------------------------------------------ launchers
struct BlockLaunch {
    const void *q, *k, *v;
    float* o;
    float* lse;
    int batch, heads, sq, sk, dim;
    float scale;
    int causal;
    int64_t q_off, k_off;
    int merge;
    int is_bf16;
    // > 0: q/o/lse (k/v) point at a row range inside (batch, head) slabs of this many rows
    int64_t q_rows_total = 0, k_rows_total = 0;
};

// What a launch needs from the device it runs on.  The ordinary entry points take it from DeviceState (whose
// status word is allocated once per device); the no-allocation entry point passes the header of its fixed array.
struct LaunchEnv {
    int* status;            // device status word the kernel reports a run-out wait in
    bool* attr_set;         // [pair form][dim == 128][bf16]: dynamic shared-memory attribute already set on this device
    int sm_count;
};

ring::BlockFwdArgs block_args(const BlockLaunch& L, const LaunchEnv& env) {
    const int64_t q_slab = L.q_rows_total > 0 ? L.q_rows_total : L.sq;
    ring::BlockFwdArgs a;
    a.o = L.o;
    a.lse = L.lse;
    a.o_row_stride = L.dim;
    a.o_head_stride = q_slab * L.dim;
    a.o_batch_stride = a.o_head_stride * L.heads;
    a.lse_head_stride = q_slab;
    a.lse_batch_stride = q_slab * L.heads;
    a.heads = L.heads;
    a.sq = L.sq;
    a.sk = L.sk;
    a.scale = L.scale;
    a.scale_log2 = L.scale * 1.4426950408889634f;
    a.causal = L.causal ? 1 : 0;
    int64_t diag = L.q_off - L.k_off;
    const int64_t lim = int64_t(1) << 30;
    diag = diag > lim ? lim : (diag < -lim ? -lim : diag);
    a.diag = static_cast<int>(diag);
    a.merge = L.merge ? 1 : 0;
    a.status = env.status;
    a.rows_per_cta = 0;
#ifdef RING_TRACE
    a.trace = g_trace;
#endif
    return a;
}

// The CTA-pair form (head dimension 128): clusters of two CTAs, 128 Q rows each; K is fetched in boxes of 64 keys.
template <class Traits>
int launch_block_pair_instance(const BlockLaunch& L, const LaunchEnv& env, cudaStream_t stream) {
    auto kernel = &ring::ring_block_attention_pair_kernel<Traits>;
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        bool& attr = env.attr_set[4 * Traits::kHalves + (Traits::kHeadDim == 128) * 2 + Traits::kIsBf16];
        if (!attr) {
            RING_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Traits::kSmemSize));
            attr = true;
        }
    }
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tensor_map(&tq, L.q, L.batch, L.heads, L.sq, L.dim, L.is_bf16, L.q_rows_total))) return rc;
    if ((rc = make_tensor_map(&tk, L.k, L.batch, L.heads, L.sk, L.dim, L.is_bf16, L.k_rows_total, 64))) return rc;
    if ((rc = make_tensor_map(&tv, L.v, L.batch, L.heads, L.sk, L.dim, L.is_bf16, L.k_rows_total))) return rc;
    ring::BlockFwdArgs a = block_args(L, env);
    a.rows_per_cta = Traits::kBlockM;
    dim3 grid(2 * ((L.sq + 255) / 256), L.batch * L.heads);  // whole pairs: a CTA whose rows lie past the end still loads its K/V halves
    kernel<<<grid, dim3(Traits::kNThreads), Traits::kSmemSize, stream>>>(tq, tk, tv, a);
    RING_CUDA(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return RING_OK;
}

template <class Traits>
int launch_block_instance(const BlockLaunch& L, const LaunchEnv& env, cudaStream_t stream) {
    auto kernel = &ring::ring_block_attention_kernel<Traits>;
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        bool& attr = env.attr_set[(Traits::kHeadDim == 128) * 2 + Traits::kIsBf16];
        if (!attr) {
            RING_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Traits::kSmemSize));
            attr = true;
        }
    }
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tensor_map(&tq, L.q, L.batch, L.heads, L.sq, L.dim, L.is_bf16, L.q_rows_total))) return rc;
    if ((rc = make_tensor_map(&tk, L.k, L.batch, L.heads, L.sk, L.dim, L.is_bf16, L.k_rows_total))) return rc;
    if ((rc = make_tensor_map(&tv, L.v, L.batch, L.heads, L.sk, L.dim, L.is_bf16, L.k_rows_total))) return rc;
    ring::BlockFwdArgs a = block_args(L, env);

    // Two Q tiles per CTA keep the tensor pipe busiest, but a grid that covers at most half of the SMs that way
    // (one head of a short shard, as in the reference's own driver) finishes sooner with one tile per CTA.
    // (RING_ROWS_PER_CTA = 128 or 256 in the environment overrides the choice; the tests use it to run both forms.)
    a.rows_per_cta = Traits::kBlockM;
    if (L.sq > 128 && ((L.sq + Traits::kBlockM - 1) / Traits::kBlockM) * L.batch * L.heads * 2 <= env.sm_count) a.rows_per_cta = 128;
    if (const char* e = std::getenv("RING_ROWS_PER_CTA")) {
        const int forced = std::atoi(e);
        if (forced == 128 || forced == Traits::kBlockM) a.rows_per_cta = forced;
    }
    dim3 grid((L.sq + a.rows_per_cta - 1) / a.rows_per_cta, L.batch * L.heads);
    dim3 block(Traits::kNThreads);
    kernel<<<grid, block, Traits::kSmemSize, stream>>>(tq, tk, tv, a);
    RING_CUDA(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return RING_OK;
}

int validate_block(const BlockLaunch& L) {
    if (!L.q || !L.k || !L.v || !L.o || !L.lse) return fail(RING_ERR_INVALID_ARGUMENT, "null tensor pointer");
    if (L.dim != 64 && L.dim != 128) return fail(RING_ERR_INVALID_ARGUMENT, "dim must be 64 or 128, got %d", L.dim);
    if (L.batch <= 0 || L.heads <= 0 || L.sq <= 0 || L.sk <= 0)
        return fail(RING_ERR_INVALID_ARGUMENT, "batch, heads and sequence lengths must be positive");
    // Any length is accepted: rows past the end of a shard are read as zero by the tensor maps, masked in the
    // softmax (keys) or simply not stored (queries).  The reference needs multiples of its 64-row tile
    // (no predication, csrc/ring_attention.cu:131,143-145).
    if (L.sq > (1 << 24) || L.sk > (1 << 24))
        return fail(RING_ERR_INVALID_ARGUMENT, "sequence lengths above 2^24 rows per shard are not supported");
    if (static_cast<int64_t>(L.batch) * L.heads > 65535)
        return fail(RING_ERR_INVALID_ARGUMENT, "batch * heads must not exceed 65535");
    if (!(L.scale > 0.f) || !std::isfinite(L.scale))
        return fail(RING_ERR_INVALID_ARGUMENT, "softmax_scale must be positive and finite");
    const uintptr_t al = reinterpret_cast<uintptr_t>(L.q) | reinterpret_cast<uintptr_t>(L.k) |
                         reinterpret_cast<uintptr_t>(L.v) | reinterpret_cast<uintptr_t>(L.o);
    if (al & 15) return fail(RING_ERR_INVALID_ARGUMENT, "tensor base pointers must be 16-byte aligned");
    return RING_OK;
}

// Shape dispatch: the reference instantiates Ring_fwd_traits<64, 64, 64, 4, half> only
// (csrc/ring_attention.cu:707-716); here <64|128, 256, 128, 12, half|bf16>.
// RING_PAIR=1 or 2 in the environment: head dimension 128 runs the CTA-pair form (clusters of two CTAs, cta_group::2
// MMAs, two S buffers) with one or two softmax threads per Q row.  Default 0: the one-CTA form.  Read at every launch
// so that tests can switch it.
int pair_form() {
    const char* e = std::getenv("RING_PAIR");
    const int v = e ? std::atoi(e) : 0;
    return (v == 1 || v == 2) ? v : 0;
}

int launch_block_env(const BlockLaunch& L, const LaunchEnv& env, cudaStream_t stream) {
    const int pair = L.dim == 128 ? pair_form() : 0;
    if (pair == 2) {
        if (L.is_bf16) return launch_block_pair_instance<Ring_pair_traits<128, __nv_bfloat16, 2>>(L, env, stream);
        return launch_block_pair_instance<Ring_pair_traits<128, __half, 2>>(L, env, stream);
    }
    if (pair == 1) {
        if (L.is_bf16) return launch_block_pair_instance<Ring_pair_traits<128, __nv_bfloat16, 1>>(L, env, stream);
        return launch_block_pair_instance<Ring_pair_traits<128, __half, 1>>(L, env, stream);
    }
    if (L.dim == 128) {
        if (L.is_bf16) return launch_block_instance<Ring_fwd_traits<128, 256, 128, 12, __nv_bfloat16>>(L, env, stream);
        return launch_block_instance<Ring_fwd_traits<128, 256, 128, 12, __half>>(L, env, stream);
    }
    if (L.is_bf16) return launch_block_instance<Ring_fwd_traits<64, 256, 128, 12, __nv_bfloat16>>(L, env, stream);
    return launch_block_instance<Ring_fwd_traits<64, 256, 128, 12, __half>>(L, env, stream);
}

int launch_block(const BlockLaunch& L, cudaStream_t stream) {
    int rc = validate_block(L);
    if (rc) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(&st))) return rc;
    return launch_block_env(L, LaunchEnv{st->d_status, st->attr_set, st->sm_count}, stream);
}

int launch_merge(float* o_acc, float* lse_acc, const float* o_part, const float* lse_part, int64_t rows, int dim,
                 cudaStream_t stream, int sms = 0) {
    if (!o_acc || !lse_acc || !o_part || !lse_part) return fail(RING_ERR_INVALID_ARGUMENT, "null tensor pointer");
    if (dim != 64 && dim != 128) return fail(RING_ERR_INVALID_ARGUMENT, "dim must be 64 or 128, got %d", dim);
    if (rows < 0) return fail(RING_ERR_INVALID_ARGUMENT, "negative row count");
    if (rows == 0) return RING_OK;
    if (sms <= 0) {
        int dev = 0;
        RING_CUDA(cudaGetDevice(&dev));
        RING_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    const int threads = 256;
    const int64_t want = (rows + 7) / 8;              // 8 warps (rows) per block
    const int64_t cap = static_cast<int64_t>(sms) * 8;  // 8 resident blocks per SM, grid-stride beyond that
    const int blocks = static_cast<int>(want < cap ? want : cap);
    if (dim == 128)
        ring::ring_lse_merge_kernel<128><<<blocks, threads, 0, stream>>>(o_acc, lse_acc, o_part, lse_part, rows);
    else
        ring::ring_lse_merge_kernel<64><<<blocks, threads, 0, stream>>>(o_acc, lse_acc, o_part, lse_part, rows);
    RING_CUDA(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return RING_OK;
}

int read_status(int* out) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    RING_CUDA(cudaDeviceSynchronize());
    RING_CUDA(cudaMemcpy(out, st->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    return RING_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------ context
constexpr int kMaxWorld = 64;

struct RingCtx {
    int rank = 0;
    int world = 1;
    int device = 0;
    bool local = false;  // virtual ranks on one GPU, exchange by device-to-device copy
    ncclComm_t comm = nullptr;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_fork = nullptr;
    cudaEvent_t ev_recv_done[kMaxWorld] = {};
    cudaEvent_t ev_comm_start[kMaxWorld] = {};
    cudaEvent_t ev_copy_start[kMaxWorld] = {};  // after the exchange's wait for its go-ahead (credit flag / previous compute)
    cudaEvent_t ev_compute_start[kMaxWorld] = {};
    cudaEvent_t ev_compute_done[kMaxWorld] = {};
    // receive buffers: recv[i] holds K then V of one shard; two of them (double buffer) unless RING_OPT_RECV_BUFFERS
    // asks for one per remote shard
    void* recv[kMaxWorld] = {};
    size_t recv_cap[kMaxWorld] = {};  // bytes
    int recv_buffers = 2;             // 0: one per remote shard (world - 1)
    // partial result of one step (separate-kernel merge mode) and an LSE buffer for callers that pass none
    float* o_part = nullptr;
    float* lse_part = nullptr;
    float* lse_own = nullptr;
    size_t o_part_cap = 0, lse_part_cap = 0, lse_own_cap = 0;  // bytes
    int merge_mode = RING_MERGE_FUSED_EPILOGUE;
    int causal_skip = 1;
    int zigzag = 0;  // causal sharding: 0 contiguous, 1 zig-zag (rank r holds half-chunks r and 2P-1-r)
    int record_timings = 0;
    int last_steps = 0;
    bool step_computed[kMaxWorld] = {};
    bool step_exchanged[kMaxWorld] = {};
    const void* local_k[kMaxWorld] = {};
    const void* local_v[kMaxWorld] = {};
    // ---- peer-copy transport (RING_TRANSPORT_PEER_COPY) ---------------------------------------------------
    int transport = RING_TRANSPORT_NCCL;
    bool peer_ready = false;          // flags exported/imported
    uint32_t* flags = nullptr;        // own flag block: ready[kMaxWorld] then credit[kMaxWorld]
    uint32_t* peer_flags[kMaxWorld] = {};
    void* recv_block = nullptr;       // one allocation holding both receive buffers (peer transport)
    size_t recv_block_half = 0;       // bytes of one receive buffer inside the block
    int recv_block_count = 0;         // receive buffers inside the block
    void* peer_recv_block[kMaxWorld] = {};
    size_t peer_recv_half[kMaxWorld] = {};
    void* xchg_dev = nullptr;         // staging for the handle all-gathers
    uint32_t call_seq = 0;
    cudaEvent_t ev_push_done = nullptr;
    cudaEvent_t ev_call_done = nullptr;  // end of the previous call on whatever stream it used
    bool have_call_done = false;
    // ---- host-buffer forward (ring_attention_fwd_host): two staging sets, copy streams, per-chunk events
    void* stage_in[2] = {nullptr, nullptr};   // [q | k | v] of one chunk
    void* stage_out[2] = {nullptr, nullptr};  // [out | lse] of one chunk
    size_t stage_in_cap[2] = {0, 0}, stage_out_cap[2] = {0, 0};
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
    cudaEvent_t ev_h2d[kMaxWorld] = {}, ev_comp[kMaxWorld] = {}, ev_d2h[kMaxWorld] = {};
    bool host_ready = false;
    bool dead = false;  // ring_ctx_abort() was called: forwards are refused, destroy does not wait for the device
};

constexpr int kFlagReady = 0;
constexpr int kFlagCredit = kMaxWorld;
constexpr size_t kXchgBlob = 128;  // bytes exchanged per rank in a handle all-gather

namespace {

RingCtx* g_default_ctx = nullptr;
RingCtx* g_solo_ctx = nullptr;  // world-1 context created on demand by ring_attention()

int ctx_common_init(RingCtx* c) {
    RING_CUDA(cudaGetDevice(&c->device));
    // The exchange stream gets the highest priority: its few CTAs (NCCL's send/recv kernel) must win an SM
    // as soon as one frees up, instead of queueing behind the block kernel's thousand pending CTAs.
    int prio_least = 0, prio_greatest = 0;
    RING_CUDA(cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest));
    RING_CUDA(cudaStreamCreateWithPriority(&c->comm_stream, cudaStreamNonBlocking, prio_greatest));
    RING_CUDA(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
    RING_CUDA(cudaEventCreateWithFlags(&c->ev_call_done, cudaEventDisableTiming));
    for (int i = 0; i < c->world; ++i) {
        RING_CUDA(cudaEventCreate(&c->ev_recv_done[i]));
        RING_CUDA(cudaEventCreate(&c->ev_comm_start[i]));
        RING_CUDA(cudaEventCreate(&c->ev_copy_start[i]));
        RING_CUDA(cudaEventCreate(&c->ev_compute_start[i]));
        RING_CUDA(cudaEventCreate(&c->ev_compute_done[i]));
    }
    DeviceState* st = nullptr;
    return device_state(&st);
}

int grow(void** buf, size_t* cap, size_t need) {
    if (need <= *cap) return RING_OK;
    // Growing is rare (first call, or a larger shape than any before) and synchronises the device.
    RING_CUDA(cudaDeviceSynchronize());
    if (*buf) RING_CUDA(cudaFree(*buf));
    *buf = nullptr;
    *cap = 0;
    RING_CUDA(cudaMalloc(buf, need));
    *cap = need;
    return RING_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------ peer-copy transport
// The K/V exchange without SMs: every rank PUSHES its own K/V shard into the destination's receive
// buffer with a device-to-device copy over NVLink (copy engines), on its exchange stream.  The receive
// buffers and a small flag block of every rank are shared with the other processes through CUDA IPC.
// Cross-process ordering uses stream memory operations on the flag blocks (no kernels, no spinning SMs):
//   ready[e]  (in the RECEIVER's block)  written by the origin rank of exchange e after its copy:
//             "the shard for your step e + 1 has landed";
//   credit[e] (in the SENDER's block)    written by the destination of exchange e:
//             "my receive buffer e & 1 is free for you" -- at the start of a call for e < 2, after
//             compute step e - 1 for e >= 2 (that step was the last reader of the buffer).
// Values are the call sequence number, compared with >=, so flags are never reset.
namespace {

int allgather_blobs(RingCtx* c, const void* mine, std::vector<char>& all) {
    NcclApi& n = nccl();
    all.assign(kXchgBlob * c->world, 0);
    char* dev = static_cast<char*>(c->xchg_dev);
    RING_CUDA(cudaMemcpyAsync(dev + kXchgBlob * (c->world + c->rank), mine, kXchgBlob, cudaMemcpyHostToDevice, c->comm_stream));
    RING_NCCL(n.AllGather(dev + kXchgBlob * (c->world + c->rank), dev, kXchgBlob, ncclInt8, c->comm, c->comm_stream));
    RING_CUDA(cudaMemcpyAsync(all.data(), dev, kXchgBlob * c->world, cudaMemcpyDeviceToHost, c->comm_stream));
    RING_CUDA(cudaStreamSynchronize(c->comm_stream));
    return RING_OK;
}

struct HandleBlob {
    cudaIpcMemHandle_t handle;
    uint64_t half_bytes;
    uint64_t valid;
};
static_assert(sizeof(HandleBlob) <= kXchgBlob, "blob size");

int peer_setup_flags(RingCtx* c) {
    StreamMemOps ops;
    int rc = stream_mem_ops(&ops);
    if (rc) return rc;
    RING_CUDA(cudaMalloc(&c->xchg_dev, kXchgBlob * 2 * kMaxWorld));
    RING_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->flags), 2 * kMaxWorld * sizeof(uint32_t)));
    RING_CUDA(cudaMemset(c->flags, 0, 2 * kMaxWorld * sizeof(uint32_t)));
    RING_CUDA(cudaEventCreateWithFlags(&c->ev_push_done, cudaEventDisableTiming));
    HandleBlob mine;
    std::memset(&mine, 0, sizeof(mine));
    cudaError_t e = cudaIpcGetMemHandle(&mine.handle, c->flags);
    mine.valid = (e == cudaSuccess) ? 1 : 0;
    if (e != cudaSuccess) (void)cudaGetLastError();
    char blob[kXchgBlob] = {0};
    std::memcpy(blob, &mine, sizeof(mine));
    std::vector<char> all;
    if ((rc = allgather_blobs(c, blob, all))) return rc;
    bool ok = true;
    for (int r = 0; r < c->world && ok; ++r) {
        HandleBlob hb;
        std::memcpy(&hb, all.data() + kXchgBlob * r, sizeof(hb));
        if (!hb.valid) { ok = false; break; }
        if (r == c->rank) { c->peer_flags[r] = c->flags; continue; }
        void* p = nullptr;
        e = cudaIpcOpenMemHandle(&p, hb.handle, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { (void)cudaGetLastError(); ok = false; break; }
        c->peer_flags[r] = static_cast<uint32_t*>(p);
    }
    // every rank must take the same decision: agree through one more all-gather
    char vote[kXchgBlob] = {0};
    vote[0] = ok ? 1 : 0;
    if ((rc = allgather_blobs(c, vote, all))) return rc;
    for (int r = 0; r < c->world; ++r)
        if (!all[kXchgBlob * r]) ok = false;
    c->peer_ready = ok;
    return RING_OK;
}

// Collective: every rank of the context calls it in the same ring_attention_fwd() with the same size.
int peer_grow_recv(RingCtx* c, size_t half_bytes, int nbuf) {
    if (half_bytes <= c->recv_block_half && nbuf <= c->recv_block_count) return RING_OK;
    if (half_bytes < c->recv_block_half) half_bytes = c->recv_block_half;
    int rc;
    std::vector<char> all;
    char blob[kXchgBlob] = {0};
    RING_CUDA(cudaDeviceSynchronize());
    if (!c->recv_block) {  // buffers an earlier NCCL-transport forward obtained with grow(): not shared, release them
        for (int i = 0; i < kMaxWorld; ++i) {
            if (c->recv[i]) RING_CUDA(cudaFree(c->recv[i]));
            c->recv[i] = nullptr;
            c->recv_cap[i] = 0;
        }
    }
    for (int r = 0; r < c->world; ++r) {  // drop the mappings of the buffers that are about to be freed
        if (r != c->rank && c->peer_recv_block[r]) RING_CUDA(cudaIpcCloseMemHandle(c->peer_recv_block[r]));
        c->peer_recv_block[r] = nullptr;
    }
    if ((rc = allgather_blobs(c, blob, all))) return rc;  // barrier: nobody still maps the old buffers
    if (c->recv_block) RING_CUDA(cudaFree(c->recv_block));
    c->recv_block = nullptr;
    c->recv_block_half = 0;
    c->recv_block_count = 0;
    RING_CUDA(cudaMalloc(&c->recv_block, static_cast<size_t>(nbuf) * half_bytes));
    c->recv_block_half = half_bytes;
    c->recv_block_count = nbuf;
    HandleBlob mine;
    std::memset(&mine, 0, sizeof(mine));
    RING_CUDA(cudaIpcGetMemHandle(&mine.handle, c->recv_block));
    mine.half_bytes = half_bytes;
    mine.valid = 1;
    std::memcpy(blob, &mine, sizeof(mine));
    if ((rc = allgather_blobs(c, blob, all))) return rc;
    for (int r = 0; r < c->world; ++r) {
        HandleBlob hb;
        std::memcpy(&hb, all.data() + kXchgBlob * r, sizeof(hb));
        c->peer_recv_half[r] = hb.half_bytes;
        if (r == c->rank) { c->peer_recv_block[r] = c->recv_block; continue; }
        RING_CUDA(cudaIpcOpenMemHandle(&c->peer_recv_block[r], hb.handle, cudaIpcMemLazyEnablePeerAccess));
    }
    for (int i = 0; i < kMaxWorld; ++i) {
        c->recv[i] = i < nbuf ? static_cast<char*>(c->recv_block) + static_cast<size_t>(i) * half_bytes : nullptr;
        c->recv_cap[i] = i < nbuf ? half_bytes : 0;
    }
    return RING_OK;
}

}  // namespace

// The reference's set_params_fprop (csrc/ring_attention.cu:361-395) with the same leading arguments.
// It only fills the struct: no allocation, no copy (the reference does three of each per call).
void set_params_fprop(Ring_fwd_params& params, const void* q, const void* k, const void* v, float* out, int npes,
                      int mype, const int* seqlen, int dim, int max_seq) {
    (void)max_seq;  // receive buffers are sized from seqlen[] by the context
    std::memset(&params, 0, sizeof(params));
    params.mype = mype;
    params.npes = npes;
    params.seqlen = nullptr;
    params.h_seqlen = const_cast<int*>(seqlen);
    params.dim = dim;
    params.softmax_scale = dim > 0 ? 1.0f / std::sqrt(static_cast<float>(dim)) : 1.0f;
    params.q_ptr = const_cast<void*>(q);
    params.k_ptr = const_cast<void*>(k);
    params.v_ptr = const_cast<void*>(v);
    params.out_ptr = out;
    params.k_buffer = nullptr;
    params.v_buffer = nullptr;
    params.batch = 1;
    params.heads = 1;
    params.lse_ptr = nullptr;
    params.causal = 0;
    params.is_bf16 = 0;
    params.stream = 0;
}

// One ring step of one rank, as pure host logic (no CUDA): which shard the step attends to, whether it
// computes at all, what is exchanged meanwhile and through which receive buffer.  run_ring_fwd() follows
// exactly this plan; it is exported so the schedule can be checked without a GPU.
//   step s attends to the shard of rank (rank + s) % world            (csrc/ring_attention.cu:463)
//   exchange s (s < world - 1) brings the shard of step s + 1 into recv buffer s & 1, pulled from its
//   ORIGIN rank (csrc/ring_attention.cu:613-617), while this rank's shard goes to (rank - s - 1) mod world.
extern "C" int ring_step_plan(int world, int rank, int step, int causal, int causal_skip_exchange, RingStepPlan* out) {
    if (!out) return fail(RING_ERR_INVALID_ARGUMENT, "null plan");
    if (world < 1 || rank < 0 || rank >= world || step < 0 || step >= world)
        return fail(RING_ERR_INVALID_ARGUMENT, "bad world/rank/step %d/%d/%d", world, rank, step);
    const bool skip_x = causal && causal_skip_exchange;
    out->src_rank = (rank + step) % world;
    out->compute = !(causal && out->src_rank > rank);  // a shard strictly after this rank's rows is fully masked
    out->compute_buffer = step == 0 ? -1 : ((step - 1) & 1);
    out->recv_buffer = step & 1;
    if (step < world - 1) {
        out->recv_from = (rank + step + 1) % world;
        out->send_to = (rank - step - 1 + 2 * world) % world;
        out->do_recv = (!skip_x || out->recv_from < rank) ? 1 : 0;  // a causal rank only reads shards at or before its own
        out->do_send = (!skip_x || out->send_to > rank) ? 1 : 0;
    } else {
        out->recv_from = out->send_to = -1;
        out->do_recv = out->do_send = 0;
    }
    return RING_OK;
}

// The ring loop.  Named after the reference's launcher (csrc/ring_attention.cu:669-704); the template
// parameter of the reference (kernel traits) is chosen at run time from params.dim by launch_block().
int run_ring_fwd(RingCtx* c, const Ring_fwd_params& p, cudaStream_t stream) {
    const int P = p.npes;
    const int r = p.mype;
    const int B = p.batch > 0 ? p.batch : 1;
    const int H = p.heads > 0 ? p.heads : 1;
    const int S = p.h_seqlen[r];
    const int D = p.dim;
    // Shards may differ in length (seqlen[] per PE, csrc/ring.h:9, csrc/ring_attention.cu:463,531): this rank ships
    // `shard_bytes` of K and of V, receives bytes_of(source) of each, and every receive buffer is laid out for the
    // longest shard (V starts at max_shard_bytes) so that sender and receiver agree without talking.
    auto bytes_of = [&](int rank) { return static_cast<size_t>(B) * H * p.h_seqlen[rank] * D * 2; };
    const size_t shard_bytes = bytes_of(r);  // one of K or V of this rank
    size_t max_shard_bytes = 0;
    std::vector<int64_t> row0(P + 1, 0);  // global index of the first row of every shard
    for (int i = 0; i < P; ++i) {
        max_shard_bytes = bytes_of(i) > max_shard_bytes ? bytes_of(i) : max_shard_bytes;
        row0[i + 1] = row0[i] + p.h_seqlen[i];
    }
    const int64_t rows = static_cast<int64_t>(B) * H * S;
    const bool causal = p.causal != 0;
    int rc;
    // Zig-zag causal sharding: the sequence is cut into 2P chunks and rank r holds chunks r and 2P-1-r (in that order),
    // so that every rank masks the same amount.  Every step then has visible keys and every shard travels.
    const bool zig = causal && c->zigzag;
    const int plan_causal = (causal && !zig) ? 1 : 0;
    if (zig) {
        for (int i = 0; i < P; ++i)
            if (p.h_seqlen[i] != S || (S & 1))
                return fail(RING_ERR_INVALID_ARGUMENT, "zig-zag sharding needs equal, even shard lengths");
    }

    const bool peer = !c->local && P > 1 && c->transport == RING_TRANSPORT_PEER_COPY;
    // Receive buffers: exchange e lands in buffer e % nbuf and compute step s >= 1 reads buffer (s - 1) % nbuf.  With two
    // (the default) exchange e must wait until step e - 1 has read the buffer; with one per remote shard no exchange
    // ever waits for a compute step.
    const int nbuf = P > 1 ? ((c->recv_buffers <= 0 || c->recv_buffers > P - 1) ? (P - 1 > 1 ? P - 1 : 1) : c->recv_buffers) : 1;
    auto compute_buf = [&](int step) { return (step - 1) % nbuf; };
    StreamMemOps ops;
    uint32_t seq = 0;
    if (peer) {
        if ((rc = stream_mem_ops(&ops))) return rc;
        if ((rc = peer_grow_recv(c, 2 * max_shard_bytes, nbuf))) return rc;
        seq = ++c->call_seq;
    } else {
        if (c->recv_block) return fail(RING_ERR_UNSUPPORTED, "switching from the peer-copy transport back to NCCL is not supported");
        for (int i = 0; i < nbuf && i < P - 1; ++i)
            if ((rc = grow(&c->recv[i], &c->recv_cap[i], 2 * max_shard_bytes))) return rc;
    }
    float* lse = static_cast<float*>(p.lse_ptr);
    if (!lse) {
        if ((rc = grow(reinterpret_cast<void**>(&c->lse_own), &c->lse_own_cap, rows * sizeof(float)))) return rc;
        lse = c->lse_own;
    }
    if (P > 1 && c->merge_mode == RING_MERGE_SEPARATE_KERNEL) {
        if ((rc = grow(reinterpret_cast<void**>(&c->o_part), &c->o_part_cap, rows * D * sizeof(float)))) return rc;
        if ((rc = grow(reinterpret_cast<void**>(&c->lse_part), &c->lse_part_cap, rows * sizeof(float)))) return rc;
    }

    // The exchange stream may touch K/V only once the compute stream's earlier work (which may have
    // produced them) is done.
    if (c->have_call_done) RING_CUDA(cudaStreamWaitEvent(stream, c->ev_call_done, 0));  // callers may change streams
    if (P > 1) {
        RING_CUDA(cudaEventRecord(c->ev_fork, stream));
        RING_CUDA(cudaStreamWaitEvent(c->comm_stream, c->ev_fork, 0));
    }
    if (peer) {
        // Every receive buffer is free here (their last readers precede this point on `stream`): tell the
        // origins of the first nbuf exchanges.
        for (int e = 0; e < nbuf && e < P - 1; ++e) {
            RingStepPlan pe;
            if ((rc = ring_step_plan(P, r, e, plan_causal, c->causal_skip, &pe))) return rc;
            if (pe.do_recv)
                RING_CU(ops.write(reinterpret_cast<CUstream>(stream),
                                  reinterpret_cast<CUdeviceptr>(c->peer_flags[pe.recv_from] + kFlagCredit + e), seq, 0));
        }
    }

    c->last_steps = P;
    bool have_partial = false;
    bool zig_have[2] = {false, false};
    bool prev_do_recv = false;
    for (int s = 0; s < P; ++s) {
        RingStepPlan plan;
        if ((rc = ring_step_plan(P, r, s, plan_causal, c->causal_skip, &plan))) return rc;
        const int src = plan.src_rank;

        // ---- exchange s: bring the shard of step s + 1 into recv[s & 1] while step s computes --------
        c->step_exchanged[s] = false;
        if (s < P - 1) {
            const int nsrc = plan.recv_from;  // whose shard arrives
            const int ndst = plan.send_to;    // who gets this rank's shard
            const bool do_recv = plan.do_recv != 0;
            const bool do_send = plan.do_send != 0;
            if (c->record_timings) RING_CUDA(cudaEventRecord(c->ev_comm_start[s], c->comm_stream));
            // buffer s % nbuf was last read by compute step s - nbuf + 1
            if (s >= nbuf && !peer) RING_CUDA(cudaStreamWaitEvent(c->comm_stream, c->ev_compute_done[s - nbuf + 1], 0));
            if (c->record_timings && !peer) RING_CUDA(cudaEventRecord(c->ev_copy_start[s], c->comm_stream));
            const int recv_buf = s % nbuf;
            char* dst_k = static_cast<char*>(c->recv[recv_buf]);
            char* dst_v = dst_k + max_shard_bytes;
            const size_t in_bytes = bytes_of(nsrc);
            if (peer) {
                if (do_send) {
                    CUstream cs = reinterpret_cast<CUstream>(c->comm_stream);
                    RING_CU(ops.wait(cs, reinterpret_cast<CUdeviceptr>(c->flags + kFlagCredit + s), seq, CU_STREAM_WAIT_VALUE_GEQ));
                    if (c->record_timings) RING_CUDA(cudaEventRecord(c->ev_copy_start[s], c->comm_stream));
                    char* remote = static_cast<char*>(c->peer_recv_block[ndst]) + static_cast<size_t>(recv_buf) * c->peer_recv_half[ndst];
                    RING_CUDA(cudaMemcpyAsync(remote, p.k_ptr, shard_bytes, cudaMemcpyDeviceToDevice, c->comm_stream));
                    RING_CUDA(cudaMemcpyAsync(remote + max_shard_bytes, p.v_ptr, shard_bytes, cudaMemcpyDeviceToDevice, c->comm_stream));
                    RING_CU(ops.write(cs, reinterpret_cast<CUdeviceptr>(c->peer_flags[ndst] + kFlagReady + s), seq, 0));
                } else if (c->record_timings) {
                    RING_CUDA(cudaEventRecord(c->ev_copy_start[s], c->comm_stream));
                }
            } else if (c->local) {
                if (do_recv) {
                    if (!c->local_k[nsrc] || !c->local_v[nsrc])
                        return fail(RING_ERR_INVALID_ARGUMENT, "local shard %d was not registered", nsrc);
                    RING_CUDA(cudaMemcpyAsync(dst_k, c->local_k[nsrc], in_bytes, cudaMemcpyDeviceToDevice, c->comm_stream));
                    RING_CUDA(cudaMemcpyAsync(dst_v, c->local_v[nsrc], in_bytes, cudaMemcpyDeviceToDevice, c->comm_stream));
                }
            } else if (do_recv || do_send) {
                // The group is closed on every path: an error between GroupStart and GroupEnd must not leave this
                // thread inside an open NCCL group.
                NcclApi& n = nccl();
                RING_NCCL(n.GroupStart());
                ncclResult_t gr = ncclSuccess;
                if (do_send) {
                    gr = n.Send(p.k_ptr, shard_bytes, ncclInt8, ndst, c->comm, c->comm_stream);
                    if (gr == ncclSuccess) gr = n.Send(p.v_ptr, shard_bytes, ncclInt8, ndst, c->comm, c->comm_stream);
                }
                if (do_recv && gr == ncclSuccess) {
                    gr = n.Recv(dst_k, in_bytes, ncclInt8, nsrc, c->comm, c->comm_stream);
                    if (gr == ncclSuccess) gr = n.Recv(dst_v, in_bytes, ncclInt8, nsrc, c->comm, c->comm_stream);
                }
                const ncclResult_t ge = n.GroupEnd();
                RING_NCCL(gr);
                RING_NCCL(ge);
            }
            c->step_exchanged[s] = do_recv || do_send;
            RING_CUDA(cudaEventRecord(c->ev_recv_done[s], c->comm_stream));
        }

        // ---- compute step s ----------------------------------------------------------------------------
        if (s >= 1) {
            if (!peer) {
                RING_CUDA(cudaStreamWaitEvent(stream, c->ev_recv_done[s - 1], 0));
            } else if (prev_do_recv) {
                RING_CU(ops.wait(reinterpret_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(c->flags + kFlagReady + (s - 1)), seq,
                                 CU_STREAM_WAIT_VALUE_GEQ));
            }
        }
        prev_do_recv = plan.do_recv != 0;
        if (c->record_timings) RING_CUDA(cudaEventRecord(c->ev_compute_start[s], stream));
        const bool compute = plan.compute != 0;
        c->step_computed[s] = compute;
        if (compute && zig) {
            // four half-shard products per step, of which the causal mask leaves two (three on the own shard)
            const int half = S / 2;
            const char* kbase = static_cast<const char*>(s == 0 ? p.k_ptr : c->recv[compute_buf(s)]);
            const char* vbase = s == 0 ? static_cast<const char*>(p.v_ptr)
                                       : static_cast<const char*>(c->recv[compute_buf(s)]) + max_shard_bytes;
            for (int qp = 0; qp < 2; ++qp) {
                for (int kp = 0; kp < 2; ++kp) {
                    const int q_chunk = qp ? 2 * P - 1 - r : r;
                    const int k_chunk = kp ? 2 * P - 1 - src : src;
                    if (k_chunk > q_chunk) continue;  // every key after every query
                    BlockLaunch L;
                    L.q = static_cast<const char*>(p.q_ptr) + static_cast<size_t>(qp) * half * D * 2;
                    L.k = kbase + static_cast<size_t>(kp) * half * D * 2;
                    L.v = vbase + static_cast<size_t>(kp) * half * D * 2;
                    L.o = static_cast<float*>(p.out_ptr) + static_cast<size_t>(qp) * half * D;
                    L.lse = lse + static_cast<size_t>(qp) * half;
                    L.batch = B; L.heads = H; L.sq = half; L.sk = half; L.dim = D;
                    L.q_rows_total = S; L.k_rows_total = S;
                    L.scale = p.softmax_scale;
                    L.causal = k_chunk == q_chunk;  // only the diagonal chunk pair is masked inside
                    L.q_off = static_cast<int64_t>(q_chunk) * half;
                    L.k_off = static_cast<int64_t>(k_chunk) * half;
                    L.is_bf16 = p.is_bf16;
                    L.merge = zig_have[qp] ? 1 : 0;
                    if ((rc = launch_block(L, stream))) return rc;
                    zig_have[qp] = true;
                }
            }
        } else if (compute) {
            BlockLaunch L;
            L.q = p.q_ptr;
            L.k = s == 0 ? p.k_ptr : c->recv[compute_buf(s)];
            L.v = s == 0 ? p.v_ptr : static_cast<char*>(c->recv[compute_buf(s)]) + max_shard_bytes;
            L.batch = B;
            L.heads = H;
            L.sq = S;
            L.sk = p.h_seqlen[src];
            L.dim = D;
            L.scale = p.softmax_scale;
            L.causal = causal;
            L.q_off = row0[r];
            L.k_off = row0[src];
            L.is_bf16 = p.is_bf16;
            if (!have_partial || c->merge_mode == RING_MERGE_FUSED_EPILOGUE) {
                L.o = static_cast<float*>(p.out_ptr);
                L.lse = lse;
                L.merge = have_partial ? 1 : 0;
                if ((rc = launch_block(L, stream))) return rc;
            } else {
                L.o = c->o_part;
                L.lse = c->lse_part;
                L.merge = 0;
                if ((rc = launch_block(L, stream))) return rc;
                if ((rc = launch_merge(static_cast<float*>(p.out_ptr), lse, c->o_part, c->lse_part, rows, D, stream)))
                    return rc;
            }
            have_partial = true;
        }
        RING_CUDA(cudaEventRecord(c->ev_compute_done[s], stream));
        if (peer && s >= 1 && s - 1 + nbuf <= P - 2) {
            // step s was the last reader of receive buffer (s - 1) % nbuf: free it for exchange s - 1 + nbuf
            const int e = s - 1 + nbuf;
            RingStepPlan pe;
            if ((rc = ring_step_plan(P, r, e, plan_causal, c->causal_skip, &pe))) return rc;
            if (pe.do_recv)
                RING_CU(ops.write(reinterpret_cast<CUstream>(stream),
                                  reinterpret_cast<CUdeviceptr>(c->peer_flags[pe.recv_from] + kFlagCredit + e), seq, 0));
        }
    }
    if (peer) {
        // the call is complete on `stream` only when this rank's own pushes are done (K/V may then be reused)
        RING_CUDA(cudaEventRecord(c->ev_push_done, c->comm_stream));
        RING_CUDA(cudaStreamWaitEvent(stream, c->ev_push_done, 0));
    }
    RING_CUDA(cudaEventRecord(c->ev_call_done, stream));
    c->have_call_done = true;
    return RING_OK;
}

namespace {

int validate_params(RingCtx* c, const Ring_fwd_params* p) {
    if (!c) return fail(RING_ERR_INVALID_ARGUMENT, "null context");
    if (c->dead) return fail(RING_ERR_UNSUPPORTED, "the context was aborted (ring_ctx_abort); destroy it and create a new one");
    if (!p) return fail(RING_ERR_INVALID_ARGUMENT, "null params");
    if (!p->q_ptr || !p->k_ptr || !p->v_ptr || !p->out_ptr) return fail(RING_ERR_INVALID_ARGUMENT, "null tensor pointer");
    if (p->npes != c->world)
        return fail(RING_ERR_INVALID_ARGUMENT, "params.npes (%d) differs from the context's world size (%d)", p->npes, c->world);
    if (p->mype < 0 || p->mype >= p->npes) return fail(RING_ERR_INVALID_ARGUMENT, "params.mype out of range");
    if (!c->local && p->mype != c->rank)
        return fail(RING_ERR_INVALID_ARGUMENT, "params.mype (%d) differs from the context's rank (%d)", p->mype, c->rank);
    if (p->dim != 64 && p->dim != 128) return fail(RING_ERR_INVALID_ARGUMENT, "dim must be 64 or 128, got %d", p->dim);
    if (!p->h_seqlen) return fail(RING_ERR_INVALID_ARGUMENT, "params.h_seqlen (host sequence-length table) is null");
    for (int i = 0; i < p->npes; ++i)
        if (p->h_seqlen[i] <= 0 || p->h_seqlen[i] > (1 << 24))
            return fail(RING_ERR_INVALID_ARGUMENT, "seqlen[%d] = %d: every rank needs between 1 and 2^24 rows", i, p->h_seqlen[i]);
    if (!(p->softmax_scale > 0.f) || !std::isfinite(p->softmax_scale))
        return fail(RING_ERR_INVALID_ARGUMENT, "softmax_scale must be positive and finite");
    int dev = -1;
    RING_CUDA(cudaGetDevice(&dev));
    if (dev != c->device)
        return fail(RING_ERR_INVALID_ARGUMENT, "current device %d is not the context's device %d", dev, c->device);
    return RING_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------ C ABI
extern "C" {

const char* ring_last_error_string(void) { return g_last_error.c_str(); }

int64_t ring_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int ring_device_status(int* status_out) {
    if (!status_out) return fail(RING_ERR_INVALID_ARGUMENT, "null status_out");
    return read_status(status_out);
}

int ring_device_status_reset(void) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    RING_CUDA(cudaDeviceSynchronize());
    RING_CUDA(cudaMemset(st->d_status, 0, sizeof(int)));
    return RING_OK;
}

// Host-side fault injection for tests: stores `code` in the device status word, as a kernel whose bounded wait
// ran out would.  Every later kernel of this library then returns at once until ring_device_status_reset().
int ring_device_status_inject(int code) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    RING_CUDA(cudaDeviceSynchronize());
    RING_CUDA(cudaMemcpy(st->d_status, &code, sizeof(int), cudaMemcpyHostToDevice));
    return RING_OK;
}

// Runs the kernels' bounded wait on an mbarrier that nothing ever completes (one CTA, one thread) and reports what
// it left in `status_out`: the wait must give up after its limit (about two seconds), record `code`, and return.
int ring_selftest_wait_timeout(int code, int* status_out, float* waited_ms) {
    if (!status_out) return fail(RING_ERR_INVALID_ARGUMENT, "null status_out");
    int* d = nullptr;
    RING_CUDA(cudaMalloc(&d, sizeof(int)));
    RING_CUDA(cudaMemset(d, 0, sizeof(int)));
    cudaEvent_t e0, e1;
    RING_CUDA(cudaEventCreate(&e0));
    RING_CUDA(cudaEventCreate(&e1));
    RING_CUDA(cudaEventRecord(e0, 0));
    ring::ring_wait_timeout_probe<<<1, 32>>>(d, code);
    RING_CUDA(cudaGetLastError());
    RING_CUDA(cudaEventRecord(e1, 0));
    RING_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    RING_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (waited_ms) *waited_ms = ms;
    RING_CUDA(cudaMemcpy(status_out, d, sizeof(int), cudaMemcpyDeviceToHost));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    RING_CUDA(cudaFree(d));
    return RING_OK;
}

int ring_get_unique_id(void* id_out) {
    if (!id_out) return fail(RING_ERR_INVALID_ARGUMENT, "null id_out");
    NcclApi& n = nccl();
    if (!n.ok) return fail(RING_ERR_NCCL, "libnccl.so.2 could not be loaded");
    static_assert(sizeof(ncclUniqueId) <= RING_UNIQUE_ID_BYTES, "unique id size");
    ncclUniqueId id;
    RING_NCCL(n.GetUniqueId(&id));
    std::memset(id_out, 0, RING_UNIQUE_ID_BYTES);
    std::memcpy(id_out, &id, sizeof(id));
    return RING_OK;
}

int ring_ctx_create(RingCtx** ctx, int rank, int world, const void* unique_id) {
    if (!ctx) return fail(RING_ERR_INVALID_ARGUMENT, "null ctx");
    *ctx = nullptr;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
        return fail(RING_ERR_INVALID_ARGUMENT, "bad rank/world %d/%d", rank, world);
    if (world > 1 && !unique_id) return fail(RING_ERR_INVALID_ARGUMENT, "world > 1 needs a unique id");
    RingCtx* c = new RingCtx();
    c->rank = rank;
    c->world = world;
    int rc = ctx_common_init(c);
    if (rc) { const std::string msg = g_last_error; ring_ctx_destroy(c); g_last_error = msg; return rc; }
    if (world > 1) {
        NcclApi& n = nccl();
        if (!n.ok) { ring_ctx_destroy(c); return fail(RING_ERR_NCCL, "libnccl.so.2 could not be loaded"); }
        ncclUniqueId id;
        std::memcpy(&id, unique_id, sizeof(id));
        // The exchange only has to keep pace with the block kernel (one K/V shard per ring step), not to
        // saturate NVLink; every CTA NCCL runs is an SM the block kernel does not get.  Cap them
        // (RING_NCCL_MAX_CTAS, default 16; 0 leaves NCCL's own choice).
        int max_ctas = 16;
        if (const char* e = std::getenv("RING_NCCL_MAX_CTAS")) max_ctas = std::atoi(e);
        ncclResult_t r;
        if (max_ctas > 0) {
            ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
            cfg.maxCTAs = max_ctas;
            cfg.minCTAs = 1;
            r = n.CommInitRankConfig(&c->comm, world, id, rank, &cfg);
        } else {
            r = n.CommInitRank(&c->comm, world, id, rank);
        }
        if (r != ncclSuccess) {
            c->comm = nullptr;
            ring_ctx_destroy(c);
            return fail(RING_ERR_NCCL, "ncclCommInitRank failed: %s", n.GetErrorString(r));
        }
        // Peer-copy transport: share the flag blocks now (collective); fall back to NCCL send/recv if the
        // processes cannot map each other's memory.
        const char* want = std::getenv("RING_TRANSPORT");
        const bool force_nccl = want && std::strcmp(want, "nccl") == 0;
        if (!force_nccl) {
            rc = peer_setup_flags(c);
            if (rc) { const std::string msg = g_last_error; ring_ctx_destroy(c); g_last_error = msg; return rc; }
            c->transport = c->peer_ready ? RING_TRANSPORT_PEER_COPY : RING_TRANSPORT_NCCL;
            if (!c->peer_ready && want && std::strcmp(want, "peer") == 0) {
                ring_ctx_destroy(c);
                return fail(RING_ERR_UNSUPPORTED, "RING_TRANSPORT=peer, but the ranks cannot map each other's memory (CUDA IPC)");
            }
        }
    }
    *ctx = c;
    return RING_OK;
}

int ring_ctx_create_local(RingCtx** ctx, int world) {
    if (!ctx) return fail(RING_ERR_INVALID_ARGUMENT, "null ctx");
    *ctx = nullptr;
    if (world < 1 || world > kMaxWorld) return fail(RING_ERR_INVALID_ARGUMENT, "bad world %d", world);
    RingCtx* c = new RingCtx();
    c->rank = 0;
    c->world = world;
    c->local = true;
    int rc = ctx_common_init(c);
    if (rc) { const std::string msg = g_last_error; ring_ctx_destroy(c); g_last_error = msg; return rc; }
    *ctx = c;
    return RING_OK;
}

int ring_ctx_set_local_shards(RingCtx* ctx, const void* const* k_shards, const void* const* v_shards) {
    if (!ctx || !ctx->local || !k_shards || !v_shards)
        return fail(RING_ERR_INVALID_ARGUMENT, "needs a local context and two pointer tables");
    for (int i = 0; i < ctx->world; ++i) {
        ctx->local_k[i] = k_shards[i];
        ctx->local_v[i] = v_shards[i];
    }
    return RING_OK;
}

int ring_ctx_set_option(RingCtx* ctx, int option, int value) {
    if (!ctx) return fail(RING_ERR_INVALID_ARGUMENT, "null context");
    switch (option) {
        case RING_OPT_MERGE_MODE:
            if (value != RING_MERGE_SEPARATE_KERNEL && value != RING_MERGE_FUSED_EPILOGUE)
                return fail(RING_ERR_INVALID_ARGUMENT, "bad merge mode %d", value);
            ctx->merge_mode = value;
            return RING_OK;
        case RING_OPT_CAUSAL_SKIP_EXCHANGE:
            ctx->causal_skip = value ? 1 : 0;
            return RING_OK;
        case RING_OPT_RECORD_TIMINGS:
            ctx->record_timings = value ? 1 : 0;
            return RING_OK;
        case RING_OPT_CAUSAL_ZIGZAG:
            ctx->zigzag = value ? 1 : 0;
            return RING_OK;
        case RING_OPT_RECV_BUFFERS:
            if (value < 0 || value == 1 || value > kMaxWorld) return fail(RING_ERR_INVALID_ARGUMENT, "bad receive-buffer count %d", value);
            ctx->recv_buffers = value;
            return RING_OK;
        case RING_OPT_TRANSPORT:
            if (value != RING_TRANSPORT_NCCL && value != RING_TRANSPORT_PEER_COPY)
                return fail(RING_ERR_INVALID_ARGUMENT, "bad transport %d", value);
            if (value == RING_TRANSPORT_PEER_COPY && !ctx->peer_ready)
                return fail(RING_ERR_UNSUPPORTED, "the peer-copy transport is not available in this context");
            ctx->transport = value;
            return RING_OK;
        default:
            return fail(RING_ERR_INVALID_ARGUMENT, "unknown option %d", option);
    }
}

int ring_ctx_get_option(RingCtx* ctx, int option, int* value) {
    if (!ctx || !value) return fail(RING_ERR_INVALID_ARGUMENT, "null argument");
    switch (option) {
        case RING_OPT_MERGE_MODE: *value = ctx->merge_mode; return RING_OK;
        case RING_OPT_CAUSAL_SKIP_EXCHANGE: *value = ctx->causal_skip; return RING_OK;
        case RING_OPT_RECORD_TIMINGS: *value = ctx->record_timings; return RING_OK;
        case RING_OPT_TRANSPORT: *value = ctx->transport; return RING_OK;
        case RING_OPT_CAUSAL_ZIGZAG: *value = ctx->zigzag; return RING_OK;
        case RING_OPT_RECV_BUFFERS: *value = ctx->recv_buffers; return RING_OK;
        default: return fail(RING_ERR_INVALID_ARGUMENT, "unknown option %d", option);
    }
}

int ring_ctx_destroy(RingCtx* c) {
    if (!c) return RING_OK;
    if (g_default_ctx == c) g_default_ctx = nullptr;
    if (g_solo_ctx == c) g_solo_ctx = nullptr;
    // An aborted context has released every wait it had queued (ring_ctx_abort) and its communicator is gone;
    // waiting for the device here could block on whatever made the caller abort.
    if (!c->dead) {
        cudaDeviceSynchronize();
    } else {
        // give the released work a bounded time to drain before its buffers go away
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(5);
        while (std::chrono::steady_clock::now() < deadline) {
            const cudaError_t e1 = c->have_call_done ? cudaEventQuery(c->ev_call_done) : cudaSuccess;
            const cudaError_t e2 = c->comm_stream ? cudaStreamQuery(c->comm_stream) : cudaSuccess;
            (void)cudaGetLastError();
            if (e1 != cudaErrorNotReady && e2 != cudaErrorNotReady) break;
            std::this_thread::sleep_for(std::chrono::milliseconds(1));
        }
    }
    if (c->comm) nccl().CommDestroy(c->comm);
    for (int i = 0; i < c->world; ++i) {
        if (c->ev_recv_done[i]) cudaEventDestroy(c->ev_recv_done[i]);
        if (c->ev_comm_start[i]) cudaEventDestroy(c->ev_comm_start[i]);
        if (c->ev_copy_start[i]) cudaEventDestroy(c->ev_copy_start[i]);
        if (c->ev_compute_start[i]) cudaEventDestroy(c->ev_compute_start[i]);
        if (c->ev_compute_done[i]) cudaEventDestroy(c->ev_compute_done[i]);
    }
    for (int i = 0; i < c->world; ++i) {
        if (i == c->rank) continue;
        if (c->peer_recv_block[i]) cudaIpcCloseMemHandle(c->peer_recv_block[i]);
        if (c->peer_flags[i]) cudaIpcCloseMemHandle(c->peer_flags[i]);
    }
    if (c->recv_block) {
        cudaFree(c->recv_block);
        for (int i = 0; i < kMaxWorld; ++i) c->recv[i] = nullptr;
    }
    if (c->flags) cudaFree(c->flags);
    if (c->xchg_dev) cudaFree(c->xchg_dev);
    for (int i = 0; i < 2; ++i) {
        if (c->stage_in[i]) cudaFree(c->stage_in[i]);
        if (c->stage_out[i]) cudaFree(c->stage_out[i]);
    }
    if (c->host_ready) {
        for (int i = 0; i < kMaxWorld; ++i) { cudaEventDestroy(c->ev_h2d[i]); cudaEventDestroy(c->ev_comp[i]); cudaEventDestroy(c->ev_d2h[i]); }
        cudaStreamDestroy(c->h2d_stream);
        cudaStreamDestroy(c->d2h_stream);
    }
    if (c->ev_push_done) cudaEventDestroy(c->ev_push_done);
    if (c->ev_call_done) cudaEventDestroy(c->ev_call_done);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    if (c->comm_stream) cudaStreamDestroy(c->comm_stream);
    for (int i = 0; i < kMaxWorld; ++i)
        if (c->recv[i]) cudaFree(c->recv[i]);
    if (c->o_part) cudaFree(c->o_part);
    if (c->lse_part) cudaFree(c->lse_part);
    if (c->lse_own) cudaFree(c->lse_own);
    delete c;
    return RING_OK;
}

int ring_set_default_ctx(RingCtx* ctx) {
    g_default_ctx = ctx;
    return RING_OK;
}

int ring_attention_fwd(RingCtx* ctx, const struct Ring_fwd_params* params) {
    int rc = validate_params(ctx, params);
    if (rc) return rc;
    return run_ring_fwd(ctx, *params, params->stream);
}

// Host-buffer forward: the (batch, head) slabs are independent, so they are taken `chunks` groups at a time and the
// host-to-device copy of group c + 1, the ring forward of group c and the device-to-host copy of group c - 1 overlap
// (PCIe is full duplex).  Every rank of the context must call it with the same shapes and chunk count.
int ring_attention_fwd_host(RingCtx* c, const struct Ring_fwd_params* hp, int chunks) {
    int rc = validate_params(c, hp);
    if (rc) return rc;
    const int B = hp->batch > 0 ? hp->batch : 1, H = hp->heads > 0 ? hp->heads : 1;
    const int slabs = B * H;
    if (chunks < 1) chunks = 1;
    if (chunks > slabs) chunks = slabs;
    if (chunks > kMaxWorld) chunks = kMaxWorld;
    const int S = hp->h_seqlen[hp->mype], D = hp->dim;
    const size_t slab_in = static_cast<size_t>(S) * D * 2, slab_out = static_cast<size_t>(S) * D * 4, slab_lse = static_cast<size_t>(S) * 4;
    const int per = (slabs + chunks - 1) / chunks;
    if (!c->host_ready) {
        RING_CUDA(cudaStreamCreateWithFlags(&c->h2d_stream, cudaStreamNonBlocking));
        RING_CUDA(cudaStreamCreateWithFlags(&c->d2h_stream, cudaStreamNonBlocking));
        for (int i = 0; i < kMaxWorld; ++i) {
            RING_CUDA(cudaEventCreateWithFlags(&c->ev_h2d[i], cudaEventDisableTiming));
            RING_CUDA(cudaEventCreateWithFlags(&c->ev_comp[i], cudaEventDisableTiming));
            RING_CUDA(cudaEventCreateWithFlags(&c->ev_d2h[i], cudaEventDisableTiming));
        }
        c->host_ready = true;
    }
    for (int i = 0; i < 2; ++i) {
        if ((rc = grow(&c->stage_in[i], &c->stage_in_cap[i], 3 * per * slab_in))) return rc;
        if ((rc = grow(&c->stage_out[i], &c->stage_out_cap[i], per * (slab_out + slab_lse)))) return rc;
    }
    cudaStream_t cs = hp->stream;
    // the copies may start once the caller's stream has reached this point (the host buffers are then ready)
    RING_CUDA(cudaEventRecord(c->ev_fork, cs));
    RING_CUDA(cudaStreamWaitEvent(c->h2d_stream, c->ev_fork, 0));
    RING_CUDA(cudaStreamWaitEvent(c->d2h_stream, c->ev_fork, 0));
    int nch = 0;
    for (int s0 = 0; s0 < slabs; s0 += per, ++nch) {
        const int n = (slabs - s0) < per ? (slabs - s0) : per;
        const int set = nch & 1;
        char* dq = static_cast<char*>(c->stage_in[set]);
        char* dk = dq + per * slab_in;
        char* dv = dk + per * slab_in;
        char* dout = static_cast<char*>(c->stage_out[set]);
        char* dlse = dout + per * slab_out;
        if (nch >= 2) RING_CUDA(cudaStreamWaitEvent(c->h2d_stream, c->ev_comp[nch - 2], 0));  // staging set reuse
        RING_CUDA(cudaMemcpyAsync(dq, static_cast<const char*>(hp->q_ptr) + s0 * slab_in, n * slab_in, cudaMemcpyHostToDevice, c->h2d_stream));
        RING_CUDA(cudaMemcpyAsync(dk, static_cast<const char*>(hp->k_ptr) + s0 * slab_in, n * slab_in, cudaMemcpyHostToDevice, c->h2d_stream));
        RING_CUDA(cudaMemcpyAsync(dv, static_cast<const char*>(hp->v_ptr) + s0 * slab_in, n * slab_in, cudaMemcpyHostToDevice, c->h2d_stream));
        RING_CUDA(cudaEventRecord(c->ev_h2d[nch], c->h2d_stream));
        RING_CUDA(cudaStreamWaitEvent(cs, c->ev_h2d[nch], 0));
        if (nch >= 2) RING_CUDA(cudaStreamWaitEvent(cs, c->ev_d2h[nch - 2], 0));
        Ring_fwd_params p = *hp;
        p.batch = 1;
        p.heads = n;
        p.q_ptr = dq; p.k_ptr = dk; p.v_ptr = dv; p.out_ptr = dout; p.lse_ptr = dlse;
        if ((rc = run_ring_fwd(c, p, cs))) return rc;
        RING_CUDA(cudaEventRecord(c->ev_comp[nch], cs));
        RING_CUDA(cudaStreamWaitEvent(c->d2h_stream, c->ev_comp[nch], 0));
        RING_CUDA(cudaMemcpyAsync(static_cast<char*>(hp->out_ptr) + s0 * slab_out, dout, n * slab_out, cudaMemcpyDeviceToHost, c->d2h_stream));
        if (hp->lse_ptr)
            RING_CUDA(cudaMemcpyAsync(static_cast<char*>(hp->lse_ptr) + s0 * slab_lse, dlse, n * slab_lse, cudaMemcpyDeviceToHost, c->d2h_stream));
        RING_CUDA(cudaEventRecord(c->ev_d2h[nch], c->d2h_stream));
    }
    // complete on the caller's stream only when the last results are on the host
    for (int i = nch > 2 ? nch - 2 : 0; i < nch; ++i) RING_CUDA(cudaStreamWaitEvent(cs, c->ev_d2h[i], 0));
    return RING_OK;
}

int ring_ctx_synchronize(RingCtx* ctx) {
    if (!ctx) return fail(RING_ERR_INVALID_ARGUMENT, "null context");
    int status = 0;
    int rc = read_status(&status);
    if (rc) return rc;
    if (ctx->comm) {
        ncclResult_t async = ncclSuccess;
        RING_NCCL(nccl().CommGetAsyncError(ctx->comm, &async));
        if (async != ncclSuccess) return fail(RING_ERR_NCCL, "NCCL async error: %s", nccl().GetErrorString(async));
    }
    if (status != 0) return fail(RING_ERR_DEVICE_TIMEOUT, "a bounded wait inside a kernel ran out (device status %d)", status);
    return RING_OK;
}

// Host-side failure detection: the same as ring_ctx_synchronize, but gives up after `timeout_ms`.  A forward
// whose peer stopped (its exchange stream then waits for a flag or an NCCL message that never comes), or whose
// stream is blocked upstream, never completes; this call notices without touching the device: it polls the
// completion event of the last forward and the exchange stream, and returns RING_ERR_HOST_TIMEOUT when the
// deadline passes.  The context is left as it is: the caller decides (wait longer, or tear the job down).
int ring_ctx_synchronize_timeout(RingCtx* ctx, int timeout_ms) {
    if (!ctx) return fail(RING_ERR_INVALID_ARGUMENT, "null context");
    if (timeout_ms < 0) return ring_ctx_synchronize(ctx);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
        cudaError_t e1 = ctx->have_call_done ? cudaEventQuery(ctx->ev_call_done) : cudaSuccess;
        cudaError_t e2 = ctx->comm_stream ? cudaStreamQuery(ctx->comm_stream) : cudaSuccess;
        cudaError_t e3 = ctx->d2h_stream ? cudaStreamQuery(ctx->d2h_stream) : cudaSuccess;
        if (e1 == cudaSuccess && e2 == cudaSuccess && e3 == cudaSuccess) break;
        (void)cudaGetLastError();  // "not ready" is recorded as the thread's last error; a later launch check must not see it
        for (cudaError_t e : {e1, e2, e3})
            if (e != cudaSuccess && e != cudaErrorNotReady) RING_CUDA(e);
        if (std::chrono::steady_clock::now() >= deadline)
            return fail(RING_ERR_HOST_TIMEOUT, "the forward did not finish within %d ms (%s%s%s still pending)", timeout_ms,
                        e1 != cudaSuccess ? "compute " : "", e2 != cudaSuccess ? "exchange " : "", e3 != cudaSuccess ? "copy-out " : "");
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    // everything this context enqueued is done: read the status word without a device-wide synchronisation
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    int status = 0;
    RING_CUDA(cudaMemcpyAsync(&status, st->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->comm_stream));
    RING_CUDA(cudaStreamSynchronize(ctx->comm_stream));
    if (ctx->comm) {
        ncclResult_t async = ncclSuccess;
        RING_NCCL(nccl().CommGetAsyncError(ctx->comm, &async));
        if (async != ncclSuccess) return fail(RING_ERR_NCCL, "NCCL async error: %s", nccl().GetErrorString(async));
    }
    if (status != 0) return fail(RING_ERR_DEVICE_TIMEOUT, "a bounded wait inside a kernel ran out (device status %d)", status);
    return RING_OK;
}

// Way out after ring_ctx_synchronize_timeout() gave up (a peer stopped, so a queued wait will never be satisfied).
// Every cross-process wait this context queues is a stream wait on a word of ITS OWN flag block, compared with >=
// against the call's sequence number (a cyclic comparison, (int32)(word - seq) >= 0): storing a value 2^30 ahead
// of the current sequence number into every word from the host releases them all, and the queued copies and kernels then drain (into receive buffers that are still mapped -- peers must
// keep theirs alive until this rank has destroyed its context).  The NCCL communicator is aborted, not destroyed
// (ncclCommDestroy waits for outstanding operations).  The context is dead afterwards: forwards are refused and
// ring_ctx_destroy() frees it without a device-wide synchronisation.  Results of the aborted forward are undefined.
int ring_ctx_abort(RingCtx* c) {
    if (!c) return fail(RING_ERR_INVALID_ARGUMENT, "null context");
    if (c->dead) return RING_OK;
    c->dead = true;
    if (c->flags) {
        // The flag block is device memory; the store must not queue behind the stuck streams.  A blocking copy on a
        // fresh non-blocking stream is independent of them.
        std::vector<uint32_t> all(2 * kMaxWorld, c->call_seq + 0x40000000u);
        cudaStream_t s = nullptr;
        RING_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        cudaError_t e = cudaMemcpyAsync(c->flags, all.data(), all.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        cudaStreamDestroy(s);
        RING_CUDA(e);
    }
    if (c->comm) {
        nccl().CommAbort(c->comm);
        c->comm = nullptr;
    }
    return RING_OK;
}

// The exchange of step i split in two: wait_ms[i] is the time its stream waited for the go-ahead (peer-copy: the
// destination's credit flag; NCCL: the compute step that last read the receive buffer), copy_ms[i] the transfer
// itself (for the peer-copy transport: this rank's PUSH of its own shard).  Needs RING_OPT_RECORD_TIMINGS.
int ring_ctx_get_exchange_timings(RingCtx* c, float* wait_ms, float* copy_ms, int n) {
    if (!c || !wait_ms || !copy_ms) return fail(RING_ERR_INVALID_ARGUMENT, "null argument");
    if (!c->record_timings) return fail(RING_ERR_INVALID_ARGUMENT, "RING_OPT_RECORD_TIMINGS is off");
    if (n < c->last_steps) return fail(RING_ERR_INVALID_ARGUMENT, "arrays too short: %d < %d", n, c->last_steps);
    const int P = c->last_steps;
    for (int s = 0; s < P; ++s) {
        wait_ms[s] = copy_ms[s] = 0.f;
        if (s < P - 1) {
            RING_CUDA(cudaEventElapsedTime(&wait_ms[s], c->ev_comm_start[s], c->ev_copy_start[s]));
            RING_CUDA(cudaEventElapsedTime(&copy_ms[s], c->ev_copy_start[s], c->ev_recv_done[s]));
        }
    }
    return RING_OK;
}

int ring_ctx_get_timings(RingCtx* c, float* compute_ms, float* comm_ms, float* exposed_ms, int n) {
    if (!c || !compute_ms || !comm_ms || !exposed_ms) return fail(RING_ERR_INVALID_ARGUMENT, "null argument");
    if (!c->record_timings) return fail(RING_ERR_INVALID_ARGUMENT, "RING_OPT_RECORD_TIMINGS is off");
    if (n < c->last_steps) return fail(RING_ERR_INVALID_ARGUMENT, "arrays too short: %d < %d", n, c->last_steps);
    const int P = c->last_steps;
    for (int s = 0; s < P; ++s) {
        compute_ms[s] = comm_ms[s] = exposed_ms[s] = 0.f;
        RING_CUDA(cudaEventElapsedTime(&compute_ms[s], c->ev_compute_start[s], c->ev_compute_done[s]));
        if (s < P - 1) {
            RING_CUDA(cudaEventElapsedTime(&comm_ms[s], c->ev_comm_start[s], c->ev_recv_done[s]));
            // idle gap of the compute stream between the end of step s and the start of step s + 1
            RING_CUDA(cudaEventElapsedTime(&exposed_ms[s], c->ev_compute_done[s], c->ev_compute_start[s + 1]));
        }
    }
    return RING_OK;
}

int ring_attention_block_fwd(const void* q, const void* k, const void* v, float* o, float* lse, int batch, int heads,
                             int sq, int sk, int dim, float softmax_scale, int causal, int64_t q_off, int64_t k_off,
                             int merge, int is_bf16, void* stream) {
    BlockLaunch L;
    L.q = q; L.k = k; L.v = v; L.o = o; L.lse = lse;
    L.batch = batch; L.heads = heads; L.sq = sq; L.sk = sk; L.dim = dim;
    L.scale = softmax_scale; L.causal = causal; L.q_off = q_off; L.k_off = k_off;
    L.merge = merge; L.is_bf16 = is_bf16;
    return launch_block(L, static_cast<cudaStream_t>(stream));
}

int ring_lse_merge(float* o_acc, float* lse_acc, const float* o_part, const float* lse_part, int64_t rows, int dim,
                   void* stream) {
    return launch_merge(o_acc, lse_acc, o_part, lse_part, rows, dim, static_cast<cudaStream_t>(stream));
}

int ring_attention_scaled(const void* q, const void* k, const void* v, float* out, int npes, int mype,
                          const int* seqlen, int dim, int max_seq, float softmax_scale) {
    if (!seqlen) return fail(RING_ERR_INVALID_ARGUMENT, "null seqlen table");
    if (npes < 1 || mype < 0 || mype >= npes) return fail(RING_ERR_INVALID_ARGUMENT, "bad npes/mype %d/%d", npes, mype);
    if (max_seq > 0 && seqlen[mype] > max_seq) return fail(RING_ERR_INVALID_ARGUMENT, "seqlen exceeds max_seq");
    RingCtx* c = g_default_ctx;
    if (!c) {
        if (npes > 1)
            return fail(RING_ERR_NO_CONTEXT, "ring_attention with npes > 1 needs ring_set_default_ctx() first");
        if (!g_solo_ctx) {
            int rc = ring_ctx_create(&g_solo_ctx, 0, 1, nullptr);
            if (rc) return rc;
        }
        c = g_solo_ctx;
    }
    Ring_fwd_params params;
    set_params_fprop(params, q, k, v, out, npes, mype, seqlen, dim, max_seq);
    params.softmax_scale = softmax_scale;
    int rc = ring_attention_fwd(c, &params);
    if (rc) return rc;
    return ring_ctx_synchronize(c);  // the reference call is synchronous (csrc/ring_attention.cu:721)
}

int ring_attention(const void* q, const void* k, const void* v, float* out, int npes, int mype, const int* seqlen,
                   int dim, int max_seq) {
    const float scale = dim > 0 ? 1.0f / std::sqrt(static_cast<float>(dim)) : 1.0f;
    return ring_attention_scaled(q, k, v, out, npes, mype, seqlen, dim, max_seq, scale);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------ no-allocation entry point
// Chunked attention whose partial-result scratch lives in a fixed device array of this library instead
// of in memory obtained from the CUDA allocator.  See include/ring_attention_b200.h for who needs it.
//
// Layout of the array (floats): [0, 64) header, word 0 = device status of this path;
// [64, 64 + 65536) row LSE of the partial; then 4 Mi floats for the partial output.
namespace {

constexpr int64_t kStaticHeaderFloats = 64;
constexpr int64_t kStaticMaxRows = RING_STATIC_MAX_ROWS;
constexpr int64_t kStaticMaxOutElems = RING_STATIC_MAX_OUT_ELEMS;

}  // namespace

static __device__ __align__(256) float g_static_scratch[kStaticHeaderFloats + kStaticMaxRows + kStaticMaxOutElems];

namespace {

struct StaticSetup {
    float* base = nullptr;  // DEVICE address of g_static_scratch on this device (the symbol itself is a host-side stand-in)
    bool attr_set[12] = {};
    int sm_count = 0;
};
std::mutex g_static_mutex;
StaticSetup g_static[64];

// Once per device, with that device current: resolve the device address of the array and read the SM count
// (neither call allocates).
int static_setup(StaticSetup** out) {
    int dev = 0;
    RING_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(RING_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticSetup& s = g_static[dev];
    if (!s.base) {
        void* p = nullptr;
        RING_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return fail(RING_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        RING_CUDA(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
        s.base = static_cast<float*>(p);
    }
    *out = &s;
    return RING_OK;
}

}  // namespace

extern "C" int ring_attention_chunked_fwd_static(const void* q, const void* k, const void* v, float* o, float* lse,
                                                 int batch, int heads, int sq, int sk, int dim, float softmax_scale,
                                                 int causal, int kv_chunk, int is_bf16, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    BlockLaunch whole;
    whole.q = q; whole.k = k; whole.v = v; whole.o = o; whole.lse = lse;
    whole.batch = batch; whole.heads = heads; whole.sq = sq; whole.sk = sk; whole.dim = dim;
    whole.scale = softmax_scale; whole.causal = causal; whole.q_off = 0; whole.k_off = 0; whole.merge = 0;
    whole.is_bf16 = is_bf16;
    int rc = validate_block(whole);
    if (rc) return rc;
    if (kv_chunk <= 0 || kv_chunk % 128 != 0)
        return fail(RING_ERR_INVALID_ARGUMENT, "kv_chunk must be a positive multiple of 128, got %d", kv_chunk);
    const int64_t rows = static_cast<int64_t>(batch) * heads * sq;
    if (rows > kStaticMaxRows || rows * dim > kStaticMaxOutElems)
        return fail(RING_ERR_INVALID_ARGUMENT,
                    "batch*heads*sq = %lld rows (x dim = %lld floats) exceeds the fixed scratch of this entry point "
                    "(%lld rows, %lld floats)", (long long)rows, (long long)(rows * dim), (long long)kStaticMaxRows,
                    (long long)kStaticMaxOutElems);
    StaticSetup* s = nullptr;
    if ((rc = static_setup(&s))) return rc;
    float* lse_part = s->base + kStaticHeaderFloats;
    float* o_part = lse_part + kStaticMaxRows;
    // The array keeps whatever the previous call left: the status word must start at zero (a stale error
    // would make every CTA return at once).  The partials need no clearing: every row is written by the
    // block kernel before the merge reads it.
    RING_CUDA(cudaMemsetAsync(s->base, 0, sizeof(int), stream));

    const LaunchEnv env{reinterpret_cast<int*>(s->base) /* header word 0 */, s->attr_set, s->sm_count};
    for (int c0 = 0; c0 < sk; c0 += kv_chunk) {
        BlockLaunch L = whole;  // K/V rows [c0, c0 + rows) of every (batch, head) slab of sk rows
        L.k = static_cast<const char*>(k) + static_cast<size_t>(c0) * dim * 2;
        L.v = static_cast<const char*>(v) + static_cast<size_t>(c0) * dim * 2;
        L.sk = (sk - c0) < kv_chunk ? (sk - c0) : kv_chunk;
        L.k_rows_total = sk;
        L.k_off = c0;
        L.o = c0 == 0 ? o : o_part;
        L.lse = c0 == 0 ? lse : lse_part;
        if ((rc = launch_block_env(L, env, stream))) return rc;
        if (c0 > 0 && (rc = launch_merge(o, lse, o_part, lse_part, rows, dim, stream, s->sm_count))) return rc;
    }
    return RING_OK;
}

extern "C" int ring_static_status(int* status_out, void* stream_) {
    if (!status_out) return fail(RING_ERR_INVALID_ARGUMENT, "null status_out");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    StaticSetup* s = nullptr;
    int rc = static_setup(&s);
    if (rc) return rc;
    RING_CUDA(cudaMemcpyAsync(status_out, s->base, sizeof(int), cudaMemcpyDeviceToHost, stream));
    RING_CUDA(cudaStreamSynchronize(stream));
    return RING_OK;
}

#ifdef RING_TRACE
extern "C" int ring_debug_set_trace(long long* buf) { g_trace = buf; return 0; }
#endif
