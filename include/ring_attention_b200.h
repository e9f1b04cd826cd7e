/*
 * C ABI of the B200 ring-attention forward.  Plain pointers and sizes only; no torch, CUDA C++ or
 * CuTe types cross this boundary (cudaStream_t and ncclUniqueId travel as void* / byte arrays).
 *
 * Each entry point cites the interface of ykcombat/RingAttention it stands in for.  The reference
 * exports no C symbols at all: its include/attention_api.cuh holds macros only and its operator
 * boundary is the C++ function ring_attention() at csrc/ring_attention.cu:706.
 *
 * Conventions
 *   - every function returns 0 on success or a negative RingStatus; nothing calls exit()
 *     (the reference prints and exits, csrc/utils.h:1-11);
 *   - device tensors are contiguous: Q, K, V  [batch, heads, seqlen_local, dim] fp16 (or bf16),
 *     O [batch, heads, seqlen_local, dim] fp32, LSE [batch, heads, seqlen_local] fp32 (natural log);
 *     per (batch, head) this is the reference's [seqlen, dim] row-major matrix
 *     (csrc/ring_attention.cu:422-454); all base pointers 16-byte aligned;
 *   - dim is 64 or 128; every rank holds at least one row; shard lengths need neither be equal (seqlen[] per PE as
 *     in csrc/ring.h:9) nor multiples of the 128-row tile (the reference has no tail predication);
 *   - one process per GPU; a context belongs to the device that was current when it was created.
 */
#ifndef RING_ATTENTION_B200_H_
#define RING_ATTENTION_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum RingStatus {
    RING_OK = 0,
    RING_ERR_INVALID_ARGUMENT = -1, /* null pointer, dim not in {64,128}, non-positive length or scale, misaligned base ... */
    RING_ERR_CUDA = -2,             /* a CUDA runtime/driver call failed; see ring_last_error_string() */
    RING_ERR_NCCL = -3,             /* an NCCL call failed or NCCL could not be loaded */
    RING_ERR_DEVICE_TIMEOUT = -4,   /* a bounded wait inside a kernel ran out; the device status word says which */
    RING_ERR_NO_CONTEXT = -5,       /* ring_attention() with npes > 1 before ring_set_default_ctx() */
    RING_ERR_UNSUPPORTED = -6,
    RING_ERR_HOST_TIMEOUT = -7      /* ring_ctx_synchronize_timeout: the deadline passed with work still pending */
} RingStatus;

#define RING_UNIQUE_ID_BYTES 128

typedef struct RingCtx RingCtx; /* opaque: communicator, side stream, events, receive buffers, workspace */

struct Ring_fwd_params; /* csrc/ring.h of this repository: the reference's struct (csrc/ring.h:5-19) plus extensions */

/* How the cross-step merge runs (ring_ctx_set_option(ctx, RING_OPT_MERGE_MODE, v)). */
#define RING_MERGE_SEPARATE_KERNEL 0 /* block kernel writes a partial, ring_lse_merge folds it in */
#define RING_MERGE_FUSED_EPILOGUE 1  /* block kernel folds its tile into the running result itself */

#define RING_OPT_MERGE_MODE 1
#define RING_OPT_CAUSAL_SKIP_EXCHANGE 2 /* 1 (default): under a causal mask, do not ship shards nobody will read */
#define RING_OPT_RECORD_TIMINGS 3       /* 1: record per-step events so ring_ctx_get_timings() works */
#define RING_OPT_TRANSPORT 4            /* how K/V shards travel between ranks, see below */
#define RING_OPT_CAUSAL_ZIGZAG 5        /* 1: causal calls assume zig-zag sharding: the sequence is cut into 2*npes chunks
                                           and rank r holds chunks r and 2*npes-1-r, in that order, in its q/k/v/out/lse.
                                           Contiguous causal sharding (the default) makes rank r do (r + 1/2) / npes of the
                                           work; zig-zag gives every rank the same.  Needs equal, even shard lengths. */

#define RING_OPT_RECV_BUFFERS 6         /* receive buffers of the exchange: 2 (default, a double buffer: an exchange waits until
                                           the compute step that last read its buffer is done) ... world - 1, or 0 = one per
                                           remote shard (no exchange ever waits for a compute step; (world - 1) x the K/V
                                           shard in memory).  Collective: every rank must use the same value. */

/* Transports of the K/V exchange.  Both keep the same schedule (ring_step_plan) and the same double buffer.
 *   NCCL:      ncclSend/ncclRecv on the exchange stream (what the reference's NCCL prototype does,
 *              test/ring_attention_with_nccl.cu:153-156).  NCCL's copy kernels occupy SMs next to the block kernel.
 *   PEER_COPY: each rank pushes its shard into the destination's receive buffer with a device-to-device copy over
 *              NVLink (copy engines, no SMs); buffers are shared through CUDA IPC and ordered with stream memory
 *              operations.  Default when the ranks can map each other's memory; NCCL otherwise.
 * The environment variable RING_TRANSPORT=nccl|peer chooses at context creation; the option switches later
 * (collectively: all ranks must switch between the same two calls). */
#define RING_TRANSPORT_NCCL 0
#define RING_TRANSPORT_PEER_COPY 1

/*
 * Replaces: ring_attention(FPC* q, FPC* k, FPC* v, float* out, int npes, int mype, int* seqlen,
 *                          int dim, int max_seq)                    -- csrc/ring_attention.cu:706-722
 * Same argument order and meaning: single batch, single head, q/k/v [seqlen[mype], dim] fp16 device
 * pointers, out [seqlen[mype], dim] fp32 device pointer, seqlen a HOST array of npes entries,
 * max_seq an upper bound on them.  Non-causal.  Synchronous like the reference
 * (which ends in cudaDeviceSynchronize, :721).  The softmax scale is 1/sqrt(dim) in the natural
 * base (the reference's kernel applies exp2 with scale 1, csrc/ring_attention.cu:389,597, which
 * disagrees with its own PyTorch check csrc/self_attention.py:22-26; see ring_attention_scaled).
 * With npes > 1 the exchange runs over the context registered by ring_set_default_ctx().
 */
int ring_attention(const void* q, const void* k, const void* v, float* out, int npes, int mype,
                   const int* seqlen, int dim, int max_seq);

/* Same call with an explicit natural-base softmax scale (1.0 gives csrc/self_attention.py:22-26). */
int ring_attention_scaled(const void* q, const void* k, const void* v, float* out, int npes, int mype,
                          const int* seqlen, int dim, int max_seq, float softmax_scale);

/*
 * Replaces: nvshmem_init / nvshmem_my_pe / nvshmem_n_pes and the symmetric allocations of
 * csrc/ring_attention.cu:754-761 and :391-393 (k_buffer / v_buffer allocated per call and leaked).
 * ring_get_unique_id: rank 0 obtains RING_UNIQUE_ID_BYTES bytes and hands them to the other ranks by any
 * host channel.  ring_ctx_create: collective over `world` processes; owns the NCCL communicator, the
 * exchange stream, events and (grown on demand, never per call in steady state) the two receive
 * buffers and the partial-result workspace.  world == 1 needs no id (pass NULL) and no NCCL.
 */
int ring_get_unique_id(void* id_out);
int ring_ctx_create(RingCtx** ctx, int rank, int world, const void* unique_id);
int ring_ctx_destroy(RingCtx* ctx);
int ring_ctx_set_option(RingCtx* ctx, int option, int value);
int ring_ctx_get_option(RingCtx* ctx, int option, int* value);
int ring_set_default_ctx(RingCtx* ctx); /* context used by ring_attention(); NULL clears it */

/*
 * Single-process stand-in for the multi-process launch of the reference (`nvshmrun -n 2`, makefile:2):
 * `world` virtual ranks share one GPU and the exchange is a device-to-device copy on the exchange
 * stream.  The caller registers every virtual rank's K and V shard, then calls ring_attention_fwd()
 * once per virtual rank (params.mype selects it).  Used to test the ring schedule on one GPU.
 */
int ring_ctx_create_local(RingCtx** ctx, int world);
int ring_ctx_set_local_shards(RingCtx* ctx, const void* const* k_shards, const void* const* v_shards);

/*
 * Replaces: set_params_fprop + run_ring_fwd<Traits> (csrc/ring_attention.cu:361-395, 669-704), i.e. the
 * whole ring loop of ring_attention_kernel (:456-619) with batch, heads, causal mask and LSE output.
 * Asynchronous on params->stream.  Step i attends to the shard of rank (mype + i) % npes
 * (csrc/ring_attention.cu:463); while it computes, the shard for step i + 1 arrives on the exchange stream.
 */
int ring_attention_fwd(RingCtx* ctx, const struct Ring_fwd_params* params);

/*
 * Same forward for callers whose tensors live in (pinned) HOST memory, as the reference's driver fills them
 * (initQKV, csrc/ring_attention.cu:731-748, builds on the host and copies).  q/k/v/out/lse of `params` are host
 * pointers; the (batch, head) slabs are processed in `chunks` groups so that the copy in of one group, the ring
 * forward of the previous and the copy out of the one before overlap.  Collective like ring_attention_fwd
 * (every rank: same shapes, same chunks).  Asynchronous on params->stream: when that stream reaches the end of the
 * call, the results are in the host buffers.
 */
int ring_attention_fwd_host(RingCtx* ctx, const struct Ring_fwd_params* params, int chunks);

/*
 * The schedule run_ring_fwd follows, as pure host logic (no GPU needed): step `step` of rank `rank`.
 * Restates the loop header of ring_attention_kernel (csrc/ring_attention.cu:456-470, 611-619): the shard
 * visited at step i is that of PE (mype + i) % npes, fetched from its origin PE.
 */
typedef struct RingStepPlan {
    int src_rank;       /* whose K/V shard this step attends to */
    int compute;        /* 0 if the shard is fully masked for this rank (causal) */
    int compute_buffer; /* -1: the rank's own shard; else index of the receive buffer holding the shard */
    int recv_buffer;    /* receive buffer the concurrent exchange fills (step & 1) */
    int recv_from;      /* origin rank of the shard for step + 1, or -1 on the last step */
    int send_to;        /* rank that receives this rank's shard meanwhile, or -1 */
    int do_recv;        /* 0 if the arriving shard would never be read (causal skip) */
    int do_send;
} RingStepPlan;
int ring_step_plan(int world, int rank, int step, int causal, int causal_skip_exchange, RingStepPlan* out);

/* Blocks until everything the context has enqueued is done and returns the device status
 * (RING_OK or RING_ERR_DEVICE_TIMEOUT / RING_ERR_CUDA). */
int ring_ctx_synchronize(RingCtx* ctx);

/*
 * The same with a deadline, for failure detection on the host: polls the completion of the last forward, the
 * exchange stream and the copy-out stream without blocking on the device, and returns RING_ERR_HOST_TIMEOUT if
 * they are not all done after timeout_ms (a peer that stopped, a stream blocked upstream).  The context is left
 * untouched; calling again waits further.  timeout_ms < 0 waits without limit.  No counterpart in the reference,
 * which ends every call in cudaDeviceSynchronize (csrc/ring_attention.cu:721) and so hangs with its peer.
 */
int ring_ctx_synchronize_timeout(RingCtx* ctx, int timeout_ms);

/*
 * Per-step timings of the last ring_attention_fwd() (needs RING_OPT_RECORD_TIMINGS = 1 and a prior
 * ring_ctx_synchronize()).  Arrays of `n` >= npes floats, milliseconds:
 *   compute_ms[i]  block kernel (+ merge) of step i;   comm_ms[i]  exchange posted during step i;
 *   exposed_ms[i]  time step i + 1 had to wait for that exchange after step i's compute was done.
 * Stands in for the cudaEvent timing of the reference driver (csrc/ring_attention.cu:773-783).
 */
int ring_ctx_get_timings(RingCtx* ctx, float* compute_ms, float* comm_ms, float* exposed_ms, int n);

/*
 * The exchange of step i in two parts (same preconditions as ring_ctx_get_timings): wait_ms[i], the time the
 * exchange stream waited for its go-ahead (peer-copy transport: the destination's "buffer free" flag; NCCL
 * transport: the compute step that last read the receive buffer), and copy_ms[i], the transfer itself (peer-copy
 * transport: this rank's push of its own shard).  Bytes moved per step / copy_ms is the achieved link rate.
 * No counterpart in the reference (its NVSHMEM get is inside the kernel, csrc/ring_attention.cu:611-619).
 */
int ring_ctx_get_exchange_timings(RingCtx* ctx, float* wait_ms, float* copy_ms, int n);

/*
 * Tear-down after a detected failure (ring_ctx_synchronize_timeout returned RING_ERR_HOST_TIMEOUT because a peer
 * stopped): releases, from the host, every stream wait this context has queued on its own flag block, aborts the
 * NCCL communicator (ncclCommAbort) and marks the context dead.  Later forwards on it return RING_ERR_UNSUPPORTED;
 * ring_ctx_destroy() then frees it without a device-wide synchronisation.  Outputs of the aborted forward are
 * undefined.  Peers that are still alive must keep their contexts (their receive buffers) until this rank has
 * destroyed its own: the released copies still land there.  No counterpart in the reference, which hangs with its
 * peer (every call ends in cudaDeviceSynchronize, csrc/ring_attention.cu:721).
 */
int ring_ctx_abort(RingCtx* ctx);

/*
 * Replaces: one pass of the flash inner loop of ring_attention_kernel over ONE source shard
 * (csrc/ring_attention.cu:536-609) plus the final normalisation (:621-664).
 * q [B,H,Sq,D], k/v [B,H,Sk,D] -> o [B,H,Sq,D] fp32, lse [B,H,Sq] fp32.  q_off / k_off are the global
 * sequence indices of row 0 of each shard (causal mask: k_off + j <= q_off + i).
 * merge = 0 overwrites o / lse; merge = 1 folds the result into the partial they already hold.
 * Asynchronous on `stream` (a cudaStream_t passed as void*; NULL = default stream).
 */
int ring_attention_block_fwd(const void* q, const void* k, const void* v, float* o, float* lse, int batch,
                             int heads, int sq, int sk, int dim, float softmax_scale, int causal,
                             int64_t q_off, int64_t k_off, int merge, int is_bf16, void* stream);

/*
 * Replaces: the implicit cross-step accumulation of csrc/ring_attention.cu:439-443, 597-598, 621-633
 * (running max / sum / O kept in registers across PEs) as a standalone pass over memory:
 * (o_acc, lse_acc) <- merge((o_acc, lse_acc), (o_part, lse_part)) for `rows` rows of `dim` floats.
 */
int ring_lse_merge(float* o_acc, float* lse_acc, const float* o_part, const float* lse_part, int64_t rows,
                   int dim, void* stream);

/*
 * No counterpart in the reference (which allocates inside every call, csrc/ring_attention.cu:384-393).
 *
 * Attention of q [B,H,Sq,D] against k/v [B,H,Sk,D] taken kv_chunk key rows at a time: the first chunk
 * writes o / lse, every further chunk is computed into a scratch partial and folded in by the merge
 * kernel -- the same two kernels and the same arithmetic as one ring step followed by ring_lse_merge,
 * so the result equals ring_attention_block_fwd over the whole K/V up to merge rounding.  Causal masks
 * keys with index j > i (row 0 of q and of k are the same sequence position).
 *
 * This variant exists for hosts that hand a component its tensors but do not let it obtain device memory
 * of its own: a serving runtime that reserved the whole GPU at start-up and gives plug-ins no allocator,
 * or a process pinned to a fixed memory budget, where cudaMalloc either fails or stalls every stream with
 * its implicit synchronisation.  The function calls no cudaMalloc / cudaFree and no allocating library
 * routine.  Its scratch is a fixed array inside this library's device image (about 16.3 MiB, held by
 * every GPU that loads the library until the process exits), which bounds the problem size:
 *     batch * heads * sq        <= RING_STATIC_MAX_ROWS        (65536 rows)
 *     batch * heads * sq * dim  <= RING_STATIC_MAX_OUT_ELEMS   (4 Mi floats)
 * Larger calls are refused with RING_ERR_INVALID_ARGUMENT and a message naming the limit.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress) and sets the
 * kernel's shared-memory attribute; make that first call before any stream capture begins.
 * All calls on a device share the one array and it keeps the last call's contents: the function clears
 * the status word it needs at zero itself, but two calls whose kernels overlap on the GPU (different
 * streams, no ordering between them) race on the partials and give wrong results.  Serialise them.
 * A bounded wait that runs out inside a kernel of this path is recorded in the array's own status word,
 * not in the word ring_device_status() reads; ring_static_status() reads it.  When it is non-zero the
 * outputs of that call are not valid.
 * Asynchronous on `stream` (cudaStream_t as void*).
 */
#define RING_STATIC_MAX_ROWS 65536
#define RING_STATIC_MAX_OUT_ELEMS (4 * 1024 * 1024)
int ring_attention_chunked_fwd_static(const void* q, const void* k, const void* v, float* o, float* lse,
                                      int batch, int heads, int sq, int sk, int dim, float softmax_scale,
                                      int causal, int kv_chunk, int is_bf16, void* stream);

/*
 * No counterpart in the reference.  Status word of the no-allocation path on the current device: waits for
 * `stream` (the one the call above was given), then stores in *status_out 0 or the code (1xx) of the bounded
 * wait that ran out inside the last ring_attention_chunked_fwd_static().  Allocates nothing either.
 */
int ring_static_status(int* status_out, void* stream);

/* Device status word of the current device: 0, or the code of the bounded wait that ran out
 * (1xx, see csrc/block_attention.cuh).  ring_device_status synchronises the device. */
int ring_device_status(int* status_out);
int ring_device_status_reset(void);

/*
 * Failure detection without a device fault.  ring_device_status_inject stores a code in the status word from the
 * host, as a timed-out kernel would; ring_selftest_wait_timeout runs the kernels' bounded wait on a barrier that
 * nothing completes and returns what it recorded and how long it waited (about two seconds).  No counterpart in
 * the reference, whose device code can only hang (its grid barrier is commented out, csrc/ring_attention.cu:457-459).
 */
int ring_device_status_inject(int code);
int ring_selftest_wait_timeout(int code, int* status_out, float* waited_ms);

/* Number of kernels this library has launched in this process (block + merge), for accounting. */
int64_t ring_kernel_launch_count(void);

/* Thread-local description of the last error returned to this thread. */
const char* ring_last_error_string(void);

#ifdef __cplusplus
}
#endif

#endif /* RING_ATTENTION_B200_H_ */
