// Block-attention kernel for sm_100a: one Q shard against one K/V shard.
//
// It replaces the reference's ring_attention_kernel (csrc/ring_attention.cu:398-666) for ONE ring
// step: S = Q K^T (:565), online softmax (:597, helpers :172-245), P = fp16(S) (:604), O += P V (:609),
// final O / l (:621-633).  Where the reference keeps the running (max, sum, O) in registers across
// ring steps, this kernel emits the step's normalised output tile together with its row
// log-sum-exp, and can fold the result into an earlier partial (merge != 0) with the same algebra as
// the standalone merge kernel.
//
// Mapping to the hardware
//   * a CTA owns two 128-row Q tiles of one (batch, head) and walks the K/V shard in 128-row blocks (one
//     tile per CTA when the two-tile grid would leave more than half of the SMs idle, args.rows_per_cta);
//   * one thread issues TMA loads (Q once, then K_j and V_j through two rings of shared-memory slots,
//     128-byte swizzle, 64-element boxes);
//   * three threads of three warps issue tcgen05.mma, because inside this kernel one thread gets only about one
//     128x128x16 instruction out per 100-115 clocks (its warp shares a scheduler with two softmax warps; alone on
//     an SM the same thread issues one per ~76, the pipe's own rate at M = 128).  The first issues S_t = Q_t K_j^T for both
//     tiles (both operands K-major in shared memory, N = 128: a narrower N would re-read Q from shared memory,
//     whose ~75 B/clock operand bandwidth is what bounds these instructions) into ONE S buffer of 128 TMEM
//     columns that the two Q tiles use in turn; the other two issue O_t += P_t V_j for tile 0 / 1, reading P_t
//     from its own 64 TMEM columns (16-bit pairs) and V_j MN-major from shared memory, so V is never transposed
//     (the reference needs ldmatrix.trans, csrc/kernel_traits.h:39,93-103) and the PV product spends no
//     shared-memory bandwidth on its A operand;
//   * two softmax warpgroups (one per Q tile, one thread per row = one TMEM lane).  A warpgroup reads its
//     S_t(j) into registers and hands the S buffer to the other tile at once; because P has columns of its
//     own, S_t(j+1) is computed while the OTHER tile runs its softmax, and the serial chain per tile is
//     softmax -> softmax rather than softmax -> PV -> QK^T.  The tiles settle half a period apart, which also
//     keeps their exponentials from competing for the MUFU all the time.  Running max / sum live in
//     registers; a new maximum is adopted only when it exceeds the one in use by more than 2^8 (the stale
//     maximum is exact algebra: it cancels in O / l and in the LSE), and then O is rescaled in TMEM;
//   * the producer warpgroup gives registers back (setmaxnreg) and the softmax warpgroups take them, so a
//     whole S row plus its packed probabilities stay in registers without spilling;
//   * the epilogue stages O through the Q tile's shared memory so that global stores (and, when folding into
//     an earlier partial, loads) cover whole row pieces.
// Every mbarrier wait is bounded (ptx::mbar_wait); on expiry the CTA records a status code, all roles
// fall through to the common exit and TMEM is released.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel_traits.h"
#include "ptx_sm100.cuh"

namespace ring {

// Values of the device status word (0 = no error).  1xx: a wait of the named role ran out.
enum DeviceStatus : int {
    kDevOk = 0,
    kDevLoadWaitEmpty = 101,
    kDevMmaWaitQ = 111,
    kDevMmaWaitKV = 112,
    kDevMmaWaitP = 113,
    kDevMmaWaitS = 114,
    kDevSoftmaxWaitS = 121,
    kDevSoftmaxWaitO = 122,
    kDevSoftmaxWaitM = 123,  // pair form: the row maximum handed over by the other warpgroup
};

struct BlockFwdArgs {
    float* o;    // [B, H, Sq, D] fp32
    float* lse;  // [B, H, Sq] fp32 (natural log)
    int64_t o_batch_stride, o_head_stride, o_row_stride;  // in elements
    int64_t lse_batch_stride, lse_head_stride;
    int heads;
    int sq;           // Q rows in the shard
    int sk;           // K/V rows in the shard
    float scale;      // natural-base softmax scale
    float scale_log2; // scale * log2(e)
    int causal;       // key j of the shard is visible to query i of the shard iff j <= i + diag
    int diag;         // (global index of Q row 0) - (global index of K row 0)
    int merge;        // 0: overwrite o/lse; 1: o/lse already hold a partial of the same rows, fold into it
    int rows_per_cta; // 256 (two Q tiles per CTA) or 128 (one tile: twice the CTAs, for grids that would leave SMs idle)
    int* status;      // device status word
#ifdef RING_TRACE
    long long* trace;  // debug builds only: clock64 stamps of CTA (0,0), 32 slots per K/V block
#endif
};

#ifdef RING_TRACE
#define RING_TRACE_STAMP(cond, slot) do { if ((cond) && a.trace && blockIdx.x == 0 && blockIdx.y == 0) a.trace[j * 32 + (slot)] = clock64(); } while (0)
#define RING_TRACE_LIFE(cond, k) do { if ((cond) && a.trace) { const int w_ = (blockIdx.x == 0 && blockIdx.y == 0) ? 0 : ((blockIdx.x == 16 && blockIdx.y == 20) ? 1 : -1); if (w_ >= 0) a.trace[((a.sk + 127) / 128) * 32 + 16 * w_ + (k)] = clock64(); } } while (0)
#else
#define RING_TRACE_STAMP(cond, slot) do { } while (0)
#define RING_TRACE_LIFE(cond, k) do { } while (0)
#endif

constexpr float kRescaleThresholdLog2 = 8.0f;
template <class T>
__global__ void __launch_bounds__(T::kNThreads, 1)
ring_block_attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_v, const BlockFwdArgs a) {
    using namespace ptx;
    constexpr int D = T::kHeadDim;
    constexpr int kStages = T::kStages;
    constexpr int kTileBytes = T::kTileBytes;
    constexpr int kBoxBytes = T::kBoxBytes;
    constexpr int kBoxes = T::kBoxesPerTile;
    constexpr uint32_t kIdescQK = umma_idesc_f16(128, T::kBlockN, false, false, T::kIsBf16);
    constexpr uint32_t kIdescPV = umma_idesc_f16(128, D, false, true, T::kIsBf16);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
    uint8_t* smem = smem_raw + (base - raw_addr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::kSmemTiles);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + T::kNumBarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* prior_error = reinterpret_cast<volatile int*>(tmem_slot + 2);

    const uint32_t bar0 = smem_u32(bars);
    auto bar_q_full = [&](int t) { return bar0 + 8u * t; };
    auto bar_kv_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto bar_kv_empty = [&](int s) { return bar0 + 8u * (2 + kStages + s); };
    auto bar_s_full = [&](int t) { return bar0 + 8u * (2 + 2 * kStages + t); };
    auto bar_p_full = [&](int t) { return bar0 + 8u * (4 + 2 * kStages + t); };
    auto bar_o_done = [&](int t) { return bar0 + 8u * (6 + 2 * kStages + t); };
    const uint32_t bar_s_free = bar0 + 8u * (8 + 2 * kStages);  // the shared S buffer has been read out
    auto smem_q = [&](int t) { return base + static_cast<uint32_t>(t * kTileBytes); };
    auto smem_kv = [&](int s) { return base + static_cast<uint32_t>((T::kQTiles + s) * kTileBytes); };

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    RING_TRACE_LIFE(tid == 0, 0);

    // Under a causal mask the CTAs of the last Q rows have the most K/V blocks to visit: launch them first.
    const int r0 = (a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x) * a.rows_per_cta;  // first Q row of this CTA
    const bool tile1_valid = a.rows_per_cta > 128 && (r0 + 128) < a.sq;
    const int ntiles = tile1_valid ? 2 : 1;

    if (tid == 0) {
        *abort_flag = 0;
        *prior_error = *reinterpret_cast<volatile int*>(a.status);
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_q_full(t), 1);
            mbar_init(bar_s_full(t), 1);
            mbar_init(bar_p_full(t), 4);  // one arrival per softmax warp
            mbar_init(bar_o_done(t), 1);
        }
        mbar_init(bar_s_free, 4);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_kv_full(s), 1);
            mbar_init(bar_kv_empty(s), ntiles);  // one tcgen05.commit per Q tile that consumed the slot
        }
        fence_mbar_init();
    }
    if (warp == T::kLoadWarp && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    __syncthreads();
    if (*prior_error != 0) return;  // an earlier CTA or launch failed: do nothing (CTA-uniform)

    if (warp == T::kMmaWarp) {
        tmem_alloc(smem_u32(tmem_slot), T::kTmemCols);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_thread_sync();
    __syncthreads();
    tcgen05_fence_after_thread_sync();
    const uint32_t tmem_base = *tmem_slot;
    RING_TRACE_LIFE(tid == 0, 1);

    // ---- work assignment --------------------------------------------------------------------------
    const int bh = blockIdx.y;
    const int b = bh / a.heads;
    const int h = bh - b * a.heads;
    int nblk = (a.sk + T::kBlockN - 1) / T::kBlockN;  // K/V blocks to visit
    if (a.causal) {
        const int last_row = min(r0 + a.rows_per_cta, a.sq) - 1;
        const int last_key = last_row + a.diag;       // last visible key index of the CTA's rows
        const int vis_blk = last_key < 0 ? 0 : last_key / T::kBlockN + 1;
        nblk = min(nblk, vis_blk);
    }

    if (warp >= T::kSoftmaxWarps) {
        // ############################################################## producer warpgroup (warps 8..11)
        setmaxnreg_dec<T::kProducerRegs>();
        if (warp == T::kLoadWarp) {
            // =================================================================== TMA producer
            if (lane == 0 && nblk > 0) {
                mbar_arrive_expect_tx(bar_q_full(0), kTileBytes);
#pragma unroll
                for (int x = 0; x < kBoxes; ++x)
                    tma_load_4d(smem_q(0) + x * kBoxBytes, &tm_q, bar_q_full(0), x * 64, r0, h, b);
                // K and V have rings of their own (kKStages and kVStages slots): a K slot is free as soon as both
                // tiles' S products have read it, which is early, so K_(j+1) never queues behind a late P V.
                bool ok = true;
#pragma unroll 1
                for (int j = 0; j < nblk && ok; ++j) {
#pragma unroll 1
                    for (int kv = 0; kv < 2; ++kv) {
                        const int nslots = kv == 0 ? T::kKStages : T::kVStages;
                        const int slot = (kv == 0 ? 0 : T::kKStages) + j % nslots;
                        const int use = j / nslots;  // how many times this slot has been filled before
                        RING_TRACE_STAMP(true, 28 + 2 * kv);
                        if (use > 0) {
                            ok = mbar_wait(bar_kv_empty(slot), (use - 1) & 1, abort_flag, a.status, kDevLoadWaitEmpty);
                            if (!ok) break;
                        }
                        mbar_arrive_expect_tx(bar_kv_full(slot), kTileBytes);
                        const CUtensorMap* tm = kv == 0 ? &tm_k : &tm_v;
#pragma unroll
                        for (int x = 0; x < kBoxes; ++x)
                            tma_load_4d(smem_kv(slot) + x * kBoxBytes, tm, bar_kv_full(slot), x * 64, j * T::kBlockN, h, b);
                        RING_TRACE_STAMP(true, 29 + 2 * kv);
                        if (j == 0 && kv == 0 && tile1_valid) {
                            mbar_arrive_expect_tx(bar_q_full(1), kTileBytes);
#pragma unroll
                            for (int x = 0; x < kBoxes; ++x)
                                tma_load_4d(smem_q(1) + x * kBoxBytes, &tm_q, bar_q_full(1), x * 64, r0 + 128, h, b);
                        }
                    }
                }
            }
            __syncwarp();
        } else if (warp == T::kMmaWarp) {
            // =================================================================== UMMA issuer: S = Q K^T, both tiles
            // (Next to the softmax warps one thread gets roughly one tcgen05.mma out per 110 clocks, so the three MMA
            //  streams of the CTA -- S for both tiles, P V for tile 0, P V for tile 1 -- are issued by three warps.)
            if (lane == 0 && nblk > 0) {
                // S = Q_t K^T into the shared S buffer: D/16 instructions of 128 x 128 x 16
                auto issue_qk = [&](int t, int kslot) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
                        umma_ss(tmem_base + T::kTmemS, umma_desc_kmajor_sw128(smem_q(t) + off),
                                umma_desc_kmajor_sw128(smem_kv(kslot) + off), kIdescQK, kk > 0 ? 1u : 0u);
                    }
                };
                // The S buffer passes S_0(0), S_1(0), S_0(1), S_1(1), ...; read-out number n completes phase n of s_free.
                int reads = 0;  // read-outs awaited so far
                bool ok = true;
#pragma unroll 1
                for (int j = 0; j < nblk && ok; ++j) {
                    const int kslot = j % T::kKStages;
                    const uint32_t kphase = static_cast<uint32_t>((j / T::kKStages) & 1);
#pragma unroll 1
                    for (int t = 0; t < ntiles; ++t) {
                        RING_TRACE_STAMP(true, 16 + 4 * t);
                        if (j == 0) ok = mbar_wait(bar_q_full(t), 0, abort_flag, a.status, kDevMmaWaitQ);
                        // the buffer is free once its previous content has been read out by the tile it was for
                        if (ok && (j > 0 || t > 0)) {
                            ok = mbar_wait(bar_s_free, reads & 1, abort_flag, a.status, kDevMmaWaitS);
                            ++reads;
                        }
                        RING_TRACE_STAMP(true, 17 + 4 * t);
                        if (ok && t == 0) ok = mbar_wait(bar_kv_full(kslot), kphase, abort_flag, a.status, kDevMmaWaitKV);
                        if (!ok) break;
                        RING_TRACE_STAMP(true, 18 + 4 * t);
                        tcgen05_fence_after_thread_sync();
                        issue_qk(t, kslot);
                        umma_commit(bar_s_full(t));
                        umma_commit(bar_kv_empty(kslot));  // one arrival per tile
                        RING_TRACE_STAMP(true, 19 + 4 * t);
                    }
                }
            }
            __syncwarp();
        } else if (warp == T::kMmaWarp + 1 || warp == T::kMmaWarp + 2) {
            // =================================================================== UMMA issuer: O_t += P_t V, one warp per tile
            const int t = warp - (T::kMmaWarp + 1);
            if (lane == 0 && nblk > 0 && t < ntiles) {
                // kBlockN/16 instructions of 128 x D x 16, A = 16-bit P in TMEM, B = V MN-major in shared memory
                bool ok = true;
#pragma unroll 1
                for (int j = 0; j < nblk && ok; ++j) {
                    const int vslot = T::kKStages + j % T::kVStages;
                    const uint32_t vphase = static_cast<uint32_t>((j / T::kVStages) & 1);
                    ok = mbar_wait(bar_p_full(t), j & 1, abort_flag, a.status, kDevMmaWaitP) &&
                         mbar_wait(bar_kv_full(vslot), vphase, abort_flag, a.status, kDevMmaWaitKV);
                    if (!ok) break;
                    RING_TRACE_STAMP(true, 24 + 2 * t);
                    tcgen05_fence_after_thread_sync();
#pragma unroll
                    for (int kk = 0; kk < T::kBlockN / 16; ++kk) {
                        umma_ts(tmem_base + T::kTmemO0 + t * D, tmem_base + T::kTmemP0 + t * T::kTmemPCols + kk * 8,
                                umma_desc_mnmajor_sw128(smem_kv(vslot) + kk * 16 * 128, kBoxBytes), kIdescPV,
                                (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(bar_o_done(t));
                    umma_commit(bar_kv_empty(vslot));  // one arrival per tile
                    RING_TRACE_STAMP(true, 25 + 2 * t);
                }
            }
            __syncwarp();
        }
    } else {
        // ############################################################## softmax warpgroups (warps 0..7)
        setmaxnreg_inc<T::kSoftmaxRegs>();
        const int t = warp >> 2;  // Q tile of this warpgroup
        const int quarter = warp & 3;
        if (t < ntiles) {
            const int row = r0 + t * 128 + quarter * 32 + lane;  // row of the Q shard == TMEM lane
            const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
            const uint32_t t_s = tmem_base + lane_addr + T::kTmemS;
            const uint32_t t_p = tmem_base + lane_addr + T::kTmemP0 + t * T::kTmemPCols;
            const uint32_t t_o = tmem_base + lane_addr + T::kTmemO0 + t * D;
            const float c = a.scale_log2;

            float m_run = -INFINITY;  // maximum the exponentials are currently taken against (raw score)
            float l_run = 0.f;        // running sum of exp2((s - m_run) c), from unrounded fp32 p
            bool ok = true;

#pragma unroll 1
            for (int j = 0; j < nblk; ++j) {
                uint32_t sr[128];
                float* s = reinterpret_cast<float*>(sr);
                ok = mbar_wait(bar_s_full(t), j & 1, abort_flag, a.status, kDevSoftmaxWaitS);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                RING_TRACE_STAMP(quarter == 0 && lane == 0, t * 8 + 0);
                RING_TRACE_LIFE(tid == 0 && j == 0, 2);
                tcgen05_fence_after_thread_sync();
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    tmem_ld_x32(t_s + 32 * i, *reinterpret_cast<uint32_t(*)[32]>(&sr[32 * i]));
                tmem_wait_ld();
                // S is in registers: hand the buffer to the other tile (its next S is computed under this softmax)
                tcgen05_fence_before_thread_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_s_free);
                RING_TRACE_STAMP(quarter == 0 && lane == 0, t * 8 + 1);

                // masking: only blocks that straddle the causal diagonal or the end of the shard
                const int col0 = j * T::kBlockN;
                int limit = a.sk - col0;                                  // valid columns of this block
                if (a.causal) limit = min(limit, row + a.diag - col0 + 1);  // visible columns of this row
                const bool masked_block = (a.sk - col0 < T::kBlockN) ||
                                          (a.causal && (r0 + t * 128 + a.diag - col0 + 1) < T::kBlockN);
                if (masked_block) {
#pragma unroll
                    for (int i = 0; i < 128; ++i)
                        if (i >= limit) s[i] = -INFINITY;
                }

                // row maximum of the block; adopt it only when it beats the one in use by more than 2^8
                // eight independent chains (a chain of dependent max instructions is latency bound), then a tree
                float mxc[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) mxc[u] = fmaxf(s[2 * u], s[2 * u + 1]);
#pragma unroll
                for (int i = 16; i < 128; i += 16) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) mxc[u] = fmax3(mxc[u], s[i + 2 * u], s[i + 2 * u + 1]);
                }
                const float mx = fmaxf(fmax3(mxc[0], mxc[1], mxc[2]), fmax3(fmax3(mxc[3], mxc[4], mxc[5]), mxc[6], mxc[7]));
                float alpha = 1.f;  // factor owed to everything accumulated before this block
                if (mx > m_run && (m_run == -INFINITY || (mx - m_run) * c > kRescaleThresholdLog2)) {
                    alpha = (m_run == -INFINITY) ? 0.f : ex2_approx((m_run - mx) * c);
                    m_run = mx;
                }
                RING_TRACE_STAMP(quarter == 0 && lane == 0, t * 8 + 2);

                // p = exp2(s c - m c), in place, fp32; the sum uses the unrounded values
                const float nms = (m_run == -INFINITY) ? 0.f : -m_run * c;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int i = 0; i < 128; i += 4) {
                    // packed fp32 pairs (fma.rn.f32x2 / add.rn.f32x2): same roundings as the scalar forms, half the
                    // issue slots; the S row sits in consecutive registers, so the pairs cost no moves
#pragma unroll
                    for (int u = 0; u < 4; u += 2) {
                        float x0, x1;
                        ffma2(x0, x1, s[i + u], s[i + u + 1], c, c, nms, nms);
                        // At head dimension 64 the kernel is bound by the MUFU (the tensor pipe has half the work per
                        // exponential): one pair in four is evaluated on the FMA pipe instead.  At 128 that costs more
                        // than it saves (measured both ways).
                        if (D == 64 && ((i + u) / 2) % 4 == 3) {
                            ex2_poly2(s[i + u], s[i + u + 1], x0, x1);
                            continue;
                        }
                        s[i + u] = ex2_approx(x0);
                        s[i + u + 1] = ex2_approx(x1);
                    }
                    fadd2(a0, a1, a0, a1, s[i], s[i + 1]);
                    fadd2(a2, a3, a2, a3, s[i + 2], s[i + 3]);
                }
                l_run = fmaf(l_run, alpha, (a0 + a1) + (a2 + a3));
                RING_TRACE_STAMP(quarter == 0 && lane == 0, t * 8 + 3);

                // P_t(j - 1) V must be complete before P_t is overwritten or O_t rescaled (it long is)
                if (j > 0) {
                    ok = mbar_wait(bar_o_done(t), (j - 1) & 1, abort_flag, a.status, kDevSoftmaxWaitO);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tcgen05_fence_after_thread_sync();
                    // O_t is rescaled only when some row of the warp adopted a new maximum (warp-collective TMEM round trip)
                    if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
                        for (int i = 0; i < D / 32; ++i) {
                            uint32_t orr[32];
                            tmem_ld_x32(t_o + 32 * i, orr);
                            tmem_wait_ld();
#pragma unroll
                            for (int x = 0; x < 32; ++x) orr[x] = __float_as_uint(__uint_as_float(orr[x]) * alpha);
                            tmem_st_x32(t_o + 32 * i, orr);
                        }
                    }
                }
                RING_TRACE_STAMP(quarter == 0 && lane == 0, t * 8 + 4);

                // P_t(j): 128 probabilities -> 64 columns of 16-bit pairs
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    uint32_t pk[32];
#pragma unroll
                    for (int x = 0; x < 32; ++x)
                        pk[x] = T::kIsBf16 ? pack_bf16x2(s[64 * i + 2 * x], s[64 * i + 2 * x + 1])
                                           : pack_f16x2(s[64 * i + 2 * x], s[64 * i + 2 * x + 1]);
                    tmem_st_x32(t_p + 32 * i, pk);
                }
                tmem_wait_st();
                tcgen05_fence_before_thread_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p_full(t));
                RING_TRACE_STAMP(quarter == 0 && lane == 0, t * 8 + 5);
            }

            RING_TRACE_LIFE(tid == 0, 3);
            // ---- epilogue: O / l, LSE, optional fold into an earlier partial -----------------------
            if (ok && nblk > 0) {
                ok = mbar_wait(bar_o_done(t), (nblk - 1) & 1, abort_flag, a.status, kDevSoftmaxWaitO);
                ok = __all_sync(0xffffffffu, ok);
                if (ok) tcgen05_fence_after_thread_sync();
            }
            if (ok) {
                const bool have = (nblk > 0) && (l_run > 0.f);
                float w_new = have ? 1.f / l_run : 0.f;  // factor applied to the accumulator in TMEM
                float lse_new = have ? m_run * a.scale + logf(l_run) : -INFINITY;
                float w_old = 0.f;
                const bool row_ok = row < a.sq;
                float* lse_ptr = a.lse + b * a.lse_batch_stride + h * a.lse_head_stride + row;
                if (a.merge && row_ok) {
                    const float lse_old = *lse_ptr;
                    const float mx = fmaxf(lse_old, lse_new);
                    if (mx == -INFINITY) {
                        w_old = 0.f;
                        w_new = 0.f;
                    } else {
                        const float e_old = expf(lse_old - mx);
                        const float e_new = expf(lse_new - mx);
                        const float tot = e_old + e_new;
                        w_old = e_old / tot;
                        w_new *= e_new / tot;
                        lse_new = mx + logf(tot);
                    }
                }
                // O goes out through shared memory so that every store instruction writes whole rows: the Q tile of
                // this warpgroup is free (its last S product has been read), each warp stages its 32 rows there, half
                // of the columns at a time, in 16-byte chunks XOR-swizzled by the row (conflict-free both ways).
                constexpr int kHalfCols = D / 2;              // columns per pass
                constexpr int kChunks = kHalfCols / 4;        // 16-byte chunks per staged row
                constexpr int kRowsPerInst = 32 / kChunks;    // rows one coalesced instruction covers
                const uint32_t stage = smem_q(t) + static_cast<uint32_t>(quarter) * (kTileBytes / 4);
                const int row_base = r0 + t * 128 + quarter * 32;
                float* o_base = a.o + b * a.o_batch_stride + h * a.o_head_stride;
#pragma unroll 1
                for (int pass = 0; pass < 2; ++pass) {
                    // when folding into an earlier partial, fetch its values first: all loads of the pass are in
                    // flight together and their latency passes under the TMEM read-out and the staging
                    float4 old[32 / kRowsPerInst];
                    if (a.merge) {
#pragma unroll
                        for (int rr = 0; rr < 32 / kRowsPerInst; ++rr) {
                            const int rl = rr * kRowsPerInst + lane / kChunks;
                            old[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (row_base + rl < a.sq)
                                old[rr] = *(reinterpret_cast<const float4*>(o_base + static_cast<int64_t>(row_base + rl) * a.o_row_stride +
                                                                            pass * kHalfCols) + lane % kChunks);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < kHalfCols / 32; ++i) {
                        uint32_t orr[32];
                        if (nblk > 0) {
                            tmem_ld_x32(t_o + pass * kHalfCols + 32 * i, orr);
                            tmem_wait_ld();
                        } else {
#pragma unroll
                            for (int x = 0; x < 32; ++x) orr[x] = 0u;
                        }
#pragma unroll
                        for (int x = 0; x < 8; ++x) {
                            const int chunk = i * 8 + x;
                            st_shared_v4(stage + lane * (kChunks * 16) + ((chunk ^ (lane & (kChunks - 1))) << 4),
                                         __float_as_uint(__uint_as_float(orr[4 * x + 0]) * w_new),
                                         __float_as_uint(__uint_as_float(orr[4 * x + 1]) * w_new),
                                         __float_as_uint(__uint_as_float(orr[4 * x + 2]) * w_new),
                                         __float_as_uint(__uint_as_float(orr[4 * x + 3]) * w_new));
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int rr = 0; rr < 32 / kRowsPerInst; ++rr) {
                        const int rl = rr * kRowsPerInst + lane / kChunks;  // row of the warp this lane serves now
                        const int ch = lane % kChunks;
                        float4 val = ld_shared_v4(stage + rl * (kChunks * 16) + ((ch ^ (rl & (kChunks - 1))) << 4));
                        const float wo = __shfl_sync(0xffffffffu, w_old, rl);
                        if (a.merge) {
                            val.x = fmaf(old[rr].x, wo, val.x);
                            val.y = fmaf(old[rr].y, wo, val.y);
                            val.z = fmaf(old[rr].z, wo, val.z);
                            val.w = fmaf(old[rr].w, wo, val.w);
                        }
                        if (row_base + rl < a.sq)
                            *(reinterpret_cast<float4*>(o_base + static_cast<int64_t>(row_base + rl) * a.o_row_stride +
                                                        pass * kHalfCols) + ch) = val;
                    }
                    __syncwarp();
                }
                if (row_ok) *lse_ptr = lse_new;
            }
        }
    }

    RING_TRACE_LIFE(tid == 0, 4);
    // ---- common exit: every thread arrives here, on success and on a timed-out wait alike ------------
    tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp == T::kMmaWarp) {
        tcgen05_fence_after_thread_sync();
        tmem_dealloc(tmem_base, T::kTmemCols);
    }
}

// One warp waits, with the same bounded wait the block kernel uses, on an mbarrier that nobody arrives at.
// It must come back after the limit with `code` in the status word (used by the library's self-test).
__global__ void ring_wait_timeout_probe(int* status, int code) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();
    const bool ok = ptx::mbar_wait(ptx::smem_u32(&bar), 0, &abort_flag, status, code);
    if (ok && threadIdx.x == 0) atomicCAS(status, 0, -1);  // the wait must NOT have succeeded
}

}  // namespace ring
