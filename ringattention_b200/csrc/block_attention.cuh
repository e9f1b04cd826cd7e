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
//   * a CTA owns two 128-row Q tiles of one (batch, head) and walks the K/V shard in 128-row blocks;
//   * one thread issues TMA loads (Q once, then K_j, V_j through a ring of kStages shared-memory
//     slots, 128-byte swizzle, 64-element boxes);
//   * one thread issues tcgen05.mma: S_t = Q_t K_j^T (both operands K-major in shared memory) into
//     TMEM columns [t*128, t*128+128), and O_t += P_t V_j with P_t read from TMEM (fp16 pairs aliased
//     onto the first 64 columns of S_t) and V_j MN-major from shared memory, so V is never transposed
//     (the reference needs ldmatrix.trans for that, csrc/kernel_traits.h:39,93-103);
//   * two softmax warpgroups (one per Q tile, one thread per row = one TMEM lane) read S with
//     tcgen05.ld, keep the running max / sum in registers, write P with tcgen05.st and rescale O in
//     TMEM only when a row maximum grew by more than 2^8 (the stale maximum is exact algebra: it
//     cancels in O / l and in the LSE);
//   * the two tiles ping-pong: while one warpgroup does softmax on S_t the tensor pipe runs the other
//     tile's MMAs.
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
    kDevSoftmaxWaitS = 121,
    kDevSoftmaxWaitO = 122,
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
    int* status;      // device status word
};

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
    auto smem_q = [&](int t) { return base + static_cast<uint32_t>(t * kTileBytes); };
    auto smem_kv = [&](int s) { return base + static_cast<uint32_t>((T::kQTiles + s) * kTileBytes); };

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        *abort_flag = 0;
        *prior_error = *reinterpret_cast<volatile int*>(a.status);
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_q_full(t), 1);
            mbar_init(bar_s_full(t), 1);
            mbar_init(bar_p_full(t), 128);
            mbar_init(bar_o_done(t), 1);
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_kv_full(s), 1);
            mbar_init(bar_kv_empty(s), 1);
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

    // ---- work assignment --------------------------------------------------------------------------
    const int bh = blockIdx.y;
    const int b = bh / a.heads;
    const int h = bh - b * a.heads;
    const int r0 = blockIdx.x * T::kBlockM;           // first Q row of this CTA
    const bool tile1_valid = (r0 + 128) < a.sq;
    int nblk = (a.sk + T::kBlockN - 1) / T::kBlockN;  // K/V blocks to visit
    if (a.causal) {
        const int last_row = min(r0 + T::kBlockM, a.sq) - 1;
        const int last_key = last_row + a.diag;       // last visible key index of the CTA's rows
        const int vis_blk = last_key < 0 ? 0 : last_key / T::kBlockN + 1;
        nblk = min(nblk, vis_blk);
    }

    if (warp == T::kLoadWarp) {
        // ======================================================================= TMA producer
        if (lane == 0 && nblk > 0) {
            mbar_arrive_expect_tx(bar_q_full(0), kTileBytes);
#pragma unroll
            for (int x = 0; x < kBoxes; ++x)
                tma_load_4d(smem_q(0) + x * kBoxBytes, &tm_q, bar_q_full(0), x * 64, r0, h, b);
            int slot = 0;
            uint32_t wrap = 0;  // how many times the ring has wrapped
            bool ok = true;
#pragma unroll 1
            for (int j = 0; j < nblk && ok; ++j) {
#pragma unroll 1
                for (int kv = 0; kv < 2; ++kv) {
                    if (wrap > 0) {
                        ok = mbar_wait(bar_kv_empty(slot), (wrap - 1) & 1, abort_flag, a.status, kDevLoadWaitEmpty);
                        if (!ok) break;
                    }
                    mbar_arrive_expect_tx(bar_kv_full(slot), kTileBytes);
                    const CUtensorMap* tm = kv == 0 ? &tm_k : &tm_v;
#pragma unroll
                    for (int x = 0; x < kBoxes; ++x)
                        tma_load_4d(smem_kv(slot) + x * kBoxBytes, tm, bar_kv_full(slot), x * 64, j * T::kBlockN, h, b);
                    if (++slot == kStages) { slot = 0; ++wrap; }
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
        // ======================================================================= UMMA issuer
        if (lane == 0 && nblk > 0) {
            int slot = 0;
            uint32_t phase = 0;
            bool ok = true;
            auto advance = [&]() { if (++slot == kStages) { slot = 0; phase ^= 1; } };
            // S_t = Q_t K^T : D/16 instructions of 128 x 128 x 16
            auto issue_qk = [&](int t, int kslot) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
                    umma_ss(tmem_base + T::kTmemS0 + t * T::kBlockN, umma_desc_kmajor_sw128(smem_q(t) + off),
                            umma_desc_kmajor_sw128(smem_kv(kslot) + off), kIdescQK, kk > 0 ? 1u : 0u);
                }
            };
            // O_t (+)= P_t V : kBlockN/16 instructions of 128 x D x 16, A = fp16 P in TMEM
            auto issue_pv = [&](int t, int vslot, bool accumulate) {
#pragma unroll
                for (int kk = 0; kk < T::kBlockN / 16; ++kk) {
                    umma_ts(tmem_base + T::kTmemO0 + t * D, tmem_base + T::kTmemS0 + t * T::kBlockN + kk * 8,
                            umma_desc_mnmajor_sw128(smem_kv(vslot) + kk * 16 * 128, kBoxBytes), kIdescPV,
                            (accumulate || kk > 0) ? 1u : 0u);
                }
            };

            // prologue: S_t(0) for both tiles
            ok = mbar_wait(bar_q_full(0), 0, abort_flag, a.status, kDevMmaWaitQ) &&
                 mbar_wait(bar_kv_full(slot), phase, abort_flag, a.status, kDevMmaWaitKV);
            if (ok) {
                tcgen05_fence_after_thread_sync();
                issue_qk(0, slot);
                umma_commit(bar_s_full(0));
                if (tile1_valid) {
                    ok = mbar_wait(bar_q_full(1), 0, abort_flag, a.status, kDevMmaWaitQ);
                    if (ok) {
                        tcgen05_fence_after_thread_sync();
                        issue_qk(1, slot);
                        umma_commit(bar_s_full(1));
                    }
                }
                umma_commit(bar_kv_empty(slot));
                advance();
            }
#pragma unroll 1
            for (int j = 0; j < nblk && ok; ++j) {
                const bool has_next = (j + 1) < nblk;
                const uint32_t pj = j & 1;
                const int vslot = slot;
                const uint32_t vphase = phase;
                advance();
                const int kslot = slot;
                const uint32_t kphase = phase;
                if (has_next) advance();

                ok = mbar_wait(bar_kv_full(vslot), vphase, abort_flag, a.status, kDevMmaWaitKV) &&
                     mbar_wait(bar_p_full(0), pj, abort_flag, a.status, kDevMmaWaitP);
                if (!ok) break;
                tcgen05_fence_after_thread_sync();
                issue_pv(0, vslot, j > 0);
                umma_commit(bar_o_done(0));
                if (has_next) {
                    ok = mbar_wait(bar_kv_full(kslot), kphase, abort_flag, a.status, kDevMmaWaitKV);
                    if (!ok) break;
                    tcgen05_fence_after_thread_sync();
                    issue_qk(0, kslot);
                    umma_commit(bar_s_full(0));
                }
                if (tile1_valid) {
                    ok = mbar_wait(bar_p_full(1), pj, abort_flag, a.status, kDevMmaWaitP);
                    if (!ok) break;
                    tcgen05_fence_after_thread_sync();
                    issue_pv(1, vslot, j > 0);
                    umma_commit(bar_o_done(1));
                }
                umma_commit(bar_kv_empty(vslot));
                if (has_next) {
                    if (tile1_valid) {
                        issue_qk(1, kslot);
                        umma_commit(bar_s_full(1));
                    }
                    umma_commit(bar_kv_empty(kslot));
                }
            }
        }
        __syncwarp();
    } else {
        // ======================================================================= softmax warpgroups
        const int t = warp >> 2;  // Q tile of this warpgroup
        const int quarter = warp & 3;
        if (t == 0 || tile1_valid) {
            const int row = r0 + t * 128 + quarter * 32 + lane;  // row of the Q shard == TMEM lane
            const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
            const uint32_t t_s = tmem_base + lane_addr + T::kTmemS0 + t * T::kBlockN;
            const uint32_t t_o = tmem_base + lane_addr + T::kTmemO0 + t * D;
            const float c = a.scale_log2;

            float m_run = -INFINITY;  // maximum the exponentials are currently taken against (raw score)
            float l_run = 0.f;        // running sum of exp2((s - m_run) c), from unrounded fp32 p
            bool ok = true;

#pragma unroll 1
            for (int j = 0; j < nblk; ++j) {
                ok = mbar_wait(bar_s_full(t), j & 1, abort_flag, a.status, kDevSoftmaxWaitS);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tcgen05_fence_after_thread_sync();

                uint32_t sr[128];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    tmem_ld_x32(t_s + 32 * i, *reinterpret_cast<uint32_t(*)[32]>(&sr[32 * i]));
                tmem_wait_ld();
                float* s = reinterpret_cast<float*>(sr);

                // masking: only blocks that straddle the causal diagonal or the end of the shard
                const int col0 = j * T::kBlockN;
                int limit = a.sk - col0;                                  // valid columns of this block
                if (a.causal) limit = min(limit, row + a.diag - col0 + 1);  // visible columns of this row
                const bool masked_block = (a.sk - col0 < T::kBlockN) ||
                                          (a.causal && (r0 + t * 128 + a.diag - col0 + 1) < T::kBlockN);
                if (masked_block) {
#pragma unroll
                    for (int cidx = 0; cidx < 128; ++cidx)
                        if (cidx >= limit) s[cidx] = -INFINITY;
                }

                float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
                for (int cidx = 4; cidx < 128; cidx += 4) {
                    mx0 = fmaxf(mx0, s[cidx]);
                    mx1 = fmaxf(mx1, s[cidx + 1]);
                    mx2 = fmaxf(mx2, s[cidx + 2]);
                    mx3 = fmaxf(mx3, s[cidx + 3]);
                }
                const float m_new = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), m_run);

                // Lazy rescale: adopt the new maximum only when it exceeds the one in use by more than
                // 2^8 in the exponent (or nothing is in use yet).  Warp-uniform, because rescaling O
                // is a warp-collective TMEM round trip.
                const bool need = (m_new > m_run) && ((m_run == -INFINITY) || ((m_new - m_run) * c > kRescaleThresholdLog2));
                if (__any_sync(0xffffffffu, need)) {
                    const float alpha = (m_run == -INFINITY) ? 0.f : ex2_approx((m_run - m_new) * c);
                    l_run *= alpha;
                    if (j > 0) {
                        ok = mbar_wait(bar_o_done(t), (j - 1) & 1, abort_flag, a.status, kDevSoftmaxWaitO);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tcgen05_fence_after_thread_sync();
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
                    m_run = m_new;
                }

                const float ms = (m_run == -INFINITY) ? 0.f : m_run * c;
                float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t pk[16];
#pragma unroll
                    for (int x = 0; x < 16; x += 2) {
                        const float p0 = ex2_approx(fmaf(s[32 * i + 2 * x + 0], c, -ms));
                        const float p1 = ex2_approx(fmaf(s[32 * i + 2 * x + 1], c, -ms));
                        const float p2 = ex2_approx(fmaf(s[32 * i + 2 * x + 2], c, -ms));
                        const float p3 = ex2_approx(fmaf(s[32 * i + 2 * x + 3], c, -ms));
                        l0 += p0; l1 += p1; l2 += p2; l3 += p3;
                        pk[x] = T::kIsBf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
                        pk[x + 1] = T::kIsBf16 ? pack_bf16x2(p2, p3) : pack_f16x2(p2, p3);
                    }
                    tmem_st_x16(t_s + 16 * i, pk);  // 32 probabilities = 16 packed columns
                }
                l_run += (l0 + l1) + (l2 + l3);
                tmem_wait_st();
                tcgen05_fence_before_thread_sync();
                mbar_arrive(bar_p_full(t));
            }

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
                float* o_ptr = a.o + b * a.o_batch_stride + h * a.o_head_stride + static_cast<int64_t>(row) * a.o_row_stride;
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
#pragma unroll
                for (int i = 0; i < D / 32; ++i) {
                    uint32_t orr[32];
                    if (nblk > 0) {
                        tmem_ld_x32(t_o + 32 * i, orr);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int x = 0; x < 32; ++x) orr[x] = 0u;
                    }
                    if (row_ok) {
                        float4* dst = reinterpret_cast<float4*>(o_ptr + 32 * i);
#pragma unroll
                        for (int x = 0; x < 8; ++x) {
                            float4 val;
                            val.x = __uint_as_float(orr[4 * x + 0]) * w_new;
                            val.y = __uint_as_float(orr[4 * x + 1]) * w_new;
                            val.z = __uint_as_float(orr[4 * x + 2]) * w_new;
                            val.w = __uint_as_float(orr[4 * x + 3]) * w_new;
                            if (a.merge) {
                                const float4 old = dst[x];
                                val.x = fmaf(old.x, w_old, val.x);
                                val.y = fmaf(old.y, w_old, val.y);
                                val.z = fmaf(old.z, w_old, val.z);
                                val.w = fmaf(old.w, w_old, val.w);
                            }
                            dst[x] = val;
                        }
                    }
                }
                if (row_ok) *lse_ptr = lse_new;
            }
        }
    }

    // ---- common exit: every thread arrives here, on success and on a timed-out wait alike ------------
    tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp == T::kMmaWarp) {
        tcgen05_fence_after_thread_sync();
        tmem_dealloc(tmem_base, T::kTmemCols);
    }
}

}  // namespace ring
