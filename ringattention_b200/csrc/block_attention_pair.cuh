// CTA-pair form of the block-attention kernel (head dimension 128): the same contract as
// ring_block_attention_kernel -- one Q shard against one K/V shard, normalised O tile + row log-sum-exp, optional
// fold into an earlier partial; it replaces the same part of the reference (csrc/ring_attention.cu:398-666,
// one ring step) -- with a different mapping to the hardware:
//
//   * a CLUSTER of two CTAs owns 256 Q rows, 128 per CTA, and the pair walks the K/V shard together.  Every
//     tcgen05.mma is a cta_group::2 instruction (M = 256: 128 rows in each CTA's tensor memory) issued by one thread
//     of the leader CTA; its B operand is split between the two CTAs' shared memories, so each CTA loads only half
//     of every K block (64 of the 128 keys) and half of every V block (64 of the 128 value columns), with plain
//     per-CTA TMA loads (each CTA fetches its own half).  Per instruction a CTA reads 6 KB of operands from shared memory instead of
//     8 KB, which brings the S product under the 64 clocks of its math;
//   * with one Q tile per CTA the tensor memory holds TWO S buffers (even and odd K/V blocks), two P buffers and O:
//     S(j + 1) is computed while block j is in its softmax, so the tensor pipe never waits for an S buffer to be
//     read out (the one-buffer form spends about a quarter of its time in that hand-off);
//   * two groups of softmax warps share the 128 rows: one takes the even K/V blocks, the other the odd ones, with
//     one thread per row in each (kHalves = 1) or two threads per row that split the block's 128 columns and exchange
//     the maxima of their halves through shared memory (kHalves = 2: four softmax warps per scheduler).  The running maximum of a row is a value in shared memory that the two
//     threads of the row hand to each other block by block (a new maximum is adopted only when it beats the one in
//     use by more than 2^8, so it rarely changes and O is rarely rescaled); each thread keeps the sum of its own
//     blocks and the two are combined at the end;
//   * cross-CTA signalling: TMA completions of both CTAs count on the LEADER's "full" barriers (the issuers wait
//     there), the softmax warps of both CTAs arrive on the leader's "S read out" / "P written" barriers, and every
//     tcgen05.commit is issued twice, once per CTA's barrier;
//   * K and V arrive through rings of four slots each, filled by two loader threads (K slots are released as
//     soon as the S product has read them, V slots only after the later P V product).
// Every mbarrier wait is bounded; on expiry the CTA records a status code and all roles fall through to the common
// exit.  The two cluster-wide hardware barriers (start and end) are reached by every thread on every path.
#pragma once

#include "block_attention.cuh"

namespace ring {

#ifdef RING_TRACE
#define RING_PTRACE(cond, j, slot) do { if ((cond) && a.trace && blockIdx.x < 2 && blockIdx.y == 0) a.trace[blockIdx.x * 4096 + (j) * 16 + (slot)] = clock64(); } while (0)
#else
#define RING_PTRACE(cond, j, slot) do { } while (0)
#endif

template <class T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T::kNThreads, 1)
ring_block_attention_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                                 const __grid_constant__ CUtensorMap tm_v, const BlockFwdArgs a) {
    using namespace ptx;
    constexpr int D = T::kHeadDim;
    constexpr int kKS = T::kKStages, kVS = T::kVStages, kStages = T::kStages;
    constexpr int kH = T::kHalves;       // threads per Q row and block parity
    constexpr int kC = 128 / kH;         // columns of a block each of them handles
    constexpr uint32_t kIdescQK = umma_idesc_f16(256, T::kBlockN, false, false, T::kIsBf16);
    constexpr uint32_t kIdescPV = umma_idesc_f16(256, D, false, true, T::kIsBf16);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment; same offset in both CTAs
    uint8_t* smem = smem_raw + (base - raw_addr);
    uint8_t* tail = smem + T::kSmemTiles;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + T::kNumBarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* prior_error = reinterpret_cast<volatile int*>(tmem_slot + 2);
    volatile float* m_sh = reinterpret_cast<volatile float*>(tail + T::kTailMaxima);   // [2][128] maximum in use after block j, at [j & 1]
    volatile float* hmax_sh = reinterpret_cast<volatile float*>(tail + T::kTailHalfMax);  // [parity][half][n & 1][128] block maximum of a column half
    volatile float* xl = reinterpret_cast<volatile float*>(tail + T::kTailSums);        // [parity * kHalves + half][128][2]: (maximum, sum) of each thread of a row

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t bar_q_full = bar0;
    auto bar_kv_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto bar_kv_empty = [&](int s) { return bar0 + 8u * (1 + kStages + s); };
    auto bar_s_full = [&](int b) { return bar0 + 8u * (1 + 2 * kStages + b); };
    auto bar_s_free = [&](int b) { return bar0 + 8u * (3 + 2 * kStages + b); };
    auto bar_p_full = [&](int b) { return bar0 + 8u * (5 + 2 * kStages + b); };
    auto bar_o_done = [&](int b) { return bar0 + 8u * (7 + 2 * kStages + b); };
    auto bar_m_pub = [&](int q) { return bar0 + 8u * (9 + 2 * kStages + q); };
    auto bar_half_max = [&](int g, int q) { return bar0 + 8u * (13 + 2 * kStages + g * 4 + q); };
    const uint32_t smem_q = base;
    auto smem_slot = [&](int s) { return base + static_cast<uint32_t>(T::kQBytes + s * T::kSlotBytes); };

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const uint32_t crank = cluster_ctarank();  // 0: leader (issues the MMAs of the pair)

    // Under a causal mask the pairs of the last Q rows have the most K/V blocks to visit: launch them first.
    const int npairs = gridDim.x >> 1;
    const int pair = a.causal ? (npairs - 1 - static_cast<int>(blockIdx.x >> 1)) : static_cast<int>(blockIdx.x >> 1);
    const int pair_r0 = pair * 256;
    const int r0 = pair_r0 + static_cast<int>(crank) * 128;  // first Q row of this CTA

    if (tid == 0) {
        *abort_flag = 0;
        *prior_error = *reinterpret_cast<volatile int*>(a.status);
        mbar_init(bar_q_full, 2);  // one expect_tx arrival per CTA's loader
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_kv_full(s), 2);   // one expect_tx arrival per CTA's loader
            mbar_init(bar_kv_empty(s), 1);  // one tcgen05.commit per use
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_s_full(b), 1);
            mbar_init(bar_s_free(b), 8 * kH);  // the parity's softmax warps of both CTAs
            mbar_init(bar_p_full(b), 8 * kH);
            mbar_init(bar_o_done(b), 1);
            for (int q = 0; q < 4; ++q) mbar_init(bar_half_max(b, q), 2);
        }
        for (int q = 0; q < 4; ++q) mbar_init(bar_m_pub(q), kH);
        fence_mbar_init();
    }
    if (warp == T::kLoadWarp && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised; its copy of the status word is readable
    // The decision to do nothing (an earlier CTA or launch failed) must be the same in both CTAs of the pair.
    const int peer_prior = static_cast<int>(ld_shared_cluster_u32(mapa_shared(smem_u32(const_cast<int*>(prior_error)), crank ^ 1u)));
    const int my_prior = *prior_error;
    cluster_sync_all();  // nobody reads a peer's shared memory after this point except through the MMAs
    if (my_prior != 0 || peer_prior != 0) return;

    if (warp == T::kQkWarp) {  // the same warp in both CTAs
        tmem_alloc_pair(smem_u32(tmem_slot), T::kTmemCols);
        tmem_relinquish_alloc_permit_pair();
    }
    tcgen05_fence_before_thread_sync();
    __syncthreads();
    tcgen05_fence_after_thread_sync();
    const uint32_t tmem_base = *tmem_slot;

    // ---- work assignment --------------------------------------------------------------------------
    const int bh = blockIdx.y;
    const int b = bh / a.heads;
    const int h = bh - b * a.heads;
    int nblk = (a.sk + T::kBlockN - 1) / T::kBlockN;  // K/V blocks the PAIR visits
    if (a.causal) {
        const int last_row = min(pair_r0 + 256, a.sq) - 1;
        const int last_key = last_row + a.diag;  // last visible key index of the pair's rows
        const int vis_blk = last_key < 0 ? 0 : last_key / T::kBlockN + 1;
        nblk = min(nblk, vis_blk);
    }

    if (warp >= T::kSoftmaxWarps) {
        // ############################################################## producer warpgroup (the last four warps)
        setmaxnreg_dec<T::kProducerRegs>();
        if (warp == T::kLoadWarp) {
            // =================================================================== TMA producer of Q and K (both CTAs)
            if (lane == 0 && nblk > 0) {
                const uint32_t lead_q = mapa_shared(bar_q_full, 0);
                mbar_arrive_expect_tx_cluster(lead_q, T::kQBytes);
#pragma unroll
                for (int x = 0; x < D / 64; ++x)
                    tma_load_4d_pair(smem_q + x * T::kBoxBytesQ, &tm_q, lead_q, x * 64, r0, h, b);
                bool ok = true;
#pragma unroll 1
                for (int j = 0; j < nblk && ok; ++j) {
                    // this CTA's 64 keys of K block j: two boxes of 64 columns x 64 rows
                    const int slot = j % kKS, use = j / kKS;
                    if (use > 0) ok = mbar_wait_cluster(bar_kv_empty(slot), (use - 1) & 1, abort_flag, a.status, kDevLoadWaitEmpty);
                    if (!ok) break;
                    const uint32_t lead = mapa_shared(bar_kv_full(slot), 0);
                    RING_PTRACE(true, j, 10);
                    mbar_arrive_expect_tx_cluster(lead, T::kSlotBytes);
#pragma unroll
                    for (int x = 0; x < D / 64; ++x)
                        tma_load_4d_pair(smem_slot(slot) + x * T::kBoxBytesK, &tm_k, lead, x * 64,
                                         j * T::kBlockN + static_cast<int>(crank) * 64, h, b);
                }
            }
            __syncwarp();
        } else if (warp == T::kLoadWarpV) {
            // =================================================================== TMA producer of V (both CTAs)
            if (lane == 0 && nblk > 0) {
                bool ok = true;
#pragma unroll 1
                for (int j = 0; j < nblk && ok; ++j) {
                    // this CTA's 64 value columns of V block j: one box of 64 columns x 128 rows
                    const int slot = kKS + j % kVS, use = j / kVS;
                    if (use > 0) ok = mbar_wait_cluster(bar_kv_empty(slot), (use - 1) & 1, abort_flag, a.status, kDevLoadWaitEmpty);
                    if (!ok) break;
                    const uint32_t lead = mapa_shared(bar_kv_full(slot), 0);
                    RING_PTRACE(true, j, 11);
                    mbar_arrive_expect_tx_cluster(lead, T::kSlotBytes);
                    tma_load_4d_pair(smem_slot(slot), &tm_v, lead, static_cast<int>(crank) * 64, j * T::kBlockN, h, b);
                }
            }
            __syncwarp();
        } else if (warp == T::kQkWarp) {
            // =================================================================== UMMA issuer (leader): S(j) = Q K_j^T
            if (crank == 0 && lane == 0 && nblk > 0) {
                const uint32_t peer_s_full0 = mapa_shared(bar_s_full(0), 1), peer_s_full1 = mapa_shared(bar_s_full(1), 1);
                bool ok = mbar_wait_cluster(bar_q_full, 0, abort_flag, a.status, kDevMmaWaitQ);
#pragma unroll 1
                for (int j = 0; j < nblk && ok; ++j) {
                    const int kslot = j % kKS, par = j & 1;
                    const uint32_t n = static_cast<uint32_t>(j >> 1);
                    ok = mbar_wait_cluster(bar_kv_full(kslot), static_cast<uint32_t>((j / kKS) & 1), abort_flag, a.status, kDevMmaWaitKV);
                    // S buffer `par` was last used by block j - 2: both CTAs' softmax warps must have read it out
                    if (ok && j >= 2) ok = mbar_wait_cluster(bar_s_free(par), (n - 1) & 1, abort_flag, a.status, kDevMmaWaitS);
                    if (!ok) break;
                    RING_PTRACE(true, j, 0);
                    tcgen05_fence_after_thread_sync();
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off_q = (kk >> 2) * T::kBoxBytesQ + (kk & 3) * 32;
                        const uint32_t off_k = (kk >> 2) * T::kBoxBytesK + (kk & 3) * 32;
                        umma_ss_pair(tmem_base + T::kTmemS0 + par * T::kBlockN, umma_desc_kmajor_sw128(smem_q + off_q),
                                     umma_desc_kmajor_sw128(smem_slot(kslot) + off_k), kIdescQK, kk > 0 ? 1u : 0u);
                    }
                    umma_commit_pair(bar_s_full(par));
                    umma_commit_pair(par ? peer_s_full1 : peer_s_full0);
                    umma_commit_pair(bar_kv_empty(kslot));
                    umma_commit_pair(mapa_shared(bar_kv_empty(kslot), 1));
                    RING_PTRACE(true, j, 1);
                }
            }
            __syncwarp();
        } else if (warp == T::kPvWarp) {
            // =================================================================== UMMA issuer (leader): O += P(j) V_j
            if (crank == 0 && lane == 0 && nblk > 0) {
                const uint32_t peer_o_done0 = mapa_shared(bar_o_done(0), 1), peer_o_done1 = mapa_shared(bar_o_done(1), 1);
                bool ok = true;
#pragma unroll 1
                for (int j = 0; j < nblk && ok; ++j) {
                    const int buf = j & 1, vslot = kKS + j % kVS;
                    const uint32_t n = static_cast<uint32_t>(j >> 1);
                    ok = mbar_wait_cluster(bar_p_full(buf), n & 1, abort_flag, a.status, kDevMmaWaitP) &&
                         mbar_wait_cluster(bar_kv_full(vslot), static_cast<uint32_t>((j / kVS) & 1), abort_flag, a.status, kDevMmaWaitKV);
                    if (!ok) break;
                    RING_PTRACE(true, j, 2);
                    tcgen05_fence_after_thread_sync();
                    // kBlockN/16 instructions of 256 x D x 16: A = 16-bit P in each CTA's tensor memory, B = V MN-major,
                    // 64 value columns from each CTA's shared memory
#pragma unroll
                    for (int kk = 0; kk < T::kBlockN / 16; ++kk) {
                        umma_ts_pair(tmem_base + T::kTmemO, tmem_base + T::kTmemP0 + buf * T::kTmemPCols + kk * 8,
                                     umma_desc_mnmajor_sw128(smem_slot(vslot) + kk * 16 * 128, T::kSlotBytes), kIdescPV,
                                     (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(bar_o_done(buf));
                    umma_commit_pair(buf ? peer_o_done1 : peer_o_done0);
                    umma_commit_pair(bar_kv_empty(vslot));
                    umma_commit_pair(mapa_shared(bar_kv_empty(vslot), 1));
                    RING_PTRACE(true, j, 3);
                }
            }
            __syncwarp();
        }
    } else {
        // ############################################################## softmax warpgroups
        setmaxnreg_inc<T::kSoftmaxRegs>();
        const int quarter = warp & 3;                       // TMEM lane quarter this warp may touch
        const int hf = kH == 2 ? ((warp >> 2) & 1) : 0;      // column half of the block (two threads per row)
        const int g = warp >> (kH == 2 ? 3 : 2);             // 0: even K/V blocks, 1: odd ones
        const int row_local = quarter * 32 + lane;          // row of the CTA's Q tile == TMEM lane
        const int row = r0 + row_local;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + lane_addr + T::kTmemS0 + g * T::kBlockN + hf * kC;
        const uint32_t t_p = tmem_base + lane_addr + T::kTmemP0 + g * T::kTmemPCols + hf * (kC / 2);
        const uint32_t t_o = tmem_base + lane_addr + T::kTmemO;
        const uint32_t lead_s_free = mapa_shared(bar_s_free(g), 0);
        const uint32_t lead_p_full = mapa_shared(bar_p_full(g), 0);
        const float c = a.scale_log2;

        float m_mine = -INFINITY;  // maximum my sum is taken against (raw score)
        float l_mine = 0.f;        // sum of exp2((s - m_mine) c) over my blocks and columns, from unrounded fp32 p
        bool ok = true;

#pragma unroll 1
        for (int j = g; j < nblk; j += 2) {
            const int n = j >> 1;  // my n-th block
            uint32_t sr[kC];
            float* s = reinterpret_cast<float*>(sr);
            ok = mbar_wait_cluster(bar_s_full(g), static_cast<uint32_t>(n & 1), abort_flag, a.status, kDevSoftmaxWaitS);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            RING_PTRACE(warp == 4 * kH * g && lane == 0, j, 4);
            tcgen05_fence_after_thread_sync();
#pragma unroll
            for (int i = 0; i < kC / 32; ++i)
                tmem_ld_x32(t_s + 32 * i, *reinterpret_cast<uint32_t(*)[32]>(&sr[32 * i]));
            tmem_wait_ld();
            // S is in registers: the buffer is free for block j + 2
            tcgen05_fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_s_free);
            RING_PTRACE(warp == 4 * kH * g && lane == 0, j, 5);

            // masking: only blocks that straddle the causal diagonal or the end of the shard
            const int col0 = j * T::kBlockN;
            int limit = a.sk - col0;                                  // valid columns of this block
            if (a.causal) limit = min(limit, row + a.diag - col0 + 1);  // visible columns of this row
            limit -= hf * kC;                                          // ... counted from this thread's first column
            const bool masked_block = (a.sk - col0 < T::kBlockN) || (a.causal && (r0 + a.diag - col0 + 1) < T::kBlockN);
            if (masked_block) {
#pragma unroll
                for (int i = 0; i < kC; ++i)
                    if (i >= limit) s[i] = -INFINITY;
            }

            // row maximum of the block (of this thread's columns): eight independent chains, then a tree
            float mxc[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) mxc[u] = fmaxf(s[2 * u], s[2 * u + 1]);
#pragma unroll
            for (int i = 16; i < kC; i += 16) {
#pragma unroll
                for (int u = 0; u < 8; ++u) mxc[u] = fmax3(mxc[u], s[i + 2 * u], s[i + 2 * u + 1]);
            }
            float mx = fmaxf(fmax3(mxc[0], mxc[1], mxc[2]), fmax3(fmax3(mxc[3], mxc[4], mxc[5]), mxc[6], mxc[7]));
            if (kH == 2) {
                // the two threads of the row exchange the maxima of their halves (slots alternate with n so that a
                // value is never overwritten before the partner has read it)
                hmax_sh[((g * 2 + hf) * 2 + (n & 1)) * 128 + row_local] = mx;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_half_max(g, quarter));
                ok = mbar_wait(bar_half_max(g, quarter), static_cast<uint32_t>(n & 1), abort_flag, a.status, kDevSoftmaxWaitM);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                mx = fmaxf(mx, hmax_sh[((g * 2 + (hf ^ 1)) * 2 + (n & 1)) * 128 + row_local]);
            }

            // The maximum in use after block j - 1 (kept by the threads of the other block parity); adopt the block's
            // own only when it beats that by more than 2^8, and hand the result on at once.  Every thread of the row
            // computes the same value; the first half stores it, all of them arrive (so that it is overwritten, two
            // blocks later, only after every reader of it has passed).
            float m_prev = -INFINITY;
            RING_PTRACE(warp == 4 * kH * g && lane == 0, j, 13);
            if (j > 0) {
                ok = mbar_wait(bar_m_pub(quarter), static_cast<uint32_t>((j - 1) & 1), abort_flag, a.status, kDevSoftmaxWaitM);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                m_prev = m_sh[((j - 1) & 1) * 128 + row_local];
            }
            RING_PTRACE(warp == 4 * kH * g && lane == 0, j, 6);
            float m_new = m_prev;
            if (mx > m_prev && (m_prev == -INFINITY || (mx - m_prev) * c > kRescaleThresholdLog2)) m_new = mx;
            if (hf == 0) m_sh[(j & 1) * 128 + row_local] = m_new;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_m_pub(quarter));
            const float alpha_o = (m_new != m_prev && m_prev != -INFINITY) ? ex2_approx((m_prev - m_new) * c) : 1.f;
            if (m_mine != m_new) {
                l_mine = (m_mine == -INFINITY) ? 0.f : l_mine * ex2_approx((m_mine - m_new) * c);
                m_mine = m_new;
            }

            // p = exp2(s c - m c), in place, fp32; the sum uses the unrounded values
            const float nms = (m_new == -INFINITY) ? 0.f : -m_new * c;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i < kC; i += 4) {
#pragma unroll
                for (int u = 0; u < 4; u += 2) {
                    float x0, x1;
                    ffma2(x0, x1, s[i + u], s[i + u + 1], c, c, nms, nms);
                    s[i + u] = ex2_approx(x0);
                    s[i + u + 1] = ex2_approx(x1);
                }
                fadd2(a0, a1, a0, a1, s[i], s[i + 1]);
                fadd2(a2, a3, a2, a3, s[i + 2], s[i + 3]);
            }
            l_mine += (a0 + a1) + (a2 + a3);
            RING_PTRACE(warp == 4 * kH * g && lane == 0, j, 7);

            // my P buffer was last read by P(j - 2) V: that product must be complete before it is overwritten
            if (n > 0) {
                ok = mbar_wait_cluster(bar_o_done(g), static_cast<uint32_t>((n - 1) & 1), abort_flag, a.status, kDevSoftmaxWaitO);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            RING_PTRACE(warp == 4 * kH * g && lane == 0, j, 8);
            // O is rescaled only when some row of the warp adopted a new maximum (the threads of a row agree, and share
            // the columns of O); P(j - 1) V (the other parity's block) must be complete first, and P(j) V cannot start
            // before this warp has written P(j)
            if (__any_sync(0xffffffffu, alpha_o != 1.f)) {
                const uint32_t par = static_cast<uint32_t>((g == 0 ? n - 1 : n) & 1);
                ok = mbar_wait_cluster(bar_o_done(g ^ 1), par, abort_flag, a.status, kDevSoftmaxWaitO);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tcgen05_fence_after_thread_sync();
#pragma unroll
                for (int i = 0; i < D / kH / 16; ++i) {  // 16 columns at a time: S is still live in registers
                    uint32_t orr[16];
                    tmem_ld_x16(t_o + hf * (D / kH) + 16 * i, orr);
                    tmem_wait_ld();
#pragma unroll
                    for (int x = 0; x < 16; ++x) orr[x] = __float_as_uint(__uint_as_float(orr[x]) * alpha_o);
                    tmem_st_x16(t_o + hf * (D / kH) + 16 * i, orr);
                }
            }

            // P(j): this thread's probabilities -> columns of 16-bit pairs
            tcgen05_fence_after_thread_sync();
#pragma unroll
            for (int i = 0; i < kC / 32; ++i) {
                uint32_t pk[16];
#pragma unroll
                for (int x = 0; x < 16; ++x)
                    pk[x] = T::kIsBf16 ? pack_bf16x2(s[32 * i + 2 * x], s[32 * i + 2 * x + 1])
                                       : pack_f16x2(s[32 * i + 2 * x], s[32 * i + 2 * x + 1]);
                tmem_st_x16(t_p + 16 * i, pk);
            }
            tmem_wait_st();
            tcgen05_fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_p_full);
            RING_PTRACE(warp == 4 * kH * g && lane == 0, j, 9);
        }

        // ---- the threads of a row meet: (maximum, sum) of each, and the earlier partial's LSE -----------
        const bool row_ok = row < a.sq;
        float* lse_ptr = a.lse + b * a.lse_batch_stride + h * a.lse_head_stride + row;
        const float lse_old = (a.merge && row_ok) ? *lse_ptr : -INFINITY;  // read before it is overwritten below
        xl[((g * kH + hf) * 128 + row_local) * 2 + 0] = m_mine;
        xl[((g * kH + hf) * 128 + row_local) * 2 + 1] = l_mine;
        asm volatile("bar.sync 1, %0;" ::"n"(T::kSoftmaxWarps * 32) : "memory");  // all softmax warps, on every path

        // ---- epilogue: O / l, LSE, optional fold into an earlier partial; every softmax warp writes its 32 rows of
        // D / (2 kHalves) columns
        if (ok && nblk > 0) {
            const int last = nblk - 1;
            ok = mbar_wait_cluster(bar_o_done(last & 1), static_cast<uint32_t>((last >> 1) & 1), abort_flag, a.status, kDevSoftmaxWaitO);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) tcgen05_fence_after_thread_sync();
        }
        if (ok) {
            const float m_f = nblk > 0 ? m_sh[((nblk - 1) & 1) * 128 + row_local] : -INFINITY;  // stored by the threads of the last block
            float l_run = 0.f;
#pragma unroll
            for (int gg = 0; gg < 2 * kH; ++gg) {
                const float mg = xl[(gg * 128 + row_local) * 2 + 0];
                const float lg = xl[(gg * 128 + row_local) * 2 + 1];
                if (mg != -INFINITY) l_run += lg * ex2_approx((mg - m_f) * c);
            }
            const bool have = (nblk > 0) && (l_run > 0.f);
            float w_new = have ? 1.f / l_run : 0.f;  // factor applied to the accumulator in TMEM
            float lse_new = have ? m_f * a.scale + logf(l_run) : -INFINITY;
            float w_old = 0.f;
            if (a.merge && row_ok) {
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
            // O goes out through shared memory so that every store instruction writes whole row pieces: the first half
            // of the softmax warps stages in the Q tile, the second half in the first two K slots (every MMA that read
            // them has completed), 16-byte chunks XOR-swizzled by the row.
            constexpr int kCols = D / (2 * kH);           // columns this warp writes
            constexpr int kChunks = kCols / 4;            // 16-byte chunks per staged row
            constexpr int kRowsPerInst = 32 / kChunks;    // rows one coalesced instruction covers
            const int pass = g * kH + hf;                 // which group of kCols columns
            const uint32_t stage = (warp < 4 * kH ? smem_q : smem_slot(0)) + static_cast<uint32_t>(warp % (4 * kH)) * (32 * kCols * 4);
            const int row_base = r0 + quarter * 32;
            float* o_base = a.o + b * a.o_batch_stride + h * a.o_head_stride;
            float4 old[32 / kRowsPerInst];
            if (a.merge) {
#pragma unroll
                for (int rr = 0; rr < 32 / kRowsPerInst; ++rr) {
                    const int rl = rr * kRowsPerInst + lane / kChunks;
                    old[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (row_base + rl < a.sq)
                        old[rr] = *(reinterpret_cast<const float4*>(o_base + static_cast<int64_t>(row_base + rl) * a.o_row_stride +
                                                                    pass * kCols) + lane % kChunks);
                }
            }
#pragma unroll
            for (int i = 0; i < kCols / 32; ++i) {
                uint32_t orr[32];
                if (nblk > 0) {
                    tmem_ld_x32(t_o + pass * kCols + 32 * i, orr);
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
                    *(reinterpret_cast<float4*>(o_base + static_cast<int64_t>(row_base + rl) * a.o_row_stride + pass * kCols) + ch) = val;
            }
            if (g == 0 && hf == 0 && row_ok) *lse_ptr = lse_new;
        }
    }

    // ---- common exit: every thread of both CTAs arrives here, on success and on a timed-out wait alike ----
    tcgen05_fence_before_thread_sync();
    __syncthreads();
    cluster_sync_all();  // the peer has finished with this CTA's shared memory, tensor memory and barriers
    if (warp == T::kQkWarp) {
        tcgen05_fence_after_thread_sync();
        tmem_dealloc_pair(tmem_base, T::kTmemCols);
    }
}

}  // namespace ring
