// Compile-time shape configuration of the block-attention kernel.
//
// Same template signature and constant names as the reference's Ring_kernel_traits /
// Ring_fwd_traits<kHeadDim, kBlockM, kBlockN, kNWarps, elem> (csrc/kernel_traits.h:11-44, 47-177):
// kNWarps, kNThreads, kBlockM, kBlockN, kHeadDim, kSmemSize, Element, ElementAccum, index_t.
// The contents are sm_100a: TMA boxes with the 128-byte swizzle instead of cp.async tiled copies,
// tcgen05 UMMA shapes instead of the mma.sync TiledMma, a TMEM column budget, a K/V stage ring and
// warp roles.  No CuTe types.
#pragma once

#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <type_traits>

template <int kHeadDim_, int kBlockM_, int kBlockN_, int kNWarps_, typename elem_type = __half>
struct Ring_kernel_traits
{
    using Element = elem_type;
    using ElementAccum = float;
    using index_t = int64_t;
    static constexpr bool kIsBf16 = std::is_same<elem_type, __nv_bfloat16>::value;

    // UMMA instruction shape (cta_group::1): M x N x 16 for 16-bit operands.
    static constexpr int kUmmaM = 128;
    static constexpr int kUmmaK = 16;
    // One TMA box / one swizzle row = 64 elements = 128 bytes.
    static constexpr int kSwizzleElems = 64;
    static constexpr int kSwizzleAtomBytes = 1024;  // 8 rows x 128 B
};

template <int kHeadDim_, int kBlockM_, int kBlockN_, int kNWarps_, typename elem_type = __half,
          typename Base = Ring_kernel_traits<kHeadDim_, kBlockM_, kBlockN_, kNWarps_, elem_type>>
struct Ring_fwd_traits : public Base
{
    using Element = typename Base::Element;
    using ElementAccum = typename Base::ElementAccum;
    using index_t = typename Base::index_t;

    static constexpr int kNWarps = kNWarps_;
    static constexpr int kNThreads = kNWarps * 32;

    static constexpr int kBlockM = kBlockM_;  // Q rows per CTA = kQTiles x 128
    static constexpr int kBlockN = kBlockN_;  // K/V rows per pipeline stage
    static constexpr int kHeadDim = kHeadDim_;

    static_assert(kHeadDim == 64 || kHeadDim == 128, "head dimension must be 64 or 128");
    static_assert(kBlockM == 256, "a CTA owns two 128-row Q tiles");
    static_assert(kBlockN == 128, "K/V blocks are 128 rows");

    // ---- warp roles -----------------------------------------------------------------------
    static constexpr int kQTiles = kBlockM / Base::kUmmaM;       // 2: ping-pong pair
    static constexpr int kSoftmaxWarps = 4 * kQTiles;            // one warpgroup per Q tile, 1 thread = 1 row
    static constexpr int kMmaWarp = kSoftmaxWarps;               // warp 8: issues S = Q K^T; warps 9, 10: P V of tile 0, 1
    static constexpr int kLoadWarp = kSoftmaxWarps + 3;          // warp 11: single-thread TMA issue
    static_assert(kNWarps == kSoftmaxWarps + 4, "8 softmax warps + one producer warpgroup (3 UMMA issuers, 1 loader)");
    // Registers after setmaxnreg: 256 softmax threads x kSoftmaxRegs + 128 producer threads x kProducerRegs <= 64 Ki
    static constexpr int kSoftmaxRegs = 216;
    static constexpr int kProducerRegs = 72;
    static_assert(256 * kSoftmaxRegs + 128 * kProducerRegs <= 65536, "register file");


    // ---- shared memory ----------------------------------------------------------------------
    static constexpr int kBoxesPerTile = kHeadDim / Base::kSwizzleElems;       // TMA boxes per 128-row tile
    static constexpr int kBoxBytes = 128 * Base::kSwizzleElems * 2;            // 16 KiB
    static constexpr int kTileBytes = kBoxesPerTile * kBoxBytes;               // one 128 x kHeadDim tile
    static constexpr int kStages = kHeadDim == 128 ? 5 : 8;                    // K/V slots in shared memory
    static constexpr int kKStages = kHeadDim == 128 ? 2 : 3;                   // ... of which the K ring
    static constexpr int kVStages = kStages - kKStages;                        // ... and the V ring
    static constexpr int kNumBarriers = 2 /*q_full*/ + 2 * kStages + 3 * kQTiles /*s_full,p_full,o_done*/ + 1 /*s_free*/;
    static constexpr int kSmemTiles = (kQTiles + kStages) * kTileBytes;
    static constexpr int kSmemSize = kSmemTiles + 1024 /*alignment slack*/ + 256 /*barriers, TMEM slot, flags*/;
    static_assert(kSmemSize <= 227 * 1024, "exceeds the 227 KiB per-CTA limit");

    // ---- tensor memory (512 columns x 128 lanes x 32 bit) ------------------------------------------
    static constexpr int kTmemCols = 512;
    static constexpr int kTmemS = 0;                  // ONE S buffer (128 fp32 columns) used by the two Q tiles in turn
    static constexpr int kTmemPCols = kBlockN / 2;    // 16-bit P of a tile: 64 columns of its own
    static constexpr int kTmemP0 = kBlockN;           // P tile t at kTmemP0 + t*kTmemPCols
    static constexpr int kTmemO0 = kBlockN + kQTiles * kTmemPCols;  // O tile t at kTmemO0 + t*kHeadDim
    static_assert(kTmemO0 + kQTiles * kHeadDim <= kTmemCols, "TMEM budget");
};

// Shape configuration of the CTA-PAIR form of the block-attention kernel (head dimension 128).
//
// Two CTAs of a cluster own 128 Q rows each and walk the K/V shard together: every tcgen05.mma is a cta_group::2
// instruction of M = 256 whose B operand is split between the two CTAs' shared memories, so each CTA loads only
// half of every K block (64 keys) and half of every V block (64 of the 128 value columns).  Per CTA that is the
// K/V stream of a 256-row CTA, which leaves shared memory for deep K/V rings and, with one Q tile instead of two,
// tensor memory for TWO S buffers: S of block j + 1 is computed while block j is still in its softmax.
// Same constant names as Ring_fwd_traits where they mean the same thing.
template <int kHeadDim_, typename elem_type = __half, int kHalves_ = 1,
          typename Base = Ring_kernel_traits<kHeadDim_, 128, 128, 8 * kHalves_ + 4, elem_type>>
struct Ring_pair_traits : public Base
{
    using Element = typename Base::Element;
    using ElementAccum = typename Base::ElementAccum;
    using index_t = typename Base::index_t;

    // kHalves = 1: one softmax thread per Q row and block parity (8 softmax warps, two per scheduler);
    // kHalves = 2: two threads per row, 64 of the block's 128 columns each (16 softmax warps, four per scheduler,
    // to overlap the latencies of the load / max / pack phases and of the barrier waits).
    static constexpr int kHalves = kHalves_;
    static_assert(kHalves == 1 || kHalves == 2, "one or two threads per row");
    static constexpr int kSoftmaxWarps = 8 * kHalves;
    static constexpr int kNWarps = kSoftmaxWarps + 4;
    static constexpr int kNThreads = kNWarps * 32;
    static constexpr int kBlockM = 128;        // Q rows per CTA (256 per pair)
    static constexpr int kBlockN = 128;        // K/V rows per block (64 of them, or 64 value columns, per CTA)
    static constexpr int kHeadDim = kHeadDim_;
    static_assert(kHeadDim == 128, "the pair form is instantiated for head dimension 128");

    // softmax warp w: TMEM lane quarter w & 3, column half (w >> 2) & (kHalves - 1), block parity w >> (1 + kHalves);
    // then one producer warpgroup: TMEM allocation and (leader CTA) issuer of S = Q K^T; (leader) issuer of O += P V;
    // TMA loads of V; TMA loads of Q and K (K slots are released early, V slots late: one thread for both would
    // hold the K loads back behind a V slot that is still being read).
    static constexpr int kQkWarp = kSoftmaxWarps;
    static constexpr int kPvWarp = kSoftmaxWarps + 1;
    static constexpr int kLoadWarpV = kSoftmaxWarps + 2;
    static constexpr int kLoadWarp = kSoftmaxWarps + 3;
    static constexpr int kSoftmaxRegs = kHalves == 1 ? 216 : 112;
    static constexpr int kProducerRegs = kHalves == 1 ? 72 : 32;
    static_assert(kSoftmaxWarps * 32 * kSoftmaxRegs + 128 * kProducerRegs <= 65536, "register file");
    // setmaxnreg.inc blocks until the CTA's own pool holds the registers, and that pool is only what setmaxnreg.dec
    // gave back (registers of the SM that the launch never assigned to the CTA do not count: a form that relied on
    // them never came back from the first setmaxnreg.inc).  Registers per thread at launch: 65536 / threads, in eights.
    static constexpr int kLaunchRegs = (65536 / kNThreads) / 8 * 8;
    static_assert((kLaunchRegs - kProducerRegs) * 128 >= (kSoftmaxRegs - kLaunchRegs) * kSoftmaxWarps * 32,
                  "the producer warpgroup must give back at least what the softmax warps take");

    static constexpr int kBoxBytesQ = 128 * Base::kSwizzleElems * 2;   // Q box: 64 columns x 128 rows = 16 KiB
    static constexpr int kQBytes = (kHeadDim / 64) * kBoxBytesQ;        // 32 KiB
    static constexpr int kBoxBytesK = 64 * Base::kSwizzleElems * 2;    // K box of this CTA: 64 columns x 64 keys = 8 KiB
    static constexpr int kSlotBytes = 16 * 1024;                        // half a K block (2 boxes) or half a V block (1 box of 128 keys)
    static constexpr int kKStages = 4;
    static constexpr int kVStages = 4;
    static constexpr int kStages = kKStages + kVStages;
    static constexpr int kNumBarriers = 1 /*q_full*/ + 2 * kStages + 2 /*s_full*/ + 2 /*s_free*/ + 2 /*p_full*/ + 2 /*o_done*/ +
                                        4 /*m_pub*/ + 8 /*half_max*/;
    static constexpr int kSmemTiles = kQBytes + kStages * kSlotBytes;
    // tail: barriers, TMEM slot, flags | running maxima [2][128] | block maxima of the halves [2][2][2][128] | (m, l) [4][128][2]
    static constexpr int kTailMaxima = 512, kTailHalfMax = 1536, kTailSums = 5632, kTailBytes = 10240;
    static constexpr int kSmemSize = kSmemTiles + 1024 /*alignment slack*/ + kTailBytes;
    static_assert(kNumBarriers * 8 + 64 <= kTailMaxima && kTailSums + 4 * 128 * 2 * 4 <= kTailBytes, "tail layout");
    static_assert(kSmemSize <= 227 * 1024, "exceeds the 227 KiB per-CTA limit");

    // tensor memory: S of even blocks, S of odd blocks, P of even / odd blocks (16-bit pairs), O
    static constexpr int kTmemCols = 512;
    static constexpr int kTmemS0 = 0;
    static constexpr int kTmemP0 = 256;
    static constexpr int kTmemPCols = 64;
    static constexpr int kTmemO = 384;
    static_assert(kTmemO + kHeadDim <= kTmemCols, "TMEM budget");
};
