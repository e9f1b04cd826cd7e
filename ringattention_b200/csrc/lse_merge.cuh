// Cross-step merge kernel: folds the partial (O, LSE) of one ring step into the running result.
//
// The reference never materialises partials: it keeps one running (max, sum, O) in registers across
// the PE loop and divides once at the end (csrc/ring_attention.cu:439-443, 456, 597-598, 621-633).
// With one kernel launch per ring step that state has to live in memory, as a normalised output and
// its natural-log row LSE; two such partials of the same rows combine as
//     lse' = mx + ln(e^{lse_a - mx} + e^{lse_b - mx}),   mx = max(lse_a, lse_b)
//     O'   = e^{lse_a - lse'} O_a + e^{lse_b - lse'} O_b
// A partial whose LSE is -inf (every key masked) contributes nothing; two such give O = 0, LSE = -inf.
//
// HBM-bound elementwise work: per row it reads 2 x (D + 1) floats and writes D + 1 floats, i.e.
// (3 D + 3) * 4 bytes.  One warp per row, 16-byte accesses, grid-stride over rows.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace ring {

template <int D>
__global__ void __launch_bounds__(256)
ring_lse_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc, const float* __restrict__ o_part,
                      const float* __restrict__ lse_part, int64_t rows) {
    static_assert(D % 128 == 0 || D == 64, "one warp covers a row with float4 (D=128) or float2 (D=64) lanes");
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t r = warp0; r < rows; r += nwarps) {
        const float la = lse_acc[r];
        const float lb = lse_part[r];
        const float mx = fmaxf(la, lb);
        float wa = 0.f, wb = 0.f, lnew = -INFINITY;
        if (mx != -INFINITY) {
            const float ea = expf(la - mx);
            const float eb = expf(lb - mx);
            const float tot = ea + eb;
            wa = ea / tot;
            wb = eb / tot;
            lnew = mx + logf(tot);
        }
        if constexpr (D == 64) {
            float2* pa = reinterpret_cast<float2*>(o_acc + r * D) + lane;
            const float2 x = *pa;
            const float2 y = *(reinterpret_cast<const float2*>(o_part + r * D) + lane);
            float2 z;
            z.x = wa * x.x + wb * y.x;
            z.y = wa * x.y + wb * y.y;
            *pa = z;
        } else {
#pragma unroll
            for (int i = 0; i < D / 128; ++i) {
                float4* pa = reinterpret_cast<float4*>(o_acc + r * D) + i * 32 + lane;
                const float4 x = *pa;
                const float4 y = *(reinterpret_cast<const float4*>(o_part + r * D) + i * 32 + lane);
                float4 z;
                z.x = wa * x.x + wb * y.x;
                z.y = wa * x.y + wb * y.y;
                z.z = wa * x.z + wb * y.z;
                z.w = wa * x.w + wb * y.w;
                *pa = z;
            }
        }
        if (lane == 0) lse_acc[r] = lnew;
    }
}

}  // namespace ring
