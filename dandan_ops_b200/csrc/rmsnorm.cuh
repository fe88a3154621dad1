// Residual add + RMSNorm of one row, shared by the standalone norm kernel and the tile kernel's fused
// prologue, so that both produce the same bits.  Rounding order of the reference
// (dandan_ops/csrc/elementwise.cu:39-62, dandan_ops/elementwise.py:118-120): the sum is rounded to FP16
// first, the normalized value is rounded to FP16 before the weight multiplies it.
#pragma once
#include "stream_kernel.cuh"

namespace b2 {

constexpr int kNormThreads = 32 * kNormSlices;       // the first 256 threads of the CTA do the work

struct NormScratch {                                   // shared memory of one row's reduction
    float slice[kNormSlices];
    float inverse;
};

// One row: summed = fp16(x + residual) (to `sums`: the caller's `summed` row, or the output row when the sum is
// not wanted), out = fp16(fp16(s * inverse_rms(s)) * weight).  Every thread of the CTA must call it (it
// contains block-wide barriers); threads beyond kNormThreads only take part in the barriers.  The sum of
// squares is added in eight lane-strided slices (one per warp), butterfly inside a slice, slices in order: a
// fixed order, so the result does not depend on the launch.
__device__ __forceinline__ void norm_row(const __half* x, const __half* residual, const __half* weight, float eps,
                                         __half* sums, __half* out, int k, NormScratch& sm) {
    const int pieces = k >> 3;
    constexpr int kStride = kNormThreads, kBatch = 4;  // loads in flight per thread; the sum keeps the order of the pieces
    const bool worker = threadIdx.x < kNormThreads;
    float sq = 0.0f;
    if (worker) {
        for (int c0 = threadIdx.x; c0 < pieces; c0 += kStride * kBatch) {
            uint4 v[kBatch], r[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                const int cc = c0 + kStride * j;
                v[j] = cc < pieces ? __ldg(reinterpret_cast<const uint4*>(x + cc * 8)) : make_uint4(0, 0, 0, 0);
                r[j] = (cc < pieces && residual) ? __ldg(reinterpret_cast<const uint4*>(residual + cc * 8)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                const int cc = c0 + kStride * j;
                if (cc < pieces) {
                    if (residual) v[j] = add_piece(v[j], r[j]);
                    *reinterpret_cast<uint4*>(sums + cc * 8) = v[j];
                    sq = sumsq_piece(v[j], sq);
                }
            }
        }
        sq = warp_sum(sq);
        if ((threadIdx.x & 31) == 0) sm.slice[threadIdx.x >> 5] = sq;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
#pragma unroll
        for (int p = 0; p < kNormSlices; ++p) total += sm.slice[p];
        sm.inverse = inverse_rms(total, k, eps);
    }
    __syncthreads();
    if (worker) {
        const float inverse = sm.inverse;
        for (int c0 = threadIdx.x; c0 < pieces; c0 += kStride * kBatch) {      // every thread re-reads only what it wrote itself
            uint4 v[kBatch], w[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                const int cc = c0 + kStride * j;
                if (cc < pieces) {
                    v[j] = *reinterpret_cast<const uint4*>(sums + cc * 8);
                    w[j] = __ldg(reinterpret_cast<const uint4*>(weight + cc * 8));
                }
            }
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                const int cc = c0 + kStride * j;
                if (cc < pieces) *reinterpret_cast<uint4*>(out + cc * 8) = norm_piece(v[j], inverse, w[j]);
            }
        }
    }
}

}  // namespace b2
