// Load-time kernels: packing, relayout between the reference tensors and the native
// image, and the exact dequantizers.  All are plain gather/scatter kernels bound by HBM
// traffic; none is on the per-token path.
#pragma once
#include "layout.cuh"

namespace b2 {

// One CTA per native block: 128 threads write 512 code words, 64 steps, 32 zero bytes.
__global__ void __launch_bounds__(128)
repack_kernel(const int32_t* __restrict__ packed, const float* __restrict__ scales,
              const int32_t* __restrict__ zeros, Dims d, uint8_t* __restrict__ native) {
    const int64_t blk = blockIdx.x;
    const int kb = int(blk / d.n16), nt = int(blk - int64_t(kb) * d.n16);
    uint8_t* base = native + blk * kBlockBytes;
    uint32_t* code = reinterpret_cast<uint32_t*>(base);
    for (int idx = threadIdx.x; idx < 512; idx += 128) {
        const int j = idx >> 7, lane = (idx >> 2) & 31, i = idx & 3;
        const int g = lane >> 2, t = lane & 3;
        const int row = nt * 16 + g + 8 * (j >> 1);
        const int grp = kb * 4 + t;
        const int k0 = kb * 256 + t * 64 + (4 * (j & 1) + i) * 8;
        uint32_t out = 0;
        if (row < d.n && grp < d.groups) {
            const uint32_t z = uint32_t(zeros[int64_t(row) * d.groups + grp]) & 15u;
            const int valid = d.k - k0;   // columns of this word that exist (may be <= 0 or >= 8)
            const uint32_t ref = valid > 0 ? uint32_t(packed[int64_t(row) * d.words + (k0 >> 3)]) : 0u;
            out = permute_word(ref, valid < 0 ? 0 : (valid > 8 ? 8 : valid), z);
        }
        code[idx] = out;
    }
    if (threadIdx.x < 64) {
        const int lane = threadIdx.x >> 1, h = threadIdx.x & 1;
        const int row = nt * 16 + (lane >> 2) + 8 * h, grp = kb * 4 + (lane & 3);
        float s = 1.0f;
        if (row < d.n && grp < d.groups) s = scales[int64_t(row) * d.groups + grp];
        reinterpret_cast<float*>(base + kStepOffset)[threadIdx.x] = s;
    } else if (threadIdx.x < 96) {
        const int lane = threadIdx.x - 64;
        const int grp = kb * 4 + (lane & 3);
        uint32_t z = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = nt * 16 + (lane >> 2) + 8 * h;
            if (row < d.n && grp < d.groups)
                z |= (uint32_t(zeros[int64_t(row) * d.groups + grp]) & 15u) << (4 * h);
        }
        base[kZeroOffset + lane] = uint8_t(z);
    }
}

// One thread per reference word / per (row, group) entry.
__global__ void __launch_bounds__(256)
unrepack_kernel(const uint8_t* __restrict__ native, Dims d, int32_t* __restrict__ packed,
                float* __restrict__ scales, int32_t* __restrict__ zeros) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t total_words = int64_t(d.n) * d.words;
    if (idx < total_words) {
        const int row = int(idx / d.words), cw = int(idx - int64_t(row) * d.words);
        const WordRef w = locate(d, row, cw);
        const uint32_t nat = reinterpret_cast<const uint32_t*>(native + w.block)[w.word];
        const int valid = d.k - cw * 8;
        packed[idx] = int32_t(unpermute_word(nat, valid > 8 ? 8 : valid));
    }
    const int64_t total_groups = int64_t(d.n) * d.groups;
    if (idx < total_groups) {
        const int row = int(idx / d.groups), grp = int(idx - int64_t(row) * d.groups);
        const WordRef w = locate(d, row, grp * 8);
        const uint8_t* base = native + w.block;
        scales[idx] = reinterpret_cast<const float*>(base + kStepOffset)[w.meta];
        zeros[idx] = (base[kZeroOffset + (w.meta >> 1)] >> (4 * (w.meta & 1))) & 15;
    }
}

// codes uint8 [N,K] -> int32 words, one thread per word.
__global__ void __launch_bounds__(256)
pack_kernel(const uint8_t* __restrict__ codes, Dims d, int32_t* __restrict__ packed) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= int64_t(d.n) * d.words) return;
    const int row = int(idx / d.words), cw = int(idx - int64_t(row) * d.words);
    const uint8_t* src = codes + int64_t(row) * d.k + cw * 8;
    const int valid = min(8, d.k - cw * 8);
    uint32_t out = 0;
    for (int c = 0; c < valid; ++c) out |= (uint32_t(src[c]) & 15u) << (4 * c);
    packed[idx] = int32_t(out);
}

// One thread per (row, eight columns): w = fp32(code - zero) * step, one FP32 rounding,
// optionally followed by the FP16 rounding of the linear path.
template <typename Out>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint8_t* __restrict__ native, Dims d, Out* __restrict__ out, int64_t ldo) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= int64_t(d.n) * d.words) return;
    const int row = int(idx / d.words), cw = int(idx - int64_t(row) * d.words);
    const WordRef w = locate(d, row, cw);
    const uint8_t* base = native + w.block;
    const uint32_t nat = reinterpret_cast<const uint32_t*>(base)[w.word];
    const float step = reinterpret_cast<const float*>(base + kStepOffset)[w.meta];
    const int zero = (base[kZeroOffset + (w.meta >> 1)] >> (4 * (w.meta & 1))) & 15;
    const int valid = min(8, d.k - cw * 8);
    Out* dst = out + int64_t(row) * ldo + cw * 8;
    for (int c = 0; c < valid; ++c) {
        const int q = int((nat >> (4 * nibble_slot(c))) & 15u);
        const float v = __fmul_rn(float(q - zero), step);
        if constexpr (sizeof(Out) == 2) dst[c] = __float2half_rn(v);
        else dst[c] = v;
    }
}

}  // namespace b2
