// Weight-streaming kernel for the decode regime (M <= 64 rows of x per launch).
//
// The kernel is bound by HBM: every weight byte is read exactly once, 0.5703 B/weight.
// A CTA of eight warps owns eight neighbouring row tiles (128 outputs) and one K-split;
// each warp walks the native blocks of its own tile along K.
//
// Weights: every warp keeps a ring of kStages blocks in shared memory, filled by bulk
// asynchronous copies (cp.async.bulk, one 2336-byte copy per block, completion counted
// on an mbarrier).  The copies need no registers, so 16 warps per SM hold ~150 KB in
// flight - several times what HBM latency x bandwidth asks for.  A lane reads its 73
// bytes of a landed block with conflict-free 16-byte shared loads and immediately hands
// the slot back to the copy engine.
//
// Activations: x for a phase of up to 2048 columns is staged in shared memory once per
// CTA, laid out [64-column chunk][row][eight 16-byte pieces, XOR-swizzled] so that the
// 16-byte read a lane makes for its MMA B fragments is conflict-free.
//
// Dequantization keeps the reference's arithmetic exactly:
//     w = fp16_rn( fp32(code - zero) * step_fp32 )
// but does the integer->FP32 conversion on the tensor cores.  `(word >> 8e) & 0x000F000F
// | 0x64006400` turns a pair of 4-bit codes into the FP16 pair (1024+code); the codes of
// the odd nibbles come out as (1024+16*code).  An m16n8k8 MMA of those raw fragments
// with a constant selection matrix (identity, or identity/16) and the accumulator
// preset to -(1024+zero) or -(64+zero) returns fp32(code - zero) for exactly the
// elements the lane holds - every product and sum is an integer below 2^11, so nothing
// is rounded.  One FP32 multiply by the step and one cvt.rn.f16x2.f32 finish the weight,
// already laid out as the A fragment of the product MMA.  x^T is the B operand
// (8 rows of x per MMA), accumulators are FP32.
//
// Split-K: partial tiles go to the workspace in fragment order; the last warp to arrive
// at a row tile (ticket counter, no waiting) adds the partials in split order - the
// result does not depend on which warp came last - writes y and re-zeroes the ticket.
//
// Every wait in the kernel is bounded: a warp that gives up on an mbarrier records
// kStatusCopyTimeout in the status word, stops computing and leaves through the normal
// exit (its outputs are then undefined; the host reads the status word on demand).
#pragma once
#include "layout.cuh"

namespace b2 {

constexpr int kStages = 4;                   // ring depth per warp
constexpr int kWarps = 8;                    // warps (row tiles) per CTA
constexpr int kBarBytes = 256;               // 8 warps x 4 stages x 8 B
constexpr int kRingBytes = kWarps * kStages * kBlockBytes;   // 74752
constexpr int kXBytes = 32768;               // staged activations per phase
constexpr int kStreamSmem = kBarBytes + kRingBytes + kXBytes;
constexpr unsigned kStatusCopyTimeout = 1u;
constexpr int kWaitLimit = 1 << 20;          // mbarrier polls before a warp gives up

struct StreamArgs {
    const __half* x;        // [M, K], row stride ldx
    const uint8_t* native;  // weight image
    __half* y;              // [M, N], row stride ldy
    float* partial;         // [splits][n16][MT][32 lanes][4] when splits > 1
    unsigned* ticket;       // [n16], zero on entry and on exit
    unsigned* status;       // sticky error word (0 = ok)
    int64_t ldx, ldy;
    int m, n, k;
    int n16, kb;            // row tiles, column blocks
    int kb_per_item;        // column blocks per K-split
    int splits;
};

// ---- small PTX helpers ------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return uint32_t(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t bits) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(bits));
    return r;
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1),
          "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
__device__ __forceinline__ void mma_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0,
                                         const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
// (lo*s, hi*s) rounded to an FP16 pair; each multiply is one IEEE FP32 rounding.
__device__ __forceinline__ uint32_t scale_pack(float lo, float hi, float s) {
    __half2 h = __floats2half2_rn(__fmul_rn(lo, s), __fmul_rn(hi, s));
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: false if the phase did not complete within kWaitLimit polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

struct BlockRegs {
    uint4 code[4];   // piece j: rows g (j<2) / g+8 (j>=2), words 4*(j&1)..4*(j&1)+3
    float2 step;     // (row g, row g+8)
    uint32_t zero;   // zero(row g) | zero(row g+8) << 4
};

__device__ __forceinline__ uint32_t pick(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// Stage x[0..MT*8) x [k0, k0 + cols) into shared memory (zero beyond M and K).
// Piece (row m, 64-column chunk T, 16-byte piece c) lands at ((T*MP + m)*8 + (c ^ key))*16
// with key = ((m & 1) << 2) | (T & 3).
template <int MT, bool XVEC>
__device__ __forceinline__ void stage_x(uint4* xs, const StreamArgs& a, int k0, int cols) {
    constexpr int MP = MT * 8;
    const int pieces_per_row = cols >> 3;
    const int total = MP * pieces_per_row;
    for (int i = threadIdx.x; i < total; i += 256) {
        const int m = i / pieces_per_row, cc = i - m * pieces_per_row;
        const int T = cc >> 3, c = cc & 7;
        const int k = k0 + cc * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < a.m && k < a.k) {
            const __half* src = a.x + int64_t(m) * a.ldx + k;
            if constexpr (XVEC) {
                v = __ldg(reinterpret_cast<const uint4*>(src));
            } else {
                uint32_t h[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    h[e] = (k + e < a.k) ? uint32_t(__half_as_ushort(__ldg(src + e))) : 0u;
                v = make_uint4(h[0] | h[1] << 16, h[2] | h[3] << 16, h[4] | h[5] << 16, h[6] | h[7] << 16);
            }
        }
        const int key = ((m & 1) << 2) | (T & 3);
        xs[(T * MP + m) * 8 + (c ^ key)] = v;
    }
}

// MT = number of 8-row tiles of x (1, 2, 4 or 8).  XVEC: x rows are 16-byte aligned and
// K is a multiple of 8, so x is read with 16-byte loads.
template <int MT, bool XVEC>
__global__ void __launch_bounds__(256, 2)
w4a16_stream_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MP = MT * 8;
    constexpr int kPhaseCols = kXBytes / (MP * 2);       // 2048, 1024, 512, 256
    constexpr int kPhaseBlocks = kPhaseCols / kBlockCols;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nt = blockIdx.x * kWarps + warp;
    const bool active = nt < a.n16;
    const int ks = blockIdx.y;
    const int kb0 = ks * a.kb_per_item;
    const int kb1 = min(a.kb, kb0 + a.kb_per_item);

    const uint32_t bar0 = smem_u32(smem) + warp * kStages * 8;
    uint8_t* ring = smem + kBarBytes + warp * kStages * kBlockBytes;
    const uint32_t ring0 = smem_u32(ring);
    uint4* xs = reinterpret_cast<uint4*>(smem + kBarBytes + kRingBytes);

    const int64_t stride = int64_t(a.n16) * kBlockBytes;
    const uint8_t* src = a.native + (int64_t(kb0) * a.n16 + (active ? nt : 0)) * kBlockBytes;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (active) {
#pragma unroll
            for (int s = 0; s < kStages; ++s)
                if (kb0 + s < kb1) {
                    mbar_expect_tx(bar0 + s * 8, kBlockBytes);
                    bulk_copy_g2s(ring0 + s * kBlockBytes, src + s * stride, kBlockBytes, bar0 + s * 8);
                }
        }
    }
    __syncwarp();

    // selection matrices of the conversion MMAs, as B fragments of this lane
    const uint32_t sel1 = (2 * t == g) ? 0x00003C00u : (2 * t + 1 == g) ? 0x3C000000u : 0u;  // 1.0
    const uint32_t sel16 = (2 * t == g) ? 0x00002C00u : (2 * t + 1 == g) ? 0x2C000000u : 0u; // 1/16
    const int xkey = ((g & 1) << 2) | t;

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mt][c] = 0.0f;

    int stage = 0;
    uint32_t parity = 0;
    bool failed = false;

    for (int p0 = kb0; p0 < kb1; p0 += kPhaseBlocks) {
        __syncthreads();                                   // everyone is done with the previous phase's x
        stage_x<MT, XVEC>(xs, a, p0 * kBlockCols, min(kPhaseBlocks, kb1 - p0) * kBlockCols);
        __syncthreads();
        if (!active || failed) continue;
        const int p1 = min(kb1, p0 + kPhaseBlocks);
        for (int kb = p0; kb < p1; ++kb) {
            if (!mbar_wait(bar0 + stage * 8, parity)) {
                failed = true;
                if (lane == 0) atomicOr(a.status, kStatusCopyTimeout);
                break;
            }
            const uint8_t* slot = ring + stage * kBlockBytes;
            BlockRegs cur;
#pragma unroll
            for (int j = 0; j < 4; ++j) cur.code[j] = *reinterpret_cast<const uint4*>(slot + j * 512 + lane * 16);
            cur.step = *reinterpret_cast<const float2*>(slot + kStepOffset + lane * 8);
            cur.zero = slot[kZeroOffset + lane];
            __syncwarp();                                  // all lanes have read the slot
            if (lane == 0 && kb + kStages < kb1) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(bar0 + stage * 8, kBlockBytes);
                bulk_copy_g2s(ring0 + stage * kBlockBytes, src + int64_t(kb - kb0 + kStages) * stride,
                              kBlockBytes, bar0 + stage * 8);
            }
            if (++stage == kStages) { stage = 0; parity ^= 1u; }

            const float zg = float(cur.zero & 15u), zh = float(cur.zero >> 4);
            const float c1[4] = {-(1024.0f + zg), -(1024.0f + zg), -(1024.0f + zh), -(1024.0f + zh)};
            const float c2[4] = {-(64.0f + zg), -(64.0f + zg), -(64.0f + zh), -(64.0f + zh)};
            const float sg = cur.step.x, sh = cur.step.y;
            const uint4* xchunk = xs + ((kb - p0) * 4 + t) * (MP * 8) + g * 8;
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) {
                const uint32_t wa = pick(cur.code[wi >> 2], wi & 3);        // row g
                const uint32_t wb = pick(cur.code[2 + (wi >> 2)], wi & 3);  // row g+8
                uint4 xv[MT];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) xv[mt] = xchunk[mt * 64 + (wi ^ xkey)];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t ua = wa >> (8 * e), ub = wb >> (8 * e);
                    float d1[4], d2[4];
                    mma_1688(d1, and_or(ua, 0x000F000Fu, 0x64006400u), and_or(ub, 0x000F000Fu, 0x64006400u),
                             sel1, c1);                     // columns 0,1 of the quad: code - zero
                    mma_1688(d2, and_or(ua, 0x00F000F0u, 0x64006400u), and_or(ub, 0x00F000F0u, 0x64006400u),
                             sel16, c2);                    // columns 2,3
                    const uint32_t w[4] = {scale_pack(d1[0], d1[1], sg), scale_pack(d1[2], d1[3], sh),
                                           scale_pack(d2[0], d2[1], sg), scale_pack(d2[2], d2[3], sh)};
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        mma_16816(acc[mt], w, e ? xv[mt].z : xv[mt].x, e ? xv[mt].w : xv[mt].y, acc[mt]);
                }
            }
        }
    }
    if (!active) return;
    if (failed) {
        // Let copies that are still in flight land before the CTA's shared memory is released.
        for (int s = 0; s < kStages; ++s) {
            bool landed = false;
            for (int i = 0; i < 4096 && !landed; ++i) landed = mbar_try_wait(bar0 + stage * 8, parity);
            if (!landed) break;
            if (++stage == kStages) { stage = 0; parity ^= 1u; }
        }
        return;
    }

    const int n0 = nt * 16 + g;
    if (a.splits > 1) {
        float4* mine = reinterpret_cast<float4*>(a.partial) + (int64_t(ks) * a.n16 + nt) * (MT * 32) + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
            __stcg(mine + mt * 32, make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]));
        __threadfence();
        __syncwarp();
        unsigned prior = 0;
        if (lane == 0) prior = atomicAdd(a.ticket + nt, 1u);
        prior = __shfl_sync(0xffffffffu, prior, 0);
        if (prior != unsigned(a.splits - 1)) return;
        __threadfence();
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mt][c] = 0.0f;
        const float4* part = reinterpret_cast<const float4*>(a.partial) + int64_t(nt) * (MT * 32) + lane;
        for (int s = 0; s < a.splits; ++s) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const float4 p = __ldcg(part + mt * 32);
                acc[mt][0] += p.x; acc[mt][1] += p.y; acc[mt][2] += p.z; acc[mt][3] += p.w;
            }
            part += int64_t(a.n16) * (MT * 32);
        }
        if (lane == 0) a.ticket[nt] = 0u;
    }

#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int m0 = mt * 8 + 2 * t;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int m = m0 + (c & 1), n = n0 + 8 * (c >> 1);
            if (m < a.m && n < a.n) a.y[int64_t(m) * a.ldy + n] = __float2half_rn(acc[mt][c]);
        }
    }
}

}  // namespace b2
