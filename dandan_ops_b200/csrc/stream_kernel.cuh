// Weight-streaming kernel for the decode regime (M <= 64 rows of x per launch).
//
// The kernel is bound by HBM and by instruction issue at the same time: every weight
// byte is read exactly once (0.5703 B/weight) and every weight costs about three
// instructions to decode exactly, so both the copy pipeline and the inner loop are kept
// as lean as the arithmetic contract allows.
//
// Work split ("stream-K").  The layer is cut into steps = (group of 16 row tiles = 256
// outputs) x (column block of 256 inputs).  Steps are numbered row-group-major and dealt
// out in equal contiguous ranges to one persistent CTA per SM, so all SMs finish
// together whatever the shape.  A CTA has 16 warps; warp w owns row tile 16*group + w
// and keeps FP32 accumulators for it while the CTA walks along K.  Where a range ends
// inside a row group, the partial tiles go to the workspace in fragment order and the
// last CTA to arrive at that row tile (ticket counter, nobody waits) adds the partials
// in contributor order - so the result does not depend on which CTA came last - writes
// y and re-zeroes the ticket.
//
// Weights: every warp keeps a ring of kStages native blocks in shared memory, filled by
// bulk asynchronous copies (cp.async.bulk, one 2336-byte copy per block, completion
// counted on an mbarrier).  The copies need no registers; with two slots per warp the 16
// warps of an SM hold ~37 KB in flight and 37 KB being decoded.  A lane reads its 73 bytes of
// a landed block with conflict-free 16-byte shared loads and immediately hands the slot back
// to the copy engine.
//
// Activations: x for a phase of up to 33 column blocks (8448 columns; fewer when more than 8
// rows are staged, more when fewer) is staged in shared memory once per CTA, laid out
// [64-column chunk][row][eight 16-byte pieces] with padded rows and chunks so that the
// 16-byte read a lane makes for its MMA B fragments is conflict-free.
//
// Dequantization keeps the reference's arithmetic exactly:
//     w = fp16_rn( fp32(code - zero) * step_fp32 )
// `(word >> 8e) & 0x000F000F | 0x64006400` turns a pair of 4-bit codes into the FP16 pair
// (1024+code); the odd nibbles come out as (1024+16*code).  One mixed-precision
// instruction per weight (add.f32.f16 / fma.f32.f16, sm_100) turns that into the exact
// FP32 integer code-zero, one FP32 multiply applies the step, and cvt.rn.f16x2.f32 rounds
// a pair to FP16 - already laid out as the A fragment of an m16n8k16 MMA whose B
// fragment is x^T (8 rows of x per MMA) and whose accumulators are FP32.
//
// Every wait in the kernel is bounded: a warp that gives up on an mbarrier records
// kStatusCopyTimeout in the status word, stops computing and leaves through the normal
// exit (its outputs are then undefined; the host reads the status word on demand).
#pragma once
#include "layout.cuh"
#include "gather_kernel.cuh"

namespace b2 {

#ifndef B2_STREAM_STAGES
#define B2_STREAM_STAGES 2
#endif
#ifndef B2_STREAM_CTAS16
#define B2_STREAM_CTAS16 1
#endif
constexpr int kStages = B2_STREAM_STAGES;    // ring depth per warp
// Shared-memory footprint of a CTA with W warps (W = 16: one CTA per SM; W = 4: four per SM,
// for layers with too few steps to feed 16-warp CTAs on every SM).
__host__ __device__ constexpr int stream_bar_bytes(int w) { return w * kStages * 8; }
__host__ __device__ constexpr int stream_ring_bytes(int w) { return w * kStages * kBlockBytes; }
// x buffer: a 16-warp CTA (one per SM) takes everything the ring leaves of the 227 KB a CTA may have - with the
// two-block rings 152 KB, i.e. 33 column blocks of 8 staged rows (K = 8448) or 16 of 16 rows; a 4-warp CTA
// (four per SM) 18.5 KB.  Ring depth 2 against 4 was measured level at M = 1 and 3-6 % ahead at M = 8 / 16 on
// the 70B-class layers: one block in flight per warp covers the copy latency (a warp spends ~1.7 us on a
// block), and K = 8192 becomes resident in x at M = 8.
__host__ __device__ constexpr int stream_x_bytes(int w) {
    return w == 16 ? ((232448 - 1024 - w * B2_STREAM_STAGES * 8 - w * B2_STREAM_STAGES * kBlockBytes - 128) / 128) * 128 / B2_STREAM_CTAS16
                   : w * 4736;
}
// Staged x: 64-column chunk T, row m, 16-byte piece c at T*chunk + m*144 + c*16.  Rows are padded
// to 144 bytes and chunks by 32 more, which spreads the eight lanes of a quarter warp (two rows x
// four chunks) over all eight 16-byte bank groups without any address arithmetic per piece.
__host__ __device__ constexpr int stream_x_chunk_bytes(int rows) { return rows * 144 + 32; }
constexpr int kStreamZeroBytes = 128;   // a row of zeros behind the x buffer: the B fragments of rows of x that do not exist
__host__ __device__ constexpr int stream_smem_bytes(int w) {
    return stream_bar_bytes(w) + stream_ring_bytes(w) + stream_x_bytes(w) + kStreamZeroBytes;
}
constexpr unsigned kStatusCopyTimeout = 1u;
constexpr int kWaitLimit = 1 << 20;          // mbarrier polls before a warp gives up

struct StreamArgs {
    const __half* x;        // [M, K], row stride ldx
    const uint8_t* native;  // weight image
    __half* y;              // [M, N], row stride ldy
    float* partial;         // [split tile][max_parts][MT][32 lanes][4]
    unsigned* ticket;       // [split tile], zero on entry and on exit
    unsigned* status;       // sticky error word (0 = ok)
    const __half* bias;     // optional [N] FP16, added to the FP16-rounded product (may be null)
    int64_t ldx, ldy;
    int m, n, k;
    int n16, kb;            // row tiles, column blocks
    int groups;             // row groups = ceil(n16 / W)
    int act;                // 0: y = x W^T (+bias); 1: rows g / g+8 of every 16-row tile are a gate/up pair,
                            //    y[:, 8*tile + g] = silu_mul(gate, up), y has n/2 columns
    int max_parts;          // partial slots per row tile
    int steps;              // groups * kb (below 2^20 for every layer the index checks admit)
    int chunk_blocks;       // w4a16_stream2d_kernel: column blocks per K chunk (all chunks but the last)
    int nchunks;            //   and the number of chunks (0 / 1 in the other kernels)
    int wait_limit;         // mbarrier polls before a warp gives up (kWaitLimit; a test passes a small number)
    int fault_step;         // -1; a test passes n >= 0: warp 0 of CTA 0 arms the barrier of its n-th weight
                            // copy but does not issue the copy, so that the wait for it runs out (only the copies
                            // of the first ring fill, n < B2_STREAM_STAGES, are looked at)
    int overlap;            // launched as a programmatic dependent of the previous kernel: request weights first,
                            // then wait for that kernel before anything else is read or written
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
// fp32(lo half of h2) + c and fp32(hi half) + c: exact conversion plus add, one instruction each.
__device__ __forceinline__ void add_mixed(uint32_t h2, float c, float& lo, float& hi) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "add.rn.f32.f16 %0, l, %3;\n\tadd.rn.f32.f16 %1, h, %3;\n\t}"
        : "=f"(lo), "=f"(hi) : "r"(h2), "f"(c));
}
// fp32(half) * (1/16) + c, exact (the product is an integer below 2^11).
__device__ __forceinline__ void fma_mixed_16th(uint32_t h2, float c, float& lo, float& hi) {
    asm("{\n\t.reg .b16 l, h, s;\n\tmov.b32 {l, h}, %2;\n\tmov.b16 s, 0x2C00;\n\t"
        "fma.rn.f32.f16 %0, l, s, %3;\n\tfma.rn.f32.f16 %1, h, s, %3;\n\t}"
        : "=f"(lo), "=f"(hi) : "r"(h2), "f"(c));
}
// The output rounding of every linear kernel: FP16(acc), then the FP16 bias added in FP16
// (the reference rounds the product first and adds bias.to(fp16) afterwards).
__device__ __forceinline__ __half finish_output(float acc, const __half* bias, int n) {
    const __half h = __float2half_rn(acc);
    return bias ? __hadd(h, bias[n]) : h;
}
// Residual add + RMSNorm on 16-byte pieces (eight FP16 values), with the reference's rounding
// order (dandan_ops/csrc/elementwise.cu:39-62, dandan_ops/elementwise.py:118-120): the sum is
// rounded to FP16 first, the normalized value is rounded to FP16 before the weight multiplies it.
// FP16 -> FP32 conversions go through the mixed-precision FMA-pipe instructions (full rate); the
// plain cvt runs at a quarter of that and made these helpers the bottleneck of the prologue.
__device__ __forceinline__ void unpack_f32(uint32_t h2, float& lo, float& hi) {     // exact, keeps the sign of zero
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "add.rn.f32.f16 %0, l, 0f80000000;\n\tadd.rn.f32.f16 %1, h, 0f80000000;\n\t}"
        : "=f"(lo), "=f"(hi) : "r"(h2));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t add_pair(uint32_t a, uint32_t b) {               // fp16(float(a) + float(b))
    float alo, ahi, lo, hi;
    unpack_f32(a, alo, ahi);
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "add.rn.f32.f16 %0, l, %3;\n\tadd.rn.f32.f16 %1, h, %4;\n\t}"
        : "=f"(lo), "=f"(hi) : "r"(b), "f"(alo), "f"(ahi));
    return pack_f16(lo, hi);
}
__device__ __forceinline__ uint32_t mul_pair(uint32_t a, uint32_t b) {               // fp16(float(a) * float(b)), product exact in FP32
    float lo, hi;
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.f16 %0, al, bl, 0f80000000;\n\tfma.rn.f32.f16 %1, ah, bh, 0f80000000;\n\t}"
        : "=f"(lo), "=f"(hi) : "r"(a), "r"(b));
    return pack_f16(lo, hi);
}
__device__ __forceinline__ uint4 add_piece(const uint4& x, const uint4& r) {
    return make_uint4(add_pair(x.x, r.x), add_pair(x.y, r.y), add_pair(x.z, r.z), add_pair(x.w, r.w));
}
__device__ __forceinline__ float sumsq_piece(const uint4& v, float acc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float lo, hi;
        unpack_f32(w[i], lo, hi);
        acc = fmaf(lo, lo, acc);
        acc = fmaf(hi, hi, acc);
    }
    return acc;
}
__device__ __forceinline__ uint4 norm_piece(const uint4& v, float inverse, const uint4& w) {
    const uint32_t a[4] = {v.x, v.y, v.z, v.w}, g[4] = {w.x, w.y, w.z, w.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float lo, hi;
        unpack_f32(a[i], lo, hi);
        o[i] = mul_pair(pack_f16(lo * inverse, hi * inverse), g[i]);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
constexpr int kNormSlices = 8;       // a row's sum of squares is added in eight lane-strided slices
// Sum over a warp in a fixed order (the same in the fused prologue and in the standalone kernel).
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float inverse_rms(float sumsq, int k, float eps) {
    return 1.0f / sqrtf(sumsq / float(k) + eps);
}

// SiLU(gate) * up on FP16 values with the reference's rounding order: the activation is rounded
// to FP16 before the multiplication (dandan_ops/csrc/elementwise.cu:70-73,
// `torch.nn.functional.silu(gate) * up` on the CPU route).
__device__ __forceinline__ __half silu_mul(__half gate, __half up) {
    const float v = __half2float(gate);
    const __half act = __float2half_rn(v / (1.0f + expf(-v)));
    return __float2half_rn(__half2float(act) * __half2float(up));
}
// Exact dequantization of one FP16 pair, `1024 + code` (even nibbles) or `1024 + 16 * code` (odd
// nibbles), to fp16_rn(fp32(code - zero) * step): a mixed-precision add (or fma by 1/16) gives
// the exact FP32 integer, one FP32 multiply applies the step (one IEEE rounding), cvt rounds the
// pair to FP16.  The two multiplies go out as one packed mul.rn.f32x2 - same rounding per element,
// one issue slot instead of two, and instruction issue is what bounds the dequantization; the
// whole pair is one asm block so that the register pairs of the packed operands need no moves,
// and the step arrives already duplicated in a 64-bit register (`twice()`, once per group).
#ifndef B2_PACKED_FMUL
#define B2_PACKED_FMUL 1
#endif
__device__ __forceinline__ uint64_t twice(float s) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(s));
    return r;
}
__device__ __forceinline__ float low_of(uint64_t s2) { return __uint_as_float(uint32_t(s2)); }
// c = -(1024 + zero)
__device__ __forceinline__ uint32_t dequant_pair_even(uint32_t h2, float c, uint64_t s2) {
#if B2_PACKED_FMUL
    uint32_t r;
    asm("{\n\t.reg .b16 l, h;\n\t.reg .f32 x, y;\n\t.reg .b64 a;\n\t"
        "mov.b32 {l, h}, %1;\n\t"
        "add.rn.f32.f16 x, l, %2;\n\tadd.rn.f32.f16 y, h, %2;\n\t"
        "mov.b64 a, {x, y};\n\tmul.rn.f32x2 a, a, %3;\n\tmov.b64 {x, y}, a;\n\t"
        "cvt.rn.f16x2.f32 %0, y, x;\n\t}"
        : "=r"(r) : "r"(h2), "f"(c), "l"(s2));
    return r;
#else
    float lo, hi;
    add_mixed(h2, c, lo, hi);
    __half2 p = __floats2half2_rn(__fmul_rn(lo, low_of(s2)), __fmul_rn(hi, low_of(s2)));
    return *reinterpret_cast<uint32_t*>(&p);
#endif
}
// c = -(64 + zero): (1024 + 16 * code) / 16 + c, exact (the product is an integer below 2^11)
__device__ __forceinline__ uint32_t dequant_pair_odd(uint32_t h2, float c, uint64_t s2) {
#if B2_PACKED_FMUL
    uint32_t r;
    asm("{\n\t.reg .b16 l, h, q;\n\t.reg .f32 x, y;\n\t.reg .b64 a;\n\t"
        "mov.b32 {l, h}, %1;\n\tmov.b16 q, 0x2C00;\n\t"
        "fma.rn.f32.f16 x, l, q, %2;\n\tfma.rn.f32.f16 y, h, q, %2;\n\t"
        "mov.b64 a, {x, y};\n\tmul.rn.f32x2 a, a, %3;\n\tmov.b64 {x, y}, a;\n\t"
        "cvt.rn.f16x2.f32 %0, y, x;\n\t}"
        : "=r"(r) : "r"(h2), "f"(c), "l"(s2));
    return r;
#else
    float lo, hi;
    fma_mixed_16th(h2, c, lo, hi);
    __half2 p = __floats2half2_rn(__fmul_rn(lo, low_of(s2)), __fmul_rn(hi, low_of(s2)));
    return *reinterpret_cast<uint32_t*>(&p);
#endif
}
// ---- the two dequantization chains behind one interface -------------------------------------
// Exact<false>: the general chain above (FP32 step, FP32 multiply, one cvt per pair).
// Exact<true> ("FP16 steps"): for layers whose steps are all exactly representable in FP16 - checkpoints
// that store FP16 scales - the product (code - zero) * step has at most 15 significant bits, so it is exact
// in FP32 and fp16_rn(fp32(code - zero) * step) == hmul2(code - zero, step): one FP16 subtract (or fma by
// 1/16 for the odd nibbles) and one FP16 multiply per pair, bit-identical to the general chain.
template <bool H16> struct GroupConst;
template <> struct GroupConst<false> {
    float c_even, c_odd;     // -(1024 + z), -(64 + z)
    uint64_t s2;             // the step, twice
};
template <> struct GroupConst<true> {
    uint32_t z_even, z_odd;  // FP16 pairs (1024 + z), -(64 + z)
    uint32_t s2;             // FP16 pair (step, step)
};
template <bool H16>
__device__ __forceinline__ GroupConst<H16> make_group(uint32_t z, float step) {
    GroupConst<H16> g;
    if constexpr (H16) {
        g.z_even = 0x64006400u + z * 0x00010001u;          // 1024 has ulp 1: z sits in the mantissa
        g.z_odd = 0xD400D400u + z * 0x00100010u;           // -(64 + z): 64 has ulp 1/16
        asm("cvt.rn.f16x2.f32 %0, %1, %1;" : "=r"(g.s2) : "f"(step));
    } else {
        // -(1024 + z) and -(64 + z) as FP32 bit patterns: z sits in the mantissa, no int-to-float conversion
        g.c_even = __uint_as_float(0xC4800000u + z * 8192u);
        g.c_odd = __uint_as_float(0xC2800000u + z * 131072u);
        g.s2 = twice(step);
    }
    return g;
}
template <bool H16>
__device__ __forceinline__ uint32_t dq_even(uint32_t h2, const GroupConst<H16>& g) {      // h2 = (1024 + code) pair
    if constexpr (H16) {
        uint32_t r;
        asm("{\n\t.reg .b32 d;\n\tsub.rn.f16x2 d, %1, %2;\n\tmul.rn.f16x2 %0, d, %3;\n\t}"
            : "=r"(r) : "r"(h2), "r"(g.z_even), "r"(g.s2));
        return r;
    } else {
        return dequant_pair_even(h2, g.c_even, g.s2);
    }
}
template <bool H16>
__device__ __forceinline__ uint32_t dq_odd(uint32_t h2, const GroupConst<H16>& g) {       // h2 = (1024 + 16 * code) pair
    if constexpr (H16) {
        uint32_t r;
        asm("{\n\t.reg .b32 d, q;\n\tmov.b32 q, 0x2C002C00;\n\tfma.rn.f16x2 d, %1, q, %2;\n\tmul.rn.f16x2 %0, d, %3;\n\t}"
            : "=r"(r) : "r"(h2), "r"(g.z_odd), "r"(g.s2));
        return r;
    } else {
        return dequant_pair_odd(h2, g.c_odd, g.s2);
    }
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int limit = kWaitLimit) {
    if (mbar_try_wait(bar, parity)) return true;           // the common case costs no loop bookkeeping
    for (int i = 1; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t pick(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// One 16-byte piece of x: global -> shared without passing through registers (XVEC) so that all
// pieces of a thread are in flight at once, or assembled from 2-byte loads for unaligned x.
template <bool XVEC, bool ASYNC = true>
__device__ __forceinline__ void stage_piece(uint8_t* dst, const __half* src, bool inside, int k, int kmax) {
    if (!inside) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    } else if constexpr (XVEC && ASYNC) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
    } else if constexpr (XVEC) {
        *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
    } else {
        uint32_t h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
            h[e] = (k + e < kmax) ? uint32_t(__half_as_ushort(__ldg(src + e))) : 0u;
        *reinterpret_cast<uint4*>(dst) = make_uint4(h[0] | h[1] << 16, h[2] | h[3] << 16, h[4] | h[5] << 16, h[6] | h[7] << 16);
    }
}
// Wait for this thread's asynchronous pieces (the caller follows with a block-wide barrier).
__device__ __forceinline__ void stage_wait() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Stage x[0..rows) x [k0, k0 + cols) into shared memory (zero beyond M and K).  `rows` = MT * 8, or, in the
// streaming kernel at MT = 1, only the rows of x that exist; `chunk` = stream_x_chunk_bytes(rows).
template <int MT, bool XVEC, int W, bool WAIT = true>
__device__ __forceinline__ void stage_x(uint8_t* xs, const StreamArgs& a, int k0, int cols, int rows = MT * 8,
                                        int chunk = stream_x_chunk_bytes(MT * 8)) {
    // Work item = (row, column block): 32 pieces, one per lane, dealt to the warps in turn
    // (`cols` is a multiple of 256).
    const int items = rows * (cols >> 8);
    const int lane = threadIdx.x & 31;
    for (int it = threadIdx.x >> 5; it < items; it += W) {
        const int blk = it / rows, m = it - blk * rows, cc = blk * 32 + lane;
        const int T = cc >> 3, c = cc & 7;
        const int k = k0 + cc * 8;
        stage_piece<XVEC>(xs + T * chunk + m * 144 + c * 16, a.x + int64_t(m) * a.ldx + k,
                          m < a.m && k < a.k, k, a.k);
    }
    if constexpr (WAIT) stage_wait();
}

// Index of the CTA whose range contains step s (ranges are [c*steps/G, (c+1)*steps/G)).
__device__ __forceinline__ int owner_of(int s, int steps, int ctas) {
    return int((unsigned(s + 1) * unsigned(ctas) - 1u) / unsigned(steps));
}

// MT = number of 8-row tiles of x (1, 2, 4 or 8).  XVEC: x rows are 16-byte aligned and
// K is a multiple of 8, so x is read with 16-byte loads.
// GATHER: the multi-GPU form.  `a.y` is this rank's column slice of a full [M, N] buffer that every rank
// holds (GatherArgs, csrc/gather_kernel.cuh).  The warp that completes a row tile stores it into the local
// buffer AND sends it to every peer's mailbox as {word, epoch} packets (plain peer stores over NVLink, as
// soon as the tile is done - the transfer overlaps the rest of the stream); a CTA that has finished its
// range polls its share of the packets the peers sent and copies them into the local buffer.  When the
// kernel ends the local buffer holds all slices: projection and all-gather in one launch.  Nothing reads a
// peer's memory; every wait is bounded (status bit 2 of the flag block on a timeout).  A CTA waits only for
// packets of OTHER GPUs, whose senders never wait before they send, so the launch needs no co-residency
// with anything but its own grid (the host checks that the whole grid fits on the device at once).
// XROWS (MT = 1 only): stage just the rows of x that exist.  The row count is then a run-time number in the
// x addressing of every block (measured: 28 more instructions per block at M = 8, 13 fewer at M = 1, where most
// lanes read the zero row), so batches of 5 to 8 rows use the compile-time layout of all 8 rows instead.
template <int MT, bool XVEC, int W, bool H16, bool GATHER, bool XROWS>
__device__ __forceinline__ void stream_body(const StreamArgs& a, const GatherArgs* ga) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MP = MT * 8;
    constexpr int kWarps = W;
    constexpr int kBarBytes = stream_bar_bytes(W), kRingBytes = stream_ring_bytes(W);
    // Up to 8 rows of x only the rows that exist are staged (rows beyond M are zero B fragments, read from a
    // 128-byte row of zeros): at M = 1 the x buffer of a 16-warp CTA then holds 244 column blocks instead of
    // 33, so x is staged once per CTA for every K up to 62 000 and the CTA never stops for an x phase again.
    const int xrows = (MT == 1 && XROWS) ? a.m : MP;
    // rows of 144 bytes, padded so that consecutive chunks sit 32 bytes apart modulo 128: the eight lanes of a
    // quarter warp (two rows, four chunks) then read eight different 16-byte bank groups for any row count
    const int kChunk = xrows * 144 + ((32 - xrows * 16) & 127);
    const int kPhaseBlocks = stream_x_bytes(W) / (4 * kChunk);      // W=16, all rows staged: 33, 16, 8, 4 column blocks
    static_assert(stream_x_bytes(W) / (4 * stream_x_chunk_bytes(MP)) >= 1, "x phase must hold at least one column block");

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ctas = gridDim.x;
    // 32-bit step arithmetic: steps * ctas stays below 2^31 (steps < 2^20, at most ~1200 CTAs)
    const int b0 = int((unsigned(a.steps) * blockIdx.x) / unsigned(ctas));
    const int b1 = int((unsigned(a.steps) * (blockIdx.x + 1)) / unsigned(ctas));

    // This warp's tile exists in every row group except possibly the last one.
    const bool in_last = (a.groups - 1) * kWarps + warp < a.n16;
    const int last_start = (a.groups - 1) * a.kb;
    const int wb1 = in_last ? b1 : (b1 < last_start ? b1 : last_start);   // end of this warp's steps

    const uint32_t bar0 = smem_u32(smem) + warp * kStages * 8;
    uint8_t* ring = smem + kBarBytes + warp * kStages * kBlockBytes;
    const uint32_t ring0 = smem_u32(ring);
    uint8_t* xs = smem + kBarBytes + kRingBytes;

    // When all of K fits in the x buffer it is staged once for the whole kernel: x does not
    // depend on the row group, so the CTA never has to stop between row groups again.  The
    // copies are issued first and awaited after the weight requests, so both latencies overlap
    // (the other order was measured 5 % slower on 24576 x 4096: every CTA reads the same lines of x,
    // and that fan-in, not the weights' first trip, is the longer way at the start).
    const bool whole_x = a.kb <= kPhaseBlocks;
    uint8_t* xzero = xs + stream_x_bytes(W);
    if (threadIdx.x < kStreamZeroBytes / 16) reinterpret_cast<uint4*>(xzero)[threadIdx.x] = make_uint4(0, 0, 0, 0);
    // Kernels launched behind this one as programmatic dependents may move onto SMs as they become free
    // (no effect otherwise).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (whole_x && !a.overlap) stage_x<MT, XVEC, W, false>(xs, a, 0, a.kb * kBlockCols, xrows, kChunk);

    // Copy-request cursor (used by lane 0): image block (fkb, 16*fgrp + warp).  Consecutive
    // column blocks of one row tile are `stride` bytes apart; at the end of a row group the
    // cursor jumps to the first column block of the next group.
    const long long stride = (long long)a.n16 * kBlockBytes;
    int fetch = b0;                // next step to request
    int fgrp = int(b0 / a.kb);
    int fkb = b0 - fgrp * a.kb;
    const uint8_t* fptr = a.native + ((long long)fkb * a.n16 + fgrp * kWarps + warp) * kBlockBytes;
    const int fault = (a.fault_step >= 0 && blockIdx.x == 0 && warp == 0) ? a.fault_step : -1;   // test hook, see StreamArgs
    auto request = [&](int slot, bool skip = false) {
        mbar_expect_tx(bar0 + slot * 8, kBlockBytes);
        if (!skip) bulk_copy_g2s(ring0 + slot * kBlockBytes, fptr, kBlockBytes, bar0 + slot * 8);
        ++fetch;
        fptr += stride;
        if (++fkb == a.kb) {
            fkb = 0;
            ++fgrp;
            fptr = a.native + (long long)(fgrp * kWarps + warp) * kBlockBytes;
        }
    };
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
#pragma unroll
        for (int s = 0; s < kStages; ++s)
            if (fetch < wb1) request(s, s == fault);       // (test hook: one of the first copies left out)
    }
    __syncwarp();
    if (a.overlap) {
        // Weights are constant; everything else (x, bias, tickets, partial tiles, y) may belong to the previous
        // kernel of the stream until it has completed and its writes are visible.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (whole_x) stage_x<MT, XVEC, W, false>(xs, a, 0, a.kb * kBlockCols, xrows, kChunk);
    }

    // With one row tile of x the sixteen MMAs of a block would be ONE dependent chain; two accumulator tiles used
    // in turn make it two chains of eight (with more row tiles the tiles are independent chains already).
    constexpr bool kTwoChains = MT == 1;
    float acc[MT][4], acc2[kTwoChains ? MT : 1][4];
    int stage = 0;
    uint32_t parity = 0;
    bool failed = false;

    if (whole_x) {
        stage_wait();
        __syncthreads();
    }

    int s0 = b0;
    while (s0 < b1) {                                       // one iteration per row group in the range
        const int grp = s0 / a.kb;
        const int k_lo = s0 - grp * a.kb;
        const int k_hi = min(a.kb, k_lo + (b1 - s0));
        const int nt = grp * kWarps + warp;
        const bool active = nt < a.n16;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                acc[mt][c] = 0.0f;
                if constexpr (kTwoChains) acc2[mt][c] = 0.0f;
            }

        for (int p0 = k_lo; p0 < k_hi; p0 += kPhaseBlocks) {
            const int p1 = min(k_hi, p0 + kPhaseBlocks);
            if (!whole_x) {
                __syncthreads();                           // everyone is done with the previous x phase
                stage_x<MT, XVEC, W>(xs, a, p0 * kBlockCols, (p1 - p0) * kBlockCols, xrows, kChunk);
                __syncthreads();
            }
            const int xorigin = whole_x ? 0 : p0;          // column block that the x buffer starts at
            if (!active || failed) continue;
            for (int kb = p0; kb < p1; ++kb) {
                if (!mbar_wait(bar0 + stage * 8, parity, a.wait_limit)) {
                    failed = true;
                    if (lane == 0) atomicOr(a.status, kStatusCopyTimeout);
                    break;
                }
                const uint8_t* slot = ring + stage * kBlockBytes;
                uint4 code[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) code[j] = *reinterpret_cast<const uint4*>(slot + j * 512 + lane * 16);
                const float2 step = *reinterpret_cast<const float2*>(slot + kStepOffset + lane * 8);
                const uint32_t zero = slot[kZeroOffset + lane];
                __syncwarp();                              // all lanes have read the slot
                if (lane == 0 && fetch < wb1) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    request(stage);
                }
                if (++stage == kStages) { stage = 0; parity ^= 1u; }

                const GroupConst<H16> gg = make_group<H16>(zero & 15u, step.x), gh = make_group<H16>(zero >> 4, step.y);
                const uint8_t* xchunk = (MT > 1 || g < xrows) ? xs + ((kb - xorigin) * 4 + t) * kChunk + g * 144 : xzero;
#pragma unroll
                for (int wi = 0; wi < 8; ++wi) {
                    const uint32_t wa = pick(code[wi >> 2], wi & 3);        // row g
                    const uint32_t wb = pick(code[2 + (wi >> 2)], wi & 3);  // row g+8
                    uint4 xv[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        xv[mt] = *reinterpret_cast<const uint4*>(xchunk + mt * (8 * 144) + wi * 16);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const uint32_t ua = wa >> (8 * e), ub = wb >> (8 * e);
                        const uint32_t w[4] = {dq_even<H16>(and_or(ua, 0x000F000Fu, 0x64006400u), gg),
                                               dq_even<H16>(and_or(ub, 0x000F000Fu, 0x64006400u), gh),
                                               dq_odd<H16>(and_or(ua, 0x00F000F0u, 0x64006400u), gg),
                                               dq_odd<H16>(and_or(ub, 0x00F000F0u, 0x64006400u), gh)};
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            if (e == 0 || !kTwoChains) mma_16816(acc[mt], w, e ? xv[mt].z : xv[mt].x, e ? xv[mt].w : xv[mt].y, acc[mt]);
                            else mma_16816(acc2[mt], w, xv[mt].z, xv[mt].w, acc2[mt]);
                    }
                }
            }
        }

        if constexpr (kTwoChains) {            // (a fixed order: results do not depend on timing)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[mt][c] += acc2[mt][c];
        }
        if (active && !failed) {
            const bool whole = (k_lo == 0 && k_hi == a.kb);
            bool write_out = whole;
            if (!whole) {
                // Contributors to this row group are the CTAs first..last; mine is slot `blockIdx.x - first`.
                const int gs = grp * a.kb;
                const int first = owner_of(gs, a.steps, ctas), last = owner_of(gs + a.kb - 1, a.steps, ctas);
                const int parts = last - first + 1;
                // Row groups that are split between CTAs are few: at most one per CTA boundary.
                // Both `grp` and `first` are unique among them; use whichever range is smaller.
                const int tile = (a.groups <= ctas ? grp : first) * kWarps + warp;
                float4* base = reinterpret_cast<float4*>(a.partial) + (long long)tile * a.max_parts * (MT * 32) + lane;
                float4* mine = base + (long long)(blockIdx.x - first) * (MT * 32);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                    __stcg(mine + mt * 32, make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]));
                __threadfence();
                __syncwarp();
                unsigned prior = 0;
                if (lane == 0) prior = atomicAdd(a.ticket + tile, 1u);
                prior = __shfl_sync(0xffffffffu, prior, 0);
                if (prior == unsigned(parts - 1)) {
                    __threadfence();
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[mt][c] = 0.0f;
                    for (int s = 0; s < parts; ++s) {
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const float4 p = __ldcg(base + (long long)s * (MT * 32) + mt * 32);
                            acc[mt][0] += p.x; acc[mt][1] += p.y; acc[mt][2] += p.z; acc[mt][3] += p.w;
                        }
                    }
                    if (lane == 0) a.ticket[tile] = 0u;
                    write_out = true;
                }
            }
            if (GATHER && write_out) {
                // Lanes g and g ^ 1 exchange one value each, so that every lane holds the two neighbouring
                // columns of one row as a 4-byte word: the unit of the local store and of a packet.
                const unsigned epoch = mailbox_epoch(*ga);
                const int64_t wpr = ga->cols >> 1;
                const bool even = (g & 1) == 0;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int m0 = mt * 8 + 2 * t;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int n = nt * 16 + g + 8 * h;
                        const unsigned v0 = (m0 < a.m && n < a.n) ? __half_as_ushort(finish_output(acc[mt][2 * h], a.bias, n)) : 0u;
                        const unsigned v1 = (m0 + 1 < a.m && n < a.n) ? __half_as_ushort(finish_output(acc[mt][2 * h + 1], a.bias, n)) : 0u;
                        const unsigned got = __shfl_xor_sync(0xffffffffu, even ? v1 : v0, 4);
                        const int row = even ? m0 : m0 + 1, col = even ? n : n - 1;
                        const unsigned word = even ? (v0 | (got << 16)) : (got | (v1 << 16));
                        if (row < a.m && col < a.n) {
                            *reinterpret_cast<unsigned*>(a.y + int64_t(row) * a.ldy + col) = word;
                            const int64_t s = int64_t(row) * wpr + (col >> 1);
                            for (int q = 0; q < ga->world; ++q)
                                if (q != ga->rank)
                                    mailbox_send(mailbox(ga->flags[q], ga->world, ga->slots, epoch & 1u, ga->rank) + s, word, epoch);
                        }
                    }
                }
            } else if (write_out) {
                const int n0 = nt * 16 + g;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int m0 = mt * 8 + 2 * t;
                    if (a.act) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {           // this thread holds the gate (row g) and up (row g+8) sums
                            const int m = m0 + c;
                            if (m < a.m && n0 + 8 < a.n)
                                a.y[int64_t(m) * a.ldy + nt * 8 + g] = silu_mul(finish_output(acc[mt][c], a.bias, n0),
                                                                               finish_output(acc[mt][c + 2], a.bias, n0 + 8));
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int m = m0 + (c & 1), n = n0 + 8 * (c >> 1);
                            if (m < a.m && n < a.n) a.y[int64_t(m) * a.ldy + n] = finish_output(acc[mt][c], a.bias, n);
                        }
                    }
                }
            }
        }
        s0 += k_hi - k_lo;
    }

    if (failed) {
        // Let copies that are still in flight land before the CTA's shared memory is released
        // (a bounded look at every slot of this warp's ring).
        for (int s = 0; s < kStages; ++s) {
            bool landed = false;
            for (int i = 0; i < 4096 && !landed; ++i) landed = mbar_try_wait(bar0 + stage * 8, parity);
            if (++stage == kStages) { stage = 0; parity ^= 1u; }
        }
    }

    if constexpr (GATHER) {
        const unsigned epoch = mailbox_epoch(*ga);
        const int64_t threads = int64_t(gridDim.x) * blockDim.x;
        mailbox_finish(*ga, epoch, mailbox_receive(*ga, epoch, int64_t(blockIdx.x) * blockDim.x + threadIdx.x, threads));
    }
}

template <int MT, bool XVEC, int W, bool H16 = false, bool XROWS = false>
__global__ void __launch_bounds__(W * 32, (W == 16 ? B2_STREAM_CTAS16 : 4))
w4a16_stream_kernel(const StreamArgs a) {
    stream_body<MT, XVEC, W, H16, false, XROWS>(a, nullptr);
}

template <int MT, int W, bool H16, bool XROWS = false>
__global__ void __launch_bounds__(W * 32, (W == 16 ? B2_STREAM_CTAS16 : 4))
w4a16_stream_gather_kernel(const StreamArgs a, const GatherArgs ga) {
    stream_body<MT, true, W, H16, true, XROWS>(a, &ga);
}

}  // namespace b2
