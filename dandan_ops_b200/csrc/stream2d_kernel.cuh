// Streaming kernel with a two-dimensional work split, for large layers whose K range does not fit in
// the x buffer (M <= 16).
//
// w4a16_stream_kernel numbers its steps row-group-major, so a CTA walks along K inside a row group and
// has to re-stage x every `phase` column blocks, between two block-wide barriers, for every row group
// it touches: measured 8 % of a 57344 x 8192 launch at M = 8 and twice that at M = 16.  Here the K
// range is cut into `nchunks` chunks that fit in the x buffer and the steps are numbered chunk-major:
//     step = (chunk, row group, column block inside the chunk)
// A CTA's contiguous range of steps then lies inside one chunk (at most it crosses one chunk
// boundary), stages that chunk's columns of x ONCE and walks down the row groups without ever
// stopping again.  The price: every row tile now gets its sum from `nchunks` (or a few more) CTAs, so
// every tile goes through the partial-tile / ticket protocol - the last CTA to arrive adds the
// partials in slot order (chunk, then CTA), which keeps the result independent of timing.  That is
// ~3 % more L2 traffic on the 70B-class layers and removes all x phases.
//
// Measured: correct and bit-reproducible, but 2-8 % SLOWER than the one-dimensional split on the 8B/70B
// projections (57344 x 8192 at M = 8: 95.6 against 90.6 us; at M = 16: 114 against 106): the fence and
// ticket round trip that now ends every (chunk, row group) segment stalls a warp longer than the x
// phases did.  It runs only when a test hook asks for it (b2_w4a16_test_hooks, stream_variant 4).
//
// Same ring of bulk copies per warp, same dequantization chains, same output stage as
// w4a16_stream_kernel; only the step order, the cursor and the slot arithmetic differ.
#pragma once
#include "stream_kernel.cuh"

namespace b2 {

// Geometry of the chunk-major numbering (cb = blocks per chunk, all chunks but the last).
struct Split2D {
    int groups, kb, cb, nchunks;
    __device__ __forceinline__ int len(int c) const { return c == nchunks - 1 ? kb - c * cb : cb; }
    __device__ __forceinline__ int offset(int c) const { return groups * c * cb; }             // first step of chunk c
    __device__ __forceinline__ void locate(int s, int& c, int& grp, int& j) const {
        c = min(s / (groups * cb), nchunks - 1);
        const int r = s - offset(c), l = len(c);
        grp = r / l;
        j = r - grp * l;
    }
};

template <int MT, bool XVEC, bool H16>
__global__ void __launch_bounds__(16 * 32, 1)
w4a16_stream2d_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int W = 16, MP = MT * 8;
    constexpr int kBarBytes = stream_bar_bytes(W), kRingBytes = stream_ring_bytes(W);
    const int xrows = MT == 1 ? a.m : MP;                       // only the rows of x that exist (see stream_kernel.cuh)
    const int kChunk = xrows * 144 + ((32 - xrows * 16) & 127);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ctas = gridDim.x;
    const int b0 = int((unsigned(a.steps) * blockIdx.x) / unsigned(ctas));
    const int b1 = int((unsigned(a.steps) * (blockIdx.x + 1)) / unsigned(ctas));
    const Split2D sp{a.groups, a.kb, a.chunk_blocks, a.nchunks};
    const bool in_last = (a.groups - 1) * W + warp < a.n16;    // this warp's tile exists in the last row group

    const uint32_t bar0 = smem_u32(smem) + warp * kStages * 8;
    uint8_t* ring = smem + kBarBytes + warp * kStages * kBlockBytes;
    const uint32_t ring0 = smem_u32(ring);
    uint8_t* xs = smem + kBarBytes + kRingBytes;
    uint8_t* xzero = xs + stream_x_bytes(W);
    if (threadIdx.x < kStreamZeroBytes / 16) reinterpret_cast<uint4*>(xzero)[threadIdx.x] = make_uint4(0, 0, 0, 0);

    // ---- copy-request cursor: (fc, fg, fj) = the step `fs`; steps of the last row group are skipped by
    // warps whose tile does not exist there (they come as whole segments in this numbering) -------------
    int fs = b0, fc, fg, fj;
    sp.locate(b0, fc, fg, fj);
    auto skip_foreign = [&]() {                                 // leave a segment of the last row group this warp has no tile in
        while (!in_last && fg == a.groups - 1 && fs < b1) {
            fs += sp.len(fc) - fj;                              // to the first step of the next chunk
            ++fc; fg = 0; fj = 0;
        }
    };
    skip_foreign();
    int fault = (a.fault_step >= 0 && blockIdx.x == 0 && warp == 0) ? a.fault_step : -1;   // test hook, see StreamArgs
    auto request = [&](int slot) {
        if (lane == 0) {
            const uint8_t* src = a.native + ((long long)(fc * sp.cb + fj) * a.n16 + fg * W + warp) * kBlockBytes;
            mbar_expect_tx(bar0 + slot * 8, kBlockBytes);
            if (fault != 0) bulk_copy_g2s(ring0 + slot * kBlockBytes, src, kBlockBytes, bar0 + slot * 8);
        }
        --fault;
        ++fs;
        if (++fj == sp.len(fc)) {
            fj = 0;
            if (++fg == a.groups) { fg = 0; ++fc; }
        }
        skip_foreign();
    };

    // x of the first chunk first (every CTA reads the same lines: the longer way at the start), then the requests
    int c0, g0, j0;
    sp.locate(b0, c0, g0, j0);
    int staged = c0;
    stage_x<MT, XVEC, W, false>(xs, a, c0 * sp.cb * kBlockCols, sp.len(c0) * kBlockCols, xrows, kChunk);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
#pragma unroll
    for (int s = 0; s < kStages; ++s)
        if (fs < b1) request(s);
    stage_wait();
    __syncthreads();

    float acc[MT][4];
    int stage = 0;
    uint32_t parity = 0;
    bool failed = false;

    int s0 = b0;
    while (s0 < b1) {                                           // one iteration per (chunk, row group) segment of the range
        int c, grp, j;
        sp.locate(s0, c, grp, j);
        const int len_c = sp.len(c);
        const int j_hi = min(len_c, j + (b1 - s0));
        if (c != staged) {                                      // the range crosses into the next chunk: once per CTA at most
            __syncthreads();
            stage_x<MT, XVEC, W>(xs, a, c * sp.cb * kBlockCols, len_c * kBlockCols, xrows, kChunk);
            __syncthreads();
            staged = c;
        }
        const int nt = grp * W + warp;
        const bool active = nt < a.n16;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][e] = 0.0f;

        if (active && !failed) {
            for (int jj = j; jj < j_hi; ++jj) {
                if (!mbar_wait(bar0 + stage * 8, parity, a.wait_limit)) {
                    failed = true;
                    if (lane == 0) atomicOr(a.status, kStatusCopyTimeout);
                    break;
                }
                const uint8_t* slot = ring + stage * kBlockBytes;
                uint4 code[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) code[q] = *reinterpret_cast<const uint4*>(slot + q * 512 + lane * 16);
                const float2 step = *reinterpret_cast<const float2*>(slot + kStepOffset + lane * 8);
                const uint32_t zero = slot[kZeroOffset + lane];
                __syncwarp();                                   // all lanes have read the slot
                if (fs < b1) {
                    if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    request(stage);
                }
                if (++stage == kStages) { stage = 0; parity ^= 1u; }

                const GroupConst<H16> gg = make_group<H16>(zero & 15u, step.x), gh = make_group<H16>(zero >> 4, step.y);
                const uint8_t* xchunk = (MT > 1 || g < xrows) ? xs + (jj * 4 + t) * kChunk + g * 144 : xzero;
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
                            mma_16816(acc[mt], w, e ? xv[mt].z : xv[mt].x, e ? xv[mt].w : xv[mt].y, acc[mt]);
                    }
                }
            }
        }

        if (active && !failed) {
            // Contributors to this row tile: for every chunk the CTAs that own a piece of its segment of this row
            // group.  Lane l looks at chunk l; a prefix sum over the lanes gives this CTA's slot (chunks in order,
            // CTAs in order inside a chunk) and the number of contributors.
            int nown = 0, first = 0;
            if (lane < sp.nchunks) {
                const int st = sp.offset(lane) + grp * sp.len(lane);
                first = owner_of(st, a.steps, ctas);
                nown = owner_of(st + sp.len(lane) - 1, a.steps, ctas) - first + 1;
            }
            int incl = nown;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int parts = __shfl_sync(0xffffffffu, incl, 31);
            const int my_slot = __shfl_sync(0xffffffffu, incl - nown, c) + (int(blockIdx.x) - __shfl_sync(0xffffffffu, first, c));
            float4* base = reinterpret_cast<float4*>(a.partial) + (long long)nt * a.max_parts * (MT * 32) + lane;
            float4* mine = base + (long long)my_slot * (MT * 32);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                __stcg(mine + mt * 32, make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]));
            __threadfence();
            __syncwarp();
            unsigned prior = 0;
            if (lane == 0) prior = atomicAdd(a.ticket + nt, 1u);
            prior = __shfl_sync(0xffffffffu, prior, 0);
            if (prior == unsigned(parts - 1)) {
                __threadfence();
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[mt][e] = 0.0f;
                for (int s = 0; s < parts; ++s) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const float4 p = __ldcg(base + (long long)s * (MT * 32) + mt * 32);
                        acc[mt][0] += p.x; acc[mt][1] += p.y; acc[mt][2] += p.z; acc[mt][3] += p.w;
                    }
                }
                if (lane == 0) a.ticket[nt] = 0u;
                const int n0 = nt * 16 + g;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int m0 = mt * 8 + 2 * t;
                    if (a.act) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {           // this thread holds the gate (row g) and up (row g+8) sums
                            const int m = m0 + e;
                            if (m < a.m && n0 + 8 < a.n)
                                a.y[int64_t(m) * a.ldy + nt * 8 + g] = silu_mul(finish_output(acc[mt][e], a.bias, n0),
                                                                               finish_output(acc[mt][e + 2], a.bias, n0 + 8));
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int m = m0 + (e & 1), n = n0 + 8 * (e >> 1);
                            if (m < a.m && n < a.n) a.y[int64_t(m) * a.ldy + n] = finish_output(acc[mt][e], a.bias, n);
                        }
                    }
                }
            }
        }
        s0 += j_hi - j;
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
}

}  // namespace b2
