// Weight-streaming kernel for large layers at M <= 16: the 32-warp form of stream_kernel.cuh.
//
// Same work split (stream-K over persistent CTAs, one per SM), same native blocks, same exact
// dequantization chain and the same ticket / partial-tile protocol as w4a16_stream_kernel; what
// changes is everything around the arithmetic, because that kernel is bound by instruction
// issue with only four warps per scheduler:
//   * 32 warps per CTA (eight per scheduler) under a 64-register cap: a warp decodes half a
//     native block at a time, so the codes of a block never sit in registers all at once;
//   * a ring of two blocks per warp (150 KB per SM in flight, as before) - with eight warps per
//     scheduler a warp takes twice as long per block, so two slots cover the same latency;
//   * the first weight copies are requested before anything else happens in the CTA;
//   * x is staged in phases of 2048 / MT columns into two buffers, the next phase fetched with
//     cp.async while the current one is used.  No block-wide barrier: each buffer has a "full"
//     mbarrier (every thread's copies have landed) and an "empty" one (every warp is done with it),
//     and a warp stages its share of the next phase half-way through the current one - by then the
//     slowest warp has normally left the previous phase, so nobody waits for anybody;
//   * a range that ends inside a row group starts with that trailing fragment: its partial tile
//     and ticket are out of the way early, and the last thing a CTA does is a plain store of a
//     whole row group instead of the fence / ticket / re-read of a split one;
//   * per-group constants come from integer arithmetic on the zero-point byte (no int->float
//     conversions at the head of a block).
#pragma once
#include "stream_kernel.cuh"

namespace b2 {

// W warps per CTA with a ring of 64 / W blocks each: 150 KB of weight copies per SM either way.
__host__ __device__ constexpr int s2_stages(int w) { return 64 / w; }
__host__ __device__ constexpr int s2_phase_blocks(int mt) { return 8 / mt; }
__host__ __device__ constexpr int s2_xbuf_bytes(int mt) { return s2_phase_blocks(mt) * 4 * stream_x_chunk_bytes(mt * 8); }
constexpr int kS2BarBytes = 64 * 8 + 64;      // 64 ring barriers + full[2], empty[2] of the x buffers (padded)
__host__ __device__ constexpr int s2_smem_bytes(int mt) {
    return kS2BarBytes + 64 * kBlockBytes + 2 * s2_xbuf_bytes(mt);
}
// Arrives on `bar` once all cp.async copies this thread has issued so far have landed.
__device__ __forceinline__ void mbar_arrive_after_copies(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

template <int MT, bool XVEC, int W>
__global__ void __launch_bounds__(W * 32, 1)
w4a16_stream2_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int S = s2_stages(W), MP = MT * 8;
    constexpr int PB = s2_phase_blocks(MT);
    constexpr int kChunk = stream_x_chunk_bytes(MP);
    constexpr int kXBuf = s2_xbuf_bytes(MT);
    constexpr int kBarBytes = kS2BarBytes, kRingBytes = W * S * kBlockBytes;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ctas = gridDim.x;
    const int b0 = int((unsigned(a.steps) * blockIdx.x) / unsigned(ctas));
    const int b1 = int((unsigned(a.steps) * (blockIdx.x + 1)) / unsigned(ctas));
    const int len = b1 - b0;
    // Steps of the trailing fragment (the range ends inside a row group that the next CTA continues):
    // they are processed first.  A range that lies inside one row group has nothing to rotate.
    int rot = b1 - (b1 / a.kb) * a.kb;
    if (rot >= len) rot = 0;
    const int nat_end = b1 - rot;

    // This warp's tile exists in every row group except possibly the last one.
    const int last_start = (a.groups - 1) * a.kb;
    const bool in_last = (a.groups - 1) * W + warp < a.n16;
    const int rot_w = (in_last || b1 <= last_start) ? rot : 0;
    const int nat_end_w = in_last ? nat_end : min(nat_end, last_start);

    const uint32_t bar0 = smem_u32(smem) + warp * S * 8;
    uint8_t* ring = smem + kBarBytes + warp * S * kBlockBytes;
    const uint32_t ring0 = smem_u32(ring);
    uint8_t* xs = smem + kBarBytes + kRingBytes;

    // ---- copy-request cursor (all lanes keep it, lane 0 issues) ---------------------------------
    // State: column block `fkb` inside the row group whose first block (for this warp) is at `fbase`;
    // `fswitch` requests from now the cursor jumps from the trailing fragment to the start of the range.
    const long long stride = (long long)a.n16 * kBlockBytes;
    int fetch_left = rot_w + max(0, nat_end_w - b0);
    int fswitch = rot_w;                              // 0: already in the natural part
    int fkb;
    const uint8_t* fbase;
    {
        const int fs = fswitch ? b1 - rot : b0;
        const int fgrp = fs / a.kb;
        fkb = fs - fgrp * a.kb;
        fbase = a.native + (long long)(fgrp * W + warp) * kBlockBytes;
    }
    int fault = (a.fault_step >= 0 && blockIdx.x == 0 && warp == 0) ? a.fault_step : -1;   // test hook, see StreamArgs
    auto request = [&](int slot) {
        if (lane == 0) {
            mbar_expect_tx(bar0 + slot * 8, kBlockBytes);
            if (fault != 0) bulk_copy_g2s(ring0 + slot * kBlockBytes, fbase + fkb * stride, kBlockBytes, bar0 + slot * 8);
        }
        --fault;
        --fetch_left;
        if (++fkb == a.kb) {
            fkb = 0;
            fbase += W * kBlockBytes;
        }
        if (--fswitch == 0) {
            const int fgrp = b0 / a.kb;
            fkb = b0 - fgrp * a.kb;
            fbase = a.native + (long long)(fgrp * W + warp) * kBlockBytes;
        }
    };
    // x buffers: full[b] completes when every thread's copies into buffer b have landed (two arrivals per
    // thread: one for its plain stores, one that fires after its cp.async copies), empty[b] when every
    // warp has finished the phase that used it.
    const uint32_t xfull = smem_u32(smem) + 64 * 8, xempty = xfull + 16;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(xfull + b * 8, 2 * W * 32);
            mbar_init(xempty + b * 8, W);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bar0 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
#pragma unroll
    for (int s = 0; s < S; ++s)
        if (fetch_left > 0) request(s);
    __syncthreads();                                  // the x barriers exist before anybody arrives on them

    // ---- x: resident when all of K fits in the two buffers, else double-buffered phases -----------
    const bool resident = a.kb <= 2 * PB;
    int part = rot ? 0 : 1;                           // 0: trailing fragment, 1: the rest of the range in order
    int ps = rot ? b1 - rot : b0;                     // first step of the current phase
    int pend = rot ? b1 : nat_end;                    // end of the current part
    int grp = ps / a.kb;
    int kbi = ps - grp * a.kb;
    if (resident) stage_x<MT, XVEC, W, false>(xs, a, 0, a.kb * kBlockCols);
    else stage_x<MT, XVEC, W, false>(xs, a, kbi * kBlockCols, min(PB, min(a.kb - kbi, pend - ps)) * kBlockCols);
    mbar_arrive(xfull);
    mbar_arrive_after_copies(xfull);

    float acc[MT][4];
    int stage = 0;
    uint32_t parity = 0;
    bool failed = false;
    int k_lo = kbi;                                   // first column block of the current segment
    bool seg_start = true;
    int phase = 0;                                    // phase j uses buffer j & 1 for the (j >> 1)-th time

    // Moves (ps, pend, part, grp, kbi) from a phase of `cnt` blocks to the next one; ps = -1 at the end.
    auto advance = [&](int& ps_, int& pend_, int& part_, int& grp_, int& kbi_, int cnt) {
        ps_ += cnt;
        kbi_ += cnt;
        if (kbi_ == a.kb) { kbi_ = 0; ++grp_; }
        if (ps_ == pend_) {
            if (part_ == 0) { part_ = 1; ps_ = b0; pend_ = nat_end; grp_ = b0 / a.kb; kbi_ = b0 - grp_ * a.kb; }
            else ps_ = -1;
        }
    };

    while (ps >= 0) {
        const int cnt = min(PB, min(a.kb - kbi, pend - ps));
        const int buf = phase & 1;
        if (!resident || phase == 0) {
            if (!mbar_wait(xfull + buf * 8, (phase >> 1) & 1, a.wait_limit) && !failed) {
                failed = true;
                if (lane == 0) atomicOr(a.status, kStatusCopyTimeout);
            }
        }
        // Half-way through the phase every warp stages its share of the next one into the other buffer,
        // once all warps have left the phase that used that buffer before.
        auto prefetch_next = [&]() {
            int ns = ps, npend = pend, npart = part, ngrp = grp, nkbi = kbi;
            advance(ns, npend, npart, ngrp, nkbi, cnt);
            if (ns < 0) return;
            if (phase >= 1 && !mbar_wait(xempty + (buf ^ 1) * 8, ((phase - 1) >> 1) & 1, a.wait_limit) && !failed) {
                failed = true;
                if (lane == 0) atomicOr(a.status, kStatusCopyTimeout);
            }
            stage_x<MT, XVEC, W, false>(xs + (buf ^ 1) * kXBuf, a, nkbi * kBlockCols,
                                        min(PB, min(a.kb - nkbi, npend - ns)) * kBlockCols);
            mbar_arrive(xfull + (buf ^ 1) * 8);
            mbar_arrive_after_copies(xfull + (buf ^ 1) * 8);
        };
        const int half = cnt >> 1;
        if (seg_start) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[mt][c] = 0.0f;
            k_lo = kbi;
            seg_start = false;
        }
        const int nt = grp * W + warp;
        const bool active = nt < a.n16;
        {
            const uint8_t* xbase = resident ? xs + (kbi * 4 + t) * kChunk + g * 144 : xs + buf * kXBuf + t * kChunk + g * 144;
            for (int kbl = 0; kbl < cnt; ++kbl) {
                if (kbl == half && !resident) prefetch_next();
                if (!active || failed) continue;
                if (!mbar_wait(bar0 + stage * 8, parity, a.wait_limit)) {
                    failed = true;
                    if (lane == 0) atomicOr(a.status, kStatusCopyTimeout);
                    continue;
                }
                const uint8_t* slot = ring + stage * kBlockBytes;
                const float2 step = *reinterpret_cast<const float2*>(slot + kStepOffset + lane * 8);
                const uint32_t zero = slot[kZeroOffset + lane];
                // -(1024 + z) and -(64 + z) as FP32 bit patterns: z sits in the mantissa
                const uint32_t zlo = zero & 15u, zhi = zero >> 4;
                const float cg = __uint_as_float(0xC4800000u + zlo * 8192u), ch = __uint_as_float(0xC4800000u + zhi * 8192u);
                const float eg = __uint_as_float(0xC2800000u + zlo * 131072u), eh = __uint_as_float(0xC2800000u + zhi * 131072u);
                const uint64_t sg = twice(step.x), sh = twice(step.y);
                const uint8_t* xrow = xbase + kbl * 4 * kChunk;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint4 ca = *reinterpret_cast<const uint4*>(slot + h * 512 + lane * 16);         // row g
                    const uint4 cb = *reinterpret_cast<const uint4*>(slot + (2 + h) * 512 + lane * 16);   // row g+8
                    if (h == 1) {
                        __syncwarp();                  // every lane has read the whole slot
                        if (fetch_left > 0) {
                            if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            request(stage);
                        }
                        if (++stage == S) { stage = 0; parity ^= 1u; }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t wa = pick(ca, i), wb = pick(cb, i);
                        uint4 xv[MT];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            xv[mt] = *reinterpret_cast<const uint4*>(xrow + mt * (8 * 144) + (h * 4 + i) * 16);
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const uint32_t ua = wa >> (8 * e), ub = wb >> (8 * e);
                            const uint32_t w[4] = {dequant_pair_even(and_or(ua, 0x000F000Fu, 0x64006400u), cg, sg),
                                                   dequant_pair_even(and_or(ub, 0x000F000Fu, 0x64006400u), ch, sh),
                                                   dequant_pair_odd(and_or(ua, 0x00F000F0u, 0x64006400u), eg, sg),
                                                   dequant_pair_odd(and_or(ub, 0x00F000F0u, 0x64006400u), eh, sh)};
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt)
                                mma_16816(acc[mt], w, e ? xv[mt].z : xv[mt].x, e ? xv[mt].w : xv[mt].y, acc[mt]);
                        }
                    }
                }
            }
        }

        if (!resident) {
            __syncwarp();                             // every lane is done with this phase's x
            if (lane == 0) mbar_arrive(xempty + buf * 8);
        }
        const bool seg_end = (kbi + cnt == a.kb) || (ps + cnt == pend);
        if (seg_end) {
            const int k_hi = kbi + cnt;
            if (active && !failed) {
                const bool whole = (k_lo == 0 && k_hi == a.kb);
                bool write_out = whole;
                if (!whole) {
                    // Contributors to this row group are the CTAs first..last; mine is slot `blockIdx.x - first`.
                    const int gs = grp * a.kb;
                    const int first = owner_of(gs, a.steps, ctas), last = owner_of(gs + a.kb - 1, a.steps, ctas);
                    const int parts = last - first + 1;
                    const int tile = (a.groups <= ctas ? grp : first) * W + warp;
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
                if (write_out) {
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
            seg_start = true;
        }
        advance(ps, pend, part, grp, kbi, cnt);
        ++phase;
    }

    if (failed && lane == 0) {
        // Let copies that are still in flight land before the CTA's shared memory is released
        // (a bounded look at every slot of this warp's ring).
        for (int s = 0; s < S; ++s) {
            bool landed = false;
            for (int i = 0; i < 4096 && !landed; ++i) landed = mbar_try_wait(bar0 + stage * 8, parity);
            if (++stage == S) { stage = 0; parity ^= 1u; }
        }
    }
}

}  // namespace b2
