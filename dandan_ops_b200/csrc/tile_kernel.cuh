// Latency-oriented kernel for small and mid-size layers in the decode regime (M <= 16).
//
// On layers of a few megabytes the streaming kernel is bound by latency, not bandwidth: a
// warp needs ~0.5 us to decode one native block, and splitting K between CTAs costs a trip
// through global memory.  This kernel puts the whole K range of one row tile (16 outputs)
// into one CTA and brings every one of its native blocks in flight at once:
//   * one bulk copy and one mbarrier per native block, all issued by the first thread before
//     anything else happens (kb * 2336 bytes in flight per CTA, several CTAs per SM);
//   * the unit of work is half a block (eight of its sixteen MMA steps); up to 16 warps take
//     consecutive units, so a block is decoded by two warps in parallel;
//   * x for the CTA's K range is staged once, unpadded: rows of 128 bytes per 64-column chunk
//     with the 16-byte pieces XOR-swizzled by the row, so the fragment reads are conflict-free
//     and two CTAs of a 4096-column layer share an SM at M = 8;
//   * the per-warp FP32 accumulator tiles are added in warp order through shared memory, so
//     the result is bit-reproducible and no workspace, ticket or partial tile is needed;
//   * layers with few row tiles and a long K run a cluster of 2 or 4 CTAs per row tile, each
//     on its share of K; the sums of CTAs 1.. reach CTA 0 through distributed shared memory.
// The dequantization chain and the MMA fragment layout are those of stream_kernel.cuh.
#pragma once
#include <type_traits>
#include "layout.cuh"
#include "stream_kernel.cuh"

namespace b2 {

constexpr int kTileMaxWarps = 16;

struct TileArgs {
    const __half* x;
    const uint8_t* native;
    __half* y;
    unsigned* status;       // may be null
    const __half* bias;     // optional [N] FP16 (may be null)
    int64_t ldx, ldy;
    int m, n, k;
    int n16, kb;
    int warps;              // warps per CTA = min(16, 2*kb)
    int act;                // as StreamArgs::act
    int wait_limit;         // mbarrier polls before a warp gives up (a test passes a small number)
    int fault_block;        // -1; a test passes b >= 0: CTA 0 arms the barrier of its b-th block but skips the copy
    int ksplit;             // 1, 2 or 4: a cluster of that many CTAs shares a row tile, each takes its share
                            // of the K blocks and the others hand their 16 x 8*MT sums to the first through
                            // distributed shared memory (layers whose row tiles leave most SMs idle)
    int overlap;            // launched as a programmatic dependent of the previous kernel: all weight copies are
                            // requested first, then the kernel waits for that one before it reads x
};

// `rows` = rows of x that exist (1..16): only those are staged, so that at M = 1 a CTA of a
// 4096-column layer needs 55 KB instead of 120 KB and four of them share an SM.
// Staged x: per 64-column chunk `rows` rows of 128 bytes, the eight 16-byte pieces of row m stored at
// piece index p ^ (m & 7), chunks 32 bytes apart modulo 128: the 16-byte fragment reads of a quarter
// warp (two rows, four chunks) fall into eight different bank groups without padding the rows.
__host__ __device__ constexpr int tile_x_chunk_bytes(int rows) { return rows * 128 + 32; }
__host__ __device__ constexpr int tile_smem_bytes(int kb, int rows, int warps) {
    // barriers (padded to 128) + blocks + staged x + reduction tiles
    return ((kb * 8 + 127) / 128) * 128 + kb * kBlockBytes + kb * 4 * tile_x_chunk_bytes(rows) +
           warps * (rows <= 8 ? 1 : 2) * 512;
}

// Element e of a row tile's 16 x (8 * MT) sums (fragment order: e = mt * 128 + 4 * lane + c) -> one output.
// GATHER: threads e and e ^ 16 hold neighbouring columns of the same row; they exchange their values so that
// the even one has a 4-byte word, which it stores into the local buffer and sends to every peer's mailbox.
// Every lane of a warp must call this in the same iteration (the callers' loops guarantee it).
template <bool GATHER>
__device__ __forceinline__ void tile_emit(const TileArgs& a, const GatherArgs* ga, int nt, int e, float sum) {
    const int mt = e >> 7, rl = (e >> 2) & 31, c = e & 3;
    const int rg = rl >> 2, rt = rl & 3;
    const int m = mt * 8 + 2 * rt + (c & 1), n = nt * 16 + rg + 8 * (c >> 1);
    const bool inside = m < a.m && n < a.n;
    if constexpr (!GATHER) {
        if (inside) a.y[int64_t(m) * a.ldy + n] = finish_output(sum, a.bias, n);
    } else {
        const unsigned v = inside ? unsigned(__half_as_ushort(finish_output(sum, a.bias, n))) : 0u;
        const unsigned other = __shfl_xor_sync(0xffffffffu, v, 16);          // column n ^ 1 of the same row
        if ((rg & 1) == 0 && inside) {
            const unsigned word = v | (other << 16);
            *reinterpret_cast<unsigned*>(a.y + int64_t(m) * a.ldy + n) = word;
            const unsigned epoch = mailbox_epoch(*ga);
            const int64_t s = int64_t(m) * (ga->cols >> 1) + (n >> 1);
            for (int q = 0; q < ga->world; ++q)
                if (q != ga->rank)
                    mailbox_send(mailbox(ga->flags[q], ga->world, ga->slots, epoch & 1u, ga->rank) + s, word, epoch);
        }
    }
}

// End of a writer CTA in the gather form: count it; the last one of the grid's n16 writers collects the peers'
// packets with all its threads and publishes the epoch.
__device__ __forceinline__ void tile_collect(const TileArgs& a, const GatherArgs* ga) {
    __shared__ int last;
    unsigned* mine = ga->flags[ga->rank];
    const unsigned epoch = mailbox_epoch(*ga);                   // read before this CTA counts itself
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(mine + kGatherTicketWord, 1u) == unsigned(a.n16) - 1u;
    __syncthreads();
    if (!last) return;
    if (mailbox_receive(*ga, epoch, threadIdx.x, blockDim.x)) atomicOr(mine + kGatherStatusWord, kStatusPeerTimeout);
    __syncthreads();
    if (threadIdx.x == 0) {
        mine[kGatherEpochWord] = epoch;
        mine[kGatherTicketWord] = 0u;
    }
}

// FULL: all MT * 8 rows of x are staged (zeros beyond M): compile-time layout, no row predicates -
// the faster form whenever the padded rows do not cost occupancy.  Otherwise only the M rows that
// exist are staged and lanes of missing rows use zero fragments.
//
// GATHER: the multi-GPU form (b2_w4a16_linear_gather).  `a.y` is this rank's column slice of a full [M, N]
// buffer; the CTA that writes a row tile stores it there and sends it to every peer's mailbox as
// {word, epoch} packets (tile_emit).  The grid of this kernel need not be resident at once, so no CTA may wait
// for a peer while others are still to be scheduled: the CTAs count themselves on the flag block's ticket
// when their tile is out, and only the LAST one - by then every packet of this rank has left - collects the
// packets the peers sent (bounded as everywhere) and publishes the epoch.
template <int MT, bool XVEC, bool FULL, bool H16, bool GATHER>
__device__ __forceinline__ void tile_body(const TileArgs& a, const GatherArgs* ga) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int rows = FULL ? MT * 8 : a.m;
    const int kChunk = tile_x_chunk_bytes(rows);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // this CTA's share of the row tile: blocks kb0 .. kb0 + kbn - 1 of K
    uint32_t part = 0;
    if (a.ksplit > 1) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(part));
        // first phase of "both CTAs are running", completed before the hand-over below touches the
        // other CTA's shared memory
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    }
    const int nt = blockIdx.x / a.ksplit;
    const int kb0 = int(part) * a.kb / a.ksplit, kbn = (int(part) + 1) * a.kb / a.ksplit - kb0;
    const int kb_max = (a.kb + a.ksplit - 1) / a.ksplit;     // both CTAs of a pair use one layout
    const int bar_bytes = ((kb_max * 8 + 127) / 128) * 128;
    uint8_t* blocks = smem + bar_bytes;
    uint8_t* xs = blocks + kb_max * kBlockBytes;
    float4* red = reinterpret_cast<float4*>(xs + kb_max * 4 * kChunk);
    const uint32_t bar0 = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int b = 0; b < kbn; ++b) mbar_init(bar0 + b * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const uint8_t* src = a.native + (int64_t(kb0) * a.n16 + nt) * kBlockBytes;
        const int64_t stride = int64_t(a.n16) * kBlockBytes;
        for (int b = 0; b < kbn; ++b) {
            mbar_expect_tx(bar0 + b * 8, kBlockBytes);
            if (!(blockIdx.x == 0 && b == a.fault_block))
                bulk_copy_g2s(smem_u32(blocks + b * kBlockBytes), src + b * stride, kBlockBytes, bar0 + b * 8);
        }
    }
    // Kernels launched behind this one as programmatic dependents may start as soon as they find room.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // The weights are constant; x, the bias and y may belong to the previous kernel until it has completed.
    if (a.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
    // stage x for all columns (zero beyond M and K)
    {
        // Copies that bypass registers (cp.async) are the faster form for the small grids of a K split
        // (2 %), loads through registers for grids that fill the device (6144 x 1024: 4.5 vs 5.2 us).
        auto stage = [&](auto async) {
            constexpr bool kAsync = decltype(async)::value;
            const int pieces_per_row = kbn * 32;
            for (int cc = threadIdx.x; cc < pieces_per_row; cc += blockDim.x) {
                const int k = kb0 * kBlockCols + cc * 8;
                uint8_t* dst = xs + (cc >> 3) * kChunk;
                const __half* src = a.x + k;
                if constexpr (FULL) {
#pragma unroll
                    for (int m = 0; m < MT * 8; ++m)
                        stage_piece<XVEC, kAsync>(dst + m * 128 + (((cc ^ m) & 7) << 4), src + int64_t(m) * a.ldx,
                                                  m < a.m && k < a.k, k, a.k);
                } else {
                    for (int m = 0; m < rows; ++m)
                        stage_piece<XVEC, kAsync>(dst + m * 128 + (((cc ^ m) & 7) << 4), src + int64_t(m) * a.ldx,
                                                  k < a.k, k, a.k);
                }
            }
            if constexpr (XVEC && kAsync) stage_wait();
        };
        if (a.ksplit > 1) stage(std::true_type{}); else stage(std::false_type{});
    }
    __syncthreads();        // x staged; barrier initialisation visible to every waiter

    // units = half blocks, dealt in consecutive runs to the warps
    const int units = kbn * 2;
    const int u0 = (units * warp) / a.warps, u1 = (units * (warp + 1)) / a.warps;
    // The eight MMAs of a unit would be one dependent chain per row tile of x; kChains accumulator tiles used in
    // turn cut it into chains of 8 / kChains (four at one row tile, two at two), added in a fixed order at the end.
    constexpr int kChains = MT == 1 ? 4 : 2;
    float acc[MT][4], accx[kChains - 1][MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            acc[mt][c] = 0.0f;
#pragma unroll
            for (int q = 0; q < kChains - 1; ++q) accx[q][mt][c] = 0.0f;
        }
    bool failed = false;
    for (int u = u0; u < u1 && !failed; ++u) {
        const int b = u >> 1, h = u & 1;
        if (!mbar_wait(bar0 + b * 8, 0, a.wait_limit)) {
            failed = true;
            if (lane == 0 && a.status) atomicOr(a.status, kStatusCopyTimeout);
            break;
        }
        const uint8_t* slot = blocks + b * kBlockBytes;
        const uint4 ca = *reinterpret_cast<const uint4*>(slot + h * 512 + lane * 16);         // row g
        const uint4 cb = *reinterpret_cast<const uint4*>(slot + (2 + h) * 512 + lane * 16);   // row g+8
        const float2 step = *reinterpret_cast<const float2*>(slot + kStepOffset + lane * 8);
        const uint32_t zero = slot[kZeroOffset + lane];
        const GroupConst<H16> gg = make_group<H16>(zero & 15u, step.x), gh = make_group<H16>(zero >> 4, step.y);
        const uint8_t* xchunk = xs + (b * 4 + t) * kChunk + g * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t wa = pick(ca, i), wb = pick(cb, i);
            uint4 xv[MT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)      // rows of x that do not exist are not staged: their columns of the product are zero
                xv[mt] = (FULL || mt * 8 + g < rows) ? *reinterpret_cast<const uint4*>(xchunk + mt * (8 * 128) + (((h * 4 + i) ^ g) << 4))
                                                     : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t ua = wa >> (8 * e), ub = wb >> (8 * e);
                const uint32_t w[4] = {dq_even<H16>(and_or(ua, 0x000F000Fu, 0x64006400u), gg),
                                       dq_even<H16>(and_or(ub, 0x000F000Fu, 0x64006400u), gh),
                                       dq_odd<H16>(and_or(ua, 0x00F000F0u, 0x64006400u), gg),
                                       dq_odd<H16>(and_or(ub, 0x00F000F0u, 0x64006400u), gh)};
                const int chain = (kChains == 4 ? 2 * (i & 1) + e : e);       // compile-time under the unrolling
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    float (&dst)[4] = chain == 0 ? acc[mt] : accx[chain == 0 ? 0 : chain - 1][mt];
                    mma_16816(dst, w, e ? xv[mt].z : xv[mt].x, e ? xv[mt].w : xv[mt].y, dst);
                }
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int q = 0; q < kChains - 1; ++q) acc[mt][c] += accx[q][mt][c];
    // Blocks this CTA requested but no warp waited for cannot exist: every block has two units.
    if (__syncthreads_or(failed) && threadIdx.x == 0) {
        // A warp gave up: copies of this CTA may still be in flight.  Look at every block's barrier
        // once more (bounded) so that nothing lands in shared memory after the CTA has left.
        for (int b = 0; b < kbn; ++b) {
            bool landed = false;
            for (int i = 0; i < 4096 && !landed; ++i) landed = mbar_try_wait(bar0 + b * 8, 0);
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
        red[(warp * MT + mt) * 32 + lane] = make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
    __syncthreads();
    if (a.ksplit > 1) {
        // The CTAs of a cluster share the row tile.  Each adds its warps' tiles in warp order; CTA p > 0
        // puts its 128 * MT sums into slot p - 1 of the first one's shared memory, and after the cluster
        // barrier the first adds the slots to its own sums in CTA order and writes y.
        float* tot = reinterpret_cast<float*>(red) + a.warps * MT * 128;       // [MT * 128] own sums
        float* peer = tot + MT * 128;                                          // [ksplit - 1][MT * 128] the others' sums
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        for (int e = threadIdx.x; e < MT * 128; e += blockDim.x) {
            const int mt = e >> 7, rl = (e >> 2) & 31, c = e & 3;
            float sum = 0.0f;
            for (int w = 0; w < a.warps; ++w)
                sum += reinterpret_cast<const float*>(red)[((w * MT + mt) * 32 + rl) * 4 + c];
            if (part == 0) {
                tot[e] = sum;
            } else {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(smem_u32(peer + (part - 1) * (MT * 128) + e)));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(sum) : "memory");
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (part != 0) return;
        if (a.act) {
            for (int e = threadIdx.x; e < MT * 64; e += blockDim.x) {
                const int mt = e >> 6, rl = (e >> 1) & 31, c = e & 1;
                const int at = (mt * 32 + rl) * 4 + c;
                float gate = tot[at], up = tot[at + 2];
                for (int p = 0; p + 1 < a.ksplit; ++p) {
                    gate += peer[p * (MT * 128) + at];
                    up += peer[p * (MT * 128) + at + 2];
                }
                const int rg = rl >> 2, rt = rl & 3;
                const int m = mt * 8 + 2 * rt + c, n = nt * 16 + rg;
                if (m < a.m && n + 8 < a.n)
                    a.y[int64_t(m) * a.ldy + nt * 8 + rg] = silu_mul(finish_output(gate, a.bias, n), finish_output(up, a.bias, n + 8));
            }
            return;
        }
        for (int e = threadIdx.x; e < MT * 128; e += blockDim.x) {
            float sum = tot[e];
            for (int p = 0; p + 1 < a.ksplit; ++p) sum += peer[p * (MT * 128) + e];
            tile_emit<GATHER>(a, ga, nt, e, sum);
        }
        if constexpr (GATHER) tile_collect(a, ga);
        return;
    }
    // thread e adds element e of every warp's tile in warp order and stores one output
    if (a.act) {
        // gate (row rg) and up (row rg + 8) of one output: elements c and c + 2 of the same fragment
        for (int e = threadIdx.x; e < MT * 64; e += blockDim.x) {
            const int mt = e >> 6, rl = (e >> 1) & 31, c = e & 1;
            float gate = 0.0f, up = 0.0f;
            for (int w = 0; w < a.warps; ++w) {
                const float* f = reinterpret_cast<const float*>(red) + ((w * MT + mt) * 32 + rl) * 4;
                gate += f[c];
                up += f[c + 2];
            }
            const int rg = rl >> 2, rt = rl & 3;
            const int m = mt * 8 + 2 * rt + c, n = nt * 16 + rg;
            if (m < a.m && n + 8 < a.n)
                a.y[int64_t(m) * a.ldy + nt * 8 + rg] = silu_mul(finish_output(gate, a.bias, n), finish_output(up, a.bias, n + 8));
        }
        return;
    }
    for (int e = threadIdx.x; e < MT * 128; e += blockDim.x) {
        const int mt = e >> 7, rl = (e >> 2) & 31, c = e & 3;
        float sum = 0.0f;
        for (int w = 0; w < a.warps; ++w)
            sum += reinterpret_cast<const float*>(red)[((w * MT + mt) * 32 + rl) * 4 + c];
        tile_emit<GATHER>(a, ga, nt, e, sum);
    }
    if constexpr (GATHER) tile_collect(a, ga);
}

template <int MT, bool XVEC, bool FULL, bool H16 = false>
__global__ void __launch_bounds__(kTileMaxWarps * 32)
w4a16_tile_kernel(const TileArgs a) {
    tile_body<MT, XVEC, FULL, H16, false>(a, nullptr);
}

template <int MT, bool FULL, bool H16>
__global__ void __launch_bounds__(kTileMaxWarps * 32)
w4a16_tile_gather_kernel(const TileArgs a, const GatherArgs ga) {
    tile_body<MT, true, FULL, H16, true>(a, &ga);
}

}  // namespace b2
