// Prefill kernel for large batches: two CTAs on neighbouring SMs (a cluster of two) compute a
// tile of 256 output columns (weight rows) by 256 rows of x with one
// tcgen05.mma.cta_group::2 instruction stream, the dequantized weights going through tensor
// memory instead of shared memory.
//
//   D[n][m] (FP32, tensor memory: 128 lanes = this CTA's weight rows, 256 columns = x rows)
//     += A[n][k] (weights, FP16, written to tensor memory by the converter warps: tcgen05.st)
//      * B[m][k] (x tile, FP16, shared memory, TMA with the 128-byte swizzle; each CTA loads
//                 128 of the 256 rows and the tensor cores of both SMs read both halves)
//
// Why this shape: per 64-column step a CTA's shared memory only takes the 16 KB x tile once
// from TMA and once into the tensor core, plus the 4.6 KB of raw 4-bit blocks - the FP16 weight
// tile (16 KB written, 16 KB read per step in the single-CTA kernel, which made shared-memory
// bandwidth the limit there) never touches it.  Every weight is converted once per 256 rows
// of x, every x byte is fetched from L2 once per 256 output columns, and eight x stages
// (128 KB) cover the TMA latency under load.
//
// Roles per CTA (10 warps):
//   warp 0      copy producer: bulk copies of this CTA's 8 native blocks per 256 columns of K,
//               TMA loads of this CTA's x rows; the loads of BOTH CTAs complete the leader's
//               full barrier (cp.async.bulk.tensor with .cta_group::2)
//   warp 1      allocates/frees tensor memory (cta_group::2, both CTAs); in the leader CTA
//               (cluster rank 0) one lane issues the MMAs and one commit per step to both CTAs
//   warps 2..9  converters: thread = weight row (tensor-memory lane); the two warps of a lane
//               quadrant take alternate 64-column steps (one 32-column tcgen05.st per step and
//               quadrant); afterwards the epilogue: tcgen05.ld gives a thread 32 rows of y for
//               ONE column, the warp transposes through the idle x ring and stores its
//               32 columns x MT/2 rows with one TMA store (2-byte global stores for unaligned y;
//               lanes l and l ^ 8 exchange sums first when the gate/up epilogue is on)
//
// Barriers (every wait is bounded, as in the single-CTA kernel):
//   raw_full/raw_free[r]   local: bulk copy done / all converter warps finished with raw stage r
//   full[s % XS]           leader only: transaction bytes of both CTAs' x loads + one arrival per
//                          converter warp of both CTAs that wrote step s
//   done[s % XS]           both CTAs: tcgen05.commit (multicast) after the MMAs of step s; frees the
//                          x stage for the producers and the tensor-memory stage for the converters
//   acc_full               both CTAs: tcgen05.commit after the last MMA
//   epi_written, epi_last  local, K-splitting only: the CTA's partial tile is in global memory /
//                          thread 64 has drawn the tile's ticket
//
// K-splitting (layers with fewer tiles than SM pairs and a long K): blockIdx.z takes a share of
// the 256-column blocks, every CTA stores its FP32 accumulator to the workspace, and the CTA that
// draws the last ticket of its half tile adds the partial tiles in split order - the same
// deterministic scheme as the streaming kernel's - and writes y.
#pragma once
#include "gemm_kernel.cuh"

namespace b2 {

constexpr int kPairRows = 128;                                   // weight rows per CTA (256 per pair)
constexpr int kPairConverters = 8;                               // converter warps per CTA
constexpr int kPairThreads = 64 + 32 * kPairConverters;
constexpr int kPairRawBytes = (kPairRows / 16) * kBlockBytes;    // 18688: 8 native blocks
constexpr uint32_t kPairWCols = kGemmBK / 2;                     // 32 columns hold 64 FP16 of a weight row
// Two shapes.  MT = rows of x per pair (the MMA's N; each CTA loads MT/2 of them):
//   MT = 256: one CTA per SM, 8 x stages, 4 weight stages, 512 tensor-memory columns
//   MT = 192: two CTAs per SM (each half the shared memory and 256 columns), so that one pair's
//             prologue and epilogue overlap the other pair's main loop
template <int MT> struct PairShape;
template <> struct PairShape<256> { static constexpr int XS = 8, WS = 4, RS = 3, CTAS = 1; };
template <> struct PairShape<192> { static constexpr int XS = 5, WS = 2, RS = 2, CTAS = 2; };
__host__ __device__ constexpr int pair_x_bytes(int mt) { return (mt / 2) * kGemmBK * 2; }
template <int MT> __host__ __device__ constexpr int pair_smem_bytes() {
    return 1024 + PairShape<MT>::XS * pair_x_bytes(MT) + PairShape<MT>::RS * kPairRawBytes + 512;
}
template <int MT> __host__ __device__ constexpr uint32_t pair_tmem_cols() { return MT + PairShape<MT>::WS * kPairWCols <= 256 ? 256 : 512; }

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in the CTA with the given cluster rank.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier that may live in the peer CTA.  CTA-scope release: the data the arrival
// publishes is in tensor memory (ordered by tcgen05.wait::st and the tcgen05 fences), and a
// cluster-scope release costs a device-wide memory barrier per arrival.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// x tile load whose completion bytes go to a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor], issued for both SMs of the pair.
__device__ __forceinline__ void umma_f16_pair_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in both CTAs once all earlier MMAs have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
                 "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
                 ::"r"(bar) : "memory");
}
// 32 registers -> 32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                   "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                   "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Tile store shared -> global; rows and columns outside the tensor are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// TMA_Y: y is 16-byte aligned with a row stride that is a multiple of 16 bytes; the epilogue
// then transposes through shared memory (the idle x ring) and stores each warp's 32 columns x
// MT/2 rows with one TMA store.  Otherwise every thread stores its 2-byte results itself.
template <int MT, bool TMA_Y, bool H16 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, PairShape<MT>::CTAS)
w4a16_gemm_pair_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap ymap, const GemmArgs a) {
    constexpr int XS = PairShape<MT>::XS, WS = PairShape<MT>::WS, RS = PairShape<MT>::RS;
    constexpr int kXBytes = pair_x_bytes(MT);
    constexpr uint32_t kTmemCols = pair_tmem_cols<MT>();
    static_assert(WS <= XS && MT % 64 == 0, "one barrier ring serves both operand rings");
    static_assert(kPairConverters * (MT / 2) * 64 <= XS * kXBytes, "the epilogue stages y in the x ring");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* x_base = smem;                                                // [XS][kXBytes]
    uint8_t* raw_base = x_base + XS * kXBytes;                             // [RS][18688]
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw_base + RS * kPairRawBytes);
    // FULL[s % XS] (leader): the x bytes of both CTAs and every converter warp's weights of step s
    // are in place.  DONE[s % XS] (both CTAs): the MMAs of step s have completed.
    constexpr int RAW_FULL = 0, RAW_FREE = RAW_FULL + RS, FULL = RAW_FREE + RS, DONE = FULL + XS,
                  ACC_FULL = DONE + XS, EPI_WRITTEN = ACC_FULL + 1, EPI_LAST = EPI_WRITTEN + 1, NBARS = EPI_LAST + 1;
    static_assert(NBARS * 8 + 12 <= 512, "barrier area");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + i * 8; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int tile_n = blockIdx.x >> 1, tile_m = blockIdx.y;
    const int m0 = tile_m * MT;                                            // first x row of the pair
    const int n0 = tile_n * (2 * kPairRows) + int(rank) * kPairRows;       // first weight row of this CTA
    // this CTA's share of K: 256-column blocks [kb0, kb1), 64-column steps s0 .. s0 + ksteps - 1
    const int split = blockIdx.z;
    const int kb0 = int(int64_t(split) * a.kb / a.splits), kb1 = int(int64_t(split + 1) * a.kb / a.splits);
    const int s0 = kb0 * 4;
    const int ksteps = min((a.k + kGemmBK - 1) / kGemmBK, kb1 * 4) - s0;

    if (threadIdx.x == 0) {
        mbar_init(bar(EPI_WRITTEN), kPairConverters);
        mbar_init(bar(EPI_LAST), 1);
        for (int i = 0; i < RS; ++i) { mbar_init(bar(RAW_FULL + i), 1); mbar_init(bar(RAW_FREE + i), kPairConverters); }
        for (int i = 0; i < XS; ++i) { mbar_init(bar(FULL + i), 1 + kPairConverters); mbar_init(bar(DONE + i), 1); }   // x bytes + 4 converter warps of each CTA
        mbar_init(bar(ACC_FULL), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tcgen05_fence_before();
    cluster_sync_all();                     // barriers of both CTAs exist before any remote arrival
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_w = tmem_base + MT;                                // weight ring behind the accumulator

    auto give_up = [&]() {
        *abort_flag = 1;
        atomicOr(a.status, kStatusGemmTimeout);
    };
    auto wait = [&](int idx, uint32_t parity) -> bool {
        for (int i = 0; i < kWaitLimit; ++i) {
            if (mbar_try_wait(bar(idx), parity)) return true;
            if ((i & 63) == 63 && *abort_flag) return false;
        }
        give_up();
        return false;
    };

    if (warp == 0) {
        // ------------------------------ copy producer ------------------------------------
        if (lane == 0) {
            const int nt0 = n0 >> 4;
            const int blocks_here = max(0, min(kPairRows / 16, a.n16 - nt0));
            const uint32_t raw_bytes = uint32_t(blocks_here) * kBlockBytes;
            const uint8_t* src = a.native + int64_t(nt0) * kBlockBytes;
            const int64_t stride = int64_t(a.n16) * kBlockBytes;
            const uint32_t full_leader = map_to_cta(bar(FULL), 0);
            for (int s = 0; s < ksteps; ++s) {
                if ((s & 3) == 0) {
                    const int kb = s >> 2, r = kb % RS;
                    if (kb >= RS && !wait(RAW_FREE + r, ((kb / RS) - 1) & 1)) break;
                    if (raw_bytes) {
                        mbar_expect_tx(bar(RAW_FULL + r), raw_bytes);
                        bulk_copy_g2s(smem_u32(raw_base + r * kPairRawBytes), src + (kb0 + kb) * stride, raw_bytes, bar(RAW_FULL + r));
                    } else {
                        mbar_arrive(bar(RAW_FULL + r));       // no weight rows here: columns beyond N, masked in the epilogue
                    }
                }
                const int st = s % XS;
                if (s >= XS && !wait(DONE + st, ((s / XS) - 1) & 1)) break;
                if (leader) mbar_expect_tx(bar(FULL + st), 2 * kXBytes);
                tma_load_2d_pair(smem_u32(x_base + st * kXBytes), &xmap, (s0 + s) * kGemmBK, m0 + int(rank) * (MT / 2), full_leader + st * 8);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (one lane of the leader CTA) -----------
        if (leader && lane == 0) {
            // D = F32, A = B = F16, both K-major, M = 256 weight rows, N = MT rows of x
            const uint32_t idesc = (1u << 4) | (uint32_t(MT >> 3) << 17) | (uint32_t(256 >> 4) << 24);
            const uint64_t desc0 = umma_desc_sw128(smem_u32(x_base));
            bool have = false;                  // the coming step's barrier was already seen complete
            int xs = 0, ws = 0;
            uint32_t par = 0;
            for (int s = 0; s < ksteps; ++s) {
                if (!have && !wait(FULL + xs, par)) break;
                tcgen05_fence_after();
                const uint64_t desc = desc0 + uint64_t((xs * kXBytes) >> 4);
                const uint32_t w_addr = tmem_w + ws * kPairWCols;
                const int xn = xs + 1 == XS ? 0 : xs + 1;
                const uint32_t parn = xs + 1 == XS ? par ^ 1 : par;
#pragma unroll
                for (int kk = 0; kk < kGemmBK / 16; ++kk) {
                    // look at the next step's barrier while the tensor cores still have work queued
                    if (kk == kGemmBK / 16 - 1) have = s + 1 < ksteps && mbar_try_wait(bar(FULL + xn), parn);
                    umma_f16_pair_ts(tmem_base, w_addr + kk * 8, desc + uint64_t(kk * 2), idesc, (s > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit_pair(bar(DONE + xs));
                if (s == ksteps - 1) umma_commit_pair(bar(ACC_FULL));
                xs = xn; par = parn;
                ws = ws + 1 == WS ? 0 : ws + 1;
            }
        }
    } else {
        // ------------------------------ converters ---------------------------------------
        const int quad = warp & 3;                      // tensor-memory lane quadrant this warp may access
        const int half = (warp - 2) >> 2;               // converts the steps with s % 2 == half; epilogue: column half
        const int r = quad * 32 + lane;                 // weight row of this CTA = tensor-memory lane
        const int blk = r >> 4, rr = r & 15, g = rr & 7, hi8 = rr >> 3;
        const uint32_t full_leader = map_to_cta(bar(FULL), 0);
        const uint32_t lane_addr = uint32_t(quad * 32) << 16;
        bool ok = true;
        int waited_kb = -1;
        // The two warps of a lane quadrant alternate steps: one 32-column tensor-memory store per
        // step and quadrant, and two steps of time for a thread's 64 weights.
        for (int s = half; s < ksteps && ok; s += 2) {
            const int kb = s >> 2, t = s & 3, rs = kb % RS;
            if (kb != waited_kb) { ok = wait(RAW_FULL + rs, (kb / RS) & 1); waited_kb = kb; }
            if (!ok) break;
            const uint8_t* nb = raw_base + rs * kPairRawBytes + blk * kBlockBytes;
            const int lane_idx = 4 * g + t;
            const uint4 code0 = *reinterpret_cast<const uint4*>(nb + (2 * hi8) * 512 + lane_idx * 16);
            const uint4 code1 = *reinterpret_cast<const uint4*>(nb + (2 * hi8 + 1) * 512 + lane_idx * 16);
            const float step = *reinterpret_cast<const float*>(nb + kStepOffset + (lane_idx * 2 + hi8) * 4);
            const GroupConst<H16> gc = make_group<H16>((nb[kZeroOffset + lane_idx] >> (4 * hi8)) & 15u, step);
            const uint32_t words[8] = {code0.x, code0.y, code0.z, code0.w, code1.x, code1.y, code1.z, code1.w};
            uint32_t o[32];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 q = dequant_word<H16>(words[i], gc);
                o[4 * i] = q.x; o[4 * i + 1] = q.y; o[4 * i + 2] = q.z; o[4 * i + 3] = q.w;
            }
            // the conversion happens in registers before the wait for the free tensor-memory stage
            if (s >= WS) ok = wait(DONE + (s - WS) % XS, ((s - WS) / XS) & 1);
            if (!ok) break;
            tcgen05_fence_after();
            tmem_st32(tmem_w + lane_addr + (s % WS) * kPairWCols, o);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(full_leader + (s % XS) * 8);
                // last step of this warp in the raw stage (its later steps belong to the next block)
                if (((s + 2) >> 2) != kb || s + 2 >= ksteps) mbar_arrive(bar(RAW_FREE + rs));
            }
        }
        // ------------------------------ epilogue -----------------------------------------
        if (ok && wait(ACC_FULL, 0)) {
            tcgen05_fence_after();
            const int n = n0 + r;
            const bool n_ok = n < a.n;
            const __half bias = (a.bias && n_ok) ? a.bias[n] : __float2half(0.0f);
            const bool split_k = a.splits > 1;
            // Partial tiles of this half tile: [split][32-column chunk][4 columns][128 weight rows] FP32 x 4,
            // so that the 32 lanes of a warp store and load 512 contiguous bytes per instruction.
            constexpr int kTileVec = kPairRows * MT / 4;             // 16-byte vectors per half tile and split
            const int64_t half_tile = (int64_t(tile_m) * (gridDim.x >> 1) + tile_n) * 2 + rank;
            uint4* part0 = reinterpret_cast<uint4*>(a.partial) + half_tile * a.splits * int64_t(kTileVec)
                           + (half * (MT / 64)) * (8 * kPairRows) + r;
            bool write_y = true;
            if (split_k) {
                uint4* mine = part0 + int64_t(split) * kTileVec;
#pragma unroll 1
                for (int cc = 0; cc < MT / 64; ++cc) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + lane_addr + half * (MT / 2) + cc * 32, v);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        mine[(cc * 8 + q) * kPairRows] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(EPI_WRITTEN));
                if (threadIdx.x == 64) {
                    if (wait(EPI_WRITTEN, 0)) {
                        __threadfence();
                        const unsigned t = atomicAdd(a.tickets + half_tile, 1u);
                        const bool last = t == unsigned(a.splits - 1);
                        if (last) a.tickets[half_tile] = 0;          // every split has arrived: ready for the next call
                        __threadfence();
                        *last_flag = last ? 1u : 0u;
                    } else {
                        *last_flag = 0u;
                    }
                    mbar_arrive(bar(EPI_LAST));
                }
                write_y = wait(EPI_LAST, 0) && *last_flag != 0;
            }
            // accumulator chunk cc of this thread: from tensor memory, or the partial tiles added in split order
            auto load_chunk = [&](int cc, uint32_t (&v)[32]) {
                if (!split_k) {
                    tmem_ld32(tmem_base + lane_addr + half * (MT / 2) + cc * 32, v);
                    return;
                }
                const uint4* src = part0 + cc * (8 * kPairRows);
#pragma unroll
                for (int q = 0; q < 8; ++q) {                          // split 0
                    const uint4 f = __ldcg(src + q * kPairRows);
                    v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
                }
                for (int sp = 1; sp < a.splits; ++sp) {                 // then 1, 2, ... in this order
                    src += kTileVec;
                    uint4 f[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) f[q] = __ldcg(src + q * kPairRows);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + __uint_as_float(f[q].x));
                        v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + __uint_as_float(f[q].y));
                        v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + __uint_as_float(f[q].z));
                        v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + __uint_as_float(f[q].w));
                    }
                }
            };
            if (!write_y) {
                // another CTA adds the partial tiles
            } else if (a.act) {
                // Gate/up epilogue.  Lanes l and l ^ 8 hold the gate and the up sum of output column
                // 8 * (row / 16) + (l & 7); the gate lane finishes x rows 0..15 of a chunk, the up lane
                // rows 16..31, each after one exchange per row with its partner.
                const bool is_up = (lane & 8) != 0;
                const __half bias_other = __shfl_xor_sync(0xffffffffu, bias, 8);
                const __half bias_g = is_up ? bias_other : bias, bias_u = is_up ? bias : bias_other;
                const int out_col = (n >> 4) * 8 + (lane & 7);          // column of y (n/2 columns in all)
                const bool out_ok = (n | 8) < a.n;                      // the tile's up row exists (n % 16 == 0 guarantees it)
                // staged tile of this warp: [MT/2 rows of y][16 columns] FP16, 32-byte rows
                uint8_t* stage = x_base + (warp - 2) * ((MT / 2) * 32);
                const int local_col = (lane >> 4) * 8 + (lane & 7);
#pragma unroll 1
                for (int cc = 0; cc < MT / 64; ++cc) {
                    const int col = half * (MT / 2) + cc * 32;
                    uint32_t v[32];
                    load_chunk(cc, v);
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const uint32_t mine = is_up ? v[e] : v[e + 16];
                        const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, 8);
                        const float gate = __uint_as_float(is_up ? theirs : v[e]);
                        const float up = __uint_as_float(is_up ? v[e + 16] : theirs);
                        __half g16 = __float2half_rn(gate), u16 = __float2half_rn(up);
                        if (a.bias) { g16 = __hadd(g16, bias_g); u16 = __hadd(u16, bias_u); }
                        const __half out = silu_mul(g16, u16);
                        const int row = cc * 32 + e + (is_up ? 16 : 0);          // row of this warp's half of the tile
                        if constexpr (TMA_Y) {
                            reinterpret_cast<__half*>(stage + row * 32)[local_col] = out;
                        } else {
                            const int m = m0 + half * (MT / 2) + row;
                            if (out_ok && m < a.m) a.y[int64_t(m) * a.ldy + out_col] = out;
                        }
                    }
                    (void)col;
                }
                if constexpr (TMA_Y) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    const int nw = (n0 + quad * 32) >> 1, mw = m0 + half * (MT / 2);
                    if (lane == 0 && n0 + quad * 32 < a.n && mw < a.m) {
                        tma_store_2d(&ymap, smem_u32(stage), nw, mw);          // box 16 columns x MT/2 rows of the [M, n/2] output
                        tma_store_wait_read();
                    }
                }
            } else if constexpr (TMA_Y) {
                // [MT/2 rows of y][32 columns] FP16, 64-byte rows: the lanes of a warp write one row per store
                uint8_t* stage = x_base + (warp - 2) * ((MT / 2) * 64);
#pragma unroll 1
                for (int cc = 0; cc < MT / 64; ++cc) {
                    uint32_t v[32];
                    load_chunk(cc, v);
                    uint16_t* row = reinterpret_cast<uint16_t*>(stage + cc * 32 * 64) + lane;
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {          // packed FP32 -> FP16 conversion, two rows of y at a time
                        uint32_t p = pack_f16(__uint_as_float(v[e]), __uint_as_float(v[e + 1]));
                        if (a.bias) {
                            const __half2 sum = __hadd2(*reinterpret_cast<const __half2*>(&p), __half2half2(bias));
                            p = *reinterpret_cast<const uint32_t*>(&sum);
                        }
                        row[e * 32] = uint16_t(p);
                        row[(e + 1) * 32] = uint16_t(p >> 16);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic-proxy stores -> TMA store
                __syncwarp();
                const int nw = n0 + quad * 32, mw = m0 + half * (MT / 2);
                if (lane == 0 && nw < a.n && mw < a.m) {
                    tma_store_2d(&ymap, smem_u32(stage), nw, mw);
                    tma_store_wait_read();                                      // shared memory is released at exit
                }
            } else {
#pragma unroll 1
                for (int cc = 0; cc < MT / 64; ++cc) {
                    const int col = half * (MT / 2) + cc * 32;           // x rows col .. col+31 of the pair tile
                    uint32_t v[32];
                    load_chunk(cc, v);
                    if (n_ok) {
                        __half* dst = a.y + int64_t(m0 + col) * a.ldy + n;
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            uint32_t p = pack_f16(__uint_as_float(v[e]), __uint_as_float(v[e + 1]));
                            if (a.bias) {
                                const __half2 sum = __hadd2(*reinterpret_cast<const __half2*>(&p), __half2half2(bias));
                                p = *reinterpret_cast<const uint32_t*>(&sum);
                            }
                            uint16_t* out16 = reinterpret_cast<uint16_t*>(dst);
                            if (m0 + col + e < a.m) out16[int64_t(e) * a.ldy] = uint16_t(p);
                            if (m0 + col + e + 1 < a.m) out16[int64_t(e + 1) * a.ldy] = uint16_t(p >> 16);
                        }
                    }
                }
            }
        }
    }
    // Neither CTA may leave (or free tensor memory) while the other can still read its shared
    // memory, arrive on its barriers or write its accumulator.
    __syncwarp();
    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace b2
