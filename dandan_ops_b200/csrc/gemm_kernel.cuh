// Prefill kernel: y[M,N] = x[M,K] @ W^T on the 5th-generation tensor cores (tcgen05).
//
// One CTA computes a tile of 128 rows of x by 128 output columns, or 256 rows by 192 columns:
//   D[m][n] (FP32, tensor memory, 128 lanes x BN columns per accumulator, MA accumulators)
//     += A[m][k] (x tile, FP16, shared memory, loaded by TMA with the 128-byte swizzle)
//      * B[n][k] (weight tile, FP16, shared memory, written by the converter warps)
// in steps of 64 columns of K (one quantization group per weight row).
//
// Warp roles (2 + BN/16 warps):
//   warp 0      copy producer: per 256-column block one bulk copy of the BN/16 native weight
//               blocks of the tile (contiguous in the image) into the raw ring, and
//               per 64-column step the TMA loads of the x tile(s)
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane) and
//               tcgen05.commit, frees tensor memory
//   warps 2..   converters: dequantize the 4-bit codes of one 64-column step exactly
//               (w = fp16_rn(fp32(code - zero) * step)) and store the FP16 tile in the
//               canonical K-major 128-byte-swizzled layout the MMA descriptor expects;
//               afterwards the same warps run the epilogue (tcgen05.ld -> FP16 -> global)
//
// Rings and barriers (every wait is bounded; a wait that gives up raises the CTA's abort
// flag, records kStatusGemmTimeout in the status word and all roles leave):
//   raw_full[r]  tx-count barrier, completed by the bulk copy of raw stage r
//   raw_free[r]  one arrival per converter warp after the last read of raw stage r
//   a_full[s]    tx-count barrier, completed by the TMA load(s) of x for step-stage s
//   b_full[s]    one arrival per converter warp (after fence.proxy.async)
//   ab_free[s]   tcgen05.commit after the MMAs that read stage s
//   acc_full     tcgen05.commit after the last MMA of the tile
//
// Tails: TMA zero-fills rows >= M and columns >= K of x, the image holds zero weights for
// rows >= N and columns >= K, the epilogue masks rows >= M and columns >= N.  The kernel
// needs K % 8 == 0 and a 16-byte aligned x (TMA strides); other calls use the streaming
// kernel.
#pragma once
#include <cuda.h>
#include "layout.cuh"
#include "stream_kernel.cuh"

namespace b2 {

// BN = output columns (weight rows) per CTA: 192 when two accumulators are used (the x tiles
// are re-read from L2 by every column tile, and L2 bandwidth is what bounds this kernel, so a
// wider tile means proportionally less traffic per flop), 128 otherwise.
constexpr int kGemmBK = 64;                     // K per step = one quantization group
constexpr int kGemmStages = 3;                  // ring of 64-column FP16 operand stages
constexpr int kGemmABytes = 128 * kGemmBK * 2;                     // 16384 per 128 rows of x
constexpr unsigned kStatusGemmTimeout = 2u;
__host__ __device__ constexpr int gemm_raw_stages(int bn) { return bn == 128 ? 3 : 2; }   // 256-column raw blocks
__host__ __device__ constexpr int gemm_raw_bytes(int bn) { return (bn / 16) * kBlockBytes; }
__host__ __device__ constexpr int gemm_b_bytes(int bn) { return bn * kGemmBK * 2; }
__host__ __device__ constexpr int gemm_threads(int bn) { return 64 + 2 * bn; }              // two roles + converters
__host__ __device__ constexpr int gemm_smem_bytes(int ma, int bn) {
    // 1024-byte alignment slack + operand stages + raw ring + barriers/flags
    return 1024 + kGemmStages * (gemm_b_bytes(bn) + ma * kGemmABytes) + gemm_raw_stages(bn) * gemm_raw_bytes(bn) + 256;
}

struct GemmArgs {
    const uint8_t* native;
    __half* y;
    unsigned* status;
    const __half* bias;     // optional [N] FP16 (may be null)
    int64_t ldy;
    int m, n, k;
    int n16, kb;
    // K-splitting (pair kernel only): blockIdx.z works on its share of the 256-column blocks and
    // the FP32 partial tiles meet in `partial`; the last CTA to arrive at a tile's ticket adds
    // them in split order (deterministic) and writes y.  splits == 1: neither pointer is used.
    float* partial;
    unsigned* tickets;
    int splits;
    // Pair kernel only: 1 = rows g / g+8 of every 16-row weight tile are a gate/up pair and y gets
    // n/2 columns, y[m][8*tile+g] = silu_mul(gate, up) (as StreamArgs::act).
    int act;
};

// ---- tcgen05 / TMA helpers ----------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and the 128-byte
// swizzle: 8-row groups are 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= uint64_t(1) << 16;                             // leading byte offset (unused for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= uint64_t(1) << 46;                             // descriptor version (sm_100)
    d |= uint64_t(2) << 61;                             // SWIZZLE_128B
    return d;
}

// Eight weights of one native word -> eight FP16 values in column order (16 bytes).
// s2 = twice(step), c_even = -(1024 + zero), c_odd = -(64 + zero).
template <bool H16>
__device__ __forceinline__ uint4 dequant_word(uint32_t w, const GroupConst<H16>& g) {
    const uint32_t u = w >> 8;
    return make_uint4(dq_even<H16>(and_or(w, 0x000F000Fu, 0x64006400u), g), dq_odd<H16>(and_or(w, 0x00F000F0u, 0x64006400u), g),
                      dq_even<H16>(and_or(u, 0x000F000Fu, 0x64006400u), g), dq_odd<H16>(and_or(u, 0x00F000F0u, 0x64006400u), g));
}
__device__ __forceinline__ uint4 dequant_word(uint32_t w, float c_even, float c_odd, uint64_t s2) {
    const uint32_t u = w >> 8;
    return make_uint4(dequant_pair_even(and_or(w, 0x000F000Fu, 0x64006400u), c_even, s2),
                      dequant_pair_odd(and_or(w, 0x00F000F0u, 0x64006400u), c_odd, s2),
                      dequant_pair_even(and_or(u, 0x000F000Fu, 0x64006400u), c_even, s2),
                      dequant_pair_odd(and_or(u, 0x00F000F0u, 0x64006400u), c_odd, s2));
}

// MA = accumulators of 128 rows of x each (1 or 2).  VEC: y rows may be written with
// 16-byte stores (N % 8 == 0, ldy % 8 == 0, y 16-byte aligned).
template <int MA, int BN, bool VEC>
__global__ void __launch_bounds__(gemm_threads(BN), 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap xmap, const GemmArgs a) {
    constexpr int kGemmBN = BN, kGemmRawStages = gemm_raw_stages(BN), kGemmRawBytes = gemm_raw_bytes(BN);
    constexpr int kGemmBBytes = gemm_b_bytes(BN), kGemmConverters = BN / 16;   // converter warps
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the swizzle pattern
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int kStageBytes = kGemmBBytes + MA * kGemmABytes;
    uint8_t* stage_base = smem;                                           // [kGemmStages][B | A0 | A1]
    uint8_t* raw_base = smem + kGemmStages * kStageBytes;                 // [kGemmRawStages][18688]
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw_base + kGemmRawStages * kGemmRawBytes);
    // barrier indices
    constexpr int RAW_FULL = 0, RAW_FREE = RAW_FULL + kGemmRawStages, A_FULL = RAW_FREE + kGemmRawStages,
                  B_FULL = A_FULL + kGemmStages, AB_FREE = B_FULL + kGemmStages, ACC_FULL = AB_FREE + kGemmStages,
                  NBARS = ACC_FULL + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + i * 8; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x, tile_m = blockIdx.y;
    const int n_tiles16 = kGemmBN / 16;
    const int ksteps = (a.k + kGemmBK - 1) / kGemmBK;   // steps that contain real columns

    if (threadIdx.x == 0) {
        for (int i = 0; i < kGemmRawStages; ++i) { mbar_init(bar(RAW_FULL + i), 1); mbar_init(bar(RAW_FREE + i), kGemmConverters); }
        for (int i = 0; i < kGemmStages; ++i) {
            mbar_init(bar(A_FULL + i), 1); mbar_init(bar(B_FULL + i), kGemmConverters); mbar_init(bar(AB_FREE + i), 1);
        }
        mbar_init(bar(ACC_FULL), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    constexpr uint32_t kTmemCols = (MA * BN <= 128) ? 128 : (MA * BN <= 256) ? 256 : 512;
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto give_up = [&]() {
        *abort_flag = 1;
        atomicOr(a.status, kStatusGemmTimeout);
    };
    // Bounded wait that also leaves when another role has given up.
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
            const uint8_t* src = a.native + (int64_t(tile_n) * n_tiles16) * kBlockBytes;
            const int64_t stride = int64_t(a.n16) * kBlockBytes;
            // the last row tile group may be short: copy only blocks that exist in the image
            const int blocks_here = min(n_tiles16, a.n16 - tile_n * n_tiles16);
            const uint32_t raw_bytes = uint32_t(blocks_here) * kBlockBytes;
            for (int s = 0; s < ksteps; ++s) {
                if ((s & 3) == 0) {
                    const int kb = s >> 2, r = kb % kGemmRawStages;
                    if (kb >= kGemmRawStages && !wait(RAW_FREE + r, ((kb / kGemmRawStages) - 1) & 1)) break;
                    mbar_expect_tx(bar(RAW_FULL + r), raw_bytes);
                    bulk_copy_g2s(smem_u32(raw_base + r * kGemmRawBytes), src + kb * stride, raw_bytes, bar(RAW_FULL + r));
                }
                const int st = s % kGemmStages;
                if (s >= kGemmStages && !wait(AB_FREE + st, ((s / kGemmStages) - 1) & 1)) break;
                mbar_expect_tx(bar(A_FULL + st), MA * kGemmABytes);
                uint8_t* adst = stage_base + st * kStageBytes + kGemmBBytes;
#pragma unroll
                for (int i = 0; i < MA; ++i)
                    tma_load_2d(smem_u32(adst + i * kGemmABytes), &xmap, s * kGemmBK, tile_m * (MA * 128) + i * 128,
                                bar(A_FULL + st));
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ---------------------------------------
        // instruction descriptor: D = F32, A = B = F16, both K-major, N = 128, M = 128
        const uint32_t idesc = (1u << 4) | (uint32_t(kGemmBN >> 3) << 17) | (uint32_t(128 >> 4) << 24);
        for (int s = 0; s < ksteps; ++s) {
            const int st = s % kGemmStages;
            const uint32_t par = (s / kGemmStages) & 1;
            if (!wait(A_FULL + st, par) || !wait(B_FULL + st, par)) break;
            tcgen05_fence_after();
            if (lane == 0) {
                const uint32_t b_addr = smem_u32(stage_base + st * kStageBytes);
#pragma unroll
                for (int i = 0; i < MA; ++i) {
                    const uint32_t a_addr = b_addr + kGemmBBytes + i * kGemmABytes;
#pragma unroll
                    for (int kk = 0; kk < kGemmBK / 16; ++kk)
                        umma_f16(tmem_base + i * BN, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32),
                                 idesc, (s > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar(AB_FREE + st));
                if (s == ksteps - 1) umma_commit(bar(ACC_FULL));
            }
            __syncwarp();
        }
    } else {
        // ------------------------------ converters ---------------------------------------
        const int ct = threadIdx.x - 64;              // 0 .. 2*BN-1
        const int r = ct >> 1, h = ct & 1;            // weight row of the tile, half of the 64-column group
        const int blk = r >> 4, rr = r & 15, g = rr & 7, hi8 = rr >> 3;
        bool ok = true;
        for (int s = 0; s < ksteps && ok; ++s) {
            const int kb = s >> 2, t = s & 3, rs = kb % kGemmRawStages, st = s % kGemmStages;
            if (t == 0) ok = wait(RAW_FULL + rs, (kb / kGemmRawStages) & 1);
            if (ok && s >= kGemmStages) ok = wait(AB_FREE + st, ((s / kGemmStages) - 1) & 1);
            if (!ok) break;
            const uint8_t* nb = raw_base + rs * kGemmRawBytes + blk * kBlockBytes;
            const int lane_idx = 4 * g + t;
            const uint4 code = *reinterpret_cast<const uint4*>(nb + (2 * hi8 + h) * 512 + lane_idx * 16);
            const float step = *reinterpret_cast<const float*>(nb + kStepOffset + (lane_idx * 2 + hi8) * 4);
            const float z = float((nb[kZeroOffset + lane_idx] >> (4 * hi8)) & 15);
            const float c_even = -(1024.0f + z), c_odd = -(64.0f + z);
            uint8_t* brow = stage_base + st * kStageBytes + r * 128;
            const uint32_t words[4] = {code.x, code.y, code.z, code.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int chunk = 4 * h + i;
                *reinterpret_cast<uint4*>(brow + ((chunk ^ (r & 7)) << 4)) = dequant_word(words[i], c_even, c_odd, twice(step));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic-proxy stores -> MMA (async proxy)
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar(B_FULL + st));
                if (t == 3 || s == ksteps - 1) mbar_arrive(bar(RAW_FREE + rs));
            }
        }
        // ------------------------------ epilogue -----------------------------------------
        if (ok && wait(ACC_FULL, 0)) {
            tcgen05_fence_after();
            const int quad = warp & 3;                 // tensor-memory lanes 32*quad .. 32*quad+31
            const int part = (warp - 2) >> 2;          // BN/64 warps share a lane quadrant, 64 columns each
#pragma unroll
            for (int i = 0; i < MA; ++i) {
                const int m = tile_m * (MA * 128) + i * 128 + quad * 32 + lane;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int col = part * 64 + cc * 32;
                    uint32_t v[32];
                    tmem_ld32(tmem_base + (uint32_t(quad * 32) << 16) + i * BN + col, v);
                    const int n0 = tile_n * kGemmBN + col;
                    if (m < a.m) {
                        __half* dst = a.y + int64_t(m) * a.ldy + n0;
                        if (VEC && n0 + 32 <= a.n) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t p[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    __half2 hh = __floats2half2_rn(__uint_as_float(v[q * 8 + 2 * e]), __uint_as_float(v[q * 8 + 2 * e + 1]));
                                    if (a.bias) hh = __hadd2(hh, *reinterpret_cast<const __half2*>(a.bias + n0 + q * 8 + 2 * e));
                                    p[e] = *reinterpret_cast<uint32_t*>(&hh);
                                }
                                *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(p[0], p[1], p[2], p[3]);
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                if (n0 + e < a.n) dst[e] = finish_output(__uint_as_float(v[e]), a.bias, n0 + e);
                        }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace b2
