// C ABI of the engine: argument checks, launch planning and kernel launches.
// Declarations and the per-function reference citations are in include/b2_w4a16.h.
#include <cuda_runtime.h>
#include <algorithm>
#include <atomic>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/b2_w4a16.h"
#include "layout.cuh"
#include "layout_kernels.cuh"
#include "stream_kernel.cuh"
#include "stream2_kernel.cuh"
#include "stream2d_kernel.cuh"
#include "gemm_kernel.cuh"
#include "gemm_pair_kernel.cuh"
#include "tile_kernel.cuh"
#include "gather_kernel.cuh"
#include "rmsnorm.cuh"

namespace {

thread_local std::string g_error;
std::atomic<int64_t> g_launches{0};

int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}

int cuda_fail(const char* what, cudaError_t e) {
    return fail(B2_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

int after_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(what, e);
    return B2_OK;
}

struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
};

// Per-device properties, read once per device.
int device_info(DeviceInfo& out) {
    static DeviceInfo cache[64];
    static std::atomic<bool> ready[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail("cudaGetDevice", e);
    if (dev < 0 || dev >= 64) return fail(B2_ERR_UNSUPPORTED, "device ordinal out of range");
    if (!ready[dev].load(std::memory_order_acquire)) {
        DeviceInfo info;
        e = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail("cudaDeviceGetAttribute", e);
        e = cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return cuda_fail("cudaDeviceGetAttribute", e);
        cache[dev] = info;
        ready[dev].store(true, std::memory_order_release);
    }
    out = cache[dev];
    return B2_OK;
}

int check_dims(int64_t n, int64_t k) {
    if (n <= 0 || k <= 0) return fail(B2_ERR_ARGUMENT, "n and k must be positive");
    if (k > INT_MAX - 256 || n > INT_MAX - 64 || n * k > INT_MAX)
        return fail(B2_ERR_RANGE, "W4A16 dimensions exceed the kernel index range");
    return B2_OK;
}

// ---------------------------------------------------------------------------------------
// Launch plan of the streaming kernel (stream-K over persistent CTAs).
// ---------------------------------------------------------------------------------------
// Test hooks (b2_w4a16_test_hooks): the poll limit of the kernels' bounded waits and a one-shot request to
// leave one weight copy out, so that a test can watch a wait run out without anything hanging.
std::atomic<int> g_wait_limit{b2::kWaitLimit};
std::atomic<int> g_fault_step{-1};
std::atomic<long long> g_gather_wait_ns{5000000000LL};   // five seconds
std::atomic<int> g_stream_variant{0};     // 0/1 = w4a16_stream_kernel; 2 = w4a16_stream2_kernel with 32 warps wherever it applies;
                                          // 3 = w4a16_stream2_kernel with 16 warps (M <= 16);
                                          // 4 = w4a16_stream2d_kernel (chunk-major split) wherever K exceeds the x buffer

struct StreamPlan {
    int mt;            // 8-row tiles of x per launch: 1, 2, 4 or 8
    int rows;          // rows of x per launch = min(m, 64)
    int warps;         // warps (row tiles) per CTA: 32 (w4a16_stream2_kernel), 16 or 4
    int groups;        // row groups = ceil(n16 / warps)
    long long steps;   // groups * column blocks
    int grid;          // persistent CTAs
    int max_parts;     // most CTAs that share one row group
    int64_t partial_bytes;
    int chunk_blocks;  // two-dimensional split (w4a16_stream2d_kernel): column blocks per K chunk, 0 = not used
    int nchunks;
};

// Column blocks of x the streaming kernels' x buffer holds for `rows` staged rows (as the kernels compute it).
int stream_x_blocks(int warps, int rows) {
    const int chunk = rows * 144 + ((32 - rows * 16) & 127);
    return b2::stream_x_bytes(warps) / (4 * chunk);
}

StreamPlan plan_stream(int64_t m, const b2::Dims& d, int sm_count) {
    StreamPlan p;
    const int sms = sm_count > 0 ? sm_count : 148;
    p.rows = int(m < B2_STREAM_MAX_M ? m : B2_STREAM_MAX_M);
    p.mt = p.rows <= 8 ? 1 : p.rows <= 16 ? 2 : p.rows <= 32 ? 4 : 8;
    // 16-warp CTAs (one per SM) when the layer has at least two steps per SM for them,
    // else 4-warp CTAs (four per SM) so that small layers still spread over the chip.
    const long long steps16 = (long long)((d.n16 + 15) / 16) * d.kb;
    p.warps = (steps16 >= 2LL * sms && p.mt <= 4) ? 16 : 4;
    if (p.mt == 8) p.warps = 16;                      // the 16 KB x buffer of a 4-warp CTA cannot hold 64 rows
    // The 32-warp form (w4a16_stream2_kernel) runs only when asked for (b2_w4a16_test_hooks): measured on the
    // 8B/70B projections it is 5-15 % behind the 16-warp kernels (more warps per scheduler, but more
    // instructions per block under the 64-register cap).
    const long long steps32 = (long long)((d.n16 + 31) / 32) * d.kb;
    const int variant = g_stream_variant.load(std::memory_order_relaxed);
    if (p.mt <= 2 && variant == 2 && steps32 >= sms) p.warps = 32;
    p.groups = (d.n16 + p.warps - 1) / p.warps;
    p.steps = (long long)p.groups * d.kb;
    long long slots = (long long)sms * (p.warps == 32 ? 1 : p.warps == 16 ? B2_STREAM_CTAS16 : 4);
    // one ticket per row tile of a split row group: at most min(groups, grid) * warps of them
    const long long ticket_slots = B2_W4A16_TICKET_BYTES / 4 - 1;
    if (p.groups > slots && slots * p.warps > ticket_slots) slots = ticket_slots / p.warps;
    p.grid = int(p.steps < slots ? p.steps : slots);
    const long long per_cta = p.steps / p.grid;       // >= 1
    long long parts = (d.kb + per_cta - 1) / per_cta + 1;
    if (parts > p.grid) parts = p.grid;
    p.max_parts = int(parts);
    const long long split_tiles = (long long)(p.groups < p.grid ? p.groups : p.grid) * p.warps;
    p.partial_bytes = p.grid > 1 ? split_tiles * p.max_parts * p.mt * 512 : 0;
    // Two-dimensional split: when K does not fit in the x buffer, cut it into chunks that do and number the
    // steps chunk-major, so that a CTA stages x once (w4a16_stream2d_kernel).  Every row tile then has a
    // ticket and nchunks or a few more partial slots.
    p.chunk_blocks = 0;
    p.nchunks = 1;
    const int xblocks = stream_x_blocks(16, (p.mt == 1 && p.rows <= 4) ? p.rows : p.mt * 8);
    // Measured 2-8 % behind the one-dimensional split on the 8B/70B projections (the fence + ticket round trip of
    // every tile costs more than the x phases it removes), so it runs only when asked for (stream_variant 4).
    if (p.warps == 16 && p.mt <= 2 && variant == 4 && d.kb > xblocks && p.grid > 1) {
        const int nch = (d.kb + xblocks - 1) / xblocks;
        const int cb = (d.kb + nch - 1) / nch;
        if (nch <= 32 && (long long)p.groups * 16 <= ticket_slots && (d.kb + cb - 1) / cb == nch) {
            p.chunk_blocks = cb;
            p.nchunks = nch;
            p.max_parts = int(nch * ((cb + per_cta - 1) / per_cta + 1));
            p.partial_bytes = (long long)p.groups * 16 * p.max_parts * p.mt * 512;
        }
    }
    return p;
}

// Plain launch, or (dependent) a launch that may begin while the previous kernel of the stream is still
// draining: its CTAs run up to their griddepcontrol.wait, which returns once that kernel has completed.
template <typename Kernel, typename... Args>
int launch_maybe_dependent(const char* name, Kernel kernel, int grid, int threads, int smem, cudaStream_t s, bool dependent,
                           const Args&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(threads));
    cfg.dynamicSmemBytes = size_t(smem);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (e != cudaSuccess) return cuda_fail(name, e);
    return B2_OK;
}

// Up to this many rows of x the streaming kernel stages only the rows that exist (template parameter XROWS).
constexpr int kStreamExactRows = 4;

template <int MT, bool XVEC, int W, bool H16 = false, bool XROWS = false>
int launch_stream_one(const b2::StreamArgs& a, int grid, cudaStream_t s) {
    if constexpr (MT == 1 && !XROWS) {
        if (a.m <= kStreamExactRows) return launch_stream_one<MT, XVEC, W, H16, true>(a, grid, s);
    }
    auto kernel = b2::w4a16_stream_kernel<MT, XVEC, W, H16, XROWS>;
    constexpr int smem = b2::stream_smem_bytes(W);
    // Opt in to >48 KB of dynamic shared memory once per device and instantiation.
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        configured.fetch_or(bit, std::memory_order_release);
    }
    return launch_maybe_dependent("w4a16_stream_kernel", kernel, grid, W * 32, smem, s, a.overlap != 0, a);
}

constexpr int kNotFused = -1000;            // internal: the fused projection + gather does not apply, use two launches

// Projection + all-gather in one launch (w4a16_stream_gather_kernel).  Its CTAs wait for packets from other
// GPUs, so the whole grid must be resident at once: checked against the occupancy the runtime reports.
template <int MT, int W, bool H16, bool XROWS = false>
int launch_stream_gather_one(const b2::StreamArgs& a, const b2::GatherArgs& ga, int grid, int sms, cudaStream_t s) {
    if constexpr (MT == 1 && !XROWS) {
        if (a.m <= kStreamExactRows) return launch_stream_gather_one<MT, W, H16, true>(a, ga, grid, sms, s);
    }
    auto kernel = b2::w4a16_stream_gather_kernel<MT, W, H16, XROWS>;
    constexpr int smem = b2::stream_smem_bytes(W);
    static std::atomic<uint64_t> configured{0};
    static std::atomic<int> per_sm[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return kNotFused;
    const uint64_t bit = 1ull << dev;
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        int blocks = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, W * 32, smem);
        if (e != cudaSuccess) return cuda_fail("cudaOccupancyMaxActiveBlocksPerMultiprocessor", e);
        per_sm[dev].store(blocks, std::memory_order_relaxed);
        configured.fetch_or(bit, std::memory_order_release);
    }
    if ((long long)grid > (long long)per_sm[dev].load(std::memory_order_relaxed) * sms) return kNotFused;
    return launch_maybe_dependent("w4a16_stream_gather_kernel", kernel, grid, W * 32, smem, s, a.overlap != 0, a, ga);
}

template <int MT, bool XVEC, int W>
int launch_stream2_one(const b2::StreamArgs& a, int grid, cudaStream_t s) {
    auto kernel = b2::w4a16_stream2_kernel<MT, XVEC, W>;
    constexpr int smem = b2::s2_smem_bytes(MT);
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        configured.fetch_or(bit, std::memory_order_release);
    }
    kernel<<<grid, W * 32, smem, s>>>(a);
    return after_launch("w4a16_stream2_kernel");
}

template <int MT, bool XVEC, bool H16>
int launch_stream2d_one(const b2::StreamArgs& a, int grid, cudaStream_t s) {
    auto kernel = b2::w4a16_stream2d_kernel<MT, XVEC, H16>;
    constexpr int smem = b2::stream_smem_bytes(16);
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        configured.fetch_or(bit, std::memory_order_release);
    }
    kernel<<<grid, 16 * 32, smem, s>>>(a);
    return after_launch("w4a16_stream2d_kernel");
}

template <int MT>
int launch_stream(const b2::StreamArgs& a, bool xvec, int warps, int grid, cudaStream_t s, bool h16) {
    if constexpr (MT <= 2) {
        if (a.nchunks > 1) {
            if (h16 && xvec) return launch_stream2d_one<MT, true, true>(a, grid, s);
            return xvec ? launch_stream2d_one<MT, true, false>(a, grid, s) : launch_stream2d_one<MT, false, false>(a, grid, s);
        }
        // FP16-step chain: up to 16 rows of an aligned x (the decode case it was built for)
        if (h16 && xvec && warps == 16) return launch_stream_one<MT, true, 16, true>(a, grid, s);
        if (h16 && xvec && warps == 4) return launch_stream_one<MT, true, 4, true>(a, grid, s);
        if (warps == 32) return xvec ? launch_stream2_one<MT, true, 32>(a, grid, s) : launch_stream2_one<MT, false, 32>(a, grid, s);
        if (warps == 16 && g_stream_variant.load(std::memory_order_relaxed) == 3)
            return xvec ? launch_stream2_one<MT, true, 16>(a, grid, s) : launch_stream2_one<MT, false, 16>(a, grid, s);
    }
    if constexpr (MT == 8) {
        return xvec ? launch_stream_one<MT, true, 16>(a, grid, s) : launch_stream_one<MT, false, 16>(a, grid, s);
    } else {
        if (warps == 16)
            return xvec ? launch_stream_one<MT, true, 16>(a, grid, s) : launch_stream_one<MT, false, 16>(a, grid, s);
        return xvec ? launch_stream_one<MT, true, 4>(a, grid, s) : launch_stream_one<MT, false, 4>(a, grid, s);
    }
}

// ---------------------------------------------------------------------------------------
// Latency-oriented tile kernel: whole K of one row tile per CTA (small and mid-size layers).
// ---------------------------------------------------------------------------------------
constexpr int kTileSmemLimit = 200 * 1024;
constexpr int64_t kTileMaxBlocks = 4096;       // native blocks (9.6 MB of image) at 9..16 rows of x; larger layers stream

// CTAs per row tile of the tile kernel (a cluster that splits K): the largest of 4 and 2 that leaves
// every CTA at least 8 half blocks (measured: a 1024 x 2048 layer gains 10 % from two CTAs of 8 warps, a
// 1024 x 1024 layer loses 15 % from two of 4) and fits all clusters on the device at once; else 1.
int tile_ksplit(const b2::Dims& d, int sms, bool clusters_ok = true) {
    if (!clusters_ok) return 1;
    for (int s = 4; s >= 2; s >>= 1)
        if (int64_t(s) * d.n16 <= sms && d.kb * 2 >= s * 8) return s;
    return 1;
}

bool tile_applicable(int64_t rows, const b2::Dims& d, int split) {
    if (rows > 16) return false;
    const int kb_cta = (d.kb + split - 1) / split;
    const int warps = kb_cta * 2 < b2::kTileMaxWarps ? kb_cta * 2 : b2::kTileMaxWarps;
    // Native blocks up to which one CTA per row tile beats the persistent streaming kernel (measured on
    // N x 4096 and 4096 x 8192 layers): the fewer rows of x, the less shared memory a CTA stages and the
    // more CTAs share an SM.
    const int64_t limit = rows == 1 ? 2 * kTileMaxBlocks : rows <= 8 ? 3 * kTileMaxBlocks / 2 : kTileMaxBlocks;
    const int smem = split > 1 ? b2::tile_smem_bytes(kb_cta, rows <= 8 ? 8 : 16, warps) + split * (rows <= 8 ? 1 : 2) * 512
                               : b2::tile_smem_bytes(d.kb, int(rows), warps);
    return int64_t(d.n16) * d.kb <= limit && smem <= kTileSmemLimit;
}

bool pair_available();

template <int MT, bool XVEC, bool FULL, bool H16 = false>
int launch_tile_one(const b2::TileArgs& a, int smem, cudaStream_t s) {
    auto kernel = b2::w4a16_tile_kernel<MT, XVEC, FULL, H16>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileSmemLimit);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        configured.fetch_or(bit, std::memory_order_release);
    }
    if (a.ksplit == 1 && !a.overlap) {
        kernel<<<a.n16, a.warps * 32, smem, s>>>(a);
        return after_launch("w4a16_tile_kernel");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(a.n16) * unsigned(a.ksplit), 1, 1);
    cfg.blockDim = dim3(unsigned(a.warps) * 32, 1, 1);
    cfg.dynamicSmemBytes = size_t(smem);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int count = 0;
    if (a.ksplit > 1) {
        attr[count].id = cudaLaunchAttributeClusterDimension;
        attr[count].val.clusterDim.x = unsigned(a.ksplit); attr[count].val.clusterDim.y = 1; attr[count].val.clusterDim.z = 1;
        ++count;
    }
    if (a.overlap) {          // may start under the previous kernel's tail, see B2_FLAG_OVERLAP_LAUNCH
        attr[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    cfg.attrs = attr;
    cfg.numAttrs = unsigned(count);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, a);
    if (le != cudaSuccess) return cuda_fail("w4a16_tile_kernel", le);
    return B2_OK;
}

// The gather form of the tile kernel collects the peers' packets with the threads of ONE CTA (the last to
// finish).  Measured on two GPUs it beats projection + gather kernel while that CTA needs a single round of
// four packets per thread (4096 x 1024 at M = 1: 6.5 vs 7.4 us) and loses beyond (M = 8: 19.8 vs 7.9 us).
bool tile_gather_pays(int64_t m, const b2::Dims& d, int ksplit, int world, int64_t slice_cols) {
    const int kb_cta = (d.kb + ksplit - 1) / ksplit;
    const int warps = kb_cta * 2 < b2::kTileMaxWarps ? kb_cta * 2 : b2::kTileMaxWarps;
    return int64_t(world - 1) * m * (slice_cols / 2) <= 4LL * warps * 32;
}

template <int MT, bool FULL, bool H16>
int launch_tile_gather_one(const b2::TileArgs& a, const b2::GatherArgs& ga, int smem, cudaStream_t s) {
    auto kernel = b2::w4a16_tile_gather_kernel<MT, FULL, H16>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileSmemLimit);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        configured.fetch_or(bit, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(a.n16) * unsigned(a.ksplit), 1, 1);
    cfg.blockDim = dim3(unsigned(a.warps) * 32, 1, 1);
    cfg.dynamicSmemBytes = size_t(smem);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int count = 0;
    if (a.ksplit > 1) {
        attr[count].id = cudaLaunchAttributeClusterDimension;
        attr[count].val.clusterDim.x = unsigned(a.ksplit); attr[count].val.clusterDim.y = 1; attr[count].val.clusterDim.z = 1;
        ++count;
    }
    if (a.overlap) {
        attr[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    cfg.attrs = attr;
    cfg.numAttrs = unsigned(count);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, a, ga);
    if (le != cudaSuccess) return cuda_fail("w4a16_tile_gather_kernel", le);
    return B2_OK;
}

int run_tile(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy, int64_t rows,
             const b2::Dims& d, void* workspace, bool xvec, cudaStream_t s, const void* bias, int act = 0, int sms = 148,
             bool h16 = false, bool overlap = false, const b2::GatherArgs* ga = nullptr) {
    if (ga && (!xvec || act)) return kNotFused;       // the gather form exists for an aligned x and the plain output
    if (ga && !tile_gather_pays(rows, d, tile_ksplit(d, sms > 0 ? sms : 148, pair_available()), ga->world, ga->slice_cols))
        return kNotFused;
    b2::TileArgs a;
    a.act = act;
    a.overlap = overlap ? 1 : 0;
    a.x = static_cast<const __half*>(x);
    a.native = static_cast<const uint8_t*>(native);
    a.y = static_cast<__half*>(y);
    a.status = workspace ? static_cast<unsigned*>(workspace) + (B2_W4A16_TICKET_BYTES / 4 - 1) : nullptr;
    a.bias = static_cast<const __half*>(bias);
    a.ldx = ldx; a.ldy = ldy;
    a.m = int(rows); a.n = d.n; a.k = d.k; a.n16 = d.n16; a.kb = d.kb;
    a.wait_limit = g_wait_limit.load(std::memory_order_relaxed);
    a.fault_block = g_fault_step.exchange(-1, std::memory_order_relaxed);
    const int mt = rows <= 8 ? 1 : 2;
    // Two CTAs per row tile (a cluster, K halved) when the tiles leave more than half of the SMs idle and
    // a CTA's 16 warps would each take more than one unit: the pair finishes in one round instead of two.
    a.ksplit = tile_ksplit(d, sms > 0 ? sms : 148, pair_available());
    const int kb_cta = (d.kb + a.ksplit - 1) / a.ksplit;
    a.warps = kb_cta * 2 < b2::kTileMaxWarps ? kb_cta * 2 : b2::kTileMaxWarps;
    if (a.ksplit > 1) {
        const int smem2 = b2::tile_smem_bytes(kb_cta, mt * 8, a.warps) + a.ksplit * mt * 512;      // padded rows: the grid is small
        if (ga) {
            if (mt == 1) return h16 ? launch_tile_gather_one<1, true, true>(a, *ga, smem2, s) : launch_tile_gather_one<1, true, false>(a, *ga, smem2, s);
            return h16 ? launch_tile_gather_one<2, true, true>(a, *ga, smem2, s) : launch_tile_gather_one<2, true, false>(a, *ga, smem2, s);
        }
        if (h16 && xvec) return mt == 1 ? launch_tile_one<1, true, true, true>(a, smem2, s) : launch_tile_one<2, true, true, true>(a, smem2, s);
        if (mt == 1) return xvec ? launch_tile_one<1, true, true>(a, smem2, s) : launch_tile_one<1, false, true>(a, smem2, s);
        return xvec ? launch_tile_one<2, true, true>(a, smem2, s) : launch_tile_one<2, false, true>(a, smem2, s);
    }
    // Stage all mt * 8 rows (zeros beyond M) unless that costs occupancy: the padded layout is the
    // faster one as long as every CTA of the grid still finds a place in the first wave.
    const int padded = b2::tile_smem_bytes(d.kb, mt * 8, a.warps);
    const int per_sm = padded <= kTileSmemLimit ? std::min(227 * 1024 / (padded + 1024), 2048 / (a.warps * 32)) : 0;
    const bool full = rows == mt * 8 || int64_t(d.n16) <= int64_t(per_sm) * (sms > 0 ? sms : 148);
    const int smem = b2::tile_smem_bytes(d.kb, full ? mt * 8 : int(rows), a.warps);
    if (ga) {
        if (mt == 1) {
            if (full) return h16 ? launch_tile_gather_one<1, true, true>(a, *ga, smem, s) : launch_tile_gather_one<1, true, false>(a, *ga, smem, s);
            return h16 ? launch_tile_gather_one<1, false, true>(a, *ga, smem, s) : launch_tile_gather_one<1, false, false>(a, *ga, smem, s);
        }
        if (full) return h16 ? launch_tile_gather_one<2, true, true>(a, *ga, smem, s) : launch_tile_gather_one<2, true, false>(a, *ga, smem, s);
        return h16 ? launch_tile_gather_one<2, false, true>(a, *ga, smem, s) : launch_tile_gather_one<2, false, false>(a, *ga, smem, s);
    }
    if (h16 && xvec) {
        if (mt == 1) return full ? launch_tile_one<1, true, true, true>(a, smem, s) : launch_tile_one<1, true, false, true>(a, smem, s);
        return full ? launch_tile_one<2, true, true, true>(a, smem, s) : launch_tile_one<2, true, false, true>(a, smem, s);
    }
    if (mt == 1) {
        if (full) return xvec ? launch_tile_one<1, true, true>(a, smem, s) : launch_tile_one<1, false, true>(a, smem, s);
        return xvec ? launch_tile_one<1, true, false>(a, smem, s) : launch_tile_one<1, false, false>(a, smem, s);
    }
    if (full) return xvec ? launch_tile_one<2, true, true>(a, smem, s) : launch_tile_one<2, false, true>(a, smem, s);
    return xvec ? launch_tile_one<2, true, false>(a, smem, s) : launch_tile_one<2, false, false>(a, smem, s);
}

int run_stream(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy, int64_t m,
               const b2::Dims& d, void* workspace, int64_t workspace_bytes, cudaStream_t s,
               const DeviceInfo& dev, const void* bias, int act = 0, bool h16 = false,
               const b2::GatherArgs* ga = nullptr, bool overlap = false) {
    const int64_t ticket_bytes = B2_W4A16_TICKET_BYTES;
    const bool xvec = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (ldx % 8 == 0) && (d.k % 8 == 0);
    for (int64_t m0 = 0; m0 < m; m0 += B2_STREAM_MAX_M) {
        const int64_t rows = (m - m0) < B2_STREAM_MAX_M ? (m - m0) : B2_STREAM_MAX_M;
        const StreamPlan p = plan_stream(rows, d, dev.sm_count);
        if (workspace == nullptr || workspace_bytes < ticket_bytes + p.partial_bytes)
            return fail(B2_ERR_WORKSPACE, "workspace smaller than b2_w4a16_workspace_bytes()");
        b2::StreamArgs a;
        a.x = static_cast<const __half*>(x) + m0 * ldx;
        a.native = static_cast<const uint8_t*>(native);
        a.y = static_cast<__half*>(y) + m0 * ldy;      // (act: at most one chunk, see linear_impl)
        a.ticket = static_cast<unsigned*>(workspace);
        a.status = a.ticket + (B2_W4A16_TICKET_BYTES / 4 - 1);
        a.bias = static_cast<const __half*>(bias);
        a.act = act;
        a.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ticket_bytes);
        a.ldx = ldx; a.ldy = ldy;
        a.m = int(rows); a.n = d.n; a.k = d.k;
        a.n16 = d.n16; a.kb = d.kb;
        a.groups = p.groups; a.max_parts = p.max_parts; a.steps = int(p.steps);
        a.chunk_blocks = p.chunk_blocks; a.nchunks = p.nchunks;
        a.wait_limit = g_wait_limit.load(std::memory_order_relaxed);
        a.fault_step = g_fault_step.exchange(-1, std::memory_order_relaxed);
        a.overlap = overlap ? 1 : 0;
        int rc;
        if (ga) {
            // one launch for projection and gather: 16 rows at most, aligned x, the shipped 16- or 4-warp kernel
            if (!xvec || p.mt > 2 || (p.warps != 16 && p.warps != 4) || p.nchunks > 1 || act) return kNotFused;
            const int sms = dev.sm_count > 0 ? dev.sm_count : 148;
            if (p.mt == 1) {
                if (p.warps == 16) return h16 ? launch_stream_gather_one<1, 16, true>(a, *ga, p.grid, sms, s) : launch_stream_gather_one<1, 16, false>(a, *ga, p.grid, sms, s);
                return h16 ? launch_stream_gather_one<1, 4, true>(a, *ga, p.grid, sms, s) : launch_stream_gather_one<1, 4, false>(a, *ga, p.grid, sms, s);
            }
            if (p.warps == 16) return h16 ? launch_stream_gather_one<2, 16, true>(a, *ga, p.grid, sms, s) : launch_stream_gather_one<2, 16, false>(a, *ga, p.grid, sms, s);
            return h16 ? launch_stream_gather_one<2, 4, true>(a, *ga, p.grid, sms, s) : launch_stream_gather_one<2, 4, false>(a, *ga, p.grid, sms, s);
        }
        switch (p.mt) {
            case 1: rc = launch_stream<1>(a, xvec, p.warps, p.grid, s, h16); break;
            case 2: rc = launch_stream<2>(a, xvec, p.warps, p.grid, s, h16); break;
            case 4: rc = launch_stream<4>(a, xvec, p.warps, p.grid, s, h16); break;
            default: rc = launch_stream<8>(a, xvec, p.warps, p.grid, s, h16); break;
        }
        if (rc != B2_OK) return rc;
    }
    return B2_OK;
}

// ---------------------------------------------------------------------------------------
// Built-in scratch for b2_w4a16_linear_static: a fixed array in device memory that every GPU
// loading this library carries until the process exits.  In host code the symbol below is
// only a handle; the kernels get the address that cudaGetSymbolAddress reports for the
// current device.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[B2_W4A16_STATIC_SCRATCH_BYTES];

int static_scratch(void** out) {
    static void* address[64];
    static std::atomic<bool> ready[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail("cudaGetDevice", e);
    if (dev < 0 || dev >= 64) return fail(B2_ERR_UNSUPPORTED, "device ordinal out of range");
    if (!ready[dev].load(std::memory_order_acquire)) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);      // address on the current device
        if (e != cudaSuccess) return cuda_fail("cudaGetSymbolAddress", e);
        address[dev] = ptr;
        ready[dev].store(true, std::memory_order_release);
    }
    *out = address[dev];
    return B2_OK;
}

int64_t stream_workspace_bytes(int64_t m, const b2::Dims& d, int sm_count) {
    // The first launch has the most rows; later chunks never need more.
    const StreamPlan p = plan_stream(m, d, sm_count);
    return B2_W4A16_TICKET_BYTES + p.partial_bytes;
}

// ---------------------------------------------------------------------------------------
// tcgen05 GEMM: tensor map for x and launch.
// ---------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static std::atomic<EncodeTiledFn> cached{nullptr};
    EncodeTiledFn fn = cached.load(std::memory_order_acquire);
    if (fn) return fn;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess || ptr == nullptr)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
    cached.store(fn, std::memory_order_release);
    return fn;
}

// B2_ROUTE_AUTO hands a batch to the tensor-memory GEMM above 64 rows, and already above 32 rows on
// layers of at least 4096 native blocks (~10 MB): measured on the 8B/70B projections the pair
// kernel takes 50 / 87 / 160 us for any M in 33..192 where the streaming kernel needs 63 / 126 /
// 224 us at M = 48 (its cost grows with every 8 rows of x); at M = 32 the streaming kernel is
// still ahead (43 / 80 / 141 us), and on small layers the two are within 15 % of each other.
bool gemm_preferred(int64_t m, const b2::Dims& d) {
    return m > B2_STREAM_MAX_M || (m > 32 && int64_t(d.n16) * d.kb >= 4096);
}

bool gemm_applicable(const void* x, int64_t ldx, const b2::Dims& d) {
    return reinterpret_cast<uintptr_t>(x) % 16 == 0 && ldx % 8 == 0 && d.k % 8 == 0;
}

template <int MA, int BN, bool VEC>
int launch_gemm_one(const CUtensorMap& map, const b2::GemmArgs& a, dim3 grid, cudaStream_t s) {
    auto kernel = b2::w4a16_gemm_kernel<MA, BN, VEC>;
    constexpr int smem = b2::gemm_smem_bytes(MA, BN);
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        configured.fetch_or(bit, std::memory_order_release);
    }
    kernel<<<grid, b2::gemm_threads(BN), smem, s>>>(map, a);
    return after_launch("w4a16_gemm_kernel");
}

template <int MT, bool TMA_Y, bool H16 = false>
int launch_gemm_pair(const CUtensorMap& map, const CUtensorMap& ymap, const b2::GemmArgs& a, dim3 grid, cudaStream_t s) {
    auto kernel = b2::w4a16_gemm_pair_kernel<MT, TMA_Y, H16>;
    constexpr int smem = b2::pair_smem_bytes<MT>();
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
        configured.fetch_or(bit, std::memory_order_release);
    }
    kernel<<<grid, b2::kPairThreads, smem, s>>>(map, ymap, a);   // clusters of two along x (__cluster_dims__)
    return after_launch("w4a16_gemm_pair_kernel");
}

// Tile shapes of the GEMM.  Single-CTA kernel: (rows of x) x (output columns) = 128 x 128,
// 256 x 128 or 256 x 192 per CTA.  Pair kernel: 256 output columns x 256 rows of x per two SMs
// (one CTA per SM), or x 192 rows with two CTAs per SM; it can also split K over up to 8 CTAs per
// tile when a layer has fewer tiles than SM pairs.  The cost of one tile per SM, measured on
// large layers, is about 10 : 12 : 15 for the single-CTA shapes and 9 / 5.25 for the pair shapes;
// prologue + epilogue cost about as much as 10 of a tile's 64-column steps, a K-split adds the
// trip of the FP32 partial tiles through L2.  The candidate with the cheapest
// waves x cost-per-tile wins.
struct GemmShape {
    int ma, bn;      // single-CTA kernel: accumulators of 128 x rows, output columns
    int pair_mt;     // pair kernel: rows of x per CTA pair (256 or 192), 0 = single-CTA kernel
    int splits;      // pair kernel: CTAs along K per tile
    int64_t tiles(int64_t m, int64_t n) const {
        if (pair_mt) return ((n + 255) / 256) * ((m + pair_mt - 1) / pair_mt);
        return ((n + bn - 1) / bn) * ((m + 128 * ma - 1) / (128 * ma));
    }
    int64_t ctas(int64_t m, int64_t n) const { return tiles(m, n) * (pair_mt ? 2 * splits : 1); }
    int64_t partial_bytes(int64_t m, int64_t n) const {
        return splits > 1 ? tiles(m, n) * splits * 256 * pair_mt * int64_t(sizeof(float)) : 0;
    }
};
constexpr GemmShape kGemmShapes[5] = {{1, 128, 0, 1}, {2, 128, 0, 1}, {2, 192, 0, 1}, {0, 0, 256, 1}, {0, 0, 192, 1}};
constexpr int kMaxSplits = 8;
std::atomic<int> g_forced_shape{0};      // B2_GEMM_SHAPE_*, 0 = automatic
std::atomic<int> g_forced_splits{0};     // K-splits of the pair kernel, 0 = automatic

// Largest split count a tile grid can use: at least four 256-column blocks per CTA and one ticket
// per half tile in the workspace's ticket area (its last word is the status word).
inline int max_splits(const GemmShape& g, int64_t m, int64_t n, int kb) {
    if (g.pair_mt == 0 || 2 * g.tiles(m, n) > B2_W4A16_TICKET_BYTES / 4 - 1) return 1;
    return std::max(1, std::min(kMaxSplits, kb / 4));
}

// Can this device co-schedule the pair kernel's two-CTA clusters at all (asked once per device)?
// A partition without two free SMs in one cluster-capable group answers no, and the GEMM then
// stays on the single-CTA shapes.
bool pair_available() {
    static std::atomic<int> state[64];          // 0 = not asked yet, 1 = yes, 2 = no
    int dev = 0;
    cudaGetDevice(&dev);
    std::atomic<int>& st = state[dev & 63];
    const int known = st.load(std::memory_order_acquire);
    if (known) return known == 1;
    auto kernel = b2::w4a16_gemm_pair_kernel<192, true>;
    constexpr int smem = b2::pair_smem_bytes<192>();
    bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess;
    if (ok) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2, 1, 1);
        cfg.blockDim = dim3(b2::kPairThreads, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        ok = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters > 0;
    }
    if (!ok) cudaGetLastError();                // clear the error of a failed query
    st.store(ok ? 1 : 2, std::memory_order_release);
    return ok;
}

inline GemmShape gemm_shape(int64_t m, int64_t n, int kb, int sms, bool pairs_ok = true) {
    const int forced = pairs_ok || g_forced_shape.load(std::memory_order_relaxed) <= 3
                           ? g_forced_shape.load(std::memory_order_relaxed) : 0;
    const int forced_splits = g_forced_splits.load(std::memory_order_relaxed);
    const int64_t pairs = sms >= 2 ? sms / 2 : 1;
    // waves x cost per tile and SM (times four).  Two co-resident 192-row tiles cost 21 each; one
    // that has its SM pair to itself takes 34, nearly as long as a 256-row tile (36): the
    // converters' latency, not the MMA, sets the pace of a lone CTA.
    const int cost4[5] = {40, 48, 60, 36, 21};
    constexpr int kLone192 = 34;
    auto wave_cost = [&](int i, const GemmShape& g, int64_t items) -> int64_t {
        if (g.pair_mt == 0) return (items + sms - 1) / sms * cost4[i];
        if (g.pair_mt == 256) return (items + pairs - 1) / pairs * cost4[i];
        const int64_t rem = items % (2 * pairs);
        return 2 * (items / (2 * pairs)) * cost4[i] + (rem == 0 ? 0 : rem <= pairs ? kLone192 : 2 * cost4[i]);
    };
    GemmShape best = kGemmShapes[1];
    int64_t best_cost = INT64_MAX;
    for (int i = 0; i < 5; ++i) {
        if (forced && i != forced - 1) continue;
        if (!pairs_ok && kGemmShapes[i].pair_mt) continue;
        GemmShape g = kGemmShapes[i];
        const int smax = max_splits(g, m, n, kb);
        for (int sp = 1; sp <= smax; ++sp) {
            if (forced_splits && sp != std::min(forced_splits, smax)) continue;
            g.splits = sp;
            const int64_t steps = int64_t((kb + sp - 1) / sp) * 4 + 10 + (sp > 1 ? 4 + 2 * sp : 0);
            const int64_t c = wave_cost(i, g, g.tiles(m, n) * sp) * steps;
            if (c < best_cost) { best_cost = c; best = g; }
        }
    }
    return best;
}

// Shape the GEMM would take for this call (workspace permitting the K-split).
GemmShape gemm_shape_for_call(int64_t m, const b2::Dims& d, int sms, int64_t workspace_bytes) {
    GemmShape shape = gemm_shape(m, d.n, d.kb, sms, pair_available());
    if (B2_W4A16_TICKET_BYTES + shape.partial_bytes(m, d.n) > workspace_bytes) shape.splits = 1;   // no room: one CTA per tile
    return shape;
}

int run_gemm(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy, int64_t m,
             const b2::Dims& d, void* workspace, int64_t workspace_bytes, cudaStream_t s, int sms, const void* bias,
             int act = 0, bool h16 = false) {
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return fail(B2_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from the driver");
    if (workspace == nullptr) return fail(B2_ERR_WORKSPACE, "workspace smaller than b2_w4a16_workspace_bytes()");
    CUtensorMap map;
    const cuuint64_t dims[2] = {cuuint64_t(d.k), cuuint64_t(m)};
    const cuuint64_t strides[1] = {cuuint64_t(ldx) * 2};
    const GemmShape shape = gemm_shape_for_call(m, d, sms, workspace_bytes);
    const int pair_mt = shape.pair_mt;
    if (act && !pair_mt) return fail(B2_ERR_UNSUPPORTED, "the fused gate/up epilogue of the GEMM exists in the pair kernel only");
    const cuuint32_t box[2] = {cuuint32_t(b2::kGemmBK), pair_mt ? cuuint32_t(pair_mt / 2) : 128u};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B2_ERR_CUDA, "cuTensorMapEncodeTiled failed");
    b2::GemmArgs a;
    a.native = static_cast<const uint8_t*>(native);
    a.y = static_cast<__half*>(y);
    a.status = static_cast<unsigned*>(workspace) + (B2_W4A16_TICKET_BYTES / 4 - 1);
    a.bias = static_cast<const __half*>(bias);
    a.ldy = ldy;
    a.m = int(m); a.n = d.n; a.k = d.k; a.n16 = d.n16; a.kb = d.kb;
    a.tickets = static_cast<unsigned*>(workspace);
    a.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + B2_W4A16_TICKET_BYTES);
    a.splits = shape.splits;
    a.act = act;
    const bool vec = reinterpret_cast<uintptr_t>(y) % 16 == 0 && ldy % 8 == 0 && d.n % 8 == 0;
    if (pair_mt) {
        const dim3 pgrid(2 * unsigned((d.n + 255) / 256), unsigned((m + pair_mt - 1) / pair_mt), unsigned(shape.splits));
        // y through TMA stores (32 columns x pair_mt/2 rows per warp) when its rows are 16-byte aligned
        const bool tma_y = reinterpret_cast<uintptr_t>(y) % 16 == 0 && ldy % 8 == 0;
        CUtensorMap ymap = map;
        if (tma_y) {
            // act: the output has n/2 columns and a warp's 32 weight rows give 16 of them
            const cuuint64_t ydims[2] = {cuuint64_t(act ? d.n / 2 : d.n), cuuint64_t(m)};
            const cuuint64_t ystrides[1] = {cuuint64_t(ldy) * 2};
            const cuuint32_t ybox[2] = {act ? 16u : 32u, cuuint32_t(pair_mt / 2)};
            if (encode(&ymap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, y, ydims, ystrides, ybox, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return fail(B2_ERR_CUDA, "cuTensorMapEncodeTiled failed for y");
            if (h16) return pair_mt == 256 ? launch_gemm_pair<256, true, true>(map, ymap, a, pgrid, s) : launch_gemm_pair<192, true, true>(map, ymap, a, pgrid, s);
            return pair_mt == 256 ? launch_gemm_pair<256, true>(map, ymap, a, pgrid, s) : launch_gemm_pair<192, true>(map, ymap, a, pgrid, s);
        }
        return pair_mt == 256 ? launch_gemm_pair<256, false>(map, ymap, a, pgrid, s) : launch_gemm_pair<192, false>(map, ymap, a, pgrid, s);
    }
    const int ma = shape.ma, bn = shape.bn;
    const dim3 grid((d.n + bn - 1) / bn, unsigned((m + 128 * ma - 1) / (128 * ma)));
    if (ma == 1) return vec ? launch_gemm_one<1, 128, true>(map, a, grid, s) : launch_gemm_one<1, 128, false>(map, a, grid, s);
    if (bn == 128) return vec ? launch_gemm_one<2, 128, true>(map, a, grid, s) : launch_gemm_one<2, 128, false>(map, a, grid, s);
    return vec ? launch_gemm_one<2, 192, true>(map, a, grid, s) : launch_gemm_one<2, 192, false>(map, a, grid, s);
}

}  // namespace

extern "C" {

int b2_w4a16_contract_version(void) { return 2; }

const char* b2_w4a16_last_error(void) { return g_error.c_str(); }

int64_t b2_w4a16_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b2_w4a16_test_hooks(int wait_limit, int skip_copy, int stream_variant) {
    if (stream_variant < 0 || stream_variant > 4) return fail(B2_ERR_ARGUMENT, "stream_variant must be 0..4");
    g_wait_limit.store(wait_limit > 0 ? wait_limit : b2::kWaitLimit, std::memory_order_relaxed);
    g_fault_step.store(skip_copy >= 0 ? skip_copy : -1, std::memory_order_relaxed);
    g_stream_variant.store(stream_variant, std::memory_order_relaxed);
    return B2_OK;
}

int b2_w4a16_gather_wait_limit(int64_t microseconds) {
    g_gather_wait_ns.store(microseconds > 0 ? microseconds * 1000LL : 5000000000LL, std::memory_order_relaxed);
    return B2_OK;
}

int b2_w4a16_set_gemm_shape(int shape, int k_splits) {
    if (shape < B2_GEMM_SHAPE_AUTO || shape > B2_GEMM_SHAPE_PAIR_192)
        return fail(B2_ERR_ARGUMENT, "unknown GEMM tile shape");
    if (k_splits < 0 || k_splits > kMaxSplits) return fail(B2_ERR_ARGUMENT, "k_splits must be 0 (automatic) to 8");
    g_forced_shape.store(shape, std::memory_order_relaxed);
    g_forced_splits.store(k_splits, std::memory_order_relaxed);
    return B2_OK;
}

int64_t b2_w4a16_native_bytes(int64_t n, int64_t k) {
    if (check_dims(n, k) != B2_OK) return 0;
    return b2::native_bytes(b2::make_dims(n, k));
}

int b2_w4a16_repack(const int32_t* packed, const float* scales, const int32_t* zeros, int64_t n,
                    int64_t k, void* native, void* stream) {
    if (!packed || !scales || !zeros || !native) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (int rc = check_dims(n, k)) return rc;
    if (reinterpret_cast<uintptr_t>(native) % 256) return fail(B2_ERR_ARGUMENT, "native image must be 256-byte aligned");
    const b2::Dims d = b2::make_dims(n, k);
    const int64_t blocks = int64_t(d.n16) * d.kb;
    b2::repack_kernel<<<unsigned(blocks), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        packed, scales, zeros, d, static_cast<uint8_t*>(native));
    return after_launch("repack_kernel");
}

int b2_w4a16_unrepack(const void* native, int64_t n, int64_t k, int32_t* packed, float* scales,
                      int32_t* zeros, void* stream) {
    if (!packed || !scales || !zeros || !native) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (int rc = check_dims(n, k)) return rc;
    const b2::Dims d = b2::make_dims(n, k);
    const int64_t total = int64_t(d.n) * d.words;
    b2::unrepack_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(native), d, packed, scales, zeros);
    return after_launch("unrepack_kernel");
}

int b2_w4a16_pack(const uint8_t* codes, int64_t n, int64_t k, int32_t* packed, void* stream) {
    if (!codes || !packed) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (int rc = check_dims(n, k)) return rc;
    const b2::Dims d = b2::make_dims(n, k);
    const int64_t total = int64_t(d.n) * d.words;
    b2::pack_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(codes, d, packed);
    return after_launch("pack_kernel");
}

int b2_w4a16_dequantize(const void* native, int64_t n, int64_t k, float* out, int64_t ldo, void* stream) {
    if (!native || !out) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (int rc = check_dims(n, k)) return rc;
    if (ldo < k) return fail(B2_ERR_ARGUMENT, "ldo must be at least k");
    const b2::Dims d = b2::make_dims(n, k);
    const int64_t total = int64_t(d.n) * d.words;
    b2::dequantize_kernel<float><<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(native), d, out, ldo);
    return after_launch("dequantize_kernel");
}

int b2_w4a16_dequantize_fp16(const void* native, int64_t n, int64_t k, void* out, int64_t ldo, void* stream) {
    if (!native || !out) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (int rc = check_dims(n, k)) return rc;
    if (ldo < k) return fail(B2_ERR_ARGUMENT, "ldo must be at least k");
    const b2::Dims d = b2::make_dims(n, k);
    const int64_t total = int64_t(d.n) * d.words;
    b2::dequantize_kernel<__half><<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(native), d, static_cast<__half*>(out), ldo);
    return after_launch("dequantize_kernel");
}

int b2_w4a16_plan(int64_t m, int64_t n, int64_t k, int* route, int* k_splits, int* grid, int* rows_per_launch) {
    if (int rc = check_dims(n, k)) return rc;
    if (m < 0) return fail(B2_ERR_ARGUMENT, "m must be non-negative");
    DeviceInfo dev;
    if (device_info(dev) != B2_OK) dev.sm_count = 148;   // planning also works without a device
    const b2::Dims d = b2::make_dims(n, k);
    const StreamPlan p = plan_stream(m > 0 ? m : 1, d, dev.sm_count);
    if (gemm_preferred(m, d) && d.k % 8 == 0) {    // assuming an aligned x, as execution_info cannot see the pointer
        const GemmShape shape = gemm_shape(m, d.n, d.kb, dev.sm_count > 0 ? dev.sm_count : 148);
        if (route) *route = B2_ROUTE_TCGEN05;
        if (k_splits) *k_splits = shape.splits;
        if (grid) *grid = int(shape.ctas(m, d.n));
        if (rows_per_launch) *rows_per_launch = int(m);
        return B2_OK;
    }
    const int split = tile_ksplit(d, dev.sm_count > 0 ? dev.sm_count : 148);
    if (m > 0 && tile_applicable(m, d, split)) {   // whole K of a row tile per CTA, or per cluster of 2 or 4 CTAs
        if (route) *route = B2_ROUTE_TILE;
        if (k_splits) *k_splits = split;
        if (grid) *grid = d.n16 * split;
        if (rows_per_launch) *rows_per_launch = int(m);
        return B2_OK;
    }
    if (route) *route = B2_ROUTE_STREAM;
    if (k_splits) *k_splits = p.max_parts;
    if (grid) *grid = p.grid;
    if (rows_per_launch) *rows_per_launch = p.rows;
    return B2_OK;
}

int b2_w4a16_status(const void* workspace, void* stream, unsigned* status_host) {
    if (!status_host) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (!workspace) {                                  // the scratch built into the library (b2_w4a16_linear_static)
        void* scratch = nullptr;
        if (int rc = static_scratch(&scratch)) return rc;
        workspace = scratch;
    }
    const unsigned* word = static_cast<const unsigned*>(workspace) + (B2_W4A16_TICKET_BYTES / 4 - 1);
    cudaError_t e = cudaMemcpyAsync(status_host, word, sizeof(unsigned), cudaMemcpyDeviceToHost,
                                    static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail("b2_w4a16_status", e);
    return B2_OK;
}

int64_t b2_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (check_dims(n, k) != B2_OK || m < 0) return B2_W4A16_TICKET_BYTES;
    DeviceInfo dev;
    if (device_info(dev) != B2_OK) dev.sm_count = 148;
    const b2::Dims d = b2::make_dims(n, k);
    int64_t need = stream_workspace_bytes(m > 0 ? m : 1, d, dev.sm_count);
    if (gemm_preferred(m, d))     // room for the partial tiles of a K-split tensor-memory GEMM
        need = std::max(need, B2_W4A16_TICKET_BYTES + gemm_shape(m, d.n, d.kb, dev.sm_count > 0 ? dev.sm_count : 148).partial_bytes(m, d.n));
    return need;
}

}  // extern "C"

namespace {

// Empty kernel: the launch floor of a graph node, for benchmarks.
__global__ void noop_kernel() {}

// Elementwise fallback of the fused gate/up epilogue for batches the decode kernels do not take:
// in[m][16 j + g] is the gate and in[m][16 j + 8 + g] the up value of output column 8 j + g.
__global__ void silu_mul_pairs_kernel(const __half* in, int64_t ld_in, __half* out, int64_t ld_out, int m, int half_n) {
    const int64_t total = int64_t(m) * half_n;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int row = int(i / half_n), col = int(i % half_n);
        const __half* src = in + row * ld_in + (col >> 3) * 16 + (col & 7);
        out[row * ld_out + col] = b2::silu_mul(src[0], src[8]);
    }
}

// Residual + RMSNorm: one CTA of eight warps per row (b2::norm_row, csrc/rmsnorm.cuh).  `summed` may alias
// nothing else; when null the sums pass through `out`.
__global__ void __launch_bounds__(b2::kNormThreads)
residual_rms_norm_kernel(const __half* x, int64_t ldx, const __half* residual, int64_t ldr,
                         const __half* weight, float eps, __half* summed, int64_t lds,
                         __half* out, int64_t ldo, int m, int k) {
    __shared__ b2::NormScratch scratch;
    // a projection launched behind this kernel as a programmatic dependent may fetch its weights meanwhile
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int row = blockIdx.x;
    __half* o = out + row * ldo;
    b2::norm_row(x + row * ldx, residual ? residual + row * ldr : nullptr, weight, eps, summed ? summed + row * lds : o, o, k, scratch);
    (void)m;
}

// Checked arguments of a gather call and which of its forms applies.
struct GatherCall {
    b2::GatherArgs a;
    bool vec;        // 16-byte pieces (push form)
    bool mailbox;    // every rank's slice fits in a mailbox half and is made of whole 4-byte words
};

int make_gather_call(void* const* y_ranks, void* const* flag_blocks, int64_t mailbox_slice_bytes, int rank, int world,
                     int64_t m, int64_t ld, int64_t n_total, int64_t slice_cols, GatherCall& c) {
    if (!y_ranks || !flag_blocks) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (world < 1 || world > b2::kGatherMaxRanks || rank < 0 || rank >= world)
        return fail(B2_ERR_ARGUMENT, "rank / world out of range (at most 16 ranks)");
    if (m < 0 || n_total < 0 || slice_cols <= 0 || ld < n_total || slice_cols * world < n_total || mailbox_slice_bytes < 0)
        return fail(B2_ERR_ARGUMENT, "slices do not cover the row");
    if (m > INT_MAX) return fail(B2_ERR_RANGE, "m exceeds the kernel index range");
    const int64_t col0 = std::min(n_total, int64_t(rank) * slice_cols);
    const int64_t cols = std::min(slice_cols, n_total - col0);
    b2::GatherArgs& a = c.a;
    bool vec = col0 % 8 == 0 && cols % 8 == 0 && ld % 8 == 0;
    bool words = slice_cols % 2 == 0 && n_total % 2 == 0 && ld % 2 == 0;
    for (int q = 0; q < b2::kGatherMaxRanks; ++q) {
        a.y[q] = q < world ? static_cast<__half*>(y_ranks[q]) : nullptr;
        a.flags[q] = q < world ? static_cast<unsigned*>(flag_blocks[q]) : nullptr;
        if (q < world) {
            if (!a.flags[q] || (!a.y[q] && m * n_total > 0)) return fail(B2_ERR_ARGUMENT, "null pointer");
            if (reinterpret_cast<uintptr_t>(a.flags[q]) % 8 || reinterpret_cast<uintptr_t>(a.y[q]) % 2)
                return fail(B2_ERR_ARGUMENT, "misaligned buffer");
            vec = vec && reinterpret_cast<uintptr_t>(a.y[q]) % 16 == 0;
            words = words && reinterpret_cast<uintptr_t>(a.y[q]) % 4 == 0;
        }
    }
    a.rank = rank; a.world = world; a.m = int(m); a.ld = ld; a.col0 = col0; a.cols = cols;
    a.n_total = n_total; a.slice_cols = slice_cols; a.slots = mailbox_slice_bytes / 4;
    a.wait_ns = g_gather_wait_ns.load(std::memory_order_relaxed);
    c.vec = vec;
    c.mailbox = words && world > 1 && m * slice_cols * 2 <= mailbox_slice_bytes && m * slice_cols > 0;
    return B2_OK;
}

// act = 1: rows g / g+8 of every 16-row tile are a gate/up pair and y gets n/2 columns.
int linear_impl(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                int64_t workspace_bytes, void* stream, int route, int act, int flags = 0,
                const b2::GatherArgs* ga = nullptr) {
    const bool h16 = (flags & B2_FLAG_FP16_STEPS) != 0;
    const void* bias = bias_fp16;
    if (bias && reinterpret_cast<uintptr_t>(bias) % 4) return fail(B2_ERR_ARGUMENT, "bias must be 4-byte aligned");
    if (m < 0) return fail(B2_ERR_ARGUMENT, "m must be non-negative");
    if (int rc = check_dims(n, k)) return rc;
    if (m == 0) return B2_OK;
    if (!x || !native || !y) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (ldx < k || ldy < (act ? n / 2 : n)) return fail(B2_ERR_ARGUMENT, "leading dimension smaller than the row length");
    if (act && n % 16 != 0) return fail(B2_ERR_UNSUPPORTED, "the fused gate/up epilogue needs N % 16 == 0");
    if (m > INT_MAX - 128 || m * k > INT_MAX || m * n > INT_MAX)
        return fail(B2_ERR_RANGE, "W4A16 dimensions exceed the kernel index range");
    if (reinterpret_cast<uintptr_t>(native) % 16) return fail(B2_ERR_ARGUMENT, "native image must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(x) % 2 || reinterpret_cast<uintptr_t>(y) % 2)
        return fail(B2_ERR_ARGUMENT, "x and y must be 2-byte aligned");
    if (workspace && reinterpret_cast<uintptr_t>(workspace) % 16)
        return fail(B2_ERR_ARGUMENT, "workspace must be 16-byte aligned");
    DeviceInfo dev;
    if (int rc = device_info(dev)) return rc;
    if (dev.cc_major != 10) return fail(B2_ERR_UNSUPPORTED, "this library contains sm_100a code only");
    const b2::Dims d = b2::make_dims(n, k);
    const int tile_split = tile_ksplit(d, dev.sm_count, pair_available());
    if (route == B2_ROUTE_AUTO)
        route = tile_applicable(m, d, tile_split) ? B2_ROUTE_TILE
              : (gemm_preferred(m, d) && gemm_applicable(x, ldx, d)) ? B2_ROUTE_TCGEN05 : B2_ROUTE_STREAM;
    if (act && route == B2_ROUTE_TCGEN05 && !gemm_shape_for_call(m, d, dev.sm_count, workspace_bytes).pair_mt) {
        // the single-CTA GEMM has no such epilogue: small batches stream, larger ones take two launches
        if (m > B2_STREAM_MAX_M)
            return fail(B2_ERR_UNSUPPORTED, "no fused gate/up epilogue for this problem: run b2_w4a16_linear, then b2_w4a16_silu_mul_pairs");
        route = B2_ROUTE_STREAM;
    }
    if (ga && route != B2_ROUTE_STREAM && route != B2_ROUTE_TILE) return kNotFused;     // the decode kernels carry the gather
    if (route == B2_ROUTE_TILE) {
        if (!tile_applicable(m, d, tile_split))
            return fail(B2_ERR_UNSUPPORTED, "the tile route needs M <= 16 and a layer whose K range fits in shared memory");
        const bool xvec = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (ldx % 8 == 0) && (d.k % 8 == 0);
        return run_tile(x, ldx, native, y, ldy, m, d, workspace, xvec, static_cast<cudaStream_t>(stream), bias, act, dev.sm_count, h16,
                        (flags & B2_FLAG_OVERLAP_LAUNCH) != 0, ga);
    }
    if (route == B2_ROUTE_STREAM)
        return run_stream(x, ldx, native, y, ldy, m, d, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream), dev, bias, act, h16, ga, (flags & B2_FLAG_OVERLAP_LAUNCH) != 0);
    if (route == B2_ROUTE_TCGEN05) {
        if (!gemm_applicable(x, ldx, d))
            return fail(B2_ERR_UNSUPPORTED, "the tcgen05 route needs K % 8 == 0 and a 16-byte aligned x");
        if (workspace_bytes < B2_W4A16_TICKET_BYTES)
            return fail(B2_ERR_WORKSPACE, "workspace smaller than b2_w4a16_workspace_bytes()");
        return run_gemm(x, ldx, native, y, ldy, m, d, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), dev.sm_count, bias, act, h16);
    }
    return fail(B2_ERR_UNSUPPORTED, "unknown route");
}

}  // namespace

extern "C" {

int b2_w4a16_linear_bias(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                         int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                         int64_t workspace_bytes, void* stream, int route) {
    return linear_impl(x, ldx, native, bias_fp16, y, ldy, m, n, k, workspace, workspace_bytes, stream, route, 0);
}

int b2_w4a16_linear_flags(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                          int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                          int64_t workspace_bytes, void* stream, int route, int flags) {
    if (flags & ~(B2_FLAG_FP16_STEPS | B2_FLAG_OVERLAP_LAUNCH)) return fail(B2_ERR_ARGUMENT, "unknown flag");
    return linear_impl(x, ldx, native, bias_fp16, y, ldy, m, n, k, workspace, workspace_bytes, stream, route, 0, flags);
}

int b2_w4a16_linear_silu_mul(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                             int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                             int64_t workspace_bytes, void* stream) {
    return linear_impl(x, ldx, native, bias_fp16, y, ldy, m, n, k, workspace, workspace_bytes, stream, B2_ROUTE_AUTO, 1);
}

int b2_w4a16_linear_silu_mul_flags(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                                   int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                                   int64_t workspace_bytes, void* stream, int flags) {
    if (flags & ~(B2_FLAG_FP16_STEPS | B2_FLAG_OVERLAP_LAUNCH)) return fail(B2_ERR_ARGUMENT, "unknown flag");
    return linear_impl(x, ldx, native, bias_fp16, y, ldy, m, n, k, workspace, workspace_bytes, stream, B2_ROUTE_AUTO, 1, flags);
}

int b2_w4a16_rmsnorm_linear(const void* x, int64_t ldx, const void* residual, int64_t ldr, const void* norm_weight,
                            float eps, void* summed, int64_t lds, void* xn_scratch, const void* native,
                            const void* bias_fp16, void* y, int64_t ldy, int64_t m, int64_t n, int64_t k,
                            void* workspace, int64_t workspace_bytes, void* stream) {
    if (m < 0) return fail(B2_ERR_ARGUMENT, "m must be non-negative");
    if (int rc = check_dims(n, k)) return rc;
    if (m == 0) return B2_OK;
    if (!x || !norm_weight || !native || !y) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (!(eps >= 0.0f) || !std::isfinite(eps)) return fail(B2_ERR_ARGUMENT, "eps must be finite and non-negative");
    if (k % 8 != 0 || ldx % 8 != 0 || (residual && ldr % 8 != 0) || (summed && lds % 8 != 0))
        return fail(B2_ERR_UNSUPPORTED, "the RMSNorm prologue needs K and the row strides to be multiples of 8");
    for (const void* p : {x, residual, norm_weight, static_cast<const void*>(summed), static_cast<const void*>(xn_scratch)})
        if (p && reinterpret_cast<uintptr_t>(p) % 16) return fail(B2_ERR_ARGUMENT, "RMSNorm operands must be 16-byte aligned");
    if (ldx < k || (residual && ldr < k) || (summed && lds < k))
        return fail(B2_ERR_ARGUMENT, "leading dimension smaller than the row length");
    if (m > INT_MAX - 128 || m * k > INT_MAX || m * n > INT_MAX)
        return fail(B2_ERR_RANGE, "W4A16 dimensions exceed the kernel index range");
    DeviceInfo dev;
    if (int rc = device_info(dev)) return rc;
    if (dev.cc_major != 10) return fail(B2_ERR_UNSUPPORTED, "this library contains sm_100a code only");
    const b2::Dims d = b2::make_dims(n, k);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!xn_scratch) return fail(B2_ERR_ARGUMENT, "xn_scratch [M, K] is required");
    residual_rms_norm_kernel<<<unsigned(m), b2::kNormThreads, 0, s>>>(
        static_cast<const __half*>(x), ldx, static_cast<const __half*>(residual), ldr,
        static_cast<const __half*>(norm_weight), eps, static_cast<__half*>(summed), lds,
        static_cast<__half*>(xn_scratch), k, int(m), int(k));
    if (int rc = after_launch("residual_rms_norm_kernel")) return rc;
    // The projection starts under the norm kernel (its weight copies do not depend on it) and reads xn_scratch
    // after that kernel has completed.  The norm kernel itself is an ordinary launch, so everything issued
    // before this call - including whatever wrote the weight image - has finished before either kernel runs.
    return linear_impl(xn_scratch, k, native, bias_fp16, y, ldy, m, n, k, workspace, workspace_bytes, stream, B2_ROUTE_AUTO, 0,
                       B2_FLAG_OVERLAP_LAUNCH);
}

int b2_w4a16_residual_rms_norm(const void* x, int64_t ldx, const void* residual, int64_t ldr, const void* norm_weight,
                               float eps, void* summed, int64_t lds, void* out, int64_t ldo, int64_t m, int64_t k,
                               void* stream) {
    if (m < 0 || k <= 0) return fail(B2_ERR_ARGUMENT, "m >= 0 and k > 0 expected");
    if (m == 0) return B2_OK;
    if (!x || !norm_weight || !out) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (!(eps >= 0.0f) || !std::isfinite(eps)) return fail(B2_ERR_ARGUMENT, "eps must be finite and non-negative");
    if (k % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0 || (residual && ldr % 8 != 0) || (summed && lds % 8 != 0))
        return fail(B2_ERR_UNSUPPORTED, "RMSNorm needs K and the row strides to be multiples of 8");
    for (const void* p : {x, residual, norm_weight, static_cast<const void*>(summed), static_cast<const void*>(out)})
        if (p && reinterpret_cast<uintptr_t>(p) % 16) return fail(B2_ERR_ARGUMENT, "RMSNorm operands must be 16-byte aligned");
    if (ldx < k || ldo < k || (residual && ldr < k) || (summed && lds < k))
        return fail(B2_ERR_ARGUMENT, "leading dimension smaller than the row length");
    if (m > INT_MAX - 128 || k > INT_MAX - 64 || m * k > INT_MAX) return fail(B2_ERR_RANGE, "dimensions exceed the kernel index range");
    residual_rms_norm_kernel<<<unsigned(m), b2::kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), ldx, static_cast<const __half*>(residual), ldr,
        static_cast<const __half*>(norm_weight), eps, static_cast<__half*>(summed), lds,
        static_cast<__half*>(out), ldo, int(m), int(k));
    return after_launch("residual_rms_norm_kernel");
}

int b2_w4a16_silu_mul_is_fused(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || check_dims(n, k) != B2_OK || n % 16 != 0) return 0;
    if (m <= B2_STREAM_MAX_M) return 1;                    // decode kernels, or the pair GEMM, or the streaming fallback
    DeviceInfo dev;
    if (device_info(dev) != B2_OK) dev.sm_count = 148;
    const b2::Dims d = b2::make_dims(n, k);
    if (d.k % 8 != 0) return 1;                            // the streaming kernel in chunks of 64 rows
    return gemm_shape_for_call(m, d, dev.sm_count > 0 ? dev.sm_count : 148, INT64_MAX).pair_mt != 0 ? 1 : 0;
}

int b2_w4a16_silu_mul_pairs(const void* y_pairs, int64_t ld_in, void* out, int64_t ld_out, int64_t m, int64_t n,
                            void* stream) {
    if (m < 0 || n <= 0 || n % 16 != 0) return fail(B2_ERR_ARGUMENT, "m >= 0 and n a positive multiple of 16 expected");
    if (m == 0) return B2_OK;
    if (!y_pairs || !out) return fail(B2_ERR_ARGUMENT, "null pointer");
    if (ld_in < n || ld_out < n / 2) return fail(B2_ERR_ARGUMENT, "leading dimension smaller than the row length");
    if (m > INT_MAX || m * n > INT_MAX) return fail(B2_ERR_RANGE, "W4A16 dimensions exceed the kernel index range");
    const int64_t total = m * (n / 2);
    const unsigned blocks = unsigned(std::min<int64_t>((total + 255) / 256, 148 * 8));
    silu_mul_pairs_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(y_pairs), ld_in, static_cast<__half*>(out), ld_out, int(m), int(n / 2));
    return after_launch("silu_mul_pairs_kernel");
}

int b2_w4a16_linear_route(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy,
                          int64_t m, int64_t n, int64_t k, void* workspace, int64_t workspace_bytes,
                          void* stream, int route) {
    return b2_w4a16_linear_bias(x, ldx, native, nullptr, y, ldy, m, n, k, workspace, workspace_bytes, stream, route);
}

int b2_w4a16_linear_static(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy,
                           int64_t m, int64_t n, int64_t k, void* stream) {
    if (m < 0) return fail(B2_ERR_ARGUMENT, "m must be non-negative");
    if (int rc = check_dims(n, k)) return rc;
    if (m > B2_STREAM_MAX_M)
        return fail(B2_ERR_RANGE, "b2_w4a16_linear_static takes at most 64 rows of x per call");
    if (m == 0) return B2_OK;
    DeviceInfo dev;
    if (int rc = device_info(dev)) return rc;
    const b2::Dims d = b2::make_dims(n, k);
    const int64_t need = stream_workspace_bytes(m, d, dev.sm_count);
    if (need > B2_W4A16_STATIC_SCRATCH_BYTES)
        return fail(B2_ERR_RANGE, "this problem needs " + std::to_string(need) +
                    " bytes of scratch; the built-in scratch of b2_w4a16_linear_static holds " +
                    std::to_string(B2_W4A16_STATIC_SCRATCH_BYTES) + " (use b2_w4a16_linear with a workspace)");
    void* scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    // The array keeps whatever the previous call left; the tickets must start at zero.  The last word
    // of the ticket area is the sticky status word, which survives (b2_w4a16_status(NULL, ...) reads it).
    const cudaError_t e = cudaMemsetAsync(scratch, 0, B2_W4A16_TICKET_BYTES - 4, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail("cudaMemsetAsync", e);
    return b2_w4a16_linear_route(x, ldx, native, y, ldy, m, n, k, scratch, B2_W4A16_STATIC_SCRATCH_BYTES, stream,
                                 B2_ROUTE_STREAM);
}

int64_t b2_w4a16_gather_block_bytes(int world, int64_t mailbox_slice_bytes) {
    if (world < 1 || world > b2::kGatherMaxRanks || mailbox_slice_bytes < 0) return 0;
    // flag words + [2 parities][world senders][one 8-byte packet per 4-byte word of a slice]
    return b2::kGatherMailboxOffset + 2 * int64_t(world) * (mailbox_slice_bytes / 4) * 8;
}

int b2_w4a16_gather(void* const* y_ranks, void* const* flag_blocks, int64_t mailbox_slice_bytes, int rank, int world,
                    int64_t m, int64_t ld, int64_t n_total, int64_t slice_cols, void* stream) {
    GatherCall c;
    if (int rc = make_gather_call(y_ranks, flag_blocks, mailbox_slice_bytes, rank, world, m, ld, n_total, slice_cols, c)) return rc;
    const b2::GatherArgs& a = c.a;
    DeviceInfo dev;
    if (int rc = device_info(dev)) return rc;
    const int sms = dev.sm_count > 0 ? dev.sm_count : 148;
    // Small slices (every rank's fits in a mailbox half): packets polled by the receiver, one NVLink crossing.
    if (c.mailbox) {
        const int64_t items = m * (slice_cols / 2) * (world - 1);
        const unsigned grid = unsigned(std::max<int64_t>(1, std::min<int64_t>((items + 255) / 256, 2LL * sms)));
        b2::gather_mailbox_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
        return after_launch("gather_mailbox_kernel");
    }
    const int64_t items = m * (c.vec ? a.cols / 8 : a.cols) * (world - 1);
    const int64_t want = (items + 255) / 256;
    const unsigned grid = unsigned(std::max<int64_t>(1, std::min<int64_t>(want, 2LL * sms)));
    if (c.vec) b2::gather_push_wait_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    else b2::gather_push_wait_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return after_launch("gather_push_wait_kernel");
}

int b2_w4a16_linear_gather(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* const* y_ranks,
                           void* const* flag_blocks, int64_t mailbox_slice_bytes, int rank, int world, int64_t m,
                           int64_t ld, int64_t n_total, int64_t slice_cols, int64_t k, void* workspace,
                           int64_t workspace_bytes, void* stream, int flags) {
    if (flags & ~(B2_FLAG_FP16_STEPS | B2_FLAG_OVERLAP_LAUNCH)) return fail(B2_ERR_ARGUMENT, "unknown flag");
    GatherCall c;
    if (int rc = make_gather_call(y_ranks, flag_blocks, mailbox_slice_bytes, rank, world, m, ld, n_total, slice_cols, c)) return rc;
    if (m == 0) return B2_OK;
    const int64_t cols = c.a.cols;
    if (cols > 0) {
        void* y_local = static_cast<__half*>(y_ranks[rank]) + c.a.col0;
        int rc = kNotFused;
        if (c.mailbox && m <= 16) rc = linear_impl(x, ldx, native, bias_fp16, y_local, ld, m, cols, k, workspace, workspace_bytes,
                                                   stream, B2_ROUTE_AUTO, 0, flags, &c.a);
        if (rc != kNotFused) return rc;
        rc = linear_impl(x, ldx, native, bias_fp16, y_local, ld, m, cols, k, workspace, workspace_bytes, stream,
                         B2_ROUTE_AUTO, 0, flags);
        if (rc != B2_OK) return rc;
    }
    return b2_w4a16_gather(y_ranks, flag_blocks, mailbox_slice_bytes, rank, world, m, ld, n_total, slice_cols, stream);
}

int b2_w4a16_linear_gather_launches(int64_t m, int64_t n_total, int64_t slice_cols, int64_t k, int rank, int world,
                                    int64_t mailbox_slice_bytes) {
    if (m <= 0 || world < 1 || rank < 0 || rank >= world || slice_cols <= 0) return 0;
    const int64_t col0 = std::min(n_total, int64_t(rank) * slice_cols);
    const int64_t cols = std::min(slice_cols, n_total - col0);
    if (cols <= 0) return 1;                                   // nothing to compute: the gather alone
    if (check_dims(cols, k) != B2_OK) return 0;
    const bool mailbox = slice_cols % 2 == 0 && n_total % 2 == 0 && world > 1 && m * slice_cols * 2 <= mailbox_slice_bytes;
    if (!mailbox || m > 16 || k % 8 != 0) return 2;
    DeviceInfo dev;
    if (device_info(dev) != B2_OK) dev.sm_count = 148;
    const b2::Dims d = b2::make_dims(cols, k);
    const int split = tile_ksplit(d, dev.sm_count, pair_available());
    if (tile_applicable(m, d, split)) return tile_gather_pays(m, d, split, world, slice_cols) ? 1 : 2;
    const StreamPlan p = plan_stream(m, d, dev.sm_count);
    return (p.warps == 16 || p.warps == 4) && p.nchunks <= 1 ? 1 : 2;
}

int b2_w4a16_gather_status(const void* flag_block, void* stream, unsigned* status_host) {
    if (!flag_block || !status_host) return fail(B2_ERR_ARGUMENT, "null pointer");
    cudaError_t e = cudaMemcpyAsync(status_host, static_cast<const unsigned*>(flag_block) + b2::kGatherStatusWord,
                                    sizeof(unsigned), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail("b2_w4a16_gather_status", e);
    return B2_OK;
}

int b2_w4a16_noop(void* stream) {
    noop_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>();
    return after_launch("noop_kernel");
}

int b2_w4a16_linear(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy, int64_t m,
                    int64_t n, int64_t k, void* workspace, int64_t workspace_bytes, void* stream) {
    return b2_w4a16_linear_route(x, ldx, native, y, ldy, m, n, k, workspace, workspace_bytes, stream,
                                 B2_ROUTE_AUTO);
}

}  // extern "C"
