// All-gather of column slices over NVLink with plain peer stores (multi-GPU form of the operator).
//
// Every rank owns the columns [col0, col0 + cols) of an [M, N] FP16 output and has already written
// them into its OWN copy of the full buffer (the projection kernels store straight into that
// slice).  This kernel pushes the slice into the same place of every peer's buffer with ordinary
// st.global through peer-mapped pointers - 16-byte stores, coalesced along a row - and then runs a
// flag exchange: the last CTA to finish publishes this call's epoch number in every peer's flag
// block (st.release.sys after a system-wide fence) and waits until every peer's epoch has arrived
// in its own block.  When the kernel ends, the local buffer holds all slices.
//
// Nothing here reads another GPU's memory, no TMA or bulk copy touches a peer, nothing is
// multicast.  The wait is bounded: after `wait_ns` nanoseconds the kernel records bit 2 in the flag
// block's status word and returns, so a rank whose peer never arrives (it crashed, or was never
// launched) gets an error status instead of a hung GPU.
//
// Small slices take a second form, gather_mailbox_kernel: latency is all that matters there, and the
// fence / ticket / flag chain above costs ~13 us.  Every 4-byte word of the slice travels as an 8-byte
// packet {word, epoch} (one single-copy-atomic store) into a mailbox behind the peer's flag block; the
// receiving rank polls the packets themselves and copies the words into its buffer as they arrive.  No
// fence, no flag round trip: one NVLink crossing per gather.  The mailbox has two halves used in turn
// (epoch parity), so a peer that is one call ahead never overwrites packets that are still being read.
//
// Flag block (one per rank, in memory every peer can write): 32 unsigned words
//   [0..15] arrive[q]  epoch of the last call whose slice from rank q has landed here (written by q)
//   [16]    epoch      number of calls this rank has completed (local)
//   [17]    ticket     CTA arrival counter of the running call (local, zero between calls)
//   [18]    status     sticky error bits (local): bit 2 = a peer's epoch did not arrive in time
// Epochs only grow, so one flag block serves every gathered layer of a process as long as all ranks
// issue the same sequence of gathers.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace b2 {

constexpr int kGatherMaxRanks = 16;
constexpr int kGatherEpochWord = 16, kGatherTicketWord = 17, kGatherStatusWord = 18;
constexpr unsigned kStatusPeerTimeout = 4u;

struct GatherArgs {
    __half* y[kGatherMaxRanks];         // every rank's [M, ld] buffer as mapped into this process; y[rank] is local
    unsigned* flags[kGatherMaxRanks];   // every rank's flag block
    int rank, world;
    int m;
    int64_t ld, col0, cols;
    long long wait_ns;                  // how long the wait for the peers' flags may last before it gives up
    // mailbox form: rank q owns columns [q * slice_cols, min(n_total, (q + 1) * slice_cols))
    int64_t n_total, slice_cols;
    int64_t slots;                      // 8-byte packets per (parity, sender) in every rank's mailbox
};
constexpr int kGatherMailboxOffset = 128;          // bytes from the flag block to its mailbox

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <bool VEC>
__global__ void __launch_bounds__(256)
gather_push_wait_kernel(const GatherArgs a) {
    __shared__ int is_last;
    const __half* src = a.y[a.rank];
    const int peers = a.world - 1;
    if (VEC) {
        const int64_t pieces = a.cols >> 3;                      // 16-byte pieces per row
        const int64_t per_peer = int64_t(a.m) * pieces;
        const int64_t total = per_peer * peers;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
            const int pi = int(i / per_peer);
            const int64_t r = i - pi * per_peer;
            const int64_t row = r / pieces, piece = r - row * pieces;
            const int64_t at = row * a.ld + a.col0 + piece * 8;
            const uint4 v = *reinterpret_cast<const uint4*>(src + at);
            *reinterpret_cast<uint4*>(a.y[pi < a.rank ? pi : pi + 1] + at) = v;
        }
    } else {
        const int64_t per_peer = int64_t(a.m) * a.cols;
        const int64_t total = per_peer * peers;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
            const int pi = int(i / per_peer);
            const int64_t r = i - pi * per_peer;
            const int64_t row = r / a.cols, col = r - row * a.cols;
            const int64_t at = row * a.ld + a.col0 + col;
            a.y[pi < a.rank ? pi : pi + 1][at] = src[at];
        }
    }
    unsigned* mine = a.flags[a.rank];
    __threadfence_system();                                      // this thread's peer stores before the ticket
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(mine + kGatherTicketWord, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence_system();
    const unsigned epoch = mine[kGatherEpochWord] + 1u;
    if (threadIdx.x < a.world && int(threadIdx.x) != a.rank) {
        const int q = threadIdx.x;
        st_release_sys(a.flags[q] + a.rank, epoch);              // my slice has landed in q's buffer
        // Bounded by the clock and by a poll count: the first polls come back to back (a flag that is a
        // microsecond away should not cost a sleep), later ones sleep 100 ns each, so the count alone ends
        // the loop even if the timer stood still.
        const unsigned long long t0 = global_ns();
        bool arrived = false;
        for (long long i = 0; i < a.wait_ns / 64 + 4096 && !arrived; ++i) {
            arrived = int(ld_acquire_sys(mine + q) - epoch) >= 0;
            if (arrived) break;
            if (i >= 4096) {
                if (global_ns() - t0 > (unsigned long long)a.wait_ns) break;
                __nanosleep(100);
            }
        }
        if (!arrived) atomicOr(mine + kGatherStatusWord, kStatusPeerTimeout);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mine[kGatherEpochWord] = epoch;
        mine[kGatherTicketWord] = 0u;
    }
}

// Mailbox of rank r: [2 parities][world senders][slots] packets of {data word, epoch}.
__device__ __forceinline__ uint2* mailbox(unsigned* flag_block, int world, int64_t slots, unsigned parity, int sender) {
    return reinterpret_cast<uint2*>(reinterpret_cast<unsigned char*>(flag_block) + kGatherMailboxOffset) +
           (int64_t(parity) * world + sender) * slots;
}

// One packet: the data word and the epoch of the call it belongs to, in one single-copy-atomic 8-byte store.
__device__ __forceinline__ void mailbox_send(uint2* slot, unsigned data, unsigned epoch) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(slot), "r"(data), "r"(epoch) : "memory");
}

// Receiving half of the mailbox form: thread `first` of `stride` polls its share of the packets of every
// peer's slice (bounded by the clock and by a poll count) and copies the words into the local buffer.
// Returns true when a packet did not arrive in time.
__device__ __forceinline__ bool mailbox_receive(const GatherArgs& a, unsigned epoch, int64_t first, int64_t stride) {
    unsigned* mine = a.flags[a.rank];
    __half* y = a.y[a.rank];
    const unsigned parity = epoch & 1u;
    bool gave_up = false;
    // One index space over all peers (a full slice has `full` words; the last rank's may be shorter), so that a
    // thread's packets from different peers are requested together: four loads in flight per thread, one trip
    // to L2 for the common case instead of one per peer.
    const int64_t full = int64_t(a.m) * (a.slice_cols >> 1);
    const int64_t total = full * (a.world - 1);
    for (int64_t i0 = first; i0 < total; i0 += 4 * stride) {
        unsigned data[4], tag[4];
        const uint2* slot[4];
        unsigned* dst[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t i = i0 + j * stride;
            slot[j] = nullptr;
            dst[j] = nullptr;
            data[j] = 0;
            tag[j] = epoch;
            if (i >= total) continue;
            const int pi = int(i / full);
            const int q = pi < a.rank ? pi : pi + 1;
            const int64_t s = i - pi * full;
            const int64_t col0 = int64_t(q) * a.slice_cols;
            const int64_t wpr = max(int64_t(0), min(a.slice_cols, a.n_total - col0)) >> 1;
            if (s >= int64_t(a.m) * wpr) continue;                         // beyond a short last slice
            const int64_t row = s / wpr, w = s - row * wpr;
            slot[j] = mailbox(mine, a.world, a.slots, parity, q) + s;
            dst[j] = reinterpret_cast<unsigned*>(y + row * a.ld + col0 + 2 * w);
            asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(data[j]), "=r"(tag[j]) : "l"(slot[j]) : "memory");
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (!slot[j]) continue;
            unsigned long long t0 = 0;
            for (long long n = 0; tag[j] != epoch && !gave_up && n < a.wait_ns / 64 + 4096; ++n) {   // bounded by the clock and by the count
                if (n == 4096) t0 = global_ns();
                if (n > 4096) {
                    if (global_ns() - t0 > (unsigned long long)a.wait_ns) { gave_up = true; break; }
                    __nanosleep(100);
                }
                asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(data[j]), "=r"(tag[j]) : "l"(slot[j]) : "memory");
            }
            if (tag[j] != epoch) { gave_up = true; continue; }
            *dst[j] = data[j];
        }
    }
    return gave_up;
}

// End of a mailbox call (every thread of every CTA calls it): record a timeout, count the CTA, and let the
// last CTA of the grid publish the new epoch and re-zero the ticket.
__device__ __forceinline__ void mailbox_finish(const GatherArgs& a, unsigned epoch, bool gave_up) {
    unsigned* mine = a.flags[a.rank];
    if (gave_up) atomicOr(mine + kGatherStatusWord, kStatusPeerTimeout);
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(mine + kGatherTicketWord, 1u) == gridDim.x - 1) {
        mine[kGatherEpochWord] = epoch;
        mine[kGatherTicketWord] = 0u;
    }
}

// The epoch of the running call.  Any thread may read it at any time before its CTA has counted itself in
// mailbox_finish: the word changes only after the last CTA of the grid has done so.
__device__ __forceinline__ unsigned mailbox_epoch(const GatherArgs& a) {
    return *reinterpret_cast<volatile unsigned*>(a.flags[a.rank] + kGatherEpochWord) + 1u;
}

__global__ void __launch_bounds__(256)
gather_mailbox_kernel(const GatherArgs a) {
    const unsigned epoch = mailbox_epoch(a);
    const unsigned parity = epoch & 1u;
    const __half* y = a.y[a.rank];
    const int64_t stride = int64_t(gridDim.x) * blockDim.x, first = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    // ---- send: every word of my slice to every peer's mailbox --------------------------------------
    {
        const int64_t wpr = a.cols >> 1;                                  // 4-byte words per row of my slice
        const int64_t words = int64_t(a.m) * wpr;
        const int peers = a.world - 1;
        for (int64_t i = first; i < words * peers; i += stride) {
            const int pi = int(i / words);
            const int64_t s = i - pi * words;
            const int64_t row = s / wpr, w = s - row * wpr;
            const unsigned data = *reinterpret_cast<const unsigned*>(y + row * a.ld + a.col0 + 2 * w);
            mailbox_send(mailbox(a.flags[pi < a.rank ? pi : pi + 1], a.world, a.slots, parity, a.rank) + s, data, epoch);
        }
    }
    // ---- receive: poll the packets of every peer's slice and copy the words into my buffer ---------
    mailbox_finish(a, epoch, mailbox_receive(a, epoch, first, stride));
}

}  // namespace b2
