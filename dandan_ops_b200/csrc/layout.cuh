// Device-native weight image shared by every kernel of the engine.
//
// The [N, K] layer is cut into blocks of 16 output rows x 256 input columns (four
// quantization groups per row).  Block (kb, nt) - kb = column block, nt = row tile -
// starts at byte ((kb * N16) + nt) * 2336, N16 = ceil(N/16): row tiles of one column
// block are adjacent, so eight warps working on eight neighbouring row tiles read one
// contiguous 18.7 KB span per step.
//
// Inside a block (offsets in bytes):
//   [   0, 2048)  512 code words.  Word index = j*128 + lane*4 + i with lane = 4*g + t:
//                 row   = g + 8*(j>>1)          (g = 0..7)
//                 group = t                      (t = 0..3, columns 64t .. 64t+63)
//                 word  = 4*(j&1) + i            (eight columns 8*word .. 8*word+7 of the group)
//                 so a warp lane reads its 64 bytes as four 16-byte pieces that are
//                 contiguous across the warp (piece j of lane l at j*512 + l*16).
//                 Inside a word, column c of the eight sits in nibble (c>>1) + 4*(c&1):
//                 nibbles p and p+4 hold an (even, odd) column pair, which makes
//                 `(word >> 8e) & 0x000F000F` a pair of FP16 mantissas.
//   [2048, 2304)  64 FP32 steps: index lane*2 + h = step of (row g + 8h, group t).
//   [2304, 2336)  32 bytes of zero points: byte lane = zero(row g, group t) | zero(row g+8, group t) << 4.
//
// This is exactly what one lane of an m16n8k16 tensor-core fragment needs: lane (g, t)
// owns rows g and g+8 of the tile and, for the sixteen MMAs of a block, the columns
// 64t + 4i .. 64t + 4i + 3 (i = 0..15), i.e. one whole quantization group per row.
//
// Padding: rows >= N and groups >= ceil(K/64) get code 0, zero point 0, step 1; columns
// >= K inside a real group get code == zero point.  Either way the padded weight is
// exactly 0.0.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace b2 {

constexpr int kTileRows = 16;
constexpr int kBlockCols = 256;
constexpr int kGroup = 64;
constexpr int kBlockBytes = 2336;
constexpr int kCodeBytes = 2048;
constexpr int kStepOffset = 2048;
constexpr int kZeroOffset = 2304;

struct Dims {
    int n, k;          // layer shape
    int n16;           // row tiles   = ceil(n / 16)
    int kb;            // col blocks  = ceil(k / 256)
    int words;         // reference words per row  = ceil(k / 8)
    int groups;        // reference groups per row = ceil(k / 64)
};

__host__ __device__ inline Dims make_dims(int64_t n, int64_t k) {
    Dims d;
    d.n = int(n); d.k = int(k);
    d.n16 = int((n + 15) / 16);
    d.kb = int((k + 255) / 256);
    d.words = int((k + 7) / 8);
    d.groups = int((k + 63) / 64);
    return d;
}

__host__ __device__ inline int64_t native_bytes(const Dims& d) {
    return int64_t(d.n16) * d.kb * kBlockBytes;
}

// Nibble position of column c (0..7) inside a native word.
__host__ __device__ inline int nibble_slot(int c) { return (c >> 1) + 4 * (c & 1); }

// Reference word (nibble c = column c) -> native word, with columns >= valid replaced by `fill`.
__host__ __device__ inline uint32_t permute_word(uint32_t ref, int valid, uint32_t fill) {
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint32_t q = c < valid ? (ref >> (4 * c)) & 15u : fill;
        out |= q << (4 * nibble_slot(c));
    }
    return out;
}

// Native word -> reference word, columns >= valid cleared.
__host__ __device__ inline uint32_t unpermute_word(uint32_t nat, int valid) {
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c)
        if (c < valid) out |= ((nat >> (4 * nibble_slot(c))) & 15u) << (4 * c);
    return out;
}

// Location of (row, column-word) inside the image.
struct WordRef {
    int64_t block;   // byte offset of the block
    int word;        // index into the 512 code words
    int meta;        // lane*2 + h : index of the step; lane = meta>>1, h = meta&1
};

__host__ __device__ inline WordRef locate(const Dims& d, int row, int col_word) {
    const int k0 = col_word * 8;
    const int kb = k0 >> 8, t = (k0 >> 6) & 3, wi = (k0 >> 3) & 7;
    const int nt = row >> 4, r = row & 15, g = r & 7, h = r >> 3;
    const int lane = 4 * g + t, j = 2 * h + (wi >> 2), i = wi & 3;
    WordRef w;
    w.block = (int64_t(kb) * d.n16 + nt) * kBlockBytes;
    w.word = j * 128 + lane * 4 + i;
    w.meta = lane * 2 + h;
    return w;
}

}  // namespace b2
