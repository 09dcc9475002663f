// Resident ("tile-major") weight layout shared by host and device code.
//
// GGUF stores a weight as [out_dim][in_dim/blk] blocks of 18 / 34 / 210 bytes, none of which is
// 16-byte aligned, and a row at a time. The GEMV feeds the tensor cores 16 rows x 32 weights per
// instruction, so on upload the blocks are regrouped into TILES of 16 consecutive rows x one
// block's worth of K, stored in the order the instruction's operand registers want them:
//
//   weight  = [row group of 16 rows][tile along K]            (tiles of a group are contiguous,
//                                                              groups follow one another)
//   Q8_0 tile, 544 B  (16 rows x 32 codes):
//       4 x 128 B "cores" (8 rows x 16 codes, row-major, 16 B per row):
//           core 0 = rows 0-7, k 0-15 | core 1 = rows 0-7, k 16-31 | core 2 = rows 8-15, k 0-15 |
//           core 3 = rows 8-15, k 16-31;   codes stored as q + 128 (unsigned bytes)
//       16 x f16 scales, in pairs (row g, row g + 8), g = 0..7
//   Q4_0 tile, 288 B  (16 rows x 32 codes):
//       32 lanes x 8 B; lane 4g + t, byte 4h + i = code(row g, k) | code(row g + 8, k) << 4
//       with k = 16h + 4t + i  (g 0..7, t 0..3, h 0..1, i 0..3)
//       16 x f16 scales, in pairs (row g, row g + 8)
//   Q4_1 tile, 320 B: the Q4_0 tile (codes 0..15 with no centring: value = d * code + m) followed by
//       16 x f16 minimums m, in pairs (row g, row g + 8)
//   Q6_K tile, 3360 B (16 rows x one 256-weight super-block):
//       8 sub-tiles of 416 B (32 consecutive weights each):
//           32 lanes x 8 B low nibbles, 32 lanes x 4 B high bit pairs (see q6k_pack below),
//           8 x 4 sub-scales as value + 128: {row g: weights 0-15, 16-31; row g + 8: weights 0-15, 16-31}
//       16 x f16 super-block scales, in pairs (row g, row g + 8)
//
// A lane of a warp (g = lane / 4, t = lane % 4) then reads its 16 codes (rows g and g + 8, weights
// 4t..4t+3 and 16+4t..16+4t+3 of the tile) with conflict-free loads, and any run of tiles of a
// row group is ONE contiguous, 16-byte-aligned byte range for a bulk async copy. Rows past out_dim
// in the last group are zero (codes and scales). No scale is widened or folded and no code is
// re-quantised: a resident tile holds exactly the bytes of its 16 GGUF blocks, and
// dequantisation reproduces the reference bit for bit.
#pragma once
#include <stdint.h>

namespace strix {

enum Fmt : int { FMT_Q4_0 = 0, FMT_Q8_0 = 1, FMT_Q6_K = 2, FMT_Q4_1 = 3 };

// ggml type ids (crates/strix-models/src/ggml_quant.rs:568-574)
constexpr int GGML_Q4_0 = 2, GGML_Q4_1 = 3, GGML_Q8_0 = 8, GGML_Q6_K = 14;

constexpr uint32_t TILE_ROWS = 16;
constexpr uint32_t Q8_TILE = 544, Q4_TILE = 288, Q41_TILE = 320, Q6_SUB = 416, Q6_TILE = 8 * Q6_SUB + 32;

struct RowLayout {
    int fmt;
    uint32_t in_dim;       // K
    uint32_t nb;           // GGUF blocks per row (32-element blocks, or 256-element super-blocks for Q6_K)
    uint32_t tile_bytes;   // bytes of one tile (16 rows x one GGUF block of K)
    uint32_t group_bytes;  // bytes of one row group = nb * tile_bytes
};

inline
#ifdef __CUDACC__
    __host__ __device__
#endif
    RowLayout
    make_layout(int fmt, uint32_t in_dim) {
    RowLayout L{};
    L.fmt = fmt;
    L.in_dim = in_dim;
    L.nb = in_dim / (fmt == FMT_Q6_K ? 256u : 32u);
    L.tile_bytes = fmt == FMT_Q4_0 ? Q4_TILE : fmt == FMT_Q4_1 ? Q41_TILE : fmt == FMT_Q8_0 ? Q8_TILE : Q6_TILE;
    L.group_bytes = L.nb * L.tile_bytes;
    return L;
}

constexpr uint32_t gguf_block_bytes(int fmt) {
    return fmt == FMT_Q4_0 ? 18u : fmt == FMT_Q4_1 ? 20u : fmt == FMT_Q8_0 ? 34u : 210u;
}
constexpr uint32_t gguf_block_elems(int fmt) { return fmt == FMT_Q6_K ? 256u : 32u; }

inline
#ifdef __CUDACC__
    __host__ __device__
#endif
    uint64_t
    resident_bytes(const RowLayout &L, uint64_t rows) {
    return ((rows + TILE_ROWS - 1) / TILE_ROWS) * (uint64_t)L.group_bytes;
}

#ifdef __CUDACC__
// ---- element accessors (checks, scale transposition, dequantise-to-f32; not the hot path) ----
// Stored code of weight k of row `row`: Q8_0 q + 128, Q4_0 the nibble, Q6_K the 6-bit code.
__device__ inline uint32_t resident_code(const uint8_t *res, const RowLayout &L, uint32_t row, uint32_t k) {
    const uint8_t *grp = res + (uint64_t)(row / TILE_ROWS) * L.group_bytes;
    const uint32_t r = row % TILE_ROWS, g = r & 7u, rh = r >> 3;
    if (L.fmt == FMT_Q8_0) {
        const uint32_t kk = k & 31u;
        return grp[(k >> 5) * Q8_TILE + (rh * 2u + (kk >> 4)) * 128u + g * 16u + (kk & 15u)];
    }
    if (L.fmt == FMT_Q4_0 || L.fmt == FMT_Q4_1) {
        const uint32_t kk = k & 31u, h = kk >> 4, t = (kk & 15u) >> 2, i = kk & 3u;
        const uint32_t b = grp[(k >> 5) * L.tile_bytes + 8u * (4u * g + t) + 4u * h + i];
        return rh ? (b >> 4) : (b & 0x0Fu);
    }
    const uint32_t e = k & 255u, st = e >> 5, kk = e & 31u, h = kk >> 4, t = (kk & 15u) >> 2, i = kk & 3u;
    const uint8_t *sub = grp + (k >> 8) * Q6_TILE + st * Q6_SUB;
    const uint32_t lane = 4u * g + t, wq = 2u * h + rh;  // which of the lane's four byte-quads
    const uint32_t lob = sub[8u * lane + 4u * h + i], hib = sub[256u + 4u * lane + i];
    return ((rh ? (lob >> 4) : lob) & 0x0Fu) | (((hib >> (2u * wq)) & 3u) << 4);
}
// f16 bits of the scale of GGUF block `blk` (32 weights; a 256-weight super-block for Q6_K) of a row.
__device__ inline uint16_t resident_scale_bits(const uint8_t *res, const RowLayout &L, uint32_t row, uint32_t blk) {
    const uint8_t *tile = res + (uint64_t)(row / TILE_ROWS) * L.group_bytes + (uint64_t)blk * L.tile_bytes;
    const uint32_t off = L.fmt == FMT_Q8_0 ? 512u : L.fmt == FMT_Q6_K ? 8u * Q6_SUB : 256u;
    const uint32_t r = row % TILE_ROWS;
    return *reinterpret_cast<const uint16_t *>(tile + off + 4u * (r & 7u) + 2u * (r >> 3));
}
// Q4_1: f16 bits of the minimum m of GGUF block `blk` of a row.
__device__ inline uint16_t resident_min_bits(const uint8_t *res, const RowLayout &L, uint32_t row, uint32_t blk) {
    const uint8_t *tile = res + (uint64_t)(row / TILE_ROWS) * L.group_bytes + (uint64_t)blk * L.tile_bytes;
    const uint32_t r = row % TILE_ROWS;
    return *reinterpret_cast<const uint16_t *>(tile + 288u + 4u * (r & 7u) + 2u * (r >> 3));
}
// Q6_K: int8 sub-scale of 16-weight group `grp16` (0 .. in_dim/16 - 1) of a row.
__device__ inline int resident_q6k_subscale(const uint8_t *res, const RowLayout &L, uint32_t row, uint32_t grp16) {
    const uint8_t *tile = res + (uint64_t)(row / TILE_ROWS) * L.group_bytes + (uint64_t)(grp16 >> 4) * L.tile_bytes;
    const uint32_t st = (grp16 >> 1) & 7u;
    const uint32_t r = row % TILE_ROWS;
    return (int)tile[st * Q6_SUB + 384u + 4u * (r & 7u) + 2u * (r >> 3) + (grp16 & 1u)] - 128;
}
#endif

}  // namespace strix
