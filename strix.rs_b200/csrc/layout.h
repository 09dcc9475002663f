// Resident ("row-planar") weight layout shared by host and device code.
//
// GGUF stores a weight as [out_dim][in_dim/blk] blocks of 18 / 34 / 210 bytes,
// none of which is 16-byte aligned. On upload every row is split into planes so
// that each plane starts on a 16-byte boundary and one whole row (or a tile of
// consecutive rows) is ONE contiguous, 16-byte-aligned byte range that a single
// bulk async copy can move into shared memory:
//
//   Q4_0 row: [ qs : nb x 16 B ][ d : nb x f16 ]                      pad to 16
//   Q8_0 row: [ qs : nb x 32 B ][ d : nb x f16 ]                      pad to 16
//   Q6_K row: [ ql : nb x 128 B ][ qh : nb x 64 B ][ sc : nb x 16 B ][ d : nb x f16 ]  pad to 16
//
// Bytes inside a plane keep their GGUF order; Q8_0 codes are stored as q + 128 (the byte with
// its top bit flipped). No scale is widened or folded, so
// a resident row is the GGUF row's size rounded up to 16 (Q4_0: exact when nb is
// a multiple of 8), and dequantisation reproduces the reference bit for bit.
#pragma once
#include <stdint.h>

namespace strix {

enum Fmt : int { FMT_Q4_0 = 0, FMT_Q8_0 = 1, FMT_Q6_K = 2 };

// ggml type ids (crates/strix-models/src/ggml_quant.rs:568-574)
constexpr int GGML_Q4_0 = 2, GGML_Q8_0 = 8, GGML_Q6_K = 14;

struct RowLayout {
    int fmt;
    uint32_t in_dim;      // K
    uint32_t nb;          // blocks per row (32-element blocks, or 256-element super-blocks for Q6_K)
    uint32_t row_stride;  // bytes per resident row, multiple of 16
    uint32_t off_qh;      // Q6_K: byte offset of the qh plane within a row
    uint32_t off_sc;      // Q6_K: byte offset of the sub-scale plane
    uint32_t off_d;       // byte offset of the f16 scale plane
};

constexpr uint32_t align16(uint32_t v) { return (v + 15u) & ~15u; }

inline
#ifdef __CUDACC__
    __host__ __device__
#endif
    RowLayout
    make_layout(int fmt, uint32_t in_dim) {
    RowLayout L{};
    L.fmt = fmt;
    L.in_dim = in_dim;
    if (fmt == FMT_Q4_0) {
        L.nb = in_dim / 32;
        L.off_d = L.nb * 16;
        L.row_stride = align16(L.nb * 18);
    } else if (fmt == FMT_Q8_0) {
        L.nb = in_dim / 32;
        L.off_d = L.nb * 32;
        L.row_stride = align16(L.nb * 34);
    } else {
        L.nb = in_dim / 256;
        L.off_qh = L.nb * 128;
        L.off_sc = L.nb * 192;
        L.off_d = L.nb * 208;
        L.row_stride = align16(L.nb * 210);
    }
    return L;
}

constexpr uint32_t gguf_block_bytes(int fmt) { return fmt == FMT_Q4_0 ? 18u : fmt == FMT_Q8_0 ? 34u : 210u; }
constexpr uint32_t gguf_block_elems(int fmt) { return fmt == FMT_Q6_K ? 256u : 32u; }

}  // namespace strix
