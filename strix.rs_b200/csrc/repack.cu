// Upload-time repack of raw GGUF blocks into the row-planar resident layout, and
// the inverse check path: dequantise a resident weight to f32.
//
// Replaces the host-side scalar split loops of the reference's upload_q4_0 /
// upload_q8_0 / upload_q6_k (crates/strix-backend-rocm/src/decode.rs:2491-2521,
// 2683-2714, 2629-2681): the raw bytes go to the device once and a kernel does
// the split, so upload cost is one H2D copy plus one pass at memory speed.
#include "common.cuh"
#include "kernels.h"
#include "layout.h"

namespace strix {

// One thread per 32-element block (Q4_0 / Q8_0).
template <int FMT>
__global__ void repack_q4q8_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ res, RowLayout L,
                                   uint32_t rows) {
    constexpr uint32_t BB = gguf_block_bytes(FMT);
    constexpr uint32_t QB = BB - 2;  // quant bytes per block
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t total = (uint64_t)rows * L.nb;
    if (idx >= total) return;
    uint32_t row = (uint32_t)(idx / L.nb), b = (uint32_t)(idx % L.nb);
    const uint8_t *src = raw + idx * BB;
    uint8_t *rowp = res + (uint64_t)row * L.row_stride;
    uint16_t d = (uint16_t)(src[0] | (src[1] << 8));
    *reinterpret_cast<uint16_t *>(rowp + L.off_d + 2 * b) = d;
    uint32_t w[QB / 4];
#pragma unroll
    for (uint32_t i = 0; i < QB / 4; i++) {
        const uint8_t *p = src + 2 + 4 * i;
        w[i] = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
        // Q8_0 codes are kept as q + 128 (unsigned bytes): the GEMV turns a byte into a float by
        // dropping it into a mantissa, which wants an unsigned value
        if (FMT == FMT_Q8_0) w[i] ^= 0x80808080u;
    }
    uint4 *dst = reinterpret_cast<uint4 *>(rowp + (uint64_t)b * QB);
#pragma unroll
    for (uint32_t i = 0; i < QB / 16; i++) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    // zero the row's padding once (block 0's thread)
    if (b == 0) {
        for (uint32_t o = L.off_d + 2 * L.nb; o < L.row_stride; o++) rowp[o] = 0;
    }
}

// Q6_K: one thread per (super-block, 16-byte piece); 13 pieces = 8 ql + 4 qh + 1 sc (+ d).
__global__ void repack_q6k_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ res, RowLayout L,
                                  uint32_t rows) {
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t total = (uint64_t)rows * L.nb * 13;
    if (idx >= total) return;
    uint32_t piece = (uint32_t)(idx % 13);
    uint64_t sbi = idx / 13;
    uint32_t row = (uint32_t)(sbi / L.nb), sb = (uint32_t)(sbi % L.nb);
    const uint8_t *src = raw + sbi * 210;
    uint8_t *rowp = res + (uint64_t)row * L.row_stride;
    uint32_t soff, doff;
    if (piece < 8) {
        soff = piece * 16;
        doff = sb * 128 + piece * 16;
    } else if (piece < 12) {
        soff = 128 + (piece - 8) * 16;
        doff = L.off_qh + sb * 64 + (piece - 8) * 16;
    } else {
        soff = 192;
        doff = L.off_sc + sb * 16;
        *reinterpret_cast<uint16_t *>(rowp + L.off_d + 2 * sb) = (uint16_t)(src[208] | (src[209] << 8));
        if (sb == 0) {
            for (uint32_t o = L.off_d + 2 * L.nb; o < L.row_stride; o++) rowp[o] = 0;
        }
    }
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint8_t *p = src + soff + 4 * i;
        w[i] = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    }
    *reinterpret_cast<uint4 *>(rowp + doff) = make_uint4(w[0], w[1], w[2], w[3]);
}

cudaError_t launch_repack(int fmt, const uint8_t *d_raw, uint8_t *d_res, const RowLayout &L, uint32_t rows,
                          cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const int T = 256;
    if (fmt == FMT_Q6_K) {
        uint64_t total = (uint64_t)rows * L.nb * 13;
        repack_q6k_kernel<<<(unsigned)((total + T - 1) / T), T, 0, stream>>>(d_raw, d_res, L, rows);
    } else {
        uint64_t total = (uint64_t)rows * L.nb;
        unsigned g = (unsigned)((total + T - 1) / T);
        if (fmt == FMT_Q4_0)
            repack_q4q8_kernel<FMT_Q4_0><<<g, T, 0, stream>>>(d_raw, d_res, L, rows);
        else
            repack_q4q8_kernel<FMT_Q8_0><<<g, T, 0, stream>>>(d_raw, d_res, L, rows);
    }
    return cudaGetLastError();
}

// Dequantise a resident weight to f32 [rows][in_dim]; one thread per 16 consecutive
// elements. Every product is a single rounded multiply (__fmul_rn), in the operand
// order of the reference's dequant_q4_0 / _q8_0 / _q6_k
// (crates/strix-models/src/ggml_quant.rs:240-262, 404-430).
__global__ void dequant_kernel(const uint8_t *__restrict__ res, float *__restrict__ out, RowLayout L,
                               uint32_t rows) {
    uint32_t upr = L.in_dim / 16;
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)rows * upr) return;
    uint32_t row = (uint32_t)(idx / upr), u = (uint32_t)(idx % upr);
    const uint8_t *rowp = res + (uint64_t)row * L.row_stride;
    float *o = out + (uint64_t)row * L.in_dim + (uint64_t)u * 16;
    if (L.fmt == FMT_Q8_0) {
        uint32_t b = u >> 1;
        float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(rowp + L.off_d + 2 * b));
        const uint8_t *q = rowp + (uint64_t)u * 16;  // resident codes are q + 128
        for (int i = 0; i < 16; i++) o[i] = __fmul_rn(d, (float)((int)q[i] - 128));
    } else if (L.fmt == FMT_Q4_0) {
        // elements 16u .. 16u+15 of block b: low nibbles (u even) or high nibbles (u odd) of bytes 0..15
        uint32_t b = u >> 1, hi = u & 1;
        float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(rowp + L.off_d + 2 * b));
        const uint8_t *qs = rowp + (uint64_t)b * 16;
        for (int j = 0; j < 16; j++) {
            int q = hi ? (qs[j] >> 4) : (qs[j] & 0x0F);
            o[j] = __fmul_rn(d, (float)(q - 8));
        }
    } else {
        // Q6_K: elements 16u..16u+15 = super-block sb, 16-element group g
        uint32_t sb = u >> 4, g = u & 15;
        uint32_t half = g >> 3, gg = g & 7, quarter = gg >> 1, l0 = (gg & 1) * 16;
        const uint8_t *ql = rowp + (uint64_t)sb * 128 + half * 64;
        const uint8_t *qh = rowp + L.off_qh + (uint64_t)sb * 64 + half * 32;
        const int8_t *sc = reinterpret_cast<const int8_t *>(rowp + L.off_sc + (uint64_t)sb * 16 + half * 8);
        float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(rowp + L.off_d + 2 * sb));
        float dsc = __fmul_rn(d, (float)sc[(l0 >> 4) + 2 * quarter]);
        for (uint32_t j = 0; j < 16; j++) {
            uint32_t l = l0 + j;
            int q;
            if (quarter == 0) q = (ql[l] & 0x0F) | ((qh[l] & 3) << 4);
            else if (quarter == 1) q = (ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4);
            else if (quarter == 2) q = (ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4);
            else q = (ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4);
            o[j] = __fmul_rn(dsc, (float)(q - 32));
        }
    }
}

cudaError_t launch_dequant(const uint8_t *d_res, float *d_out, const RowLayout &L, uint32_t rows,
                           cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    uint64_t total = (uint64_t)rows * (L.in_dim / 16);
    const int T = 256;
    dequant_kernel<<<(unsigned)((total + T - 1) / T), T, 0, stream>>>(d_res, d_out, L, rows);
    return cudaGetLastError();
}

}  // namespace strix
