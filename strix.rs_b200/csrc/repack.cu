// Upload-time repack of raw GGUF blocks into the tile-major resident layout, and
// the inverse check path: dequantise a resident weight to f32.
//
// Replaces the host-side scalar split loops of the reference's upload_q4_0 /
// upload_q8_0 / upload_q6_k (crates/strix-backend-rocm/src/decode.rs:2491-2521,
// 2683-2714, 2629-2681): the raw bytes go to the device once and a kernel does
// the regrouping, so upload cost is one H2D copy plus one pass at memory speed.
#include "common.cuh"
#include "kernels.h"
#include "layout.h"

namespace strix {

__device__ __forceinline__ uint32_t rd32(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

// One thread per (row group, tile, lane): it gathers the lane's 16 codes (rows g and g + 8,
// weights 4t..4t+3 and 16+4t..16+4t+3 of the block) from the raw rows of this chunk.
//   raw: GGUF rows [row0, row0 + n) of the shard; res: the whole resident shard; row0 % 16 == 0.
//   gemm_codes (Q8_0 only, may be null): [rows][in_dim] codes as q + 128, row-major, for the prefill GEMM.
template <int FMT>
__global__ void repack_q4q8_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ res,
                                   uint8_t *__restrict__ gemm_codes, RowLayout L, uint32_t row0, uint32_t n) {
    constexpr uint32_t BB = gguf_block_bytes(FMT);
    const uint32_t groups = (n + TILE_ROWS - 1) / TILE_ROWS;
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)groups * L.nb * 32u) return;
    const uint32_t lane = (uint32_t)(idx & 31u), g = lane >> 2, t = lane & 3u;
    const uint32_t kb = (uint32_t)((idx >> 5) % L.nb), rgl = (uint32_t)((idx >> 5) / L.nb);
    uint8_t *tile = res + (uint64_t)(row0 / TILE_ROWS + rgl) * L.group_bytes + (uint64_t)kb * L.tile_bytes;
    const uint32_t r_lo = rgl * TILE_ROWS + g, r_hi = r_lo + 8u;  // chunk-relative rows
    const uint8_t *b_lo = raw + ((uint64_t)r_lo * L.nb + kb) * BB, *b_hi = raw + ((uint64_t)r_hi * L.nb + kb) * BB;
    const bool v_lo = r_lo < n, v_hi = r_hi < n;
    if (FMT == FMT_Q8_0) {
        // codes are kept as q + 128 (unsigned bytes): the f16 path turns a byte into a float by
        // dropping it into a mantissa, which wants an unsigned value; rows past the end hold q = 0
#pragma unroll
        for (uint32_t kh = 0; kh < 2; kh++) {
            const uint32_t k = 16u * kh + 4u * t;
            const uint32_t w_lo = (v_lo ? rd32(b_lo + 2 + k) : 0u) ^ 0x80808080u;
            const uint32_t w_hi = (v_hi ? rd32(b_hi + 2 + k) : 0u) ^ 0x80808080u;
            *reinterpret_cast<uint32_t *>(tile + (0u + kh) * 128u + g * 16u + 4u * t) = w_lo;
            *reinterpret_cast<uint32_t *>(tile + (2u + kh) * 128u + g * 16u + 4u * t) = w_hi;
            if (gemm_codes) {
                if (v_lo) *reinterpret_cast<uint32_t *>(gemm_codes + (uint64_t)(row0 + r_lo) * L.in_dim + kb * 32u + k) = w_lo;
                if (v_hi) *reinterpret_cast<uint32_t *>(gemm_codes + (uint64_t)(row0 + r_hi) * L.in_dim + kb * 32u + k) = w_hi;
            }
        }
    } else {
        // byte 4h + i of the lane = code(row g, k) | code(row g + 8, k) << 4, k = 16h + 4t + i; GGUF keeps
        // weight k < 16 in the low nibble of byte k and weight k >= 16 in the high nibble of byte k - 16
#pragma unroll
        for (uint32_t h = 0; h < 2; h++) {
            // (rows past the end: Q4_0 code 8 is the value 0; Q4_1 code 0 with d = m = 0 is)
            constexpr uint32_t QO = FMT == FMT_Q4_1 ? 4u : 2u, PAD = FMT == FMT_Q4_1 ? 0u : 0x88888888u;
            const uint32_t q_lo = v_lo ? rd32(b_lo + QO + 4u * t) : PAD;
            const uint32_t q_hi = v_hi ? rd32(b_hi + QO + 4u * t) : PAD;
            const uint32_t n_lo = (h ? (q_lo >> 4) : q_lo) & 0x0F0F0F0Fu, n_hi = (h ? (q_hi >> 4) : q_hi) & 0x0F0F0F0Fu;
            *reinterpret_cast<uint32_t *>(tile + 8u * lane + 4u * h) = n_lo | (n_hi << 4);
        }
    }
    if (lane < TILE_ROWS) {
        const uint32_t r = rgl * TILE_ROWS + lane;
        const uint8_t *b = raw + ((uint64_t)r * L.nb + kb) * BB;
        const uint16_t d = r < n ? (uint16_t)(b[0] | (b[1] << 8)) : (uint16_t)0;
        // scales sit in pairs (row g, row g + 8), so that a lane reads both with one 32-bit load
        *reinterpret_cast<uint16_t *>(tile + (FMT == FMT_Q8_0 ? 512u : 256u) + 4u * (lane & 7u) + 2u * (lane >> 3)) = d;
        if (FMT == FMT_Q4_1) {
            const uint16_t m = r < n ? (uint16_t)(b[2] | (b[3] << 8)) : (uint16_t)0;
            *reinterpret_cast<uint16_t *>(tile + 288u + 4u * (lane & 7u) + 2u * (lane >> 3)) = m;
        }
    }
}

// GGUF Q6_K code (0..63) of element e (0..255) of a 210-byte super-block
// (element order of dequant_q6_k, crates/strix-models/src/ggml_quant.rs:404-430).
__device__ __forceinline__ uint32_t q6k_code(const uint8_t *blk, uint32_t e) {
    const uint32_t half = e >> 7, quarter = (e >> 5) & 3u, l = e & 31u;
    const uint32_t qlb = blk[half * 64u + l + (quarter & 1u) * 32u];
    const uint32_t lo = (quarter & 2u) ? (qlb >> 4) : (qlb & 0x0Fu);
    const uint32_t hi = (blk[128u + half * 32u + l] >> (2u * quarter)) & 3u;
    return lo | (hi << 4);
}

// Q6_K: one thread per (row group, super-block, sub-tile, lane). The lane's 16 codes form four
// byte-quads W0 (row g, weights 4t..4t+3), W1 (row g + 8, same), W2 (row g, 16+4t..), W3 (row g + 8),
// stored as  L0 = lo4(W0) | lo4(W1) << 4,  L1 = lo4(W2) | lo4(W3) << 4  (8 bytes of low nibbles)
// and  H = hi2(W0) | hi2(W1) << 2 | hi2(W2) << 4 | hi2(W3) << 6  (4 bytes of high bit pairs).
__global__ void repack_q6k_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ res, RowLayout L,
                                  uint32_t row0, uint32_t n) {
    const uint32_t groups = (n + TILE_ROWS - 1) / TILE_ROWS;
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)groups * L.nb * 256u) return;
    const uint32_t lane = (uint32_t)(idx & 31u), g = lane >> 2, t = lane & 3u, st = (uint32_t)((idx >> 5) & 7u);
    const uint32_t sb = (uint32_t)((idx >> 8) % L.nb), rgl = (uint32_t)((idx >> 8) / L.nb);
    uint8_t *tile = res + (uint64_t)(row0 / TILE_ROWS + rgl) * L.group_bytes + (uint64_t)sb * L.tile_bytes;
    uint8_t *sub = tile + st * Q6_SUB;
    const uint32_t r_lo = rgl * TILE_ROWS + g, r_hi = r_lo + 8u;
    const uint8_t *b_lo = raw + ((uint64_t)r_lo * L.nb + sb) * 210u, *b_hi = raw + ((uint64_t)r_hi * L.nb + sb) * 210u;
    uint32_t W[4] = {0, 0, 0, 0};
#pragma unroll
    for (uint32_t h = 0; h < 2; h++)
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            const uint32_t e = 32u * st + 16u * h + 4u * t + i;
            W[2 * h] |= (r_lo < n ? q6k_code(b_lo, e) : 32u) << (8u * i);
            W[2 * h + 1] |= (r_hi < n ? q6k_code(b_hi, e) : 32u) << (8u * i);
        }
    const uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x03030303u;
    *reinterpret_cast<uint32_t *>(sub + 8u * lane) = (W[0] & M4) | ((W[1] & M4) << 4);
    *reinterpret_cast<uint32_t *>(sub + 8u * lane + 4u) = (W[2] & M4) | ((W[3] & M4) << 4);
    *reinterpret_cast<uint32_t *>(sub + 256u + 4u * lane) =
        ((W[0] >> 4) & M2) | (((W[1] >> 4) & M2) << 2) | (((W[2] >> 4) & M2) << 4) | (((W[3] >> 4) & M2) << 6);
    if (lane < TILE_ROWS) {
        const uint32_t r = rgl * TILE_ROWS + lane;
        const uint8_t *b = raw + ((uint64_t)r * L.nb + sb) * 210u;
        const bool v = r < n;
        // sub-scales as value + 128, four per g: {row g: first, last 16 weights; row g + 8: first, last 16};
        // super-block scales in pairs (row g, row g + 8)
        const uint32_t so = 384u + 4u * (lane & 7u) + 2u * (lane >> 3);
        sub[so] = (uint8_t)((v ? b[192u + 2u * st] : 0) ^ 0x80);
        sub[so + 1u] = (uint8_t)((v ? b[192u + 2u * st + 1u] : 0) ^ 0x80);
        if (st == 0)
            *reinterpret_cast<uint16_t *>(tile + 8u * Q6_SUB + 4u * (lane & 7u) + 2u * (lane >> 3)) =
                v ? (uint16_t)(b[208] | (b[209] << 8)) : (uint16_t)0;
    }
}

cudaError_t launch_repack(int fmt, const uint8_t *d_raw, uint8_t *d_res, uint8_t *d_gemm_codes, const RowLayout &L,
                          uint32_t row0, uint32_t n, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const int T = 256;
    const uint64_t groups = (n + TILE_ROWS - 1) / TILE_ROWS;
    if (fmt == FMT_Q6_K) {
        const uint64_t total = groups * L.nb * 256u;
        repack_q6k_kernel<<<(unsigned)((total + T - 1) / T), T, 0, stream>>>(d_raw, d_res, L, row0, n);
    } else {
        const uint64_t total = groups * L.nb * 32u;
        const unsigned gr = (unsigned)((total + T - 1) / T);
        if (fmt == FMT_Q4_0)
            repack_q4q8_kernel<FMT_Q4_0><<<gr, T, 0, stream>>>(d_raw, d_res, nullptr, L, row0, n);
        else if (fmt == FMT_Q4_1)
            repack_q4q8_kernel<FMT_Q4_1><<<gr, T, 0, stream>>>(d_raw, d_res, nullptr, L, row0, n);
        else
            repack_q4q8_kernel<FMT_Q8_0><<<gr, T, 0, stream>>>(d_raw, d_res, d_gemm_codes, L, row0, n);
    }
    return cudaGetLastError();
}

// Dequantise a resident weight to f32 [rows][in_dim]; one thread per 16 consecutive
// elements. Every product is a single rounded multiply (__fmul_rn), in the operand
// order of the reference's dequant_q4_0 / _q8_0 / _q6_k
// (crates/strix-models/src/ggml_quant.rs:240-262, 404-430).
__global__ void dequant_kernel(const uint8_t *__restrict__ res, float *__restrict__ out, RowLayout L,
                               uint32_t rows) {
    const uint32_t upr = L.in_dim / 16;
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)rows * upr) return;
    const uint32_t row = (uint32_t)(idx / upr), u = (uint32_t)(idx % upr);
    float *o = out + (uint64_t)row * L.in_dim + (uint64_t)u * 16;
    if (L.fmt == FMT_Q6_K) {
        // elements 16u..16u+15 = super-block u/16, one 16-element sub-scale group
        const float d = f16_bits_to_f32(resident_scale_bits(res, L, row, u >> 4));
        const float dsc = __fmul_rn(d, (float)resident_q6k_subscale(res, L, row, u));
        for (uint32_t j = 0; j < 16; j++) o[j] = __fmul_rn(dsc, (float)((int)resident_code(res, L, row, 16u * u + j) - 32));
    } else if (L.fmt == FMT_Q4_1) {
        // d * code + m: multiply, then add, two roundings (dequant_q4_1, ggml_quant.rs:264-275)
        const float d = f16_bits_to_f32(resident_scale_bits(res, L, row, u >> 1));
        const float m = f16_bits_to_f32(resident_min_bits(res, L, row, u >> 1));
        for (uint32_t j = 0; j < 16; j++) o[j] = __fadd_rn(__fmul_rn(d, (float)resident_code(res, L, row, 16u * u + j)), m);
    } else {
        const float d = f16_bits_to_f32(resident_scale_bits(res, L, row, u >> 1));
        const int bias = L.fmt == FMT_Q8_0 ? 128 : 8;
        for (uint32_t j = 0; j < 16; j++) o[j] = __fmul_rn(d, (float)((int)resident_code(res, L, row, 16u * u + j) - bias));
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
