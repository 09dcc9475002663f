// Device code shared by the dequant-GEMV kernels (gemv.cu: one launch per step; chain.cu: a list of
// steps in one persistent launch): shared-memory loads, the tensor-core tile (one 16 x 32 tile of
// resident codes against the activation operands of its block), the shared-memory layout of those
// operands, and the activation prologue that builds them.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"
#include "strix_cuda.h"

namespace strix {

// SwiGLU / GeGLU gates with the fast exponential (as the reference's device kernels do:
// silu_quant uses __expf, kernels.rs:879-892); relative error ~1e-6, far inside the 1e-3 contract.
__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
    const float C = 0.7978846f;
    const float t = C * (x + 0.044715f * x * x * x);
    const float th = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * t));  // tanh(t)
    return 0.5f * x * (1.0f + th);
}

// ---- shared-memory loads on 32-bit shared addresses ----
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f16(uint32_t a) { return f16_bits_to_f32((uint16_t)lds_u16(a)); }

// bytes (I, I+1) of w -> packed f16 pair (1024 + b_I, 1024 + b_I+1)
template <int I>
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t w) {
    return __byte_perm(w, 0x64646464u, I == 0 ? 0x4140u : 0x4342u);
}

// D(16x8, f32) += A(16x16, f16) * B(16x8, f16)
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// int (|v| < 2^22) -> float without the conversion unit: drop it into the mantissa of 1.5 * 2^23
__device__ __forceinline__ float int_to_float_magic(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }

__device__ __forceinline__ int quant1(float x, float inv) {
    int q = (int)rintf(x * inv);
    return max(-127, min(127, q));
}
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}
__device__ __forceinline__ int sum4(uint32_t w) { return dp4a_ss(w, 0x01010101u, 0); }
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}

// Work geometry: a work item is one row group (16 rows) of one of the launch's matrices.
struct GroupRef {
    uint32_t mat, row0, rows;
    const uint8_t *src;
};
__device__ __forceinline__ GroupRef group_ref(const GemvArgs &A, uint32_t t) {
    uint32_t m = 0;
    if (A.nmat > 1 && t >= A.mat[1].tile0) m = 1;
    if (A.nmat > 2 && t >= A.mat[2].tile0) m = 2;
    GroupRef r;
    r.mat = m;
    const uint32_t gl = t - A.mat[m].tile0;
    r.row0 = gl * TILE_ROWS;
    r.rows = min(TILE_ROWS, A.mat[m].rows - r.row0);
    uint32_t gs = gl;  // the row group inside the resident stack
    if (A.sel_ids) {
        const uint32_t sel = gl / A.sel_groups;
        gs = min((uint32_t)A.sel_ids[sel], A.sel_experts - 1u) * A.sel_groups + (gl - sel * A.sel_groups);
    }
    r.src = A.mat[m].w + (uint64_t)gs * A.L.group_bytes;
    return r;
}

// Shared-memory map of gemv_kernel (offsets in bytes):
//   0     full[96]   mbarriers: a stage's bulk copy has landed             (producer arms, copy completes)
//   768   empty[96]  mbarriers: the stage's consumer warps are done with it (one arrival per warp of the slot)
//   1536  ctl[0]     abort flag (a bounded wait ran out)
//   1600  (64 words spare)
//   1856  oscale[8]  factor applied to the outputs of activation row j: the RMSNorm scale (which is
//                    linear, so it is applied after the product) / the power-of-two scale of the f16 split
//   1920  part       24 warps x 32 lanes x NV partial sums (rows split along K over the warps of a slot)
//   ...   x          the B operands, block sums and scales of the activations (see the prologue)
//   ...   stages     slots x n_stages x stage_bytes, 128-byte aligned; a stage = a run of tiles of one row group
constexpr uint32_t SMEM_EMPTY_OFF = 768, SMEM_CTL_OFF = 1536, SMEM_RED_OFF = 1600, SMEM_OSCALE_OFF = 1856;
constexpr uint32_t SMEM_PART_OFF = 1920;

// Values each lane carries per row group: rows g and g + 8 of one activation row (NV = 2), or of two
// (integer form with more than one activation row: C columns 2t and 2t + 1 are rows 2t, 2t + 1).
__host__ __device__ constexpr int lane_values(int act, bool multi) { return (act == STRIX_ACT_Q8DOT && multi) ? 4 : 2; }

// Kernel-internal third activation form (Q6_K, Q8_0 and Q4_0, one f32 activation row): the row is carried as THREE
// int8 digit rows, x = d * (q1 + q2 / 254 + q3 / 254^2) per 32-weight block (d = amax / 127, what is
// left over is below 2^-24 of the block's largest value), and runs through the integer form as if
// they were three activation rows; the epilogue adds the three partial results. The weight codes
// then feed the u8 x s8 MMA as they are stored: no conversion to f16, which was a third of the f32
// form's instructions for this format. For Q8_0 the f16 form is close to the memory pipeline's pace in a burst, but
// it is the one kernel of the family that slows down under sustained load (74.9 against 65.3 us on 151936 x 2560
// after half a second; the integer forms hold their burst time): its byte -> f16 conversions and two f16 MMAs per
// tile are the most work per byte of all forms.
constexpr int ACT_F32_DIGITS = 2;
constexpr uint32_t N_DIGITS = 3;

// Where the activation operands live in shared memory (all offsets from x_off, computed the same
// way by gemv_plan).
//   f32 form:      xB  uint4 [K/32][8 b]  lane 4c + t of block blk: B registers of column c (= 2j + hl:
//                                         hi / lo half of activation row j) for the block's two MMAs
//                  rec (Q4_1 only) [K/32][4] f32: the block's sum of row j's activations, scaled like xB
//   integer form:  xB  uint2 [K/32][4 b]  lane 4j + t: int8 codes k 4t..4t+3 and 16+4t..16+4t+3 of row j
//                  (Q6_K: [K/32][8 b], column 2j + h = row j against the first / last 16 weights only:
//                   the other word is zero)
//                  rec, per 32-weight block: what turns the block's integer sum into its contribution,
//                  d_x (block scale of x) and kf = -bias * d_x * sum(codes) (removes the +128 / +8 / +32
//                  the stored weight codes carry):
//                      Q4_0 / Q8_0, one row:   [K/32]    { d_x, kf }
//                      Q4_0 / Q8_0, 2..8 rows: [K/32][4] { d_x(2t), d_x(2t+1), kf(2t), kf(2t+1) }
//                      Q6_K:                   [K/32][4] { d_x(t), -32 * sum(codes of row t, first 16) as an int,
//                                                          the same for the last 16, 0 }
//   digit form:    the integer form's Q6_K layout with three rows (the digits of the one f32 row), for Q8_0 weights
//                  too (their MMA then adds the two halves' columns)
struct XLayout {
    uint32_t xb, rec, end;
    uint32_t xb_stride, rec_stride;  // bytes per 32-weight block
    uint32_t cols;                   // MMA columns in use (a power of two <= 8)
};
__host__ __device__ inline XLayout x_layout(int fmt, int act, uint32_t K, uint32_t b, uint32_t x_off) {
    XLayout X;
    const uint32_t nb32 = K / 32u;
    X.xb = x_off;
    if (act == ACT_F32_DIGITS) b = N_DIGITS;
    if (act == STRIX_ACT_F32) {
        X.cols = 2u * b;
        X.xb_stride = X.cols * 4u * 16u;
        X.rec_stride = fmt == FMT_Q4_1 ? 16u : 0u;  // Q4_1: the block's sum of (scaled) activations, per row
    } else {
        X.cols = (fmt == FMT_Q6_K || act == ACT_F32_DIGITS) ? 2u * b : b;
        X.xb_stride = X.cols * 4u * 8u;
        X.rec_stride = (fmt == FMT_Q6_K || b > 1) ? 64u : 8u;
    }
    X.rec = X.xb + nb32 * X.xb_stride;
    X.end = X.rec + nb32 * X.rec_stride;
    return X;
}

__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}
// byte I of w (an int8 stored as value + 128) -> float, through the mantissa of 2^23
template <int I>
__device__ __forceinline__ float biased_byte_to_float(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | I)) - 8388736.0f;
}
// byte I of w as a sign-extended int: one byte permute (a selector nibble with its top bit set copies
// the sign of the byte it names)
template <int I>
__device__ __forceinline__ int sext_byte(uint32_t w) {
    int d;
    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(d) : "r"(w), "n"(0x8880 + 0x1111 * I));
    return d;
}
// (a & b) | c in one instruction, all three from registers
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// packed f16 subtract (exact here: both operands are small integers)
__device__ __forceinline__ uint32_t hsub2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t mad_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// a constant the compiler keeps in a register (it cannot see through the asm)
__device__ __forceinline__ uint32_t reg_const(uint32_t v) {
    uint32_t d;
    asm volatile("mov.b32 %0, %1;" : "=r"(d) : "r"(v));
    return d;
}

// D(16x8, f32) = A(16x16, f16) * B(16x8, f16)  (zero accumulator: no registers to initialise)
__device__ __forceinline__ void mma_f16_z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// D(16x8, s32) = A(16x32, u8) * B(32x8, s8) + C, C kept in registers of its own (never written)
__device__ __forceinline__ void mma_u8s8_c(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1, const int (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// Loop-invariant registers of the tile code: masks and packed-f16 constants (kept in registers so
// that every field extraction is ONE three-input logic instruction), and the integer form's
// accumulator input 1.5 * 2^23 as an int (the MMA adds the block's integer sum into its mantissa).
struct TileConsts {
    uint32_t m000f, m00f0, k6400, k5400, bias_a, bias_b;
    int magic[4];
};
template <int FMT, int ACT>
__device__ __forceinline__ TileConsts tile_consts() {
    TileConsts C;
    C.m000f = reg_const(0x000F000Fu);
    C.m00f0 = reg_const(0x00F000F0u);
    C.k6400 = reg_const(0x64006400u);
    C.k5400 = reg_const(0x54005400u);
    // f16 pairs: 1024 + 8 and 64 + 8 (Q4_0), 1024 and 64 (Q4_1: codes are not centred), 1024 + 128 (Q8_0),
    // 1024 + 32 (Q6_K)
    C.bias_a = reg_const(FMT == FMT_Q4_0 ? 0x64086408u : FMT == FMT_Q4_1 ? 0x64006400u : FMT == FMT_Q8_0 ? 0x64806480u : 0x64206420u);
    C.bias_b = reg_const(FMT == FMT_Q4_1 ? 0x54005400u : 0x54805480u);
#pragma unroll
    for (int i = 0; i < 4; i++) C.magic[i] = (int)reg_const(0x4B400000u);
    return C;
}

// One tile (16 rows x 32 weights) against the activation operands of its block.
//   ta: shared address of the tile (Q6_K: of the 416-byte sub-tile); da: Q6_K only, shared address of
//   the super-block's scale pairs; xb_a / xr_a: this lane's B-operand and record addresses for the
//   block. acc: see lane_values().
//   Q6D = false (Q6_K only): the super-block scale is left out (the caller applies it once per
//   super-block to what this adds into acc).
template <int FMT, int ACT, bool MULTI, bool Q6D = true>
__device__ __forceinline__ void tile_mac(uint32_t ta, uint32_t da, uint32_t xb_a, uint32_t xr_a, const TileConsts &C,
                                         uint32_t lane, float (&acc)[lane_values(ACT, MULTI)]) {
    const uint32_t g = lane >> 2;
    constexpr uint32_t M4 = 0x0F0F0F0Fu, M30 = 0x30303030u;
    // ---- the 16 codes of this lane: A operand words (bytes) W0 (row g, k 4t..), W1 (row g+8, k 4t..),
    //      W2 (row g, k 16+4t..), W3 (row g+8, k 16+4t..); block scales of rows g and g + 8 ----
    uint32_t W0, W1, W2, W3;
    float2 d, mn = make_float2(0.f, 0.f);
    if (FMT == FMT_Q8_0) {
        W0 = lds32(ta + 4u * lane);
        W2 = lds32(ta + 128u + 4u * lane);
        W1 = lds32(ta + 256u + 4u * lane);
        W3 = lds32(ta + 384u + 4u * lane);
        d = h2_to_f2(lds32(ta + 512u + 4u * g));
    } else if (FMT == FMT_Q4_0 || FMT == FMT_Q4_1) {
        const uint2 n = lds64(ta + 8u * lane);
        W0 = n.x;  // nibbles: kept packed for the f32 form, split below for the integer form
        W2 = n.y;
        W1 = W3 = 0;
        d = h2_to_f2(lds32(ta + 256u + 4u * g));
        if (FMT == FMT_Q4_1) mn = h2_to_f2(lds32(ta + 288u + 4u * g));  // the block minimums of rows g and g + 8
    } else {
        const uint2 lo = lds64(ta + 8u * lane);
        const uint32_t H = lds32(ta + 256u + 4u * lane);
        W0 = (lo.x & M4) | ((H << 4) & M30);
        W1 = ((lo.x >> 4) & M4) | ((H << 2) & M30);
        W2 = (lo.y & M4) | (H & M30);
        W3 = ((lo.y >> 4) & M4) | ((H >> 2) & M30);
        d = Q6D ? h2_to_f2(lds32(da + 4u * g)) : make_float2(1.f, 1.f);
    }
    // Q6_K: the int8 sub-scales of the two 16-weight halves of rows g and g + 8, stored + 128:
    // {row g: first, last 16; row g + 8: first, last 16}
    uint32_t sc = 0u;
    if (FMT == FMT_Q6_K) sc = lds32(ta + 384u + 4u * g);

    if (ACT == STRIX_ACT_F32) {
        const uint4 xb = lds128(xb_a);
        float c0[4];
        if (FMT == FMT_Q4_0 || FMT == FMT_Q4_1) {
            // nibble in bits 0..3 of a half-word: 0x6400 | n = 1024 + n; in bits 4..7: 0x5400 | (n << 4) = 64 + n;
            // minus 1024 + 8 / 64 + 8 gives the signed weight, exactly. Even nibbles are row g, odd ones row g + 8.
            const uint32_t w8 = W0 >> 8, v8 = W2 >> 8;
            mma_f16_z(c0, hsub2_bits(and_or(W0, C.m000f, C.k6400), C.bias_a), hsub2_bits(and_or(W0, C.m00f0, C.k5400), C.bias_b),
                      hsub2_bits(and_or(w8, C.m000f, C.k6400), C.bias_a), hsub2_bits(and_or(w8, C.m00f0, C.k5400), C.bias_b),
                      xb.x, xb.y);
            mma_f16(c0, hsub2_bits(and_or(W2, C.m000f, C.k6400), C.bias_a), hsub2_bits(and_or(W2, C.m00f0, C.k5400), C.bias_b),
                    hsub2_bits(and_or(v8, C.m000f, C.k6400), C.bias_a), hsub2_bits(and_or(v8, C.m00f0, C.k5400), C.bias_b),
                    xb.z, xb.w);
            if (FMT == FMT_Q4_1) {
                // value = d * code + m: the minimum meets the block's sum of activations (scaled like the
                // operands; the record holds it per activation row), q4_1_gemv_dp's term (kernels.rs:289-320)
                const float xs = __uint_as_float(lds32(xr_a));
                acc[0] = fmaf(mn.x, xs, acc[0]);
                acc[1] = fmaf(mn.y, xs, acc[1]);
            }
            acc[0] = fmaf(d.x, c0[0] + c0[1], acc[0]);
            acc[1] = fmaf(d.y, c0[2] + c0[3], acc[1]);
        } else if (FMT == FMT_Q8_0) {
            mma_f16_z(c0, hsub2_bits(bytes_to_h2<0>(W0), C.bias_a), hsub2_bits(bytes_to_h2<0>(W1), C.bias_a),
                      hsub2_bits(bytes_to_h2<2>(W0), C.bias_a), hsub2_bits(bytes_to_h2<2>(W1), C.bias_a), xb.x, xb.y);
            mma_f16(c0, hsub2_bits(bytes_to_h2<0>(W2), C.bias_a), hsub2_bits(bytes_to_h2<0>(W3), C.bias_a),
                    hsub2_bits(bytes_to_h2<2>(W2), C.bias_a), hsub2_bits(bytes_to_h2<2>(W3), C.bias_a), xb.z, xb.w);
            acc[0] = fmaf(d.x, c0[0] + c0[1], acc[0]);
            acc[1] = fmaf(d.y, c0[2] + c0[3], acc[1]);
        } else {
            // (d * sub-scale) per half and row
            float s_lo0 = biased_byte_to_float<0>(sc), s_lo1 = biased_byte_to_float<1>(sc);
            float s_hi0 = biased_byte_to_float<2>(sc), s_hi1 = biased_byte_to_float<3>(sc);
            if (Q6D) {
                s_lo0 *= d.x; s_lo1 *= d.x; s_hi0 *= d.y; s_hi1 *= d.y;
            }
            float c1[4];
            mma_f16_z(c0, hsub2_bits(bytes_to_h2<0>(W0), C.bias_a), hsub2_bits(bytes_to_h2<0>(W1), C.bias_a),
                      hsub2_bits(bytes_to_h2<2>(W0), C.bias_a), hsub2_bits(bytes_to_h2<2>(W1), C.bias_a), xb.x, xb.y);
            mma_f16_z(c1, hsub2_bits(bytes_to_h2<0>(W2), C.bias_a), hsub2_bits(bytes_to_h2<0>(W3), C.bias_a),
                      hsub2_bits(bytes_to_h2<2>(W2), C.bias_a), hsub2_bits(bytes_to_h2<2>(W3), C.bias_a), xb.z, xb.w);
            acc[0] = fmaf(s_lo0, c0[0] + c0[1], acc[0]);
            acc[0] = fmaf(s_lo1, c1[0] + c1[1], acc[0]);
            acc[1] = fmaf(s_hi0, c0[2] + c0[3], acc[1]);
            acc[1] = fmaf(s_hi1, c1[2] + c1[3], acc[1]);
        }
    } else {
        if (FMT == FMT_Q4_0 || FMT == FMT_Q4_1) {
            const uint32_t n0 = W0, n1 = W2;
            W0 = n0 & M4;
            W1 = (n0 >> 4) & M4;
            W2 = n1 & M4;
            W3 = (n1 >> 4) & M4;
        }
        const uint2 xq = lds64(xb_a);
        int c[4];
        if (FMT == FMT_Q6_K) {
            // columns (2j, 2j + 1) = activation row j against the first / last 16 weights of the tile.
            // All in integers up to the block scale: the record's -32 * sum(x codes) of each half goes in
            // as the accumulator (it removes the +32 the stored weight codes carry), and the two halves
            // meet their int8 sub-scales in integer multiply-adds (|result| < 2^26):
            // y += (d_w * d_x) * (sc_first * (isum_first - 32 sum_first) + sc_last * (isum_last - 32 sum_last))
            const uint4 r = lds128(xr_a);
            const int cin[4] = {(int)r.y, (int)r.z, (int)r.y, (int)r.z};
            mma_u8s8_c(c, W0, W1, W2, W3, xq.x, xq.y, cin);
            const uint32_t ss = sc ^ 0x80808080u;  // signed bytes; the selectors below sign-extend one byte each
            const int s0 = sext_byte<0>(ss), s1 = sext_byte<1>(ss), s2 = sext_byte<2>(ss), s3 = sext_byte<3>(ss);
            const float dx = __uint_as_float(r.x);
            acc[0] = fmaf(Q6D ? dx * d.x : dx, (float)(s0 * c[0] + s1 * c[1]), acc[0]);
            acc[1] = fmaf(Q6D ? dx * d.y : dx, (float)(s2 * c[2] + s3 * c[3]), acc[1]);
            return;
        }
        if (ACT == ACT_F32_DIGITS) {
            // Q8_0 / Q4_0 against the digit operands (the Q6_K layout: columns 2j, 2j + 1 = digit j against the first /
            // last 16 weights; the record holds d_x(j) and -32 * sum(codes) of each half, the stored weight codes carry
            // +128 / +8): y += (d_w * d_x) * (isum_first + isum_last - bias * sum(codes))
            const uint4 r = lds128(xr_a);
            // (-32 * sum is a multiple of 32: the shift is exact)
            const int k0 = FMT == FMT_Q8_0 ? 4 * (int)r.y : ((int)r.y >> 2), k1 = FMT == FMT_Q8_0 ? 4 * (int)r.z : ((int)r.z >> 2);
            const int cin[4] = {k0, k1, k0, k1};
            mma_u8s8_c(c, W0, W1, W2, W3, xq.x, xq.y, cin);
            const float dx = __uint_as_float(r.x);
            acc[0] = fmaf(dx * d.x, (float)(c[0] + c[1]), acc[0]);
            acc[1] = fmaf(dx * d.y, (float)(c[2] + c[3]), acc[1]);
            return;
        }
        mma_u8s8_c(c, W0, W1, W2, W3, xq.x, xq.y, C.magic);
        // the integer sums arrive inside the mantissa of 1.5 * 2^23: one subtraction makes them floats.
        // y += d_w * (d_x * (float)isum + kf)  =  (d_w * d_x) * (float)(isum - bias * sum(codes)), the block
        // term of q8i_gemv / q4_gemv_dp (kernels.rs:894-912, 259-287)
        const float f0 = __int_as_float(c[0]) - 12582912.0f, f2 = __int_as_float(c[2]) - 12582912.0f;
        if constexpr (MULTI) {
            const uint4 r = lds128(xr_a);
            const float f1 = __int_as_float(c[1]) - 12582912.0f, f3 = __int_as_float(c[3]) - 12582912.0f;
            const float dx0 = __uint_as_float(r.x), dx1 = __uint_as_float(r.y);
            const float k0 = __uint_as_float(r.z), k1 = __uint_as_float(r.w);
            if (FMT == FMT_Q4_1) {
                // Q4_1: the record's k is d_x * sum(x codes); y += d_w * d_x * isum + m_w * k (kernels.rs:316)
                acc[0] = fmaf(d.x, dx0 * f0, fmaf(mn.x, k0, acc[0]));
                acc[1] = fmaf(d.x, dx1 * f1, fmaf(mn.x, k1, acc[1]));
                acc[2] = fmaf(d.y, dx0 * f2, fmaf(mn.y, k0, acc[2]));
                acc[3] = fmaf(d.y, dx1 * f3, fmaf(mn.y, k1, acc[3]));
            } else {
                acc[0] = fmaf(d.x, fmaf(dx0, f0, k0), acc[0]);
                acc[1] = fmaf(d.x, fmaf(dx1, f1, k1), acc[1]);
                acc[2] = fmaf(d.y, fmaf(dx0, f2, k0), acc[2]);
                acc[3] = fmaf(d.y, fmaf(dx1, f3, k1), acc[3]);
            }
        } else {
            const uint2 r = lds64(xr_a);
            const float dx = __uint_as_float(r.x), k0 = __uint_as_float(r.y);
            if (FMT == FMT_Q4_1) {
                acc[0] = fmaf(d.x, dx * f0, fmaf(mn.x, k0, acc[0]));
                acc[1] = fmaf(d.y, dx * f2, fmaf(mn.y, k0, acc[1]));
            } else {
                acc[0] = fmaf(d.x, fmaf(dx, f0, k0), acc[0]);
                acc[1] = fmaf(d.y, fmaf(dx, f2, k0), acc[1]);
            }
        }
    }
}

// The activation after the optional pre-op, four consecutive elements (e4 = float4 index). RMSNorm is
// applied WITHOUT its scalar 1/rms (the caller multiplies the outputs by it); `ss` collects the
// squares of the raw values for it.
template <int PRE>
__device__ __forceinline__ float4 load_pre(const float *Aa, const float *Ab, uint32_t e4, float &ss) {
    float4 a4 = __ldcg(reinterpret_cast<const float4 *>(Aa) + e4);
    if (PRE != STRIX_PRE_NONE) {
        const float4 b4 = __ldcg(reinterpret_cast<const float4 *>(Ab) + e4);
        if (PRE == STRIX_PRE_RMSNORM) {
            ss = fmaf(a4.x, a4.x, ss); ss = fmaf(a4.y, a4.y, ss); ss = fmaf(a4.z, a4.z, ss); ss = fmaf(a4.w, a4.w, ss);
            a4.x *= b4.x; a4.y *= b4.y; a4.z *= b4.z; a4.w *= b4.w;
        } else if (PRE == STRIX_PRE_SWIGLU) {
            a4.x = silu_f(a4.x) * b4.x; a4.y = silu_f(a4.y) * b4.y;
            a4.z = silu_f(a4.z) * b4.z; a4.w = silu_f(a4.w) * b4.w;
        } else {
            a4.x = gelu_tanh_f(a4.x) * b4.x; a4.y = gelu_tanh_f(a4.y) * b4.y;
            a4.z = gelu_tanh_f(a4.z) * b4.z; a4.w = gelu_tanh_f(a4.w) * b4.w;
        }
    }
    return a4;
}

// x * s (s a power of two) split into two f16 numbers hi + lo
__device__ __forceinline__ void split_h(float x, float s, __half &hi, __half &lo) {
    const float v = x * s;
    hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
}

// Per-thread view of the CTA: geometry that is the same for every step a CTA runs, and the ring
// positions that carry over from one step to the next.
struct Cta {
    uint8_t *smem;
    uint32_t tid, lane, warp, grid, bid;
    uint32_t wc, n_slots, n_cons, Sk, stage_bytes, stage_off;
    uint32_t *status;
    // producer: stage hand-overs every slot has seen so far; consumer: position in the slot's ring and
    // the parity of the phase to wait for
    uint32_t tq_base, sl, ph;
};
__device__ __forceinline__ uint64_t *cta_full(const Cta &C) { return reinterpret_cast<uint64_t *>(C.smem); }
__device__ __forceinline__ uint64_t *cta_empty(const Cta &C) { return reinterpret_cast<uint64_t *>(C.smem + SMEM_EMPTY_OFF); }
__device__ __forceinline__ volatile uint32_t *cta_ctl(const Cta &C) {
    return reinterpret_cast<volatile uint32_t *>(C.smem + SMEM_CTL_OFF);
}

// What the activation prologue reads: B activation rows of K floats (a_stride / b_stride floats apart),
// `b` the norm weight (RMSNorm) or the up vector (SwiGLU / GeGLU), and where in shared memory the
// operands go (see x_layout).
struct ActIn {
    const float *a, *b;
    uint32_t K, B, a_stride, b_stride, x_off;
    float eps;
};
__device__ __forceinline__ ActIn act_in(const GemvArgs &A) {
    ActIn I;
    I.a = A.a; I.b = A.b; I.K = A.L.in_dim; I.B = A.nbatch; I.a_stride = A.a_stride; I.b_stride = A.b_stride;
    I.x_off = A.x_off; I.eps = A.eps;
    return I;
}

// ---- consumers: operands prepared elsewhere ----
// The operand region arrives as an image in global memory (launch_xop_prepare wrote it once for all CTAs):
// thread 0 fetches it with bulk copies of at most 32 KB on an mbarrier of its own, everybody waits (bounded).
constexpr uint32_t SMEM_XBAR_OFF = SMEM_CTL_OFF + 32u;
__device__ __forceinline__ void image_prologue(const uint8_t *image, uint32_t x_off, uint32_t bytes, uint32_t nrows, const Cta &C) {
    uint64_t *bar = reinterpret_cast<uint64_t *>(C.smem + SMEM_XBAR_OFF);
    const uint32_t ct = C.n_cons * 32u;
    if (C.tid == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
        mbar_arrive_expect_tx(bar, bytes);
        for (uint32_t o = 0; o < bytes; o += 32768u)
            bulk_g2s(C.smem + x_off + o, image + o, min(32768u, bytes - o), bar);
    }
    if (C.tid < 8u) reinterpret_cast<float *>(C.smem + SMEM_OSCALE_OFF)[C.tid] = 1.0f;  // (the image is fully scaled)
    asm volatile("bar.sync 15, %0;" ::"r"(ct) : "memory");  // the barrier is initialised for everyone
    if (!mbar_wait_bounded(bar, 0u, C.status)) cta_ctl(C)[0] = 1;
    (void)nrows;
}

// ---- consumers: activation prologue ----
// The activation (after the optional RMSNorm / SwiGLU / GeGLU) is turned ONCE per CTA,
// cooperatively, into the B operands of the tensor-core instructions, in shared memory (see
// x_layout). It sits on the critical path of a small launch (the weights of such a launch are all
// in flight before it ends), so it is one trip to global memory: thread tid owns the float4s
// tid, tid + ct, ... of the row (eight consecutive threads = one 32-element block) and keeps
// them in registers across the one block-wide reduction. RMSNorm's scalar 1/rms is not applied
// here at all: the product is linear in it, so it multiplies the outputs (oscale).
// (Activations are read past L1: inside a chain kernel another CTA wrote them a moment ago.)
#define STRIX_CONS_BAR() asm volatile("bar.sync 15, %0;" ::"r"(ct) : "memory")
// (The pre-op is a template parameter: with all four inlined at every unrolled load the prologue
// alone was most of the kernel's code, and a small launch spent its time fetching instructions.)
template <int FMT, int ACT, bool MULTI, int PRE>
__device__ __forceinline__ void consumer_prologue(const ActIn &A, const Cta &C) {
    uint8_t *smem = C.smem;
    float *oscale = reinterpret_cast<float *>(smem + SMEM_OSCALE_OFF);
    const uint32_t tid = C.tid, lane = C.lane, warp = C.warp, n_cons = C.n_cons;
    const uint32_t K = A.K, B = A.B;
    const uint32_t ct = n_cons * 32u;  // consumer threads = tid < ct
    const XLayout XL = x_layout(FMT, ACT, K, B, A.x_off);
    {
        constexpr uint32_t NI = 6;  // float4s a thread keeps in registers; longer rows re-load the rest
        const uint32_t K4 = K / 4u, l8 = lane & 7u;
        const bool need_max = ACT == STRIX_ACT_F32;
        const bool need_red = need_max || PRE == STRIX_PRE_RMSNORM;
        if (XL.end > XL.rec && (B > 1 || ACT == ACT_F32_DIGITS)) {
            // records of columns that carry no activation row stay zero (what they produce is never stored)
            uint32_t *z = reinterpret_cast<uint32_t *>(smem + XL.rec);
            for (uint32_t i = tid; i < (XL.end - XL.rec) / 4u; i += ct) z[i] = 0u;
            STRIX_CONS_BAR();
        }
        // With several activation rows the warps split into one group per row and the rows are
        // prepared side by side (their trips to global memory overlap); a group meets at a named
        // barrier of its own. gt / gct: this thread's index in its group / threads per group.
        // (Long rows stay with all warps, one row after the other: a group of three warps would have to
        // re-read most of a 15360-long row, which measured slower than taking turns.)
        const bool grouped = B > 1 && K <= 8192u;
        const uint32_t wpg = grouped ? n_cons / B : n_cons;  // warps per group
        const uint32_t n_groups = grouped ? B : 1u;
        const uint32_t grp = warp / wpg, gw = warp - grp * wpg;
        const uint32_t gt = gw * 32u + lane, gct = wpg * 32u;
        float *scr = reinterpret_cast<float *>(smem + SMEM_PART_OFF);  // [row][2][32]: the partial-sum area is idle here
#define STRIX_ROW_BAR() asm volatile("bar.sync %0, %1;" ::"r"(grouped ? 1u + grp : 15u), "r"(gct) : "memory")
        for (uint32_t bi = grp; bi < B && grp < n_groups; bi += n_groups) {
            const float *Aa = A.a + (size_t)bi * A.a_stride;
            const float *Ab = A.b ? A.b + (size_t)bi * A.b_stride : nullptr;
            // phase A: load, apply the pre-op (without the RMSNorm scalar), partial sum of squares / maximum
            float4 v[NI];
            float ss = 0.f, amax = 0.f;
#pragma unroll
            for (uint32_t i = 0; i < NI; i++) {
                const uint32_t e4 = gt + i * gct;
                v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e4 < K4) v[i] = load_pre<PRE>(Aa, Ab, e4, ss);
                amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v[i].x), fabsf(v[i].y))), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
            }
            for (uint32_t e4 = gt + NI * gct; e4 < K4; e4 += gct) {
                const float4 t4 = load_pre<PRE>(Aa, Ab, e4, ss);
                amax = fmaxf(fmaxf(amax, fmaxf(fabsf(t4.x), fabsf(t4.y))), fmaxf(fabsf(t4.z), fabsf(t4.w)));
            }
            float s = 1.0f;  // f32 form: power-of-two scale before the f16 split
            if (need_red) {
                ss = warp_sum(ss);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                if (lane == 0) {
                    scr[bi * 64u + gw] = ss;
                    scr[bi * 64u + 32u + gw] = amax;
                }
                STRIX_ROW_BAR();
                float tot = 0.f, am = 0.f;
                for (uint32_t w2 = 0; w2 < wpg; w2++) {
                    tot += scr[bi * 64u + w2];
                    am = fmaxf(am, scr[bi * 64u + 32u + w2]);
                }
                // rmsnorm (crates/strix-backend-cpu/src/qwen3.rs:107-114): x * (1/sqrt(mean(x^2)+eps)) * w
                float os = PRE == STRIX_PRE_RMSNORM ? 1.0f / sqrtf(tot / (float)K + A.eps) : 1.0f;
                if (need_max) {
                    // largest magnitude -> power-of-two scale that puts it in [2^13, 2^14): keeps hi inside the
                    // f16 range, and lo (the 11 bits below hi) out of the subnormals except for values
                    // 2^-27 of the largest, whose contribution is below f32 resolution anyway.
                    // s = 2^(13 - floor(log2(am))), from the exponent field; 1 for zero, denormal or non-finite input
                    const int ex = (int)((__float_as_uint(am) >> 23) & 0xffu);
                    if (ex > 0 && ex < 255) {
                        const int se = max(1, min(254, 127 + 13 - (ex - 127)));  // biased exponent of s
                        s = __uint_as_float((uint32_t)se << 23);
                        os *= __uint_as_float((uint32_t)(254 - se) << 23);  // times 1/s, exact
                    }
                }
                if (gt == 0) oscale[bi] = os;
            } else if (gt == 0) {
                oscale[bi] = 1.0f;
            }
            // phase B: build the operands
            for (uint32_t i = 0;; i++) {
                const uint32_t e4 = gt + i * gct;
                if ((gt - lane) + i * gct >= K4) break;  // the whole warp is past the row's end (the loop body shuffles)
                const bool live = e4 < K4;
                float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < NI) {
                    // (static indexing keeps v[] in registers)
#pragma unroll
                    for (uint32_t k = 0; k < NI; k++)
                        if (k == i) t4 = v[k];
                } else if (live) {
                    float dummy = 0.f;
                    t4 = load_pre<PRE>(Aa, Ab, e4, dummy);
                }
                const uint32_t blk = e4 >> 3, t = l8 & 3u, hf = l8 >> 2;
                if (ACT == STRIX_ACT_F32) {
                    // this thread's four values are one MMA's worth of k for column pair (hi, lo) of row bi:
                    // words {b0, b1} of the first (hf = 0) or second (hf = 1) MMA of the block.
                    // Q8_0 / Q6_K pair the codes (k0,k1), (k2,k3); the Q4_0 nibble decoder (k0,k2), (k1,k3).
                    __half h[4], l[4];
                    split_h(t4.x, s, h[0], l[0]); split_h(t4.y, s, h[1], l[1]);
                    split_h(t4.z, s, h[2], l[2]); split_h(t4.w, s, h[3], l[3]);
                    uint2 uh, ul;
                    if (FMT == FMT_Q4_0 || FMT == FMT_Q4_1) {
                        uh = make_uint2(pack_h2(h[0], h[2]), pack_h2(h[1], h[3]));
                        ul = make_uint2(pack_h2(l[0], l[2]), pack_h2(l[1], l[3]));
                    } else {
                        uh = make_uint2(pack_h2(h[0], h[1]), pack_h2(h[2], h[3]));
                        ul = make_uint2(pack_h2(l[0], l[1]), pack_h2(l[2], l[3]));
                    }
                    if (live) {
                        uint2 *xb2 = reinterpret_cast<uint2 *>(smem + XL.xb);
                        xb2[(blk * 8u * B + (2u * bi) * 4u + t) * 2u + hf] = uh;
                        xb2[(blk * 8u * B + (2u * bi + 1u) * 4u + t) * 2u + hf] = ul;
                    }
                    if (FMT == FMT_Q4_1) {
                        float bs = ((t4.x + t4.y) + (t4.z + t4.w)) * s;  // s is a power of two: exact
                        bs += __shfl_xor_sync(0xffffffffu, bs, 1);
                        bs += __shfl_xor_sync(0xffffffffu, bs, 2);
                        bs += __shfl_xor_sync(0xffffffffu, bs, 4);
                        if (live && l8 == 0) reinterpret_cast<float *>(smem + XL.rec)[blk * 4u + bi] = bs;
                    }
                } else if (ACT == ACT_F32_DIGITS) {
                    // three int8 digits per value, base 254: q1 = rint(x / d), r = x / d - q1 (|r| <= 1/2),
                    // q2 = rint(254 r), q3 = rint(254 (254 r - q2)); digit j is activation row j of the
                    // integer form's Q6_K layout, with block scale d / 254^j
                    uint32_t *xbw = reinterpret_cast<uint32_t *>(smem + XL.xb);
                    float *rec = reinterpret_cast<float *>(smem + XL.rec);
                    float bm = fmaxf(fmaxf(fabsf(t4.x), fabsf(t4.y)), fmaxf(fabsf(t4.z), fabsf(t4.w)));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
                    const float d = bm / 127.0f;
                    float mul = d > 0.f ? 1.0f / d : 0.f, dj = d;
                    float r0 = t4.x, r1 = t4.y, r2 = t4.z, r3 = t4.w;
#pragma unroll
                    for (uint32_t j = 0; j < N_DIGITS; j++) {
                        const int q0 = quant1(r0, mul), q1 = quant1(r1, mul), q2 = quant1(r2, mul), q3 = quant1(r3, mul);
                        r0 = fmaf(r0, mul, -(float)q0); r1 = fmaf(r1, mul, -(float)q1);
                        r2 = fmaf(r2, mul, -(float)q2); r3 = fmaf(r3, mul, -(float)q3);
                        const uint32_t wq = pack4(q0, q1, q2, q3);
                        int cs = sum4(wq);
                        cs += __shfl_xor_sync(0xffffffffu, cs, 1);
                        cs += __shfl_xor_sync(0xffffffffu, cs, 2);  // over this lane's 16-weight half of the block
                        if (live) {
                            xbw[(blk * 8u * N_DIGITS + (2u * j + hf) * 4u + t) * 2u + hf] = wq;
                            xbw[(blk * 8u * N_DIGITS + (2u * j + hf) * 4u + t) * 2u + (hf ^ 1u)] = 0u;
                            if (l8 == 0) rec[blk * 16u + j * 4u] = dj;
                            if (t == 0) rec[blk * 16u + j * 4u + 1u + hf] = __int_as_float(-32 * cs);
                        }
                        mul = 254.0f;
                        dj *= (1.0f / 254.0f);
                    }
                } else {
                    // per-32 quantiser (xquant8, kernels.rs:864-876): d = amax/127, inv = d>0 ? 1/d : 0,
                    // q = clamp(rintf(x*inv)); eight lanes per block, four elements each
                    uint32_t *xbw = reinterpret_cast<uint32_t *>(smem + XL.xb);
                    float *rec = reinterpret_cast<float *>(smem + XL.rec);
                    // (Q4_1 is not centred: its record keeps +d_x * sum(codes) for the minimum's term)
                    constexpr int BIAS = FMT == FMT_Q8_0 ? 128 : FMT == FMT_Q4_0 ? 8 : FMT == FMT_Q4_1 ? -1 : 32;
                    float bm = fmaxf(fmaxf(fabsf(t4.x), fabsf(t4.y)), fmaxf(fabsf(t4.z), fabsf(t4.w)));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
                    const float d = bm / 127.0f;
                    const float inv = d > 0.f ? 1.0f / d : 0.f;
                    const uint32_t wq = pack4(quant1(t4.x, inv), quant1(t4.y, inv), quant1(t4.z, inv), quant1(t4.w, inv));
                    int cs = sum4(wq);
                    cs += __shfl_xor_sync(0xffffffffu, cs, 1);
                    cs += __shfl_xor_sync(0xffffffffu, cs, 2);
                    const int half_sum = cs;  // over this lane's 16-weight half of the block
                    cs += __shfl_xor_sync(0xffffffffu, cs, 4);
                    if (live) {
                        // lane l8 holds codes 4 l8 .. 4 l8 + 3 of the block = word hf of B-register pair t
                        if (FMT == FMT_Q6_K) {
                            // column 2 bi + hf sees only its own 16 weights: the other word stays zero
                            xbw[(blk * 8u * B + (2u * bi + hf) * 4u + t) * 2u + hf] = wq;
                            xbw[(blk * 8u * B + (2u * bi + hf) * 4u + t) * 2u + (hf ^ 1u)] = 0u;
                            if (l8 == 0) rec[blk * 16u + bi * 4u] = d;
                            if (t == 0) rec[blk * 16u + bi * 4u + 1u + hf] = __int_as_float(-BIAS * half_sum);
                        } else {
                            xbw[(blk * 4u * B + bi * 4u + t) * 2u + hf] = wq;
                            if (l8 == 0) {
                                const float kf = -(float)BIAS * d * (float)cs;
                                if (B > 1) {
                                    rec[blk * 16u + (bi >> 1) * 4u + (bi & 1u)] = d;
                                    rec[blk * 16u + (bi >> 1) * 4u + 2u + (bi & 1u)] = kf;
                                } else {
                                    rec[blk * 2u] = d;
                                    rec[blk * 2u + 1u] = kf;
                                }
                            }
                        }
                    }
                }
            }
        }
    }
#undef STRIX_ROW_BAR
    STRIX_CONS_BAR();
}
#undef STRIX_CONS_BAR

}  // namespace strix
