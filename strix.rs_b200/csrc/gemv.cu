// Fused dequant -> GEMV over resident tile-major weights (Q4_0 / Q8_0 / Q6_K), f32-activation
// and int8-activation (integer-dot) forms, for 1 to 8 activation rows per pass over the weights.
//
// Replaces the reference's batch-1 decode kernels (crates/strix-backend-rocm/src/kernels.rs:
// q4_gemv :141-176, q4_gemv_dp :259-287, q6k_gemv :178-237, q8_gemv :239-257, q8i_gemv :894-912,
// and the batched-verify GEMVs) and the CPU loops they mirror (crates/strix-backend-cpu/src/
// qwen3.rs:62-105 qmatmul / dot_f32).
//
// Shape of the kernel (one persistent CTA per SM, 24 consumer warps + 1 producer warp):
//   * The weights stream through shared memory: the producer warp issues 1-D bulk async copies
//     (cp.async.bulk, mbarrier complete_tx) of runs of tiles into per-slot rings of stages; DRAM
//     traffic is exactly the resident bytes, once.
//   * A slot is a group of wc warps that works on one row group (16 rows) at a time; the slots of
//     a CTA work on different row groups, the warps of a slot on different tiles of the group.
//   * A tile (16 rows x 32 weights) is one tensor-core instruction: mma.sync m16n8k32 u8 x s8 -> s32
//     for the integer-dot form, two m16n8k16 f16 x f16 -> f32 for the f32 form. The tile's codes are
//     the A operand straight from shared memory (bytes for the integer form; for the f32 form a byte
//     becomes the f16 value 1024 + code by one byte permute, exactly). The activation is the B
//     operand: column j of the int8 codes, or columns (2j, 2j + 1) = (hi, lo) halves of x split into
//     two f16 numbers (x = hi + lo to 2^-22), so that the f32 result keeps f32 accuracy. The code
//     biases (+128, +8, +32, +1024) are removed with the per-block sums of x, and the block scale is
//     applied to the block's sum, as the reference does.
//   * Without the tensor cores the kernel was bound by instruction issue (about 85 instructions per
//     16 weights x 32 lanes for Q8_0, more for Q6_K); a tile now costs about 25, which leaves the
//     memory pipeline as the limit and makes activation rows 2..8 almost free.
//   * Every wait is bounded: on expiry the kernel flags STATUS_WAIT_TIMEOUT, stops issuing copies,
//     stops waiting, and runs out.
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
    r.src = A.mat[m].w + (uint64_t)gl * A.L.group_bytes;
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

// Kernel-internal third activation form (Q6_K, one f32 activation row): the row is carried as THREE
// int8 digit rows, x = d * (q1 + q2 / 254 + q3 / 254^2) per 32-weight block (d = amax / 127, what is
// left over is below 2^-24 of the block's largest value), and runs through the integer form as if
// they were three activation rows; the epilogue adds the three partial results. The weight codes
// then feed the u8 x s8 MMA as they are stored: no conversion to f16, which was a third of the f32
// form's instructions for this format.
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
//   digit form:    the integer form's Q6_K layout with three rows (the digits of the one f32 row)
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
        X.cols = fmt == FMT_Q6_K ? 2u * b : b;
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
// row groups of one step are dealt round-robin to the CTAs, starting at a CTA that moves with the
// step (so that the CTAs that get one group more are not always the same ones)
__device__ __forceinline__ uint32_t cta_rank(const Cta &C, const GemvArgs &A) {
    const uint32_t r = C.bid + A.rot;
    return r >= C.grid ? r - C.grid : r;
}
__device__ __forceinline__ uint32_t cta_groups(const Cta &C, const GemvArgs &A) {
    const uint32_t r = cta_rank(C, A);
    return A.n_tiles > r ? (A.n_tiles - r + C.grid - 1) / C.grid : 0;
}

// ---- producer (one warp): one bulk copy per stage (a run of CT tiles of one row group). Slot k owns
//      stages k Sk .. k Sk + Sk - 1 and takes the CTA's row groups k, k + slots, ...; copies are issued in
//      the order (round of row groups, chunk, slot), so every slot's ring fills at the same pace. A
//      slot without a row group in the last round still gets its (empty) hand-overs, so that all rings
//      stay in step. The 32 lanes share the work: each pass they look at the next 32 entries, poll
//      their stages once, and the leading run of free ones is issued - strictly in order, so a lane
//      that polls a stage for lap n can rely on lap n - 1 having been issued. ----
__device__ __forceinline__ void producer_step(const GemvArgs &A, Cta &C) {
    uint64_t *full = cta_full(C), *empty = cta_empty(C);
    volatile uint32_t *ctl = cta_ctl(C);
    uint8_t *stages = C.smem + C.stage_off;
    const uint32_t n_slots = C.n_slots, Sk = C.Sk, lane = C.lane;
    const uint32_t my_n = cta_groups(C, A), rank = cta_rank(C, A);
    const uint32_t CT = A.chunk_tiles, NC = A.n_chunks;
    const uint32_t rounds = (my_n + n_slots - 1) / n_slots;
    uint32_t total = rounds * NC * n_slots;
    // (measurement mode "stop after the prologue": only the copies that need no consumer are issued)
    if ((A.debug & 4u) && total > n_slots * Sk) total = n_slots * Sk;
    const uint32_t win = n_slots * Sk < 32u ? n_slots * Sk : 32u;
    uint32_t base = 0, idle = 0;
    while (base < total && !ctl[0]) {  // after an abort nothing more is issued
        const uint32_t q = base + lane;
        bool ready = false, live = false;
        uint32_t s = 0, n = 0, c = 0;
        if (lane < win && q < total) {
            const uint32_t tq = q / n_slots, k = q - tq * n_slots;  // tq: this step's hand-over number in slot k
            const uint32_t r = tq / NC;
            c = tq - r * NC;
            n = r * n_slots + k;
            live = n < my_n;
            const uint32_t gq = C.tq_base + tq, lap = gq / Sk;
            s = k * Sk + (gq - lap * Sk);
            ready = lap == 0 || mbar_try_wait(&empty[s], (lap - 1u) & 1u);
        }
        const uint32_t m = __ballot_sync(0xffffffffu, ready);
        const uint32_t nrun = (m == 0xffffffffu) ? 32u : (uint32_t)__ffs((int)~m) - 1u;  // leading run of ready lanes
        if (lane < nrun && q < total) {
            if (live) {
                const GroupRef gr = group_ref(A, rank + n * C.grid);
                const uint32_t nbk = min(CT, A.L.nb - c * CT);
                const uint32_t bytes = nbk * A.L.tile_bytes;
                mbar_arrive_expect_tx(&full[s], bytes);
                bulk_g2s(stages + (uint64_t)s * C.stage_bytes, gr.src + (uint64_t)c * CT * A.L.tile_bytes, bytes, &full[s]);
            } else {
                mbar_arrive(&full[s]);  // an empty hand-over: the phase completes at once
            }
        }
        base += nrun;
        // bounded like every other wait: 2^22 passes without progress
        if (nrun) {
            idle = 0;
        } else if (++idle >= (1u << 22)) {
            if (lane == 0) {
                if (C.status) atomicOr(C.status, STATUS_WAIT_TIMEOUT);
                ctl[0] = 1;
            }
            idle = 0;
        }
        __syncwarp();
    }
    if (ctl[0]) {
        // after an abort consumers stop waiting: let the copies still in flight land (bounded) before
        // the CTA's shared memory is released. Lane k looks after slot k's last Sk hand-overs.
        if (lane < n_slots && base > lane) {
            const uint32_t tq_last = C.tq_base + (base - 1u - lane) / n_slots;
            for (uint32_t gq = (tq_last + 1u > Sk ? tq_last + 1u - Sk : 0u); gq <= tq_last; gq++) {
                uint64_t *bar = &full[lane * Sk + gq % Sk];
                for (uint32_t it = 0; it < (1u << 16); ++it)
                    if (mbar_try_wait(bar, (gq / Sk) & 1u)) break;
            }
        }
    } else {
        C.tq_base += rounds * NC;
    }
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
__device__ __forceinline__ void consumer_prologue(const GemvArgs &A, const Cta &C) {
    uint8_t *smem = C.smem;
    float *oscale = reinterpret_cast<float *>(smem + SMEM_OSCALE_OFF);
    const uint32_t tid = C.tid, lane = C.lane, warp = C.warp, n_cons = C.n_cons;
    const uint32_t K = A.L.in_dim, B = A.nbatch;
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

// ---- consumers: stream the row groups. Slot k takes the CTA's groups k, k + slots, ...; within a
//      stage the wc warps of the slot take tiles w, w + wc, ... ----
template <int FMT, int ACT, bool MULTI>
__device__ __forceinline__ void consumer_groups(const GemvArgs &A, Cta &C) {
    constexpr int NV = lane_values(ACT, MULTI);
    uint8_t *smem = C.smem;
    uint64_t *full = cta_full(C), *empty = cta_empty(C);
    volatile uint32_t *ctl = cta_ctl(C);
    const float *oscale = reinterpret_cast<const float *>(smem + SMEM_OSCALE_OFF);
    float *part = reinterpret_cast<float *>(smem + SMEM_PART_OFF);
    // (the warp index through a shuffle: the compiler then knows it is the same in every lane and keeps
    // the loop control that depends on it off the per-lane logic pipe)
    const uint32_t lane = C.lane, warp = __shfl_sync(0xffffffffu, C.warp, 0), wc = C.wc, n_slots = C.n_slots, Sk = C.Sk;
    const RowLayout L = A.L;
    const uint32_t B = A.nbatch, CT = A.chunk_tiles, NC = A.n_chunks;
    const uint32_t my_n = cta_groups(C, A), rank = cta_rank(C, A);
    const uint32_t rounds = (my_n + n_slots - 1) / n_slots;
    const XLayout XL = x_layout(FMT, ACT, L.in_dim, B, A.x_off);
    const uint32_t slot = warp / wc, w = warp - slot * wc;
    const uint32_t st0 = smem_u32(smem + C.stage_off) + slot * Sk * C.stage_bytes;
    const bool skip = (A.debug & 1u) != 0u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    // this lane's B-operand and record addresses for block 0 (see x_layout). Lanes whose MMA column
    // carries no activation row re-read a column that does: what they produce is never stored.
    const uint32_t xs0 = smem_u32(smem);
    // (a duplicate stays inside its own half of the warp, whose 16 lanes then touch one 128-byte run: a
    // duplicate of the other half's address would land on the same banks as this half's own lanes)
    const uint32_t n_op = XL.cols * 4u;
    const uint32_t lane_eff = (n_op > 16u && lane >= 16u) ? 16u + (lane - 16u) % (n_op - 16u) : lane % n_op;
    const uint32_t xb_l = xs0 + XL.xb + lane_eff * (ACT == STRIX_ACT_F32 ? 16u : 8u);
    const uint32_t xr_l = xs0 + XL.rec + ((FMT == FMT_Q6_K || MULTI) ? 16u * t : (FMT == FMT_Q4_1 && ACT == STRIX_ACT_F32) ? 4u * t : 0u);
    const TileConsts TC = tile_consts<FMT, ACT>();
    const uint32_t xb_step = wc * XL.xb_stride, xr_step = wc * XL.rec_stride, ta_step = wc * L.tile_bytes;
    const uint32_t q6_step = wc * Q6_SUB;
    float *my_part = part + (size_t)(warp * 32u + lane) * NV;
    for (uint32_t r = 0; r < rounds; r++) {
        const uint32_t n = r * n_slots + slot;
        const bool live = n < my_n;  // in the last round a slot may have no row group: its hand-overs are empty
        float acc[NV];
#pragma unroll
        for (int v = 0; v < NV; v++) acc[v] = 0.f;
        for (uint32_t c = 0; c < NC; c++) {
            // once any wait has run out, nobody waits again: the loop runs to its end on whatever is in
            // shared memory and the status word reports it
            if (!ctl[0] && !mbar_wait_bounded(&full[slot * Sk + C.sl], C.ph, C.status)) ctl[0] = 1;
            const uint32_t base = st0 + C.sl * C.stage_bytes;
            const uint32_t nbk = min(CT, L.nb - c * CT);
            if (live && !skip) {
                // tiles w, w + wc, ... of the stage; block index of tile i = first block of the stage + i
                constexpr uint32_t SUB = FMT == FMT_Q6_K ? 8u : 1u;
                const uint32_t blk0 = c * CT * SUB + w;
                uint32_t xb_a = mad_u32(blk0, XL.xb_stride, xb_l), xr_a = mad_u32(blk0, XL.rec_stride, xr_l);
                if (FMT == FMT_Q6_K && (wc == 1 || wc == 2 || wc == 4 || wc == 8)) {
                    // a warp's sub-tiles of one super-block share the super-block scale: it is applied
                    // once to their sum
                    uint32_t tb = base;
                    for (uint32_t sb = 0; sb < nbk; sb++, tb += Q6_TILE) {
                        const float2 d = h2_to_f2(lds32(tb + 8u * Q6_SUB + 4u * g));
                        float part_sb[NV];
#pragma unroll
                        for (int v = 0; v < NV; v++) part_sb[v] = 0.f;
                        uint32_t ta = tb + w * Q6_SUB;
                        // two sub-tiles per pass: two independent chains for the scheduler to interleave
                        float part_2[NV];
#pragma unroll
                        for (int v = 0; v < NV; v++) part_2[v] = 0.f;
                        if (wc == 4u) {
                            // (the large-launch geometry: exactly two sub-tiles per warp and super-block, no loop)
                            tile_mac<FMT, ACT, MULTI, false>(ta, 0u, xb_a, xr_a, TC, lane, part_sb);
                            tile_mac<FMT, ACT, MULTI, false>(ta + 4u * Q6_SUB, 0u, xb_a + xb_step, xr_a + xr_step, TC, lane, part_2);
                            xb_a += 2u * xb_step;
                            xr_a += 2u * xr_step;
                        } else {
                            for (uint32_t st = w; st < 8u; st += 2u * wc, ta += 2u * q6_step) {
                                tile_mac<FMT, ACT, MULTI, false>(ta, 0u, xb_a, xr_a, TC, lane, part_sb);
                                xb_a += xb_step;
                                xr_a += xr_step;
                                if (st + wc < 8u) {
                                    tile_mac<FMT, ACT, MULTI, false>(ta + q6_step, 0u, xb_a, xr_a, TC, lane, part_2);
                                    xb_a += xb_step;
                                    xr_a += xr_step;
                                }
                            }
                        }
                        part_sb[0] += part_2[0];
                        part_sb[1] += part_2[1];
                        acc[0] = fmaf(d.x, part_sb[0], acc[0]);
                        acc[1] = fmaf(d.y, part_sb[1], acc[1]);
                    }
                } else if (FMT == FMT_Q6_K) {
                    for (uint32_t i = w; i < nbk * 8u; i += wc, xb_a += xb_step, xr_a += xr_step) {
                        const uint32_t tb = mad_u32(i >> 3, Q6_TILE, base);
                        tile_mac<FMT, ACT, MULTI>(mad_u32(i & 7u, Q6_SUB, tb), tb + 8u * Q6_SUB, xb_a, xr_a, TC, lane, acc);
                    }
                } else {
                    // two tiles per pass: two independent chains for the scheduler to interleave
                    uint32_t ta = base + w * L.tile_bytes, i = w;
                    float acc2[NV];
#pragma unroll
                    for (int v = 0; v < NV; v++) acc2[v] = 0.f;
                    for (; i + wc < nbk; i += 2u * wc, ta += 2u * ta_step, xb_a += 2u * xb_step, xr_a += 2u * xr_step) {
                        tile_mac<FMT, ACT, MULTI>(ta, 0u, xb_a, xr_a, TC, lane, acc);
                        tile_mac<FMT, ACT, MULTI>(ta + ta_step, 0u, xb_a + xb_step, xr_a + xr_step, TC, lane, acc2);
                    }
                    if (i < nbk) tile_mac<FMT, ACT, MULTI>(ta, 0u, xb_a, xr_a, TC, lane, acc);
#pragma unroll
                    for (int v = 0; v < NV; v++) acc[v] += acc2[v];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot * Sk + C.sl]);  // this warp's reads of the stage are complete
            if (++C.sl == Sk) { C.sl = 0; C.ph ^= 1u; }
        }
        if (!live) continue;
        const GroupRef gr = group_ref(A, rank + n * C.grid);
        // ---- the row group is complete: add up the slot's partial sums (warp order) and store ----
        if (wc > 1) {
            // (first barrier: warp 0 has finished reading the previous group's partial sums)
            asm volatile("bar.sync %0, %1;" ::"r"(1u + slot), "r"(wc * 32u) : "memory");
#pragma unroll
            for (int v = 0; v < NV; v++) my_part[v] = acc[v];
            asm volatile("bar.sync %0, %1;" ::"r"(1u + slot), "r"(wc * 32u) : "memory");
            if (w != 0) continue;
            for (uint32_t k = 1; k < wc; k++) {
#pragma unroll
                for (int v = 0; v < NV; v++) acc[v] += my_part[(size_t)k * 32u * NV + v];
            }
        }
        if (ACT == ACT_F32_DIGITS) {
            // lane t of a quad holds digit t's share of rows g and g + 8: their sum is the output (lane 0 stores it)
#pragma unroll
            for (int v = 0; v < NV; v++) {
                float a = t < N_DIGITS ? acc[v] : 0.f;
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                acc[v] = a;
            }
        }
        // lane (g, t): NV = 2 -> rows g, g + 8 of activation row t; NV = 4 -> rows g, g + 8 of rows 2t, 2t + 1
#pragma unroll
        for (int v = 0; v < NV; v++) {
            const uint32_t row = g + ((NV == 2 ? v : (v >> 1)) ? 8u : 0u);
            const uint32_t j = NV == 2 ? t : 2u * t + (uint32_t)(v & 1);
            if (j < B && row < gr.rows) {
                float val = acc[v];
                val *= oscale[j];
                const size_t o = (size_t)j * A.mat[gr.mat].ystride + gr.row0 + row;
                const GemvMat &M = A.mat[gr.mat];
                if (M.res) val += __ldcg(M.res + o);
                if (M.y) M.y[o] = val;
                // row-sharded form: the row also goes straight into every accelerator's full vector
                // (plain stores over NVLink peer memory; what makes them visible is the end of this
                // kernel, which the barrier that follows it on the stream waits for)
                for (uint32_t p = 0; p < M.n_peer; p++) M.peer_y[p][(size_t)M.row_base + o] = val;
            }
        }
    }
}

__device__ __forceinline__ Cta cta_init(uint8_t *smem, uint32_t wc, uint32_t n_slots, uint32_t Sk, uint32_t stage_bytes,
                                        uint32_t stage_off, uint32_t *status) {
    Cta C;
    C.smem = smem;
    C.tid = threadIdx.x;
    C.lane = C.tid & 31u;
    C.warp = C.tid >> 5;
    C.grid = gridDim.x;
    C.bid = blockIdx.x;
    C.wc = wc;
    C.n_slots = n_slots;
    C.n_cons = n_slots * wc;  // consumer warps; warp n_cons is the producer
    C.Sk = Sk;
    C.stage_bytes = stage_bytes;
    C.stage_off = stage_off;
    C.status = status;
    C.tq_base = C.sl = C.ph = 0;
    if (C.tid < n_slots * Sk) {
        mbar_init(&cta_full(C)[C.tid], 1);
        mbar_init(&cta_empty(C)[C.tid], wc);
        if (C.tid == 0) cta_ctl(C)[0] = 0;
        mbar_fence_init();
    }
    __syncthreads();
    return C;
}

// One launch = one step: up to three weights that share an activation.
template <int FMT, int ACT, bool MULTI, int PRE>
__global__ void __launch_bounds__((GEMV_WARPS + 1) * 32, 1) gemv_kernel(const __grid_constant__ GemvArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    // Programmatic dependent launch: the next kernel of the stream may start on an SM as soon as this
    // kernel's CTA there has gone; it prefetches its weights and only then waits for this grid (below).
    asm volatile("griddepcontrol.launch_dependents;");
    if (A.debug & 2u) return;  // measurement only: cost of an empty launch of this shape
    Cta C = cta_init(smem, A.wc, A.slots, A.n_stages, A.stage_bytes, A.stage_off, A.status);
    if (C.warp == C.n_cons) {
        producer_step(A, C);
        return;
    }
    // Everything above (and the producer's copies) touches only this launch's weights. The activation
    // and the outputs belong to the stream's order: wait for the preceding grid here.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (A.sync_epoch) {
        // multi-GPU: the activations were stored here by the other ranks' previous kernels; each of them
        // released the epoch this rank has reached into its flag word when its kernel had finished.
        // (The producer warp is already prefetching weights: the wait hides behind that.)
        // (after one wait of the chain has run out nobody waits again: the status word says so)
        const bool gave_up = A.status && (*reinterpret_cast<volatile uint32_t *>(A.status) & STATUS_WAIT_TIMEOUT);
        if (C.tid < A.sync_world && !gave_up) {
            const uint32_t want = *reinterpret_cast<volatile uint32_t *>(A.sync_epoch);
            bool ok = false;
            for (uint32_t it = 0; it < (1u << 21) && !ok; ++it) {
                uint32_t seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(A.sync_local + C.tid) : "memory");
                ok = (int32_t)(seen - want) >= 0;
            }
            if (!ok && A.status) atomicOr(A.status, STATUS_WAIT_TIMEOUT);  // bounded: report and go on
        }
        asm volatile("bar.sync 15, %0;" ::"r"(C.n_cons * 32u) : "memory");
    }
    consumer_prologue<FMT, ACT, MULTI, PRE>(A, C);
    if (A.debug & 4u) return;  // measurement only: stop after the activation prologue
    consumer_groups<FMT, ACT, MULTI>(A, C);
    if (A.sync_epoch) {
        // this CTA's rows are stored (locally and on every peer); the last CTA of the grid to get here
        // tells the other ranks
        asm volatile("bar.sync 15, %0;" ::"r"(C.n_cons * 32u) : "memory");
        if (C.tid == 0) {
            __threadfence_system();
            if (atomicAdd(A.sync_done, 1u) == gridDim.x - 1u) {
                *A.sync_done = 0u;
                const uint32_t e = *reinterpret_cast<volatile uint32_t *>(A.sync_epoch) + 1u;
                *reinterpret_cast<volatile uint32_t *>(A.sync_epoch) = e;
                __threadfence_system();
                for (uint32_t p = 0; p < A.sync_world; p++)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(A.sync_peer[p] + A.sync_rank), "r"(e) : "memory");
            }
        }
    }
}

template <int FMT, int ACT>
__device__ __forceinline__ void chain_prologue(const GemvArgs &A, const Cta &C) {
    switch (A.pre) {
        case STRIX_PRE_NONE: consumer_prologue<FMT, ACT, false, STRIX_PRE_NONE>(A, C); break;
        case STRIX_PRE_RMSNORM: consumer_prologue<FMT, ACT, false, STRIX_PRE_RMSNORM>(A, C); break;
        case STRIX_PRE_SWIGLU: consumer_prologue<FMT, ACT, false, STRIX_PRE_SWIGLU>(A, C); break;
        default: consumer_prologue<FMT, ACT, false, STRIX_PRE_GEGLU>(A, C); break;
    }
}

// A whole chain of steps in ONE cooperative launch (one CTA per SM, all resident): the decode
// projection chain. Every step needs the outputs of the one before it, so between steps the CTAs
// meet at a grid-wide barrier (a counter in global memory; the wait is bounded like every other).
// What the single launches cannot do happens here: the producer warp does not wait at that barrier -
// it goes on filling the rings with the NEXT steps' weights (they depend on nothing) while the
// consumers finish this step and exchange activations, so HBM never idles between projections.
template <int ACT>
__global__ void __launch_bounds__((GEMV_WARPS + 1) * 32, 1)
gemv_chain_kernel(const GemvArgs *__restrict__ steps, uint32_t n_steps, uint32_t *gbar, unsigned long long *trace) {
    extern __shared__ __align__(128) uint8_t smem[];
    const GemvArgs &A0 = steps[0];
    Cta C = cta_init(smem, A0.wc, A0.slots, A0.n_stages, A0.stage_bytes, A0.stage_off, A0.status);
    volatile uint32_t *ctl = cta_ctl(C);
    if (C.warp == C.n_cons) {
        for (uint32_t s = 0; s < n_steps && !ctl[0]; s++) producer_step(steps[s], C);
        return;
    }
    const uint32_t ct = C.n_cons * 32u;
    for (uint32_t s = 0; s < n_steps; s++) {
        const GemvArgs &A = steps[s];
        if (s > 0) {
            // grid barrier: every CTA has stored the outputs of step s - 1
            STRIX_CONS_BAR();
            if (C.tid == 0) {
                __threadfence();
                atomicAdd(gbar, 1u);
                const uint32_t want = s * C.grid;
                bool ok = ctl[0] != 0;
                for (uint32_t it = 0; it < (1u << 22) && !ok; ++it) {
                    uint32_t seen;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(gbar) : "memory");
                    ok = seen >= want;
                    // another CTA gave up: do not sit out the full bound
                    if (!ok && (it & 1023u) == 1023u && C.status && (*(volatile uint32_t *)C.status & STATUS_WAIT_TIMEOUT)) break;
                }
                if (!ok) {
                    if (C.status) atomicOr(C.status, STATUS_WAIT_TIMEOUT);
                    ctl[0] = 1;
                }
            }
            STRIX_CONS_BAR();
        }
        // (measurement only: with a trace buffer, CTA 0 notes the time after the barrier, after the
        // prologue and after its row groups)
#define STRIX_TRACE(slot_)                                                                  \
    if (trace && C.bid == 0 && C.tid == 0) {                                                \
        unsigned long long t_;                                                              \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                              \
        trace[3u * s + (slot_)] = t_;                                                       \
    }
        STRIX_TRACE(0)
        switch (A.L.fmt) {
            case FMT_Q4_0:
                chain_prologue<FMT_Q4_0, ACT>(A, C);
                STRIX_TRACE(1)
                consumer_groups<FMT_Q4_0, ACT, false>(A, C);
                break;
            case FMT_Q4_1:
                chain_prologue<FMT_Q4_1, ACT>(A, C);
                STRIX_TRACE(1)
                consumer_groups<FMT_Q4_1, ACT, false>(A, C);
                break;
            case FMT_Q8_0:
                chain_prologue<FMT_Q8_0, ACT>(A, C);
                STRIX_TRACE(1)
                consumer_groups<FMT_Q8_0, ACT, false>(A, C);
                break;
            default:
                chain_prologue<FMT_Q6_K, ACT>(A, C);
                STRIX_TRACE(1)
                consumer_groups<FMT_Q6_K, ACT, false>(A, C);
                break;
        }
        STRIX_TRACE(2)
#undef STRIX_TRACE
    }
}
#undef STRIX_CONS_BAR

// ------------------------------------------------------------------ host side
static inline uint32_t align128u(uint32_t v) { return (v + 127u) & ~127u; }

bool gemv_plan(GemvArgs &a, int num_sms, size_t smem_optin) {
    const uint32_t K = a.L.in_dim;
    if (K == 0 || K % 32 != 0) return false;
    const uint32_t pool = (uint32_t)GEMV_WARPS;
    const uint32_t budget = (uint32_t)smem_optin - 1024u;
    const uint32_t nbt = a.nbatch ? a.nbatch : 1u;
    a.nbatch = nbt;
    // activation rows one pass can carry: the f32 form spends two MMA columns per row (hi, lo), and
    // so does Q6_K's integer form (two 16-weight halves); the other integer forms one
    const uint32_t bmax = (a.act == STRIX_ACT_F32 || a.L.fmt == FMT_Q6_K) ? 4u : 8u;
    if (nbt > bmax) return false;
    const bool multi = a.act == STRIX_ACT_Q8DOT && a.L.fmt != FMT_Q6_K && nbt > 1;
    const uint32_t nv = (uint32_t)lane_values(a.act, multi);
    a.x_off = align128u(SMEM_PART_OFF + pool * 32u * nv * 4u);
    // Q6_K with one f32 row: the digit form (its operands take 8 bytes of shared memory per weight
    // column, so long rows, which would starve the rings, keep the f16 form)
    uint32_t digit_rule = 1;
    if (const char *e = getenv("STRIX_GEMV_DIGITS")) digit_rule = (uint32_t)atoi(e);  // 0 = never, 2 = whenever it fits
    a.digits = (a.L.fmt == FMT_Q6_K && a.act == STRIX_ACT_F32 && nbt == 1 && digit_rule != 0 &&
                (K <= 8192u || digit_rule == 2))
                   ? 1u
                   : 0u;
    XLayout XL = x_layout(a.L.fmt, a.digits ? ACT_F32_DIGITS : a.act, K, nbt, a.x_off);
    if (a.digits && align128u(XL.end) + 2u * align128u(a.L.tile_bytes) > budget) {
        a.digits = 0;
        XL = x_layout(a.L.fmt, a.act, K, nbt, a.x_off);
    }
    const uint32_t stage_off = align128u(XL.end);
    if (stage_off + 2u * align128u(a.L.tile_bytes) > budget) return false;  // in_dim beyond what one SM can hold
    const uint32_t avail = budget - stage_off;

    // Geometry. A slot of wc warps works on one row group at a time, fed through its own ring of Sk
    // stages; a stage is a run of CT tiles (a multiple of wc, so every warp of the slot gets the same
    // share). More warps per group shorten the serial work of a small launch; more slots keep more row
    // groups in flight and waste less on the cross-warp sum. Every feasible wc is costed in "tiles on
    // the busiest warp" and the cheapest wins.
    uint64_t groups = 0;
    for (int k = 0; k < a.nmat; k++) groups += (a.mat[k].rows + TILE_ROWS - 1) / TILE_ROWS;
    if (groups == 0) groups = 1;
    const uint64_t ctas = groups < (uint64_t)num_sms ? groups : (uint64_t)num_sms;
    const uint64_t per_cta = (groups + ctas - 1) / ctas;
    const uint32_t nb = a.L.nb, tb = a.L.tile_bytes;
    const uint32_t sub = a.L.fmt == FMT_Q6_K ? 8u : 1u;  // MMA tiles per GGUF block
    static const uint32_t wcs[] = {1, 2, 3, 4, 6, 8, 12, 24};
    uint32_t force_wc = 0, force_ct = 0, force_sk = 0;
    if (const char *e = getenv("STRIX_GEMV_WC")) force_wc = (uint32_t)atoi(e);  // tuning knobs
    if (const char *e = getenv("STRIX_GEMV_CT")) force_ct = (uint32_t)atoi(e);
    if (const char *e = getenv("STRIX_GEMV_STAGES")) force_sk = (uint32_t)atoi(e);
    // Q6_K launches with at least two row groups for every warp of the grid: one warp per group (a warp
    // then owns whole super-blocks and nothing is exchanged between warps) measured 66.0 us against 70.1
    // for four warps per group on 151936 x 2560 inside the benchmark step; Q8_0 loses by it (84 against 68).
    const bool q6k_many = a.L.fmt == FMT_Q6_K && groups >= (uint64_t)num_sms * pool * 2u && !force_wc;
    uint32_t best_wc = 0, best_ct = 0, best_sk = 0;
    double best_cost = 1e300;
    for (uint32_t wc : wcs) {
        if (force_wc && wc != force_wc) continue;
        if (wc > nb * sub) break;
        const uint32_t slots = pool / wc;
        if (wc > 1 && slots > 12) continue;  // named barriers 1..12 serve the slots
        // stage size: aim at 3 stages per slot inside what is left of shared memory, at most 16 KB
        uint32_t target = avail / (slots * 3u);
        if (target > 16384u) target = 16384u;
        const uint32_t quantum = (wc + sub - 1) / sub;  // GGUF blocks that give every warp of the slot one tile
        uint32_t ct = (target / tb) / quantum * quantum;
        if (ct < quantum) ct = quantum;
        if (ct > nb) ct = nb;
        if (force_ct) ct = force_ct < nb ? force_ct : nb;
        const uint32_t sb = align128u(ct * tb);
        uint32_t sk = avail / (slots * sb);
        if (sk > 8u) sk = 8u;
        if (slots * sk > (uint32_t)GEMV_MAX_STAGES) sk = (uint32_t)GEMV_MAX_STAGES / slots;
        if (force_sk && force_sk <= sk) sk = force_sk;
        if (sk < 2u) continue;
        const uint64_t rounds = (per_cta + slots - 1) / slots;
        const uint32_t tiles = (nb * sub + wc - 1) / wc;       // tiles per warp per row group
        const uint32_t chunks = (nb + ct - 1) / ct;            // stage hand-overs per row group
        // (small stages cost copy efficiency: measured 83 us with 2.8 KB stages against 72 us with 10.9 KB
        // on the same 414 MB weight)
        const double cost = (double)rounds * (tiles + 0.5 * chunks + (wc > 1 ? 4.0 : 1.5)) * (sk >= 3u ? 1.0 : 1.3) *
                            (1.0 + 1500.0 / sb);
        if (cost < best_cost) { best_cost = cost; best_wc = wc; best_ct = ct; best_sk = sk; }
        if (q6k_many && wc == 1u) break;  // feasible: taken
    }
    if (best_wc == 0) return false;
    a.wc = best_wc;
    a.slots = pool / best_wc;
    a.chunk_tiles = best_ct;
    a.n_chunks = (nb + best_ct - 1) / best_ct;
    a.n_stages = best_sk;
    a.stage_bytes = align128u(best_ct * tb);
    a.stage_off = stage_off;
    uint32_t tile = 0;
    for (int m = 0; m < a.nmat; m++) {
        a.mat[m].tile0 = tile;
        tile += (a.mat[m].rows + TILE_ROWS - 1) / TILE_ROWS;
    }
    a.n_tiles = tile;
    a.rows_per_tile = TILE_ROWS;
    a.multi = multi ? 1u : 0u;
    a.pdl = 1;
    if (const char *e = getenv("STRIX_GEMV_PDL")) a.pdl = (uint32_t)atoi(e);  // 0 = plain stream order
    a.debug = 0;
    if (const char *e = getenv("STRIX_GEMV_DEBUG")) a.debug = (uint32_t)atoi(e);  // 1 = stream only, no arithmetic
    a.smem_bytes = stage_off + a.slots * a.n_stages * a.stage_bytes;
    a.grid = a.n_tiles < (uint32_t)num_sms ? a.n_tiles : (uint32_t)num_sms;
    return true;
}

template <int FMT, int ACT, bool MULTI>
static cudaError_t launch_t(const GemvArgs &a, cudaStream_t stream) {
    const uint32_t threads = (a.slots * a.wc + 1u) * 32u;  // consumer warps + one producer warp
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = a.smem_bytes;
    cfg.stream = stream;
    // programmatic stream serialization: this launch may begin (weight prefetch) while the previous
    // kernel of the stream drains; the kernel itself waits before it touches activations or outputs
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.pdl ? 1u : 0u;
    switch (a.pre) {
        case STRIX_PRE_NONE: return cudaLaunchKernelEx(&cfg, gemv_kernel<FMT, ACT, MULTI, STRIX_PRE_NONE>, a);
        case STRIX_PRE_RMSNORM: return cudaLaunchKernelEx(&cfg, gemv_kernel<FMT, ACT, MULTI, STRIX_PRE_RMSNORM>, a);
        case STRIX_PRE_SWIGLU: return cudaLaunchKernelEx(&cfg, gemv_kernel<FMT, ACT, MULTI, STRIX_PRE_SWIGLU>, a);
        case STRIX_PRE_GEGLU: return cudaLaunchKernelEx(&cfg, gemv_kernel<FMT, ACT, MULTI, STRIX_PRE_GEGLU>, a);
        default: return cudaErrorInvalidValue;
    }
}

template <int FMT>
static cudaError_t launch_fmt(const GemvArgs &a, cudaStream_t stream) {
    if constexpr (FMT == FMT_Q6_K) {
        if (a.digits) return launch_t<FMT, ACT_F32_DIGITS, false>(a, stream);
    }
    if (a.act == STRIX_ACT_F32) return launch_t<FMT, STRIX_ACT_F32, false>(a, stream);
    if constexpr (FMT != FMT_Q6_K) {
        if (a.multi) return launch_t<FMT, STRIX_ACT_Q8DOT, true>(a, stream);
    }
    return launch_t<FMT, STRIX_ACT_Q8DOT, false>(a, stream);
}

cudaError_t launch_gemv(const GemvArgs &a, cudaStream_t stream) {
    if (a.n_tiles == 0) return cudaSuccess;
    switch (a.L.fmt) {
        case FMT_Q4_0: return launch_fmt<FMT_Q4_0>(a, stream);
        case FMT_Q4_1: return launch_fmt<FMT_Q4_1>(a, stream);
        case FMT_Q8_0: return launch_fmt<FMT_Q8_0>(a, stream);
        default: return launch_fmt<FMT_Q6_K>(a, stream);
    }
}

// Geometry for a chain of steps run by one cooperative launch: the rings (warps per row group, slots,
// stages per slot, stage size) and the activation region are the same for every step, because the
// rings carry over from step to step; only the run of tiles per stage follows each step's tile size.
bool gemv_chain_plan(GemvArgs *steps, uint32_t n, int num_sms, size_t smem_optin, uint32_t *smem_bytes) {
    if (n == 0) return false;
    const uint32_t pool = (uint32_t)GEMV_WARPS;
    const uint32_t budget = (uint32_t)smem_optin - 1024u;
    uint32_t wc = 8;
    if (const char *e = getenv("STRIX_CHAIN_WC")) wc = (uint32_t)atoi(e);  // tuning knob
    if (wc < 2 || pool % wc != 0 || pool / wc > 12) return false;
    const uint32_t slots = pool / wc;
    uint32_t sk = 4;
    if (const char *e = getenv("STRIX_CHAIN_STAGES")) sk = (uint32_t)atoi(e);
    if (sk < 2 || slots * sk > (uint32_t)GEMV_MAX_STAGES) return false;
    const uint32_t x_off = align128u(SMEM_PART_OFF + pool * 32u * 2u * 4u);
    uint32_t x_end = x_off;
    for (uint32_t i = 0; i < n; i++) {
        GemvArgs &a = steps[i];
        if (a.act != steps[0].act || a.L.in_dim == 0 || a.L.in_dim % 32 != 0) return false;
        a.nbatch = 1;
        const XLayout XL = x_layout(a.L.fmt, a.act, a.L.in_dim, 1, x_off);
        if (XL.end > x_end) x_end = XL.end;
    }
    const uint32_t stage_off = align128u(x_end);
    if (stage_off >= budget) return false;
    uint32_t sb = ((budget - stage_off) / (slots * sk)) & ~127u;
    if (sb > 16384u) sb = 16384u;
    for (uint32_t i = 0; i < n; i++) {
        GemvArgs &a = steps[i];
        const uint32_t sub = a.L.fmt == FMT_Q6_K ? 8u : 1u;
        const uint32_t quantum = (wc + sub - 1) / sub;
        uint32_t ct = (sb / a.L.tile_bytes) / quantum * quantum;
        if (ct == 0) return false;  // a stage cannot hold one tile per warp of the slot
        if (ct > a.L.nb) ct = a.L.nb;
        a.wc = wc;
        a.slots = slots;
        a.n_stages = sk;
        a.stage_bytes = sb;
        a.stage_off = stage_off;
        a.x_off = x_off;
        a.chunk_tiles = ct;
        a.n_chunks = (a.L.nb + ct - 1) / ct;
        uint32_t tile = 0;
        for (int m = 0; m < a.nmat; m++) {
            a.mat[m].tile0 = tile;
            tile += (a.mat[m].rows + TILE_ROWS - 1) / TILE_ROWS;
        }
        a.n_tiles = tile;
        a.rows_per_tile = TILE_ROWS;
        a.multi = 0;
        a.digits = 0;
        a.pdl = 0;
        a.debug = 0;
        if (const char *e = getenv("STRIX_GEMV_DEBUG")) a.debug = (uint32_t)atoi(e) & 1u;  // 1 = no arithmetic
        a.rot = (i * 37u) % (uint32_t)num_sms;
        a.grid = (uint32_t)num_sms;
        a.smem_bytes = stage_off + slots * sk * sb;
    }
    *smem_bytes = steps[0].smem_bytes;
    return true;
}

cudaError_t launch_gemv_chain(const GemvArgs *d_steps, uint32_t n_steps, int act, uint32_t *d_gbar, int num_sms,
                              uint32_t smem_bytes, unsigned long long *d_trace, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(d_gbar, 0, sizeof(uint32_t), stream);
    if (e != cudaSuccess) return e;
    void *args[4] = {(void *)&d_steps, (void *)&n_steps, (void *)&d_gbar, (void *)&d_trace};
    const dim3 grid((unsigned)num_sms), block((GEMV_WARPS + 1) * 32);
    // cooperative: the CTAs wait on one another between steps, so all of them must be resident
    if (act == STRIX_ACT_F32)
        return cudaLaunchCooperativeKernel((const void *)gemv_chain_kernel<STRIX_ACT_F32>, grid, block, args, smem_bytes, stream);
    return cudaLaunchCooperativeKernel((const void *)gemv_chain_kernel<STRIX_ACT_Q8DOT>, grid, block, args, smem_bytes, stream);
}

template <int FMT>
static cudaError_t optin_fmt(size_t b) {
    cudaError_t e = cudaSuccess;
#define STRIX_ATTR1(ACT_, MULTI_, PRE_)                                                                                \
    if (e == cudaSuccess)                                                                                              \
        e = cudaFuncSetAttribute(gemv_kernel<FMT, ACT_, MULTI_, PRE_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)b);
#define STRIX_ATTR(ACT_, MULTI_)                                                                 \
    STRIX_ATTR1(ACT_, MULTI_, STRIX_PRE_NONE) STRIX_ATTR1(ACT_, MULTI_, STRIX_PRE_RMSNORM)      \
    STRIX_ATTR1(ACT_, MULTI_, STRIX_PRE_SWIGLU) STRIX_ATTR1(ACT_, MULTI_, STRIX_PRE_GEGLU)
    STRIX_ATTR(STRIX_ACT_F32, false) STRIX_ATTR(STRIX_ACT_Q8DOT, false)
    if constexpr (FMT != FMT_Q6_K) { STRIX_ATTR(STRIX_ACT_Q8DOT, true) }
    if constexpr (FMT == FMT_Q6_K) { STRIX_ATTR(ACT_F32_DIGITS, false) }
#undef STRIX_ATTR
#undef STRIX_ATTR1
    return e;
}

cudaError_t gemv_prepare_device(size_t smem_optin) {
    cudaError_t e;
    if ((e = optin_fmt<FMT_Q4_0>(smem_optin)) != cudaSuccess) return e;
    if ((e = optin_fmt<FMT_Q4_1>(smem_optin)) != cudaSuccess) return e;
    if ((e = optin_fmt<FMT_Q8_0>(smem_optin)) != cudaSuccess) return e;
    if ((e = optin_fmt<FMT_Q6_K>(smem_optin)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemv_chain_kernel<STRIX_ACT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)smem_optin)) != cudaSuccess)
        return e;
    return cudaFuncSetAttribute(gemv_chain_kernel<STRIX_ACT_Q8DOT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)smem_optin);
}

// ---- cross-GPU barrier (one rank per GPU; never run two ranks of it on one GPU) ----
struct PeerFlags {
    uint32_t *p[GEMV_MAX_PEERS];
};
__global__ void peer_barrier_kernel(uint32_t *epoch, volatile uint32_t *local_flags, PeerFlags peers, int rank, int world,
                                    uint32_t *status) {
    __shared__ uint32_t seq;
    if (threadIdx.x == 0) seq = ++(*epoch);
    __syncthreads();
    const uint32_t want = seq;
    if ((int)threadIdx.x < world) {
        // the kernels before this one on the stream have completed: their stores to peer memory are done
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.p[threadIdx.x] + rank), "r"(want) : "memory");
        bool ok = status && (*reinterpret_cast<volatile uint32_t *>(status) & STATUS_WAIT_TIMEOUT);  // gave up before
        for (uint32_t it = 0; it < (1u << 22) && !ok; ++it) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(local_flags + threadIdx.x) : "memory");
            ok = (int32_t)(seen - want) >= 0;
        }
        if (!ok && status) atomicOr(status, STATUS_WAIT_TIMEOUT);  // bounded: report and go on
    }
}

cudaError_t launch_peer_barrier(uint32_t *d_epoch, uint32_t *d_local_flags, uint32_t *const *peer_flags, int rank,
                                int world, uint32_t *d_status, cudaStream_t stream) {
    if (world < 1 || world > GEMV_MAX_PEERS) return cudaErrorInvalidValue;
    PeerFlags pf{};
    for (int i = 0; i < world; i++) pf.p[i] = peer_flags[i];
    peer_barrier_kernel<<<1, 32, 0, stream>>>(d_epoch, d_local_flags, pf, rank, world, d_status);
    return cudaGetLastError();
}

// ---- the activation quantiser on its own (xquant8_rows, kernels.rs:1000-1013) ----
__global__ void xquant8_kernel(const float *__restrict__ x, int8_t *__restrict__ q, float *__restrict__ d,
                               uint32_t nblk) {
    const uint32_t blk = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    if (blk >= nblk) return;
    const float v = x[(uint64_t)blk * 32u + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax / 127.0f;
    const float inv = sc > 0.f ? 1.0f / sc : 0.f;
    q[(uint64_t)blk * 32u + lane] = (int8_t)quant1(v, inv);
    if (lane == 0) d[blk] = sc;
}

cudaError_t launch_xquant8(const float *d_x, int8_t *d_q, float *d_d, uint32_t n, cudaStream_t stream) {
    const uint32_t nblk = n / 32;
    if (nblk == 0) return cudaSuccess;
    const uint32_t T = 256, per = T / 32;
    xquant8_kernel<<<(nblk + per - 1) / per, T, 0, stream>>>(d_x, d_q, d_d, nblk);
    return cudaGetLastError();
}

}  // namespace strix
