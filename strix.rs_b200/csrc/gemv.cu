// Fused dequant -> GEMV over resident GGUF Q4_0 / Q8_0 / Q6_K rows, f32-activation
// and int8-activation (integer-dot) forms, for sm_100a.
//
// Replaces the reference's q4_gemv, q8_0_gemv, q6_gemv, q8i_gemv, q4_gemv_dp,
// q4_gemv_dp2/dp3 and the xquant / rmsnorm_xquant / silu_xquant / geglu_xquant
// launches in front of them (crates/strix-backend-rocm/src/kernels.rs:41-69,
// 646-668, 607-640, 894-912, 228-361, 75-226).
//
// Design (HBM-bound streaming kernel, no tensor cores):
//  * one persistent CTA per SM; the weight rows of a launch are cut into tiles of
//    consecutive rows (one contiguous byte range each, see layout.h);
//  * a producer warp streams tiles HBM -> shared memory through a ring of stages
//    with 1-D bulk async copies (cp.async.bulk, no multicast) that complete on
//    "full" mbarriers; consumer warps hand a stage back through an "empty"
//    mbarrier. Bytes in flight per SM do not depend on occupancy or registers;
//  * the activation vector never touches shared memory: K is cut into units of 16
//    elements, a consumer warp owns NCH runs of 32 units for the whole kernel
//    ("column stationary") and keeps their x values (f32 pairs, or int8 after the
//    per-32 quantiser) in registers; wc warps cover one row between them, and
//    `slots` such groups work on different rows of a tile;
//  * a warp carries RB (2 or 4) rows at once: NCH x RB independent load/dot chains
//    per lane, then ONE transposed shuffle reduction for the batch;
//  * when wc > 1 the wc partial sums of a row meet in shared memory behind a named
//    barrier of just those warps and are added in a fixed order (reproducible);
//  * byte -> f32 conversion avoids the conversion unit: a PRMT/LOP3 drops two codes
//    into the mantissas of a packed f16 pair (1024 + code), a mixed-precision add
//    (f16 + f32 -> f32) removes the bias exactly, and packed f32x2 FMAs accumulate;
//  * every mbarrier wait is bounded; on expiry the kernel raises
//    STATUS_WAIT_TIMEOUT in the accelerator's status word and runs out its loops
//    without waiting again.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "strix_cuda.h"

namespace strix {

// First element (within the row) of the g-th group of four x values of unit u.
// A unit is the 16 elements that one lane multiplies per row:
//   Q8_0: 16 consecutive elements (half a block);
//   Q4_0: bytes 8hf..8hf+7 of block b: elements 8hf+i (low nibbles) and 16+8hf+i (high);
//   Q6_K: word c4 of ql/ql+32/qh in half h of super-block sb: elements 32k + 4c4 + j, k<4, j<4.
template <int FMT>
__device__ __forceinline__ uint32_t unit_elem(uint32_t u, uint32_t g) {
    if (FMT == FMT_Q8_0) return 16u * u + 4u * g;
    if (FMT == FMT_Q4_0) return 32u * (u >> 1) + 8u * (u & 1u) + (g >> 1) * 16u + (g & 1u) * 4u;
    uint32_t sb = u >> 4, r = u & 15u;
    return 256u * sb + 128u * (r >> 3) + 32u * g + 4u * (r & 7u);
}

// SwiGLU / GeGLU gates with the fast exponential (as the reference's device kernels do:
// silu_quant uses __expf, kernels.rs:879-892); relative error ~1e-6, far inside the 1e-3 contract.
__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
    const float C = 0.7978846f;
    const float t = C * (x + 0.044715f * x * x * x);
    const float th = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * t));  // tanh(t)
    return 0.5f * x * (1.0f + th);
}

// ---- shared-memory loads on 32-bit shared addresses (always LDS, 32-bit address arithmetic) ----
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
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
__device__ __forceinline__ float lds_f16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return f16_bits_to_f32(v);
}

// (f16 pair) + bias -> (f32 pair), one mixed-precision add per half. With the halves holding
// 1024 + code (or 64 + code) and bias = -(1024 + offset) the result is (code - offset) exactly.
__device__ __forceinline__ float2 unbias_pair(uint32_t h2, float bias) {
    float2 r;
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "add.rn.f32.f16 %0, lo, %3;\n\t"
        "add.rn.f32.f16 %1, hi, %3;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "r"(h2), "f"(bias));
    return r;
}
// bytes (I, I+1) of w -> packed f16 pair (1024 + b_I, 1024 + b_I+1)
template <int I>
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t w) {
    return __byte_perm(w, 0x64646464u, I == 0 ? 0x4140u : 0x4342u);
}
// sign-extended byte of w; sel4 from sext_sel(). (__byte_perm keeps only 3 bits per selector
// nibble, so the sign-replicating form goes through prmt.b32 itself.)
__device__ __forceinline__ int sext_byte(uint32_t w, uint32_t sel4) {
    int d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0u), "r"(sel4));
    return d;
}
__host__ __device__ constexpr uint32_t sext_sel(uint32_t i) { return i | ((i | 8u) << 4) | ((i | 8u) << 8) | ((i | 8u) << 12); }

// Per-lane activation state: NCH units (unit c = first_unit + 32 c), in registers for the whole kernel.
template <int FMT, int ACT, int NCH>
struct LaneX {
    static constexpr int ND = (FMT == FMT_Q6_K) ? 4 : 1;
    // f32 form: the 16 values of a unit as 8 pairs, ordered to match the packed f16 pairs the
    // decoder produces (see pair_index)
    float2 v2[ACT == STRIX_ACT_F32 ? NCH : 1][8];
    // int8 form: 16 codes as 4 words, per-32 scale(s), bias * sum of the codes
    uint32_t q[ACT == STRIX_ACT_Q8DOT ? NCH : 1][4];
    float d[ACT == STRIX_ACT_Q8DOT ? NCH : 1][ND];
    int qs[ACT == STRIX_ACT_Q8DOT ? NCH : 1][ND];
    // byte offsets (within a resident row) of unit 0's fields; unit c adds a compile-time step
    uint32_t off_w, off_s, off_hh, off_sc;
    uint32_t sel_a, sel_b;  // Q6_K: sign-extending PRMT selectors of this lane's sub-scale bytes
    uint32_t valid;         // bit c set: unit c lies inside the row
};

// Which two of a unit's 16 x values (order of unit_elem: v[4g + i]) go into pair p.
//   Q8_0 / Q6_K: natural order, pair p = (v[2p], v[2p+1]).
//   Q4_0: the nibble decoder yields, per code word wd (bytes 4wd..4wd+3), the pairs
//         (b0.lo, b2.lo), (b1.lo, b3.lo), (b0.hi, b2.hi), (b1.hi, b3.hi); low nibbles are
//         v[0..7], high nibbles v[8..15].
template <int FMT>
__device__ __forceinline__ void pair_index(int p, int &i0, int &i1) {
    if (FMT == FMT_Q4_0) {
        const int wd = p >> 2, k = p & 3;  // k: 0 lo(0,2)  1 lo(1,3)  2 hi(0,2)  3 hi(1,3)
        const int base = 4 * wd + (k & 1) + ((k & 2) ? 8 : 0);
        i0 = base;
        i1 = base + 2;
    } else {
        i0 = 2 * p;
        i1 = 2 * p + 1;
    }
}

__device__ __forceinline__ int quant1(float x, float inv) {
    int q = (int)rintf(x * inv);
    return max(-127, min(127, q));
}
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}

template <int FMT, int ACT, int NCH>
__device__ __forceinline__ void set_unit_x(LaneX<FMT, ACT, NCH> &X, int c, const float (&v)[16]) {
#pragma unroll
    for (int p = 0; p < 8; p++) {
        int i0, i1;
        pair_index<FMT>(p, i0, i1);
        X.v2[c][p] = make_float2(v[i0], v[i1]);
    }
}

__device__ __forceinline__ int sum4(uint32_t w) { return dp4a_ss(w, 0x01010101u, 0); }

// Integer-dot form: read unit u's 16 int8 codes (4 words in the decoder's order: the CTA's
// quantised activation is stored unit-major, so this is one 16-byte load), the block scale(s),
// and bias * sum(codes).
template <int FMT, int ACT, int NCH>
__device__ __forceinline__ void load_unit_q(LaneX<FMT, ACT, NCH> &X, int c, uint32_t u, const uint4 *xq4,
                                            const float *sd) {
    const uint4 w = xq4[u];
    X.q[c][0] = w.x; X.q[c][1] = w.y; X.q[c][2] = w.z; X.q[c][3] = w.w;
    if (FMT == FMT_Q8_0) {
        X.d[c][0] = sd[u >> 1];
        X.qs[c][0] = 128 * (sum4(w.x) + sum4(w.y) + sum4(w.z) + sum4(w.w));  // resident codes are q + 128
    } else if (FMT == FMT_Q4_0) {
        X.d[c][0] = sd[u >> 1];
        X.qs[c][0] = 8 * (sum4(w.x) + sum4(w.y) + sum4(w.z) + sum4(w.w));  // nibbles carry +8
    } else {
        const uint32_t blk0 = unit_elem<FMT>(u, 0) >> 5;  // group k of the unit lies in block blk0 + k
#pragma unroll
        for (uint32_t k = 0; k < 4; k++) {
            X.d[c][k] = sd[blk0 + k];
            X.qs[c][k] = 32 * sum4(X.q[c][k]);  // 6-bit codes carry +32
        }
    }
}

// Byte step between unit c and unit c+1 of a lane (32 units further along the row).
template <int FMT> struct Step;
template <> struct Step<FMT_Q8_0> { static constexpr uint32_t w = 512, s = 32, hh = 0, sc = 0; };
template <> struct Step<FMT_Q4_0> { static constexpr uint32_t w = 256, s = 32, hh = 0, sc = 0; };
template <> struct Step<FMT_Q6_K> { static constexpr uint32_t w = 256, s = 4, hh = 128, sc = 32; };

// Contribution of unit c of one resident row to that row's dot product.
// `rb` = 32-bit shared address of the row's first byte.
template <int FMT, int ACT, int NCH>
__device__ __forceinline__ float unit_dot(uint32_t rb, const LaneX<FMT, ACT, NCH> &X, int c) {
    const uint32_t cu = (uint32_t)c;
    if (FMT == FMT_Q8_0) {
        // resident codes are q + 128 (unsigned bytes)
        const uint4 w = lds128(rb + X.off_w + cu * Step<FMT>::w);
        const float d = lds_f16(rb + X.off_s + cu * Step<FMT>::s);
        if (ACT == STRIX_ACT_F32) {
            const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
            float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);
#pragma unroll
            for (int g = 0; g < 4; g++) {
                acc_a = __ffma2_rn(unbias_pair(bytes_to_h2<0>(ws[g]), -1152.0f), X.v2[c][2 * g], acc_a);
                acc_b = __ffma2_rn(unbias_pair(bytes_to_h2<2>(ws[g]), -1152.0f), X.v2[c][2 * g + 1], acc_b);
            }
            acc_a = __fadd2_rn(acc_a, acc_b);
            return d * (acc_a.x + acc_a.y);
        } else {
            int isum = dp4a_us(w.x, X.q[c][0], -X.qs[c][0]);  // sum((q+128) xq) - 128 sum(xq)
            isum = dp4a_us(w.y, X.q[c][1], isum);
            isum = dp4a_us(w.z, X.q[c][2], isum);
            isum = dp4a_us(w.w, X.q[c][3], isum);
            return (d * X.d[c][0]) * (float)isum;
        }
    } else if (FMT == FMT_Q4_0) {
        const uint2 w = lds64(rb + X.off_w + cu * Step<FMT>::w);
        const float d = lds_f16(rb + X.off_s + cu * Step<FMT>::s);
        if (ACT == STRIX_ACT_F32) {
            float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);
            const uint32_t wd[2] = {w.x, w.y};
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const uint32_t w0 = wd[k], w8 = wd[k] >> 8;
                // nibble in bits 0..3 of a half: 0x6400 | n = 1024 + n;  in bits 4..7: 0x5400 | (n << 4) = 64 + n
                const uint32_t lo02 = (w0 & 0x000F000Fu) | 0x64006400u, lo13 = (w8 & 0x000F000Fu) | 0x64006400u;
                const uint32_t hi02 = (w0 & 0x00F000F0u) | 0x54005400u, hi13 = (w8 & 0x00F000F0u) | 0x54005400u;
                acc_a = __ffma2_rn(unbias_pair(lo02, -1032.0f), X.v2[c][4 * k + 0], acc_a);
                acc_b = __ffma2_rn(unbias_pair(lo13, -1032.0f), X.v2[c][4 * k + 1], acc_b);
                acc_a = __ffma2_rn(unbias_pair(hi02, -72.0f), X.v2[c][4 * k + 2], acc_a);
                acc_b = __ffma2_rn(unbias_pair(hi13, -72.0f), X.v2[c][4 * k + 3], acc_b);
            }
            acc_a = __fadd2_rn(acc_a, acc_b);
            return d * (acc_a.x + acc_a.y);
        } else {
            const uint32_t lo0 = w.x & 0x0F0F0F0Fu, lo1 = w.y & 0x0F0F0F0Fu;
            const uint32_t hi0 = (w.x >> 4) & 0x0F0F0F0Fu, hi1 = (w.y >> 4) & 0x0F0F0F0Fu;
            int isum = dp4a_us(lo0, X.q[c][0], -X.qs[c][0]);  // raw nibbles, minus 8 * sum(xq)
            isum = dp4a_us(lo1, X.q[c][1], isum);
            isum = dp4a_us(hi0, X.q[c][2], isum);
            isum = dp4a_us(hi1, X.q[c][3], isum);
            return (d * X.d[c][0]) * (float)isum;
        }
    } else {
        const uint32_t ow = rb + X.off_w + cu * Step<FMT>::w;
        const uint32_t a = lds32(ow), b = lds32(ow + 32u), hh = lds32(rb + X.off_hh + cu * Step<FMT>::hh);
        const uint2 scw = lds64(rb + X.off_sc + cu * Step<FMT>::sc);  // the half's 8 sub-scales
        const float d = lds_f16(rb + X.off_s + cu * Step<FMT>::s);
        const uint32_t qw[4] = {(a & 0x0F0F0F0Fu) | ((hh & 0x03030303u) << 4),
                                (b & 0x0F0F0F0Fu) | ((hh & 0x0C0C0C0Cu) << 2),
                                ((a >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u),
                                ((b >> 4) & 0x0F0F0F0Fu) | ((hh >> 2) & 0x30303030u)};
        const float sc[4] = {(float)sext_byte(scw.x, X.sel_a), (float)sext_byte(scw.x, X.sel_b),
                             (float)sext_byte(scw.y, X.sel_a), (float)sext_byte(scw.y, X.sel_b)};
        if (ACT == STRIX_ACT_F32) {
            float2 t2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                float2 acc = __ffma2_rn(unbias_pair(bytes_to_h2<0>(qw[k]), -1056.0f), X.v2[c][2 * k], make_float2(0.f, 0.f));
                acc = __ffma2_rn(unbias_pair(bytes_to_h2<2>(qw[k]), -1056.0f), X.v2[c][2 * k + 1], acc);
                t2 = __ffma2_rn(make_float2(sc[k], sc[k]), acc, t2);
            }
            return d * (t2.x + t2.y);
        } else {
            float t = 0.f;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int isum = dp4a_us(qw[k], X.q[c][k], -X.qs[c][k]);  // minus 32 * sum(xq)
                t = fmaf(sc[k] * X.d[c][k], (float)isum, t);
            }
            return d * t;
        }
    }
}

// Sums RB per-lane values across the warp with fewer shuffles than RB separate butterflies: lanes
// trade the halves they do not keep (xor 16, then xor 8 for RB = 4), which leaves one row per lane,
// then a plain butterfly over the remaining lane bits. On return lane (32/RB) k holds the sum of row k.
template <int RB>
__device__ __forceinline__ float batch_reduce(const float (&v)[RB], uint32_t lane) {
    static_assert(RB == 1 || RB == 2 || RB == 4, "batch_reduce is written for 1, 2 or 4 rows");
    const bool up16 = (lane & 16u) != 0u;
    float k;
    if constexpr (RB == 1) {
        k = v[0] + __shfl_xor_sync(0xffffffffu, v[0], 16);
        k += __shfl_xor_sync(0xffffffffu, k, 8);
    } else if constexpr (RB == 4) {
        const bool up8 = (lane & 8u) != 0u;
        // after this step lanes 0-15 hold rows 0,1 and lanes 16-31 hold rows 2,3
        float k0 = up16 ? v[2] : v[0], s0 = up16 ? v[0] : v[2];
        float k1 = up16 ? v[3] : v[1], s1 = up16 ? v[1] : v[3];
        k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
        k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
        // lanes with bit 3 clear keep the even row of their pair, the others the odd one
        k = up8 ? k1 : k0;
        const float sx = up8 ? k0 : k1;
        k += __shfl_xor_sync(0xffffffffu, sx, 8);
    } else {
        k = up16 ? v[RB - 1] : v[0];
        const float sx = up16 ? v[0] : v[RB - 1];
        k += __shfl_xor_sync(0xffffffffu, sx, 16);
        k += __shfl_xor_sync(0xffffffffu, k, 8);
    }
    k += __shfl_xor_sync(0xffffffffu, k, 4);
    k += __shfl_xor_sync(0xffffffffu, k, 2);
    k += __shfl_xor_sync(0xffffffffu, k, 1);
    return k;
}

struct TileRef {
    uint32_t mat, row0, rows;
    const uint8_t *src;
};

__device__ __forceinline__ TileRef tile_ref(const GemvArgs &A, uint32_t t) {
    uint32_t m = 0;
    if (A.nmat > 1 && t >= A.mat[1].tile0) m = 1;
    if (A.nmat > 2 && t >= A.mat[2].tile0) m = 2;
    TileRef r;
    r.mat = m;
    r.row0 = (t - A.mat[m].tile0) * A.rows_per_tile;
    r.rows = min(A.rows_per_tile, A.mat[m].rows - r.row0);
    r.src = A.mat[m].w + (uint64_t)r.row0 * A.L.row_stride;
    return r;
}

// Shared-memory map of gemv_kernel (offsets in bytes):
//   0     full[64]   mbarriers: a stage's bulk copy has landed            (producer arms, copy completes)
//   512   empty[64]  mbarriers: the stage's consumer warps are done with it (one arrival per warp of the slot)
//   1024  ctl[0]     abort flag (a bounded wait ran out)
//   1088  red[32]    block reduction scratch (RMSNORM prologue)
//   1280  part       per slot: 2 x wc x 4 partial sums (rows split along K over wc warps)
//   2304  seq[64]    batch index last issued into each stage
//   2560  x          the activations: B x K f32, or K f32 staging + B x (K int8 codes + K/32 f32 block scales)
//   ...   stages     n_stages x stage_bytes, 128-byte aligned; one stage = one batch of RB rows
constexpr uint32_t SMEM_EMPTY_OFF = 512, SMEM_CTL_OFF = 1024, SMEM_RED_OFF = 1088, SMEM_PART_OFF = 1280;
constexpr uint32_t SMEM_SEQ_OFF = 2304, SMEM_X_OFF = 2560;

// Inverse of unit_elem for groups of four elements: natural float4 index e4 -> (unit, group).
template <int FMT>
__device__ __forceinline__ void elem4_to_unit(uint32_t e4, uint32_t &u, uint32_t &g) {
    if (FMT == FMT_Q8_0) {
        u = e4 >> 2;
        g = e4 & 3u;
    } else if (FMT == FMT_Q4_0) {
        const uint32_t e = e4 * 4u, w = e & 31u;
        u = 2u * (e >> 5) + ((w & 15u) >> 3);
        g = 2u * (w >> 4) + ((w & 7u) >> 2);
    } else {
        const uint32_t e = e4 * 4u;
        u = 16u * (e >> 8) + 8u * ((e >> 7) & 1u) + ((e & 31u) >> 2);
        g = (e >> 5) & 3u;
    }
}

template <int FMT, int ACT, int RB>
__global__ void __launch_bounds__((GEMV_WARPS + 1) * 32, 1) gemv_kernel(const __grid_constant__ GemvArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    if (A.debug & 2u) return;  // measurement only: cost of an empty launch of this shape
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem + SMEM_EMPTY_OFF);
    volatile uint32_t *ctl = reinterpret_cast<volatile uint32_t *>(smem + SMEM_CTL_OFF);
    float *red = reinterpret_cast<float *>(smem + SMEM_RED_OFF);
    float *part = reinterpret_cast<float *>(smem + SMEM_PART_OFF);
    volatile uint32_t *seq = reinterpret_cast<volatile uint32_t *>(smem + SMEM_SEQ_OFF);
    uint8_t *stages = smem + A.stage_off;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t wc = A.wc, n_slots = A.slots;
    const uint32_t n_cons = n_slots * wc;  // consumer warps; warp n_cons is the producer
    const uint32_t S = A.n_stages, grid = gridDim.x, bid = blockIdx.x;
    const uint32_t my_n = (A.n_tiles > bid) ? (A.n_tiles - bid + grid - 1) / grid : 0;
    const RowLayout L = A.L;
    const uint32_t U = L.in_dim / 16u, K = L.in_dim, B = A.nbatch;
    const uint32_t C = (U + 31u) / 32u;  // runs of 32 units along a row

    if (tid == 0) {
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], wc);
        }
        ctl[0] = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == n_cons) {
        // ---- producer: one bulk copy per batch of RB rows, into a ring of S stages. The first S copies
        //      start at once (they overlap the activation prologue); after that a stage is refilled as
        //      soon as the warps of the slot that consumed it have released it ----
        // The 32 lanes share the work: issuing one copy costs a few hundred cycles of dependent
        // instructions, which a single lane cannot hide at one copy per 5 KB. Each pass the lanes look
        // at the next 32 batches (lane l at batch base + l), poll their stages once, and the leading
        // run of free ones is issued. Issue stays strictly in batch order: a lane that polls stage s for
        // lap n can then rely on lap n - 1 having been issued, so the parity it tests cannot be
        // mistaken for the phase two laps back.
        const uint32_t win = S < 32u ? S : 32u;
        uint32_t base = 0, idle = 0;
        while (base < my_n && !ctl[0]) {  // after an abort nothing more is issued
            const uint32_t i = base + lane;
            bool ready = false;
            uint32_t s = 0;
            if (lane < win && i < my_n) {
                const uint32_t lap = i / S;
                s = i - lap * S;
                ready = lap == 0 || mbar_try_wait(&empty[s], (lap - 1u) & 1u);
            }
            const uint32_t m = __ballot_sync(0xffffffffu, ready);
            const uint32_t n = (m == 0xffffffffu) ? 32u : (uint32_t)__ffs((int)~m) - 1u;  // leading run of ready lanes
            if (lane < n) {
                TileRef t = tile_ref(A, bid + i * grid);
                const uint32_t bytes = t.rows * L.row_stride;
                seq[s] = i;  // consumers check it: tells this lap's completion from an older one's
                mbar_arrive_expect_tx(&full[s], bytes);
                bulk_g2s(stages + (uint64_t)s * A.stage_bytes, t.src, bytes, &full[s]);
            }
            base += n;
            // bounded like every other wait: 2^22 passes without progress
            if (n) {
                idle = 0;
            } else if (++idle >= (1u << 22)) {
                if (lane == 0) {
                    if (A.status) atomicOr(A.status, STATUS_WAIT_TIMEOUT);
                    ctl[0] = 1;
                }
                idle = 0;
            }
            __syncwarp();
        }
        if (lane == 0 && ctl[0]) {
            // after an abort consumers stop waiting: let the copies still in flight land (bounded)
            // before the CTA's shared memory is released
            for (uint32_t k = (base > S ? base - S : 0); k < base; k++)
                mbar_wait_bounded(&full[k % S], (k / S) & 1u, nullptr);
        }
        return;
    }

    // ---- consumers: activation prologue ----
    // The activation (after the optional RMSNorm / SwiGLU / GeGLU) is produced ONCE per CTA,
    // cooperatively, into shared memory, and stays there: a lane re-reads the 16 values of a unit
    // for every batch of rows (one conflict-free 16-byte load per group of four; the f32 form is
    // stored unit-major for that). Keeping x out of the register file is what lets 24 consumer
    // warps run per SM; the extra shared-memory reads are shared by the RB rows of a batch.
    //   f32 form:          xs4[b][g][U]   float4 = group g of unit u of activation row b
    //   integer-dot form:  xs[K] f32 staging (natural order, reused per activation row),
    //                      xq[b][U][16] int8 codes (unit-major), sd[b][K/32] block scales
    const uint32_t ct = n_cons * 32u;  // consumer threads = tid < ct
    float *xs0 = reinterpret_cast<float *>(smem + A.x_off);
    int8_t *xq0 = reinterpret_cast<int8_t *>(smem + A.x_off + K * 4u);
    float *sd0 = reinterpret_cast<float *>(smem + A.x_off + K * 4u + B * K);
#define STRIX_CONS_BAR() asm volatile("bar.sync 15, %0;" ::"r"(ct) : "memory")
    for (uint32_t bi = 0; bi < B; bi++) {
        const float *Aa = A.a + (size_t)bi * A.a_stride;
        const float *Ab = A.b ? A.b + (size_t)bi * A.b_stride : nullptr;
        float *xs = (ACT == STRIX_ACT_F32) ? xs0 + bi * K : xs0;
        float scale = 1.0f;
        if (A.pre == STRIX_PRE_RMSNORM) {
            // rmsnorm (crates/strix-backend-cpu/src/qwen3.rs:107-114): x * (1/sqrt(mean(x^2)+eps)) * w
            float ss = 0.f;
            for (uint32_t e4 = tid; e4 < K / 4u; e4 += ct) {
                const float4 t = __ldg(reinterpret_cast<const float4 *>(Aa) + e4);
                ss = fmaf(t.x, t.x, ss); ss = fmaf(t.y, t.y, ss); ss = fmaf(t.z, t.z, ss); ss = fmaf(t.w, t.w, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) red[warp] = ss;
            STRIX_CONS_BAR();
            float tot = 0.f;
            for (uint32_t w = 0; w < n_cons; w++) tot += red[w];
            scale = 1.0f / sqrtf(tot / (float)K + A.eps);
            if (B > 1) STRIX_CONS_BAR();  // red[] is rewritten for the next activation row
        }
        for (uint32_t e4 = tid; e4 < K / 4u; e4 += ct) {
            float4 a4 = __ldg(reinterpret_cast<const float4 *>(Aa) + e4);
            if (A.pre != STRIX_PRE_NONE) {
                const float4 b4 = __ldg(reinterpret_cast<const float4 *>(Ab) + e4);
                if (A.pre == STRIX_PRE_RMSNORM) {
                    a4.x = (a4.x * scale) * b4.x; a4.y = (a4.y * scale) * b4.y;
                    a4.z = (a4.z * scale) * b4.z; a4.w = (a4.w * scale) * b4.w;
                } else if (A.pre == STRIX_PRE_SWIGLU) {
                    a4.x = silu_f(a4.x) * b4.x; a4.y = silu_f(a4.y) * b4.y;
                    a4.z = silu_f(a4.z) * b4.z; a4.w = silu_f(a4.w) * b4.w;
                } else {
                    a4.x = gelu_tanh_f(a4.x) * b4.x; a4.y = gelu_tanh_f(a4.y) * b4.y;
                    a4.z = gelu_tanh_f(a4.z) * b4.z; a4.w = gelu_tanh_f(a4.w) * b4.w;
                }
            }
            if (ACT == STRIX_ACT_F32) {
                uint32_t u, g;
                elem4_to_unit<FMT>(e4, u, g);
                reinterpret_cast<float4 *>(xs)[g * U + u] = a4;
            } else {
                reinterpret_cast<float4 *>(xs)[e4] = a4;
            }
        }
        STRIX_CONS_BAR();
        if (ACT == STRIX_ACT_Q8DOT) {
            // per-32 quantiser (xquant8, kernels.rs:864-876): d = amax/127, inv = d>0 ? 1/d : 0,
            // q = clamp(rintf(x*inv)); eight lanes per block (four elements each), four blocks per warp pass
            int8_t *xq = xq0 + bi * K;
            float *sd = sd0 + bi * (K / 32u);
            const uint32_t sub = lane >> 3, l8 = lane & 7u;
            for (uint32_t blk = warp * 4u + sub; blk < K / 32u; blk += n_cons * 4u) {
                const float4 v = *reinterpret_cast<const float4 *>(xs + blk * 32u + l8 * 4u);
                float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                // (the trip count is uniform within each group of eight lanes only, hence the masks)
                const uint32_t mask = 0xffu << (sub * 8u);
                amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 4));
                const float d = amax / 127.0f;
                const float inv = d > 0.f ? 1.0f / d : 0.f;
                uint32_t qu, qg;
                elem4_to_unit<FMT>(blk * 8u + l8, qu, qg);
                reinterpret_cast<uint32_t *>(xq)[qu * 4u + qg] =
                    pack4(quant1(v.x, inv), quant1(v.y, inv), quant1(v.z, inv), quant1(v.w, inv));
                if (l8 == 0) sd[blk] = d;
            }
            STRIX_CONS_BAR();
        }
    }
#undef STRIX_CONS_BAR
    if (A.debug & 4u) return;  // measurement only: stop after the activation prologue

    // byte offsets (within a resident row) of the fields of this lane's unit in run 0
    LaneX<FMT, ACT, 1> X;
    uint32_t b_w, b_s, b_hh = 0, b_sc = 0;
    X.off_hh = X.off_sc = X.sel_a = X.sel_b = 0;
    X.valid = 1;
    if (FMT == FMT_Q8_0) {
        b_w = lane * 16u;
        b_s = L.off_d + 2u * (lane >> 1);
    } else if (FMT == FMT_Q4_0) {
        b_w = lane * 8u;
        b_s = L.off_d + 2u * (lane >> 1);
    } else {
        const uint32_t sb = lane >> 4, r = lane & 15u, h = r >> 3, c4 = r & 7u;
        b_w = sb * 128u + h * 64u + c4 * 4u;
        b_hh = L.off_qh + sb * 64u + h * 32u + c4 * 4u;
        b_sc = L.off_sc + sb * 16u + h * 8u;
        b_s = L.off_d + 2u * sb;
        X.sel_a = sext_sel(c4 >> 2);         // sub-scale byte (c4>>2)     of a word: groups 0 and 2
        X.sel_b = sext_sel((c4 >> 2) + 2u);  // sub-scale byte (c4>>2) + 2 of a word: groups 1 and 3
    }

    // ---- stream the batches: slot k (wc warps) takes batches k, k + n_slots, ... of this CTA; the
    //      wc warps of a slot split the runs of a row between them (warp w: runs w, w + wc, ...) ----
    const uint32_t slot = warp / wc, w = warp - slot * wc;
    const uint32_t st0 = smem_u32(stages);
    const bool skip = (A.debug & 1u) != 0u;
    constexpr uint32_t LPR = 32u / RB;  // after batch_reduce lane LPR*k holds row k
    b_w += w * Step<FMT>::w; b_s += w * Step<FMT>::s; b_hh += w * Step<FMT>::hh; b_sc += w * Step<FMT>::sc;
    const uint32_t d_w = wc * Step<FMT>::w, d_s = wc * Step<FMT>::s, d_hh = wc * Step<FMT>::hh, d_sc = wc * Step<FMT>::sc;
    float *my_part = part + slot * (2u * wc * 4u);
    uint32_t par = 0;
    uint32_t s = slot % S, ph = (slot / S) & 1u;
    for (uint32_t i = slot; i < my_n; i += n_slots) {
        // once any wait has run out, nobody waits again: the loop runs to its end on whatever is in
        // shared memory and the status word reports it
        // (a stage is used by different slots on different laps, so a slot does not see every phase of
        // full[s] go by; the batch index the producer left in seq[s] tells this lap's completion from
        // that of the lap before last, which has the same parity)
        if (!ctl[0]) {
            bool got = false;
            for (uint32_t it = 0; it < (1u << 22) && !got; ++it) got = mbar_try_wait(&full[s], ph) && seq[s] == i;
            if (!got) {
                if (A.status) atomicOr(A.status, STATUS_WAIT_TIMEOUT);
                ctl[0] = 1;
            }
        }
        const TileRef t = tile_ref(A, bid + i * grid);
        const uint32_t rb0 = st0 + s * A.stage_bytes;
        // Rows past the matrix's end read whatever the stage still holds; their sums are dropped.
        for (uint32_t bi = 0; bi < B && !skip; bi++) {
            float *y = A.mat[t.mat].y + (size_t)bi * A.mat[t.mat].ystride + t.row0;
            const float *res = A.mat[t.mat].res ? A.mat[t.mat].res + (size_t)bi * A.mat[t.mat].ystride + t.row0 : nullptr;
            const float4 *xs4 = reinterpret_cast<const float4 *>(xs0 + bi * K);
            const uint4 *xq4 = reinterpret_cast<const uint4 *>(xq0 + bi * K);
            const float *sd = sd0 + bi * (K / 32u);
            float acc[RB];
#pragma unroll
            for (int j = 0; j < RB; j++) acc[j] = 0.f;
            X.off_w = b_w; X.off_s = b_s; X.off_hh = b_hh; X.off_sc = b_sc;
            for (uint32_t u = w * 32u + lane; u < C * 32u; u += wc * 32u) {
                if (u < U) {
                    if (ACT == STRIX_ACT_F32) {
                        float v[16];
#pragma unroll
                        for (uint32_t g = 0; g < 4; g++) {
                            const float4 a4 = xs4[g * U + u];
                            v[4 * g] = a4.x; v[4 * g + 1] = a4.y; v[4 * g + 2] = a4.z; v[4 * g + 3] = a4.w;
                        }
                        set_unit_x<FMT, ACT, 1>(X, 0, v);
                    } else {
                        load_unit_q<FMT, ACT, 1>(X, 0, u, xq4, sd);
                    }
#pragma unroll
                    for (int j = 0; j < RB; j++)
                        acc[j] += unit_dot<FMT, ACT, 1>(rb0 + (uint32_t)j * L.row_stride, X, 0);
                }
                X.off_w += d_w; X.off_s += d_s; X.off_hh += d_hh; X.off_sc += d_sc;
            }
            const float tot = batch_reduce<RB>(acc, lane);
            const uint32_t rr = lane / LPR;
            const bool leader = (lane & (LPR - 1u)) == 0u;
            if (wc == 1) {
                if (leader && rr < t.rows) y[rr] = res ? tot + res[rr] : tot;
            } else {
                // partial sums of the slot's warps meet in shared memory (double-buffered, so one
                // barrier per batch is enough); warp 0 of the slot adds them in warp order
                float *pp = my_part + par * (wc * 4u);
                if (leader) pp[w * 4u + rr] = tot;
                asm volatile("bar.sync %0, %1;" ::"r"(1u + slot), "r"(wc * 32u) : "memory");
                if (w == 0 && lane < RB && lane < t.rows) {
                    float sum = pp[lane];
                    for (uint32_t k = 1; k < wc; k++) sum += pp[k * 4u + lane];
                    y[lane] = res ? sum + res[lane] : sum;
                }
                par ^= 1u;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);  // this warp's reads of the stage are complete
        s += n_slots;
        while (s >= S) { s -= S; ph ^= 1u; }
    }
}

// ------------------------------------------------------------------ host side
static inline uint32_t align128u(uint32_t v) { return (v + 127u) & ~127u; }

bool gemv_plan(GemvArgs &a, int num_sms, size_t smem_optin) {
    const uint32_t K = a.L.in_dim;
    if (K == 0 || K % 32 != 0) return false;
    const uint32_t pool = (uint32_t)GEMV_WARPS;
    const uint32_t U = K / 16, C = (U + 31) / 32;
    const uint32_t stride = a.L.row_stride;
    const uint32_t budget = (uint32_t)smem_optin - 1024u;
    const uint32_t nbt = a.nbatch ? a.nbatch : 1u;
    a.nbatch = nbt;
    // the CTA's activation: K f32 values; for the integer-dot form also K int8 codes and K/32 scales
    a.x_off = SMEM_X_OFF;
    const uint32_t stage_off =
        a.x_off + align128u(a.act == STRIX_ACT_Q8DOT ? K * 4u + nbt * (K + K / 8u) : nbt * K * 4u);
    if (stage_off + 2u * align128u(stride) > budget) return false;  // in_dim beyond what one SM can hold
    const uint32_t avail = budget - stage_off;

    // Geometry: a slot of wc warps works on one batch of rb rows (= one stage of the ring) at a time,
    // the 24 / wc slots on different batches. What must fit in shared memory is one stage per slot
    // plus the copies in flight (about 64 KB per SM keeps HBM busy). More rows per batch re-use each
    // x value read from shared memory and share one reduction; more warps per row shorten the serial
    // work of a small launch and shrink the footprint of long rows. Every feasible (rb, wc) is
    // costed in "unit-dots on the busiest warp" and the cheapest wins.
    uint64_t total_rows = 0;
    for (int k = 0; k < a.nmat; k++) total_rows += a.mat[k].rows;
    uint32_t best_rb = 0, best_wc = 0, best_S = 0;
    double best_cost = 1e300;
    static const uint32_t wcs[] = {1, 2, 3, 4, 6, 8, 12};
    uint32_t force_rb = 0, force_wc = 0;
    if (const char *e = getenv("STRIX_GEMV_RB")) force_rb = (uint32_t)atoi(e);  // tuning knobs
    if (const char *e = getenv("STRIX_GEMV_WC")) force_wc = (uint32_t)atoi(e);
    for (uint32_t flight = 65536u; flight >= 8192u && best_rb == 0; flight >>= 1) {
        for (uint32_t rb = 4; rb >= 1; rb >>= 1) {
            if (force_rb && rb != force_rb) continue;
            const uint32_t sb = align128u(rb * stride);
            uint32_t S = avail / sb;
            if (S > (uint32_t)GEMV_MAX_STAGES) S = (uint32_t)GEMV_MAX_STAGES;
            if (S < 2) continue;
            uint64_t batches = 0;
            for (int k = 0; k < a.nmat; k++) batches += (a.mat[k].rows + rb - 1) / rb;
            if (batches == 0) batches = 1;
            const uint64_t ctas = batches < (uint64_t)num_sms ? batches : (uint64_t)num_sms;
            const uint64_t per_cta = (batches + ctas - 1) / ctas;
            for (uint32_t wc : wcs) {
                if (force_wc && wc != force_wc) continue;
                if (wc > C) break;
                const uint32_t slots = pool / wc;
                uint64_t need = slots + (flight + sb - 1) / sb;
                if (need > per_cta) need = per_cta;  // a short launch never has more in the ring
                if (S < need) continue;
                const uint64_t rounds = (per_cta + slots - 1) / slots;
                const uint32_t passes = (C + wc - 1) / wc;
                const double cost = (double)rounds * nbt * (passes * (rb + 0.5) + 2.5 + (wc > 1 ? 2.0 : 0.0));
                if (cost < best_cost) { best_cost = cost; best_rb = rb; best_wc = wc; best_S = S; }
            }
        }
    }
    if (best_rb == 0) return false;
    const uint32_t rb = best_rb;
    a.rb = rb;
    a.wc = best_wc;
    a.slots = pool / best_wc;
    a.nch = 0;
    uint32_t tile = 0;
    for (int m = 0; m < a.nmat; m++) {
        a.mat[m].tile0 = tile;
        tile += (a.mat[m].rows + rb - 1) / rb;
    }
    a.n_tiles = tile;
    a.rows_per_tile = rb;
    a.stage_off = stage_off;
    a.stage_bytes = align128u(rb * stride);
    uint32_t S = best_S;
    if (const char *e = getenv("STRIX_GEMV_STAGES")) {  // tuning knob
        const uint32_t v = (uint32_t)atoi(e);
        if (v >= 2 && v <= (uint32_t)GEMV_MAX_STAGES && v * a.stage_bytes <= avail) S = v;
    }
    a.debug = 0;
    if (const char *e = getenv("STRIX_GEMV_DEBUG")) a.debug = (uint32_t)atoi(e);  // 1 = stream only, no arithmetic
    a.n_stages = S;
    a.smem_bytes = stage_off + S * a.stage_bytes;
    a.grid = a.n_tiles < (uint32_t)num_sms ? a.n_tiles : (uint32_t)num_sms;
    return true;
}

template <int FMT, int ACT>
static cudaError_t launch_t(const GemvArgs &a, cudaStream_t stream) {
    const uint32_t threads = (a.slots * a.wc + 1u) * 32u;  // consumer warps + one producer warp
    if (a.rb == 4)
        gemv_kernel<FMT, ACT, 4><<<a.grid, threads, a.smem_bytes, stream>>>(a);
    else if (a.rb == 2)
        gemv_kernel<FMT, ACT, 2><<<a.grid, threads, a.smem_bytes, stream>>>(a);
    else
        gemv_kernel<FMT, ACT, 1><<<a.grid, threads, a.smem_bytes, stream>>>(a);
    return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_fmt(const GemvArgs &a, cudaStream_t stream) {
    if (a.act == STRIX_ACT_F32) return launch_t<FMT, STRIX_ACT_F32>(a, stream);
    return launch_t<FMT, STRIX_ACT_Q8DOT>(a, stream);
}

cudaError_t launch_gemv(const GemvArgs &a, cudaStream_t stream) {
    if (a.n_tiles == 0) return cudaSuccess;
    switch (a.L.fmt) {
        case FMT_Q4_0: return launch_fmt<FMT_Q4_0>(a, stream);
        case FMT_Q8_0: return launch_fmt<FMT_Q8_0>(a, stream);
        default: return launch_fmt<FMT_Q6_K>(a, stream);
    }
}

template <int FMT>
static cudaError_t optin_fmt(size_t b) {
    cudaError_t e = cudaSuccess;
#define STRIX_ATTR(ACT_, RB_)                                                                               \
    if (e == cudaSuccess)                                                                                   \
        e = cudaFuncSetAttribute(gemv_kernel<FMT, ACT_, RB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)b);
    STRIX_ATTR(STRIX_ACT_F32, 1) STRIX_ATTR(STRIX_ACT_F32, 2) STRIX_ATTR(STRIX_ACT_F32, 4)
    STRIX_ATTR(STRIX_ACT_Q8DOT, 1) STRIX_ATTR(STRIX_ACT_Q8DOT, 2) STRIX_ATTR(STRIX_ACT_Q8DOT, 4)
#undef STRIX_ATTR
    return e;
}

cudaError_t gemv_prepare_device(size_t smem_optin) {
    cudaError_t e;
    if ((e = optin_fmt<FMT_Q4_0>(smem_optin)) != cudaSuccess) return e;
    if ((e = optin_fmt<FMT_Q8_0>(smem_optin)) != cudaSuccess) return e;
    return optin_fmt<FMT_Q6_K>(smem_optin);
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
