// Fused dequant -> GEMV over resident GGUF Q4_0 / Q8_0 / Q6_K rows, f32-activation
// and int8-activation (integer-dot) forms, for sm_100a.
//
// Replaces the reference's q4_gemv, q8_0_gemv, q6_gemv, q8i_gemv, q4_gemv_dp,
// q4_gemv_dp2/dp3 and the xquant / rmsnorm_xquant / silu_xquant / geglu_xquant
// launches in front of them (crates/strix-backend-rocm/src/kernels.rs:41-69,
// 646-668, 607-640, 894-912, 228-361, 75-226).
//
// Design (HBM-bound streaming kernel, no tensor cores):
//  * one persistent CTA per SM; the weight rows of a launch are cut into tiles
//    of consecutive rows (one contiguous byte range each, see layout.h);
//  * tiles stream HBM -> shared memory through a ring of up to 8 stages filled
//    by 1-D bulk async copies (cp.async.bulk, no multicast) that complete on
//    mbarriers, so the bytes in flight per SM do not depend on occupancy or on
//    registers;
//  * the activation vector never touches shared memory: K is cut into units of
//    16 elements, a warp owns the same units for the whole kernel ("column
//    stationary") and keeps their x values (f32, or int8 after the per-32
//    quantiser) in registers; wc warps cover one row between them and `slots`
//    such groups work on different rows of a tile;
//  * a row's wc partial sums meet in shared memory and are added in a fixed
//    order, so results are reproducible run to run;
//  * every mbarrier wait is bounded; on expiry the kernel raises
//    STATUS_WAIT_TIMEOUT in the accelerator's status word and leaves.
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

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
    const float C = 0.7978846f;
    return 0.5f * x * (1.0f + tanhf(C * (x + 0.044715f * x * x * x)));
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

// Byte -> f32 without a conversion instruction: one PRMT drops byte i of `w` into the mantissa of
// a constant, so the result is (2^k + byte) exactly.
//   magic15: byte lands in bits 8..15 of 0x47000000 -> 32768 + byte   (any byte 0..255)
//   magic7 : byte lands in bits 16..23 of 0x43000000 -> 128 + byte    (byte < 128 only)
template <int I>
__device__ __forceinline__ float magic15(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x47000000u, 0x7404u | (I << 4)));
}
template <int I>
__device__ __forceinline__ float magic7(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x43000000u, 0x7044u | (I << 8)));
}
// sign-extended byte i of w (selector nibbles with bit 3 set replicate the byte's sign)
// (the __byte_perm intrinsic keeps only 3 bits per selector nibble, so this goes through prmt.b32 itself)
__device__ __forceinline__ int sext_byte(uint32_t w, uint32_t sel4) {
    int d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0u), "r"(sel4));
    return d;
}
__host__ __device__ constexpr uint32_t sext_sel(uint32_t i) { return i | ((i | 8u) << 4) | ((i | 8u) << 8) | ((i | 8u) << 12); }

// Per-lane activation state for one unit (16 x values), held in registers for the whole kernel.
template <int FMT, int ACT>
struct UnitX {
    // f32 form: the 16 values as 8 pairs (operands of the packed f32x2 FMA)
    float2 v2[ACT == STRIX_ACT_F32 ? 8 : 1];
    // bias correction folded into the accumulator's start value:
    //   Q4_0: (128 + 8) * sum of the 16 x;  Q6_K: (128 + 32) * sum of each group of 4;  Q8_0: unused
    float corr[ACT == STRIX_ACT_F32 ? (FMT == FMT_Q6_K ? 4 : 1) : 1];
    // int8 form
    uint32_t q[ACT == STRIX_ACT_Q8DOT ? 4 : 1];
    float d[ACT == STRIX_ACT_Q8DOT ? (FMT == FMT_Q6_K ? 4 : 1) : 1];
    int qs[ACT == STRIX_ACT_Q8DOT ? (FMT == FMT_Q6_K ? 4 : 1) : 1];  // bias * sum of the int8 values
    // byte offsets of this unit's fields within a resident row
    uint32_t off_w, off_s, off_hh, off_sc;
    uint32_t sel_a, sel_b;  // Q6_K: sign-extending PRMT selectors of this unit's sub-scale bytes
};

__device__ __forceinline__ int quant1(float x, float inv) {
    int q = (int)rintf(x * inv);
    return max(-127, min(127, q));
}

template <int FMT, int ACT>
__device__ __forceinline__ void make_unit_x(UnitX<FMT, ACT> &X, const float (&v)[16], uint32_t u, const RowLayout &L) {
    if (FMT == FMT_Q8_0) {
        X.off_w = u * 16u;
        X.off_s = L.off_d + 2u * (u >> 1);
    } else if (FMT == FMT_Q4_0) {
        X.off_w = u * 8u;
        X.off_s = L.off_d + 2u * (u >> 1);
    } else {
        const uint32_t sb = u >> 4, r = u & 15u, h = r >> 3, c4 = r & 7u;
        X.off_w = sb * 128u + h * 64u + c4 * 4u;
        X.off_hh = L.off_qh + sb * 64u + h * 32u + c4 * 4u;
        X.off_sc = L.off_sc + sb * 16u + h * 8u;
        X.off_s = L.off_d + 2u * sb;
        X.sel_a = sext_sel(c4 >> 2);         // sub-scale byte (c4>>2)     of the word: groups 0 and 2
        X.sel_b = sext_sel((c4 >> 2) + 2u);  // sub-scale byte (c4>>2) + 2 of the word: groups 1 and 3
    }
    if (ACT == STRIX_ACT_F32) {
#pragma unroll
        for (int i = 0; i < 8; i++) X.v2[i] = make_float2(v[2 * i], v[2 * i + 1]);
        if (FMT == FMT_Q4_0) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) s += v[i];
            X.corr[0] = 136.0f * s;
        } else if (FMT == FMT_Q6_K) {
#pragma unroll
            for (int k = 0; k < 4; k++) X.corr[k] = 160.0f * ((v[4 * k] + v[4 * k + 1]) + (v[4 * k + 2] + v[4 * k + 3]));
        }
    } else {
        // per-32 quantiser (xquant8, kernels.rs:864-876): d = amax/127, inv = d>0 ? 1/d : 0,
        // q = clamp(rintf(x*inv)). The 32 elements of a block sit in 2 lanes (Q4_0, Q8_0)
        // or in the 8 lanes that share (sb, half) (Q6_K).
        if (FMT != FMT_Q6_K) {
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            float d = amax / 127.0f;
            float inv = d > 0.f ? 1.0f / d : 0.f;
            int sum = 0;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                int q0 = quant1(v[4 * g], inv), q1 = quant1(v[4 * g + 1], inv);
                int q2 = quant1(v[4 * g + 2], inv), q3 = quant1(v[4 * g + 3], inv);
                sum += q0 + q1 + q2 + q3;
                X.q[g] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                         ((uint32_t)(q3 & 0xff) << 24);
            }
            X.d[0] = d;
            X.qs[0] = 8 * sum;
        } else {
#pragma unroll
            for (int k = 0; k < 4; k++) {
                float amax = fmaxf(fmaxf(fabsf(v[4 * k]), fabsf(v[4 * k + 1])),
                                   fmaxf(fabsf(v[4 * k + 2]), fabsf(v[4 * k + 3])));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                float d = amax / 127.0f;
                float inv = d > 0.f ? 1.0f / d : 0.f;
                int q0 = quant1(v[4 * k], inv), q1 = quant1(v[4 * k + 1], inv);
                int q2 = quant1(v[4 * k + 2], inv), q3 = quant1(v[4 * k + 3], inv);
                X.q[k] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                         ((uint32_t)(q3 & 0xff) << 24);
                X.d[k] = d;
                X.qs[k] = 32 * (q0 + q1 + q2 + q3);
            }
        }
    }
}

// sum over 4 bytes of (2^k + byte_i) * x_i on two packed-f32x2 accumulators
template <bool M7>
__device__ __forceinline__ void fma4(uint32_t w, const float2 &xa, const float2 &xb, float2 &acc_a, float2 &acc_b) {
    float2 p, q;
    if (M7) {
        p = make_float2(magic7<0>(w), magic7<1>(w));
        q = make_float2(magic7<2>(w), magic7<3>(w));
    } else {
        p = make_float2(magic15<0>(w), magic15<1>(w));
        q = make_float2(magic15<2>(w), magic15<3>(w));
    }
    acc_a = __ffma2_rn(p, xa, acc_a);
    acc_b = __ffma2_rn(q, xb, acc_b);
}

// Contribution of one unit of one resident row to that row's dot product.
// `rb` = 32-bit shared address of the row's first byte.
template <int FMT, int ACT>
__device__ __forceinline__ float unit_dot(uint32_t rb, const UnitX<FMT, ACT> &X) {
    if (FMT == FMT_Q8_0) {
        const uint4 w = lds128(rb + X.off_w);
        const float d = lds_f16(rb + X.off_s);
        if (ACT == STRIX_ACT_F32) {
            // q + 128 is an unsigned byte; (32768 + 128 + q) - 32896 = q exactly, then packed FMAs
            const uint32_t ws[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
            const float2 bias = make_float2(-32896.0f, -32896.0f);
            float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);
#pragma unroll
            for (int g = 0; g < 4; g++) {
                float2 p = make_float2(magic15<0>(ws[g]), magic15<1>(ws[g]));
                float2 q = make_float2(magic15<2>(ws[g]), magic15<3>(ws[g]));
                p = __fadd2_rn(p, bias);
                q = __fadd2_rn(q, bias);
                acc_a = __ffma2_rn(p, X.v2[2 * g], acc_a);
                acc_b = __ffma2_rn(q, X.v2[2 * g + 1], acc_b);
            }
            return d * ((acc_a.x + acc_a.y) + (acc_b.x + acc_b.y));
        } else {
            int isum = dp4a_ss(w.x, X.q[0], 0);
            isum = dp4a_ss(w.y, X.q[1], isum);
            isum = dp4a_ss(w.z, X.q[2], isum);
            isum = dp4a_ss(w.w, X.q[3], isum);
            return (d * X.d[0]) * (float)isum;
        }
    } else if (FMT == FMT_Q4_0) {
        const uint2 w = lds64(rb + X.off_w);
        const float d = lds_f16(rb + X.off_s);
        const uint32_t lo0 = w.x & 0x0F0F0F0Fu, lo1 = w.y & 0x0F0F0F0Fu;
        const uint32_t hi0 = (w.x >> 4) & 0x0F0F0F0Fu, hi1 = (w.y >> 4) & 0x0F0F0F0Fu;
        if (ACT == STRIX_ACT_F32) {
            // sum((128 + nib) x) - 136 sum(x) = sum((nib - 8) x); the second term starts the accumulator
            float2 acc_a = make_float2(-X.corr[0], 0.f), acc_b = make_float2(0.f, 0.f);
            fma4<true>(lo0, X.v2[0], X.v2[1], acc_a, acc_b);
            fma4<true>(lo1, X.v2[2], X.v2[3], acc_a, acc_b);
            fma4<true>(hi0, X.v2[4], X.v2[5], acc_a, acc_b);
            fma4<true>(hi1, X.v2[6], X.v2[7], acc_a, acc_b);
            return d * ((acc_a.x + acc_a.y) + (acc_b.x + acc_b.y));
        } else {
            int isum = dp4a_us(lo0, X.q[0], -X.qs[0]);  // raw nibbles, minus 8 * sum(xq)
            isum = dp4a_us(lo1, X.q[1], isum);
            isum = dp4a_us(hi0, X.q[2], isum);
            isum = dp4a_us(hi1, X.q[3], isum);
            return (d * X.d[0]) * (float)isum;
        }
    } else {
        const uint32_t a = lds32(rb + X.off_w), b = lds32(rb + X.off_w + 32u), hh = lds32(rb + X.off_hh);
        const uint2 scw = lds64(rb + X.off_sc);  // the half's 8 sub-scales
        const float d = lds_f16(rb + X.off_s);
        const uint32_t qw[4] = {(a & 0x0F0F0F0Fu) | ((hh & 0x03030303u) << 4),
                                (b & 0x0F0F0F0Fu) | ((hh & 0x0C0C0C0Cu) << 2),
                                ((a >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u),
                                ((b >> 4) & 0x0F0F0F0Fu) | ((hh >> 2) & 0x30303030u)};
        const float sc[4] = {(float)sext_byte(scw.x, X.sel_a), (float)sext_byte(scw.x, X.sel_b),
                             (float)sext_byte(scw.y, X.sel_a), (float)sext_byte(scw.y, X.sel_b)};
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            if (ACT == STRIX_ACT_F32) {
                float2 acc_a = make_float2(-X.corr[k], 0.f), acc_b = make_float2(0.f, 0.f);
                fma4<true>(qw[k], X.v2[2 * k], X.v2[2 * k + 1], acc_a, acc_b);
                t = fmaf(sc[k], (acc_a.x + acc_a.y) + (acc_b.x + acc_b.y), t);
            } else {
                const int isum = dp4a_us(qw[k], X.q[k], -X.qs[k]);  // minus 32 * sum(xq)
                t = fmaf(sc[k] * X.d[k], (float)isum, t);
            }
        }
        return d * t;
    }
}

// Sums GEMV_RB (= 4) per-lane values across the warp with 6 shuffles instead of 20: lanes trade the
// halves they do not keep (xor 16, then xor 8), which leaves one row per lane, then a 3-step
// butterfly over xor 4/2/1. On return lane 8k (k = 0..3) holds the full sum of row k.
__device__ __forceinline__ float batch_reduce(const float (&v)[GEMV_RB], uint32_t lane) {
    static_assert(GEMV_RB == 4, "batch_reduce is written for 4 rows");
    const bool up16 = (lane & 16u) != 0u, up8 = (lane & 8u) != 0u;
    // after this step lanes 0-15 hold rows 0,1 and lanes 16-31 hold rows 2,3
    float k0 = up16 ? v[2] : v[0], s0 = up16 ? v[0] : v[2];
    float k1 = up16 ? v[3] : v[1], s1 = up16 ? v[1] : v[3];
    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    // lanes with bit 3 clear keep the even row of their pair, the others the odd one
    float k = up8 ? k1 : k0, sx = up8 ? k0 : k1;
    k += __shfl_xor_sync(0xffffffffu, sx, 8);
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

template <int FMT, int ACT, int NCH>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32, 1) gemv_kernel(const __grid_constant__ GemvArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);        // GEMV_MAX_STAGES barriers
    uint32_t *ctl = reinterpret_cast<uint32_t *>(smem + 64);    // [0] = abort flag
    float *red = reinterpret_cast<float *>(smem + 128);         // 32 floats: block reduction
    float *part = reinterpret_cast<float *>(smem + 256);        // 2 x rows_per_tile x wc partial sums
    uint8_t *stages = smem + 256 + ((2u * A.rows_per_tile * A.wc * 4u + 127u) & ~127u);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t S = A.n_stages, grid = gridDim.x, bid = blockIdx.x;
    const uint32_t my_n = (A.n_tiles > bid) ? (A.n_tiles - bid + grid - 1) / grid : 0;
    const RowLayout L = A.L;
    const uint32_t U = L.in_dim / 16u;

    if (tid == 0) {
        for (uint32_t s = 0; s < S; s++) mbar_init(&full[s], 1);
        ctl[0] = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Start the first S tile copies before the activation prologue so that they overlap it.
    if (tid == 0) {
        const uint32_t n0 = min(S, my_n);
        for (uint32_t i = 0; i < n0; i++) {
            TileRef t = tile_ref(A, bid + i * grid);
            const uint32_t bytes = t.rows * L.row_stride;
            mbar_arrive_expect_tx(&full[i], bytes);
            bulk_g2s(stages + (uint64_t)i * A.stage_bytes, t.src, bytes, &full[i]);
        }
    }

    // ---- activation prologue: this lane's x values, kept in registers for the whole kernel ----
    float scale = 1.0f;
    if (A.pre == STRIX_PRE_RMSNORM) {
        // rmsnorm (crates/strix-backend-cpu/src/qwen3.rs:107-114): x * (1/sqrt(mean(x^2)+eps)) * w
        float ss = 0.f;
        for (uint32_t i = tid; i < L.in_dim; i += blockDim.x) {
            float t = __ldg(A.a + i);
            ss = fmaf(t, t, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (uint32_t w = 0; w < (blockDim.x >> 5); w++) tot += red[w];
        scale = 1.0f / sqrtf(tot / (float)L.in_dim + A.eps);
    }
    const uint32_t cw = warp % A.wc, slot = warp / A.wc;
    UnitX<FMT, ACT> X[NCH];
#pragma unroll
    for (int c = 0; c < NCH; c++) {
        const uint32_t u = (cw + (uint32_t)c * A.wc) * 32u + lane;
        const bool valid = u < U;
        float v[16];
#pragma unroll
        for (uint32_t g = 0; g < 4; g++) {
            float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (valid) {
                const uint32_t e = unit_elem<FMT>(u, g);
                a4 = __ldg(reinterpret_cast<const float4 *>(A.a + e));
                if (A.pre != STRIX_PRE_NONE) {
                    const float4 b4 = __ldg(reinterpret_cast<const float4 *>(A.b + e));
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
            }
            v[4 * g] = a4.x; v[4 * g + 1] = a4.y; v[4 * g + 2] = a4.z; v[4 * g + 3] = a4.w;
        }
        make_unit_x<FMT, ACT>(X[c], v, u, L);
    }

    // ---- stream the tiles ----
    uint32_t buf = 0;
    bool aborted = false;
    uint32_t i = 0;
    for (; i < my_n; i++) {
        const uint32_t s = i % S, ph = (i / S) & 1u;
        const bool ok = mbar_wait_bounded(&full[s], ph, A.status);
        if (!ok) ctl[0] = 1;
        const TileRef t = tile_ref(A, bid + i * grid);
        float *pp = part + buf * (A.rows_per_tile * A.wc);
        if (ok) {
            const uint32_t st = smem_u32(stages) + s * A.stage_bytes;
            // A slot works on GEMV_RB consecutive rows at a time: RB independent load/dot chains per
            // lane, then one transposed warp reduction for the whole batch. Rows past the tile's end
            // read whatever the stage still holds from an earlier tile; their sums are dropped below.
            for (uint32_t r0 = slot * GEMV_RB; r0 < t.rows; r0 += A.slots * GEMV_RB) {
                float acc[GEMV_RB];
#pragma unroll
                for (int j = 0; j < GEMV_RB; j++) acc[j] = 0.f;
                const uint32_t rb0 = st + r0 * L.row_stride;
#pragma unroll
                for (int c = 0; c < NCH; c++) {
                    const uint32_t u = (cw + (uint32_t)c * A.wc) * 32u + lane;
                    if (u < U) {
#pragma unroll
                        for (int j = 0; j < GEMV_RB; j++)
                            acc[j] += unit_dot<FMT, ACT>(rb0 + (uint32_t)j * L.row_stride, X[c]);
                    }
                }
                const float tot = batch_reduce(acc, lane);
                // lane 8k now holds the sum of row r0 + k
                const uint32_t rr = r0 + (lane >> 3);
                if ((lane & 7u) == 0u && rr < t.rows) pp[rr * A.wc + cw] = tot;
            }
        }
        __syncthreads();
        if (ctl[0]) { aborted = true; break; }
        if (tid == 0 && i + S < my_n) {
            // the stage is drained (barrier above): refill it with the tile S steps ahead
            fence_proxy_async_smem();
            TileRef n = tile_ref(A, bid + (i + S) * grid);
            const uint32_t bytes = n.rows * L.row_stride;
            mbar_arrive_expect_tx(&full[s], bytes);
            bulk_g2s(stages + (uint64_t)s * A.stage_bytes, n.src, bytes, &full[s]);
        }
        if (tid < t.rows) {
            float sum = 0.f;
            for (uint32_t c = 0; c < A.wc; c++) sum += pp[tid * A.wc + c];
            A.mat[t.mat].y[t.row0 + tid] = sum;
        }
        buf ^= 1u;
    }
    if (aborted && tid == 0) {
        // Copies already issued for later tiles are still in flight: give them a bounded
        // chance to land before the CTA's shared memory is released.
        for (uint32_t j = i + 1; j < min(my_n, i + S); j++) mbar_wait_bounded(&full[j % S], (j / S) & 1u, nullptr);
    }
}

// ------------------------------------------------------------------ host side
static inline uint32_t align128u(uint32_t v) { return (v + 127u) & ~127u; }

bool gemv_plan(GemvArgs &a, int num_sms, size_t smem_optin) {
    const uint32_t K = a.L.in_dim;
    if (K == 0 || K % 32 != 0) return false;
    const uint32_t U = K / 16, C = (U + 31) / 32;
    const uint32_t nch = (C + GEMV_MAX_WARPS - 1) / GEMV_MAX_WARPS;
    if (nch > 4) return false;
    const uint32_t wc = (C + nch - 1) / nch;
    const uint32_t slots = GEMV_MAX_WARPS / wc > 0 ? GEMV_MAX_WARPS / wc : 1;
    const uint32_t stride = a.L.row_stride;
    const uint32_t budget = (uint32_t)smem_optin - 1024u;

    // A tile is a whole number of row batches for every slot: a multiple of slots * GEMV_RB rows,
    // about 24-48 KB, capped at 160 rows. Among candidate heights pick the one with the least
    // work on the busiest CTA (bytes streamed plus a fixed charge per tile).
    const uint32_t quantum = slots * GEMV_RB;
    uint32_t mmax = 40960u / (quantum * stride);
    if (mmax < 1) mmax = 1;
    while (mmax > 1 && mmax * quantum > 160) mmax--;
    uint32_t best_rt = quantum;
    uint64_t best_cost = ~0ull;
    for (uint32_t m = mmax; m >= 1 && 2 * m >= mmax; m--) {
        const uint32_t rt = m * quantum;
        uint64_t tiles = 0;
        for (int k = 0; k < a.nmat; k++) tiles += (a.mat[k].rows + rt - 1) / rt;
        if (tiles == 0) tiles = 1;
        const uint64_t per_cta = (tiles + (uint64_t)num_sms - 1) / (uint64_t)num_sms;
        const uint64_t cost = per_cta * ((uint64_t)rt * stride + 2048u);
        if (cost < best_cost) { best_cost = cost; best_rt = rt; }
    }
    const uint32_t rt = best_rt;
    uint32_t tile = 0;
    for (int m = 0; m < a.nmat; m++) {
        a.mat[m].tile0 = tile;
        tile += (a.mat[m].rows + rt - 1) / rt;
    }
    a.n_tiles = tile;
    a.rows_per_tile = rt;
    a.wc = wc;
    a.slots = slots;
    a.nch = nch;
    const uint32_t stage_off = 256u + align128u(2u * rt * wc * 4u);
    a.stage_bytes = align128u(rt * stride);
    if (budget < stage_off + 2u * a.stage_bytes) return false;
    uint32_t S = (budget - stage_off) / a.stage_bytes;
    if (S > GEMV_MAX_STAGES) S = GEMV_MAX_STAGES;
    a.n_stages = S;
    a.smem_bytes = stage_off + S * a.stage_bytes;
    a.grid = a.n_tiles < (uint32_t)num_sms ? a.n_tiles : (uint32_t)num_sms;
    return true;
}

template <int FMT, int ACT, int NCH>
static cudaError_t launch_t(const GemvArgs &a, cudaStream_t stream) {
    const uint32_t threads = a.wc * a.slots * 32u;
    gemv_kernel<FMT, ACT, NCH><<<a.grid, threads, a.smem_bytes, stream>>>(a);
    return cudaGetLastError();
}

template <int FMT, int ACT>
static cudaError_t launch_nch(const GemvArgs &a, cudaStream_t stream) {
    switch (a.nch) {
        case 1: return launch_t<FMT, ACT, 1>(a, stream);
        case 2: return launch_t<FMT, ACT, 2>(a, stream);
        case 3: return launch_t<FMT, ACT, 3>(a, stream);
        default: return launch_t<FMT, ACT, 4>(a, stream);
    }
}

template <int FMT>
static cudaError_t launch_act(const GemvArgs &a, cudaStream_t stream) {
    return a.act == STRIX_ACT_Q8DOT ? launch_nch<FMT, STRIX_ACT_Q8DOT>(a, stream)
                                    : launch_nch<FMT, STRIX_ACT_F32>(a, stream);
}

cudaError_t launch_gemv(const GemvArgs &a, cudaStream_t stream) {
    if (a.n_tiles == 0) return cudaSuccess;
    switch (a.L.fmt) {
        case FMT_Q4_0: return launch_act<FMT_Q4_0>(a, stream);
        case FMT_Q8_0: return launch_act<FMT_Q8_0>(a, stream);
        default: return launch_act<FMT_Q6_K>(a, stream);
    }
}

template <int FMT, int ACT, int NCH>
static cudaError_t optin_one(size_t bytes) {
    return cudaFuncSetAttribute(gemv_kernel<FMT, ACT, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}
template <int FMT, int ACT>
static cudaError_t optin_nch(size_t b) {
    cudaError_t e;
    if ((e = optin_one<FMT, ACT, 1>(b)) != cudaSuccess) return e;
    if ((e = optin_one<FMT, ACT, 2>(b)) != cudaSuccess) return e;
    if ((e = optin_one<FMT, ACT, 3>(b)) != cudaSuccess) return e;
    return optin_one<FMT, ACT, 4>(b);
}
template <int FMT>
static cudaError_t optin_fmt(size_t b) {
    cudaError_t e = optin_nch<FMT, STRIX_ACT_F32>(b);
    return e != cudaSuccess ? e : optin_nch<FMT, STRIX_ACT_Q8DOT>(b);
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
