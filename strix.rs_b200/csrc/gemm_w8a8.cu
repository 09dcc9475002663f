// W8A8 prefill GEMM for sm_100a: Q8_0 weights x per-32 int8 activations on tcgen05
// int8 MMA with TMEM accumulators fed by TMA.
//
//   Y[m][n] = sum_kb  d_w[n,kb] * d_x[m,kb] * (float) isum[m,n,kb],
//   isum[m,n,kb] = sum_{i<32} W[n,kb,i] * X[m,kb,i]          (int32, exact)
//
// Replaces the reference's xquant8_rows + q8w_gemm32 / q8w_gemm
// (crates/strix-backend-rocm/src/kernels.rs:1000-1013, 1308-1443; dispatch
// decode.rs:1742-1766, entry decode.rs:3257-3297) and the split-K form of its
// prefill GEMM (kernels.rs:539-601).
//
// Both operands carry a scale per 32 elements of K, so the int32 sum of one
// K-block cannot be carried into the next: every tcgen05.mma (K = 32 for int8)
// writes a FRESH accumulator, and CUDA cores fold it into f32 with the two
// scales. The kernel is organised around that drain:
//   * CTA tile 128 tokens x 128 weight rows; warp 0 issues TMA loads (activations
//     and weights as 128-byte-swizzled K-major tiles, the K-block's weight scales
//     as an f32 row), warp 1 issues one MMA per K-block into one of four
//     128-column TMEM buffers and commits it to an mbarrier;
//   * sixteen epilogue warps (TMEM lane group = warp % 4, column quarter = index / 4)
//     read a finished buffer with tcgen05.ld, re-arm it, hand it back, and run
//     acc[n] += d_w[n] * (d_x[m] * isum) as packed f32x2 ops, 32 columns per thread;
//   * int32 -> f32 costs no conversion instruction: the integer r = isum + 128 * sum(x codes) that
//     comes back from TMEM (weight codes are resident as q + 128, the MMA runs u8 x s8) is ADDED to
//     the bit pattern of 1.5 * 2^23 (an integer add, off the FMA pipe), which is the float
//     12582912 + r. The quantiser leaves c = -d_x * (12582912 + 128 * sum) per (token, K-block),
//     so d_x * isum = fma(d_x, 12582912 + r, c): TWO packed FMAs per pair of elements (this one and
//     the accumulation with d_w). The MMA overwrites its buffer (no accumulator input), so a
//     drained buffer needs nothing written into it and goes back to the MMA warp as soon as its
//     contents are in registers: the hand-over, not the arithmetic, is what bounds this kernel
//     (four buffers of 128 columns are all of TMEM, and an MMA takes ~500 clocks from issue to
//     completion). c is rounded once, which moves
//     each block term by at most 0.75 d_x, i.e. ~1e-5 of a typical block sum, against a contract of
//     1e-3; the bit-exact tier (MODE 1 below) recovers isum with the exact subtract;
//   * the kernel is a template over MODE: 0 = the product path; 1 = the SAME producer / MMA / TMEM
//     pipeline with an epilogue that stores every int32 block sum isum[m][n][kb] (the bit-exact
//     tier of the contract, checked on the tensor-core path itself); 2 = the epilogue only hands
//     the buffers back (no TMEM read, no arithmetic): what the TMA + tensor pipeline sustains
//     without the drain; 3 = as 2 and no loads either (operands stay whatever shared memory
//     holds): the MMA issue loop with its buffer hand-overs but no data movement; 4 = the MMAs alone,
//     issued back to back by one thread with a single commit at the end: the measured int8 peak;
//   * split-K (grid.z) writes f32 partials that a second kernel adds in a fixed
//     order: reproducible, unlike the reference's atomicAdd;
//   * every wait is bounded; after a timeout nothing waits again, the status word
//     is raised, and the CTA still frees its TMEM before it returns.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace strix {

constexpr uint32_t GM_BM = 128, GM_BN = 128;      // CTA tile: tokens x weight rows
constexpr uint32_t GM_KB_STAGE = 4;               // K-blocks (of 32) per shared-memory stage = one 128-byte atom
constexpr uint32_t GM_STAGES = 5;
constexpr uint32_t GM_TBUF = 4;                   // TMEM accumulator buffers of GM_BN columns
constexpr uint32_t GM_A_BYTES = GM_BM * 128, GM_B_BYTES = GM_BN * 128, GM_S_BYTES = GM_KB_STAGE * GM_BN * 4;
constexpr uint32_t GM_XD_BYTES = GM_BM * GM_KB_STAGE * 4;  // [K-block][token]: activation scales / un-bias terms (MODE 1: code sums)
constexpr uint32_t GM_OFF_S = GM_A_BYTES + GM_B_BYTES, GM_OFF_XD = GM_OFF_S + GM_S_BYTES, GM_OFF_XS = GM_OFF_XD + GM_XD_BYTES;
constexpr uint32_t GM_STAGE_BYTES = GM_OFF_XS + GM_XD_BYTES;  // 38912 = 38 KB
constexpr uint32_t GM_EPI_WARPS = 16, GM_EPI_WARP0 = 2, GM_THREADS = (GM_EPI_WARP0 + GM_EPI_WARPS) * 32;
constexpr uint32_t GM_MAGIC = 0x4B400000u;  // bits of 12582912.0f = 1.5 * 2^23: ulp 1, room for |isum| < 2^22
static_assert(GM_KB_STAGE == GM_TBUF, "a TMEM buffer is reused by the same K-block slot of the next stage");
constexpr uint32_t GM_SMEM = 1024 /* barriers */ + GM_STAGES * GM_STAGE_BYTES + 1024 /* alignment slack */;

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] = A[smem desc] * B[smem desc], int8 inputs, int32 result (the accumulator input is disabled: every
// K-block gets a fresh sum, and nothing has to be written into the buffer before it is used again).
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): start address >> 4,
// leading byte offset 1 (ignored for swizzled K-major), stride byte offset = 8 rows x 128 B = 1024
// (>> 4 = 64), descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B). The tile base must
// be 1024-byte aligned. Stepping 32 bytes along K inside the atom adds 2 to the start field.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)1u << 16;
    d |= (uint64_t)64u << 32;
    d |= (uint64_t)1u << 46;
    d |= (uint64_t)2u << 61;
    return d;
}
// Instruction descriptor (kind::i8): D = s32 (bits 4-5 = 2), A = signed int8 (bits 7-9 = 1),
// B = unsigned int8 (bits 10-12 = 0), both K-major (bits 15, 16 = 0), N >> 3 in bits 17-22,
// M >> 4 in bits 24-28.
constexpr uint32_t GM_IDESC = (2u << 4) | (1u << 7) | (0u << 10) | ((GM_BN >> 3) << 17) | ((GM_BM >> 4) << 24);

struct GemmArgs {
    float *y;           // [splits][M][ldy] (splits > 1: partials) or [M][ldy]
    uint32_t M, N, nb, ldy, ldx;  // ldx: leading dimension of xs / xd (nb rounded up to 4: TMA strides are multiples of 16 B)
    uint32_t kb_per_split;  // K-blocks per grid.z slice, a multiple of GM_KB_STAGE
    int32_t *dump;          // MODE 1: isum[M][N][nb]
    uint32_t *status;
};

template <int MODE>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_w8a8_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_xd,
                 const __grid_constant__ CUtensorMap map_xs, const __grid_constant__ GemmArgs A) {
    extern __shared__ uint8_t smem_raw[];
    // barriers in the first KB, stages from the next 1024-byte boundary (the swizzle atom wants it)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);             // [GM_STAGES] TMA landed
    uint64_t *empty = full + GM_STAGES;                              // [GM_STAGES] MMA + epilogue done with the stage
    uint64_t *tfull = empty + GM_STAGES;                             // [GM_TBUF] MMA result ready in TMEM
    uint64_t *tempty = tfull + GM_TBUF;                              // [GM_TBUF] epilogue has read the buffer
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + GM_TBUF);
    volatile uint32_t *ctl = tmem_slot + 1;
    uint8_t *stages = smem + 1024;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t n0 = blockIdx.x * GM_BN, m0 = blockIdx.y * GM_BM;
    const uint32_t kb0 = blockIdx.z * A.kb_per_split;
    const uint32_t kb1 = min(A.nb, kb0 + A.kb_per_split);
    const uint32_t n_stage_iters = (kb1 - kb0 + GM_KB_STAGE - 1) / GM_KB_STAGE;

    if (tid == 0) {
        for (uint32_t s = 0; s < GM_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1 + GM_EPI_WARPS);
        }
        for (uint32_t b = 0; b < GM_TBUF; b++) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], GM_EPI_WARPS);
        }
        *ctl = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        // 512 columns = four accumulator buffers; this CTA is alone on its SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(GM_TBUF * GM_BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (MODE == 4) {
        // measurement: the bare issue rate of tcgen05.mma kind::i8 - one thread issues this CTA's MMAs back to back
        // on whatever shared memory holds, into the four buffers in turn, with one commit at the end
        if (warp == 1 && lane == 0) {
            const uint32_t sa = smem_u32(stages);
            const uint64_t adesc = smem_desc_sw128(sa), bdesc = smem_desc_sw128(sa + GM_A_BYTES);
            if (A.dump) {
                // (A.dump non-null: every MMA is committed and waited for before the next one: its issue-to-completion latency)
                for (uint32_t g = 0; g < kb1 - kb0; g++) {
                    tc_mma_i8(tmem_base + (g % GM_TBUF) * GM_BN, adesc + 2u * (g & 3u), bdesc + 2u * (g & 3u), GM_IDESC);
                    tc_commit(&tfull[0]);
                    mbar_wait_bounded(&tfull[0], g & 1u, A.status);
                }
            } else {
                for (uint32_t g = 0; g < kb1 - kb0; g++) tc_mma_i8(tmem_base + (g % GM_TBUF) * GM_BN, adesc + 2u * (g & 3u), bdesc + 2u * (g & 3u), GM_IDESC);
                tc_commit(&tfull[0]);
                mbar_wait_bounded(&tfull[0], 0u, A.status);
            }
        }
    } else if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (uint32_t it = 0; it < n_stage_iters; it++) {
                const uint32_t s = it % GM_STAGES;
                if (it >= GM_STAGES && !*ctl && !mbar_wait_bounded(&empty[s], ((it / GM_STAGES) - 1u) & 1u, A.status))
                    *ctl = 1;
                uint8_t *st = stages + s * GM_STAGE_BYTES;
                const uint32_t kb = kb0 + it * GM_KB_STAGE;
                if (MODE == 3) {
                    mbar_arrive(&full[s]);  // nothing is loaded: the phase completes at once
                    continue;
                }
                mbar_arrive_expect_tx(&full[s], GM_STAGE_BYTES);
                tma_load_2d(st, &map_x, (int)(kb * 32u), (int)m0, &full[s]);
                tma_load_2d(st + GM_A_BYTES, &map_w, (int)(kb * 32u), (int)n0, &full[s]);
                tma_load_2d(st + GM_OFF_S, &map_s, (int)n0, (int)kb, &full[s]);
                tma_load_2d(st + GM_OFF_XD, &map_xd, (int)m0, (int)kb, &full[s]);
                tma_load_2d(st + GM_OFF_XS, &map_xs, (int)m0, (int)kb, &full[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t g = 0;  // K-block counter of this CTA
            uint32_t aborted = 0;  // (once a wait has run out nobody waits again; other warps learn it through *ctl)
            for (uint32_t it = 0; it < n_stage_iters; it++) {
                if ((it & 7u) == 7u) aborted |= *ctl;
                const uint32_t s = it % GM_STAGES;
                if (!aborted && !mbar_wait_bounded(&full[s], (it / GM_STAGES) & 1u, A.status)) *ctl = aborted = 1;
                tc_fence_after();
                const uint32_t sa = smem_u32(stages + s * GM_STAGE_BYTES);
                const uint64_t adesc = smem_desc_sw128(sa), bdesc = smem_desc_sw128(sa + GM_A_BYTES);
                const uint32_t nkb = min(GM_KB_STAGE, kb1 - (kb0 + it * GM_KB_STAGE));
                for (uint32_t j = 0; j < nkb; j++, g++) {
                    const uint32_t buf = g % GM_TBUF, use = g / GM_TBUF;
                    // the epilogue warps pre-load every buffer (first use included) before it may be accumulated into
                    if (!aborted && !mbar_wait_bounded(&tempty[buf], use & 1u, A.status)) *ctl = aborted = 1;
                    tc_fence_after();
                    tc_mma_i8(tmem_base + buf * GM_BN, adesc + 2u * j, bdesc + 2u * j, GM_IDESC);
                    tc_commit(&tfull[buf]);  // arrives when this MMA (and all before it) has completed
                }
                tc_commit(&empty[s]);  // the stage's operand tiles are no longer being read
            }
        }
    } else {
        // ---------------- epilogue: drain TMEM, apply the block scales ----------------
        const uint32_t lg = warp & 3u, cq = (warp - GM_EPI_WARP0) >> 2;  // TMEM lane group (fixed by warp % 4), column quarter
        const uint32_t m = m0 + lg * 32u + lane;                         // this thread's token
        const bool m_ok = m < A.M;
        const uint32_t taddr0 = tmem_base + ((lg * 32u) << 16) + cq * 32u;
        const uint32_t trow = lg * 32u + lane;  // this thread's row in the tile
        // the four buffers start out free
        if (lane == 0)
            for (uint32_t j = 0; j < GM_TBUF; j++) mbar_arrive(&tempty[j]);
        float2 acc[16];
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = make_float2(0.f, 0.f);
        uint32_t aborted = 0;
        for (uint32_t it = 0; it < n_stage_iters; it++) {
            const uint32_t s = it % GM_STAGES;
            const uint32_t kb = kb0 + it * GM_KB_STAGE;
            aborted |= *ctl;
            if (!aborted && !mbar_wait_bounded(&full[s], (it / GM_STAGES) & 1u, A.status)) *ctl = aborted = 1;
            const uint8_t *stg = stages + s * GM_STAGE_BYTES;
            const float *sw = reinterpret_cast<const float *>(stg + GM_OFF_S) + cq * 32u;
            // [K-block][token]: consecutive lanes read consecutive words
            const float *sxd = reinterpret_cast<const float *>(stg + GM_OFF_XD) + trow;
            const float *sxc = reinterpret_cast<const float *>(stg + GM_OFF_XS) + trow;
            const uint32_t nkb = min(GM_KB_STAGE, kb1 - kb);  // uniform across the CTA
#pragma unroll 1
            for (uint32_t j = 0; j < nkb; j++) {
                if (MODE >= 2) {
                    // measurement: the buffer goes straight back (no TMEM read, no arithmetic)
                    if (!aborted && !mbar_wait_bounded(&tfull[j], it & 1u, A.status)) *ctl = aborted = 1;
                    tc_fence_after();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tempty[j]);
                    continue;
                }
                // this token's scale and un-bias term for the K-block (rows past M were zero-filled by TMA)
                const float dxj = sxd[j * GM_BM];
                const float cj = sxc[j * GM_BM];
                if (!aborted && !mbar_wait_bounded(&tfull[j], it & 1u, A.status)) *ctl = aborted = 1;
                tc_fence_after();
                uint32_t r[32];
                tc_ld32(taddr0 + j * GM_BN, r);
                tc_wait_ld();
                // the sums are in registers: the buffer goes back to the MMA warp before the arithmetic, not after it
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty[j]);
                if (MODE == 1) {
                    // bit-exact tier: r = isum + 128 * sum(x codes) as an integer (weight codes are resident as q + 128);
                    // the K-block's code sum arrives where the product path has c
                    const int32_t off = 128 * __float_as_int(cj);
                    if (m_ok) {
#pragma unroll
                        for (int q = 0; q < 32; q++) {
                            const uint32_t n = n0 + cq * 32u + (uint32_t)q;
                            if (n < A.N) A.dump[((uint64_t)m * A.N + n) * A.nb + kb + j] = (int32_t)r[q] - off;
                        }
                    }
                } else {
                    // int -> float without the conversion unit: adding the integer to the bit pattern of 1.5 * 2^23 gives
                    // the float 12582912 + r (|r| < 2^22); acc[n] += d_w[n] * (d_x * isum), d_x * isum = fma(d_x, 12582912 + r, c)
                    const float2 dx2 = make_float2(dxj, dxj), c2 = make_float2(cj, cj);
                    const float4 *swj = reinterpret_cast<const float4 *>(sw + j * GM_BN);
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const float4 w4 = swj[q];
                        const float2 g0 = __ffma2_rn(dx2, make_float2(__uint_as_float(r[4 * q] + GM_MAGIC), __uint_as_float(r[4 * q + 1] + GM_MAGIC)), c2);
                        const float2 g1 = __ffma2_rn(dx2, make_float2(__uint_as_float(r[4 * q + 2] + GM_MAGIC), __uint_as_float(r[4 * q + 3] + GM_MAGIC)), c2);
                        acc[2 * q] = __ffma2_rn(make_float2(w4.x, w4.y), g0, acc[2 * q]);
                        acc[2 * q + 1] = __ffma2_rn(make_float2(w4.z, w4.w), g1, acc[2 * q + 1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);  // done with the stage's scale rows
        }
        // write this thread's 32 outputs (one token, 32 consecutive weight rows)
        if (MODE == 0 && m_ok) {
            float *yrow = A.y + ((uint64_t)blockIdx.z * A.M + m) * A.ldy + n0 + cq * 32u;
            const uint32_t nleft = (A.N > n0 + cq * 32u) ? A.N - (n0 + cq * 32u) : 0u;
            if (nleft >= 32u && (A.ldy & 3u) == 0u) {
#pragma unroll
                for (int i = 0; i < 8; i++)
                    reinterpret_cast<float4 *>(yrow)[i] = make_float4(acc[2 * i].x, acc[2 * i].y, acc[2 * i + 1].x, acc[2 * i + 1].y);
            } else {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    if (2u * i < nleft) yrow[2 * i] = acc[i].x;
                    if (2u * i + 1u < nleft) yrow[2 * i + 1] = acc[i].y;
                }
            }
        }
    }
    // ---------------- teardown: every warp arrives; TMEM goes back before the CTA ends ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(GM_TBUF * GM_BN)
                     : "memory");
    }
}

// y[m][n] = sum over splits of part[z][m][n], in z order.
__global__ void splitk_reduce_kernel(const float *__restrict__ part, float *__restrict__ y, uint32_t M, uint32_t N,
                                     uint32_t ldp, uint32_t splits) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)M * N) return;
    const uint32_t m = (uint32_t)(i / N), n = (uint32_t)(i % N);
    float s = 0.f;
    for (uint32_t z = 0; z < splits; z++) s += part[((uint64_t)z * M + m) * ldp + n];
    y[(uint64_t)m * N + n] = s;
}

// Activation quantiser for the GEMM (xquant8_rows, kernels.rs:1000-1013) that also emits, per block, the
// sum of the codes and the un-bias term the GEMM's epilogue adds: c = -d * (12582912 + 128 * sum).
// One warp per 32-element block. d / xs / xc are [nb][ldm] (K-block major: a GEMM stage fetches the
// values of 128 consecutive tokens for 4 K-blocks as one box).
__global__ void xquant8_sum_kernel(const float *__restrict__ x, int8_t *__restrict__ q, float *__restrict__ d,
                                   int32_t *__restrict__ xs, float *__restrict__ xc, uint32_t nblk, uint32_t nb,
                                   uint32_t ldm) {
    const uint32_t blk = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    if (blk >= nblk) return;
    const uint32_t o = (blk % nb) * ldm + blk / nb;
    const float v = x[(uint64_t)blk * 32u + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax / 127.0f;
    const float inv = sc > 0.f ? 1.0f / sc : 0.f;
    int qi = (int)rintf(v * inv);
    qi = max(-127, min(127, qi));
    q[(uint64_t)blk * 32u + lane] = (int8_t)qi;
    int sum = qi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) {
        d[o] = sc;
        xs[o] = sum;
        xc[o] = -sc * (12582912.0f + 128.0f * (float)sum);  // the sum in brackets is an integer below 2^24: exact
    }
}

// f32 copy of a Q8_0 weight's scales, transposed to [nb][lds] so that one K-block's scales for
// 128 consecutive rows are one contiguous run (what the GEMM's TMA box fetches).
__global__ void scales_transpose_kernel(const uint8_t *__restrict__ res, float *__restrict__ out, RowLayout L,
                                        uint32_t rows, uint32_t lds) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)L.nb * lds) return;
    const uint32_t kb = (uint32_t)(i / lds), n = (uint32_t)(i % lds);
    float v = 0.f;
    if (n < rows) v = f16_bits_to_f32(resident_scale_bits(res, L, n, kb));
    out[i] = v;
}

// Q4_0 weights for the same GEMM (the reference's q4_gemm_w bakes the nibbles into signed bytes while it
// stages them, kernels.rs:443-537): the codes once more, row-major [rows][in_dim], one byte each as
// (nibble - 8) + 128 - the Q8_0 convention, so that the kernel, its un-bias term and the block scales are
// the same. Built on the first GEMM with the weight, from the resident tile-major form.
__global__ void expand_q4_codes_kernel(const uint8_t *__restrict__ res, uint8_t *__restrict__ out, RowLayout L, uint32_t rows) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 4 codes
    const uint64_t total = (uint64_t)rows * L.in_dim / 4u;
    if (i >= total) return;
    const uint32_t row = (uint32_t)(i / (L.in_dim / 4u)), k = (uint32_t)(i % (L.in_dim / 4u)) * 4u;
    uint32_t w = 0;
#pragma unroll
    for (uint32_t j = 0; j < 4; j++) w |= (resident_code(res, L, row, k + j) + 120u) << (8u * j);
    reinterpret_cast<uint32_t *>(out)[i] = w;
}

cudaError_t launch_expand_q4_codes(const uint8_t *d_res, uint8_t *d_out, const RowLayout &L, uint32_t rows, cudaStream_t stream) {
    const uint64_t total = (uint64_t)rows * L.in_dim / 4u;
    if (total == 0) return cudaSuccess;
    expand_q4_codes_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(d_res, d_out, L, rows);
    return cudaGetLastError();
}

// int32 block sums isum[m][n][kb] of a Q8_0 weight with int8 activations, one thread each:
// the bit-exact tier of the GEMM contract, computed the plain way (no tensor cores).
// `codes`: the weight's codes row-major [rows][in_dim], stored as q + 128.
__global__ void block_isums_kernel(const uint8_t *__restrict__ codes, const int8_t *__restrict__ xq, int32_t *__restrict__ out,
                                   RowLayout L, uint32_t M, uint32_t rows) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)M * rows * L.nb) return;
    const uint32_t kb = (uint32_t)(i % L.nb);
    const uint32_t n = (uint32_t)((i / L.nb) % rows), m = (uint32_t)(i / ((uint64_t)L.nb * rows));
    const uint8_t *w = codes + (uint64_t)n * L.in_dim + (uint64_t)kb * 32u;
    const int8_t *x = xq + (uint64_t)m * L.in_dim + (uint64_t)kb * 32u;
    int s = 0;
    for (int k = 0; k < 32; k++) s += ((int)w[k] - 128) * (int)x[k];
    out[i] = s;
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static bool make_map_2d(CUtensorMap *map, CUtensorMapDataType dt, void *base, uint64_t dim0, uint64_t dim1,
                        uint64_t stride1_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {dim0, dim1};
    cuuint64_t strides[1] = {stride1_bytes};
    cuuint32_t box[2] = {box0, box1};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

uint32_t gemm_scales_ld(uint32_t rows) { return (rows + 3u) & ~3u; }

cudaError_t launch_scales_transpose(const uint8_t *d_res, float *d_out, const RowLayout &L, uint32_t rows,
                                    cudaStream_t stream) {
    const uint32_t lds = gemm_scales_ld(rows);
    const uint64_t total = (uint64_t)L.nb * lds;
    if (total == 0) return cudaSuccess;
    scales_transpose_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(d_res, d_out, L, rows, lds);
    return cudaGetLastError();
}

uint32_t gemm_x_ld(uint32_t m) { return (m + 3u) & ~3u; }

// x[m][nb*32] -> q[m][nb*32] int8 and, K-block major with ldm = gemm_x_ld(m): d[nb][ldm] f32 block scales,
// xs[nb][ldm] int32 code sums, xc[nb][ldm] f32 un-bias terms
cudaError_t launch_xquant8_sum(const float *d_x, int8_t *d_q, float *d_d, int32_t *d_xs, float *d_xc, uint32_t m,
                               uint32_t nb, cudaStream_t stream) {
    const uint64_t nblk = (uint64_t)m * nb;
    if (nblk == 0) return cudaSuccess;
    const uint32_t T = 256, per = T / 32;
    xquant8_sum_kernel<<<(unsigned)((nblk + per - 1) / per), T, 0, stream>>>(d_x, d_q, d_d, d_xs, d_xc, (uint32_t)nblk, nb,
                                                                               gemm_x_ld(m));
    return cudaGetLastError();
}

cudaError_t launch_block_isums(const uint8_t *d_res, const int8_t *d_xq, int32_t *d_out, const RowLayout &L, uint32_t M,
                               uint32_t rows, cudaStream_t stream) {
    const uint64_t total = (uint64_t)M * rows * L.nb;
    if (total == 0) return cudaSuccess;
    block_isums_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(d_res, d_xq, d_out, L, M, rows);
    return cudaGetLastError();
}

cudaError_t gemm_prepare_device() {
    cudaError_t e = cudaFuncSetAttribute(gemm_w8a8_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GM_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_w8a8_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GM_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_w8a8_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GM_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_w8a8_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GM_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_w8a8_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GM_SMEM);
    // the small kernels of the GEMM path: asking for their attributes makes the driver load their code now
    // (module loading is lazy), so that a later call that must not allocate finds everything in place
    cudaFuncAttributes fa;
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, xquant8_sum_kernel);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, scales_transpose_kernel);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, splitk_reduce_kernel);
    return e;
}

uint32_t gemm_pick_splits(uint32_t M, uint32_t rows, uint32_t nb, int num_sms) {
    // Split K when the output tiles alone leave most SMs idle (ffn_down: few rows, long K).
    const uint32_t tiles = ((M + GM_BM - 1) / GM_BM) * ((rows + GM_BN - 1) / GM_BN);
    const uint32_t stages = (nb + GM_KB_STAGE - 1) / GM_KB_STAGE;
    uint32_t splits = 1;
    while (tiles * splits * 2 <= (uint32_t)num_sms && splits * 2 <= stages && splits < 8) splits *= 2;
    // one more slice if that fills a wave better
    if (tiles * splits < (uint32_t)num_sms && tiles * (splits + 1) <= (uint32_t)num_sms && splits + 1 <= stages) {
        const uint32_t s1 = (uint32_t)num_sms / tiles;
        if (s1 > splits && s1 <= 8 && s1 <= stages) splits = s1;
    }
    return splits;
}

size_t gemm_workspace_floats(uint32_t M, uint32_t rows, uint32_t splits) {
    return splits > 1 ? (size_t)splits * M * gemm_scales_ld(rows) : 0;
}

// d_y[M][rows] = W8A8 GEMM. d_part: workspace of gemm_workspace_floats() floats when splits > 1.
// mode: 0 = the product; 1 = int32 block sums into d_dump[M][rows][nb] (d_y untouched); 2, 3 = measurement
// (no drain / no drain and no loads; nothing is written).
cudaError_t launch_gemm_w8a8(const uint8_t *d_res, const RowLayout &L, uint32_t rows, const float *d_scalesT,
                             const int8_t *d_xq, const float *d_xd, const int32_t *d_xs, const float *d_xc, uint32_t M,
                             float *d_y, float *d_part, uint32_t splits, int mode, int32_t *d_dump, uint32_t *d_status,
                             cudaStream_t stream) {
    if (M == 0 || rows == 0) return cudaSuccess;
    CUtensorMap mx, mw, ms, mxd, mxs;
    const uint32_t lds = gemm_scales_ld(rows), ldm = gemm_x_ld(M);
    // activations: [M][K] int8, K innermost; weights: [rows][K] bytes (codes as q + 128), K innermost;
    // weight scales: [nb][lds] f32; token scales and un-bias terms (mode 1: code sums): [nb][ldm].
    // Coordinates past a dimension read as zero.
    const void *fifth = mode == 1 ? (const void *)d_xs : (const void *)d_xc;
    if (!make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, const_cast<int8_t *>(d_xq), L.in_dim, M, L.in_dim, 128, GM_BM,
                     CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, const_cast<uint8_t *>(d_res), L.in_dim, rows, L.in_dim, 128,
                     GM_BN, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_2d(&ms, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, const_cast<float *>(d_scalesT), lds, L.nb, (uint64_t)lds * 4,
                     GM_BN, GM_KB_STAGE, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !make_map_2d(&mxd, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, const_cast<float *>(d_xd), ldm, L.nb, (uint64_t)ldm * 4,
                     GM_BM, GM_KB_STAGE, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !make_map_2d(&mxs, CU_TENSOR_MAP_DATA_TYPE_INT32, const_cast<void *>(fifth), ldm, L.nb, (uint64_t)ldm * 4,
                     GM_BM, GM_KB_STAGE, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    GemmArgs a{};
    a.M = M;
    a.N = rows;
    a.nb = L.nb;
    a.ldx = ldm;
    a.dump = d_dump;
    a.status = d_status;
    const uint32_t stages = (L.nb + GM_KB_STAGE - 1) / GM_KB_STAGE;
    if (splits < 1) splits = 1;
    if (splits > stages) splits = stages;
    a.kb_per_split = ((stages + splits - 1) / splits) * GM_KB_STAGE;
    splits = (L.nb + a.kb_per_split - 1) / a.kb_per_split;
    if (splits > 1) {
        a.y = d_part;
        a.ldy = lds;
    } else {
        a.y = d_y;
        a.ldy = rows;
    }
    dim3 grid((rows + GM_BN - 1) / GM_BN, (M + GM_BM - 1) / GM_BM, splits);
    switch (mode) {
        case 0: gemm_w8a8_kernel<0><<<grid, GM_THREADS, GM_SMEM, stream>>>(mx, mw, ms, mxd, mxs, a); break;
        case 1: gemm_w8a8_kernel<1><<<grid, GM_THREADS, GM_SMEM, stream>>>(mx, mw, ms, mxd, mxs, a); break;
        case 2: gemm_w8a8_kernel<2><<<grid, GM_THREADS, GM_SMEM, stream>>>(mx, mw, ms, mxd, mxs, a); break;
        case 3: gemm_w8a8_kernel<3><<<grid, GM_THREADS, GM_SMEM, stream>>>(mx, mw, ms, mxd, mxs, a); break;
        case 4: gemm_w8a8_kernel<4><<<grid, GM_THREADS, GM_SMEM, stream>>>(mx, mw, ms, mxd, mxs, a); break;
        case 5:  // measurement: mode 4 with every MMA waited for before the next is issued
            a.dump = reinterpret_cast<int32_t *>(d_y);
            gemm_w8a8_kernel<4><<<grid, GM_THREADS, GM_SMEM, stream>>>(mx, mw, ms, mxd, mxs, a);
            break;
        default: return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (mode == 0 && splits > 1) {
        const uint64_t total = (uint64_t)M * rows;
        splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(d_part, d_y, M, rows, lds, splits);
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace strix
