// A list of dequant-GEMV steps in ONE persistent cooperative launch: the decode projection chain
// (four dependent steps per layer plus the lm_head: crates/strix-backend-rocm/src/decode.rs:5047-5531
// runs them as 12 launches per layer), and any batch of independent GEMVs (gemv_batch, decode.rs:3227-3255).
//
// Why one launch. A decode step moves 6-28 MB of weights (1-4 us of HBM time), but as its own launch
// it costs ~9 us: launch, first-byte latency of the weight stream, activation prologue, drain. Here
//   * the producer warp of every CTA streams the weights of step after step through ONE ring of
//     stages (1-D bulk async copies, mbarrier complete_tx) and never waits for another CTA - weights
//     depend on nothing - so HBM keeps streaming while activations are exchanged;
//   * all consumer warps of a CTA work on every stage: the CTA's tiles of a step form one flat
//     list and tile u belongs to warp u mod CH_WARPS, whatever row group it is in, so small steps (160 row
//     groups on 148 SMs) still use every warp. A warp keeps the partial sums of the row group it is
//     in; they wait in shared memory, per (row group, warp), and are added in warp order (deterministic)
//     once per step (or per 12 row groups);
//   * a step's outputs are published into EXCHANGE VECTORS of 8-byte entries {f32 value, epoch}
//     (one 64-bit store each, so value and flag arrive together); the consumers of the next step poll
//     the entries they need until each carries the epoch of the producing step of this launch. There
//     is no grid barrier and no fence: the step-to-step latency is one store and one load through L2.
//     With the rows sharded over GPUs the same stores also go to every peer's vector over NVLink
//     (plain peer stores, no multicast), and the exchange needs no collective and no extra launch;
//   * RMSNorm and the per-32 int8 quantiser (rmsnorm_xquant / xquant8, kernels.rs:101-147, 864-876)
//     run in the prologue in the reference's operand order ((x * 1/rms) * w, then d = amax/127, rintf);
//     SwiGLU / GeGLU (silu_xquant, geglu_xquant, kernels.rs:151-226) run in the epilogue of the
//     gate|up step, which handles row group g of both matrices in the same warps; the residual add
//     runs in the epilogue of the o / down steps.
// Every wait is bounded. A wait on an exchange vector that runs out raises STATUS_WAIT_TIMEOUT, after
// which nobody polls again (the launch runs to its end on whatever the vectors hold); the weight
// pipeline is local to the CTA and keeps its own bounded mbarrier waits.
#include <algorithm>

#include "gemv_tiles.cuh"

namespace strix {

// Shared-memory map (bytes). 0..1919 as in gemv_tiles.cuh (full / empty mbarriers, control words, oscale);
// the activation prologues use [SMEM_PART_OFF, +2048) as reduction scratch.
// Consumer warps: fifteen, i.e. sixteen warps with the producer. Every phase of a 2 us step is run by all consumer
// warps and its bookkeeping (stage hand-overs, polls, barriers) is per warp, so fewer warps mean fewer instructions
// competing for issue slots; the compiler gives a thread 128 registers for any CTA of 13 to 16 warps (24 warps: 72,
// with spills in the tile loop), so sixteen is the most that costs no registers. Measured on the 36-layer decode
// chain, ms per token on one box: 11 warps 1.384, 12 1.386, 14 1.394, 15 1.345-1.353; 24 warps 1.35 against 1.37
// for 12 in an earlier revision. Row-sharded over two GPUs: 1.151 with 15 against 1.160-1.168 with 12.
#ifndef STRIX_CHAIN_WARPS
#define STRIX_CHAIN_WARPS 15
#endif
constexpr uint32_t CH_WARPS = STRIX_CHAIN_WARPS;
constexpr uint32_t CH_PART_OFF = SMEM_PART_OFF + 2048u;  // [CHAIN_PART_SLOTS][CH_WARPS][16] f32 partial sums
// Step descriptors in shared memory: a step's fields are read many times by every warp, and from global
// memory each first touch of a line costs an L2 round trip on the critical path of a 2 us step. Warp 0
// copies step s + 1 in while step s runs (three slots: the threads still storing step s - 1's rows read
// theirs); the producer warp, which runs steps ahead of the consumers, keeps a slot of its own.
constexpr uint32_t CH_STEP_BYTES = 512;
static_assert(sizeof(ChainStep) <= CH_STEP_BYTES && sizeof(ChainStep) % 16 == 0, "one 16-byte word per lane of a warp");
constexpr uint32_t CH_STEP_OFF = CH_PART_OFF + CHAIN_PART_SLOTS * CH_WARPS * 16u * 4u;  // 3 consumer slots + 1 producer slot
constexpr uint32_t CH_X_OFF = (CH_STEP_OFF + 4u * CH_STEP_BYTES + 127u) & ~127u;
constexpr int CH_NORM_NI = 2;  // float4s a thread keeps across the RMSNorm reduction: normed rows up to 2 * 4 * 384 = 3072

struct ChainCta {
    Cta c;
    uint32_t n_stages, stage_bytes, stage_off, x_off;
    uint32_t sl, ph;       // ring position and phase parity (producer: stage to fill; consumers: stage to read)
    uint32_t lap0;         // producer: still on the ring's first lap (nothing to wait for)
    uint32_t ubase;        // consumers: tiles of this step seen so far, mod CH_WARPS
    uint32_t poll_limit;
    uint32_t epoch_base;
    unsigned long long *trace;  // measurement only: this step's clock words (CTA 0), or null
    uint32_t debug;             // measurement only: bit 0 = no arithmetic, bit 1 = polls do not wait
    long long wait_clk;         // measurement only: SM clocks this thread spent waiting for weight stages
};
static_assert(CHAIN_ACT_DIGITS == ACT_F32_DIGITS, "one code for the digit form");

__device__ __forceinline__ void ch_trace(const ChainCta &C, uint32_t k) {
    if (C.trace && C.c.tid == 0) C.trace[k] = (unsigned long long)clock64();
}

__device__ __forceinline__ volatile uint32_t *ch_ctl(const ChainCta &C) { return cta_ctl(C.c); }
// one warp: steps[s] -> shared-memory slot, 16 bytes per lane, as an asynchronous copy (the warp does not
// wait for the data; ch_fetch_wait before the barrier that hands the slot to the other warps)
__device__ __forceinline__ void ch_fetch_step(const ChainStep *steps, uint32_t s, uint8_t *slot, uint32_t lane) {
    if (lane * 16u < sizeof(ChainStep))
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(slot + lane * 16u)),
                     "l"(reinterpret_cast<const uint8_t *>(steps + s) + lane * 16u)
                     : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void ch_fetch_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// ctl[0]: a wait of the CTA's weight pipeline ran out. ctl[1]: a wait on an exchange vector ran out
// somewhere: nobody polls again.

__device__ __forceinline__ uint32_t ch_rank(const ChainCta &C, const ChainStep &S) {
    const uint32_t r = C.c.bid + S.rot;
    return r >= C.c.grid ? r - C.c.grid : r;
}
__device__ __forceinline__ uint32_t ch_items(const ChainCta &C, const ChainStep &S) {
    const uint32_t r = ch_rank(C, S);
    return S.n_items > r ? (S.n_items - r + C.c.grid - 1u) / C.c.grid : 0u;
}

struct ItemRef {
    uint32_t mat, row0, rows;
    const uint8_t *src0, *src1;
};
__device__ __forceinline__ ItemRef item_ref(const ChainStep &S, uint32_t item) {
    ItemRef r;
    uint32_t m = 0;
    if (!S.pair) {
        if (S.nmat > 1 && item >= S.mat[1].item0) m = 1;
        if (S.nmat > 2 && item >= S.mat[2].item0) m = 2;
    }
    const uint32_t gl = item - S.mat[m].item0;
    r.mat = m;
    r.row0 = gl * TILE_ROWS;
    r.rows = min(TILE_ROWS, S.mat[m].rows - r.row0);
    r.src0 = S.mat[m].w + (uint64_t)gl * S.L.group_bytes;
    r.src1 = S.pair ? S.mat[1].w + (uint64_t)gl * S.L.group_bytes : nullptr;
    return r;
}

// ---- producer: lane 0 of the producer warp fills the ring, item after item, chunk after chunk ----
__device__ __forceinline__ void chain_produce(const ChainStep &S, ChainCta &C) {
    uint64_t *full = cta_full(C.c), *empty = cta_empty(C.c);
    volatile uint32_t *ctl = ch_ctl(C);
    uint8_t *stages = C.c.smem + C.stage_off;
    const uint32_t my_n = ch_items(C, S), rank = ch_rank(C, S);
    const uint32_t CT = S.chunk_tiles, NC = S.n_chunks, tb = S.L.tile_bytes;
    for (uint32_t n = 0; n < my_n; n++) {
        const ItemRef it = item_ref(S, rank + n * C.c.grid);
        for (uint32_t c = 0; c < NC; c++) {
            if (!C.lap0 && !mbar_wait_suspended(&empty[C.sl], C.ph ^ 1u, C.c.status, 100u)) ctl[0] = 1;
            if (ctl[0]) return;  // after an abort nothing more is issued
            const uint32_t nbk = min(CT, S.L.nb - c * CT), bytes = nbk * tb;
            uint8_t *dst = stages + (uint64_t)C.sl * C.stage_bytes;
            mbar_arrive_expect_tx(&full[C.sl], S.pair ? 2u * bytes : bytes);
            bulk_g2s(dst, it.src0 + (uint64_t)c * CT * tb, bytes, &full[C.sl]);
            if (S.pair) bulk_g2s(dst + CT * tb, it.src1 + (uint64_t)c * CT * tb, bytes, &full[C.sl]);
            if (++C.sl == C.n_stages) { C.sl = 0; C.ph ^= 1u; C.lap0 = 0; }
        }
    }
}

// ---- exchange vectors ----
__device__ __forceinline__ void ll_store(unsigned long long *p, float v, uint32_t epoch) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)epoch << 32);
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_load2(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p));
}
// One entry, waited for (bounded) by the calling thread alone.
__device__ __forceinline__ float ll_wait1(const unsigned long long *p, uint32_t want, ChainCta &C) {
    volatile uint32_t *ctl = ch_ctl(C);
    unsigned long long w = 0;
    for (uint32_t it = 0;; ++it) {
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
        if ((uint32_t)(w >> 32) == want || ctl[1] || (C.debug & 2u)) break;
        if (it >= C.poll_limit) {
            if (C.c.status) atomicOr(C.c.status, STATUS_WAIT_TIMEOUT);
            ctl[1] = 1;
            break;
        }
    }
    return __uint_as_float((uint32_t)w);
}

#define CH_CONS_BAR() asm volatile("bar.sync 15, %0;" ::"r"(CH_WARPS * 32u) : "memory")

// ---- prologue of an integer-dot step (one activation row): the activation, plain or from an exchange
//      vector, through the optional RMSNorm into the per-32 int8 operands of the tiles (see x_layout).
//      Thread tid owns float4s tid, tid + 768, ... (eight consecutive threads = one 32-element block).
//      The row is taken in passes of NIP float4s per thread: all of a pass's entries are requested before
//      the first is looked at (one trip to L2 per pass) and, without a norm, quantised and stored before
//      the next pass, so a long row (ffn 9728) needs no more registers than a short one. With RMSNorm
//      the values stay in registers across the block-wide sum of squares (rows up to 4 x NIP x 3072).
//      Every warp of all 148 CTAs runs this, on the critical path of a 2 us step: what counts is its
//      instruction count. Warps past the end of the row only meet the barriers. ----
__device__ __forceinline__ void quant_store(const float4 t4, uint32_t e4, bool live, uint32_t l8, bool q6, int bias, uint32_t *xbw,
                                            float *rec) {
    // per-32 quantiser (xquant8, kernels.rs:864-876): d = amax/127, inv = d>0 ? 1/d : 0, q = clamp(rintf(x*inv));
    // eight lanes per block, four elements each
    const uint32_t blk = e4 >> 3, t = l8 & 3u, hf = l8 >> 2;
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
        if (q6) {
            xbw[(blk * 8u + hf * 4u + t) * 2u + hf] = wq;
            xbw[(blk * 8u + hf * 4u + t) * 2u + (hf ^ 1u)] = 0u;
            if (l8 == 0) rec[blk * 16u] = d;
            if (t == 0) rec[blk * 16u + 1u + hf] = __int_as_float(-bias * half_sum);
        } else {
            xbw[(blk * 4u + t) * 2u + hf] = wq;
            if (l8 == 0) {
                rec[blk * 2u] = d;
                rec[blk * 2u + 1u] = -(float)bias * d * (float)cs;
            }
        }
    }
}

// One pass: NIP float4s per thread starting at float4 index e0 (this thread's first), ct apart.
template <int NIP>
__device__ __forceinline__ void fetch_pass(const ChainStep &S, ChainCta &C, uint32_t e0, uint32_t ct, uint32_t K4, float4 (&v)[NIP]) {
    volatile uint32_t *ctl = ch_ctl(C);
    if (S.a_ll) {
        const uint32_t want = C.epoch_base + S.in_step + 1u;
        uint32_t pend = 0;
#pragma unroll
        for (int i = 0; i < NIP; i++) {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e0 + i * ct < K4) pend |= 1u << i;
        }
        for (uint32_t it = 0; pend != 0u; ++it) {
            unsigned long long e[NIP][4];
#pragma unroll
            for (int i = 0; i < NIP; i++) {
                if (pend & (1u << i)) {
                    const unsigned long long *p = S.a_ll + (size_t)(e0 + i * ct) * 4u;
                    ll_load2(p, e[i][0], e[i][1]);
                    ll_load2(p + 2, e[i][2], e[i][3]);
                }
            }
#pragma unroll
            for (int i = 0; i < NIP; i++) {
                if (pend & (1u << i)) {
                    if ((uint32_t)(e[i][0] >> 32) == want && (uint32_t)(e[i][1] >> 32) == want &&
                        (uint32_t)(e[i][2] >> 32) == want && (uint32_t)(e[i][3] >> 32) == want)
                        pend &= ~(1u << i);
                    v[i] = make_float4(__uint_as_float((uint32_t)e[i][0]), __uint_as_float((uint32_t)e[i][1]),
                                       __uint_as_float((uint32_t)e[i][2]), __uint_as_float((uint32_t)e[i][3]));
                }
            }
            if (pend == 0u || ctl[1] || (C.debug & 2u)) break;  // (a wait ran out somewhere: nobody polls again)
            if (it >= C.poll_limit) {
                if (C.c.status) atomicOr(C.c.status, STATUS_WAIT_TIMEOUT);
                ctl[1] = 1;
                break;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < NIP; i++) {
            const uint32_t e4 = e0 + i * ct;
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e4 < K4) v[i] = __ldcg(reinterpret_cast<const float4 *>(S.a) + e4);
        }
    }
}

template <int PRE>
__device__ __forceinline__ void chain_prologue_q8(const ChainStep &S, ChainCta &C, bool q6, int bias) {
    uint8_t *smem = C.c.smem;
    float *scr = reinterpret_cast<float *>(smem + SMEM_PART_OFF);
    const uint32_t tid = C.c.tid, lane = C.c.lane, warp = C.c.warp;
    const uint32_t K = S.L.in_dim, K4 = K / 4u, ct = CH_WARPS * 32u, l8 = lane & 7u;
    const XLayout XL = x_layout(q6 ? FMT_Q6_K : FMT_Q4_0, STRIX_ACT_Q8DOT, K, 1, C.x_off);
    uint32_t *xbw = reinterpret_cast<uint32_t *>(smem + XL.xb);
    float *rec = reinterpret_cast<float *>(smem + XL.rec);
    const uint32_t wbase = tid - lane;  // this warp's first float4
    if constexpr (PRE == STRIX_PRE_RMSNORM) {
        // rmsnorm (crates/strix-backend-cpu/src/qwen3.rs:107-114): (x * (1 / sqrt(mean(x^2) + eps))) * w.
        // Up to CH_NORM_NI float4s per thread stay in registers across the sum of squares.
        float4 v[CH_NORM_NI], w[CH_NORM_NI];
        float ss = 0.f;
        if (wbase < K4) {
            // the norm weights depend on nothing: on their way before the wait
#pragma unroll
            for (int i = 0; i < CH_NORM_NI; i++) {
                const uint32_t e4 = tid + i * ct;
                w[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e4 < K4) w[i] = __ldg(reinterpret_cast<const float4 *>(S.b) + e4);
            }
            fetch_pass<CH_NORM_NI>(S, C, tid, ct, K4, v);
#pragma unroll
            for (int i = 0; i < CH_NORM_NI; i++) {
                ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
                ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
            }
            ss = warp_sum(ss);
        }
        ch_trace(C, 1);
        if (lane == 0) scr[warp] = ss;
        CH_CONS_BAR();
        if (wbase < K4) {
            float tot = 0.f;
#pragma unroll
            for (uint32_t w2 = 0; w2 < CH_WARPS; w2++) tot += scr[w2];
            const float sc = 1.0f / sqrtf(tot / (float)K + S.eps);
#pragma unroll
            for (int i = 0; i < CH_NORM_NI; i++) {
                if (wbase + i * ct >= K4) break;  // the whole warp is past the row's end (quant_store shuffles)
                const float4 x4 = make_float4((v[i].x * sc) * w[i].x, (v[i].y * sc) * w[i].y, (v[i].z * sc) * w[i].z,
                                              (v[i].w * sc) * w[i].w);
                quant_store(x4, tid + i * ct, tid + i * ct < K4, l8, q6, bias, xbw, rec);
            }
        }
    } else {
        // no norm: each pass (up to 2 float4s per thread, both requested at once) is quantised and stored before
        // the next one is fetched. Threads past the row's end carry zeros through the shuffles and store nothing.
        const uint32_t per = (K4 + ct - 1u) / ct;  // float4s per thread
        if (per <= 1u) {
            float4 v[1];
            fetch_pass<1>(S, C, tid, ct, K4, v);
            quant_store(v[0], tid, tid < K4, l8, q6, bias, xbw, rec);
        } else if (per <= 2u) {
            float4 v[2];
            fetch_pass<2>(S, C, tid, ct, K4, v);
#pragma unroll
            for (int i = 0; i < 2; i++) quant_store(v[i], tid + i * ct, tid + i * ct < K4, l8, q6, bias, xbw, rec);
        } else {
            // (Two float4s per thread and pass. Four measured slower - the registers they take are spilled in the
            // tile loop - and even writing this loop over a pass size with its first store under the same test as the
            // second cost 11 %, 1.54 against 1.39 ms per token: the kernel's register allocation is that tight.)
            for (uint32_t e0 = tid; e0 - lane < K4; e0 += 2u * ct) {
                float4 v[2];
                fetch_pass<2>(S, C, e0, ct, K4, v);
                quant_store(v[0], e0, e0 < K4, l8, q6, bias, xbw, rec);
                if (e0 - lane + ct < K4) quant_store(v[1], e0 + ct, e0 + ct < K4, l8, q6, bias, xbw, rec);
            }
        }
        ch_trace(C, 1);
    }
    if (tid == 0) *reinterpret_cast<float *>(smem + SMEM_OSCALE_OFF) = 1.0f;
    CH_CONS_BAR();
}

// ---- epilogue: add up the partial sums of the row groups waiting in shared memory (warp order) and
//      publish the rows. Thread r of item `it` owns row r of that row group. ----
// The residual of the row this thread will publish in the step's FIRST reduction, fetched before the tiles
// are run so that its trip to L2 is off the critical path. ok = 0: nothing fetched (no residual, a row of a
// later reduction, or an entry that has not arrived yet): chain_flush then reads it itself.
struct EarlyRes {
    float v;
    uint32_t ok;
};
template <bool PAIR>
__device__ __forceinline__ EarlyRes chain_early_res(const ChainStep &S, ChainCta &C, uint32_t my_n) {
    EarlyRes E{0.f, 0u};
    constexpr uint32_t CAP = PAIR ? (uint32_t)CHAIN_PART_SLOTS / 2u : (uint32_t)CHAIN_PART_SLOTS;
    const uint32_t tid = C.c.tid, n0 = my_n < CAP ? my_n : CAP;
    if (tid >= n0 * TILE_ROWS) return E;
    const uint32_t it = tid / TILE_ROWS, r = tid % TILE_ROWS;
    const ItemRef ref = item_ref(S, ch_rank(C, S) + it * C.c.grid);
    if (r >= ref.rows) return E;
    const ChainMat &M = S.mat[ref.mat];
    const size_t o = ref.row0 + r;
    if (M.res) {
        E.v = __ldcg(M.res + o);
        E.ok = 1u;
    }
    if (M.res_ll) {
        unsigned long long w;
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(M.res_ll + M.row_base + o) : "memory");
        if ((uint32_t)(w >> 32) == C.epoch_base + S.res_step + 1u) {
            E.v += __uint_as_float((uint32_t)w);
            E.ok |= 2u;
        }
    }
    return E;
}

template <bool PAIR>
__device__ __forceinline__ void chain_flush(const ChainStep &S, ChainCta &C, uint32_t first_n, uint32_t n_wait, float osc,
                                            uint32_t epoch, EarlyRes E) {
    const uint32_t tid = C.c.tid;
    if (tid >= n_wait * TILE_ROWS) return;
    const float *part = reinterpret_cast<const float *>(C.c.smem + CH_PART_OFF);
    const uint32_t it = tid / TILE_ROWS, r = tid % TILE_ROWS;
    const ItemRef ref = item_ref(S, ch_rank(C, S) + (first_n + it) * C.c.grid);
    if (r >= ref.rows) return;
    const uint32_t slot = PAIR ? 2u * it : it;
    float val = 0.f;
#pragma unroll
    for (uint32_t w = 0; w < CH_WARPS; w++) val += part[(slot * CH_WARPS + w) * 16u + r];
    val *= osc;
    if (PAIR) {
        float up = 0.f;
#pragma unroll
        for (uint32_t w = 0; w < CH_WARPS; w++) up += part[((slot + 1u) * CH_WARPS + w) * 16u + r];
        up *= osc;
        val = (S.pair == STRIX_PRE_SWIGLU ? silu_f(val) : gelu_tanh_f(val)) * up;
    }
    const ChainMat &M = S.mat[ref.mat];
    const size_t o = ref.row0 + r;
    if (first_n == 0u) val += E.v;  // (the early fetch covers the first reduction's rows)
    if (M.res && !(first_n == 0u && (E.ok & 1u))) val += __ldcg(M.res + o);
    if (M.res_ll && !(first_n == 0u && (E.ok & 2u))) val += ll_wait1(M.res_ll + M.row_base + o, C.epoch_base + S.res_step + 1u, C);
    if (M.y) M.y[o] = val;
    for (uint32_t p = 0; p < M.n_out_ll; p++) ll_store(M.out_ll[p] + M.row_base + o, val, epoch);
}

// ---- consumers: all warps on every stage; tile u of the CTA's flat list of this step belongs to warp u mod CH_WARPS ----
template <int FMT, int ACT, bool PAIR>
__device__ __forceinline__ void chain_consume(const ChainStep &S, ChainCta &C, uint32_t epoch) {
    uint8_t *smem = C.c.smem;
    uint64_t *full = cta_full(C.c), *empty = cta_empty(C.c);
    volatile uint32_t *ctl = ch_ctl(C);
    float *part = reinterpret_cast<float *>(smem + CH_PART_OFF);
    const uint32_t lane = C.c.lane, warp = __shfl_sync(0xffffffffu, C.c.warp, 0);
    const RowLayout L = S.L;
    constexpr uint32_t SUB = FMT == FMT_Q6_K ? 8u : 1u;
    const uint32_t CT = S.chunk_tiles, NC = S.n_chunks;
    const uint32_t my_n = ch_items(C, S);
    const XLayout XL = x_layout(FMT, ACT, L.in_dim, 1, C.x_off);
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t xs0 = smem_u32(smem), st0 = xs0 + C.stage_off;
    // this lane's B-operand and record addresses for block 0 (as in gemv_kernel: lanes whose MMA column
    // carries no activation row re-read one that does; what they produce is never stored)
    const uint32_t n_op = XL.cols * 4u;
    const uint32_t lane_eff = (n_op > 16u && lane >= 16u) ? 16u + (lane - 16u) % (n_op - 16u) : lane % n_op;
    const uint32_t xb_l = xs0 + XL.xb + lane_eff * (ACT == STRIX_ACT_F32 ? 16u : 8u);
    const uint32_t xr_l = xs0 + XL.rec + (FMT == FMT_Q6_K ? 16u * t : (FMT == FMT_Q4_1 && ACT == STRIX_ACT_F32) ? 4u * t : 0u);
    const TileConsts TC = tile_consts<FMT, ACT>();
    const float osc = *reinterpret_cast<const float *>(smem + SMEM_OSCALE_OFF);
    const uint32_t half_off = CT * L.tile_bytes;  // a pair's stage: gate tiles, then up tiles
    constexpr uint32_t PER = PAIR ? 2u : 1u;
    uint32_t waiting = 0, first_n = 0;  // row groups whose partial sums wait in shared memory; the first of them
    const EarlyRes early = chain_early_res<PAIR>(S, C, my_n);
    for (uint32_t n = 0; n < my_n; n++) {
        float acc[2] = {0.f, 0.f}, up[2] = {0.f, 0.f};
        for (uint32_t c = 0; c < NC; c++) {
            if (C.trace) {
                const long long c0 = clock64();
                if (!ctl[0] && !mbar_wait_bounded(&full[C.sl], C.ph, C.c.status)) ctl[0] = 1;
                C.wait_clk += clock64() - c0;
            } else if (!ctl[0] && !mbar_wait_bounded(&full[C.sl], C.ph, C.c.status)) {
                ctl[0] = 1;
            }
            const uint32_t base = st0 + C.sl * C.stage_bytes;
            const uint32_t nbk = min(CT, L.nb - c * CT), U = nbk * SUB;
            uint32_t j = warp >= C.ubase ? warp - C.ubase : warp + CH_WARPS - C.ubase;
            const uint32_t blk0 = c * CT * SUB;
            auto mac = [&](uint32_t u, float (&a)[2], float (&b)[2]) {
                const uint32_t xb_a = mad_u32(blk0 + u, XL.xb_stride, xb_l), xr_a = mad_u32(blk0 + u, XL.rec_stride, xr_l);
                uint32_t ta, da = 0u;
                if (FMT == FMT_Q6_K) {
                    const uint32_t tb = mad_u32(u >> 3, Q6_TILE, base);
                    ta = mad_u32(u & 7u, Q6_SUB, tb);
                    da = tb + 8u * Q6_SUB;
                } else {
                    ta = mad_u32(u, L.tile_bytes, base);
                }
                tile_mac<FMT, ACT, false>(ta, da, xb_a, xr_a, TC, lane, a);
                if (PAIR) tile_mac<FMT, ACT, false>(ta + half_off, da + half_off, xb_a, xr_a, TC, lane, b);
            };
            // (one call site, not unrolled: a second copy of the tile code costs registers that the compiler then
            // spills inside this loop, which measured slower than the latency the second chain would hide)
            if (!(C.debug & 1u)) {
#pragma unroll 1
                for (; j < U; j += CH_WARPS) mac(j, acc, up);
            }
            C.ubase = (C.ubase + U) % CH_WARPS;
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[C.sl]);  // this warp's reads of the stage are complete
            if (++C.sl == C.n_stages) { C.sl = 0; C.ph ^= 1u; }
        }
        // the row group is complete for this warp: its partial sums wait for the reduction
        if (ACT == CHAIN_ACT_DIGITS) {
            // lane t of a quad holds digit t's share of rows g and g + 8
#pragma unroll
            for (int v = 0; v < 2; v++) {
                float a = t < N_DIGITS ? acc[v] : 0.f;
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                acc[v] = a;
            }
        }
        if (t == 0) {
            float *p = part + (waiting * CH_WARPS + warp) * 16u;
            p[g] = acc[0];
            p[g + 8u] = acc[1];
            if (PAIR) {
                p[CH_WARPS * 16u + g] = up[0];
                p[CH_WARPS * 16u + g + 8u] = up[1];
            }
        }
        waiting += PER;
        const bool last = n + 1u == my_n;
        if (last || waiting + PER > (uint32_t)CHAIN_PART_SLOTS) {
            if (last) {
                ch_trace(C, 3);
                if (warp == 0) ch_fetch_wait();  // the next step's descriptor has landed: this barrier hands it over
            }
            CH_CONS_BAR();
            chain_flush<PAIR>(S, C, first_n, waiting / PER, osc, epoch, early);
            // (after the step's last row group nothing waits here: the next write to this area lies behind
            // the barriers of the next prologue, which the threads still adding up pass last)
            if (!last) CH_CONS_BAR();
            first_n = n + 1u;
            waiting = 0;
        }
    }
}

template <int FMT>
__device__ __forceinline__ void chain_step_fmt(const ChainStep &S, ChainCta &C, uint32_t epoch) {
    if (S.act == STRIX_ACT_Q8DOT) {
        ch_trace(C, 2);
        if (S.pair) chain_consume<FMT, STRIX_ACT_Q8DOT, true>(S, C, epoch);
        else chain_consume<FMT, STRIX_ACT_Q8DOT, false>(S, C, epoch);
        return;
    }
#ifndef CHAIN_MIN
    // f32 activations (plain input, no pre-op: independent GEMVs of a batch)
    ActIn I;
    I.a = S.a; I.b = nullptr; I.K = S.L.in_dim; I.B = 1; I.a_stride = 0; I.b_stride = 0; I.x_off = C.x_off; I.eps = 0.f;
    if constexpr (FMT == FMT_Q6_K) {
        if (S.act == CHAIN_ACT_DIGITS) {
            consumer_prologue<FMT, ACT_F32_DIGITS, false, STRIX_PRE_NONE>(I, C.c);
            ch_trace(C, 2);
            chain_consume<FMT, ACT_F32_DIGITS, false>(S, C, epoch);
            return;
        }
    }
    consumer_prologue<FMT, STRIX_ACT_F32, false, STRIX_PRE_NONE>(I, C.c);
    ch_trace(C, 2);
    chain_consume<FMT, STRIX_ACT_F32, false>(S, C, epoch);
#endif
}

__global__ void __launch_bounds__((CH_WARPS + 1) * 32, 1)
chain_kernel(const ChainStep *__restrict__ steps, uint32_t n_steps, ChainGeom G, uint32_t *gctl, uint32_t *status,
             uint32_t poll_limit, uint32_t debug, unsigned long long *trace) {
    extern __shared__ __align__(128) uint8_t smem[];
    ChainCta C;
    C.c.smem = smem;
    C.c.tid = threadIdx.x;
    C.c.lane = C.c.tid & 31u;
    C.c.warp = C.c.tid >> 5;
    C.c.grid = gridDim.x;
    C.c.bid = blockIdx.x;
    C.c.wc = CH_WARPS;
    C.c.n_slots = 1;
    C.c.n_cons = CH_WARPS;
    C.c.Sk = G.n_stages;
    C.c.stage_bytes = G.stage_bytes;
    C.c.stage_off = G.stage_off;
    C.c.status = status;
    C.c.tq_base = C.c.sl = C.c.ph = 0;
    C.n_stages = G.n_stages;
    C.stage_bytes = G.stage_bytes;
    C.stage_off = G.stage_off;
    C.x_off = G.x_off;
    C.sl = C.ph = C.ubase = 0;
    C.lap0 = 1;
    C.poll_limit = poll_limit;
    C.debug = debug;
    C.trace = nullptr;
    C.wait_clk = 0;
    // the epoch base of this launch: every CTA reads it before it can leave, and the last CTA to leave
    // moves it on (below), so no launch ever sees a value change under it
    C.epoch_base = *reinterpret_cast<volatile uint32_t *>(gctl);
    if (C.c.tid < G.n_stages) {
        mbar_init(&cta_full(C.c)[C.c.tid], 1);
        mbar_init(&cta_empty(C.c)[C.c.tid], CH_WARPS);
        if (C.c.tid == 0) {
            ch_ctl(C)[0] = 0;
            ch_ctl(C)[1] = 0;
        }
        mbar_fence_init();
    }
    __syncthreads();
    if (C.c.warp == CH_WARPS) {
        // ---------------- producer warp ----------------
        uint8_t *slot = smem + CH_STEP_OFF + 3u * CH_STEP_BYTES;
        const ChainStep &S = *reinterpret_cast<const ChainStep *>(slot);
        uint32_t issued = 0;
        for (uint32_t s = 0; s < n_steps && !ch_ctl(C)[0]; s++) {
            __syncwarp();
            ch_fetch_step(steps, s, slot, C.c.lane);
            ch_fetch_wait();
            __syncwarp();
            if (C.c.lane == 0) {
                chain_produce(S, C);
                issued += ch_items(C, S) * S.n_chunks;
            }
        }
        if (C.c.lane == 0) {
            if (ch_ctl(C)[0]) {
                // after an abort the consumers stop waiting: let the copies still in flight land (bounded)
                // before the CTA's shared memory is released
                const uint32_t back = issued < C.n_stages ? issued : C.n_stages;
                uint32_t sl = C.sl, ph = C.ph;
                for (uint32_t k = 0; k < back; k++) {
                    if (sl == 0) { sl = C.n_stages; ph ^= 1u; }
                    --sl;
                    for (uint32_t it = 0; it < (1u << 16); ++it)
                        if (mbar_try_wait(&cta_full(C.c)[sl], ph)) break;
                }
            }
        }
        return;
    }
    // ---------------- consumer warps ----------------
    if (C.c.warp == 0) {
        ch_fetch_step(steps, 0, smem + CH_STEP_OFF, C.c.lane);
        ch_fetch_wait();
    }
    CH_CONS_BAR();
    for (uint32_t s = 0; s < n_steps; s++) {
        const ChainStep &S = *reinterpret_cast<const ChainStep *>(smem + CH_STEP_OFF + (s % 3u) * CH_STEP_BYTES);
        // the next step's descriptor comes in while this step runs; what makes it visible to the other warps
        // is a barrier of this step (the prologue's, or the one below for a CTA without rows in this step)
        if (C.c.warp == 0 && s + 1u < n_steps) ch_fetch_step(steps, s + 1u, smem + CH_STEP_OFF + ((s + 1u) % 3u) * CH_STEP_BYTES, C.c.lane);
        C.trace = (trace && C.c.bid == 0) ? trace + (size_t)CHAIN_TRACE_WORDS * s : nullptr;
        C.wait_clk = 0;
        ch_trace(C, 0);
        if (ch_items(C, S) == 0u) {
            if (C.c.warp == 0) ch_fetch_wait();
            CH_CONS_BAR();
        }
        if (ch_items(C, S) != 0u) {
            const uint32_t epoch = C.epoch_base + s + 1u;
            if (S.act == STRIX_ACT_Q8DOT) {
                // (one copy of the prologue for all formats: they differ in the operand layout of Q6_K and in the
                // bias of the stored codes; Q4_1 is not centred: its record keeps +d_x * sum(codes))
                const int fmt = S.L.fmt;
                const int bias = fmt == FMT_Q8_0 ? 128 : fmt == FMT_Q4_0 ? 8 : fmt == FMT_Q4_1 ? -1 : 32;
                if (S.pre == STRIX_PRE_RMSNORM) chain_prologue_q8<STRIX_PRE_RMSNORM>(S, C, fmt == FMT_Q6_K, bias);
                else chain_prologue_q8<STRIX_PRE_NONE>(S, C, fmt == FMT_Q6_K, bias);
            }
            switch (S.L.fmt) {
                case FMT_Q4_0: chain_step_fmt<FMT_Q4_0>(S, C, epoch); break;
#ifndef CHAIN_MIN
                case FMT_Q4_1: chain_step_fmt<FMT_Q4_1>(S, C, epoch); break;
                case FMT_Q8_0: chain_step_fmt<FMT_Q8_0>(S, C, epoch); break;
#endif
                default: chain_step_fmt<FMT_Q6_K>(S, C, epoch); break;
            }
        }
        ch_trace(C, 4);
        if (C.trace && C.c.tid == 0) C.trace[5] = (unsigned long long)C.wait_clk;
    }
    // the last CTA to leave moves the epoch base past this launch's steps
    CH_CONS_BAR();
    if (C.c.tid == 0) {
        __threadfence();
        if (atomicAdd(gctl + 1, 1u) == gridDim.x - 1u) {
            gctl[1] = 0u;
            *reinterpret_cast<volatile uint32_t *>(gctl) = C.epoch_base + n_steps;
        }
    }
}
#undef CH_CONS_BAR

// ------------------------------------------------------------------ host side
static inline uint32_t align128u(uint32_t v) { return (v + 127u) & ~127u; }

bool chain_plan(ChainStep *steps, uint32_t n, int num_sms, size_t smem_optin, ChainGeom *geom) {
    if (n == 0 || !geom) return false;
    const uint32_t budget = (uint32_t)smem_optin - 1024u;
    uint32_t x_end = CH_X_OFF;
    for (uint32_t i = 0; i < n; i++) {
        ChainStep &s = steps[i];
        const uint32_t K = s.L.in_dim;
        if (K == 0 || K % 32u != 0 || s.nmat < 1 || s.nmat > GEMV_MAX_MATS) return false;
        if (s.act == STRIX_ACT_Q8DOT) {
            // the RMSNorm prologue keeps the whole row in registers
            if (s.pre == STRIX_PRE_RMSNORM && K > (uint32_t)CH_NORM_NI * 4u * CH_WARPS * 32u) return false;
            if (s.pre != STRIX_PRE_NONE && s.pre != STRIX_PRE_RMSNORM) return false;
            if (s.pre == STRIX_PRE_RMSNORM && !s.b) return false;
            if (!s.a && !s.a_ll) return false;
        } else {
            if (s.act != STRIX_ACT_F32 && !(s.act == CHAIN_ACT_DIGITS && s.L.fmt == FMT_Q6_K)) return false;
            if (s.pre != STRIX_PRE_NONE || s.a_ll || !s.a || s.pair) return false;
        }
        if (s.pair) {
            if (s.pair != STRIX_PRE_SWIGLU && s.pair != STRIX_PRE_GEGLU) return false;
            if (s.nmat != 2 || s.mat[0].rows != s.mat[1].rows) return false;
        }
        if (s.a_ll && s.in_step >= i) return false;  // an exchange vector holds an EARLIER step's outputs
        for (int m = 0; m < s.nmat; m++)
            if (s.mat[m].res_ll && s.res_step >= i) return false;
        const XLayout XL = x_layout(s.L.fmt, s.act == CHAIN_ACT_DIGITS ? ACT_F32_DIGITS : s.act, K, 1, CH_X_OFF);
        if (XL.end > x_end) x_end = XL.end;
    }
    const uint32_t stage_off = align128u(x_end);
    uint32_t max_tile = 0;
    for (uint32_t i = 0; i < n; i++) max_tile = std::max(max_tile, steps[i].L.tile_bytes * (steps[i].pair ? 2u : 1u));
    if (stage_off + 2u * align128u(max_tile) > budget) return false;
    // the ring: 8 stages of what is left (at most 32 KB each); fewer, larger ones if a tile would not fit
    uint32_t sk = 8;
    uint32_t sb = ((budget - stage_off) / sk) & ~127u;
    while (sb < max_tile && sk > 2) {
        sk--;
        sb = ((budget - stage_off) / sk) & ~127u;
    }
    if (sb < max_tile) return false;
    if (sb > 32768u) sb = 32768u;
    for (uint32_t i = 0; i < n; i++) {
        ChainStep &s = steps[i];
        const uint32_t per = s.pair ? 2u : 1u;
        uint32_t ct = sb / (s.L.tile_bytes * per);
        if (ct > s.L.nb) ct = s.L.nb;
        // even chunks: 304 blocks in runs of 84 would end on a short one (84 84 84 52); 76 x 4 keeps every stage full
        const uint32_t nc = (s.L.nb + ct - 1) / ct;
        ct = (s.L.nb + nc - 1) / nc;
        s.chunk_tiles = ct;
        s.n_chunks = (s.L.nb + ct - 1) / ct;
        uint32_t item = 0;
        for (int m = 0; m < s.nmat; m++) {
            s.mat[m].item0 = s.pair ? 0u : item;
            if (!s.pair || m == 0) item += (s.mat[m].rows + TILE_ROWS - 1) / TILE_ROWS;
        }
        s.n_items = item;
        s.rot = (i * 37u) % (uint32_t)num_sms;
    }
    geom->n_stages = sk;
    geom->stage_bytes = sb;
    geom->stage_off = stage_off;
    geom->x_off = CH_X_OFF;
    geom->smem_bytes = stage_off + sk * sb;
    return true;
}

cudaError_t chain_prepare_device(size_t smem_optin) {
    return cudaFuncSetAttribute(chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_optin);
}

cudaError_t launch_chain(const ChainStep *d_steps, uint32_t n_steps, const ChainGeom &geom, uint32_t *d_ctl,
                         uint32_t *d_status, uint32_t poll_limit, uint32_t debug, unsigned long long *d_trace, int num_sms,
                         cudaStream_t stream) {
    if (n_steps == 0) return cudaSuccess;
    ChainGeom g = geom;
    void *args[8] = {(void *)&d_steps, (void *)&n_steps, (void *)&g, (void *)&d_ctl, (void *)&d_status, (void *)&poll_limit,
                     (void *)&debug, (void *)&d_trace};
    const dim3 grid((unsigned)num_sms), block((CH_WARPS + 1) * 32);
    // cooperative: CTAs wait for one another's outputs, so all of them must be resident
    return cudaLaunchCooperativeKernel((const void *)chain_kernel, grid, block, args, geom.smem_bytes, stream);
}

}  // namespace strix
