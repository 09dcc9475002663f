// Fused dequant -> GEMV over resident tile-major weights (Q4_0 / Q8_0 / Q6_K), f32-activation
// and int8-activation (integer-dot) forms, for 1 to 8 activation rows per pass over the weights.
//
// Replaces the reference's batch-1 decode kernels (crates/strix-backend-rocm/src/kernels.rs:
// q4_gemv :41-69, q4_gemv_dp :259-287 with its fused forms dp2 / dp3 :324-361, q4_1_gemv_dp :292-320,
// q6_gemv :607-640, q8_0_gemv :646-668, q8i_gemv :894-912, and the batched-verify GEMVs) and the CPU
// loops they mirror (crates/strix-backend-cpu/src/qwen3.rs:90-105, 173-182 dot_f32 / qmatmul).
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
//   * One f32 activation row of up to 8192 elements (Q4_0, Q8_0, Q6_K) does not take the f16 tiles: it is carried
//     as three int8 digits per value and runs through the integer tile as three activation rows (gemv_tiles.cuh,
//     ACT_F32_DIGITS): no byte -> f16 conversion, one MMA per tile, f32 accuracy; the form that holds its burst
//     time under sustained load.
//   * Without the tensor cores the kernel was bound by instruction issue (about 85 instructions per
//     16 weights x 32 lanes for Q8_0, more for Q6_K); a tile now costs about 25, which leaves the
//     memory pipeline as the limit and makes activation rows 2..8 almost free.
//   * Every wait is bounded: on expiry the kernel flags STATUS_WAIT_TIMEOUT, stops issuing copies,
//     stops waiting, and runs out.
//   * gemv_multi_kernel runs several independent GEMVs (the items of a gemv_batch) side by side in one
//     launch: the CTAs are dealt out among the problems and each runs this same pipeline on its own.
//   * The launches of one batch do not wait for one another (GemvArgs::order): the first waits for what the
//     batch follows and only then lets its dependents be scheduled; a later one runs as its CTAs get an SM
//     and waits for the grid before it at its END. Measured on the six-weight benchmark step: the second
//     launch's first tile is consumed 2.5 us after its CTA starts instead of 3.3-4.4 us after the LAST CTA
//     of the launch before has gone; 157.6 -> 152.7 us per step.
#include <utility>

#include "gemv_tiles.cuh"

namespace strix {

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
    const uint32_t xr_l = xs0 + XL.rec + ((FMT == FMT_Q6_K || MULTI || ACT == ACT_F32_DIGITS) ? 16u * t
                                          : (FMT == FMT_Q4_1 && ACT == STRIX_ACT_F32)             ? 4u * t
                                                                                                   : 0u);
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
    // (A.order: 1 = first kernel of a batch of independent items, 2 = a later one; see GemvArgs)
    if (A.order != 1u) asm volatile("griddepcontrol.launch_dependents;");
    if (A.debug & 2u) return;  // measurement only: cost of an empty launch of this shape
    Cta C = cta_init(smem, A.wc, A.slots, A.n_stages, A.stage_bytes, A.stage_off, A.status);
    if (C.warp == C.n_cons) {
        producer_step(A, C);
        return;
    }
    // Everything above (and the producer's copies) touches only this launch's weights. The activation
    // and the outputs belong to the stream's order: wait for the preceding grid here. A later item of a batch has
    // nothing to wait for (its activation was there before the batch's first kernel started, its outputs are
    // its own): it only keeps the order of completion, at its end.
    if (A.order != 2u) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (A.order == 1u) asm volatile("griddepcontrol.launch_dependents;");
    if (A.xop) {
        const XLayout XL = x_layout(FMT, ACT, A.L.in_dim, A.nbatch, A.x_off);
        image_prologue(A.xop, XL.xb, (XL.end - XL.xb + 15u) & ~15u, A.nbatch, C);
    } else {
        consumer_prologue<FMT, ACT, MULTI, PRE>(act_in(A), C);
    }
    if (A.debug & 4u) return;  // measurement only: stop after the activation prologue
    consumer_groups<FMT, ACT, MULTI>(A, C);
    if (A.order == 2u) asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Several INDEPENDENT GEMVs side by side in one launch (the items of a gemv_batch: gemv_batch, decode.rs:3227-3255).
// A small GEMV (20-30 MB of weights, 3-4 us of HBM time) costs a launch of its own ~9 us in fill and drain, and
// nothing of another launch overlaps it because one CTA fills an SM. Here the CTAs of ONE launch are dealt out
// among the problems in proportion to their bytes (gemv_multi_plan), every CTA runs the ordinary pipeline on its
// own problem (its own format, activation form, in_dim, geometry), and the launch fills and drains once.
// One kernel carries every (format, activation form) body, pre-op none, one activation row; a CTA runs one of them.
template <int FMT, int ACT>
__device__ __forceinline__ void multi_body(const GemvArgs &A, Cta &C) {
    consumer_prologue<FMT, ACT, false, STRIX_PRE_NONE>(act_in(A), C);
    consumer_groups<FMT, ACT, false>(A, C);
}
template <int FMT>
__device__ __forceinline__ void multi_fmt(const GemvArgs &A, Cta &C) {
    if constexpr (FMT == FMT_Q6_K || FMT == FMT_Q8_0 || FMT == FMT_Q4_0) {
        if (A.digits) return multi_body<FMT, ACT_F32_DIGITS>(A, C);
    }
    if (A.act == STRIX_ACT_F32) return multi_body<FMT, STRIX_ACT_F32>(A, C);
    return multi_body<FMT, STRIX_ACT_Q8DOT>(A, C);
}
__global__ void __launch_bounds__((GEMV_WARPS + 1) * 32, 1) gemv_multi_kernel(const __grid_constant__ GemvMultiArgs M) {
    extern __shared__ __align__(128) uint8_t smem[];
    if (M.order != 1u) asm volatile("griddepcontrol.launch_dependents;");
    uint32_t i = 0;
    while (i + 1u < M.n && blockIdx.x >= M.cta0[i + 1u]) i++;
    const GemvArgs &A = M.p[i];
    Cta C = cta_init(smem, A.wc, A.slots, A.n_stages, A.stage_bytes, A.stage_off, A.status);
    C.bid = blockIdx.x - M.cta0[i];  // the problem's CTAs are numbered from 0 among themselves
    C.grid = M.cta0[i + 1u] - M.cta0[i];
    if (C.warp == C.n_cons) {
        producer_step(A, C);
        return;
    }
    if (M.order != 2u) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (M.order == 1u) asm volatile("griddepcontrol.launch_dependents;");
    switch (A.L.fmt) {
        case FMT_Q4_0: multi_fmt<FMT_Q4_0>(A, C); break;
        case FMT_Q4_1: multi_fmt<FMT_Q4_1>(A, C); break;
        case FMT_Q8_0: multi_fmt<FMT_Q8_0>(A, C); break;
        default: multi_fmt<FMT_Q6_K>(A, C); break;
    }
    if (M.order == 2u) asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- the activation operands of an integer-dot launch, prepared once for all CTAs ----
// One CTA per activation row (rows past nbatch only clear their record slots, which must read zero).
// Pre-ops as the reference's fused quantisers: RMSNorm in its operand order ((x * 1/rms) * w, kernels.rs:101-147),
// SwiGLU / GeGLU (kernels.rs:151-226), then xquant8 (kernels.rs:864-876). The image is the shared-memory
// operand region of gemv_kernel in x_layout order, so a CTA fetches it with plain bulk copies.
constexpr uint32_t XOP_THREADS = 1024, XOP_NI = 4;  // rows up to 4 * 4 * 1024 = 16384 elements
template <int PRE>
__global__ void __launch_bounds__(XOP_THREADS, 1)
xop_prepare_kernel(const float *__restrict__ a, const float *__restrict__ b, uint32_t a_stride, uint32_t b_stride, float eps,
                   uint32_t K, uint32_t B, int q6, int bias, uint8_t *__restrict__ image) {
    __shared__ float scr[32];
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, l8 = lane & 7u, bi = blockIdx.x;
    const uint32_t nb32 = K / 32u;
    // Without a norm nothing ties a row's blocks together: gridDim.y CTAs share a row, each takes a run of whole
    // 32-blocks (float4 indices [lo4, lo4 + K4)). With RMSNorm the launch has one CTA per row.
    const uint32_t lo4 = blockIdx.y * (K / 4u / gridDim.y), K4 = K / 4u / gridDim.y;
    const XLayout XL = x_layout(q6 ? FMT_Q6_K : FMT_Q4_0, STRIX_ACT_Q8DOT, K, B, 0u);
    uint32_t *xbw = reinterpret_cast<uint32_t *>(image + XL.xb);
    float *rec = reinterpret_cast<float *>(image + XL.rec);
    // the image (and the activations) belong to the stream's order: the launch before this one may still read them
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (bi >= B) {
        // a record slot without an activation row reads zero (what its MMA column produces is never stored)
        if (blockIdx.y != 0u) return;
        if (q6) {
            for (uint32_t blk = tid; blk < nb32; blk += XOP_THREADS)
                reinterpret_cast<float4 *>(rec)[blk * 4u + bi] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (uint32_t blk = tid; blk < nb32; blk += XOP_THREADS) {
                rec[blk * 16u + (bi >> 1) * 4u + (bi & 1u)] = 0.f;
                rec[blk * 16u + (bi >> 1) * 4u + 2u + (bi & 1u)] = 0.f;
            }
        }
        return;
    }
    const float *Aa = a + (size_t)bi * a_stride;
    const float *Ab = b ? b + (size_t)bi * b_stride : nullptr;
    float4 v[XOP_NI];
    float ss = 0.f;
#pragma unroll
    for (uint32_t i = 0; i < XOP_NI; i++) {
        const uint32_t e4 = tid + i * XOP_THREADS;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e4 < K4) {
            float4 a4 = __ldcg(reinterpret_cast<const float4 *>(Aa) + lo4 + e4);
            if (PRE == STRIX_PRE_RMSNORM) {
                ss = fmaf(a4.x, a4.x, ss); ss = fmaf(a4.y, a4.y, ss); ss = fmaf(a4.z, a4.z, ss); ss = fmaf(a4.w, a4.w, ss);
            } else if (PRE != STRIX_PRE_NONE) {
                const float4 b4 = __ldcg(reinterpret_cast<const float4 *>(Ab) + lo4 + e4);
                if (PRE == STRIX_PRE_SWIGLU) {
                    a4.x = silu_f(a4.x) * b4.x; a4.y = silu_f(a4.y) * b4.y; a4.z = silu_f(a4.z) * b4.z; a4.w = silu_f(a4.w) * b4.w;
                } else {
                    a4.x = gelu_tanh_f(a4.x) * b4.x; a4.y = gelu_tanh_f(a4.y) * b4.y;
                    a4.z = gelu_tanh_f(a4.z) * b4.z; a4.w = gelu_tanh_f(a4.w) * b4.w;
                }
            }
            v[i] = a4;
        }
    }
    if (PRE == STRIX_PRE_RMSNORM) {
        ss = warp_sum(ss);
        if (lane == 0) scr[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (uint32_t w2 = 0; w2 < XOP_THREADS / 32u; w2++) tot += scr[w2];
        const float sc = 1.0f / sqrtf(tot / (float)K + eps);   // (one CTA per row here: K4 is the whole row)
#pragma unroll
        for (uint32_t i = 0; i < XOP_NI; i++) {
            const uint32_t e4 = tid + i * XOP_THREADS;
            if (e4 < K4) {
                const float4 w4 = __ldg(reinterpret_cast<const float4 *>(b) + e4);  // the norm weight is shared by the rows
                v[i].x = (v[i].x * sc) * w4.x; v[i].y = (v[i].y * sc) * w4.y;
                v[i].z = (v[i].z * sc) * w4.z; v[i].w = (v[i].w * sc) * w4.w;
            }
        }
    }
#pragma unroll
    for (uint32_t i = 0; i < XOP_NI; i++) {
        const uint32_t e4 = tid + i * XOP_THREADS;
        if ((tid - lane) + i * XOP_THREADS >= K4) break;  // the whole warp is past the row's end (the body shuffles)
        const bool live = e4 < K4;
        const float4 t4 = v[i];
        const uint32_t blk = (lo4 + e4) >> 3, t = l8 & 3u, hf = l8 >> 2;
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
        const int half_sum = cs;
        cs += __shfl_xor_sync(0xffffffffu, cs, 4);
        if (live) {
            if (q6) {
                xbw[(blk * 8u * B + (2u * bi + hf) * 4u + t) * 2u + hf] = wq;
                xbw[(blk * 8u * B + (2u * bi + hf) * 4u + t) * 2u + (hf ^ 1u)] = 0u;
                if (l8 == 0) rec[blk * 16u + bi * 4u] = d;
                if (t == 0) rec[blk * 16u + bi * 4u + 1u + hf] = __int_as_float(-bias * half_sum);
                if (l8 == 0) rec[blk * 16u + bi * 4u + 3u] = 0.f;
            } else {
                xbw[(blk * 4u * B + bi * 4u + t) * 2u + hf] = wq;
                if (l8 == 0) {
                    const float kf = -(float)bias * d * (float)cs;
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

size_t xop_image_bytes(int fmt, uint32_t in_dim, uint32_t nbatch) {
    const XLayout XL = x_layout(fmt, STRIX_ACT_Q8DOT, in_dim, nbatch, 0u);
    return ((size_t)(XL.end - XL.xb) + 15u) & ~(size_t)15u;
}

cudaError_t launch_xop_prepare(int fmt, uint32_t in_dim, uint32_t nbatch, const float *d_a, const float *d_b,
                               uint32_t a_stride, uint32_t b_stride, float eps, int pre, uint8_t *d_image, bool pdl,
                               cudaStream_t stream) {
    if (in_dim > XOP_NI * 4u * XOP_THREADS || in_dim % 32u != 0) return cudaErrorInvalidValue;
    const bool q6 = fmt == FMT_Q6_K;
    const int bias = fmt == FMT_Q8_0 ? 128 : fmt == FMT_Q4_0 ? 8 : fmt == FMT_Q4_1 ? -1 : 32;
    cudaLaunchConfig_t cfg = {};
    // one CTA per record slot of the layout: rows without an activation clear theirs
    // (pre-ops other than RMSNorm work element by element: four CTAs per row, or two, when the row's blocks divide)
    const uint32_t nb32 = in_dim / 32u;
    const uint32_t parts = pre == STRIX_PRE_RMSNORM ? 1u : nb32 % 4u == 0u ? 4u : nb32 % 2u == 0u ? 2u : 1u;
    cfg.gridDim = dim3(nbatch > 1 || q6 ? (q6 ? 4u : 8u) : 1u, parts);
    cfg.blockDim = dim3(XOP_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1u : 0u;
    const int q6i = q6 ? 1 : 0;
    switch (pre) {
        case STRIX_PRE_NONE:
            return cudaLaunchKernelEx(&cfg, xop_prepare_kernel<STRIX_PRE_NONE>, d_a, d_b, a_stride, b_stride, eps, in_dim, nbatch, q6i, bias, d_image);
        case STRIX_PRE_RMSNORM:
            return cudaLaunchKernelEx(&cfg, xop_prepare_kernel<STRIX_PRE_RMSNORM>, d_a, d_b, a_stride, b_stride, eps, in_dim, nbatch, q6i, bias, d_image);
        case STRIX_PRE_SWIGLU:
            return cudaLaunchKernelEx(&cfg, xop_prepare_kernel<STRIX_PRE_SWIGLU>, d_a, d_b, a_stride, b_stride, eps, in_dim, nbatch, q6i, bias, d_image);
        case STRIX_PRE_GEGLU:
            return cudaLaunchKernelEx(&cfg, xop_prepare_kernel<STRIX_PRE_GEGLU>, d_a, d_b, a_stride, b_stride, eps, in_dim, nbatch, q6i, bias, d_image);
        default: return cudaErrorInvalidValue;
    }
}

// ------------------------------------------------------------------ host side
static inline uint32_t align128u(uint32_t v) { return (v + 127u) & ~127u; }

bool gemv_plan(GemvArgs &a, int num_sms, size_t smem_optin, const GemvTune &tune) {
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
    // (Q8_0 takes the same form by a rule of its own: its f16 form is the faster one in a burst on small launches)
    const uint32_t digit_rule = a.L.fmt == FMT_Q8_0   ? tune.q8_digits_rule
                                : a.L.fmt == FMT_Q4_0 ? tune.q4_digits_rule
                                                      : tune.digits_rule;  // 0 = never, 1 = K <= 8192, 2 = whenever it fits
    a.digits = ((a.L.fmt == FMT_Q6_K || a.L.fmt == FMT_Q8_0 || a.L.fmt == FMT_Q4_0) && a.act == STRIX_ACT_F32 && nbt == 1 && digit_rule != 0 &&
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
    const uint32_t force_wc = tune.force_wc, force_ct = tune.force_ct, force_sk = tune.force_sk;  // tuning knobs (0 = planned)
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
    a.pdl = tune.pdl;      // 0 = plain stream order
    a.debug = tune.debug;  // measurement modes (see GemvTune)
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
    if constexpr (FMT == FMT_Q6_K || FMT == FMT_Q8_0 || FMT == FMT_Q4_0) {
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

// Deals num_sms CTAs out among n planned-to-be problems (nmat = 1, one activation row, pre-op none) and plans each
// on its share: every problem gets one CTA, then the problem whose busiest CTA carries the most bytes gets the next
// one, until none is left or nobody can use another. False when a problem cannot run this way.
bool gemv_multi_plan(GemvMultiArgs &m, int num_sms, size_t smem_optin, const GemvTune &tune) {
    const uint32_t n = m.n;
    if (n < 1 || n > (uint32_t)GEMV_MULTI_MAX || n > (uint32_t)num_sms) return false;
    uint32_t nc[GEMV_MULTI_MAX], groups[GEMV_MULTI_MAX];
    for (uint32_t i = 0; i < n; i++) {
        const GemvArgs &a = m.p[i];
        if (a.nmat != 1 || a.pre != STRIX_PRE_NONE || a.nbatch > 1 || a.xop || a.sel_ids) return false;
        groups[i] = (a.mat[0].rows + TILE_ROWS - 1) / TILE_ROWS;
        nc[i] = 1;
    }
    // what a row group costs a CTA, in bytes streamed at the rate a CTA sustains for this format and activation form
    // (Q8_0 runs at the memory pipeline's pace; the others are bound by instruction issue: measured fractions of
    // the copy peak on large launches are 0.93 Q8_0, 0.74 Q6_K as digits or int8, 0.60 Q6_K and Q4_0 on f16 tiles,
    // 0.74 Q4_0 int8)
    auto slow = [&](uint32_t i) -> uint64_t {
        const GemvArgs &a = m.p[i];
        const uint32_t rule = a.L.fmt == FMT_Q6_K ? tune.digits_rule : a.L.fmt == FMT_Q4_0 ? tune.q4_digits_rule : 0u;
        const bool f16_tiles = a.act == STRIX_ACT_F32 && !(rule != 0 && (a.L.in_dim <= 8192u || rule == 2));
        if (a.L.fmt == FMT_Q8_0) return 100;
        return f16_tiles ? 155 : 125;
    };
    auto load = [&](uint32_t i) { return (uint64_t)((groups[i] + nc[i] - 1u) / nc[i]) * m.p[i].L.group_bytes * slow(i); };
    for (uint32_t left = (uint32_t)num_sms - n; left > 0; left--) {
        uint32_t worst = n;
        for (uint32_t i = 0; i < n; i++)
            if (nc[i] < groups[i] && (worst == n || load(i) > load(worst))) worst = i;
        if (worst == n) break;  // (more CTAs than row groups help nobody)
        nc[worst]++;
    }
    // The CTAs of a launch start in the order of their index, as the launch before lets go of its SMs (a spread of
    // 3-4 us): the problem whose CTAs have the most to do takes the first CTAs, the lightest the last (insertion sort by
    // load; measured per CTA with the planner's own dealing, the heaviest problem used to start last and end 3 us
    // behind the others).
    for (uint32_t i = 1; i < n; i++)
        for (uint32_t j = i; j > 0 && load(j) > load(j - 1); j--) {
            std::swap(m.p[j], m.p[j - 1]);
            std::swap(nc[j], nc[j - 1]);
            std::swap(groups[j], groups[j - 1]);
        }
    uint32_t c0 = 0, smem = 0;
    for (uint32_t i = 0; i < n; i++) {
        GemvArgs &a = m.p[i];
        a.nbatch = 1;
        if (!gemv_plan(a, (int)nc[i], smem_optin, tune)) return false;
        a.rot = 0;
        m.cta0[i] = c0;
        c0 += a.grid ? a.grid : 1u;  // (a problem without rows keeps one idle CTA: the CTA ranges stay well-formed)
        if (a.smem_bytes > smem) smem = a.smem_bytes;
    }
    m.cta0[n] = c0;
    m.grid = c0;
    m.smem_bytes = smem;
    m.pdl = tune.pdl;
    return true;
}

cudaError_t launch_gemv_multi(const GemvMultiArgs &m, cudaStream_t stream) {
    if (m.n == 0 || m.grid == 0) return cudaSuccess;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(m.grid);
    cfg.blockDim = dim3((GEMV_WARPS + 1) * 32);
    cfg.dynamicSmemBytes = m.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = m.pdl ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, gemv_multi_kernel, m);
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
    if constexpr (FMT == FMT_Q6_K || FMT == FMT_Q8_0 || FMT == FMT_Q4_0) { STRIX_ATTR(ACT_F32_DIGITS, false) }
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
    return cudaFuncSetAttribute(gemv_multi_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_optin);
}

// ---- cross-GPU barrier (one rank per GPU; never run two ranks of it on one GPU) ----
struct PeerFlags {
    uint32_t *p[GEMV_MAX_PEERS];
};
__global__ void peer_barrier_kernel(uint32_t *epoch, volatile uint32_t *local_flags, PeerFlags peers, int rank, int world,
                                    uint32_t *status, uint32_t limit) {
    __shared__ uint32_t seq;
    if (threadIdx.x == 0) seq = ++(*epoch);
    __syncthreads();
    const uint32_t want = seq;
    if ((int)threadIdx.x < world) {
        // the kernels before this one on the stream have completed: their stores to peer memory are done
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.p[threadIdx.x] + rank), "r"(want) : "memory");
        bool ok = status && (*reinterpret_cast<volatile uint32_t *>(status) & STATUS_WAIT_TIMEOUT);  // gave up before
        for (uint32_t it = 0; it < limit && !ok; ++it) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(local_flags + threadIdx.x) : "memory");
            ok = (int32_t)(seen - want) >= 0;
        }
        if (!ok && status) atomicOr(status, STATUS_WAIT_TIMEOUT);  // bounded: report and go on
    }
}

cudaError_t launch_peer_barrier(uint32_t *d_epoch, uint32_t *d_local_flags, uint32_t *const *peer_flags, int rank,
                                int world, uint32_t *d_status, uint32_t poll_limit, cudaStream_t stream) {
    if (world < 1 || world > GEMV_MAX_PEERS) return cudaErrorInvalidValue;
    PeerFlags pf{};
    for (int i = 0; i < world; i++) pf.p[i] = peer_flags[i];
    peer_barrier_kernel<<<1, 32, 0, stream>>>(d_epoch, d_local_flags, pf, rank, world, d_status, poll_limit);
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
