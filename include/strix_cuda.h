/*
 * strix_cuda.h -- C ABI of the B200 (sm_100a) weight accelerator for strix.rs.
 *
 * One `strix_cuda` handle is one accelerator bound to one CUDA device. The
 * entry points mirror, one to one, the methods of the reference trait
 * `WeightAccel` (crates/strix-core/src/accel.rs:147-507) that lie on the
 * quantized-matmul hot path; each declaration cites the trait method (and the
 * ROCm implementation) it replaces. A Rust `impl WeightAccel` binds these with
 * a plain `extern "C"` block.
 *
 * Return convention (the trait has no Result at this seam, accel.rs:144-146):
 *    1  adopted / Some(..) / true
 *    0  declined / None / false   -- the caller keeps the weight on the CPU
 *   <0  device or argument error; text via strix_cuda_last_error()
 * There is no CPU fallback inside the library.
 *
 * Buffers named `bytes`, `x`, `xs`, `h` are HOST memory borrowed for the call;
 * outputs `y`, `logits` are HOST memory owned by the caller. Entry points whose
 * name ends in `_dev` take DEVICE pointers and a cudaStream_t (as void*), do no
 * host<->device copy and do not synchronise; they exist for measurement and for
 * callers that keep activations resident.
 *
 * Threading: like the reference (decode.rs:559-562) a handle is not re-entrant;
 * serialise calls on one handle.
 */
#ifndef STRIX_CUDA_H
#define STRIX_CUDA_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define STRIX_API __attribute__((visibility("default")))
#else
#define STRIX_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct strix_cuda strix_cuda;

/* Activation arithmetic of a GEMV. F32 = the reference's q4_gemv / q8_0_gemv /
 * q6_gemv (kernels.rs:41-69, 646-668, 607-640). Q8DOT = the integer-dot
 * variant: x is quantised per 32 to int8 (xquant8, kernels.rs:864-876) and the
 * dot runs in int32 (q8i_gemv :894-912, q4_gemv_dp :259-287). */
enum { STRIX_ACT_F32 = 0, STRIX_ACT_Q8DOT = 1 };

/* Elementwise op fused in front of a device-resident GEMV's activation. */
enum {
    STRIX_PRE_NONE = 0,
    STRIX_PRE_RMSNORM = 1, /* x = rmsnorm(a, w, eps)        (rmsnorm_xquant, kernels.rs:101-147) */
    STRIX_PRE_SWIGLU = 2,  /* x = silu(a) * b               (silu_xquant,    kernels.rs:151-188) */
    STRIX_PRE_GEGLU = 3    /* x = gelu_tanh(a) * b          (geglu_xquant,   kernels.rs:190-226) */
};

typedef struct strix_cuda_opts {
    /* Row-sharding across a group of accelerators (one process per GPU).
     * rank r of `world` adopts rows [shard_begin(r), shard_begin(r+1)) of every
     * uploaded weight; world <= 1 means no sharding. No counterpart in the
     * reference, which is single-device (hip.rs:149). */
    int rank;
    int world;
    /* 1 = time every launch with CUDA events and keep per-kernel totals
     * (the reference's STRIX_PROF, decode.rs:25-69); read them with
     * strix_cuda_profile_dump. Launches no longer overlap while it is on (an
     * event sits between them), and launches made inside a stream capture are
     * not timed. */
    int profile;
    int reserved[5];
} strix_cuda_opts;

/* prof_dump (decode.rs:36-69): the per-kernel totals gathered since the last call (opts.profile or
 * set_option("profile", 1)), most expensive first, as text. Waits for the device. Returns the length of the whole
 * text; with buf != NULL at most cap - 1 characters and a 0 are written to it and the totals are reset; with
 * buf == NULL (a sizing call) nothing is reset. */
STRIX_API size_t strix_cuda_profile_dump(strix_cuda *h, char *buf, size_t cap);

/* RocmWeightAccel::new (decode.rs:565-829). `opts` may be NULL. */
STRIX_API int strix_cuda_create(int device, const strix_cuda_opts *opts, strix_cuda **out);
STRIX_API void strix_cuda_destroy(strix_cuda *h);
/* Text of the last error on this handle ("" if none). Valid until the next call. */
STRIX_API const char *strix_cuda_last_error(strix_cuda *h);
/* Error text for a failed strix_cuda_create (no handle exists then). */
STRIX_API const char *strix_cuda_create_error(void);

/* WeightAccel::name (accel.rs:405), ::resident_count (accel.rs:402). */
STRIX_API const char *strix_cuda_name(strix_cuda *h);
STRIX_API size_t strix_cuda_resident_count(strix_cuda *h);

/* WeightAccel::upload_q4_0 (accel.rs:150; decode.rs:2491-2521),
 * ::upload_q8_0 (accel.rs:163; decode.rs:2683-2714),
 * ::upload_q6_k (accel.rs:159; decode.rs:2629-2681).
 * `bytes` = raw GGUF blocks, row-major [out_dim][in_dim/blk][blk_bytes], copied
 * before return. Declines (0) when in_dim is not a multiple of the block size
 * or len != out_dim * (in_dim/blk) * blk_bytes, as the reference does. */
STRIX_API int strix_cuda_upload_q4_0(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len,
                           size_t in_dim, size_t out_dim);
STRIX_API int strix_cuda_upload_q8_0(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len,
                           size_t in_dim, size_t out_dim);
STRIX_API int strix_cuda_upload_q6_k(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len,
                           size_t in_dim, size_t out_dim);
/* WeightAccel::upload_q4_1 (accel.rs:154; decode.rs:2588-2627): 20-byte blocks [d f16][m f16][16 code bytes],
 * value = d * code + m; llama.cpp keeps early-layer ffn_down in this format. Same guards as upload_q4_0. */
STRIX_API int strix_cuda_upload_q4_1(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len,
                           size_t in_dim, size_t out_dim);
/* WeightAccel::upload_f32 (accel.rs:413; decode.rs:3908-3912): norm weights. */
STRIX_API int strix_cuda_upload_f32(strix_cuda *h, const char *key, const float *data, size_t n);

/* Shape of an adopted weight: rows held by THIS accelerator (its shard) and the
 * first global row of the shard. 0 if `key` is not resident. */
STRIX_API int strix_cuda_weight_info(strix_cuda *h, const char *key, size_t *in_dim, size_t *out_dim_total,
                           size_t *shard_row0, size_t *shard_rows, int *ggml_type);

/* WeightAccel::gemv (accel.rs:391; decode.rs:3827-3898): y = W x on a resident
 * weight; H2D x, one launch, sync, D2H y. 0 when `key` is not resident or
 * k != in_dim (the reference returns None). y receives this accelerator's
 * shard rows (all rows when unsharded); y_cap is y's capacity in floats.
 * `act` selects STRIX_ACT_F32 or STRIX_ACT_Q8DOT. */
STRIX_API int strix_cuda_gemv(strix_cuda *h, const char *key, const float *x, size_t k, float *y, size_t y_cap,
                    int act);
/* WeightAccel::gemv_batch (accel.rs:397-399; decode.rs:3227-3255): n GEMVs, one
 * sync. status[i] receives 1/0 per item as gemv would return. */
STRIX_API int strix_cuda_gemv_batch(strix_cuda *h, size_t n, const char *const *keys, const float *const *xs,
                          const size_t *ks, float *const *ys, const size_t *y_caps, int act, int *status);

/* Device-resident GEMV: d_y[shard_rows] = W * pre(d_a, d_b) on `stream`.
 * `pre` is a STRIX_PRE_* op: NONE reads x = d_a; RMSNORM uses d_b as the norm
 * weight and `eps`; SWIGLU/GEGLU combine gate d_a with up d_b. No copy, no sync.
 * Up to 3 weights that share the activation run as one launch (the reference's
 * q4_gemv_dp2 / _dp3, kernels.rs:228-255, 324-361): pass their keys and outputs. */
STRIX_API int strix_cuda_gemv_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_a,
                        const float *d_b, float eps, int pre, int act, float *const *d_ys, void *stream);
/* The same with a fused residual add: d_ys[m][r] = (W_m x)[r] + d_res[m][r] (d_res[m] may be null; it
 * may equal d_ys[m]). This is the reference's q4_gemv_w_add / accumulate-into-h form of the o and down
 * projections (decode.rs:5390-5400, 5470-5477). With row shards, d_res[m] points at this shard's
 * rows of the residual vector. */
STRIX_API int strix_cuda_gemv_res_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_a,
                            const float *d_b, float eps, int pre, int act, float *const *d_ys,
                            const float *const *d_res, void *stream);

/* Row-sharded multi-GPU form of the device GEMV (no counterpart in the reference, which is
 * single-GPU): instead of a local output shard, every output row r of weight m is stored into
 * peer_ys[m * n_peers + p][row0_m + r] for p < n_peers - the FULL output vectors of all accelerators
 * of the group (peer-mapped device memory, this accelerator's own copy among them), so that no
 * all-gather follows. d_res (may be null, entries may be null) are this shard's rows of residual
 * vectors. The stores are plain peer stores; they are complete when the kernel is, and
 * strix_cuda_peer_barrier_dev after it on every rank's stream makes them safe to read.
 * A chain of such launches needs that barrier between steps; the persistent chain kernel behind
 * strix_cuda_configure_decode on a sharded handle carries the exchange inside one launch instead. */
STRIX_API int strix_cuda_gemv_peers_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_a,
                              const float *d_b, float eps, int pre, int act, const float *const *d_res,
                              int n_peers, float *const *peer_ys, void *stream);
/* Lets kernels of this accelerator's device store into memory of `peer_device` (as mapped into this
 * process, e.g. through CUDA IPC). 1 = enabled (or already so), 0 = the devices cannot reach each other. */
STRIX_API int strix_cuda_enable_peer_access(strix_cuda *h, int peer_device);
/* Maps memory that another process exported with cudaIpcGetMemHandle (64 bytes) for the kernels of this
 * accelerator's device; *out is the base of the exported allocation. Open a given handle once. */
STRIX_API int strix_cuda_ipc_open(strix_cuda *h, const void *handle, size_t handle_len, void **out);
STRIX_API int strix_cuda_ipc_close(strix_cuda *h, void *p);
/* The CUDA IPC handle (64 bytes) of the device allocation that starts at d_ptr (e.g. the exchange block of
 * strix_cuda_decode_exchange_info), for another process to open with strix_cuda_ipc_open. */
STRIX_API int strix_cuda_ipc_export(strix_cuda *h, const void *d_ptr, void *handle, size_t handle_cap);
/* One 32-bit word of device (or peer-mapped) memory, by a copy engine transfer: lets a caller check a
 * mapping it was handed before any kernel stores through it. */
STRIX_API int strix_cuda_peek_u32(strix_cuda *h, const void *d_ptr, uint32_t *out);
/* The counterpart: writes one word (e.g. the mark a peer then reads back through its mapping). */
STRIX_API int strix_cuda_poke_u32(strix_cuda *h, void *d_ptr, uint32_t value);
/* Cross-GPU barrier for the form above: one launch per rank (opts.rank / opts.world of the handle), one
 * rank per GPU. d_epoch: one zero-initialised word of this rank; d_local_flags: `world` zero-initialised
 * words of this rank; peer_flags[i]: rank i's flag array as mapped into this process. The wait is
 * bounded; on expiry the handle's status word gets the time-out bit and the kernel returns. */
STRIX_API int strix_cuda_peer_barrier_dev(strix_cuda *h, uint32_t *d_epoch, uint32_t *d_local_flags,
                                uint32_t *const *peer_flags, void *stream);

/* WeightAccel::gemv_batch (accel.rs:397-399; decode.rs:3227-3255) for device-resident vectors: n INDEPENDENT GEMVs,
 * d_ys[i] = W(keys[i]) d_xs[i], enqueued from `stream` (no copies, no synchronisation). Independent means: no item
 * reads or writes what another writes; the items then need not run in the order given. Items whose weights are at
 * most "batch_small_bytes" (set_option; 256 MiB) run SIDE BY SIDE in one launch, up to 6 per launch: its CTAs are
 * dealt out among the items by their bytes, so the launch fills and drains once for all of them (a launch of its
 * own costs such an item more in fill and drain than its weights take to stream). The others get a launch each,
 * before it. The host-pointer form strix_cuda_gemv_batch splits a batch the same way.
 * set_option("batch_side_by_side", 0) gives every item its own launch, 2 runs all items side by side.
 * Because the items are independent, only the batch's FIRST launch waits for the work that precedes the call on
 * `stream`; every later launch starts its row groups as soon as its CTAs get an SM, beside the tail of the launch
 * before it, and waits for that launch only at its own end, so that the batch still completes in stream order
 * (set_option("batch_overlap", 0): every launch waits before it reads its activation, as an ordinary GEMV does).
 * All activations must therefore come from work that precedes the call on `stream` (or be complete already); none may
 * be written by an item of the batch.
 * 0 = an unknown key or a null vector. */
STRIX_API int strix_cuda_gemv_batch_dev(strix_cuda *h, size_t n, const char *const *keys, const float *const *d_xs,
                              float *const *d_ys, int act, void *stream);
/* The row-sharded form of strix_cuda_gemv_batch_dev (no counterpart in the reference, which is single-device,
 * hip.rs:149; BASELINE's "output all-gather" fused into the kernels): item i's rows are stored by the kernels
 * themselves into the FULL output vector of weight i on every accelerator of the group,
 * peer_ys[i * n_peers + p][row0 + r] for p < n_peers (peer-mapped device memory, see strix_cuda_ipc_open; this GPU's
 * own copy is one of them), with plain stores over NVLink. No collective follows; strix_cuda_peer_barrier_dev on the
 * same stream makes the vectors safe to read on every rank. */
STRIX_API int strix_cuda_gemv_batch_peers_dev(strix_cuda *h, size_t n, const char *const *keys, const float *const *d_xs,
                                    int n_peers, float *const *peer_ys, int act, void *stream);
/* WeightAccel::prefill_q8_gemm (accel.rs:213; decode.rs:3257-3297): y[m][rows] = W8A8 GEMM of m
 * token rows xs[m][in_dim] with a resident Q8_0 weight: per-32 int8 activations (xquant8_rows,
 * kernels.rs:1000-1013), int32 block sums on tcgen05, f32 combine with both block scales
 * (q8w_gemm32, kernels.rs:1373-1443); split-K over long in_dim (the reference's q4_gemm_w_sk,
 * kernels.rs:539-601, with a fixed-order reduction instead of atomics). 0 when `key` is not a
 * resident Q8_0 weight. Unlike the reference (m <= 256, out_dim <= 8192) any m is accepted. */
STRIX_API int strix_cuda_prefill_q8_gemm(strix_cuda *h, const char *key, const float *xs, size_t m, float *y,
                               size_t y_cap);
/* The same on device pointers: d_y[m][rows] from d_xs[m][in_dim] on `stream`; no copy, no sync. */
STRIX_API int strix_cuda_prefill_q8_gemm_dev(strix_cuda *h, const char *key, const float *d_xs, size_t m, float *d_y,
                                   void *stream);
/* The prefill GEMM with a resident Q4_0 weight: the reference's q4_gemm_w / q4_gemm_w_sk (kernels.rs:443-601;
 * dispatch decode.rs:5655-5720), Q4_0 weights x per-32 int8 activations, int32 block sums (sum of (nibble - 8) * xq,
 * exact), f32 combine with both block scales, split-K with a fixed-order reduction. Runs on the same tcgen05 kernel:
 * on first use the weight gets a byte-per-code copy ((nibble - 8) + 128, row-major) next to its tile-major form.
 * 0 when `key` is not a resident Q4_0 weight. */
STRIX_API int strix_cuda_prefill_q4_gemm(strix_cuda *h, const char *key, const float *xs, size_t m, float *y,
                               size_t y_cap);
STRIX_API int strix_cuda_prefill_q4_gemm_dev(strix_cuda *h, const char *key, const float *d_xs, size_t m, float *d_y,
                                   void *stream);

/* No counterpart in the reference. The W8A8 GEMM for callers that must not allocate device memory
 * (a server whose arena owns the whole device; a latency-critical path that cannot risk the
 * device-wide synchronisation of cudaMalloc/cudaFree): same kernels and result as
 * strix_cuda_prefill_q8_gemm_dev, but ALL scratch comes from one fixed device array built into the
 * library (strix_cuda_noalloc_scratch_bytes() = 32 MiB per GPU, held until process exit). Calls no
 * cudaMalloc/cudaFree. A shape whose scratch exceeds the array returns <0 with the sizes in the
 * error text. The driver materialises the array's memory and the kernels' code when they are first
 * touched, which can allocate: strix_cuda_create does that touching (address look-up with the handle's
 * device current, kernel attributes), so create the handle before the arena takes the device. (Only for
 * a device with no handle from strix_cuda_create would the first call do the look-up itself: keep
 * that call outside any stream capture.) Every call shares the array (it keeps the last call's contents; nothing needs
 * zeroing), so calls whose kernels overlap on the GPU race: serialise them. */
STRIX_API int strix_cuda_prefill_q8_gemm_noalloc(strix_cuda *h, const char *key, const float *d_xs, size_t m,
                                       float *d_y, void *stream);
STRIX_API size_t strix_cuda_noalloc_scratch_bytes(void);

/* WeightAccel::upload_moe_q8 / upload_moe_q6 (accel.rs:167-196; decode.rs:2717-2831): adopt a whole
 * mixture-of-experts layer: gate and up hold ne experts of [eff][hidden] raw GGUF blocks back to back, down ne
 * experts of [hidden][eff] (Q8_0 34-byte blocks / Q6_K 210-byte super-blocks). 1 = adopted, 0 = declined as the
 * reference declines (hidden or eff not whole blocks or above 4096, a length that does not match) or on a
 * row-sharded handle, <0 = error. The experts of a projection become one resident stack that the GEMV kernel
 * indexes by expert id. */
STRIX_API int strix_cuda_upload_moe_q8(strix_cuda *h, size_t layer, const uint8_t *gate, size_t gate_len, const uint8_t *up,
                             size_t up_len, const uint8_t *down, size_t down_len, size_t hidden, size_t eff, size_t ne);
STRIX_API int strix_cuda_upload_moe_q6(strix_cuda *h, size_t layer, const uint8_t *gate, size_t gate_len, const uint8_t *up,
                             size_t up_len, const uint8_t *down, size_t down_len, size_t hidden, size_t eff, size_t ne);
/* WeightAccel::moe_ffn (accel.rs:198-211; decode.rs:2833-2870): y[hidden] = sum_i wexp[i] *
 * down_{ids[i]}(silu(gate_{ids[i]} x) * up_{ids[i]} x) over the k <= 16 routed experts of one token, in the order
 * given, plus sgate * the shared expert (blk.<layer>.ffn_{gate,up,down}_shexp.weight, resident through the usual
 * uploads) when sgate != 0. act: STRIX_ACT_F32 (the reference's default kernels) or STRIX_ACT_Q8DOT (its
 * integer-dot kernels, q8i_moe_*). 1 = done, 0 = None in the reference (layer not adopted, a length mismatch,
 * k = 0 or > 16, an id outside [0, ne), a shared expert asked for but not resident), <0 = error. */
STRIX_API int strix_cuda_moe_ffn(strix_cuda *h, size_t layer, const int *ids, const float *wexp, size_t k, const float *x,
                       size_t x_len, float sgate, int act, float *y, size_t y_cap);
/* The same with ids, weights, x and y on the device, enqueued on `stream`, no synchronisation (the router's top-k
 * can stay on the device: strix_cuda_topk_router_dev). An id outside [0, ne) is clamped into the range. */
STRIX_API int strix_cuda_moe_ffn_dev(strix_cuda *h, size_t layer, const int *d_ids, const float *d_wexp, size_t k,
                           const float *d_x, float sgate, int act, float *d_y, void *stream);
/* WeightAccel::moe_expert_ffn (accel.rs:220-223; decode.rs:3299-3356): m grouped tokens xs[m][hidden] through
 * expert e: y[m][hidden] = down_e(silu(gate_e xs) * up_e xs), the weights read once per 8 tokens. */
STRIX_API int strix_cuda_moe_expert_ffn(strix_cuda *h, size_t layer, size_t e, const float *xs, size_t m, int act, float *y,
                              size_t y_cap);
/* WeightAccel::moe_layer_ffn (accel.rs:236-246; decode.rs:3552-3630): plan[n_plan] pairs (expert id, row count);
 * xs[rows][hidden] gathered expert-major in plan order; y[rows][hidden] the experts' outputs in the same order.
 * 0 = None (unknown layer, an id out of range, counts that do not add up to rows). */
STRIX_API int strix_cuda_moe_layer_ffn(strix_cuda *h, size_t layer, const int *plan, size_t n_plan, const float *xs, size_t rows,
                             int act, float *y, size_t y_cap);
/* The router's top-k (mellum.rs:1590-1609; the reference's topk_router kernel, kernels.rs:1846-1873): softmax over
 * logits[ne <= 128], the k <= 16 most probable experts (a tie goes to the lower index), weights = their
 * probabilities divided by the sum of the chosen ones. 0 = sizes out of range. */
STRIX_API int strix_cuda_topk_router(strix_cuda *h, const float *logits, size_t ne, size_t k, int *ids, float *w);
STRIX_API int strix_cuda_topk_router_dev(strix_cuda *h, const float *d_logits, size_t ne, size_t k, int *d_ids, float *d_w,
                               void *stream);

/* Plain-data mirror of GpuLayerCfg / GpuDecodeConfig (crates/strix-core/src/accel.rs:19-72). */
typedef struct strix_gpu_layer_cfg {
    uint32_t head_dim, n_kv;
    int k_eq_v;
    float rope_theta;
    int is_local;
    float output_scale;
    int no_rope, rope_norm;
} strix_gpu_layer_cfg;
typedef struct strix_gpu_decode_config {
    uint32_t hidden, n_heads, ffn, vocab, n_layers;
    float eps, final_softcap;
    int attn_rsqrt, norm_v, qk_norm, post_norm, act_gelu, gpu_prefill;
    uint32_t n_swa, max_seq;
    const strix_gpu_layer_cfg *layers; /* n_layers entries; may be NULL (unused by the projection chain) */
    /* Not in the reference struct: */
    int attn_standin_q; /* 1: projection chain only, Wo is fed with q (no KV cache). 0: real attention over a KV cache
                         * of max_seq rows in the flavours of the reference's forwards; `layers` must then describe
                         * every layer (see strix_cuda_configure_decode) */
    int act;            /* STRIX_ACT_F32 or STRIX_ACT_Q8DOT for every projection */
} strix_gpu_decode_config;

/* WeightAccel::configure_decode (accel.rs:417; decode.rs:4528-4622). Call after every weight
 * (blk.N.attn_q/attn_k/attn_v/attn_output/ffn_gate/ffn_up/ffn_down.weight, output.weight or
 * token_embd.weight) and norm (blk.N.attn_norm/ffn_norm.weight, output_norm.weight via upload_f32)
 * is uploaded; with qk_norm also blk.N.attn_q_norm / attn_k_norm.weight (head_dim floats); with post_norm
 * blk.N.post_attention_norm / post_ffw_norm.weight (hidden floats); optionally rope_freqs.weight.
 * Real attention (attn_standin_q = 0) follows the reference's forwards field by field:
 *   head_dim, n_kv   per layer (<= 512, a multiple of 4; n_heads a multiple of n_kv)
 *   k_eq_v           no V projection on that layer: V is the raw K projection, taken before the K-norm
 *   norm_v           V RMS-normalised per head without a weight
 *   qk_norm          per-head RMSNorm of q and k before the rope
 *   no_rope, rope_norm (pairs (2k, 2k+1) instead of (k, k + head_dim/2)), rope_theta per layer. The angle of
 *                    pair j is pos * theta^(-2j/hd) / rope_freqs[j] (factors on non-local layers, when uploaded)
 *                    for a post_norm model (the Gemma forward, ops.rs:159-176), else the running product
 *                    pos * (theta^(-2/hd))^j of the Qwen3 / SmolLM3 forwards (qwen3.rs:126-138)
 *   is_local + n_swa a local layer attends only to the last n_swa cached rows (decode.rs:5312-5325)
 *   attn_rsqrt       scores scaled by 1/sqrt(head_dim), else by 1
 *   post_norm        h += rmsnorm(Wo a) * post_attention_norm; h = (h + rmsnorm(Wd act) * post_ffw_norm) * output_scale
 *   final_softcap    > 0: logits = cap * tanh(logits / cap) on every logits-returning call (the argmax calls skip it)
 * set_option("kv_f16", 1) before this call keeps the cache in f16 (the reference's STRIX_F16_KV), rows rounded
 * to nearest with ties away from zero as the reference's stores do (kernels.rs:18-32).
 * 0 = declined (a weight or norm missing, a head size out of range, or a sharded handle asking for anything
 * but the integer-dot projection chain without post_norm): the model keeps its per-weight gemv path. Any later
 * upload drops the configuration. */
STRIX_API int strix_cuda_configure_decode(strix_cuda *h, const strix_gpu_decode_config *cfg);
/* WeightAccel::decode_step (accel.rs:433; decode.rs:5047-5531): logits[vocab] from the embedded hidden
 * state hvec[hidden]. With the attention stand-in and integer-dot activations the whole chain is ONE
 * persistent launch (steps hand their outputs on through exchange vectors, no barrier between them);
 * otherwise four GEMV launches per layer (plus three small attention kernels with real attention),
 * replayed from a CUDA graph. With real attention row `pos` of the KV cache is written and
 * rows 0..pos are attended to (pos >= max_seq is an error); with the stand-in `pos` has no effect.
 * 0 = not configured. */
STRIX_API int strix_cuda_decode_step(strix_cuda *h, const float *hvec, size_t pos, float *logits, size_t logits_cap);
/* WeightAccel::decode_step_argmax (accel.rs:437-442; decode.rs:5497-5515, 5533-5538): the same step,
 * then the argmax over the logits on the device; only the winning token id crosses back (4 bytes
 * instead of vocab * 4). Ties resolve to the lowest index, NaN never wins, as in the reference's
 * argmax_f32 (kernels.rs:2088-2110). 0 = not configured, or a row-sharded handle. */
STRIX_API int strix_cuda_decode_step_argmax(strix_cuda *h, const float *hvec, size_t pos, uint32_t *id);
/* WeightAccel::lm_head_argmax_rows (accel.rs:216-219; decode.rs:3631-3689): ids[t] = argmax over the
 * rows of W xs[t], t < m, with one pass over the weights per chunk of activation rows and the argmax
 * on the device. xs_len must be m * in_dim and m <= 16, else 0 (None), as in the reference; unlike
 * the reference any resident format is accepted (`act` picks the f32 or the integer-dot GEMV).
 * ids are row indices of the whole weight; a row-sharded handle returns the winner among ITS rows, and
 * vals (may be null) receives the winning values so that the caller can fold the shards. */
STRIX_API int strix_cuda_lm_head_argmax_rows(strix_cuda *h, const char *key, const float *xs, size_t xs_len, size_t m,
                                             int act, uint32_t *ids, float *vals);
/* Folds the per-shard winners of a row-sharded lm_head_argmax_rows (ids / vals: [n_shards][m], shards in rank order)
 * into the winners over the whole weight with the kernel's rule: a value replaces the running best (-3.0e38, row 0)
 * only if it is greater, or equal with a lower row index; NaN never wins (argmax_f32, kernels.rs:2088-2110).
 * Host-side; needs no handle. */
STRIX_API void strix_cuda_fold_argmax_shards(size_t n_shards, size_t m, const uint32_t *ids, const float *vals,
                                             uint32_t *out_ids, float *out_vals);
/* argmax per row of a device matrix d_x[rows][stride] (n entries per row, rows <= 16) on `stream`;
 * d_ids[rows] / d_vals[rows] (either may be null) are device pointers. No sync. The per-block winners, tickets and
 * results are one scratch set per handle: argmax calls on one handle must be serialised (one stream at a time). */
STRIX_API int strix_cuda_argmax_dev(strix_cuda *h, const float *d_x, size_t n, size_t stride, size_t rows,
                                    uint32_t *d_ids, float *d_vals, void *stream);
/* WeightAccel::prefill (accel.rs:464-473; decode.rs:5555-6394): m tokens hs[m][hidden] at positions
 * start_pos .. start_pos + m - 1 in ONE pass over the weights per projection (the rows ride through the
 * batched GEMV as extra tensor-core columns), causal attention row after row, KV cache filled for those
 * positions; logits[vocab] of the LAST token. 0 = not configured, m == 0 or m > strix_cuda_prefill_max
 * (the caller chunks, as with the reference's M_CHUNK). */
STRIX_API int strix_cuda_prefill(strix_cuda *h, const float *hs, size_t start_pos, size_t m, float *logits,
                                 size_t logits_cap);
/* WeightAccel::verify (accel.rs:500-506; decode.rs:5548-5553): the same, logits[m][vocab] of ALL tokens
 * (speculative-decoding verify of gamma + 1 rows). */
STRIX_API int strix_cuda_verify(strix_cuda *h, const float *hs, size_t start_pos, size_t m, float *logits,
                                size_t logits_cap);
/* verify, greedy form: ids[m] = argmax of each of the m rows' logits, taken on the device (4 m bytes come back instead
 * of m * vocab floats): what the speculative loops compare the proposals with (generate.rs:644-651, 873-878). */
STRIX_API int strix_cuda_verify_argmax(strix_cuda *h, const float *hs, size_t start_pos, size_t m, uint32_t *ids);
/* WeightAccel::prefill_max (accel.rs:475-479): tokens one prefill / verify call accepts (8), 0 = no decode configured. */
STRIX_API size_t strix_cuda_prefill_max(strix_cuda *h);
/* WeightAccel::seed_decode_kv (accel.rs:421-427): fill cache rows 0 .. tokens-1 of layer il from a prefill
 * done elsewhere (k normed and roped, v raw, token-major [tokens][n_kv * head_dim]). 0 = no real-attention
 * configuration, il or tokens out of range. */
STRIX_API int strix_cuda_seed_decode_kv(strix_cuda *h, size_t il, const float *k, const float *v, size_t tokens);
/* Row-sharded decode (no counterpart in the reference, which is single-device): on handles created with
 * world > 1, configure_decode accepts the projection chain (attn_standin_q = 1, STRIX_ACT_Q8DOT). Every
 * rank runs the persistent chain kernel over its row shards and publishes each step's rows into the
 * exchange block of EVERY rank with plain peer stores (8-byte {value, epoch} entries; no collective, no
 * barrier launch, no multicast); a rank's consumers poll their own block. strix_cuda_decode_exchange_info
 * returns this rank's block (one cudaMalloc allocation, exportable with strix_cuda_ipc_export; its last 128
 * bytes are spare, for a mark that lets the peers check their mapping before any kernel stores through it);
 * strix_cuda_decode_set_peers hands over all ranks' blocks as mapped into this process (entry `rank` may
 * be null). Until the group is wired a rank publishes into its own block only, so its waits for the other
 * ranks' rows run out: bounded (option "poll_limit"), the status word gets the time-out bit, the call
 * returns -2 and the handle stays usable. decode_step / decode_chain_dev then return this rank's shard of
 * the logits (rows shard_row0 .. of the head). All ranks must make the same sequence of decode calls. */
STRIX_API int strix_cuda_decode_exchange_info(strix_cuda *h, void **base, size_t *bytes);
STRIX_API int strix_cuda_decode_set_peers(strix_cuda *h, int n, void *const *blocks);
/* The same chain on device pointers (d_h is updated in place; a row-sharded handle leaves it as it was),
 * enqueued on `stream`; no copy, no sync. */
STRIX_API int strix_cuda_decode_chain_dev(strix_cuda *h, float *d_h, float *d_logits, void *stream);

/* Batched GEMV for speculative verify (the reference runs its verify rows through the 128-token
 * prefill GEMM, decode.rs:5548-5553, 6366-6410): ys[b][rows] = W xs[b][in_dim] for b activation rows
 * with ONE pass over the weights per chunk of up to 8 rows. Host buffers, one sync. */
STRIX_API int strix_cuda_gemv_rows(strix_cuda *h, const char *key, const float *xs, size_t b, float *y, size_t y_cap,
                         int act);
/* The same on device pointers, up to 3 weights that share the activations per launch; no copy, no sync. */
STRIX_API int strix_cuda_gemv_rows_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_xs, size_t b,
                             int act, float *const *d_ys, void *stream);

/* Device status word written by kernels whose bounded waits ran out
 * (0 = clean). Synchronises `stream`. */
STRIX_API int strix_cuda_device_status(strix_cuda *h, void *stream, uint32_t *status);
/* Resets the status word (the host-buffer entry points do so themselves when they report it with -2; a
 * caller of the _dev entry points that has seen a non-zero status clears it here). Synchronises `stream`. */
STRIX_API int strix_cuda_clear_device_status(strix_cuda *h, void *stream);

/* ---- test / measurement extras (not part of the trait) ---- */

/* Planning and measurement knobs of one handle, by name (the reference reads such knobs from the
 * environment, e.g. STRIX_NO_SPLITK / STRIX_SK / STRIX_PROF, decode.rs:5652-5671, 25-31; here nothing on
 * the call path reads the environment). 1 = set, 0 = unknown name. Any configured decode chain and cached
 * graph is dropped. Names: "q6k_digits" (0 never / 1 in_dim <= 8192 / 2 whenever it fits: Q6_K f32 row as
 * three int8 digit rows), "q8_0_digits" / "q4_0_digits" (the same for Q8_0 / Q4_0), "gemv_warps_per_group", "gemv_blocks_per_stage", "gemv_stages" (0 = planned),
 * "gemv_pdl" (programmatic dependent launch between GEMVs), "rows_operand_image" (batched integer-dot GEMV:
 * the activation operands are prepared once by a kernel of their own and fetched by every CTA; 0 = every CTA
 * quantises all rows itself), "operand_image_min_k" (a single row is prepared that way too from this in_dim on;
 * 8192), "gemv_debug" (bit 0: stream the weights without
 * arithmetic, bit 1: empty launches, bit 2: stop after the activation prologue), "batch_graph" (gemv_batch
 * replays a cached CUDA graph), "batch_side_by_side" / "batch_small_bytes" (which items of a gemv_batch share a launch,
 * see strix_cuda_gemv_batch_dev), "batch_overlap" (later launches of a batch do not wait for earlier ones; 1),
 * "decode_chain" (the projection chain as one persistent launch),
 * "kv_f16" (real attention keeps its KV cache in f16),
 * "chain_trace" (per-step clocks, see strix_cuda_decode_trace), "chain_debug" (bit 0: the chain kernel skips
 * the arithmetic, bit 1: its waits on exchange vectors do not wait; results are then meaningless), "poll_limit" (bound, in polls, of a wait on
 * an exchange vector; 0 = default), "profile" (as strix_cuda_opts.profile). */
STRIX_API int strix_cuda_set_option(strix_cuda *h, const char *name, long long value);
/* After set_option("chain_trace", 1): per step of the last decode-chain launch, 6 words from its CTA 0: the
 * clock (ns) at the step's start, when its activations had arrived, after its prologue, after its last row
 * group, after its reduction and stores; and the SM clocks spent waiting for weight stages. Returns the
 * number of steps (0 = no trace, or `cap_words` too small). Synchronises. */
STRIX_API int strix_cuda_decode_trace(strix_cuda *h, unsigned long long *out, size_t cap_words);

/* Dequantise a resident weight back to f32 [shard_rows][in_dim] on the host:
 * must equal dequantize_into (ggml_quant.rs:139-183) bit for bit. */
STRIX_API int strix_cuda_dequant_to_f32(strix_cuda *h, const char *key, float *out, size_t out_cap);
/* The activation quantiser alone (xquant8_rows, kernels.rs:1000-1013):
 * q[n] int8 and d[n/32] f32 from x[n], n a multiple of 32. */
STRIX_API int strix_cuda_xquant8(strix_cuda *h, const float *x, size_t n, int8_t *q, float *d);

/* int32 block sums isum[m][rows][in_dim/32] of a resident Q8_0 or Q4_0 weight with the int8 codes of
 * xs[m][in_dim] (the bit-exact tier of the GEMM, q8w_gemm32's per-block accumulator, kernels.rs:1417-1428),
 * computed by a plain integer loop without tensor cores. */
STRIX_API int strix_cuda_debug_block_isums(strix_cuda *h, const char *key, const float *xs, size_t m, int32_t *out,
                                 size_t out_cap);
/* The same sums as the prefill GEMM's own tcgen05 kernel produces them: its producer, MMA and TMEM pipeline
 * unchanged, with an epilogue that stores each block's integer instead of folding it into f32. `splits`:
 * split-K slices (0 = what strix_cuda_prefill_q8_gemm would pick). An entry the kernel does not write reads -1. */
STRIX_API int strix_cuda_debug_gemm_isums(strix_cuda *h, const char *key, const float *xs, size_t m, uint32_t splits,
                                int32_t *out, size_t out_cap);
/* Measurement: quantise d_xs[m][in_dim] once, then launch the GEMM kernel `reps` times on `stream` in `mode`:
 * 0 = the product into d_y[m][rows]; 2 = without the accumulator drain (TMA + tensor pipeline alone);
 * 3 = without drain and loads (the issue loop with its buffer hand-overs only); 4 = the MMAs alone, issued
 * back to back with one commit at the end (the issue rate of tcgen05.mma kind::i8: the measured int8 peak).
 * No sync. */
STRIX_API int strix_cuda_debug_gemm_mode_dev(strix_cuda *h, const char *key, const float *d_xs, size_t m, float *d_y,
                                   int mode, int reps, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* STRIX_CUDA_H */
