// Host-callable launchers of the CUDA kernels (internal to the library).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "layout.h"

namespace strix {

// Regroups raw GGUF rows [row0, row0 + n) of a shard (row0 a multiple of 16) into the resident shard;
// for Q8_0, d_gemm_codes (may be null) also receives the codes row-major for the prefill GEMM.
cudaError_t launch_repack(int fmt, const uint8_t *d_raw, uint8_t *d_res, uint8_t *d_gemm_codes, const RowLayout &L,
                          uint32_t row0, uint32_t n, cudaStream_t stream);
cudaError_t launch_dequant(const uint8_t *d_res, float *d_out, const RowLayout &L, uint32_t rows,
                           cudaStream_t stream);

// ---- dequant-GEMV -------------------------------------------------------
constexpr int GEMV_MAX_MATS = 3;
constexpr int GEMV_MAX_PEERS = 8;
constexpr int GEMV_MAX_STAGES = 96;
// Consumer warps per CTA (plus one producer warp), one CTA per SM: six per scheduler.
constexpr int GEMV_WARPS = 24;
constexpr int gemv_warps(int /*act*/) { return GEMV_WARPS; }

struct GemvMat {
    const uint8_t *w;  // resident rows of this accelerator's shard
    float *y;          // output, one float per resident row
    const float *res;  // optional residual added to the output (y = W x + res); may alias y
    uint32_t rows;
    uint32_t ystride;  // floats between the outputs (and residuals) of consecutive activation rows
    uint32_t tile0;  // index of this matrix's first tile in the launch-wide tile list
    // Row-sharded multi-GPU form: every output is also stored into the FULL output vector of each of
    // n_peer accelerators (peer-mapped device memory, this GPU's own copy included), at row_base + row.
    float *peer_y[GEMV_MAX_PEERS];
    uint32_t n_peer;
    uint32_t row_base;
};

struct GemvArgs {
    GemvMat mat[GEMV_MAX_MATS];  // tile0 = index of the matrix's first row group in the launch-wide list
    int nmat;
    RowLayout L;
    const float *a;  // activation (or gate) vector, in_dim floats
    const float *b;  // norm weight (RMSNORM) or up vector (SWIGLU/GEGLU); unused for NONE
    uint32_t nbatch;             // activation rows that share the weights (1 = plain GEMV)
    uint32_t a_stride, b_stride;  // floats between consecutive activation rows of a / b (0 = shared)
    float eps;
    int pre;  // STRIX_PRE_*
    int act;  // STRIX_ACT_*
    uint32_t rows_per_tile;  // rows of a row group (16)
    uint32_t n_tiles;        // row groups of the launch, over all its matrices
    uint32_t stage_bytes;    // multiple of 128
    uint32_t stage_off;      // byte offset of the first stage in dynamic shared memory
    uint32_t x_off;          // byte offset of the activation operands in dynamic shared memory
    uint32_t n_stages;       // stages in each slot's ring
    uint32_t wc;             // warps that share a row group (they split its tiles along K)
    uint32_t slots;          // groups of wc warps, each working on a different row group
    uint32_t chunk_tiles;    // GGUF blocks of K per stage
    uint32_t n_chunks;       // stages per row group
    uint32_t multi;          // integer form with more than one activation row (Q4_0 / Q8_0)
    uint32_t digits;         // f32 activations carried as three int8 digits per value (Q6_K, one activation row)
    uint32_t pdl;            // launch with programmatic stream serialization
    uint32_t rot;            // chain kernel: CTA that takes the step's first row group
    // Place among the launches of a batch of INDEPENDENT items (activations all there before the batch starts, outputs
    // disjoint), which have no reason to wait for one another. 0 = an ordinary launch: dependents may be scheduled
    // from its start, and it waits for the grid before it ahead of its activation prologue. 1 = the batch's first
    // launch: waits the same way, but lets dependents be scheduled only AFTER that wait, so that nothing of the batch
    // starts before the work the batch follows is complete. 2 = a later launch of the batch: runs its prologue and its
    // row groups as soon as its CTAs get an SM, and waits for the grid before it only at its end (completion stays in
    // stream order). Between two such launches no SM idles while the slowest CTA of the first one finishes.
    uint32_t order;
    // Integer-dot form with the activation operands prepared ONCE by a kernel of their own (launch_xop_prepare)
    // instead of by every CTA: the image of the shared-memory operand region (x_layout order) in global
    // memory, which each CTA fetches with bulk copies. Null = the CTA builds its operands itself.
    const uint8_t *xop;
    // Expert indirection (mixture-of-experts layers): every matrix of the launch is a stack of experts of
    // sel_groups row groups each; the launch's virtual matrix is the stack of the experts sel_ids[0], sel_ids[1], ...
    // (device words, read by the kernel), so mat[].rows = selections * rows per expert. Null = none.
    const int *sel_ids;
    uint32_t sel_groups;
    uint32_t sel_experts;  // experts in the stack; an id outside [0, sel_experts) is clamped into it (never read out of bounds)
    uint32_t grid;
    uint32_t smem_bytes;
    uint32_t debug;  // measurement only: bit 0 = stream the tiles but skip the arithmetic
    uint32_t *status;
};

// Planning knobs of one accelerator (strix_cuda_set_option; the defaults are what the planner picks).
struct GemvTune {
    uint32_t digits_rule = 1;  // Q6_K with one f32 row as three int8 digit rows: 0 never, 1 for in_dim <= 8192, 2 whenever it fits
    uint32_t q8_digits_rule = 1;  // the same for Q8_0
    uint32_t q4_digits_rule = 1;  // ... and for Q4_0
    uint32_t force_wc = 0, force_ct = 0, force_sk = 0;  // warps per row group / blocks per stage / stages per slot (0 = planned)
    uint32_t pdl = 1;          // programmatic stream serialization between GEMV launches
    uint32_t xop = 1;          // batched integer-dot GEMV: operands prepared once by a kernel of their own (0 = by every CTA)
    uint32_t xop_single_min_k = 8192;  // ... and a single activation row too, from this in_dim on (measured: decode chain 1.365 -> 1.300 ms per token
                               // with its 9728-long rows prepared this way, 1.32 from 4096 on, 1.37 from 2560 on; verify step 2.08 -> 1.98 ms)
    uint32_t debug = 0;        // measurement only: bit 0 stream the tiles without arithmetic, bit 1 empty launch,
                               // bit 2 stop after the activation prologue
};

// Fills the launch geometry (rows_per_tile .. smem_bytes, tile0 of each matrix)
// from L, mat[].rows and the device's SM count. Returns false when in_dim is
// too large for the shared-memory pipeline.
bool gemv_plan(GemvArgs &a, int num_sms, size_t smem_optin, const GemvTune &tune);
cudaError_t gemv_prepare_device(size_t smem_optin);  // opt in to large dynamic shared memory, once per device
cudaError_t launch_gemv(const GemvArgs &a, cudaStream_t stream);
// Several independent GEMVs side by side in one launch (see gemv_multi_kernel): p[i] as for launch_gemv (one weight,
// one activation row, no pre-op), planned by gemv_multi_plan, which also deals the CTAs out: problem i runs on CTAs
// [cta0[i], cta0[i + 1]).
constexpr int GEMV_MULTI_MAX = 6;
struct GemvMultiArgs {
    GemvArgs p[GEMV_MULTI_MAX];
    uint32_t n;
    uint32_t cta0[GEMV_MULTI_MAX + 1];
    uint32_t grid, smem_bytes, pdl;
    uint32_t order;  // as GemvArgs::order
};
static_assert(sizeof(GemvMultiArgs) <= 4000, "passed by value: kernel parameters are limited to 4 KB");
bool gemv_multi_plan(GemvMultiArgs &m, int num_sms, size_t smem_optin, const GemvTune &tune);
cudaError_t launch_gemv_multi(const GemvMultiArgs &m, cudaStream_t stream);
// Bytes of the operand image of nbatch activation rows (what GemvArgs::xop points at), and the kernel that
// writes it: the pre-op (RMSNorm in the reference's operand order, SwiGLU, GeGLU) and the per-32 int8
// quantiser, one CTA per activation row. a / b / strides / eps / pre as in GemvArgs.
size_t xop_image_bytes(int fmt, uint32_t in_dim, uint32_t nbatch);
cudaError_t launch_xop_prepare(int fmt, uint32_t in_dim, uint32_t nbatch, const float *d_a, const float *d_b,
                               uint32_t a_stride, uint32_t b_stride, float eps, int pre, uint8_t *d_image, bool pdl,
                               cudaStream_t stream);
// ---- step lists in one persistent launch (chain.cu) ------------------------------------------
// A list of GEMV steps run by ONE cooperative kernel (one CTA per SM): the producer warp of every CTA
// streams the weights of step after step through one ring of stages without ever waiting for another
// CTA, while the consumer warps run the steps in order. A step whose activation is the output of an
// earlier step reads it from an EXCHANGE VECTOR: 8-byte entries {f32 value, epoch}, written by the
// step that produces them (into the vector of every rank when the rows are sharded over GPUs) and
// polled by the consumers until every entry carries the epoch of this launch's producing step - the
// flag travels with the data, so there is no grid barrier, no fence and, across GPUs, no collective.
constexpr int CHAIN_PART_SLOTS = 12;    // row groups whose per-warp partial sums wait in shared memory for one reduction
constexpr int CHAIN_ACT_DIGITS = 2;     // ChainStep::act: one f32 row as three int8 digit rows (Q6_K)
constexpr uint32_t CHAIN_MAX_STAGES = 16;
constexpr uint32_t CHAIN_POLL_LIMIT = 1u << 21;  // default bound of a wait on an exchange vector (about a second)

struct ChainMat {
    const uint8_t *w;   // resident rows of this accelerator's shard
    uint32_t rows;      // rows held here
    uint32_t item0;     // index of this matrix's first row group in the step's item list
    uint32_t row_base;  // first global row of the shard: entries row_base + r of res_ll / out_ll belong to local row r
    float *y;           // plain output [rows], or null
    const float *res;   // plain residual [rows] added to the output, or null
    const unsigned long long *res_ll;             // residual taken from an exchange vector, or null
    unsigned long long *out_ll[GEMV_MAX_PEERS];   // exchange vectors the rows are published into (every rank's, own included)
    uint32_t n_out_ll;
};

struct ChainStep {
    ChainMat mat[GEMV_MAX_MATS];
    int nmat;
    RowLayout L;
    int act;   // STRIX_ACT_F32, STRIX_ACT_Q8DOT or CHAIN_ACT_DIGITS
    int pre;   // STRIX_PRE_* applied to the activation (an exchange-vector input takes NONE or RMSNORM)
    int pair;  // 0, or STRIX_PRE_SWIGLU / STRIX_PRE_GEGLU: mat[0] = gate, mat[1] = up (same rows); a work item is row
               // group g of both, and what mat[0]'s outputs receive is act(gate) * up (the next step's activation)
    const float *a, *b;           // plain activation (null with a_ll) / norm weight or up vector
    const unsigned long long *a_ll;  // activation as an exchange vector of in_dim entries, or null
    uint32_t in_step, res_step;   // steps of this list whose outputs a_ll / res_ll hold
    float eps;
    // filled by chain_plan:
    uint32_t n_items;      // work items: row groups over all matrices (pairs count once)
    uint32_t chunk_tiles;  // GGUF blocks of K per stage (per matrix of a pair)
    uint32_t n_chunks;     // stages per work item
    uint32_t rot;          // CTA that takes the step's first item
    uint32_t pad_[2];      // sizeof a multiple of 16: a warp copies a step into shared memory as 16-byte words
};
static_assert(sizeof(ChainStep) % 16 == 0 && sizeof(ChainStep) <= 512, "ChainStep: whole 16-byte words, at most 32 of them");

struct ChainGeom {
    uint32_t n_stages, stage_bytes, stage_off, x_off, smem_bytes;
};
// Fills the geometry of steps[0..n) and the launch-wide ring; false when a step cannot run this way
// (activation operands too large for shared memory, an exchange-vector input with an unsupported form).
bool chain_plan(ChainStep *steps, uint32_t n, int num_sms, size_t smem_optin, ChainGeom *geom);
cudaError_t chain_prepare_device(size_t smem_optin);
// d_steps: the planned list in device memory. d_ctl: two words {epoch base, exit ticket}, zero-initialised once
// and then owned by the launches (each adds n_steps to the base when its last CTA leaves). d_trace: null, or
// CHAIN_TRACE_WORDS * n_steps device words (measurement only) that receive, from CTA 0 and per step: the clock (ns)
// at its start, when its activations have arrived, after its prologue, after its last row group, after its
// reduction and stores; and the SM clocks its first thread spent waiting for weight stages. poll_limit: bound
// of every wait on an exchange vector, in polls. debug (measurement only): bit 0 = no arithmetic, bit 1 = the
// waits on exchange vectors do not wait.
constexpr int CHAIN_TRACE_WORDS = 6;
cudaError_t launch_chain(const ChainStep *d_steps, uint32_t n_steps, const ChainGeom &geom, uint32_t *d_ctl,
                         uint32_t *d_status, uint32_t poll_limit, uint32_t debug, unsigned long long *d_trace,
                         int num_sms, cudaStream_t stream);

// ---- W8A8 prefill GEMM (tcgen05 int8 MMA) ----------------------------------
cudaError_t gemm_prepare_device();
cudaError_t noalloc_prepare_device(int device);  // gemm_noalloc.cu: materialises the fixed scratch array on the current device
uint32_t gemm_scales_ld(uint32_t rows);  // leading dimension (floats) of the transposed f32 scale plane
cudaError_t launch_scales_transpose(const uint8_t *d_res, float *d_out, const RowLayout &L, uint32_t rows,
                                    cudaStream_t stream);  // d_res: the resident (tile-major) weight
// Q4_0: the weight's codes as bytes (nibble - 8) + 128, row-major [rows][in_dim], for the GEMM's TMA boxes
cudaError_t launch_expand_q4_codes(const uint8_t *d_res, uint8_t *d_out, const RowLayout &L, uint32_t rows,
                                   cudaStream_t stream);
uint32_t gemm_x_ld(uint32_t m);  // leading dimension (tokens) of the K-block-major per-token arrays
// x[m][nb*32] -> q int8 [m][nb*32]; block scales d, code sums xs and un-bias terms xc, each [nb][gemm_x_ld(m)]
cudaError_t launch_xquant8_sum(const float *d_x, int8_t *d_q, float *d_d, int32_t *d_xs, float *d_xc, uint32_t m,
                               uint32_t nb, cudaStream_t stream);
cudaError_t launch_block_isums(const uint8_t *d_res, const int8_t *d_xq, int32_t *d_out, const RowLayout &L, uint32_t M,
                               uint32_t rows, cudaStream_t stream);
uint32_t gemm_pick_splits(uint32_t M, uint32_t rows, uint32_t nb, int num_sms);
size_t gemm_workspace_floats(uint32_t M, uint32_t rows, uint32_t splits);
// mode 0: d_y[M][rows]; mode 1: the kernel's int32 block sums into d_dump[M][rows][nb]; modes 2, 3: measurement
// (no accumulator drain / no drain and no loads), nothing written.
cudaError_t launch_gemm_w8a8(const uint8_t *d_res, const RowLayout &L, uint32_t rows, const float *d_scalesT,
                             const int8_t *d_xq, const float *d_xd, const int32_t *d_xs, const float *d_xc, uint32_t M,
                             float *d_y, float *d_part, uint32_t splits, int mode, int32_t *d_dump, uint32_t *d_status,
                             cudaStream_t stream);

// Cross-GPU barrier on flag words in peer-mapped memory (one launch per rank, one rank per GPU):
// bumps *d_epoch, stores the new value into flag word `rank` of every rank's flag array and waits
// (bounded) until all `world` words of this rank's own array have reached it.
// (bounded: poll_limit polls)
cudaError_t launch_peer_barrier(uint32_t *d_epoch, uint32_t *d_local_flags, uint32_t *const *peer_flags, int rank,
                                int world, uint32_t *d_status, uint32_t poll_limit, cudaStream_t stream);

// The activation quantiser on its own: q[n] int8, d[n/32] f32 from x[n].
cudaError_t launch_xquant8(const float *d_x, int8_t *d_q, float *d_d, uint32_t n, cudaStream_t stream);

// One layer's attention for `rows` tokens at once (attention.cu): per-head norm and rope of q (in place) and k, k / v
// appended to the cache at the tokens' positions, then softmax(q k^T * scale) v over the cached rows into attn.
// q / k / v / attn are [rows][dim]; pos[rows] ascending (so that attention is causal among the rows).
// part: rows * n_heads * ceil(max_seq / ATT_SPLIT_TOKENS) * (hd + 2) floats.
constexpr uint32_t ATT_SPLIT_TOKENS = 64;
constexpr uint32_t ATT_MAX_HD = 512;
enum { ATT_ROPE_NONE = 0, ATT_ROPE_CHAIN = 1, ATT_ROPE_POW = 2 };
struct AttnArgs {
    float *q;
    const float *k, *v;            // v = the raw k vector on a layer that shares K and V
    const float *q_norm, *k_norm;  // [hd] each, null = no QK-norm
    const float *freq;             // [hd / 2] frequency factors of ATT_ROPE_POW, or null
    void *kc, *vc;                 // [max_seq][n_kv * hd] of float, or of f16 when kv_f16
    float *part, *attn;
    const uint32_t *pos;
    uint32_t n_heads, n_kv, hd, max_seq, rows;
    uint32_t window;        // 0 = attend to every cached row; else to the last `window` rows
    uint32_t kv_f16, norm_v, rope, rope_adjacent;
    float eps, theta_scale /* ATT_ROPE_CHAIN */, theta /* ATT_ROPE_POW */, scale;
    uint32_t *status;
};
cudaError_t launch_attention_step(const AttnArgs &A, cudaStream_t stream);
// h[r] = (h[r] + rmsnorm(x[r]) * w) * out_scale for `rows` vectors of `dim`
cudaError_t launch_addnorm(float *d_h, const float *d_x, const float *d_w, uint32_t dim, float eps, float out_scale,
                           uint32_t rows, cudaStream_t stream);
// x = cap * tanh(x / cap)
cudaError_t launch_softcap(float *d_x, size_t n, float cap, cudaStream_t stream);
void f32_to_f16_ref(const float *src, unsigned short *dst, size_t n);

}  // namespace strix
