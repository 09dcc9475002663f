// Internal definition of the accelerator handle (shared by the .cu files that
// implement groups of C-ABI entry points).
#pragma once
#include <map>
#include <cuda_runtime.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "kernels.h"
#include "strix_cuda.h"

namespace strix {

// One adopted weight: this accelerator's shard of rows in the tile-major layout.
struct Resident {
    int fmt;
    RowLayout L;
    size_t out_total;  // rows of the whole weight
    size_t row0;       // first global row held here
    size_t rows;       // rows held here
    uint8_t *dev;
    size_t bytes;
    uint8_t *gemm_codes;  // Q8_0 only: the codes once more, row-major [rows][in_dim] as q + 128 (the prefill GEMM's
                          // TMA boxes want K-major rows; the GEMV's tile-major order does not give them)
    float *scalesT;  // Q8_0 only, built on the first GEMM: f32 scales transposed to [nb][ld] (see gemm_w8a8.cu)
};

struct DevBuf {
    float *p = nullptr;
    size_t cap = 0;  // floats
};
struct PinBuf {
    void *p = nullptr;
    size_t cap = 0;  // bytes
};

}  // namespace strix

struct strix_decode_state;  // decode.cu

struct strix_cuda {
    int device = 0;
    int rank = 0, world = 1, profile = 0;
    strix::GemvTune tune;             // planning knobs (strix_cuda_set_option)
    int use_batch_graph = 1;          // gemv_batch replays a cached CUDA graph
    uint32_t chain_debug = 0;         // measurement: see launch_chain
    int chain_trace = 0;              // measurement: the chain kernel records per-step clocks (strix_cuda_decode_trace)
    int kv_f16 = 0;                   // real attention keeps its KV cache in f16 (the reference's STRIX_F16_KV, decode.rs:513-516)
    int decode_chain = -1;            // the decode projection chain as one persistent launch: 1 on, 0 off, -1 = on for a
                                      // row-sharded handle (the only way it can run), off otherwise (a launch per step
                                      // measured 1.33 against 1.39 ms per token on one GPU)
    uint32_t poll_limit = strix::CHAIN_POLL_LIMIT;  // bound of a wait on an exchange vector, in polls
    int num_sms = 0;
    size_t smem_optin = 0;
    std::string name, err;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;        // gemv_batch: outputs leave here while later kernels run
    std::vector<cudaEvent_t> batch_events;     // gemv_batch: (kernel done, copy done) per call slot
    // gemv_batch replays the last batch shape from a CUDA graph (one launch instead of ~5 runtime calls
    // per item): the graph, what it was captured for, and the pinned words its copies raise as each
    // output lands (the host copies that output out while later kernels still run)
    struct BatchGraph {
        cudaGraphExec_t exec = nullptr;
        int act = 0;
        std::vector<const uint8_t *> w_dev;   // resident buffers of the items, in order (null = skipped item)
        std::vector<size_t> rows, in_dim;
        std::vector<int> fmt;
        int side_by_side = 0;                 // the options the graph was captured under
        size_t small_bytes = 0;
        const void *x = nullptr, *y = nullptr, *pin_in = nullptr, *pin_out = nullptr;
    } batch_graph;
    // gemv_batch / gemv_batch_dev: the small items of a batch (independent GEMVs that would each pay a launch's fill
    // and drain, ~9 us against 3-4 us of HBM time) run side by side in one launch (gemv_multi_kernel)
    int batch_side_by_side = 1;       // 0 = a launch per item, 1 = items up to batch_small_bytes share launches, 2 = all items do
    int batch_overlap = 1;            // later launches of a batch do not wait for the earlier ones (GemvArgs::order)
    size_t batch_small_bytes = (size_t)256 << 20;  // (measured on 1/2 and 1/4 row shards of the benchmark step: 87 against 95 us, 50 against 61 us with 64 MiB)
    volatile uint32_t *batch_flags = nullptr;  // pinned, BATCH_GRAPH_MAX words
    uint32_t *d_one = nullptr;                 // device word holding 1
    uint32_t *d_status = nullptr;
    uint32_t status_host = 0;
    std::unordered_map<std::string, strix::Resident> weights;
    std::unordered_map<std::string, strix::DevBuf> f32s;
    // staging for the host-pointer entry points (grown on demand, never shrunk; like the
    // reference's persistent gemv_x / gemv_y, decode.rs:3827-3832)
    uint8_t *xop = nullptr;  // operand image of a batched integer-dot GEMV (launch_xop_prepare), grown on demand
    size_t xop_cap = 0;
    strix::DevBuf x, y;
    strix::PinBuf pin_in, pin_out;
    // scratch of the prefill GEMM (grown on demand): f32 activations, their int8 codes, block scales,
    // block code sums, f32 output, split-K partials
    strix::DevBuf gm_x, gm_y, gm_part, gm_xd, gm_xc;
    // Per-kernel timing (opts.profile / option "profile"; the reference's STRIX_PROF, decode.rs:25-69): every launch
    // site brackets its kernel with two CUDA events; strix_cuda_profile_dump folds them into per-kernel totals.
    struct ProfPending {
        const char *name;
        cudaEvent_t a, b;
    };
    std::vector<ProfPending> prof_pending;
    std::map<std::string, std::pair<double, uint32_t>> prof_total;  // name -> (milliseconds, launches)
    strix_decode_state *decode = nullptr;  // configured projection chain (decode.cu), or null
    // mixture-of-experts layers adopted by upload_moe_q8 / upload_moe_q6 (moe.cu): the experts of a projection are one
    // resident stack "moe.<layer>.gate|up|down" of n_expert * rows-per-expert rows
    struct MoeLayer {
        int fmt = 0;
        uint32_t hidden = 0, eff = 0, n_expert = 0;
    };
    std::unordered_map<size_t, MoeLayer> moe;
    strix::DevBuf moe_g, moe_u, moe_dy, moe_out, moe_w, moe_sh;  // scratch: gate / up rows, down rows, result, weights, shared expert
    int *moe_ids = nullptr;
    // argmax scratch (argmax.cu), allocated on first use: per-block winners, per-row tickets, results
    void *am_part = nullptr;
    uint32_t *am_ticket = nullptr, *am_idx = nullptr;
    float *am_val = nullptr;
    uint32_t *am_pin = nullptr;  // pinned: ids (16) then the status word
    int8_t *gm_xq = nullptr;
    size_t gm_xq_cap = 0;
    int32_t *gm_xs = nullptr;
    size_t gm_xs_cap = 0;
};

namespace strix {
// Brackets the launches made while it lives with two events on `s`, when profiling is on and `s` is not being
// captured (events inside a capture cannot be timed). `name` must be a string literal.
struct ProfScope {
    strix_cuda *h;
    cudaStream_t s;
    const char *name;
    cudaEvent_t a = nullptr, b = nullptr;
    ProfScope(strix_cuda *h_, cudaStream_t s_, const char *name_);
    ~ProfScope();
};
void prof_fold(strix_cuda *h);  // waits for the pending event pairs and adds them to the totals
const char *gemv_prof_name(const GemvArgs &a);
size_t shard_begin(size_t rows, int world, int r);
int ensure_f32(strix_cuda *h, DevBuf &b, size_t n);
int ensure_pinned(strix_cuda *h, PinBuf &b, size_t bytes);
int ensure_xop(strix_cuda *h, size_t bytes);
const Resident *find_weight(strix_cuda *h, const char *key);
// Repack + upload of raw GGUF blocks [out_dim][in_dim] under `key` (1 adopted, 0 declined, <0 error). gemm_copy: Q8_0
// weights also keep the row-major code copy the prefill GEMM reads.
int upload_quant(strix_cuda *h, int fmt, const char *key, const uint8_t *bytes, size_t len, size_t in_dim, size_t out_dim,
                 bool gemm_copy);
// argmax per row of d_x[rows][stride] (n entries each, rows <= 16) into h->am_idx (and h->am_val) on `stream`
int argmax_rows_enqueue(strix_cuda *h, const float *d_x, size_t n, size_t stride, size_t rows, cudaStream_t stream);
Resident *find_weight_mut(strix_cuda *h, const char *key);
// One GEMV launch over up to 3 resident weights that share the activation; d_res (may be null)
// gives per-weight residual vectors added to the outputs.
int gemv_launch_rows(strix_cuda *h, int nmat, const Resident *const *ws, const float *d_a, const float *d_b, float eps,
                     int pre, int act, float *const *d_ys, const float *const *d_res, uint32_t b, uint32_t a_stride,
                     uint32_t b_stride, cudaStream_t stream);
int gemv_fill_args(strix_cuda *h, int nmat, const Resident *const *ws, const float *d_a, const float *d_b, float eps,
                   int pre, int act, float *const *d_ys, const float *const *d_res, GemvArgs *out);
void batch_release(strix_cuda *h);   // drops the cached gemv_batch graph (it holds weight pointers)
void decode_trace_enable(strix_cuda *h);  // see decode.cu
void decode_release(strix_cuda *h);  // drops a configured decode chain (its graph holds weight pointers)
int gemv_launch(strix_cuda *h, int nmat, const Resident *const *ws, const float *d_a, const float *d_b, float eps,
                int pre, int act, float *const *d_ys, const float *const *d_res, cudaStream_t stream);
}  // namespace strix
