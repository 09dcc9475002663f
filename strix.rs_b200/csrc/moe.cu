// Mixture-of-experts FFN over resident expert stacks: WeightAccel::upload_moe_q8 / upload_moe_q6 / moe_ffn /
// moe_expert_ffn / moe_layer_ffn (crates/strix-core/src/accel.rs:167-246) and the router's top-k.
//
// Replaces the reference's MoE kernels (crates/strix-backend-rocm/src/kernels.rs:670-797 q8_moe_gemv_gu /
// q8_moe_down, :1561-1600 q6_moe_gemv, :1738-1752 moe_silu_mul / shexp_add, :1846-1882 topk_router / moe_wsum;
// call sites decode.rs:1820-1923 queue_shexp / moe6_launches, :1923-2130 moe_launches, :2717-2870 uploads and
// moe_ffn, :3299-3356 moe_expert_ffn, :3552-3630 moe_layer_ffn) and agrees with the CPU forward they must match
// (crates/strix-backend-cpu/src/mellum.rs:1582-1663).
//
// Layout: the ne experts of a projection are ONE resident stack of ne * rows-per-expert rows in the GEMV's
// tile-major order ("moe.<layer>.gate", ".up": rows = eff per expert, in_dim = hidden; ".down": rows = hidden per
// expert, in_dim = eff); an expert is a run of whole row groups, so the GEMV kernel reaches it by an index, not a copy.
//
// One token (moe_ffn), three GEMV-kernel launches instead of the reference's 2 k + 3:
//   gate|up   one launch over 2 k virtual matrices: the kernel's expert indirection (GemvArgs::sel_ids) makes the
//             launch's row-group list the stack of experts ids[0..k) of both projections; x is shared
//   down      one launch per chunk of up to 8 selections: the k activation vectors silu(g_s) * u_s ride as the
//             activation rows of a batched GEMV over the stack of the selected down experts. The MMA gives every
//             (activation row, expert) pair; only the pairs (s, s) are wanted, and the extra columns are free (the
//             MMA is 8 columns wide whatever the row count). The fold reads that diagonal
//   fold      out[o] = sum_s w[s] * dy[s][o], s ascending, multiply then add as the CPU forward does
//             (mellum.rs:1655-1657), plus sgate * the shared expert's output where the layer has one
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "accel.h"

using namespace strix;

#define CU_TRY(h, expr)                                                    \
    do {                                                                   \
        cudaError_t _e = (expr);                                           \
        if (_e != cudaSuccess) {                                           \
            (h)->err = std::string(#expr) + ": " + cudaGetErrorString(_e); \
            return -1;                                                     \
        }                                                                  \
    } while (0)

namespace {

constexpr uint32_t MOE_MAX_K = 16;       // routed experts per token (the reference's limit, decode.rs:2842)
constexpr uint32_t MOE_MAX_EXPERTS = 128;  // router width (kernels.rs:1846-1851: four logits per lane)

// out[o] (+)= sum_{s < n} w[s] * dyy[s][s * hidden + o]: the diagonal of the batched down launch, folded with the
// routing weights in selection order. dyy: [n][n * hidden]. accumulate = 0 starts from zero.
__global__ void moe_fold_kernel(const float *__restrict__ dyy, const float *__restrict__ w, uint32_t n, uint32_t hidden,
                                float *__restrict__ out, int accumulate) {
    const uint32_t o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= hidden) return;
    float s = accumulate ? out[o] : 0.f;
    for (uint32_t e = 0; e < n; e++) s = __fadd_rn(s, __fmul_rn(w[e], dyy[(size_t)e * n * hidden + (size_t)e * hidden + o]));
    out[o] = s;
}

// out[i] += sd[i] * sgate (kernels.rs:1747-1752 shexp_add)
__global__ void moe_shared_add_kernel(float *__restrict__ out, const float *__restrict__ sd, float sgate, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(out[i], __fmul_rn(sd[i], sgate));
}

// Router top-k (mellum.rs:1590-1609; kernels.rs:1846-1873): p = exp(l - max) / sum over all experts, the k largest
// (a tie goes to the lower index), weights p / (sum of the chosen p). One warp; the two sums run in index /
// selection order on one lane, as the CPU forward's do.
__global__ void __launch_bounds__(32) topk_router_kernel(const float *__restrict__ logits, uint32_t ne, uint32_t k,
                                                         int *__restrict__ ids, float *__restrict__ w) {
    __shared__ float p[MOE_MAX_EXPERTS];
    const uint32_t l = threadIdx.x;
    float mx = -3.0e38f;
    for (uint32_t e = l; e < ne; e += 32) mx = fmaxf(mx, logits[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (uint32_t e = l; e < ne; e += 32) p[e] = expf(logits[e] - mx);
    __syncwarp();
    float sum = 0.f;
    if (l == 0)
        for (uint32_t e = 0; e < ne; e++) sum += p[e];
    sum = __shfl_sync(0xffffffffu, sum, 0);
    for (uint32_t e = l; e < ne; e += 32) p[e] = p[e] / sum;
    __syncwarp();
    float ws = 0.f;
    for (uint32_t i = 0; i < k; i++) {
        float b = -1.f;
        uint32_t bi = 0xffffffffu;
        for (uint32_t e = l; e < ne; e += 32)
            if (p[e] > b) {  // ascending scan: the lower index keeps a tie
                b = p[e];
                bi = e;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, b, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > b || (ob == b && oi < bi)) {
                b = ob;
                bi = oi;
            }
        }
        if (l == 0) {
            ids[i] = (int)bi;
            w[i] = b;
            p[bi] = -2.f;  // taken
        }
        ws += b;
        __syncwarp();
    }
    if (l == 0)
        for (uint32_t i = 0; i < k; i++) w[i] = w[i] / ws;
}

std::string moe_key(size_t layer, const char *what) { return "moe." + std::to_string(layer) + "." + what; }

int moe_upload(strix_cuda *h, int fmt, size_t layer, const uint8_t *gate, size_t gate_len, const uint8_t *up, size_t up_len,
               const uint8_t *down, size_t down_len, size_t hidden, size_t eff, size_t ne) {
    if (!h || !gate || !up || !down) return -1;
    h->err.clear();
    const size_t be = gguf_block_elems(fmt), bb = gguf_block_bytes(fmt);
    // the reference's own limits (decode.rs:2727-2735, 2803-2811): whole blocks, eff and hidden <= 4096, exact lengths
    if (hidden == 0 || eff == 0 || ne == 0 || hidden % be != 0 || eff % be != 0 || eff > 4096 || hidden > 4096) return 0;
    if (ne > MOE_MAX_EXPERTS * 8 || (eff % TILE_ROWS) != 0 || (hidden % TILE_ROWS) != 0) return 0;
    const size_t gate_eb = (hidden / be) * bb * eff, down_eb = (eff / be) * bb * hidden;
    if (gate_len != gate_eb * ne || up_len != gate_eb * ne || down_len != down_eb * ne) return 0;
    if (h->world > 1) return 0;  // expert stacks are not row-sharded: the model keeps its per-expert path
    int rc = upload_quant(h, fmt, moe_key(layer, "gate").c_str(), gate, gate_len, hidden, eff * ne, false);
    if (rc == 1) rc = upload_quant(h, fmt, moe_key(layer, "up").c_str(), up, up_len, hidden, eff * ne, false);
    if (rc == 1) rc = upload_quant(h, fmt, moe_key(layer, "down").c_str(), down, down_len, eff, hidden * ne, false);
    if (rc != 1) return rc;
    strix_cuda::MoeLayer L;
    L.fmt = fmt;
    L.hidden = (uint32_t)hidden;
    L.eff = (uint32_t)eff;
    L.n_expert = (uint32_t)ne;
    h->moe[layer] = L;
    return 1;
}

struct MoeW {
    const strix_cuda::MoeLayer *L;
    const Resident *gate, *up, *down;
};
bool moe_find(strix_cuda *h, size_t layer, MoeW *out) {
    auto it = h->moe.find(layer);
    if (it == h->moe.end()) return false;
    out->L = &it->second;
    out->gate = find_weight(h, moe_key(layer, "gate").c_str());
    out->up = find_weight(h, moe_key(layer, "up").c_str());
    out->down = find_weight(h, moe_key(layer, "down").c_str());
    return out->gate && out->up && out->down;
}

int moe_scratch(strix_cuda *h, const strix_cuda::MoeLayer &L, size_t rows) {
    // g / u: one row of eff per (token, selection); dy: the batched down launch's [n][n * hidden] for n <= 8,
    // or rows of hidden for the grouped-token paths
    const size_t r = std::max<size_t>(rows, MOE_MAX_K);
    if (ensure_f32(h, h->moe_g, r * L.eff) < 0 || ensure_f32(h, h->moe_u, r * L.eff) < 0) return -1;
    if (ensure_f32(h, h->moe_dy, std::max<size_t>(64 * (size_t)L.hidden, rows * L.hidden)) < 0) return -1;
    if (ensure_f32(h, h->moe_out, std::max<size_t>(rows, 1) * L.hidden) < 0) return -1;
    if (ensure_f32(h, h->moe_w, MOE_MAX_K) < 0) return -1;
    if (!h->moe_ids) CU_TRY(h, cudaMalloc(&h->moe_ids, MOE_MAX_K * sizeof(int)));
    return 0;
}

// One planned launch of the GEMV kernel over (a chunk of) an expert stack.
int moe_launch(strix_cuda *h, GemvArgs &c, uint32_t rows_nbatch, int pre, const float *a, const float *b, uint32_t a_stride,
               uint32_t b_stride, cudaStream_t s) {
    c.nbatch = rows_nbatch;
    c.a = a;
    c.b = b;
    c.a_stride = a_stride;
    c.b_stride = b_stride;
    c.pre = pre;
    if (!gemv_plan(c, h->num_sms, h->smem_optin, h->tune)) {
        h->err = "moe: in_dim too large for the shared-memory pipeline";
        return -1;
    }
    if (c.act == STRIX_ACT_Q8DOT && rows_nbatch >= 2 && h->tune.xop != 0) {
        // several activation rows in the integer-dot form: operands prepared once (see gemv_launch_rows)
        if (ensure_xop(h, xop_image_bytes(c.L.fmt, c.L.in_dim, rows_nbatch)) < 0) return -1;
        CU_TRY(h, launch_xop_prepare(c.L.fmt, c.L.in_dim, rows_nbatch, a, b, a_stride, b_stride, 0.f, pre, h->xop,
                                     h->tune.pdl != 0, s));
        c.xop = h->xop;
        c.pre = STRIX_PRE_NONE;
        if (!gemv_plan(c, h->num_sms, h->smem_optin, h->tune)) {
            h->err = "moe: in_dim too large for the shared-memory pipeline";
            return -1;
        }
    }
    ProfScope prof(h, s, "gemv.moe");
    CU_TRY(h, launch_gemv(c, s));
    return 0;
}

// The routed experts of one token: d_x[hidden] -> d_out[hidden], ids / weights already on the device.
int moe_token_enqueue(strix_cuda *h, size_t layer, const MoeW &W, const int *d_ids, const float *d_w, uint32_t k,
                      const float *d_x, float sgate, float *d_out, int act, cudaStream_t s) {
    const strix_cuda::MoeLayer &L = *W.L;
    const uint32_t eff = L.eff, hidden = L.hidden;
    {   // gate|up over the k selected experts, x shared
        const Resident *ws[2] = {W.gate, W.up};
        float *ys[2] = {h->moe_g.p, h->moe_u.p};
        GemvArgs a{};
        if (gemv_fill_args(h, 2, ws, d_x, nullptr, 0.f, STRIX_PRE_NONE, act, ys, nullptr, &a) < 0) return -1;
        for (int m = 0; m < 2; m++) {
            a.mat[m].rows = k * eff;
            a.mat[m].ystride = k * eff;
        }
        a.sel_ids = d_ids;
        a.sel_groups = eff / TILE_ROWS;
        a.sel_experts = L.n_expert;
        if (moe_launch(h, a, 1, STRIX_PRE_NONE, d_x, nullptr, 0, 0, s) < 0) return -1;
    }
    // down: the selections' activations as the rows of a batched launch over the stack of their experts; as many
    // selections per launch as the shared-memory plan takes (8 at most; Q6_K stacks 4)
    const uint32_t max_rows = W.down->fmt == FMT_Q6_K ? 4u : 8u;
    for (uint32_t c0 = 0; c0 < k;) {
        const Resident *ws[1] = {W.down};
        float *ys[1] = {h->moe_dy.p};
        GemvArgs a{};
        if (gemv_fill_args(h, 1, ws, nullptr, nullptr, 0.f, STRIX_PRE_SWIGLU, act, ys, nullptr, &a) < 0) return -1;
        a.sel_ids = d_ids + c0;
        a.sel_groups = hidden / TILE_ROWS;
        a.sel_experts = L.n_expert;
        uint32_t n = std::min(max_rows, k - c0);
        for (;; n = (n + 1) / 2) {
            GemvArgs t = a;
            t.mat[0].rows = n * hidden;
            t.nbatch = n;
            if (gemv_plan(t, h->num_sms, h->smem_optin, h->tune)) break;
            if (n == 1) {
                h->err = "moe: expert width too large for the shared-memory pipeline";
                return -1;
            }
        }
        a.mat[0].rows = n * hidden;
        a.mat[0].ystride = n * hidden;
        if (moe_launch(h, a, n, STRIX_PRE_SWIGLU, h->moe_g.p + (size_t)c0 * eff, h->moe_u.p + (size_t)c0 * eff, eff, eff, s) < 0)
            return -1;
        moe_fold_kernel<<<(hidden + 255) / 256, 256, 0, s>>>(h->moe_dy.p, d_w + c0, n, hidden, d_out, c0 != 0);
        CU_TRY(h, cudaGetLastError());
        c0 += n;
    }
    if (sgate != 0.f) {
        // shared expert (decode.rs:1820-1856): dense residents blk.<layer>.ffn_{gate,up,down}_shexp.weight
        const std::string b = "blk." + std::to_string(layer) + ".";
        const Resident *g = find_weight(h, (b + "ffn_gate_shexp.weight").c_str());
        const Resident *u = find_weight(h, (b + "ffn_up_shexp.weight").c_str());
        const Resident *d = find_weight(h, (b + "ffn_down_shexp.weight").c_str());
        if (!g || !u || !d || g->L.in_dim != hidden || u->L.in_dim != hidden || g->rows != u->rows || d->L.in_dim != g->rows ||
            d->rows != hidden || g->fmt != u->fmt)
            return 0;
        const size_t sff = g->rows;
        if (ensure_f32(h, h->moe_sh, 2 * sff + hidden) < 0) return -1;
        float *sg = h->moe_sh.p, *su = sg + sff, *sd = su + sff;
        const Resident *w2[2] = {g, u};
        float *y2[2] = {sg, su};
        if (gemv_launch(h, 2, w2, d_x, nullptr, 0.f, STRIX_PRE_NONE, act, y2, nullptr, s) < 0) return -1;
        const Resident *w1[1] = {d};
        float *y1[1] = {sd};
        if (gemv_launch(h, 1, w1, sg, su, 0.f, STRIX_PRE_SWIGLU, act, y1, nullptr, s) < 0) return -1;
        moe_shared_add_kernel<<<(hidden + 255) / 256, 256, 0, s>>>(d_out, sd, sgate, hidden);
        CU_TRY(h, cudaGetLastError());
    }
    return 1;
}

// m tokens through ONE expert: d_xs[m][hidden] -> d_y[m][hidden] (gate|up rows, SwiGLU, down rows).
int moe_expert_enqueue(strix_cuda *h, const MoeW &W, uint32_t e, const float *d_xs, uint32_t m, float *d_g, float *d_u,
                       float *d_y, int act, cudaStream_t s) {
    const strix_cuda::MoeLayer &L = *W.L;
    // views of the expert's rows inside the stacks: whole row groups, so a pointer offset is all it takes
    Resident gv = *W.gate, uv = *W.up, dv = *W.down;
    const size_t g_bytes = (size_t)(L.eff / TILE_ROWS) * gv.L.group_bytes, d_bytes = (size_t)(L.hidden / TILE_ROWS) * dv.L.group_bytes;
    gv.dev += (size_t)e * g_bytes;
    uv.dev += (size_t)e * g_bytes;
    dv.dev += (size_t)e * d_bytes;
    gv.rows = gv.out_total = uv.rows = uv.out_total = L.eff;
    dv.rows = dv.out_total = L.hidden;
    const Resident *w2[2] = {&gv, &uv};
    float *y2[2] = {d_g, d_u};
    if (gemv_launch_rows(h, 2, w2, d_xs, nullptr, 0.f, STRIX_PRE_NONE, act, y2, nullptr, m, L.hidden, 0, s) < 0) return -1;
    const Resident *w1[1] = {&dv};
    float *y1[1] = {d_y};
    if (gemv_launch_rows(h, 1, w1, d_g, d_u, 0.f, STRIX_PRE_SWIGLU, act, y1, nullptr, m, L.eff, L.eff, s) < 0) return -1;
    return 1;
}

int finish(strix_cuda *h, const char *who) {
    CU_TRY(h, cudaMemcpyAsync(&h->status_host, h->d_status, 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaStreamSynchronize(h->stream));
    if (h->status_host != 0) {
        h->err = std::string(who) + ": device status " + std::to_string(h->status_host);
        cudaMemsetAsync(h->d_status, 0, 4, h->stream);
        return -2;
    }
    return 1;
}

}  // namespace

extern "C" {

int strix_cuda_upload_moe_q8(strix_cuda *h, size_t layer, const uint8_t *gate, size_t gate_len, const uint8_t *up, size_t up_len,
                             const uint8_t *down, size_t down_len, size_t hidden, size_t eff, size_t ne) {
    return moe_upload(h, FMT_Q8_0, layer, gate, gate_len, up, up_len, down, down_len, hidden, eff, ne);
}
int strix_cuda_upload_moe_q6(strix_cuda *h, size_t layer, const uint8_t *gate, size_t gate_len, const uint8_t *up, size_t up_len,
                             const uint8_t *down, size_t down_len, size_t hidden, size_t eff, size_t ne) {
    return moe_upload(h, FMT_Q6_K, layer, gate, gate_len, up, up_len, down, down_len, hidden, eff, ne);
}

int strix_cuda_moe_ffn(strix_cuda *h, size_t layer, const int *ids, const float *wexp, size_t k, const float *x, size_t x_len,
                       float sgate, int act, float *y, size_t y_cap) {
    if (!h || !ids || !wexp || !x || !y) return -1;
    h->err.clear();
    MoeW W{};
    if (!moe_find(h, layer, &W)) return 0;
    const strix_cuda::MoeLayer &L = *W.L;
    // None in the reference: a length mismatch, more than 16 experts (decode.rs:2840-2844, 2859-2862)
    if (x_len != L.hidden || k == 0 || k > MOE_MAX_K || y_cap < L.hidden) return 0;
    for (size_t i = 0; i < k; i++)
        if (ids[i] < 0 || (uint32_t)ids[i] >= L.n_expert) return 0;
    if (act != STRIX_ACT_F32 && act != STRIX_ACT_Q8DOT) return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    if (moe_scratch(h, L, 1) < 0) return -1;
    if (ensure_f32(h, h->x, L.hidden) < 0) return -1;
    if (ensure_pinned(h, h->pin_in, (L.hidden + 2 * MOE_MAX_K) * 4) < 0 || ensure_pinned(h, h->pin_out, L.hidden * 4) < 0) return -1;
    float *pin = static_cast<float *>(h->pin_in.p);
    memcpy(pin, x, L.hidden * 4);
    memcpy(pin + L.hidden, wexp, k * 4);
    memcpy(pin + L.hidden + MOE_MAX_K, ids, k * 4);
    cudaStream_t s = h->stream;
    CU_TRY(h, cudaMemcpyAsync(h->x.p, pin, L.hidden * 4, cudaMemcpyHostToDevice, s));
    CU_TRY(h, cudaMemcpyAsync(h->moe_w.p, pin + L.hidden, k * 4, cudaMemcpyHostToDevice, s));
    CU_TRY(h, cudaMemcpyAsync(h->moe_ids, pin + L.hidden + MOE_MAX_K, k * 4, cudaMemcpyHostToDevice, s));
    const int rc = moe_token_enqueue(h, layer, W, h->moe_ids, h->moe_w.p, (uint32_t)k, h->x.p, sgate, h->moe_out.p, act, s);
    if (rc != 1) {
        cudaStreamSynchronize(s);
        return rc;
    }
    CU_TRY(h, cudaMemcpyAsync(h->pin_out.p, h->moe_out.p, L.hidden * 4, cudaMemcpyDeviceToHost, s));
    const int fr = finish(h, "moe_ffn");
    if (fr < 0) return fr;
    memcpy(y, h->pin_out.p, L.hidden * 4);
    return 1;
}

int strix_cuda_moe_ffn_dev(strix_cuda *h, size_t layer, const int *d_ids, const float *d_wexp, size_t k, const float *d_x,
                           float sgate, int act, float *d_y, void *stream) {
    if (!h || !d_ids || !d_wexp || !d_x || !d_y) return -1;
    h->err.clear();
    MoeW W{};
    if (!moe_find(h, layer, &W)) return 0;
    if (k == 0 || k > MOE_MAX_K || (act != STRIX_ACT_F32 && act != STRIX_ACT_Q8DOT)) return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    if (moe_scratch(h, *W.L, 1) < 0) return -1;
    return moe_token_enqueue(h, layer, W, d_ids, d_wexp, (uint32_t)k, d_x, sgate, d_y, act, static_cast<cudaStream_t>(stream));
}

int strix_cuda_moe_expert_ffn(strix_cuda *h, size_t layer, size_t e, const float *xs, size_t m, int act, float *y, size_t y_cap) {
    const int plan[2] = {(int)e, (int)m};
    return strix_cuda_moe_layer_ffn(h, layer, plan, 1, xs, m, act, y, y_cap);
}

int strix_cuda_moe_layer_ffn(strix_cuda *h, size_t layer, const int *plan, size_t n_plan, const float *xs, size_t rows, int act,
                             float *y, size_t y_cap) {
    if (!h || !plan || !xs || !y) return -1;
    h->err.clear();
    MoeW W{};
    if (!moe_find(h, layer, &W)) return 0;
    const strix_cuda::MoeLayer &L = *W.L;
    size_t total = 0;
    for (size_t i = 0; i < n_plan; i++) {
        if (plan[2 * i] < 0 || (uint32_t)plan[2 * i] >= L.n_expert || plan[2 * i + 1] < 0) return 0;
        total += (size_t)plan[2 * i + 1];
    }
    if (rows == 0 || total != rows || y_cap < rows * L.hidden || (act != STRIX_ACT_F32 && act != STRIX_ACT_Q8DOT)) return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    if (moe_scratch(h, L, rows) < 0) return -1;
    if (ensure_f32(h, h->x, rows * L.hidden) < 0) return -1;
    if (ensure_pinned(h, h->pin_in, rows * L.hidden * 4) < 0 || ensure_pinned(h, h->pin_out, rows * L.hidden * 4) < 0) return -1;
    {   // the batched GEMV's operand image, sized before any launch
        const size_t need = std::max(xop_image_bytes(L.fmt, L.hidden, 8), xop_image_bytes(L.fmt, L.eff, 8));
        if (ensure_xop(h, need) < 0) return -1;
    }
    cudaStream_t s = h->stream;
    memcpy(h->pin_in.p, xs, rows * L.hidden * 4);
    CU_TRY(h, cudaMemcpyAsync(h->x.p, h->pin_in.p, rows * L.hidden * 4, cudaMemcpyHostToDevice, s));
    size_t off = 0;
    for (size_t i = 0; i < n_plan; i++) {
        const uint32_t m = (uint32_t)plan[2 * i + 1];
        if (m == 0) continue;
        const int rc = moe_expert_enqueue(h, W, (uint32_t)plan[2 * i], h->x.p + off * L.hidden, m, h->moe_g.p + off * L.eff,
                                          h->moe_u.p + off * L.eff, h->moe_out.p + off * L.hidden, act, s);
        if (rc != 1) {
            cudaStreamSynchronize(s);
            return rc;
        }
        off += m;
    }
    CU_TRY(h, cudaMemcpyAsync(h->pin_out.p, h->moe_out.p, rows * L.hidden * 4, cudaMemcpyDeviceToHost, s));
    const int fr = finish(h, "moe_layer_ffn");
    if (fr < 0) return fr;
    memcpy(y, h->pin_out.p, rows * L.hidden * 4);
    return 1;
}

int strix_cuda_topk_router_dev(strix_cuda *h, const float *d_logits, size_t ne, size_t k, int *d_ids, float *d_w, void *stream) {
    if (!h || !d_logits || !d_ids || !d_w) return -1;
    h->err.clear();
    if (ne == 0 || ne > MOE_MAX_EXPERTS || k == 0 || k > MOE_MAX_K || k > ne) return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    topk_router_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(d_logits, (uint32_t)ne, (uint32_t)k, d_ids, d_w);
    CU_TRY(h, cudaGetLastError());
    return 1;
}

int strix_cuda_topk_router(strix_cuda *h, const float *logits, size_t ne, size_t k, int *ids, float *w) {
    if (!h || !logits || !ids || !w) return -1;
    h->err.clear();
    if (ne == 0 || ne > MOE_MAX_EXPERTS || k == 0 || k > MOE_MAX_K || k > ne) return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    if (ensure_f32(h, h->x, ne) < 0 || ensure_f32(h, h->moe_w, MOE_MAX_K) < 0) return -1;
    if (!h->moe_ids) CU_TRY(h, cudaMalloc(&h->moe_ids, MOE_MAX_K * sizeof(int)));
    CU_TRY(h, cudaMemcpyAsync(h->x.p, logits, ne * 4, cudaMemcpyHostToDevice, h->stream));
    const int rc = strix_cuda_topk_router_dev(h, h->x.p, ne, k, h->moe_ids, h->moe_w.p, h->stream);
    if (rc != 1) return rc;
    CU_TRY(h, cudaMemcpyAsync(ids, h->moe_ids, k * 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaMemcpyAsync(w, h->moe_w.p, k * 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaStreamSynchronize(h->stream));
    return 1;
}

}  // extern "C"
