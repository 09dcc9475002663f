// Host side of the accelerator: the handle, resident-weight bookkeeping, and the
// extern "C" entry points declared in include/strix_cuda.h.
//
// Mirrors RocmWeightAccel (crates/strix-backend-rocm/src/decode.rs:445-557,
// 2491-2714, 3227-3297, 3827-3912) for the quantized-matmul path only. There is
// no CPU fallback: a call either runs on the GPU, declines (0) so that the caller
// keeps the weight on its own CPU path, or fails (<0).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "accel.h"

using namespace strix;

static thread_local std::string g_create_error;

#define CU_TRY(h, expr)                                                                                  \
    do {                                                                                                 \
        cudaError_t _e = (expr);                                                                         \
        if (_e != cudaSuccess) {                                                                         \
            (h)->err = std::string(#expr) + ": " + cudaGetErrorString(_e);                               \
            return -1;                                                                                   \
        }                                                                                                \
    } while (0)

namespace strix {

size_t shard_begin(size_t rows, int world, int r) {
    if (world <= 1) return r <= 0 ? 0 : rows;
    size_t q = rows / (size_t)world, rem = rows % (size_t)world;
    return (size_t)r * q + std::min((size_t)r, rem);
}

int ensure_f32(strix_cuda *h, DevBuf &b, size_t n) {
    if (b.cap >= n) return 1;
    if (b.p) cudaFree(b.p);
    b.p = nullptr;
    b.cap = 0;
    size_t want = std::max<size_t>(n, 4096);
    CU_TRY(h, cudaMalloc(&b.p, want * sizeof(float)));
    b.cap = want;
    return 1;
}

int ensure_pinned(strix_cuda *h, PinBuf &b, size_t bytes) {
    if (b.cap >= bytes) return 1;
    if (b.p) cudaFreeHost(b.p);
    b.p = nullptr;
    b.cap = 0;
    size_t want = std::max<size_t>(bytes, 1 << 16);
    CU_TRY(h, cudaMallocHost(&b.p, want));
    b.cap = want;
    return 1;
}

// The operand image of a batched integer-dot GEMV (grown on demand; a caller that captures launches into a
// graph sizes it beforehand, since nothing may be allocated during a capture).
int ensure_xop(strix_cuda *h, size_t bytes) {
    if (h->xop_cap >= bytes) return 1;
    if (h->xop) cudaFree(h->xop);
    h->xop = nullptr;
    h->xop_cap = 0;
    CU_TRY(h, cudaMalloc(&h->xop, bytes));
    h->xop_cap = bytes;
    return 1;
}

const Resident *find_weight(strix_cuda *h, const char *key) {
    auto it = h->weights.find(key);
    return it == h->weights.end() ? nullptr : &it->second;
}
Resident *find_weight_mut(strix_cuda *h, const char *key) {
    auto it = h->weights.find(key);
    return it == h->weights.end() ? nullptr : &it->second;
}

}  // namespace strix

namespace strix {
int upload_quant(strix_cuda *h, int fmt, const char *key, const uint8_t *bytes, size_t len, size_t in_dim, size_t out_dim,
                 bool gemm_copy) {
    if (!h || !key || !bytes) return -1;
    h->err.clear();
    const size_t be = gguf_block_elems(fmt), bb = gguf_block_bytes(fmt);
    // the reference declines, it does not fail, on these (decode.rs:2492-2499, 2630-2636, 2684-2691)
    if (in_dim == 0 || in_dim % be != 0) return 0;
    const size_t nb = in_dim / be;
    if (len != nb * out_dim * bb) return 0;
    if (in_dim > 0x7fffffffu || out_dim > 0x7fffffffu) return 0;
    CU_TRY(h, cudaSetDevice(h->device));

    Resident r{};
    r.fmt = fmt;
    r.L = make_layout(fmt, (uint32_t)in_dim);
    r.out_total = out_dim;
    r.row0 = shard_begin(out_dim, h->world, h->rank);
    r.rows = shard_begin(out_dim, h->world, h->rank + 1) - r.row0;
    {
        // the shared-memory pipeline must be able to hold two stages of one row
        GemvArgs probe{};
        probe.L = r.L;
        probe.nmat = 1;
        probe.mat[0].rows = (uint32_t)std::max<size_t>(r.rows, 1);
        if (!gemv_plan(probe, h->num_sms, h->smem_optin, h->tune)) return 0;
    }
    r.bytes = (size_t)resident_bytes(r.L, r.rows);
    CU_TRY(h, cudaMalloc(&r.dev, std::max<size_t>(r.bytes, 16)));
    if (fmt == FMT_Q8_0 && gemm_copy) {
        const cudaError_t eg = cudaMalloc(&r.gemm_codes, std::max<size_t>(r.rows * in_dim, 16));
        if (eg != cudaSuccess) {
            cudaFree(r.dev);
            h->err = std::string("upload (GEMM copy): ") + cudaGetErrorString(eg);
            return -1;
        }
    }

    // Raw GGUF bytes go up in chunks of whole row groups; a kernel regroups each chunk into tiles.
    const size_t raw_row = nb * bb;
    const size_t chunk_rows = std::max<size_t>(1, (size_t)(128u << 20) / raw_row / TILE_ROWS) * TILE_ROWS;
    uint8_t *d_raw = nullptr;
    cudaError_t e = cudaMalloc(&d_raw, std::min(chunk_rows, std::max<size_t>(r.rows, 1)) * raw_row);
    if (e != cudaSuccess) {
        cudaFree(r.dev);
        if (r.gemm_codes) cudaFree(r.gemm_codes);
        h->err = std::string("upload staging: ") + cudaGetErrorString(e);
        return -1;
    }
    for (size_t at = 0; at < r.rows && e == cudaSuccess; at += chunk_rows) {
        const size_t n = std::min(chunk_rows, r.rows - at);
        e = cudaMemcpyAsync(d_raw, bytes + (r.row0 + at) * raw_row, n * raw_row, cudaMemcpyHostToDevice, h->stream);
        if (e == cudaSuccess)
            e = launch_repack(fmt, d_raw, r.dev, r.gemm_codes, r.L, (uint32_t)at, (uint32_t)n, h->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);  // `bytes` is borrowed; d_raw is reused
    }
    cudaFree(d_raw);
    if (e != cudaSuccess) {
        cudaFree(r.dev);
        if (r.gemm_codes) cudaFree(r.gemm_codes);
        h->err = std::string("upload: ") + cudaGetErrorString(e);
        return -1;
    }
    decode_release(h);  // a configured chain may hold the pointer this upload replaces
    batch_release(h);   // so may the cached gemv_batch graph and programs (the allocator can hand the old address
                        // back to a weight of another format or shape)
    auto it = h->weights.find(key);
    if (it != h->weights.end()) {
        cudaFree(it->second.dev);
        if (it->second.gemm_codes) cudaFree(it->second.gemm_codes);
        if (it->second.scalesT) cudaFree(it->second.scalesT);
        it->second = r;
    } else {
        h->weights.emplace(key, r);
    }
    return 1;
}
}  // namespace strix

namespace strix {
ProfScope::ProfScope(strix_cuda *h_, cudaStream_t s_, const char *name_) : h(h_), s(s_), name(name_) {
    if (!h->profile) return;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return;
    }
    if (h->prof_pending.size() >= 8192) prof_fold(h);  // (bounded: fold what has run so far)
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) {
        cudaGetLastError();
        if (a) cudaEventDestroy(a);
        a = b = nullptr;
        return;
    }
    cudaEventRecord(a, s);
}
ProfScope::~ProfScope() {
    if (!a) return;
    cudaEventRecord(b, s);
    h->prof_pending.push_back({name, a, b});
}
void prof_fold(strix_cuda *h) {
    for (auto &p : h->prof_pending) {
        float ms = 0.f;
        if (cudaEventSynchronize(p.b) == cudaSuccess && cudaEventElapsedTime(&ms, p.a, p.b) == cudaSuccess) {
            auto &t = h->prof_total[p.name];
            t.first += ms;
            t.second += 1;
        } else {
            cudaGetLastError();
        }
        cudaEventDestroy(p.a);
        cudaEventDestroy(p.b);
    }
    h->prof_pending.clear();
}

void batch_release(strix_cuda *h) {
    if (h->batch_graph.exec) {
        cudaGraphExecDestroy(h->batch_graph.exec);
        h->batch_graph.exec = nullptr;
    }
}

// Items idx of a batch (independent GEMVs ws[i], d_xs[i] -> d_ys[i]) side by side: up to GEMV_MULTI_MAX problems
// per launch (gemv_multi_kernel), the CTAs dealt out among them by their bytes. What cannot be planned that way
// gets a launch of its own.
// peer_ys (may be null): the row-sharded multi-GPU form - item i's rows go straight into the FULL output vector of
// every accelerator of the group, peer_ys[i * n_peers + p] (peer-mapped device memory, this GPU's own copy among
// them), at row_base + row, instead of into d_ys[i].
static void batch_set_peers(GemvArgs &a, const Resident *w, float *const *peer_ys, size_t i, int n_peers) {
    if (!peer_ys) return;
    a.mat[0].y = nullptr;
    a.mat[0].n_peer = (uint32_t)n_peers;
    a.mat[0].row_base = (uint32_t)w->row0;
    for (int p = 0; p < n_peers; p++) a.mat[0].peer_y[p] = peer_ys[i * (size_t)n_peers + (size_t)p];
}
// The place of each launch among the launches of one batch (GemvArgs::order): the items are independent, so only the
// first launch waits for what the batch follows and the later ones overlap their predecessors' tails. Off when an
// item that runs as a launch of its own gets its operands from a preparation launch (that launch writes what the
// next one reads); items that run side by side always build their operands themselves.
struct BatchOrder {
    bool overlap = false;
    uint32_t launched = 0;
    uint32_t next() { return overlap ? (launched++ ? 2u : 1u) : 0u; }
};
static bool batch_item_prepares_operands(const strix_cuda *h, const Resident *w, int act) {
    return act == STRIX_ACT_Q8DOT && h->tune.xop != 0 && w->L.in_dim >= h->tune.xop_single_min_k && w->L.in_dim <= 16384u;
}
static BatchOrder batch_order(const strix_cuda *h, size_t n, const Resident *const *ws, int act, const std::vector<char> &is_small) {
    BatchOrder o;
    o.overlap = h->batch_overlap != 0 && h->tune.pdl != 0;
    for (size_t i = 0; o.overlap && i < n; i++)
        if (ws[i] && !is_small[i] && batch_item_prepares_operands(h, ws[i], act)) o.overlap = false;
    return o;
}
// one item as a launch of its own
static int batch_enqueue_one(strix_cuda *h, size_t i, const Resident *const *ws, const float *const *d_xs, float *const *d_ys,
                             float *const *peer_ys, int n_peers, int act, cudaStream_t s, BatchOrder &order) {
    const Resident *w1[1] = {ws[i]};
    float *y1[1] = {d_ys ? d_ys[i] : nullptr};
    if (!peer_ys && !order.overlap) return gemv_launch(h, 1, w1, d_xs[i], nullptr, 0.f, STRIX_PRE_NONE, act, y1, nullptr, s);
    GemvArgs a{};
    if (gemv_fill_args(h, 1, w1, d_xs[i], nullptr, 0.f, STRIX_PRE_NONE, act, y1, nullptr, &a) < 0) return -1;
    batch_set_peers(a, ws[i], peer_ys, i, n_peers);
    a.nbatch = 1;
    if (!gemv_plan(a, h->num_sms, h->smem_optin, h->tune)) {
        h->err = "gemv_batch: in_dim too large for the shared-memory pipeline";
        return -1;
    }
    a.order = order.next();
    ProfScope prof(h, s, gemv_prof_name(a));
    CU_TRY(h, launch_gemv(a, s));
    return 1;
}
static int batch_enqueue_side_by_side(strix_cuda *h, const std::vector<size_t> &idx, const Resident *const *ws,
                                      const float *const *d_xs, float *const *d_ys, int act, cudaStream_t s,
                                      BatchOrder &order, float *const *peer_ys = nullptr, int n_peers = 0) {
    for (size_t at = 0; at < idx.size(); at += GEMV_MULTI_MAX) {
        const size_t cnt = std::min<size_t>(GEMV_MULTI_MAX, idx.size() - at);
        GemvMultiArgs m{};
        m.n = (uint32_t)cnt;
        bool ok = cnt >= 2;
        for (size_t k = 0; ok && k < cnt; k++) {
            const size_t i = idx[at + k];
            const Resident *w1[1] = {ws[i]};
            float *y1[1] = {d_ys ? d_ys[i] : nullptr};
            if (gemv_fill_args(h, 1, w1, d_xs[i], nullptr, 0.f, STRIX_PRE_NONE, act, y1, nullptr, &m.p[k]) < 0) return -1;
            batch_set_peers(m.p[k], ws[i], peer_ys, i, n_peers);
        }
        if (ok) ok = gemv_multi_plan(m, h->num_sms, h->smem_optin, h->tune);
        if (ok) {
            m.order = order.next();
            ProfScope prof(h, s, "gemv_multi");
            CU_TRY(h, launch_gemv_multi(m, s));
            continue;
        }
        for (size_t k = 0; k < cnt; k++)
            if (batch_enqueue_one(h, idx[at + k], ws, d_xs, d_ys, peer_ys, n_peers, act, s, order) < 0) return -1;
    }
    return 1;
}

// Which items of a batch run side by side in one launch: those whose weights are at most batch_small_bytes (a large
// weight saturates the memory system from a launch of its own), if there are at least two of them.
static std::vector<size_t> batch_small_items(const strix_cuda *h, size_t n, const Resident *const *ws) {
    std::vector<size_t> small;
    if (h->batch_side_by_side == 0) return small;
    for (size_t i = 0; i < n; i++)
        if (ws[i] && (h->batch_side_by_side == 2 || ws[i]->bytes <= h->batch_small_bytes)) small.push_back(i);
    if (small.size() < 2) small.clear();
    return small;
}
}  // namespace strix

namespace strix {
// "gemv.<format>.<activation form>" of a planned launch (string literals: ProfScope keeps the pointer)
const char *gemv_prof_name(const GemvArgs &a) {
    static const char *const names[4][3] = {{"gemv.q4_0.f32", "gemv.q4_0.q8dot", "gemv.q4_0.f32_digits"},
                                            {"gemv.q8_0.f32", "gemv.q8_0.q8dot", "gemv.q8_0.f32_digits"},
                                            {"gemv.q6_k.f32", "gemv.q6_k.q8dot", "gemv.q6_k.f32_digits"},
                                            {"gemv.q4_1.f32", "gemv.q4_1.q8dot", "gemv.q4_1.q8dot"}};
    const int f = a.L.fmt == FMT_Q4_0 ? 0 : a.L.fmt == FMT_Q8_0 ? 1 : a.L.fmt == FMT_Q6_K ? 2 : 3;
    return names[f][a.digits ? 2 : a.act == STRIX_ACT_Q8DOT ? 1 : 0];
}
}  // namespace strix

// Per-kernel totals since the last reset, as text (most expensive first; the reference's prof_dump, decode.rs:36-69).
// Returns the length of the whole text; with a buffer, at most cap - 1 characters of it are copied and the totals are
// reset; without one (a sizing call) they are kept.
size_t strix_cuda_profile_dump(strix_cuda *h, char *buf, size_t cap) {
    if (!h) return 0;
    cudaSetDevice(h->device);
    prof_fold(h);
    std::vector<std::pair<std::string, std::pair<double, uint32_t>>> v(h->prof_total.begin(), h->prof_total.end());
    std::sort(v.begin(), v.end(), [](const auto &x, const auto &y) { return x.second.first > y.second.first; });
    double total = 0;
    for (auto &e : v) total += e.second.first;
    std::string out;
    char line[256];
    snprintf(line, sizeof line, "== strix profile: total kernel time %.3f ms ==\n", total);
    out += line;
    for (auto &e : v) {
        snprintf(line, sizeof line, "  %24s  %9.3f ms  %6u calls  %5.1f%%  (%.4f ms/call)\n", e.first.c_str(), e.second.first,
                 e.second.second, total > 0 ? e.second.first / total * 100.0 : 0.0, e.second.first / e.second.second);
        out += line;
    }
    if (buf && cap) {
        const size_t n = std::min(out.size(), cap - 1);
        memcpy(buf, out.data(), n);
        buf[n] = 0;
        h->prof_total.clear();  // (a call without a buffer only asks for the length)
    }
    return out.size();
}

// One GEMV launch over up to 3 resident weights that share the activation.
namespace strix {
int gemv_launch(strix_cuda *h, int nmat, const Resident *const *ws, const float *d_a, const float *d_b, float eps,
                int pre, int act, float *const *d_ys, const float *const *d_res, cudaStream_t stream) {
    return gemv_launch_rows(h, nmat, ws, d_a, d_b, eps, pre, act, d_ys, d_res, 1, 0, 0, stream);
}

// b activation rows (a_stride / b_stride floats apart; outputs rows-of-the-weight floats apart) share
// one pass over the weights. Rows are taken in chunks when their activations do not fit in shared
// memory next to at least two pipeline stages.
// The launch arguments of one step (everything but the geometry, which a plan fills in).
int gemv_fill_args(strix_cuda *h, int nmat, const Resident *const *ws, const float *d_a, const float *d_b, float eps,
                   int pre, int act, float *const *d_ys, const float *const *d_res, GemvArgs *out) {
    if (nmat < 1 || nmat > GEMV_MAX_MATS) {
        h->err = "gemv: between 1 and 3 weights per launch";
        return -1;
    }
    if (act != STRIX_ACT_F32 && act != STRIX_ACT_Q8DOT) {
        h->err = "gemv: unknown activation mode";
        return -1;
    }
    GemvArgs a{};
    a.nmat = nmat;
    a.L = ws[0]->L;
    for (int m = 0; m < nmat; m++) {
        if (ws[m]->fmt != ws[0]->fmt || ws[m]->L.in_dim != ws[0]->L.in_dim) {
            h->err = "gemv: fused weights must share format and in_dim";
            return -1;
        }
        a.mat[m].w = ws[m]->dev;
        a.mat[m].y = d_ys[m];
        a.mat[m].res = d_res ? d_res[m] : nullptr;
        a.mat[m].rows = (uint32_t)ws[m]->rows;
        a.mat[m].ystride = (uint32_t)ws[m]->rows;
    }
    a.a = d_a;
    a.b = d_b;
    a.eps = eps;
    a.pre = pre;
    a.act = act;
    a.status = h->d_status;
    *out = a;
    return 1;
}

int gemv_launch_rows(strix_cuda *h, int nmat, const Resident *const *ws, const float *d_a, const float *d_b, float eps,
                     int pre, int act, float *const *d_ys, const float *const *d_res, uint32_t b, uint32_t a_stride,
                     uint32_t b_stride, cudaStream_t stream) {
    GemvArgs a{};
    if (gemv_fill_args(h, nmat, ws, d_a, d_b, eps, pre, act, d_ys, d_res, &a) < 0) return -1;
    a.a_stride = a_stride;
    a.b_stride = b_stride;
    uint32_t done = 0;
    while (done < b) {
        uint32_t chunk = std::min<uint32_t>(b - done, 8u);
        GemvArgs c = a;
        for (;; chunk = (chunk + 1) / 2) {
            c = a;
            c.nbatch = chunk;
            if (gemv_plan(c, h->num_sms, h->smem_optin, h->tune)) break;
            if (chunk == 1) {
                h->err = "gemv: in_dim too large for the shared-memory pipeline";
                return -1;
            }
        }
        c.a = d_a + (size_t)done * a_stride;
        c.b = d_b ? d_b + (size_t)done * b_stride : nullptr;
        // Several activation rows in the integer-dot form: their operands are prepared ONCE by a kernel of its own
        // and fetched by every CTA, instead of being quantised by each of the 148 CTAs (8 rows of 15360 cost a CTA
        // ~15 us of prologue, on the critical path of a launch whose weights stream in 5 us). One row stays with
        // the in-kernel prologue while it is short: there a second launch costs more than it saves; from
        // xop_single_min_k elements on (the ffn-long rows of the down projections) it is prepared the same way.
        if (act == STRIX_ACT_Q8DOT && (chunk >= 2 || a.L.in_dim >= h->tune.xop_single_min_k) && a.L.in_dim <= 16384u && h->tune.xop != 0) {
            if (ensure_xop(h, xop_image_bytes(a.L.fmt, a.L.in_dim, chunk)) < 0) return -1;
            ProfScope prof(h, stream, "xop_prepare");
            CU_TRY(h, launch_xop_prepare(a.L.fmt, a.L.in_dim, chunk, c.a, pre == STRIX_PRE_RMSNORM ? d_b : c.b, a_stride,
                                         b_stride, eps, pre, h->xop, h->tune.pdl != 0, stream));
            c.xop = h->xop;
            c.pre = STRIX_PRE_NONE;
        }
        for (int m = 0; m < nmat; m++) {
            c.mat[m].y = d_ys[m] + (size_t)done * c.mat[m].ystride;
            c.mat[m].res = (d_res && d_res[m]) ? d_res[m] + (size_t)done * c.mat[m].ystride : nullptr;
        }
        {
            ProfScope prof(h, stream, gemv_prof_name(c));
            CU_TRY(h, launch_gemv(c, stream));
        }
        done += chunk;
    }
    return 1;
}
}  // namespace strix

extern "C" {

int strix_cuda_create(int device, const strix_cuda_opts *opts, strix_cuda **out) {
    if (!out) return -1;
    *out = nullptr;
    g_create_error.clear();
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        g_create_error = std::string("cudaSetDevice: ") + cudaGetErrorString(e);
        return -1;
    }
    cudaDeviceProp p{};
    e = cudaGetDeviceProperties(&p, device);
    if (e != cudaSuccess) {
        g_create_error = std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e);
        return -1;
    }
    if (p.major != 10) {
        // Kernels are built for sm_100a only; there is no other code path.
        g_create_error = std::string("device ") + p.name + " is not sm_100 (Blackwell B200); no fallback exists";
        return -1;
    }
    strix_cuda *h = new strix_cuda();
    h->device = device;
    h->rank = opts ? opts->rank : 0;
    h->world = opts && opts->world > 1 ? opts->world : 1;
    h->profile = opts ? opts->profile : 0;
    if (h->rank < 0 || h->rank >= h->world) {
        g_create_error = "rank outside [0, world)";
        delete h;
        return -1;
    }
    h->num_sms = p.multiProcessorCount;
    h->smem_optin = p.sharedMemPerBlockOptin;
    h->name = std::string("cuda:") + std::to_string(device) + " " + p.name + " (sm_" + std::to_string(p.major) +
              std::to_string(p.minor) + "a)";
    e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&h->d_status, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = gemv_prepare_device(h->smem_optin);
    if (e == cudaSuccess) e = chain_prepare_device(h->smem_optin);
    if (e == cudaSuccess) e = gemm_prepare_device();
    if (e == cudaSuccess) e = noalloc_prepare_device(device);
    // the operand image of a GEMV whose activations are prepared by a kernel of their own: at most 8 rows of 16384
    // elements (320 bytes per 32-block), allocated here because its first use may lie inside a stream capture
    if (e == cudaSuccess) {
        const size_t image_max = (size_t)512 * 320 + 4096;
        e = cudaMalloc(&h->xop, image_max);
        if (e == cudaSuccess) h->xop_cap = image_max;
    }
    if (e != cudaSuccess) {
        g_create_error = std::string("create: ") + cudaGetErrorString(e);
        if (h->xop) cudaFree(h->xop);
        if (h->d_status) cudaFree(h->d_status);
        if (h->stream) cudaStreamDestroy(h->stream);
        delete h;
        return -1;
    }
    *out = h;
    return 1;
}

void strix_cuda_destroy(strix_cuda *h) {
    if (!h) return;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->stream);
    decode_release(h);
    prof_fold(h);
    if (h->copy_stream) cudaStreamDestroy(h->copy_stream);
    for (cudaEvent_t e : h->batch_events) cudaEventDestroy(e);
    batch_release(h);
    if (h->batch_flags) cudaFreeHost((void *)h->batch_flags);
    if (h->d_one) cudaFree(h->d_one);
    for (auto &kv : h->weights) {
        cudaFree(kv.second.dev);
        if (kv.second.gemm_codes) cudaFree(kv.second.gemm_codes);
        if (kv.second.scalesT) cudaFree(kv.second.scalesT);
    }
    for (float *p : {h->gm_x.p, h->gm_y.p, h->gm_part.p, h->gm_xd.p, h->gm_xc.p})
        if (p) cudaFree(p);
    if (h->gm_xq) cudaFree(h->gm_xq);
    for (float *p : {h->moe_g.p, h->moe_u.p, h->moe_dy.p, h->moe_out.p, h->moe_w.p, h->moe_sh.p})
        if (p) cudaFree(p);
    if (h->moe_ids) cudaFree(h->moe_ids);
    if (h->am_part) cudaFree(h->am_part);  // one allocation: winners, tickets, ids, values
    if (h->am_pin) cudaFreeHost(h->am_pin);
    if (h->gm_xs) cudaFree(h->gm_xs);
    for (auto &kv : h->f32s) cudaFree(kv.second.p);
    if (h->xop) cudaFree(h->xop);
    if (h->x.p) cudaFree(h->x.p);
    if (h->y.p) cudaFree(h->y.p);
    if (h->pin_in.p) cudaFreeHost(h->pin_in.p);
    if (h->pin_out.p) cudaFreeHost(h->pin_out.p);
    cudaFree(h->d_status);
    cudaStreamDestroy(h->stream);
    delete h;
}

int strix_cuda_set_option(strix_cuda *h, const char *name, long long value) {
    if (!h || !name) return -1;
    h->err.clear();
    const std::string n = name;
    const uint32_t v = (uint32_t)value;
    if (n == "q6k_digits") h->tune.digits_rule = v;
    else if (n == "q8_0_digits") h->tune.q8_digits_rule = v;
    else if (n == "q4_0_digits") h->tune.q4_digits_rule = v;
    else if (n == "gemv_warps_per_group") h->tune.force_wc = v;
    else if (n == "gemv_blocks_per_stage") h->tune.force_ct = v;
    else if (n == "gemv_stages") h->tune.force_sk = v;
    else if (n == "gemv_pdl") h->tune.pdl = v;
    else if (n == "gemv_debug") h->tune.debug = v;
    else if (n == "rows_operand_image") h->tune.xop = v;
    else if (n == "operand_image_min_k") h->tune.xop_single_min_k = v;
    else if (n == "batch_graph") h->use_batch_graph = value != 0;
    else if (n == "kv_f16") h->kv_f16 = value != 0;
    else if (n == "decode_chain") h->decode_chain = value < 0 ? -1 : value != 0;
    else if (n == "chain_debug") h->chain_debug = v;
    else if (n == "poll_limit") h->poll_limit = v ? v : CHAIN_POLL_LIMIT;
    // (what follows leaves a configured decode chain as it is)
    else if (n == "batch_side_by_side") { h->batch_side_by_side = (int)v; return 1; }
    else if (n == "batch_small_bytes") { h->batch_small_bytes = (size_t)value; return 1; }
    else if (n == "batch_overlap") { h->batch_overlap = (int)v; batch_release(h); return 1; }
    else if (n == "profile") { h->profile = value != 0; return 1; }
    else if (n == "chain_trace") {
        h->chain_trace = value != 0;
        if (h->chain_trace) decode_trace_enable(h);
        return 1;
    }
    else return 0;
    // plans made under the old value must not be replayed
    decode_release(h);
    if (h->batch_graph.exec) {
        cudaGraphExecDestroy(h->batch_graph.exec);
        h->batch_graph.exec = nullptr;
    }
    return 1;
}

const char *strix_cuda_last_error(strix_cuda *h) { return h ? h->err.c_str() : ""; }
const char *strix_cuda_create_error(void) { return g_create_error.c_str(); }
const char *strix_cuda_name(strix_cuda *h) { return h ? h->name.c_str() : ""; }
size_t strix_cuda_resident_count(strix_cuda *h) { return h ? h->weights.size() : 0; }

int strix_cuda_upload_q4_0(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len, size_t in_dim,
                           size_t out_dim) {
    return upload_quant(h, FMT_Q4_0, key, bytes, len, in_dim, out_dim, true);
}
int strix_cuda_upload_q8_0(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len, size_t in_dim,
                           size_t out_dim) {
    return upload_quant(h, FMT_Q8_0, key, bytes, len, in_dim, out_dim, true);
}
int strix_cuda_upload_q6_k(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len, size_t in_dim,
                           size_t out_dim) {
    return upload_quant(h, FMT_Q6_K, key, bytes, len, in_dim, out_dim, true);
}
int strix_cuda_upload_q4_1(strix_cuda *h, const char *key, const uint8_t *bytes, size_t len, size_t in_dim, size_t out_dim) {
    return upload_quant(h, FMT_Q4_1, key, bytes, len, in_dim, out_dim, true);
}

int strix_cuda_upload_f32(strix_cuda *h, const char *key, const float *data, size_t n) {
    if (!h || !key || !data) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    DevBuf b{};
    CU_TRY(h, cudaMalloc(&b.p, std::max<size_t>(n, 4) * sizeof(float)));
    b.cap = n;
    cudaError_t e = cudaMemcpy(b.p, data, n * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(b.p);
        h->err = std::string("upload_f32: ") + cudaGetErrorString(e);
        return -1;
    }
    decode_release(h);
    auto it = h->f32s.find(key);
    if (it != h->f32s.end()) {
        cudaFree(it->second.p);
        it->second = b;
    } else {
        h->f32s.emplace(key, b);
    }
    return 1;
}

int strix_cuda_weight_info(strix_cuda *h, const char *key, size_t *in_dim, size_t *out_dim_total,
                           size_t *shard_row0, size_t *shard_rows, int *ggml_type) {
    if (!h || !key) return -1;
    const Resident *r = find_weight(h, key);
    if (!r) return 0;
    if (in_dim) *in_dim = r->L.in_dim;
    if (out_dim_total) *out_dim_total = r->out_total;
    if (shard_row0) *shard_row0 = r->row0;
    if (shard_rows) *shard_rows = r->rows;
    if (ggml_type)
        *ggml_type = r->fmt == FMT_Q4_0 ? GGML_Q4_0 : r->fmt == FMT_Q4_1 ? GGML_Q4_1 : r->fmt == FMT_Q8_0 ? GGML_Q8_0 : GGML_Q6_K;
    return 1;
}

int strix_cuda_gemv_batch(strix_cuda *h, size_t n, const char *const *keys, const float *const *xs,
                          const size_t *ks, float *const *ys, const size_t *y_caps, int act, int *status) {
    if (!h || (n && (!keys || !xs || !ks || !ys || !y_caps))) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    std::vector<const Resident *> ws(n, nullptr);
    int any = 0;
    for (size_t i = 0; i < n; i++) {
        const Resident *r = find_weight(h, keys[i]);
        // the reference returns None for an unknown key or a length mismatch (decode.rs:3833-3836)
        if (!r || ks[i] != r->L.in_dim || y_caps[i] < r->rows) {
            if (status) status[i] = 0;
            continue;
        }
        ws[i] = r;
        if (status) status[i] = 1;
        any = 1;
    }
    if (!any) return n ? 0 : 1;
    // The items are independent, so the device may take them in any order. Units of work, in the order they run:
    // every large item as a launch of its own, first (their outputs, the big ones, leave while later kernels run),
    // then the small items side by side in one launch (gemv_multi_kernel), whose outputs are all that is left to
    // copy when the last kernel ends. Activations and outputs lie back to back in the staging buffers in
    // that order.
    const std::vector<size_t> small = batch_small_items(h, n, ws.data());
    std::vector<char> is_small(n, 0);
    for (size_t i : small) is_small[i] = 1;
    std::vector<std::vector<size_t>> units;
    for (size_t i = 0; i < n; i++)
        if (ws[i] && !is_small[i]) units.push_back({i});
    if (!small.empty()) units.push_back(small);
    const size_t nu = units.size();
    std::vector<size_t> xoff(n, 0), yoff(n, 0), unit_y0(nu, 0), unit_y1(nu, 0);
    size_t xtot = 0, ytot = 0;
    for (size_t u = 0; u < nu; u++) {
        unit_y0[u] = ytot;
        for (size_t i : units[u]) {
            xoff[i] = xtot;
            yoff[i] = ytot;
            xtot += (ws[i]->L.in_dim + 3) & ~(size_t)3;  // keep every x 16-byte aligned
            ytot += (ws[i]->rows + 3) & ~(size_t)3;      // and every y
        }
        unit_y1[u] = ytot;
    }
    if (ensure_f32(h, h->x, xtot) < 0 || ensure_f32(h, h->y, std::max<size_t>(ytot, 1)) < 0) return -1;
    if (ensure_pinned(h, h->pin_in, xtot * 4) < 0 || ensure_pinned(h, h->pin_out, std::max<size_t>(ytot, 1) * 4) < 0)
        return -1;
    float *pin = static_cast<float *>(h->pin_in.p), *pout = static_cast<float *>(h->pin_out.p);
    for (size_t i = 0; i < n; i++)
        if (ws[i]) memcpy(pin + xoff[i], xs[i], ws[i]->L.in_dim * sizeof(float));
    // Outputs leave on a second stream, each as soon as its kernel is done, so that the copies (and the
    // host's own copy out of the pinned buffer) overlap the kernels still to run.
    if (!h->copy_stream) CU_TRY(h, cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking));
    while (h->batch_events.size() < 2 * nu) {
        cudaEvent_t e = nullptr;
        CU_TRY(h, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        h->batch_events.push_back(e);
    }
    // Outputs leave in groups: an event between two launches keeps the second from starting early behind the
    // first (programmatic dependent launch), so small outputs wait for a later unit and only an output that
    // brings the pending bytes to 256 KB (or the last unit) closes a group. group_end[u]: the unit whose
    // event covers unit u's outputs; group_begin[e]: first unit of the group that e closes.
    std::vector<size_t> group_end(nu, 0), group_begin(nu, 0);
    {
        size_t pending = 0, first = nu;
        for (size_t u = 0; u < nu; u++) {
            if (first == nu) first = u;
            pending += (unit_y1[u] - unit_y0[u]) * 4;
            if (pending >= (256u << 10) || u + 1 == nu) {
                for (size_t j = first; j <= u; j++) group_end[j] = u;
                group_begin[u] = first;
                pending = 0;
                first = nu;
            }
        }
    }
    std::vector<const float *> dxs(n, nullptr);
    std::vector<float *> dys(n, nullptr);
    for (size_t i = 0; i < n; i++)
        if (ws[i]) {
            dxs[i] = h->x.p + xoff[i];
            dys[i] = h->y.p + yoff[i];
        }
    constexpr size_t BATCH_GRAPH_MAX = 64;
    // What the device does for this batch: H2D of the activations, then per unit its kernel(s) on the main
    // stream and, on the copy stream, its outputs' D2H followed by a one-word copy that raises the unit's
    // pinned flag. `graph`: the same sequence is being captured (the copy stream joins the main one at the
    // end, the events are capture-internal); otherwise the events are real and the host waits on them.
    auto enqueue = [&](bool graph) -> int {
        CU_TRY(h, cudaMemcpyAsync(h->x.p, pin, xtot * 4, cudaMemcpyHostToDevice, h->stream));
        cudaEvent_t last = nullptr;
        BatchOrder order = batch_order(h, n, ws.data(), act, is_small);
        for (size_t u = 0; u < nu; u++) {
            if (units[u].size() > 1) {
                if (batch_enqueue_side_by_side(h, units[u], ws.data(), dxs.data(), dys.data(), act, h->stream, order) < 0) return -1;
            } else {
                for (size_t i : units[u])
                    if (batch_enqueue_one(h, i, ws.data(), dxs.data(), dys.data(), nullptr, 0, act, h->stream, order) < 0) return -1;
            }
            if (group_end[u] != u) continue;  // its outputs leave with a later unit's (see group_end)
            cudaEvent_t done = h->batch_events[2 * u], copied = h->batch_events[2 * u + 1];
            CU_TRY(h, cudaEventRecord(done, h->stream));
            CU_TRY(h, cudaStreamWaitEvent(h->copy_stream, done, 0));
            // the group's outputs are contiguous in the staging buffers: one copy
            const size_t y0 = unit_y0[group_begin[u]], bytes = (unit_y1[u] - y0) * 4;
            if (bytes) CU_TRY(h, cudaMemcpyAsync(pout + y0, h->y.p + y0, bytes, cudaMemcpyDeviceToHost, h->copy_stream));
            if (graph)
                CU_TRY(h, cudaMemcpyAsync((void *)(h->batch_flags + u), h->d_one, 4, cudaMemcpyDeviceToHost, h->copy_stream));
            CU_TRY(h, cudaEventRecord(copied, h->copy_stream));
            last = copied;
        }
        if (graph && last) CU_TRY(h, cudaStreamWaitEvent(h->stream, last, 0));
        // (the status word goes to ordinary host memory: that copy stays outside the graph)
        if (!graph) CU_TRY(h, cudaMemcpyAsync((void *)(h->batch_flags + BATCH_GRAPH_MAX), h->d_status, 4, cudaMemcpyDeviceToHost, h->stream));
        return 1;
    };
    // (with per-kernel timing on, the launches are made directly: events inside a captured graph cannot be timed)
    const bool use_graph = n <= BATCH_GRAPH_MAX && h->use_batch_graph && !h->profile;
    if (!h->batch_flags) {
        // pinned: one word per unit of a captured batch, and after them the copy of the device status word (into
        // pageable memory that copy would hold the host until the whole batch has run, and no output could be
        // handed over while later kernels still run)
        CU_TRY(h, cudaMallocHost((void **)&h->batch_flags, (BATCH_GRAPH_MAX + 1) * 4));
        CU_TRY(h, cudaMalloc(&h->d_one, 4));
        const uint32_t one = 1;
        CU_TRY(h, cudaMemcpy(h->d_one, &one, 4, cudaMemcpyHostToDevice));
    }
    if (use_graph) {
        // the cached graph fits if every pointer and shape its nodes hold is the same as last time
        auto &bg = h->batch_graph;
        bool same = bg.exec && bg.act == act && bg.w_dev.size() == n && bg.x == h->x.p && bg.y == h->y.p &&
                    bg.pin_in == h->pin_in.p && bg.pin_out == h->pin_out.p && bg.side_by_side == h->batch_side_by_side &&
                    bg.small_bytes == h->batch_small_bytes;
        for (size_t i = 0; same && i < n; i++)
            same = bg.w_dev[i] == (ws[i] ? ws[i]->dev : nullptr) &&
                   (!ws[i] || (bg.rows[i] == ws[i]->rows && bg.in_dim[i] == ws[i]->L.in_dim && bg.fmt[i] == ws[i]->fmt));
        if (!same) {
            if (bg.exec) cudaGraphExecDestroy(bg.exec);
            bg.exec = nullptr;
            cudaGraph_t g = nullptr;
            CU_TRY(h, cudaStreamBeginCapture(h->stream, cudaStreamCaptureModeThreadLocal));
            const int rc = enqueue(true);
            const cudaError_t e = cudaStreamEndCapture(h->stream, &g);
            if (rc < 0 || e != cudaSuccess) {
                if (g) cudaGraphDestroy(g);
                if (rc >= 0) h->err = std::string("gemv_batch: graph capture: ") + cudaGetErrorString(e);
                return -1;
            }
            const cudaError_t ei = cudaGraphInstantiate(&bg.exec, g, 0);
            cudaGraphDestroy(g);
            if (ei != cudaSuccess) {
                bg.exec = nullptr;
                h->err = std::string("gemv_batch: graph instantiate: ") + cudaGetErrorString(ei);
                return -1;
            }
            bg.act = act;
            bg.w_dev.assign(n, nullptr);
            bg.rows.assign(n, 0);
            bg.in_dim.assign(n, 0);
            bg.fmt.assign(n, 0);
            for (size_t i = 0; i < n; i++)
                if (ws[i]) {
                    bg.w_dev[i] = ws[i]->dev;
                    bg.rows[i] = ws[i]->rows;
                    bg.in_dim[i] = ws[i]->L.in_dim;
                    bg.fmt[i] = ws[i]->fmt;
                }
            bg.x = h->x.p;
            bg.y = h->y.p;
            bg.pin_in = h->pin_in.p;
            bg.pin_out = h->pin_out.p;
            bg.side_by_side = h->batch_side_by_side;
            bg.small_bytes = h->batch_small_bytes;
        }
        for (size_t u = 0; u < nu; u++) h->batch_flags[u] = 0u;
        CU_TRY(h, cudaGraphLaunch(bg.exec, h->stream));
        CU_TRY(h, cudaMemcpyAsync((void *)(h->batch_flags + BATCH_GRAPH_MAX), h->d_status, 4, cudaMemcpyDeviceToHost, h->stream));
        // hand each output to the caller as its flag comes up (bounded: once the stream has drained,
        // everything has landed whatever the flag says)
        for (size_t u = 0; u < nu; u++) {
            for (uint64_t spin = 0; h->batch_flags[group_end[u]] == 0u; spin++)
                if ((spin & 0xfffu) == 0xfffu && cudaStreamQuery(h->stream) != cudaErrorNotReady) break;
            for (size_t i : units[u]) memcpy(ys[i], pout + yoff[i], ws[i]->rows * sizeof(float));
        }
    } else {
        if (enqueue(false) < 0) return -1;
        // hand each output to the caller as its copy lands
        for (size_t u = 0; u < nu; u++) {
            CU_TRY(h, cudaEventSynchronize(h->batch_events[2 * group_end[u] + 1]));
            for (size_t i : units[u]) memcpy(ys[i], pout + yoff[i], ws[i]->rows * sizeof(float));
        }
    }
    CU_TRY(h, cudaStreamSynchronize(h->stream));
    const uint32_t st = h->batch_flags[BATCH_GRAPH_MAX];
    if (st != 0) {
        h->err = "gemv: device status " + std::to_string(st) + " (a bounded wait ran out)";
        cudaMemsetAsync(h->d_status, 0, 4, h->stream);
        return -2;
    }
    return 1;
}

// WeightAccel::gemv_batch for device-resident vectors: n independent GEMVs enqueued from `stream`, no copies and
// no synchronisation. Large items first, a launch each; then the small ones side by side in one launch.
static int gemv_batch_device(strix_cuda *h, size_t n, const char *const *keys, const float *const *d_xs, float *const *d_ys,
                             float *const *peer_ys, int n_peers, int act, cudaStream_t s, const char *who) {
    h->err.clear();
    if (act != STRIX_ACT_F32 && act != STRIX_ACT_Q8DOT) {
        h->err = std::string(who) + ": unknown activation mode";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    std::vector<const Resident *> ws(n, nullptr);
    for (size_t i = 0; i < n; i++) {
        ws[i] = find_weight(h, keys[i]);
        if (!ws[i] || !d_xs[i] || (d_ys && !d_ys[i])) return 0;
        for (int p = 0; peer_ys && p < n_peers; p++)
            if (!peer_ys[i * (size_t)n_peers + (size_t)p]) return 0;
    }
    const std::vector<size_t> small = batch_small_items(h, n, ws.data());
    std::vector<char> is_small(n, 0);
    for (size_t i : small) is_small[i] = 1;
    BatchOrder order = batch_order(h, n, ws.data(), act, is_small);
    for (size_t i = 0; i < n; i++)
        if (!is_small[i] && batch_enqueue_one(h, i, ws.data(), d_xs, d_ys, peer_ys, n_peers, act, s, order) < 0) return -1;
    if (!small.empty() && batch_enqueue_side_by_side(h, small, ws.data(), d_xs, d_ys, act, s, order, peer_ys, n_peers) < 0) return -1;
    return 1;
}

int strix_cuda_gemv_batch_dev(strix_cuda *h, size_t n, const char *const *keys, const float *const *d_xs, float *const *d_ys,
                              int act, void *stream) {
    if (!h || (n && (!keys || !d_xs || !d_ys))) return -1;
    return gemv_batch_device(h, n, keys, d_xs, d_ys, nullptr, 0, act, static_cast<cudaStream_t>(stream), "gemv_batch_dev");
}

// The row-sharded form of gemv_batch_dev: every item's rows are stored into the full output vector of every
// accelerator of the group (peer_ys[i * n_peers + p], this GPU's own copy included) by the kernels themselves, over
// peer memory, so no collective follows: strix_cuda_peer_barrier_dev on the same stream makes them safe to read.
int strix_cuda_gemv_batch_peers_dev(strix_cuda *h, size_t n, const char *const *keys, const float *const *d_xs, int n_peers,
                                    float *const *peer_ys, int act, void *stream) {
    if (!h || (n && (!keys || !d_xs || !peer_ys))) return -1;
    if (n_peers < 1 || n_peers > GEMV_MAX_PEERS) {
        h->err = "gemv_batch_peers_dev: between 1 and 8 peers";
        return -1;
    }
    return gemv_batch_device(h, n, keys, d_xs, nullptr, peer_ys, n_peers, act, static_cast<cudaStream_t>(stream),
                             "gemv_batch_peers_dev");
}

int strix_cuda_gemv(strix_cuda *h, const char *key, const float *x, size_t k, float *y, size_t y_cap, int act) {
    if (!h || !key || !x || !y) return -1;
    int status = 0;
    const char *keys[1] = {key};
    const float *xs[1] = {x};
    float *ys[1] = {y};
    int rc = strix_cuda_gemv_batch(h, 1, keys, xs, &k, ys, &y_cap, act, &status);
    if (rc < 0) return rc;
    return status;
}

int strix_cuda_gemv_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_a, const float *d_b,
                        float eps, int pre, int act, float *const *d_ys, void *stream) {
    if (!h || !keys || !d_a || !d_ys) return -1;
    h->err.clear();
    if (nmat < 1 || nmat > GEMV_MAX_MATS) {
        h->err = "gemv_dev: between 1 and 3 weights per launch";
        return -1;
    }
    if (pre != STRIX_PRE_NONE && !d_b) {
        h->err = "gemv_dev: this prologue needs d_b";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    const Resident *ws[GEMV_MAX_MATS];
    for (int m = 0; m < nmat; m++) {
        ws[m] = find_weight(h, keys[m]);
        if (!ws[m]) return 0;
    }
    return gemv_launch(h, nmat, ws, d_a, d_b, eps, pre, act, d_ys, nullptr, static_cast<cudaStream_t>(stream));
}

int strix_cuda_gemv_res_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_a, const float *d_b,
                            float eps, int pre, int act, float *const *d_ys, const float *const *d_res, void *stream) {
    if (!h || !keys || !d_a || !d_ys || !d_res) return -1;
    h->err.clear();
    if (nmat < 1 || nmat > GEMV_MAX_MATS) {
        h->err = "gemv_res_dev: between 1 and 3 weights per launch";
        return -1;
    }
    if (pre != STRIX_PRE_NONE && !d_b) {
        h->err = "gemv_res_dev: this prologue needs d_b";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    const Resident *ws[GEMV_MAX_MATS];
    for (int m = 0; m < nmat; m++) {
        ws[m] = find_weight(h, keys[m]);
        if (!ws[m]) return 0;
    }
    return gemv_launch(h, nmat, ws, d_a, d_b, eps, pre, act, d_ys, d_res, static_cast<cudaStream_t>(stream));
}

int strix_cuda_gemv_peers_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_a, const float *d_b,
                              float eps, int pre, int act, const float *const *d_res, int n_peers,
                              float *const *peer_ys, void *stream) {
    if (!h || !keys || !d_a || !peer_ys) return -1;
    h->err.clear();
    if (nmat < 1 || nmat > GEMV_MAX_MATS || n_peers < 1 || n_peers > GEMV_MAX_PEERS) {
        h->err = "gemv_peers_dev: between 1 and 3 weights, 1 and 8 peers per launch";
        return -1;
    }
    if (pre != STRIX_PRE_NONE && !d_b) {
        h->err = "gemv_peers_dev: this prologue needs d_b";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    const Resident *ws[GEMV_MAX_MATS];
    float *no_y[GEMV_MAX_MATS] = {nullptr, nullptr, nullptr};
    for (int m = 0; m < nmat; m++) {
        ws[m] = find_weight(h, keys[m]);
        if (!ws[m]) return 0;
    }
    GemvArgs a{};
    if (gemv_fill_args(h, nmat, ws, d_a, d_b, eps, pre, act, no_y, d_res, &a) < 0) return -1;
    for (int m = 0; m < nmat; m++) {
        a.mat[m].n_peer = (uint32_t)n_peers;
        a.mat[m].row_base = (uint32_t)ws[m]->row0;
        for (int p = 0; p < n_peers; p++) a.mat[m].peer_y[p] = peer_ys[m * n_peers + p];
    }
    a.nbatch = 1;
    if (!gemv_plan(a, h->num_sms, h->smem_optin, h->tune)) {
        h->err = "gemv_peers_dev: in_dim too large for the shared-memory pipeline";
        return -1;
    }
    {
        ProfScope prof(h, static_cast<cudaStream_t>(stream), gemv_prof_name(a));
        CU_TRY(h, launch_gemv(a, static_cast<cudaStream_t>(stream)));
    }
    return 1;
}

int strix_cuda_enable_peer_access(strix_cuda *h, int peer_device) {
    if (!h) return -1;
    h->err.clear();
    if (peer_device == h->device) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    int can = 0;
    CU_TRY(h, cudaDeviceCanAccessPeer(&can, h->device, peer_device));
    if (!can) return 0;
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();  // not an error: clear it
        return 1;
    }
    CU_TRY(h, e);
    return 1;
}

int strix_cuda_ipc_open(strix_cuda *h, const void *handle, size_t handle_len, void **out) {
    if (!h || !handle || !out) return -1;
    h->err.clear();
    if (handle_len != sizeof(cudaIpcMemHandle_t)) {
        h->err = "ipc_open: a CUDA IPC memory handle is " + std::to_string(sizeof(cudaIpcMemHandle_t)) + " bytes";
        return -1;
    }
    // opened with THIS accelerator's device current: that is the device whose kernels will store into the
    // memory, and the flag lets the runtime set up peer access to the device that owns it
    CU_TRY(h, cudaSetDevice(h->device));
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle, sizeof(hd));
    void *p = nullptr;
    CU_TRY(h, cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess));
    *out = p;
    return 1;
}

int strix_cuda_peek_u32(strix_cuda *h, const void *d_ptr, uint32_t *out) {
    if (!h || !d_ptr || !out) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    CU_TRY(h, cudaMemcpy(out, d_ptr, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    return 1;
}

int strix_cuda_poke_u32(strix_cuda *h, void *d_ptr, uint32_t value) {
    if (!h || !d_ptr) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    CU_TRY(h, cudaMemcpy(d_ptr, &value, sizeof(uint32_t), cudaMemcpyHostToDevice));
    return 1;
}

int strix_cuda_ipc_export(strix_cuda *h, const void *d_ptr, void *handle, size_t handle_cap) {
    if (!h || !d_ptr || !handle) return -1;
    h->err.clear();
    if (handle_cap < sizeof(cudaIpcMemHandle_t)) {
        h->err = "ipc_export: a CUDA IPC memory handle is " + std::to_string(sizeof(cudaIpcMemHandle_t)) + " bytes";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    cudaIpcMemHandle_t hd;
    CU_TRY(h, cudaIpcGetMemHandle(&hd, const_cast<void *>(d_ptr)));
    memcpy(handle, &hd, sizeof(hd));
    return 1;
}

int strix_cuda_ipc_close(strix_cuda *h, void *p) {
    if (!h || !p) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    CU_TRY(h, cudaIpcCloseMemHandle(p));
    return 1;
}

int strix_cuda_peer_barrier_dev(strix_cuda *h, uint32_t *d_epoch, uint32_t *d_local_flags, uint32_t *const *peer_flags,
                                void *stream) {
    if (!h || !d_epoch || !d_local_flags || !peer_flags) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    CU_TRY(h, launch_peer_barrier(d_epoch, d_local_flags, peer_flags, h->rank, h->world, h->d_status, h->poll_limit,
                                  static_cast<cudaStream_t>(stream)));
    return 1;
}

int strix_cuda_gemv_rows_dev(strix_cuda *h, int nmat, const char *const *keys, const float *d_xs, size_t b, int act,
                             float *const *d_ys, void *stream) {
    if (!h || !keys || !d_xs || !d_ys) return -1;
    h->err.clear();
    if (nmat < 1 || nmat > GEMV_MAX_MATS) {
        h->err = "gemv_rows_dev: between 1 and 3 weights per launch";
        return -1;
    }
    if (b == 0) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    const Resident *ws[GEMV_MAX_MATS];
    for (int m = 0; m < nmat; m++) {
        ws[m] = find_weight(h, keys[m]);
        if (!ws[m]) return 0;
    }
    return gemv_launch_rows(h, nmat, ws, d_xs, nullptr, 0.f, STRIX_PRE_NONE, act, d_ys, nullptr, (uint32_t)b,
                            ws[0]->L.in_dim, 0, static_cast<cudaStream_t>(stream));
}

int strix_cuda_gemv_rows(strix_cuda *h, const char *key, const float *xs, size_t b, float *y, size_t y_cap, int act) {
    if (!h || !key || !xs || !y) return -1;
    h->err.clear();
    const Resident *r = find_weight(h, key);
    if (!r) return 0;
    if (b == 0) return 1;
    if (y_cap < b * r->rows) {
        h->err = "gemv_rows: output too small";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    const size_t K = r->L.in_dim;
    if (ensure_f32(h, h->x, b * K) < 0 || ensure_f32(h, h->y, std::max<size_t>(b * r->rows, 1)) < 0) return -1;
    CU_TRY(h, cudaMemcpyAsync(h->x.p, xs, b * K * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    const Resident *w1[1] = {r};
    float *y1[1] = {h->y.p};
    if (gemv_launch_rows(h, 1, w1, h->x.p, nullptr, 0.f, STRIX_PRE_NONE, act, y1, nullptr, (uint32_t)b, (uint32_t)K, 0,
                         h->stream) < 0)
        return -1;
    if (r->rows) CU_TRY(h, cudaMemcpyAsync(y, h->y.p, b * r->rows * sizeof(float), cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaMemcpyAsync(&h->status_host, h->d_status, 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaStreamSynchronize(h->stream));
    if (h->status_host != 0) {
        h->err = "gemv_rows: device status " + std::to_string(h->status_host) + " (a bounded wait ran out)";
        cudaMemsetAsync(h->d_status, 0, 4, h->stream);
        return -2;
    }
    return 1;
}

int strix_cuda_device_status(strix_cuda *h, void *stream, uint32_t *status) {
    if (!h || !status) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CU_TRY(h, cudaMemcpyAsync(&h->status_host, h->d_status, 4, cudaMemcpyDeviceToHost, s));
    CU_TRY(h, cudaStreamSynchronize(s));
    *status = h->status_host;
    return 1;
}

int strix_cuda_clear_device_status(strix_cuda *h, void *stream) {
    if (!h) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CU_TRY(h, cudaMemsetAsync(h->d_status, 0, 4, s));
    CU_TRY(h, cudaStreamSynchronize(s));
    return 1;
}

int strix_cuda_dequant_to_f32(strix_cuda *h, const char *key, float *out, size_t out_cap) {
    if (!h || !key || !out) return -1;
    h->err.clear();
    const Resident *r = find_weight(h, key);
    if (!r) return 0;
    const size_t n = r->rows * (size_t)r->L.in_dim;
    if (out_cap < n) {
        h->err = "dequant_to_f32: output too small";
        return -1;
    }
    if (n == 0) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    float *d = nullptr;
    CU_TRY(h, cudaMalloc(&d, n * sizeof(float)));
    cudaError_t e = launch_dequant(r->dev, d, r->L, (uint32_t)r->rows, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, d, n * sizeof(float), cudaMemcpyDeviceToHost, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    cudaFree(d);
    if (e != cudaSuccess) {
        h->err = std::string("dequant_to_f32: ") + cudaGetErrorString(e);
        return -1;
    }
    return 1;
}

int strix_cuda_xquant8(strix_cuda *h, const float *x, size_t n, int8_t *q, float *d) {
    if (!h || !x || !q || !d) return -1;
    h->err.clear();
    if (n % 32 != 0 || n > 0x7fffffffu) {
        h->err = "xquant8: n must be a multiple of 32";
        return -1;
    }
    if (n == 0) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    float *dx = nullptr, *dd = nullptr;
    int8_t *dq = nullptr;
    cudaError_t e = cudaMalloc(&dx, n * 4);
    if (e == cudaSuccess) e = cudaMalloc(&dd, n / 32 * 4);
    if (e == cudaSuccess) e = cudaMalloc(&dq, n);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dx, x, n * 4, cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess) e = launch_xquant8(dx, dq, dd, (uint32_t)n, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(q, dq, n, cudaMemcpyDeviceToHost, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d, dd, n / 32 * 4, cudaMemcpyDeviceToHost, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    cudaFree(dx);
    cudaFree(dd);
    cudaFree(dq);
    if (e != cudaSuccess) {
        h->err = std::string("xquant8: ") + cudaGetErrorString(e);
        return -1;
    }
    return 1;
}

}  // extern "C"
