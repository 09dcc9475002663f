// Resident decode step: the per-token projection chain, four GEMV launches per layer.
//
// Mirrors the projection part of RocmWeightAccel::configure_decode / decode_step
// (crates/strix-backend-rocm/src/decode.rs:4528-4622, 5047-5531) and the CPU forward it
// must agree with (crates/strix-backend-cpu/src/qwen3.rs:818-899):
//
//   per layer:  n = rmsnorm(h, attn_norm);  q,k,v = Wq n, Wk n, Wv n      (one launch, norm fused)
//               a = attention(q, k, v)                                     -- NOT on this path
//               h += Wo a                                                  (one launch, residual fused)
//               n = rmsnorm(h, ffn_norm);  g,u = Wg n, Wu n                (one launch, norm fused)
//               h += Wd (act(g) * u)                                       (one launch, SwiGLU/GeGLU + residual fused)
//   logits = Whead rmsnorm(h, output_norm)                                 (one launch, norm fused)
//
// The reference needs 12 launches per layer for the same work (decode.rs:5239-5477); here the
// norm, the activation quantiser, the gate activation and the residual add live inside the GEMV.
// Attention comes in two forms. `attn_standin_q = 1` feeds Wo with q itself (n_heads * head_dim
// values): the projection chain alone, which is what the benchmark's decode configuration times.
// `attn_standin_q = 0` runs real attention (attention.cu) between the q/k/v step and the o step, in the
// flavours of the reference's three forwards: dense Qwen3 (QK-norm, half-split rope), SmolLM3 (no QK-norm,
// adjacent-pair rope, layers without rope) and Gemma (per-layer head sizes, V = raw K on layers without a V
// projection, weightless V-norm, frequency factors, sliding window on local layers, scale 1 or 1/sqrt(hd),
// sandwich post-norm residuals with a per-layer output scale, final logit soft-cap), with an f32 or f16 KV cache.
//
// With the attention stand-in and integer-dot activations the whole chain runs as ONE persistent
// cooperative kernel (chain.cu): the steps above become a list the kernel walks; its producer warps
// prefetch the next steps' weights without pause and the activations pass from step to step through
// exchange vectors of {value, epoch} entries (no grid barrier). SwiGLU / GeGLU then sit in the epilogue
// of the gate|up step. The list holds device pointers, so it is built (and uploaded) once per
// (hidden-state, logits) buffer pair, outside any stream capture; a pair first seen inside a capture,
// f32 activations and real attention take the launch-per-step path.
//
// The step is captured into a CUDA graph on the first call and replayed afterwards
// (one H2D of h, one graph launch, one D2H of the logits, one sync per token).
#include <algorithm>
#include <cmath>
#include <cstdio>
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

struct strix_decode_state {
    strix_gpu_decode_config cfg{};
    struct Layer {
        const Resident *q, *k, *v, *o, *gate, *up, *down;  // v = null: the layer shares K and V (gemma.rs:796-803)
        const float *attn_norm, *ffn_norm;
        const float *q_norm = nullptr, *k_norm = nullptr;  // real attention with QK-norm only
        const float *post_attn = nullptr, *post_ffw = nullptr;  // sandwich post-norm weights (post_norm models)
        float out_scale = 1.f;                                  // per-layer output scale of a post_norm model
        size_t qdim = 0, kvdim = 0;                             // rows of Wq, of Wk
        // real attention
        uint32_t hd = 0, n_kv = 0, window = 0;
        int rope = ATT_ROPE_CHAIN, rope_adjacent = 0;
        float theta_scale = 1.f;  // rope base ^ (-2 / head_dim), computed on the host (ATT_ROPE_CHAIN)
        float theta = 0.f;        // rope base (ATT_ROPE_POW)
        const float *freq = nullptr;
        float scale = 1.f;
        void *kc = nullptr, *vc = nullptr;  // this layer's cache rows inside kv_block
    };
    std::vector<Layer> layers;
    const Resident *head = nullptr;
    const float *out_norm = nullptr;
    // activations (device)
    float *h = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *gate = nullptr, *up = nullptr, *logits = nullptr;
    void *pin_h = nullptr, *pin_logits = nullptr;
    cudaGraphExec_t exec = nullptr;
    // real attention (attn_standin_q = 0): KV cache (per layer [max_seq][n_kv * hd] for k and for v, f32 or f16,
    // one allocation), the softmax partials, the attention output, and the position word the kernels read (a graph
    // replays unchanged)
    bool real_attn = false, kv_f16 = false;
    void *kv_block = nullptr;
    float *att_part = nullptr, *attn = nullptr;
    float *t = nullptr;  // a projection's output before its sandwich post-norm (post_norm models)
    uint32_t *d_pos = nullptr, *pin_pos = nullptr;
    // batched rows (prefill / verify, up to ROWS_MAX tokens per call): [m][dim] activations, [m] positions
    float *r_h = nullptr, *r_q = nullptr, *r_k = nullptr, *r_v = nullptr, *r_attn = nullptr, *r_gate = nullptr,
          *r_up = nullptr, *r_logits = nullptr, *r_t = nullptr;
    uint32_t *r_pos = nullptr;
    void *r_pin_in = nullptr, *r_pin_out = nullptr;
    cudaGraphExec_t r_exec[2][9] = {};  // [all logits?][rows]: the batched chain captured once per shape
    size_t qdim = 0, kvdim = 0;  // the largest layer's
    // chain-kernel programs, one per (h, logits) buffer pair
    struct Program {
        const float *h;
        const float *logits;
        ChainStep *d_steps;
        uint32_t n_steps;
        ChainGeom geom;
    };
    std::vector<Program> programs;
    // exchange vectors of the chain kernel ({f32 value, epoch} entries): q, the hidden state before and
    // after the attention block, the gated FFN activation; and the kernel's two control words
    // (one allocation, so that a group of accelerators can map each other's block through one IPC handle;
    // peer[r] = rank r's block as mapped into this process, own block included, once the group is wired)
    unsigned long long *ll_block = nullptr;
    size_t ll_off[4] = {0, 0, 0, 0}, ll_words = 0;  // q, h_a, h_b, act: offsets in entries
    unsigned long long *peer[GEMV_MAX_PEERS] = {};
    int n_peer = 0;
    uint32_t *d_ctl = nullptr;
    unsigned long long *d_trace = nullptr;  // measurement only (option "chain_trace"): per-step clocks of CTA 0
    uint32_t trace_n = 0;
    bool chain_ok = true;  // false once a plan has failed: every call takes the launch-per-step path
};

static void decode_free(strix_decode_state *d) {
    if (!d) return;
    for (float *p : {d->h, d->q, d->k, d->v, d->gate, d->up, d->logits, d->att_part, d->attn, d->t})
        if (p) cudaFree(p);
    if (d->kv_block) cudaFree(d->kv_block);
    for (float *p : {d->r_h, d->r_q, d->r_k, d->r_v, d->r_attn, d->r_gate, d->r_up, d->r_logits, d->r_t})
        if (p) cudaFree(p);
    for (auto &row : d->r_exec)
        for (cudaGraphExec_t g : row)
            if (g) cudaGraphExecDestroy(g);
    if (d->r_pos) cudaFree(d->r_pos);
    if (d->r_pin_in) cudaFreeHost(d->r_pin_in);
    if (d->r_pin_out) cudaFreeHost(d->r_pin_out);
    if (d->d_pos) cudaFree(d->d_pos);
    if (d->pin_pos) cudaFreeHost(d->pin_pos);
    if (d->pin_h) cudaFreeHost(d->pin_h);
    if (d->pin_logits) cudaFreeHost(d->pin_logits);
    if (d->exec) cudaGraphExecDestroy(d->exec);
    for (auto &p : d->programs) cudaFree(p.d_steps);
    for (unsigned long long *p : {d->ll_block, d->d_trace})
        if (p) cudaFree(p);
    if (d->d_ctl) cudaFree(d->d_ctl);
    delete d;
}

namespace strix {
void decode_release(strix_cuda *h) {
    decode_free(h->decode);
    h->decode = nullptr;
}
// Option "chain_trace" switched on for a chain that is already configured (and, row-sharded, already wired to its
// peers): the trace words are allocated now, and the captured token step, which holds the old null pointer, goes.
void decode_trace_enable(strix_cuda *h) {
    strix_decode_state *d = h->decode;
    if (!d || d->d_trace) return;
    const size_t n = 4 * d->layers.size() + 1;
    const size_t nb = (size_t)CHAIN_TRACE_WORDS * n * sizeof(unsigned long long);
    if (cudaMalloc(&d->d_trace, nb) != cudaSuccess) {
        cudaGetLastError();
        d->d_trace = nullptr;
        return;
    }
    cudaMemset(d->d_trace, 0, nb);
    cudaDeviceSynchronize();
    d->trace_n = (uint32_t)n;
    if (d->exec) {
        cudaGraphExecDestroy(d->exec);
        d->exec = nullptr;
    }
}
}  // namespace strix

static const float *f32_of(strix_cuda *h, const std::string &key, size_t n) {
    auto it = h->f32s.find(key);
    if (it == h->f32s.end() || it->second.cap < n) return nullptr;
    return it->second.p;
}

// The chain as a list of steps, handed one at a time to `emit` (launch it, or collect it).
// `mid(layer index)` runs between the q/k/v step and the o step and returns the vector Wo is fed with
// (q itself for the stand-in; the attention output otherwise), or null on error. In a post_norm model the o and
// down steps write into d->t and `post(layer index, 0 | 1)` folds that into h (sandwich norm, residual, output scale).
template <typename Emit, typename Mid, typename Post>
static int walk_chain(strix_decode_state *d, Emit emit, Mid mid, Post post) {
    const float eps = d->cfg.eps;
    const int gate_pre = d->cfg.act_gelu ? STRIX_PRE_GEGLU : STRIX_PRE_SWIGLU;
    const bool sandwich = d->cfg.post_norm != 0;
    for (size_t il = 0; il < d->layers.size(); il++) {
        auto &L = d->layers[il];
        {
            const Resident *w[3] = {L.q, L.k, L.v};
            float *y[3] = {d->q, d->k, d->v};
            if (emit(L.v ? 3 : 2, w, d->h, L.attn_norm, eps, STRIX_PRE_RMSNORM, y, nullptr) < 0) return -1;
        }
        {   // h += Wo a, a = the attention output (or q itself: the stand-in)
            const float *a = mid(il);
            if (!a) return -1;
            const Resident *w[1] = {L.o};
            float *y[1] = {sandwich ? d->t : d->h};
            const float *r[1] = {d->h};
            if (emit(1, w, a, nullptr, 0.f, STRIX_PRE_NONE, y, sandwich ? nullptr : r) < 0) return -1;
            if (sandwich && post(il, 0) < 0) return -1;
        }
        {
            const Resident *w[2] = {L.gate, L.up};
            float *y[2] = {d->gate, d->up};
            if (emit(2, w, d->h, L.ffn_norm, eps, STRIX_PRE_RMSNORM, y, nullptr) < 0) return -1;
        }
        {
            const Resident *w[1] = {L.down};
            float *y[1] = {sandwich ? d->t : d->h};
            const float *r[1] = {d->h};
            if (emit(1, w, d->gate, d->up, 0.f, gate_pre, y, sandwich ? nullptr : r) < 0) return -1;
            if (sandwich && post(il, 1) < 0) return -1;
        }
    }
    const Resident *w[1] = {d->head};
    float *y[1] = {d->logits};
    return emit(1, w, d->h, d->out_norm, eps, STRIX_PRE_RMSNORM, y, nullptr);
}

// One layer's attention over `rows` tokens whose q / k / v sit in the given buffers.
static int attention_enqueue(strix_cuda *h, strix_decode_state *d, const strix_decode_state::Layer &L, float *q, const float *k,
                             const float *v, float *attn, const uint32_t *pos, uint32_t rows, cudaStream_t s) {
    AttnArgs A{};
    A.q = q;
    A.k = k;
    A.v = L.v ? v : k;
    A.q_norm = L.q_norm;
    A.k_norm = L.k_norm;
    A.freq = L.freq;
    A.kc = L.kc;
    A.vc = L.vc;
    A.part = d->att_part;
    A.attn = attn;
    A.pos = pos;
    A.n_heads = d->cfg.n_heads;
    A.n_kv = L.n_kv;
    A.hd = L.hd;
    A.max_seq = d->cfg.max_seq;
    A.rows = rows;
    A.window = L.window;
    A.kv_f16 = d->kv_f16 ? 1u : 0u;
    A.norm_v = d->cfg.norm_v ? 1u : 0u;
    A.rope = (uint32_t)L.rope;
    A.rope_adjacent = (uint32_t)L.rope_adjacent;
    A.eps = d->cfg.eps;
    A.theta_scale = L.theta_scale;
    A.theta = L.theta;
    A.scale = L.scale;
    A.status = h->d_status;
    ProfScope prof(h, s, "attention");
    const cudaError_t e = launch_attention_step(A, s);
    if (e != cudaSuccess) {
        h->err = std::string("attention: ") + cudaGetErrorString(e);
        return -1;
    }
    return 0;
}

// The sandwich residual after the o (which = 0) or down (which = 1) projection of a post_norm model.
static int post_enqueue(strix_cuda *h, strix_decode_state *d, const strix_decode_state::Layer &L, int which, float *hid,
                        const float *t, uint32_t rows, cudaStream_t s) {
    ProfScope prof(h, s, "addnorm");
    const cudaError_t e = launch_addnorm(hid, t, which ? L.post_ffw : L.post_attn, d->cfg.hidden, d->cfg.eps,
                                         which ? L.out_scale : 1.0f, rows, s);
    if (e != cudaSuccess) {
        h->err = std::string("post-norm: ") + cudaGetErrorString(e);
        return -1;
    }
    return 0;
}

// The chain-kernel program for the current d->h / d->logits, built on first use. Null when the
// chain kernel cannot be used (plan failed, switched off, or a new buffer pair inside a stream capture).
static const strix_decode_state::Program *chain_program(strix_cuda *h, strix_decode_state *d, cudaStream_t s) {
    // (attention is not a GEMV step, and the exchange-vector prologue is the integer-dot one: launches otherwise)
    const bool want_chain = h->decode_chain < 0 ? h->world > 1 : h->decode_chain != 0;
    if (!d->chain_ok || d->real_attn || d->cfg.post_norm || !want_chain || d->cfg.act != STRIX_ACT_Q8DOT) return nullptr;
    for (auto &p : d->programs)
        if (p.h == d->h && p.logits == d->logits) return &p;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return nullptr;
    auto fail = [&]() -> const strix_decode_state::Program * {
        d->chain_ok = false;
        return nullptr;
    };
    if (!d->ll_block) return fail();
    // where a step publishes its rows: into the exchange block of every rank of the group (this rank's own
    // among them); a lone accelerator, or a group not wired yet, into its own block only
    auto publish = [&](ChainMat &m, int which) {
        if (d->n_peer > 1) {
            m.n_out_ll = (uint32_t)d->n_peer;
            for (int r = 0; r < d->n_peer; r++) m.out_ll[r] = d->peer[r] + d->ll_off[which];
        } else {
            m.n_out_ll = 1;
            m.out_ll[0] = d->ll_block + d->ll_off[which];
        }
    };
    const unsigned long long *ll_q = d->ll_block + d->ll_off[0], *ll_ha = d->ll_block + d->ll_off[1],
                             *ll_hb = d->ll_block + d->ll_off[2], *ll_act = d->ll_block + d->ll_off[3];
    const bool sharded = h->world > 1;
    std::vector<ChainStep> steps;
    const int gate_pair = d->cfg.act_gelu ? STRIX_PRE_GEGLU : STRIX_PRE_SWIGLU;
    const size_t nl = d->layers.size();
    auto mat = [&](ChainStep &st, int m, const Resident *w) {
        st.mat[m].w = w->dev;
        st.mat[m].rows = (uint32_t)w->rows;
        st.mat[m].row_base = (uint32_t)w->row0;
    };
    for (size_t il = 0; il < nl; il++) {
        const auto &L = d->layers[il];
        const uint32_t s0 = (uint32_t)(4 * il);
        ChainStep qkv{};
        qkv.nmat = 3;
        qkv.L = L.q->L;
        qkv.act = STRIX_ACT_Q8DOT;
        qkv.pre = STRIX_PRE_RMSNORM;
        qkv.b = L.attn_norm;
        qkv.eps = d->cfg.eps;
        if (il == 0) qkv.a = d->h;
        else { qkv.a_ll = ll_ha; qkv.in_step = s0 - 1; }
        mat(qkv, 0, L.q); mat(qkv, 1, L.k); mat(qkv, 2, L.v);
        publish(qkv.mat[0], 0);
        qkv.mat[0].y = d->q;
        qkv.mat[1].y = d->k;
        qkv.mat[2].y = d->v;
        steps.push_back(qkv);
        ChainStep o{};  // h += Wo q (the stand-in feeds Wo with q itself)
        o.nmat = 1;
        o.L = L.o->L;
        o.act = STRIX_ACT_Q8DOT;
        o.pre = STRIX_PRE_NONE;
        o.a_ll = ll_q;
        o.in_step = s0;
        mat(o, 0, L.o);
        if (il == 0) o.mat[0].res = d->h + L.o->row0;  // (this shard's rows of the hidden state)
        else { o.mat[0].res_ll = ll_ha; o.res_step = s0 - 1; }
        publish(o.mat[0], 2);
        steps.push_back(o);
        ChainStep gu{};  // act(Wg n) * (Wu n), n = rmsnorm(h)
        gu.nmat = 2;
        gu.L = L.gate->L;
        gu.act = STRIX_ACT_Q8DOT;
        gu.pre = STRIX_PRE_RMSNORM;
        gu.pair = gate_pair;
        gu.b = L.ffn_norm;
        gu.eps = d->cfg.eps;
        gu.a_ll = ll_hb;
        gu.in_step = s0 + 1;
        mat(gu, 0, L.gate); mat(gu, 1, L.up);
        publish(gu.mat[0], 3);
        steps.push_back(gu);
        ChainStep dn{};  // h += Wd (...)
        dn.nmat = 1;
        dn.L = L.down->L;
        dn.act = STRIX_ACT_Q8DOT;
        dn.pre = STRIX_PRE_NONE;
        dn.a_ll = ll_act;
        dn.in_step = s0 + 2;
        mat(dn, 0, L.down);
        dn.mat[0].res_ll = ll_hb;
        dn.res_step = s0 + 1;
        publish(dn.mat[0], 1);
        if (il + 1 == nl && !sharded) dn.mat[0].y = d->h;  // the hidden state after the last layer, for the caller
        steps.push_back(dn);
    }
    {
        ChainStep hd{};
        hd.nmat = 1;
        hd.L = d->head->L;
        hd.act = STRIX_ACT_Q8DOT;
        hd.pre = STRIX_PRE_RMSNORM;
        hd.b = d->out_norm;
        hd.eps = d->cfg.eps;
        if (nl == 0) hd.a = d->h;
        else { hd.a_ll = ll_ha; hd.in_step = (uint32_t)(4 * nl - 1); }
        mat(hd, 0, d->head);
        hd.mat[0].y = d->logits;
        steps.push_back(hd);
    }
    strix_decode_state::Program p{};
    if (!chain_plan(steps.data(), (uint32_t)steps.size(), h->num_sms, h->smem_optin, &p.geom)) return fail();
    p.h = d->h;
    p.logits = d->logits;
    p.n_steps = (uint32_t)steps.size();
    if (h->chain_trace && !d->d_trace) {
        const size_t nb = (size_t)CHAIN_TRACE_WORDS * steps.size() * sizeof(unsigned long long);
        if (cudaMalloc(&d->d_trace, nb) == cudaSuccess) {
            cudaMemset(d->d_trace, 0, nb);
            d->trace_n = (uint32_t)steps.size();
        }
    }
    if (cudaMalloc(&p.d_steps, steps.size() * sizeof(ChainStep)) != cudaSuccess ||
        cudaMemcpy(p.d_steps, steps.data(), steps.size() * sizeof(ChainStep), cudaMemcpyHostToDevice) != cudaSuccess) {
        if (p.d_steps) cudaFree(p.d_steps);
        return fail();
    }
    d->programs.push_back(p);
    return &d->programs.back();
}

// Enqueue the whole chain on `s`. Returns 1, or <0 with h->err set.
static int enqueue_chain(strix_cuda *h, strix_decode_state *d, cudaStream_t s) {
    if (const strix_decode_state::Program *p = chain_program(h, d, s)) {
        ProfScope prof(h, s, "chain");
        CU_TRY(h, launch_chain(p->d_steps, p->n_steps, p->geom, d->d_ctl, h->d_status, h->poll_limit, h->chain_debug,
                               h->chain_trace ? d->d_trace : nullptr, h->num_sms, s));
        return 1;
    }
    if (h->world > 1) {
        // (a row shard cannot run the chain launch by launch: every step needs the other shards' rows)
        h->err = "decode: the row-sharded chain needs the persistent chain kernel (planning failed, or it is switched off)";
        return -1;
    }
    const int act = d->cfg.act;
    return walk_chain(d, [&](int nmat, const Resident *const *w, const float *a, const float *b, float eps, int pre,
                             float *const *y, const float *const *r) {
        return gemv_launch(h, nmat, w, a, b, eps, pre, act, y, r, s);
    }, [&](size_t il) -> const float * {
        if (!d->real_attn) return d->q;
        if (attention_enqueue(h, d, d->layers[il], d->q, d->k, d->v, d->attn, d->d_pos, 1, s) < 0) return nullptr;
        return d->attn;
    }, [&](size_t il, int which) { return post_enqueue(h, d, d->layers[il], which, d->h, d->t, 1, s); });
}

extern "C" {

int strix_cuda_configure_decode(strix_cuda *h, const strix_gpu_decode_config *cfg) {
    if (!h || !cfg) return -1;
    h->err.clear();
    decode_release(h);
    const bool real_attn = !cfg->attn_standin_q;
    if (real_attn) {
        // per-layer head sizes within what attention.cu handles (16-byte cache rows, <= ATT_MAX_HD), grouped-query heads
        if (!cfg->layers || cfg->max_seq == 0 || cfg->n_heads == 0) return 0;
        for (uint32_t il = 0; il < cfg->n_layers; il++) {
            const strix_gpu_layer_cfg &lc = cfg->layers[il];
            if (lc.head_dim == 0 || lc.head_dim > ATT_MAX_HD || (lc.head_dim & 3u) || lc.n_kv == 0 || cfg->n_heads % lc.n_kv != 0 ||
                (!lc.no_rope && !(lc.rope_theta > 0.f)))
                return 0;
        }
    }
    if (cfg->act != STRIX_ACT_F32 && cfg->act != STRIX_ACT_Q8DOT) return 0;
    // A sharded handle holds row shards only: the chain then runs as the persistent kernel alone (projection
    // chain with the stand-in, integer-dot form), every rank publishing its rows into all ranks' exchange vectors.
    if (h->world > 1 && (real_attn || cfg->post_norm || cfg->act != STRIX_ACT_Q8DOT || h->decode_chain == 0 || h->world > GEMV_MAX_PEERS))
        return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    auto *d = new strix_decode_state();
    d->cfg = *cfg;
    d->cfg.layers = nullptr;
    d->kv_f16 = real_attn && h->kv_f16 != 0;
    const size_t hidden = cfg->hidden, ffn = cfg->ffn;
    size_t qdim = 0, kvdim = 0, hd_max = 0, cache_bytes = 0;
    auto need = [&](const std::string &key, size_t in_dim, size_t out_dim) -> const Resident * {
        const Resident *r = find_weight(h, key.c_str());
        if (!r || r->L.in_dim != in_dim || (out_dim && r->out_total != out_dim)) return nullptr;
        return r;
    };
    const size_t kv_elem = d->kv_f16 ? 2 : 4;
    bool ok = true;
    for (uint32_t il = 0; il < cfg->n_layers && ok; il++) {
        const std::string b = "blk." + std::to_string(il) + ".";
        strix_decode_state::Layer L{};
        const bool shared_kv = real_attn && cfg->layers[il].k_eq_v;
        L.q = need(b + "attn_q.weight", hidden, 0);
        L.k = need(b + "attn_k.weight", hidden, 0);
        L.v = shared_kv ? nullptr : need(b + "attn_v.weight", hidden, 0);
        ok = L.q && L.k && L.q->fmt == L.k->fmt && (shared_kv || (L.v && L.k->out_total == L.v->out_total && L.q->fmt == L.v->fmt));
        if (!ok) break;
        L.qdim = L.q->out_total;
        L.kvdim = L.k->out_total;
        // the stand-in keeps one q size for all layers (its exchange vectors are sized once)
        ok = real_attn || il == 0 || (L.qdim == qdim && L.kvdim == kvdim);
        qdim = std::max(qdim, L.qdim);
        kvdim = std::max(kvdim, L.kvdim);
        L.o = need(b + "attn_output.weight", L.qdim, hidden);
        L.gate = need(b + "ffn_gate.weight", hidden, ffn);
        L.up = need(b + "ffn_up.weight", hidden, ffn);
        L.down = need(b + "ffn_down.weight", ffn, hidden);
        L.attn_norm = f32_of(h, b + "attn_norm.weight", hidden);
        L.ffn_norm = f32_of(h, b + "ffn_norm.weight", hidden);
        if (cfg->post_norm) {
            // gemma.rs:876-879, 896-906: h += norm(Wo a) * post_attention_norm; h = (h + norm(Wd act) * post_ffw_norm) * scale
            L.post_attn = f32_of(h, b + "post_attention_norm.weight", hidden);
            L.post_ffw = f32_of(h, b + "post_ffw_norm.weight", hidden);
            L.out_scale = cfg->layers ? cfg->layers[il].output_scale : 1.0f;
            ok = ok && L.post_attn && L.post_ffw;
        }
        if (real_attn) {
            const strix_gpu_layer_cfg &lc = cfg->layers[il];
            L.hd = lc.head_dim;
            L.n_kv = lc.n_kv;
            hd_max = std::max<size_t>(hd_max, L.hd);
            if (cfg->qk_norm) {
                L.q_norm = f32_of(h, b + "attn_q_norm.weight", L.hd);
                L.k_norm = f32_of(h, b + "attn_k_norm.weight", L.hd);
                ok = ok && L.q_norm && L.k_norm;
            }
            // Which angle formula: the Gemma forward (the post_norm family) evaluates base^(-2j/hd) per pair and divides
            // by the frequency factors on its global layers (ops.rs:159-176, gemma.rs:819-829); the Qwen3 and SmolLM3
            // forwards multiply the angle by base^(-2/hd) pair after pair (qwen3.rs:126-138, smollm3.rs:126-138).
            if (lc.no_rope) L.rope = ATT_ROPE_NONE;
            else if (cfg->post_norm) {
                L.rope = ATT_ROPE_POW;
                L.theta = lc.rope_theta;
                if (!lc.is_local) L.freq = f32_of(h, "rope_freqs.weight", L.hd / 2);  // absent: no factors
            } else {
                L.rope = ATT_ROPE_CHAIN;
                // theta_scale = freq_base.powf(-2.0 / n_dims) (qwen3.rs:128), evaluated in f32 on the host
                L.theta_scale = powf(lc.rope_theta, -2.0f / (float)L.hd);
            }
            L.rope_adjacent = lc.rope_norm ? 1 : 0;
            L.window = (lc.is_local && cfg->n_swa > 0) ? cfg->n_swa : 0;  // decode.rs:5312-5320
            L.scale = cfg->attn_rsqrt ? 1.0f / sqrtf((float)L.hd) : 1.0f;
            ok = ok && L.qdim == (size_t)cfg->n_heads * L.hd && L.kvdim == (size_t)L.n_kv * L.hd;
            cache_bytes += 2 * (((size_t)cfg->max_seq * L.kvdim * kv_elem + 255) & ~(size_t)255);
        }
        ok = ok && L.o && L.gate && L.up && L.down && L.attn_norm && L.ffn_norm && L.gate->fmt == L.up->fmt;
        d->layers.push_back(L);
    }
    if (ok) {
        d->head = need("output.weight", hidden, cfg->vocab);
        if (!d->head) d->head = need("token_embd.weight", hidden, cfg->vocab);  // tied embedding (qwen3.rs:891-895)
        d->out_norm = f32_of(h, "output_norm.weight", hidden);
        ok = d->head && d->out_norm;
    }
    if (!ok) {  // a weight the chain needs was not adopted: decline, the model keeps per-weight gemv
        decode_free(d);
        return 0;
    }
    cudaError_t e = cudaSuccess;
    auto alloc = [&](float **p, size_t n) {
        if (e == cudaSuccess) e = cudaMalloc(p, std::max<size_t>(n, 4) * sizeof(float));
    };
    alloc(&d->h, hidden);
    alloc(&d->q, qdim);
    alloc(&d->k, kvdim);
    alloc(&d->v, kvdim);
    alloc(&d->gate, ffn);
    alloc(&d->up, ffn);
    alloc(&d->logits, cfg->vocab);
    if (cfg->post_norm) alloc(&d->t, hidden);
    if (real_attn) {
        d->real_attn = true;
        const size_t splits = (cfg->max_seq + ATT_SPLIT_TOKENS - 1) / ATT_SPLIT_TOKENS;
        if (e == cudaSuccess) e = cudaMalloc(&d->kv_block, std::max<size_t>(cache_bytes, 256));
        size_t off = 0;
        for (auto &L : d->layers) {
            const size_t bytes = ((size_t)cfg->max_seq * L.kvdim * kv_elem + 255) & ~(size_t)255;
            L.kc = static_cast<char *>(d->kv_block) + off;
            L.vc = static_cast<char *>(d->kv_block) + off + bytes;
            off += 2 * bytes;
        }
        alloc(&d->att_part, 8 * (size_t)cfg->n_heads * splits * (hd_max + 2));  // up to 8 rows per call (prefill / verify)
        alloc(&d->attn, qdim);
        if (e == cudaSuccess) e = cudaMalloc(&d->d_pos, 4);
        if (e == cudaSuccess) e = cudaMemset(d->d_pos, 0, 4);
        if (e == cudaSuccess) e = cudaMallocHost(&d->pin_pos, 4);
    }
    if (!real_attn && cfg->act == STRIX_ACT_Q8DOT) {
        // exchange vectors of the chain kernel, one allocation: q | h_a | h_b | act, each 128-byte aligned.
        // Epoch 0 = never written: the first launch's steps carry epochs 1, 2, ...
        size_t off = 0;
        const size_t lens[4] = {qdim, hidden, hidden, ffn};
        for (int i = 0; i < 4; i++) {
            d->ll_off[i] = off;
            off += (lens[i] + 15) & ~(size_t)15;
        }
        d->ll_words = off + 16;  // (16 spare entries at the end: room for a mapping-check mark)
        if (e == cudaSuccess) e = cudaMalloc(&d->ll_block, d->ll_words * 8);
        if (e == cudaSuccess) e = cudaMemset(d->ll_block, 0, d->ll_words * 8);
        if (e == cudaSuccess) e = cudaMalloc(&d->d_ctl, 8);
        if (e == cudaSuccess) e = cudaMemset(d->d_ctl, 0, 8);
    }
    if (e == cudaSuccess) e = cudaMallocHost(&d->pin_h, hidden * sizeof(float));
    if (e == cudaSuccess) e = cudaMallocHost(&d->pin_logits, (size_t)cfg->vocab * sizeof(float));
    if (e != cudaSuccess) {
        h->err = std::string("configure_decode: ") + cudaGetErrorString(e);
        decode_free(d);
        return -1;
    }
    d->qdim = qdim;
    d->kvdim = kvdim;
    h->decode = d;
    return 1;
}

}  // extern "C"

// Tokens per prefill / verify call: what one batched-GEMV pass carries (the speculative-verify sizes,
// gamma + 1 <= 8; generate.rs:604-607, 850-853). Longer prompts are chunked by the caller (prefill_max).
static constexpr size_t ROWS_MAX = 8;

static int rows_alloc(strix_cuda *h, strix_decode_state *d) {
    if (d->r_h) return 0;
    {
        // the batched GEMV's operand image, sized for the largest step before anything is captured into a graph
        size_t need = 0;
        auto see = [&](const Resident *w) {
            need = std::max(need, xop_image_bytes(w->fmt, w->L.in_dim, w->fmt == FMT_Q6_K ? 4u : (uint32_t)ROWS_MAX));
        };
        for (auto &L : d->layers)
            for (const Resident *w : {L.q, L.o, L.gate, L.down}) see(w);
        see(d->head);
        if (ensure_xop(h, need) < 0) return -1;
    }
    cudaError_t e = cudaSuccess;
    auto alloc = [&](float **p, size_t n) {
        if (e == cudaSuccess) e = cudaMalloc(p, ROWS_MAX * std::max<size_t>(n, 4) * sizeof(float));
    };
    alloc(&d->r_h, d->cfg.hidden);
    alloc(&d->r_q, d->qdim);
    alloc(&d->r_k, d->kvdim);
    alloc(&d->r_v, d->kvdim);
    alloc(&d->r_attn, d->qdim);
    alloc(&d->r_gate, d->cfg.ffn);
    alloc(&d->r_up, d->cfg.ffn);
    alloc(&d->r_logits, d->cfg.vocab);
    if (d->cfg.post_norm) alloc(&d->r_t, d->cfg.hidden);
    if (e == cudaSuccess) e = cudaMalloc(&d->r_pos, ROWS_MAX * 4);
    if (e == cudaSuccess) e = cudaMallocHost(&d->r_pin_in, ROWS_MAX * (d->cfg.hidden * sizeof(float) + 4));
    if (e == cudaSuccess) e = cudaMallocHost(&d->r_pin_out, ROWS_MAX * (size_t)d->cfg.vocab * sizeof(float));
    if (e != cudaSuccess) {
        h->err = std::string("prefill scratch: ") + cudaGetErrorString(e);
        return -1;
    }
    return 0;
}

static int rows_enqueue(strix_cuda *h, strix_decode_state *d, size_t m, bool all_logits, cudaStream_t s);

// m tokens (rows) through the chain in one pass over the weights per step: the batched GEMV carries
// the rows as extra MMA columns; attention takes all rows in one launch per kernel (their keys and values
// enter the cache first, then row t attends to rows 0 .. its own position: causal). all_logits: the head for every row, else for the last one.
// ids (may be null): the rows' greedy tokens instead of their logits (argmax on the device).
static int rows_run(strix_cuda *h, strix_decode_state *d, const float *hs, size_t start_pos, size_t m, bool all_logits,
                    float *out, size_t out_cap, const char *who, uint32_t *ids = nullptr) {
    if (m == 0 || m > ROWS_MAX) return 0;  // the caller chunks (the reference's `m > M_CHUNK -> None`, decode.rs:5559)
    const size_t hidden = d->cfg.hidden, vocab = d->cfg.vocab, n_out = all_logits ? m : 1;
    if (!ids && out_cap < n_out * vocab) {
        h->err = std::string(who) + ": logits buffer too small";
        return -1;
    }
    if (d->real_attn && start_pos + m > d->cfg.max_seq) {
        h->err = std::string(who) + ": positions up to " + std::to_string(start_pos + m - 1) + " beyond max_seq " +
                 std::to_string(d->cfg.max_seq);
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    if (rows_alloc(h, d) < 0) return -1;
    cudaStream_t s = h->stream;
    float *pin = static_cast<float *>(d->r_pin_in);
    uint32_t *pin_pos = reinterpret_cast<uint32_t *>(pin + ROWS_MAX * hidden);
    memcpy(pin, hs, m * hidden * sizeof(float));
    for (size_t t = 0; t < m; t++) pin_pos[t] = (uint32_t)(start_pos + t);
    CU_TRY(h, cudaMemcpyAsync(d->r_h, pin, m * hidden * sizeof(float), cudaMemcpyHostToDevice, s));
    CU_TRY(h, cudaMemcpyAsync(d->r_pos, pin_pos, m * 4, cudaMemcpyHostToDevice, s));
    // The kernels of one (rows, all-logits) shape are captured into a CUDA graph on first use and replayed
    // afterwards: a call is ~250 launches, and issuing them one by one costs the host about a millisecond.
    // (Positions and activations live in fixed device buffers, so the graph does not depend on them.)
    cudaGraphExec_t &exec = d->r_exec[all_logits ? 1 : 0][m];
    if (!exec) {
        cudaGraph_t g = nullptr;
        CU_TRY(h, cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        const int rc = rows_enqueue(h, d, m, all_logits, s);
        const cudaError_t e = cudaStreamEndCapture(s, &g);
        if (rc < 0 || e != cudaSuccess) {
            if (g) cudaGraphDestroy(g);
            if (rc >= 0) h->err = std::string(who) + ": graph capture: " + cudaGetErrorString(e);
            return -1;
        }
        const cudaError_t ei = cudaGraphInstantiate(&exec, g, 0);
        cudaGraphDestroy(g);
        if (ei != cudaSuccess) {
            exec = nullptr;
            h->err = std::string(who) + ": graph instantiate: " + cudaGetErrorString(ei);
            return -1;
        }
    }
    CU_TRY(h, cudaGraphLaunch(exec, s));
    if (ids) {
        if (argmax_rows_enqueue(h, d->r_logits, vocab, vocab, n_out, s) < 0) return -1;
        CU_TRY(h, cudaMemcpyAsync(h->am_pin, h->am_idx, n_out * 4, cudaMemcpyDeviceToHost, s));
    } else {
        if (d->cfg.final_softcap > 0.f) CU_TRY(h, launch_softcap(d->r_logits, n_out * vocab, d->cfg.final_softcap, s));  // decode.rs:6382-6393
        CU_TRY(h, cudaMemcpyAsync(d->r_pin_out, d->r_logits, n_out * vocab * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    CU_TRY(h, cudaMemcpyAsync(&h->status_host, h->d_status, 4, cudaMemcpyDeviceToHost, s));
    CU_TRY(h, cudaStreamSynchronize(s));
    if (h->status_host != 0) {
        h->err = std::string(who) + ": device status " + std::to_string(h->status_host);
        cudaMemsetAsync(h->d_status, 0, 4, s);
        return -2;
    }
    if (ids)
        for (size_t t = 0; t < n_out; t++) ids[t] = h->am_pin[t];
    else
        memcpy(out, d->r_pin_out, n_out * vocab * sizeof(float));
    return 1;
}

static int rows_enqueue(strix_cuda *h, strix_decode_state *d, size_t m, bool all_logits, cudaStream_t s) {
    const size_t hidden = d->cfg.hidden, n_out = all_logits ? m : 1;
    const int act = d->cfg.act;
    const float eps = d->cfg.eps;
    const int gate_pre = d->cfg.act_gelu ? STRIX_PRE_GEGLU : STRIX_PRE_SWIGLU;
    const uint32_t b = (uint32_t)m, ffn = d->cfg.ffn;
    const bool sandwich = d->cfg.post_norm != 0;
    for (size_t il = 0; il < d->layers.size(); il++) {
        auto &L = d->layers[il];
        {
            const Resident *w[3] = {L.q, L.k, L.v};
            float *y[3] = {d->r_q, d->r_k, d->r_v};
            if (gemv_launch_rows(h, L.v ? 3 : 2, w, d->r_h, L.attn_norm, eps, STRIX_PRE_RMSNORM, act, y, nullptr, b, (uint32_t)hidden, 0, s) < 0)
                return -1;
        }
        const float *a = d->r_q;  // the stand-in feeds Wo with q
        if (d->real_attn) {
            if (attention_enqueue(h, d, L, d->r_q, d->r_k, d->r_v, d->r_attn, d->r_pos, b, s) < 0) return -1;
            a = d->r_attn;
        }
        {
            const Resident *w[1] = {L.o};
            float *y[1] = {sandwich ? d->r_t : d->r_h};
            const float *r[1] = {d->r_h};
            if (gemv_launch_rows(h, 1, w, a, nullptr, 0.f, STRIX_PRE_NONE, act, y, sandwich ? nullptr : r, b, (uint32_t)L.qdim, 0, s) < 0)
                return -1;
            if (sandwich && post_enqueue(h, d, L, 0, d->r_h, d->r_t, b, s) < 0) return -1;
        }
        {
            const Resident *w[2] = {L.gate, L.up};
            float *y[2] = {d->r_gate, d->r_up};
            if (gemv_launch_rows(h, 2, w, d->r_h, L.ffn_norm, eps, STRIX_PRE_RMSNORM, act, y, nullptr, b, (uint32_t)hidden, 0, s) < 0)
                return -1;
        }
        {
            const Resident *w[1] = {L.down};
            float *y[1] = {sandwich ? d->r_t : d->r_h};
            const float *r[1] = {d->r_h};
            if (gemv_launch_rows(h, 1, w, d->r_gate, d->r_up, 0.f, gate_pre, act, y, sandwich ? nullptr : r, b, ffn, ffn, s) < 0) return -1;
            if (sandwich && post_enqueue(h, d, L, 1, d->r_h, d->r_t, b, s) < 0) return -1;
        }
    }
    {
        const Resident *w[1] = {d->head};
        float *y[1] = {d->r_logits};
        const float *x = all_logits ? d->r_h : d->r_h + (m - 1) * hidden;
        if (gemv_launch_rows(h, 1, w, x, d->out_norm, eps, STRIX_PRE_RMSNORM, act, y, nullptr, (uint32_t)n_out, (uint32_t)hidden, 0, s) < 0)
            return -1;
    }
    return 1;
}

extern "C" {

// WeightAccel::prefill (accel.rs:464-473; decode.rs:5555-6394): logits of the LAST of m tokens.
int strix_cuda_prefill(strix_cuda *h, const float *hs, size_t start_pos, size_t m, float *logits, size_t logits_cap) {
    if (!h || !hs || !logits) return -1;
    h->err.clear();
    if (!h->decode) return 0;
    return rows_run(h, h->decode, hs, start_pos, m, false, logits, logits_cap, "prefill");
}
// WeightAccel::verify (accel.rs:500-506; decode.rs:5548-5553): logits of ALL m tokens, token-major.
int strix_cuda_verify(strix_cuda *h, const float *hs, size_t start_pos, size_t m, float *logits, size_t logits_cap) {
    if (!h || !hs || !logits) return -1;
    h->err.clear();
    if (!h->decode) return 0;
    return rows_run(h, h->decode, hs, start_pos, m, true, logits, logits_cap, "verify");
}
int strix_cuda_verify_argmax(strix_cuda *h, const float *hs, size_t start_pos, size_t m, uint32_t *ids) {
    if (!h || !hs || !ids) return -1;
    h->err.clear();
    if (!h->decode || h->world > 1) return 0;
    return rows_run(h, h->decode, hs, start_pos, m, true, nullptr, 0, "verify_argmax", ids);
}
// WeightAccel::prefill_max (accel.rs:475-479): 0 = prefill unsupported (no decode configured).
size_t strix_cuda_prefill_max(strix_cuda *h) { return (h && h->decode) ? ROWS_MAX : 0; }

// WeightAccel::seed_decode_kv (accel.rs:421-427): cache rows 0 .. tokens-1 of layer il from a prefill done
// elsewhere: k already normed and roped, v raw, token-major [tokens][n_kv * head_dim].
int strix_cuda_seed_decode_kv(strix_cuda *h, size_t il, const float *k, const float *v, size_t tokens) {
    if (!h || !k || !v) return -1;
    h->err.clear();
    strix_decode_state *d = h->decode;
    if (!d || !d->real_attn || il >= d->layers.size() || tokens > d->cfg.max_seq) return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    const auto &L = d->layers[il];
    const size_t n = tokens * L.kvdim;
    if (d->kv_f16) {  // the cache holds f16: round on the host the way the cache's own stores do
        std::vector<unsigned short> kh(n), vh(n);
        f32_to_f16_ref(k, kh.data(), n);
        f32_to_f16_ref(v, vh.data(), n);
        CU_TRY(h, cudaMemcpyAsync(L.kc, kh.data(), n * 2, cudaMemcpyHostToDevice, h->stream));
        CU_TRY(h, cudaMemcpyAsync(L.vc, vh.data(), n * 2, cudaMemcpyHostToDevice, h->stream));
        CU_TRY(h, cudaStreamSynchronize(h->stream));
        return 1;
    }
    CU_TRY(h, cudaMemcpyAsync(L.kc, k, n * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    CU_TRY(h, cudaMemcpyAsync(L.vc, v, n * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    CU_TRY(h, cudaStreamSynchronize(h->stream));  // k and v are borrowed for the call
    return 1;
}

// Device-resident form: runs the chain on d_h[hidden] (updated in place) into d_logits[vocab] on `stream`.
int strix_cuda_decode_chain_dev(strix_cuda *h, float *d_h, float *d_logits, void *stream) {
    if (!h || !d_h || !d_logits) return -1;
    h->err.clear();
    strix_decode_state *d = h->decode;
    if (!d || d->real_attn) return 0;  // (the position travels with decode_step only)
    CU_TRY(h, cudaSetDevice(h->device));
    float *save_h = d->h, *save_l = d->logits;
    d->h = d_h;
    d->logits = d_logits;
    int rc = enqueue_chain(h, d, static_cast<cudaStream_t>(stream));
    d->h = save_h;
    d->logits = save_l;
    return rc;
}

// Row-sharded groups: this accelerator's exchange block (one device allocation) so that the caller can
// export it (cudaIpcGetMemHandle) to the other ranks.
int strix_cuda_decode_exchange_info(strix_cuda *h, void **base, size_t *bytes) {
    if (!h || !base || !bytes) return -1;
    h->err.clear();
    strix_decode_state *d = h->decode;
    if (!d || !d->ll_block) return 0;
    *base = d->ll_block;
    *bytes = d->ll_words * 8;
    return 1;
}

// Wires the group: blocks[r] = rank r's exchange block as mapped into this process (blocks[rank] may be null =
// this accelerator's own). From now on every step publishes its rows into all n blocks.
int strix_cuda_decode_set_peers(strix_cuda *h, int n, void *const *blocks) {
    if (!h || !blocks) return -1;
    h->err.clear();
    strix_decode_state *d = h->decode;
    if (!d || !d->ll_block) return 0;
    if (n != h->world || n > GEMV_MAX_PEERS) {
        h->err = "decode_set_peers: one block per rank of the group (at most 8)";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    CU_TRY(h, cudaDeviceSynchronize());
    for (int r = 0; r < n; r++) {
        d->peer[r] = (r == h->rank || !blocks[r]) ? d->ll_block : static_cast<unsigned long long *>(blocks[r]);
        if (r != h->rank && !blocks[r]) {
            h->err = "decode_set_peers: a null block for another rank";
            return -1;
        }
    }
    d->n_peer = n;
    for (auto &p : d->programs) cudaFree(p.d_steps);  // programs built before hold the old destinations
    d->programs.clear();
    if (d->exec) {
        cudaGraphExecDestroy(d->exec);
        d->exec = nullptr;
    }
    d->chain_ok = true;
    return 1;
}

// Measurement only: after set_option("chain_trace", 1) the chain kernel's CTA 0 notes, per step, the clock (ns)
// at its start, when its activations have arrived, after its prologue, after its last row group and after its
// reduction and stores, and the SM clocks spent waiting for weight stages (CHAIN_TRACE_WORDS = 6 words per
// step); this copies out the words of the last launch. Returns the number of steps, 0 without a trace.
int strix_cuda_decode_trace(strix_cuda *h, unsigned long long *out, size_t cap_words) {
    if (!h || !out) return -1;
    h->err.clear();
    strix_decode_state *d = h->decode;
    if (!d || !d->d_trace || cap_words < (size_t)CHAIN_TRACE_WORDS * d->trace_n) return 0;
    CU_TRY(h, cudaSetDevice(h->device));
    CU_TRY(h, cudaDeviceSynchronize());
    CU_TRY(h, cudaMemcpy(out, d->d_trace, (size_t)CHAIN_TRACE_WORDS * d->trace_n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return (int)d->trace_n;
}

// H2D of the hidden state and one replay of the captured chain on the handle's stream (captured on
// the first call); the logits are then in d->logits.
static int decode_enqueue_step(strix_cuda *h, strix_decode_state *d, const float *hvec, size_t pos) {
    CU_TRY(h, cudaSetDevice(h->device));
    if (d->real_attn && pos >= d->cfg.max_seq) {
        h->err = "decode_step: position " + std::to_string(pos) + " beyond max_seq " + std::to_string(d->cfg.max_seq);
        return -1;
    }
    if (!d->exec) {
        cudaGraph_t g = nullptr;
        (void)chain_program(h, d, h->stream);  // built (and uploaded) before the capture starts
        CU_TRY(h, cudaStreamBeginCapture(h->stream, cudaStreamCaptureModeThreadLocal));
        int rc = enqueue_chain(h, d, h->stream);
        cudaError_t e = cudaStreamEndCapture(h->stream, &g);
        if (rc < 0 || e != cudaSuccess) {
            if (g) cudaGraphDestroy(g);
            if (rc >= 0) h->err = std::string("decode_step: graph capture: ") + cudaGetErrorString(e);
            return -1;
        }
        e = cudaGraphInstantiate(&d->exec, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) {
            d->exec = nullptr;
            h->err = std::string("decode_step: graph instantiate: ") + cudaGetErrorString(e);
            return -1;
        }
    }
    memcpy(d->pin_h, hvec, d->cfg.hidden * sizeof(float));
    CU_TRY(h, cudaMemcpyAsync(d->h, d->pin_h, d->cfg.hidden * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    if (d->real_attn) {
        // the captured kernels read the position from this word: row `pos` of the cache is (re)written, rows
        // 0..pos are attended to. (The previous step's copy has completed: every step ends with a sync.)
        *d->pin_pos = (uint32_t)pos;
        CU_TRY(h, cudaMemcpyAsync(d->d_pos, d->pin_pos, 4, cudaMemcpyHostToDevice, h->stream));
    }
    CU_TRY(h, cudaGraphLaunch(d->exec, h->stream));
    return 1;
}

static int decode_finish(strix_cuda *h, const char *who) {
    CU_TRY(h, cudaMemcpyAsync(&h->status_host, h->d_status, 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaStreamSynchronize(h->stream));
    if (h->status_host != 0) {
        h->err = std::string(who) + ": device status " + std::to_string(h->status_host) + " (a bounded wait ran out)";
        cudaMemsetAsync(h->d_status, 0, 4, h->stream);
        return -2;
    }
    return 1;
}

int strix_cuda_decode_step(strix_cuda *h, const float *hvec, size_t pos, float *logits, size_t logits_cap) {
    if (!h || !hvec || !logits) return -1;  // (with the attention stand-in `pos` has no effect)
    h->err.clear();
    strix_decode_state *d = h->decode;
    if (!d) return 0;  // not configured: None, the model falls back to per-weight gemv
    const size_t n_out = d->head->rows;  // the whole vocabulary, or this accelerator's shard of it
    if (logits_cap < n_out) {
        h->err = "decode_step: logits buffer too small";
        return -1;
    }
    int rc = decode_enqueue_step(h, d, hvec, pos);
    if (rc < 0) return rc;
    // the final logit soft-cap (decode.rs:5516-5527); the greedy entry point skips it: cap * tanh(x / cap) is monotone
    if (d->cfg.final_softcap > 0.f) CU_TRY(h, launch_softcap(d->logits, n_out, d->cfg.final_softcap, h->stream));
    CU_TRY(h, cudaMemcpyAsync(d->pin_logits, d->logits, n_out * sizeof(float), cudaMemcpyDeviceToHost, h->stream));
    if ((rc = decode_finish(h, "decode_step")) < 0) return rc;
    memcpy(logits, d->pin_logits, n_out * sizeof(float));
    return 1;
}

// Greedy decode of one token: the chain, then the argmax on the device; 4 bytes come back instead of
// the vocabulary-wide logits (decode.rs:5497-5515, 5533-5538). Ties resolve to the lowest index.
// A row-sharded accelerator (world > 1) holds only its own logits and declines (0): the caller folds
// the shards' winners itself.
int strix_cuda_decode_step_argmax(strix_cuda *h, const float *hvec, size_t pos, uint32_t *id) {
    if (!h || !hvec || !id) return -1;
    h->err.clear();
    strix_decode_state *d = h->decode;
    if (!d || h->world > 1) return 0;
    int rc = decode_enqueue_step(h, d, hvec, pos);
    if (rc < 0) return rc;
    if (argmax_rows_enqueue(h, d->logits, d->cfg.vocab, d->cfg.vocab, 1, h->stream) < 0) return -1;
    CU_TRY(h, cudaMemcpyAsync(h->am_pin, h->am_idx, 4, cudaMemcpyDeviceToHost, h->stream));
    if ((rc = decode_finish(h, "decode_step_argmax")) < 0) return rc;
    *id = h->am_pin[0];
    return 1;
}

}  // extern "C"
