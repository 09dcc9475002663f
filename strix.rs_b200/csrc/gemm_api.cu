// C-ABI entry points of the W8A8 prefill GEMM (see gemm_w8a8.cu for the kernels).
#include <algorithm>
#include <cstring>
#include <string>

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

template <typename T>
static int ensure_raw(strix_cuda *h, T *&p, size_t &cap, size_t n) {
    if (cap >= n) return 1;
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
    CU_TRY(h, cudaMalloc(&p, std::max<size_t>(n, 256) * sizeof(T)));
    cap = std::max<size_t>(n, 256);
    return 1;
}

// Builds the weight's transposed f32 scale plane on first use.
static int ensure_scales(strix_cuda *h, Resident *r, cudaStream_t stream) {
    if (r->scalesT) return 1;
    const size_t n = (size_t)r->L.nb * gemm_scales_ld((uint32_t)r->rows);
    float *p = nullptr;
    CU_TRY(h, cudaMalloc(&p, std::max<size_t>(n, 4) * sizeof(float)));
    cudaError_t e = launch_scales_transpose(r->dev, p, r->L, (uint32_t)r->rows, stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        h->err = std::string("scales transpose: ") + cudaGetErrorString(e);
        return -1;
    }
    r->scalesT = p;
    return 1;
}

// A Q4_0 weight gets its byte-per-code copy for the GEMM on first use (Q8_0 weights have theirs from the upload).
static int ensure_codes(strix_cuda *h, Resident *r, cudaStream_t stream) {
    if (r->gemm_codes) return 1;
    if (r->fmt != FMT_Q4_0) {
        h->err = "prefill GEMM: this weight has no byte-per-code copy";
        return -1;
    }
    uint8_t *p = nullptr;
    CU_TRY(h, cudaMalloc(&p, std::max<size_t>(r->rows * (size_t)r->L.in_dim, 16)));
    const cudaError_t e = launch_expand_q4_codes(r->dev, p, r->L, (uint32_t)r->rows, stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        h->err = std::string("expand q4 codes: ") + cudaGetErrorString(e);
        return -1;
    }
    r->gemm_codes = p;
    return 1;
}

// Scratch of the activation quantiser for m token rows of a weight with nb K-blocks.
static int ensure_quant(strix_cuda *h, size_t m, size_t K, size_t nb) {
    const size_t n = nb * gemm_x_ld((uint32_t)m);
    if (ensure_raw(h, h->gm_xq, h->gm_xq_cap, m * K) < 0) return -1;
    if (ensure_raw(h, h->gm_xs, h->gm_xs_cap, n) < 0) return -1;
    if (ensure_f32(h, h->gm_xd, n) < 0 || ensure_f32(h, h->gm_xc, n) < 0) return -1;
    return 1;
}

// Quantise d_xs[m][in_dim] and run the GEMM into d_y[m][rows]; all scratch from the handle.
static int gemm_device(strix_cuda *h, Resident *r, const float *d_xs, size_t m, float *d_y, cudaStream_t stream) {
    const size_t K = r->L.in_dim, nb = r->L.nb;
    if (ensure_codes(h, r, stream) < 0 || ensure_scales(h, r, stream) < 0) return -1;
    if (ensure_quant(h, m, K, nb) < 0) return -1;
    const uint32_t splits = gemm_pick_splits((uint32_t)m, (uint32_t)r->rows, (uint32_t)nb, h->num_sms);
    const size_t wsf = gemm_workspace_floats((uint32_t)m, (uint32_t)r->rows, splits);
    if (wsf && ensure_f32(h, h->gm_part, wsf) < 0) return -1;
    ProfScope prof(h, stream, "gemm_w8a8");  // (quantiser, GEMM and split-K reduction together)
    CU_TRY(h, launch_xquant8_sum(d_xs, h->gm_xq, h->gm_xd.p, h->gm_xs, h->gm_xc.p, (uint32_t)m, (uint32_t)nb, stream));
    CU_TRY(h, launch_gemm_w8a8(r->gemm_codes, r->L, (uint32_t)r->rows, r->scalesT, h->gm_xq, h->gm_xd.p, h->gm_xs, h->gm_xc.p,
                              (uint32_t)m, d_y, h->gm_part.p, splits, 0, nullptr, h->d_status, stream));
    return 1;
}

extern "C" {

static int prefill_gemm_host(strix_cuda *h, int fmt, const char *key, const float *xs, size_t m, float *y, size_t y_cap) {
    if (!h || !key || !xs || !y) return -1;
    h->err.clear();
    Resident *r = find_weight_mut(h, key);
    // None for an unknown key or a weight of another format (decode.rs:3258 looks only in the q8 map)
    if (!r || r->fmt != fmt) return 0;
    if (m == 0) return 1;
    if (m > 0x7fffffffu / std::max<size_t>(r->L.in_dim, 1)) return 0;
    if (y_cap < m * r->rows) {
        h->err = "prefill_q8_gemm: output too small";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    const size_t K = r->L.in_dim;
    if (ensure_f32(h, h->gm_x, m * K) < 0 || ensure_f32(h, h->gm_y, std::max<size_t>(m * r->rows, 1)) < 0) return -1;
    CU_TRY(h, cudaMemcpyAsync(h->gm_x.p, xs, m * K * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    if (gemm_device(h, r, h->gm_x.p, m, h->gm_y.p, h->stream) < 0) return -1;
    if (r->rows) CU_TRY(h, cudaMemcpyAsync(y, h->gm_y.p, m * r->rows * sizeof(float), cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaMemcpyAsync(&h->status_host, h->d_status, 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaStreamSynchronize(h->stream));
    if (h->status_host != 0) {
        h->err = "prefill_q8_gemm: device status " + std::to_string(h->status_host) + " (a bounded wait ran out)";
        cudaMemsetAsync(h->d_status, 0, 4, h->stream);
        return -2;
    }
    return 1;
}

int strix_cuda_prefill_q8_gemm(strix_cuda *h, const char *key, const float *xs, size_t m, float *y, size_t y_cap) {
    return prefill_gemm_host(h, FMT_Q8_0, key, xs, m, y, y_cap);
}

int strix_cuda_prefill_q4_gemm(strix_cuda *h, const char *key, const float *xs, size_t m, float *y, size_t y_cap) {
    return prefill_gemm_host(h, FMT_Q4_0, key, xs, m, y, y_cap);
}

int strix_cuda_prefill_q4_gemm_dev(strix_cuda *h, const char *key, const float *d_xs, size_t m, float *d_y, void *stream) {
    if (!h || !key || !d_xs || !d_y) return -1;
    h->err.clear();
    Resident *r = find_weight_mut(h, key);
    if (!r || r->fmt != FMT_Q4_0) return 0;
    if (m == 0) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    return gemm_device(h, r, d_xs, m, d_y, static_cast<cudaStream_t>(stream));
}

int strix_cuda_prefill_q8_gemm_dev(strix_cuda *h, const char *key, const float *d_xs, size_t m, float *d_y, void *stream) {
    if (!h || !key || !d_xs || !d_y) return -1;
    h->err.clear();
    Resident *r = find_weight_mut(h, key);
    if (!r || r->fmt != FMT_Q8_0) return 0;
    if (m == 0) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    return gemm_device(h, r, d_xs, m, d_y, static_cast<cudaStream_t>(stream));
}

// mode 0: the GEMM's tensor-core kernel with the epilogue that stores its int32 block sums; mode 1: a plain
// integer loop (no tensor cores) over the same codes. `splits`: 0 = as the product path picks, else forced.
static int block_isums(strix_cuda *h, const char *key, const float *xs, size_t m, int32_t *out, size_t out_cap, bool tensor,
                       uint32_t splits) {
    if (!h || !key || !xs || !out) return -1;
    h->err.clear();
    Resident *r = find_weight_mut(h, key);
    if (!r || (r->fmt != FMT_Q8_0 && r->fmt != FMT_Q4_0)) return 0;
    const size_t K = r->L.in_dim, nb = r->L.nb, total = m * r->rows * nb;
    if (out_cap < total) {
        h->err = "debug isums: output too small";
        return -1;
    }
    if (total == 0) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    if (ensure_f32(h, h->gm_x, m * K) < 0 || ensure_quant(h, m, K, nb) < 0 || ensure_codes(h, r, h->stream) < 0) return -1;
    if (tensor && ensure_scales(h, r, h->stream) < 0) return -1;
    if (tensor && splits == 0) splits = gemm_pick_splits((uint32_t)m, (uint32_t)r->rows, (uint32_t)nb, h->num_sms);
    int32_t *d_out = nullptr;
    CU_TRY(h, cudaMalloc(&d_out, total * sizeof(int32_t)));
    cudaError_t e = cudaMemsetAsync(d_out, 0xff, total * sizeof(int32_t), h->stream);  // an entry nobody writes shows as -1
    if (e == cudaSuccess) e = cudaMemcpyAsync(h->gm_x.p, xs, m * K * sizeof(float), cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess)
        e = launch_xquant8_sum(h->gm_x.p, h->gm_xq, h->gm_xd.p, h->gm_xs, h->gm_xc.p, (uint32_t)m, (uint32_t)nb, h->stream);
    if (e == cudaSuccess) {
        if (tensor)
            e = launch_gemm_w8a8(r->gemm_codes, r->L, (uint32_t)r->rows, r->scalesT, h->gm_xq, h->gm_xd.p, h->gm_xs, h->gm_xc.p,
                                 (uint32_t)m, nullptr, nullptr, splits, 1, d_out, h->d_status, h->stream);
        else
            e = launch_block_isums(r->gemm_codes, h->gm_xq, d_out, r->L, (uint32_t)m, (uint32_t)r->rows, h->stream);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, d_out, total * sizeof(int32_t), cudaMemcpyDeviceToHost, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&h->status_host, h->d_status, 4, cudaMemcpyDeviceToHost, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    cudaFree(d_out);
    if (e != cudaSuccess) {
        h->err = std::string("debug isums: ") + cudaGetErrorString(e);
        return -1;
    }
    if (h->status_host != 0) {
        h->err = "debug isums: device status " + std::to_string(h->status_host) + " (a bounded wait ran out)";
        cudaMemsetAsync(h->d_status, 0, 4, h->stream);
        return -2;
    }
    return 1;
}

int strix_cuda_debug_block_isums(strix_cuda *h, const char *key, const float *xs, size_t m, int32_t *out, size_t out_cap) {
    return block_isums(h, key, xs, m, out, out_cap, false, 0);
}

int strix_cuda_debug_gemm_isums(strix_cuda *h, const char *key, const float *xs, size_t m, uint32_t splits, int32_t *out,
                                size_t out_cap) {
    return block_isums(h, key, xs, m, out, out_cap, true, splits);
}

// Measurement: quantises d_xs[m][in_dim] once, then launches the GEMM kernel `reps` times in `mode`
// (0 the product into d_y; 2 without the accumulator drain; 3 without drain and loads) on `stream`.
int strix_cuda_debug_gemm_mode_dev(strix_cuda *h, const char *key, const float *d_xs, size_t m, float *d_y, int mode,
                                   int reps, void *stream) {
    if (!h || !key || !d_xs || !d_y) return -1;
    h->err.clear();
    if (mode != 0 && (mode < 2 || mode > 5)) {
        h->err = "debug_gemm_mode_dev: mode 0, 2, 3, 4 or 5";
        return -1;
    }
    Resident *r = find_weight_mut(h, key);
    if (!r || r->fmt != FMT_Q8_0) return 0;
    if (m == 0 || reps <= 0) return 1;
    CU_TRY(h, cudaSetDevice(h->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t K = r->L.in_dim, nb = r->L.nb;
    if (ensure_scales(h, r, st) < 0 || ensure_quant(h, m, K, nb) < 0) return -1;
    const uint32_t splits = gemm_pick_splits((uint32_t)m, (uint32_t)r->rows, (uint32_t)nb, h->num_sms);
    const size_t wsf = gemm_workspace_floats((uint32_t)m, (uint32_t)r->rows, splits);
    if (wsf && ensure_f32(h, h->gm_part, wsf) < 0) return -1;
    ProfScope prof(h, st, "gemm_w8a8");
    CU_TRY(h, launch_xquant8_sum(d_xs, h->gm_xq, h->gm_xd.p, h->gm_xs, h->gm_xc.p, (uint32_t)m, (uint32_t)nb, st));
    for (int i = 0; i < reps; i++)
        CU_TRY(h, launch_gemm_w8a8(r->gemm_codes, r->L, (uint32_t)r->rows, r->scalesT, h->gm_xq, h->gm_xd.p, h->gm_xs,
                                  h->gm_xc.p, (uint32_t)m, d_y, h->gm_part.p, splits, mode, nullptr, h->d_status, st));
    return 1;
}

}  // extern "C"
