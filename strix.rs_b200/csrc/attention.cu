// Single-token attention of the resident decode step (dense Qwen3 flavour): per-head QK RMSNorm,
// NEOX RoPE, KV append, single-query softmax(q k^T / sqrt(hd)) v with grouped-query heads.
//
// Replaces the reference's qkv_post + sdpa kernels (crates/strix-backend-rocm/src/kernels.rs:1935-1998,
// 2114-2200; call sites decode.rs:5262-5388) and agrees with the CPU forward they must match
// (crates/strix-backend-cpu/src/qwen3.rs:117-138 rmsnorm_inplace / rope_neox, :823-873 the step).
//
// Everything a CUDA graph replays unchanged: the position is read from a device word, and the
// softmax runs as a fixed grid of (head, split) blocks (flash-decoding: every split of 64 cached
// tokens keeps its own maximum, sum and weighted value sum; a second kernel folds them). Splits
// past the current length write an empty partial and leave.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "kernels.h"

namespace strix {

constexpr uint32_t ATT_SPLIT = ATT_SPLIT_TOKENS;  // cached tokens per softmax split
constexpr uint32_t ATT_THREADS = 256;

// grid = n_heads + 2 n_kv blocks of 128 threads: blocks [0, n_heads) treat a q head in place,
// [n_heads, n_heads + n_kv) a k head (normed, rotated, then stored into the cache row of `pos`),
// the rest copy a v head into the cache. hd <= 256, even.
__global__ void __launch_bounds__(128) qk_post_kernel(float *__restrict__ q, const float *__restrict__ k,
                                                      const float *__restrict__ v, const float *__restrict__ q_norm,
                                                      const float *__restrict__ k_norm, float *__restrict__ kc,
                                                      float *__restrict__ vc, const uint32_t *__restrict__ d_pos,
                                                      uint32_t n_heads, uint32_t n_kv, uint32_t hd, float eps,
                                                      float theta_scale, uint32_t max_seq, uint32_t *status) {
    __shared__ float xs[256], th[128], red[4];
    // blockIdx.y = activation row (token) of a batched call: its own q / k / v vectors and position
    q += (size_t)blockIdx.y * n_heads * hd;
    k += (size_t)blockIdx.y * n_kv * hd;
    v += (size_t)blockIdx.y * n_kv * hd;
    const uint32_t b = blockIdx.x, t = threadIdx.x, pos = d_pos[blockIdx.y], half = hd / 2;
    if (pos >= max_seq) {  // the cache is full: report, touch nothing
        if (t == 0 && b == 0 && status) atomicOr(status, STATUS_BAD_ARGS);
        return;
    }
    const uint32_t kvdim = n_kv * hd;
    if (b >= n_heads + n_kv) {  // v head: straight into the cache
        const uint32_t hh = b - n_heads - n_kv;
        for (uint32_t i = t; i < hd; i += 128) vc[(size_t)pos * kvdim + hh * hd + i] = v[hh * hd + i];
        return;
    }
    const bool is_q = b < n_heads;
    const uint32_t hh = is_q ? b : b - n_heads;
    const float *src = is_q ? q + hh * hd : k + hh * hd;
    const float *w = is_q ? q_norm : k_norm;
    float ss = 0.f;
    for (uint32_t i = t; i < hd; i += 128) {
        const float x = src[i];
        xs[i] = x;
        ss += x * x;
    }
    ss = warp_sum(ss);
    if ((t & 31u) == 0) red[t >> 5] = ss;
    // rope_neox (qwen3.rs:126-138): theta starts at pos and is multiplied by theta_scale once per pair,
    // in f32, one after the other; the same chain of roundings is replayed here by one thread
    if (t == 127) {
        float theta = (float)pos;
        for (uint32_t kk = 0; kk < half; kk++) {
            th[kk] = theta;
            theta = __fmul_rn(theta, theta_scale);
        }
    }
    __syncthreads();
    const float tot = (red[0] + red[1]) + (red[2] + red[3]);
    const float scale = w ? 1.0f / sqrtf(tot / (float)hd + eps) : 1.0f;  // rmsnorm_inplace (qwen3.rs:117-124)
    for (uint32_t kk = t; kk < half; kk += 128) {
        float x0 = xs[kk], x1 = xs[kk + half];
        if (w) {
            x0 = x0 * scale * w[kk];
            x1 = x1 * scale * w[kk + half];
        }
        float s, c;
        sincosf(th[kk], &s, &c);
        const float y0 = x0 * c - x1 * s, y1 = x0 * s + x1 * c;
        if (is_q) {
            q[hh * hd + kk] = y0;
            q[hh * hd + kk + half] = y1;
        } else {
            kc[(size_t)pos * kvdim + hh * hd + kk] = y0;
            kc[(size_t)pos * kvdim + hh * hd + kk + half] = y1;
        }
    }
}

// grid = (n_heads, max_splits), 256 threads. part: [n_heads][max_splits][hd + 2] = {max, sum, out[hd]}.
// A split is short (64 cached tokens) so that a long context spreads over many SMs: the work per
// token is a few hundred bytes and its latency, not its bandwidth, is what a block waits for.
__global__ void __launch_bounds__(ATT_THREADS) sdpa_split_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                                                                 const float *__restrict__ vc, float *__restrict__ part,
                                                                 const uint32_t *__restrict__ d_pos, uint32_t n_heads,
                                                                 uint32_t n_kv, uint32_t hd, float scale, uint32_t max_seq) {
    __shared__ float sc[ATT_SPLIT], red[ATT_THREADS / 32];
    __shared__ __align__(16) float vsum[4 * ATT_THREADS];
    const uint32_t hh = blockIdx.x, sp = blockIdx.y, row = blockIdx.z, t = threadIdx.x, lane = t & 31u, warp = t >> 5;
    const uint32_t len = min(d_pos[row] + 1u, max_seq);
    q += (size_t)row * n_heads * hd;
    float *my = part + (((size_t)row * n_heads + hh) * gridDim.y + sp) * (hd + 2u);
    const uint32_t t0 = sp * ATT_SPLIT;
    if (t0 >= len) {
        if (t == 0) {
            my[0] = -3.0e38f;
            my[1] = 0.f;
        }
        return;
    }
    const uint32_t n = min(ATT_SPLIT, len - t0), kvdim = n_kv * hd, kvh = hh / (n_heads / n_kv);
    const uint32_t nq = hd / 4u;  // float4 columns of a head (hd % 4 == 0: rows of the cache are 16-byte aligned)
    // scores: a warp takes tokens warp, warp + 8, ...; a lane keeps its float4 slice(s) of q in registers
    // and reads the same slice of each key row with one 16-byte load; four tokens per pass
    constexpr uint32_t NW = ATT_THREADS / 32;
    const float4 *q4 = reinterpret_cast<const float4 *>(q + hh * hd);
    const float4 qa = lane < nq ? q4[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 qb = lane + 32u < nq ? q4[lane + 32u] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t j0 = warp; j0 < n; j0 += 4u * NW) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (uint32_t u = 0; u < 4; u++) {
            const uint32_t j = j0 + u * NW;
            if (j < n) {
                const float4 *kr = reinterpret_cast<const float4 *>(kc + (size_t)(t0 + j) * kvdim + kvh * hd);
                if (lane < nq) {
                    const float4 kv = kr[lane];
                    a[u] = fmaf(qa.x, kv.x, fmaf(qa.y, kv.y, fmaf(qa.z, kv.z, qa.w * kv.w)));
                }
                if (lane + 32u < nq) {
                    const float4 kv = kr[lane + 32u];
                    a[u] = fmaf(qb.x, kv.x, fmaf(qb.y, kv.y, fmaf(qb.z, kv.z, fmaf(qb.w, kv.w, a[u]))));
                }
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < 4; u++) {
            const float r = warp_sum(a[u]);
            if (lane == 0 && j0 + u * NW < n) sc[j0 + u * NW] = r * scale;
        }
    }
    __syncthreads();
    float m = -3.0e38f;
    for (uint32_t j = t; j < n; j += ATT_THREADS) m = fmaxf(m, sc[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
    for (uint32_t w2 = 1; w2 < NW; w2++) m = fmaxf(m, red[w2]);
    __syncthreads();
    float l = 0.f;
    for (uint32_t j = t; j < n; j += ATT_THREADS) {
        const float e = expf(sc[j] - m);
        sc[j] = e;
        l += e;
    }
    l = warp_sum(l);
    if (lane == 0) red[warp] = l;
    __syncthreads();
    if (t == 0) {
        float tot = 0.f;
        for (uint32_t w2 = 0; w2 < NW; w2++) tot += red[w2];
        my[0] = m;
        my[1] = tot;
    }
    // weighted value sum: the 256 threads form `parts` groups of hd / 4 lanes; a lane owns four output
    // elements and group p takes tokens p, p + parts, ... (16-byte loads, rows of the cache coalesced); the
    // groups' sums meet in shared memory, in group order
    const uint32_t parts = ATT_THREADS / nq;  // >= 4: hd <= 256
    const uint32_t p = t / nq, c4 = t - p * nq;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p < parts) {
        const float4 *vr = reinterpret_cast<const float4 *>(vc + (size_t)t0 * kvdim + kvh * hd) + c4;
        const uint32_t row4 = kvdim / 4u;
        for (uint32_t j = p; j < n; j += parts) {
            const float4 v = vr[(size_t)j * row4];
            const float w = sc[j];
            o.x = fmaf(w, v.x, o.x);
            o.y = fmaf(w, v.y, o.y);
            o.z = fmaf(w, v.z, o.z);
            o.w = fmaf(w, v.w, o.w);
        }
        reinterpret_cast<float4 *>(vsum)[t] = o;  // as floats: vsum[p * hd + 4 c4 + e]
    }
    __syncthreads();
    if (t < hd) {
        float tot = vsum[t];
        for (uint32_t k2 = 1; k2 < parts; k2++) tot += vsum[k2 * hd + t];
        my[2u + t] = tot;
    }
}

// grid = n_heads, hd threads: fold the splits' partials into attn[n_heads * hd].
__global__ void sdpa_fold_kernel(const float *__restrict__ part, float *__restrict__ attn, const uint32_t *__restrict__ d_pos,
                                 uint32_t hd, uint32_t max_splits, uint32_t max_seq) {
    const uint32_t hh = blockIdx.x, row = blockIdx.y, i = threadIdx.x;
    const uint32_t len = min(d_pos[row] + 1u, max_seq), ns = min(max_splits, (len + ATT_SPLIT - 1) / ATT_SPLIT);
    const float *p = part + ((size_t)row * gridDim.x + hh) * max_splits * (hd + 2u);
    attn += (size_t)row * gridDim.x * hd;
    float M = -3.0e38f;
    for (uint32_t s = 0; s < ns; s++) M = fmaxf(M, p[(size_t)s * (hd + 2u)]);
    float L = 0.f, o = 0.f;
    for (uint32_t s = 0; s < ns; s++) {
        const float *ps = p + (size_t)s * (hd + 2u);
        const float f = expf(ps[0] - M);
        L = fmaf(f, ps[1], L);
        if (i < hd) o = fmaf(f, ps[2u + i], o);
    }
    if (i < hd) attn[hh * hd + i] = o * (1.0f / L);
}

cudaError_t launch_attention_step(float *d_q, const float *d_k, const float *d_v, const float *d_q_norm,
                                  const float *d_k_norm, float *d_kc, float *d_vc, float *d_part, float *d_attn,
                                  const uint32_t *d_pos, uint32_t n_heads, uint32_t n_kv, uint32_t hd, float eps,
                                  float theta_scale, float scale, uint32_t max_seq, uint32_t rows, uint32_t *d_status,
                                  cudaStream_t stream) {
    const uint32_t max_splits = (max_seq + ATT_SPLIT - 1) / ATT_SPLIT;
    // all rows' keys and values enter the cache first; then every row attends to rows 0 .. its own position
    // (causal: a later row's key is in the cache but beyond an earlier row's length)
    qk_post_kernel<<<dim3(n_heads + 2u * n_kv, rows), 128, 0, stream>>>(d_q, d_k, d_v, d_q_norm, d_k_norm, d_kc, d_vc, d_pos, n_heads,
                                                             n_kv, hd, eps, theta_scale, max_seq, d_status);
    sdpa_split_kernel<<<dim3(n_heads, max_splits, rows), ATT_THREADS, 0, stream>>>(d_q, d_kc, d_vc, d_part, d_pos, n_heads, n_kv,
                                                                             hd, scale, max_seq);
    sdpa_fold_kernel<<<dim3(n_heads, rows), ((hd + 31u) / 32u) * 32u, 0, stream>>>(d_part, d_attn, d_pos, hd, max_splits, max_seq);
    return cudaGetLastError();
}

}  // namespace strix
