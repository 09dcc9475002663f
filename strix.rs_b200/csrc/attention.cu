// Single-token attention of the resident decode step: per-head QK RMSNorm, RoPE, KV append, single-query
// softmax(q k^T * scale) v with grouped-query heads, in the flavours the reference's models ask for.
//
// Replaces the reference's qkv_post + sdpa kernels (crates/strix-backend-rocm/src/kernels.rs:1935-1998,
// 2114-2200; call sites decode.rs:5262-5388) and agrees with the CPU forwards they must match:
//   dense Qwen3   crates/strix-backend-cpu/src/qwen3.rs:117-138, 823-873   QK-norm, pairs (k, k + half), angle chain
//   SmolLM3       crates/strix-backend-cpu/src/smollm3.rs:126-138, 557-648 no QK-norm, pairs (2k, 2k + 1), layers without rope
//   Gemma         crates/strix-backend-cpu/src/gemma.rs:779-872            QK-norm, V = raw K on some layers, V RMS-normed
//                 (ops.rs:159-176 rope_in_place_ff)                         without weight, angle = pos * base^(-2j/hd) / ff[j],
//                                                                          sliding window on local layers, scale 1 or 1/sqrt(hd)
// and the f16 KV cache of the reference's GPU path (kernels.rs:18-35 f2h / h2f / KVLD; decode.rs:513-516).
//
// Everything a CUDA graph replays unchanged: the position is read from a device word, and the
// softmax runs as a fixed grid of (head, split) blocks (flash-decoding: every split of 64 cached
// tokens keeps its own maximum, sum and weighted value sum; a second kernel folds them). Splits
// outside [window start, current length) write an empty partial and leave.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"

namespace strix {

constexpr uint32_t ATT_SPLIT = ATT_SPLIT_TOKENS;  // cached tokens per softmax split
constexpr uint32_t ATT_THREADS = 256;

// f32 -> f16 bits the way the reference's cache stores round (kernels.rs:18-32): to nearest, a tie away from
// zero; beyond the f16 range (and NaN) -> infinity; below half of the smallest subnormal -> zero. On the magnitude
// bits `a`: a normal result is (a + half of the dropped 13 bits) >> 13 with the exponent re-biased (a carry walks
// into the exponent by itself); a subnormal one shifts the mantissa with its hidden bit by 126 - exponent field.
__host__ __device__ inline unsigned short f2h_ref_bits(uint32_t x) {
    const uint32_t sign = (x >> 16) & 0x8000u, a = x & 0x7fffffffu;
    uint32_t h;
    if (a >= 0x47800000u) h = 0x7c00u;
    else if (a >= 0x38800000u) h = ((a + 0x1000u) >> 13) - (112u << 10);
    else if (a < 0x33000000u) h = 0u;
    else h = ((((a & 0x7fffffu) | 0x800000u) >> (125u - (a >> 23))) + 1u) >> 1;
    return (unsigned short)(sign | h);
}
__device__ __forceinline__ unsigned short f2h_ref(float f) { return f2h_ref_bits(__float_as_uint(f)); }
__device__ __forceinline__ void kv_store(float *p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void kv_store(__half *p, size_t i, float v) {
    reinterpret_cast<unsigned short *>(p)[i] = f2h_ref(v);
}
// four consecutive cache elements starting at element 4 * i4 of a row
__device__ __forceinline__ float4 kv_load4(const float *row, uint32_t i4) { return reinterpret_cast<const float4 *>(row)[i4]; }
__device__ __forceinline__ float4 kv_load4(const __half *row, uint32_t i4) {
    const uint2 u = reinterpret_cast<const uint2 *>(row)[i4];
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// grid = (n_heads + 2 n_kv, rows) blocks of 128 threads: blocks [0, n_heads) treat a q head in place,
// [n_heads, n_heads + n_kv) a k head (normed, rotated, then stored into the cache row of `pos`),
// the rest put a v head into the cache (from A.v, which is the RAW k vector on a layer that shares K and V:
// gemma.rs:796-803 takes V before the K-norm). hd <= 512, even.
template <typename T>
__global__ void __launch_bounds__(128) qk_post_kernel(const AttnArgs A) {
    __shared__ float xs[ATT_MAX_HD], th[ATT_MAX_HD / 2], red[4];
    const uint32_t n_heads = A.n_heads, n_kv = A.n_kv, hd = A.hd;
    // blockIdx.y = activation row (token) of a batched call: its own q / k / v vectors and position
    float *q = A.q + (size_t)blockIdx.y * n_heads * hd;
    const float *k = A.k + (size_t)blockIdx.y * n_kv * hd;
    const float *v = A.v + (size_t)blockIdx.y * n_kv * hd;
    T *kc = static_cast<T *>(A.kc), *vc = static_cast<T *>(A.vc);
    const uint32_t b = blockIdx.x, t = threadIdx.x, pos = A.pos[blockIdx.y], half = hd / 2;
    if (pos >= A.max_seq) {  // the cache is full: report, touch nothing
        if (t == 0 && b == 0 && A.status) atomicOr(A.status, STATUS_BAD_ARGS);
        return;
    }
    const uint32_t kvdim = n_kv * hd;
    if (b >= n_heads + n_kv) {  // v head: into the cache, RMS-normed without a weight where the model asks (gemma.rs:804-813)
        const uint32_t hh = b - n_heads - n_kv;
        float scale = 1.f;
        if (A.norm_v) {
            float ss = 0.f;
            for (uint32_t i = t; i < hd; i += 128) {
                const float x = v[hh * hd + i];
                ss += x * x;
            }
            ss = warp_sum(ss);
            if ((t & 31u) == 0) red[t >> 5] = ss;
            __syncthreads();
            scale = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)hd + A.eps);
        }
        for (uint32_t i = t; i < hd; i += 128) kv_store(vc, (size_t)pos * kvdim + hh * hd + i, v[hh * hd + i] * scale);
        return;
    }
    const bool is_q = b < n_heads;
    const uint32_t hh = is_q ? b : b - n_heads;
    const float *src = is_q ? q + hh * hd : k + hh * hd;
    const float *w = is_q ? A.q_norm : A.k_norm;
    float ss = 0.f;
    for (uint32_t i = t; i < hd; i += 128) {
        const float x = src[i];
        xs[i] = x;
        ss += x * x;
    }
    ss = warp_sum(ss);
    if ((t & 31u) == 0) red[t >> 5] = ss;
    if (A.rope == ATT_ROPE_CHAIN) {
        // qwen3.rs:126-138 / smollm3.rs:126-138: theta starts at pos and is multiplied by theta_scale once per
        // pair, in f32, one after the other; the same chain of roundings is replayed here by one thread
        if (t == 127) {
            float theta = (float)pos;
            for (uint32_t kk = 0; kk < half; kk++) {
                th[kk] = theta;
                theta = __fmul_rn(theta, A.theta_scale);
            }
        }
    } else if (A.rope == ATT_ROPE_POW) {
        // ops.rs:159-176: inv_freq = theta^(-(2 j) / hd), divided by the frequency factor where the layer has
        // them, angle = pos * inv_freq, all in f32 (the power itself through double, then rounded once)
        for (uint32_t kk = t; kk < half; kk += 128) {
            const float ex = -(2.0f * (float)kk) / (float)hd;
            float inv = (float)pow((double)A.theta, (double)ex);
            if (A.freq) inv = inv / A.freq[kk];
            th[kk] = (float)pos * inv;
        }
    }
    __syncthreads();
    const float tot = (red[0] + red[1]) + (red[2] + red[3]);
    const float scale = w ? 1.0f / sqrtf(tot / (float)hd + A.eps) : 1.0f;  // rmsnorm_inplace (qwen3.rs:117-124)
    for (uint32_t kk = t; kk < half; kk += 128) {
        // pairs (k, k + half), or the adjacent pairs (2k, 2k + 1) of a Llama-permuted model
        const uint32_t ia = A.rope_adjacent ? 2u * kk : kk, ib = A.rope_adjacent ? 2u * kk + 1u : kk + half;
        float x0 = xs[ia], x1 = xs[ib];
        if (w) {
            x0 = x0 * scale * w[ia];
            x1 = x1 * scale * w[ib];
        }
        float y0 = x0, y1 = x1;
        if (A.rope != ATT_ROPE_NONE) {
            float s, c;
            sincosf(th[kk], &s, &c);
            y0 = x0 * c - x1 * s;
            y1 = x0 * s + x1 * c;
        }
        if (is_q) {
            q[hh * hd + ia] = y0;
            q[hh * hd + ib] = y1;
        } else {
            kv_store(kc, (size_t)pos * kvdim + hh * hd + ia, y0);
            kv_store(kc, (size_t)pos * kvdim + hh * hd + ib, y1);
        }
    }
}

// grid = (n_heads, max_splits, rows), 256 threads. part: [rows][n_heads][max_splits][hd + 2] = {max, sum, out[hd]}.
// A split is short (64 cached tokens) so that a long context spreads over many SMs: the work per
// token is a few hundred bytes and its latency, not its bandwidth, is what a block waits for.
// A.window > 0: only the last `window` cached tokens are attended to (decode.rs:5312-5325).
template <typename T>
__global__ void __launch_bounds__(ATT_THREADS) sdpa_split_kernel(const AttnArgs A) {
    __shared__ float sc[ATT_SPLIT], red[ATT_THREADS / 32];
    __shared__ __align__(16) float vsum[4 * ATT_THREADS];
    const uint32_t n_heads = A.n_heads, n_kv = A.n_kv, hd = A.hd;
    const uint32_t hh = blockIdx.x, sp = blockIdx.y, row = blockIdx.z, t = threadIdx.x, lane = t & 31u, warp = t >> 5;
    const uint32_t len = min(A.pos[row] + 1u, A.max_seq);
    const uint32_t first = (A.window && len > A.window) ? len - A.window : 0u;
    const float *q = A.q + (size_t)row * n_heads * hd;
    const T *kc = static_cast<const T *>(A.kc), *vc = static_cast<const T *>(A.vc);
    float *my = A.part + (((size_t)row * n_heads + hh) * gridDim.y + sp) * (hd + 2u);
    const uint32_t t0 = max(sp * ATT_SPLIT, first), t1 = min(len, (sp + 1u) * ATT_SPLIT);
    if (t0 >= t1) {
        if (t == 0) {
            my[0] = -3.0e38f;
            my[1] = 0.f;
        }
        return;
    }
    const uint32_t n = t1 - t0, kvdim = n_kv * hd, kvh = hh / (n_heads / n_kv);
    const uint32_t nq = hd / 4u;  // 4-element columns of a head (hd % 4 == 0)
    // scores: a warp takes tokens warp, warp + 8, ...; a lane keeps its 4-element slices of q in registers
    // and reads the same slices of each key row; four tokens per pass
    constexpr uint32_t NW = ATT_THREADS / 32, NSL = ATT_MAX_HD / 128;
    const float4 *q4 = reinterpret_cast<const float4 *>(q + hh * hd);
    float4 qs[NSL];
#pragma unroll
    for (uint32_t u = 0; u < NSL; u++) qs[u] = lane + 32u * u < nq ? q4[lane + 32u * u] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t j0 = warp; j0 < n; j0 += 4u * NW) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (uint32_t u = 0; u < 4; u++) {
            const uint32_t j = j0 + u * NW;
            if (j < n) {
                const T *kr = kc + (size_t)(t0 + j) * kvdim + kvh * hd;
#pragma unroll
                for (uint32_t s = 0; s < NSL; s++) {
                    if (lane + 32u * s < nq) {
                        const float4 kv = kv_load4(kr, lane + 32u * s);
                        a[u] = fmaf(qs[s].x, kv.x, fmaf(qs[s].y, kv.y, fmaf(qs[s].z, kv.z, fmaf(qs[s].w, kv.w, a[u]))));
                    }
                }
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < 4; u++) {
            const float r = warp_sum(a[u]);
            if (lane == 0 && j0 + u * NW < n) sc[j0 + u * NW] = r * A.scale;
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
    // elements and group p takes tokens p, p + parts, ... (rows of the cache coalesced); the
    // groups' sums meet in shared memory, in group order
    const uint32_t parts = ATT_THREADS / nq;  // >= 2: hd <= 512
    const uint32_t p = t / nq, c4 = t - p * nq;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p < parts) {
        const T *vr = vc + (size_t)t0 * kvdim + kvh * hd;
        for (uint32_t j = p; j < n; j += parts) {
            const float4 v = kv_load4(vr + (size_t)j * kvdim, c4);
            const float w = sc[j];
            o.x = fmaf(w, v.x, o.x);
            o.y = fmaf(w, v.y, o.y);
            o.z = fmaf(w, v.z, o.z);
            o.w = fmaf(w, v.w, o.w);
        }
        reinterpret_cast<float4 *>(vsum)[t] = o;  // as floats: vsum[p * hd + 4 c4 + e]
    }
    __syncthreads();
    for (uint32_t i = t; i < hd; i += ATT_THREADS) {
        float tot = vsum[i];
        for (uint32_t k2 = 1; k2 < parts; k2++) tot += vsum[k2 * hd + i];
        my[2u + i] = tot;
    }
}

// grid = (n_heads, rows), hd threads (rounded up to a warp): fold the splits' partials into attn[n_heads * hd].
// Splits before the window or past the length hold {-3e38, 0} and add nothing.
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
        if (ps[1] == 0.f) continue;  // an empty split
        const float f = expf(ps[0] - M);
        L = fmaf(f, ps[1], L);
        if (i < hd) o = fmaf(f, ps[2u + i], o);
    }
    if (i < hd) attn[hh * hd + i] = o * (1.0f / L);
}

// h[i] = (h[i] + x[i] * rs * w[i]) * out_scale, rs = 1 / sqrt(mean(x^2) + eps): the sandwich residual of the Gemma
// forward (gemma.rs:876-879, 896-906; the reference's addnorm kernel, kernels.rs:1899-1911). grid = rows, 256 threads.
__global__ void __launch_bounds__(256) addnorm_kernel(float *__restrict__ h, const float *__restrict__ x,
                                                      const float *__restrict__ w, uint32_t dim, float eps, float out_scale) {
    __shared__ float red[8];
    h += (size_t)blockIdx.x * dim;
    x += (size_t)blockIdx.x * dim;
    const uint32_t t = threadIdx.x;
    float ss = 0.f;
    for (uint32_t i = t; i < dim; i += 256) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    if ((t & 31u) == 0) red[t >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float rs = 1.0f / sqrtf(tot / (float)dim + eps);
    for (uint32_t i = t; i < dim; i += 256) h[i] = (h[i] + x[i] * rs * w[i]) * out_scale;
}

// x[i] = cap * tanh(x[i] / cap) (ops.rs:127-135 softcap_inplace; the reference's softcap kernel, kernels.rs:2081-2086).
__global__ void softcap_kernel(float *__restrict__ x, size_t n, float cap, float inv) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] * inv);
}

cudaError_t launch_attention_step(const AttnArgs &A, cudaStream_t stream) {
    const uint32_t max_splits = (A.max_seq + ATT_SPLIT - 1) / ATT_SPLIT;
    // all rows' keys and values enter the cache first; then every row attends to rows 0 .. its own position
    // (causal: a later row's key is in the cache but beyond an earlier row's length)
    const dim3 g1(A.n_heads + 2u * A.n_kv, A.rows), g2(A.n_heads, max_splits, A.rows);
    if (A.kv_f16) {
        qk_post_kernel<__half><<<g1, 128, 0, stream>>>(A);
        sdpa_split_kernel<__half><<<g2, ATT_THREADS, 0, stream>>>(A);
    } else {
        qk_post_kernel<float><<<g1, 128, 0, stream>>>(A);
        sdpa_split_kernel<float><<<g2, ATT_THREADS, 0, stream>>>(A);
    }
    sdpa_fold_kernel<<<dim3(A.n_heads, A.rows), ((A.hd + 31u) / 32u) * 32u, 0, stream>>>(A.part, A.attn, A.pos, A.hd, max_splits,
                                                                                     A.max_seq);
    return cudaGetLastError();
}

cudaError_t launch_addnorm(float *d_h, const float *d_x, const float *d_w, uint32_t dim, float eps, float out_scale,
                           uint32_t rows, cudaStream_t stream) {
    addnorm_kernel<<<rows, 256, 0, stream>>>(d_h, d_x, d_w, dim, eps, out_scale);
    return cudaGetLastError();
}

cudaError_t launch_softcap(float *d_x, size_t n, float cap, cudaStream_t stream) {
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(d_x, n, cap, 1.0f / cap);
    return cudaGetLastError();
}

// host f32 -> f16 words with the cache's rounding (seeding the cache from a prefill done elsewhere)
void f32_to_f16_ref(const float *src, unsigned short *dst, size_t n) {
    for (size_t i = 0; i < n; i++) {
        uint32_t x;
        memcpy(&x, src + i, 4);
        dst[i] = f2h_ref_bits(x);
    }
}

}  // namespace strix
