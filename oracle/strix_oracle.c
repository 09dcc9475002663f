/*
 * CPU oracle for the quantized-matmul hot path of strix.rs.
 *
 * TEST INFRASTRUCTURE ONLY. This file is a plain-C restatement of the
 * reference's CPU arithmetic (and, where the reference has no CPU code, of its
 * device kernels' arithmetic). It exists so that the CUDA backend can be
 * checked against it and so that a CPU baseline can be timed beside the GPU
 * numbers. Nothing in the shipped backend links, loads or calls it.
 *
 * Every function names the reference lines it restates (paths are relative to
 * the reference project root).
 *
 * Parity status:
 *   - block dequantisation (Q4_0 / Q4_1 / Q8_0 / Q6_K): PINNED by the
 *     reference's own known-answer tests
 *     (crates/strix-models/src/ggml_quant.rs:443-469, 497-514, 562-565), which
 *     tests/test_oracle_golden.py replays against this file.
 *   - dot_f32 / qmatmul accumulation order: follows the source text
 *     (crates/strix-backend-cpu/src/qwen3.rs:90-105, 173-182); the reference
 *     holds no test for it -- parity unpinned.
 *   - activation quantiser, integer-dot GEMV, W8A8 GEMM: the reference has no
 *     CPU implementation and no test; restated from the device kernels
 *     (crates/strix-backend-rocm/src/kernels.rs:864-876, 894-912, 259-287,
 *     1373-1443) -- parity unpinned.
 *
 * Third-party arithmetic restated here: `half` 2.7.1 (Cargo.lock:623-624),
 * f16::to_f32 -- exact IEEE binary16 -> binary32 widening, subnormals included.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (Rust does not contract
 * a*b+c into an FMA, so neither may this file).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SO_Q4_0 2
#define SO_Q4_1 3
#define SO_Q8_0 8
#define SO_Q6_K 14

/* ggml type ids as in crates/strix-models/src/ggml_quant.rs:568-574. */

/* half::f16::to_f32 (half 2.7.1), called at ggml_quant.rs:186-188. Exact. */
float so_f16_to_f32(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) & 1u, e = (uint32_t)(h >> 10) & 0x1fu, m = h & 0x3ffu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) {
            u = s << 31;
        } else {
            /* subnormal: m * 2^-24, normalise */
            int sh = 0;
            while (!(m & 0x400u)) { m <<= 1; sh++; }
            m &= 0x3ffu;
            u = (s << 31) | ((uint32_t)(113 - sh) << 23) | (m << 13);
        }
    } else if (e == 31) {
        u = (s << 31) | 0x7f800000u | (m << 13);
    } else {
        u = (s << 31) | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* block geometry: ggml_quant.rs:88-124 */
int so_block_elems(int ty) {
    switch (ty) {
        case SO_Q4_0: case SO_Q4_1: case SO_Q8_0: return 32;
        case SO_Q6_K: return 256;
        default: return 0;
    }
}
int so_block_bytes(int ty) {
    switch (ty) {
        case SO_Q4_0: return 18;
        case SO_Q4_1: return 20;
        case SO_Q8_0: return 34;
        case SO_Q6_K: return 210;
        default: return 0;
    }
}

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ggml_quant.rs:240-247 */
static void dequant_q8_0(const uint8_t *b, float *out, size_t nblk) {
    for (size_t i = 0; i < nblk; i++, b += 34, out += 32) {
        float d = so_f16_to_f32(rd16(b));
        for (int j = 0; j < 32; j++) out[j] = d * (float)(int8_t)b[2 + j];
    }
}
/* ggml_quant.rs:251-262 */
static void dequant_q4_0(const uint8_t *b, float *out, size_t nblk) {
    for (size_t i = 0; i < nblk; i++, b += 18, out += 32) {
        float d = so_f16_to_f32(rd16(b));
        const uint8_t *qs = b + 2;
        for (int j = 0; j < 16; j++) {
            int lo = (int)(qs[j] & 0x0F) - 8;
            int hi = (int)(qs[j] >> 4) - 8;
            out[j] = d * (float)lo;
            out[j + 16] = d * (float)hi;
        }
    }
}
/* ggml_quant.rs:264-275 (multiply, then add; no fusion) */
static void dequant_q4_1(const uint8_t *b, float *out, size_t nblk) {
    for (size_t i = 0; i < nblk; i++, b += 20, out += 32) {
        float d = so_f16_to_f32(rd16(b));
        float m = so_f16_to_f32(rd16(b + 2));
        const uint8_t *qs = b + 4;
        for (int j = 0; j < 16; j++) {
            float p0 = d * (float)(qs[j] & 0x0F);
            float p1 = d * (float)(qs[j] >> 4);
            out[j] = p0 + m;
            out[j + 16] = p1 + m;
        }
    }
}
/* ggml_quant.rs:404-430. `d * sc as f32 * q as f32` is (d*sc)*q: two roundings. */
static void dequant_q6_k(const uint8_t *b, float *out, size_t nblk) {
    for (size_t i = 0; i < nblk; i++, b += 210, out += 256) {
        const uint8_t *ql0 = b, *qh0 = b + 128;
        const int8_t *sc0 = (const int8_t *)(b + 192);
        float d = so_f16_to_f32(rd16(b + 208));
        for (int half = 0; half < 2; half++) {
            const uint8_t *ql = ql0 + half * 64, *qh = qh0 + half * 32;
            const int8_t *sc = sc0 + half * 8;
            float *y = out + half * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q1 = (int)((ql[l] & 0x0F) | ((qh[l] & 3) << 4)) - 32;
                int q2 = (int)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                float s1 = d * (float)sc[is], s2 = d * (float)sc[is + 2];
                float s3 = d * (float)sc[is + 4], s4 = d * (float)sc[is + 6];
                y[l] = s1 * (float)q1;
                y[l + 32] = s2 * (float)q2;
                y[l + 64] = s3 * (float)q3;
                y[l + 96] = s4 * (float)q4;
            }
        }
    }
}

/*
 * dequantize_into, ggml_quant.rs:139-183. Returns 0 on success,
 * -1 if n is not a multiple of the block size, -2 if too few bytes (extra
 * bytes are ignored, as in the reference), -3 for an unsupported type.
 */
int so_dequantize_into(int ty, const uint8_t *bytes, size_t nbytes, float *out, size_t n) {
    int be = so_block_elems(ty);
    if (be == 0) return -3;
    if (n % (size_t)be != 0) return -1;
    size_t nblk = n / (size_t)be;
    if (nbytes < nblk * (size_t)so_block_bytes(ty)) return -2;
    switch (ty) {
        case SO_Q8_0: dequant_q8_0(bytes, out, nblk); break;
        case SO_Q4_0: dequant_q4_0(bytes, out, nblk); break;
        case SO_Q4_1: dequant_q4_1(bytes, out, nblk); break;
        case SO_Q6_K: dequant_q6_k(bytes, out, nblk); break;
        default: return -3;
    }
    return 0;
}

/* dot_f32, crates/strix-backend-cpu/src/qwen3.rs:90-105 */
float so_dot_f32(const float *a, const float *b, size_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t chunks = n / 8;
    for (size_t c = 0; c < chunks; c++) {
        size_t i = c * 8;
        for (int k = 0; k < 8; k++) {
            float p = a[i + k] * b[i + k];
            acc[k] = acc[k] + p;
        }
    }
    float s = (acc[0] + acc[1]) + (acc[2] + acc[3]) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    for (size_t i = chunks * 8; i < n; i++) {
        float p = a[i] * b[i];
        s = s + p;
    }
    return s;
}

/* ---- row-parallel driver: the stand-in for rayon's par_iter_mut over rows ---- */
typedef void (*row_fn)(size_t row, void *ctx, float *scratch);
typedef struct {
    size_t r0, r1, scratch_len;
    row_fn fn;
    void *ctx;
} span_t;

static void *span_main(void *p) {
    span_t *s = (span_t *)p;
    float *scratch = s->scratch_len ? (float *)malloc(s->scratch_len * sizeof(float)) : NULL;
    for (size_t r = s->r0; r < s->r1; r++) s->fn(r, s->ctx, scratch);
    free(scratch);
    return NULL;
}

static void par_rows(size_t rows, int nthreads, size_t scratch_len, row_fn fn, void *ctx) {
    if (nthreads < 1) nthreads = 1;
    if ((size_t)nthreads > rows) nthreads = rows ? (int)rows : 1;
    span_t *sp = (span_t *)calloc((size_t)nthreads, sizeof(span_t));
    pthread_t *th = (pthread_t *)calloc((size_t)nthreads, sizeof(pthread_t));
    size_t per = rows / (size_t)nthreads, rem = rows % (size_t)nthreads, at = 0;
    for (int t = 0; t < nthreads; t++) {
        size_t cnt = per + ((size_t)t < rem ? 1 : 0);
        sp[t].r0 = at; sp[t].r1 = at + cnt; sp[t].scratch_len = scratch_len;
        sp[t].fn = fn; sp[t].ctx = ctx;
        at += cnt;
    }
    for (int t = 1; t < nthreads; t++) pthread_create(&th[t], NULL, span_main, &sp[t]);
    span_main(&sp[0]);
    for (int t = 1; t < nthreads; t++) pthread_join(th[t], NULL);
    free(sp); free(th);
}

/* ---- qmatmul / qmatmul_batch ---- */
typedef struct {
    float *out; const float *xs; const uint8_t *bytes;
    int ty; size_t in_dim, out_dim, m, bpr;
} mm_ctx;

static void qmatmul_row(size_t o, void *c, float *scratch) {
    mm_ctx *k = (mm_ctx *)c;
    so_dequantize_into(k->ty, k->bytes + o * k->bpr, k->bpr, scratch, k->in_dim);
    for (size_t t = 0; t < k->m; t++)
        k->out[t * k->out_dim + o] = so_dot_f32(scratch, k->xs + t * k->in_dim, k->in_dim);
}

/*
 * qmatmul, qwen3.rs:173-182: per output row dequantise the whole row into an
 * f32 scratch, then dot_f32 with x. Returns 0, or <0 on a shape error.
 */
int so_qmatmul(float *out, const float *x, const uint8_t *bytes, int ty, size_t in_dim,
               size_t out_dim, int nthreads) {
    int be = so_block_elems(ty);
    if (be == 0 || in_dim % (size_t)be != 0) return -1;
    mm_ctx c = {out, x, bytes, ty, in_dim, out_dim, 1, (in_dim / (size_t)be) * (size_t)so_block_bytes(ty)};
    par_rows(out_dim, nthreads, in_dim, qmatmul_row, &c);
    return 0;
}

/*
 * qmatmul_batch, crates/strix-backend-cpu/src/mellum.rs:244-271 (same as
 * qwen3.rs:432-449): each row dequantised once, dotted with every token.
 * xs is [m][in_dim], out is [m][out_dim] (token-major).
 */
int so_qmatmul_batch(float *out, const float *xs, size_t m, const uint8_t *bytes, int ty,
                     size_t in_dim, size_t out_dim, int nthreads) {
    int be = so_block_elems(ty);
    if (be == 0 || in_dim % (size_t)be != 0) return -1;
    mm_ctx c = {out, xs, bytes, ty, in_dim, out_dim, m, (in_dim / (size_t)be) * (size_t)so_block_bytes(ty)};
    par_rows(out_dim, nthreads, in_dim, qmatmul_row, &c);
    return 0;
}

/* rmsnorm, qwen3.rs:107-114: sequential f32 sum of squares, 1/sqrt, x*scale*w */
void so_rmsnorm(float *out, const float *x, const float *w, size_t n, float eps) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) {
        float p = x[i] * x[i];
        ss = ss + p;
    }
    float scale = 1.0f / sqrtf(ss / (float)n + eps);
    for (size_t i = 0; i < n; i++) {
        float t = x[i] * scale;
        out[i] = t * w[i];
    }
}

/* SwiGLU combine, qwen3.rs:881-884: gate[i] = (g / (1 + exp(-g))) * up[i] */
void so_swiglu(float *gate, const float *up, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float g = gate[i];
        float s = g / (1.0f + expf(-g));
        gate[i] = s * up[i];
    }
}

/* gelu_tanh + geglu, crates/strix-backend-cpu/src/ops.rs:110-122 */
void so_geglu(float *out, const float *gate, const float *up, size_t n) {
    const float C = 0.7978846f;
    for (size_t i = 0; i < n; i++) {
        float x = gate[i];
        float x3 = 0.044715f * x * x * x;
        float t = tanhf(C * (x + x3));
        float g = 0.5f * x * (1.0f + t);
        out[i] = g * up[i];
    }
}

/*
 * Activation quantiser, hot-path form (device kernel xquant8,
 * crates/strix-backend-rocm/src/kernels.rs:864-876; rows form :1000-1013):
 * per 32 elements d = amax/127, inv = d>0 ? 1/d : 0,
 * q = clamp(rintf(x*inv), -127, 127); d kept as f32. rintf rounds ties to even.
 * n must be a multiple of 32. Returns the number of elements whose scaled value
 * lay exactly on a .5 tie (so that the rounding rule's effect is visible).
 */
size_t so_xquant8(const float *x, size_t n, int8_t *q, float *d) {
    size_t ties = 0;
    for (size_t b = 0; b < n / 32; b++) {
        const float *xb = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(xb[i]));
        float sc = amax / 127.0f;
        float inv = sc > 0.0f ? 1.0f / sc : 0.0f;
        for (int i = 0; i < 32; i++) {
            float v = xb[i] * inv;
            if (fabsf(v - truncf(v)) == 0.5f) ties++;
            int qi = (int)rintf(v);
            if (qi > 127) qi = 127;
            if (qi < -127) qi = -127;
            q[b * 32 + i] = (int8_t)qi;
        }
        d[b] = sc;
    }
    return ties;
}

/* ---- integer-dot GEMV ---- */
typedef struct {
    float *y; const uint8_t *bytes; const int8_t *xq; const float *xd;
    int ty; size_t in_dim, out_dim, m, bpr; int32_t *isums;
} id_ctx;

/* int32 block sum of a Q8_0 weight block with an int8 activation block:
 * the inner term of q8i_gemv (kernels.rs:894-912) and q8w_gemm32 (:1373-1443) */
static inline int32_t isum_q8(const uint8_t *blk, const int8_t *xq) {
    int32_t s = 0;
    for (int i = 0; i < 32; i++) s += (int32_t)(int8_t)blk[2 + i] * (int32_t)xq[i];
    return s;
}
/* q4_gemv_dp (kernels.rs:259-287): raw nibbles dotted with xq, minus 8*sum(xq).
 * Equal, in int32, to sum((nib-8)*xq). Element order follows the Q4_0 block:
 * byte j low nibble = element j, high nibble = element j+16. */
static inline int32_t isum_q4(const uint8_t *blk, const int8_t *xq) {
    int32_t s = 0, xs = 0;
    for (int j = 0; j < 16; j++) {
        s += (int32_t)(blk[2 + j] & 0x0F) * (int32_t)xq[j];
        s += (int32_t)(blk[2 + j] >> 4) * (int32_t)xq[j + 16];
    }
    for (int i = 0; i < 32; i++) xs += xq[i];
    return s - 8 * xs;
}

static void idot_row(size_t o, void *c, float *scratch) {
    (void)scratch;
    id_ctx *k = (id_ctx *)c;
    const uint8_t *row = k->bytes + o * k->bpr;
    for (size_t t = 0; t < k->m; t++) {
        const int8_t *xq = k->xq + t * k->in_dim;
        float acc = 0.0f;
        if (k->ty == SO_Q8_0 || k->ty == SO_Q4_0) {
            size_t nb = k->in_dim / 32;
            const float *xd = k->xd + t * nb;
            size_t bb = (k->ty == SO_Q8_0) ? 34 : 18;
            for (size_t b = 0; b < nb; b++) {
                const uint8_t *blk = row + b * bb;
                int32_t s = (k->ty == SO_Q8_0) ? isum_q8(blk, xq + b * 32) : isum_q4(blk, xq + b * 32);
                if (k->isums) k->isums[(t * k->out_dim + o) * nb + b] = s;
                float dw = so_f16_to_f32(rd16(blk));
                float sc = dw * xd[b];          /* ws*xd, then *(float)s: left to right */
                float term = sc * (float)s;
                acc = acc + term;
            }
        } else if (k->ty == SO_Q4_1) {
            /* q4_1_gemv_dp (kernels.rs:289-320): value = d * code + m, codes 0..15 not centred; per block
             * acc += xd[b] * (dw * (float)isum + mw * (float)xsum[b]) */
            size_t nb = k->in_dim / 32;
            const float *xd = k->xd + t * nb;
            for (size_t b = 0; b < nb; b++) {
                const uint8_t *blk = row + b * 20;
                const int8_t *a = xq + b * 32;
                int32_t s = 0, xs = 0;
                for (int j = 0; j < 16; j++) {
                    s += (int32_t)(blk[4 + j] & 0x0F) * (int32_t)a[j];
                    s += (int32_t)(blk[4 + j] >> 4) * (int32_t)a[j + 16];
                }
                for (int i = 0; i < 32; i++) xs += a[i];
                if (k->isums) k->isums[(t * k->out_dim + o) * nb + b] = s;
                float dw = so_f16_to_f32(rd16(blk)), mw = so_f16_to_f32(rd16(blk + 2));
                float inner = dw * (float)s;
                float mterm = mw * (float)xs;
                inner = inner + mterm;
                float term = xd[b] * inner;
                acc = acc + term;
            }
        } else { /* SO_Q6_K: no reference kernel; per 16-element sub-scale group */
            size_t nsb = k->in_dim / 256;
            const float *xd = k->xd + t * (k->in_dim / 32);
            for (size_t sb = 0; sb < nsb; sb++) {
                const uint8_t *blk = row + sb * 210;
                const uint8_t *ql0 = blk, *qh0 = blk + 128;
                const int8_t *sc0 = (const int8_t *)(blk + 192);
                float d = so_f16_to_f32(rd16(blk + 208));
                for (int g = 0; g < 16; g++) { /* group g covers elements 16g .. 16g+15 */
                    int half = g / 8, gg = g % 8;      /* gg: 16-element group within the half */
                    int quarter = gg / 2, l0 = (gg % 2) * 16;
                    const uint8_t *ql = ql0 + half * 64, *qh = qh0 + half * 32;
                    int32_t s = 0;
                    for (int l = l0; l < l0 + 16; l++) {
                        int q;
                        switch (quarter) {
                            case 0: q = (ql[l] & 0x0F) | ((qh[l] & 3) << 4); break;
                            case 1: q = (ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4); break;
                            case 2: q = (ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4); break;
                            default: q = (ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4); break;
                        }
                        s += (int32_t)(q - 32) * (int32_t)xq[sb * 256 + half * 128 + quarter * 32 + l];
                    }
                    /* sub-scale index: is + 2*quarter with is = l/16, within the half */
                    float dsc = d * (float)sc0[half * 8 + (l0 / 16) + 2 * quarter];
                    float w = dsc * xd[sb * 8 + half * 4 + quarter];
                    float term = w * (float)s;
                    acc = acc + term;
                }
            }
        }
        k->y[t * k->out_dim + o] = acc;
    }
}

/*
 * Integer-dot GEMV / W8A8 GEMM over m quantised activation rows:
 *   y[t][o] = sum_kb (d_w[o,kb] * d_x[t,kb]) * (float)isum[t,o,kb], summed in
 * f32 in block order. Q8_0 restates q8i_gemv (kernels.rs:894-912) and
 * q8w_gemm32 (:1417-1428); Q4_0 restates q4_gemv_dp (:259-287), Q4_1 q4_1_gemv_dp (:289-320). Q6_K has no
 * integer-dot kernel in the reference: it is defined here per 16-element
 * sub-scale group with weight (d*sc)*d_x. The contract fixes the int32 block
 * sums exactly and y within rel-L2 1e-3; the reference's own lane/shuffle
 * summation order is not reproduced.
 * If isums != NULL (Q8_0/Q4_0 only) it receives [m][out_dim][in_dim/32] int32.
 */
int so_idot_gemm(float *y, const uint8_t *bytes, int ty, const int8_t *xq, const float *xd,
                 size_t m, size_t in_dim, size_t out_dim, int32_t *isums, int nthreads) {
    int be = so_block_elems(ty);
    if (be == 0 || in_dim % (size_t)be != 0) return -1;
    id_ctx c = {y, bytes, xq, xd, ty, in_dim, out_dim, m,
                (in_dim / (size_t)be) * (size_t)so_block_bytes(ty), isums};
    par_rows(out_dim, nthreads, 0, idot_row, &c);
    return 0;
}

int so_version(void) { return 1; }
