// Greedy argmax over logits on the device, and the two trait methods built on it.
//
//   argmax_f32                    crates/strix-backend-rocm/src/kernels.rs:2088-2110
//   decode_step_argmax            crates/strix-core/src/accel.rs:437-442; decode.rs:5497-5515, 5533-5538
//   lm_head_argmax_rows           crates/strix-core/src/accel.rs:216-219; decode.rs:3631-3689
//
// Semantics of the reference kernel, kept exactly: the running best starts at (-3.0e38, index 0), a
// value replaces it only if it is GREATER (so NaN never wins and values at or below -3.0e38 leave
// index 0), and ties resolve to the LOWEST index. The reference scans with one block of 1024
// threads; here every SM takes a slice of the row and the last block to finish folds the per-block
// winners (a ticket counter, no block waits for another), so a 151936-entry row costs a few
// microseconds instead of a single SM's read of 600 KB. The result does not depend on the split:
// "greater, then lower index" is a total order.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <string>

#include "accel.h"
#include "kernels.h"

namespace strix {

constexpr int ARGMAX_THREADS = 256;
constexpr int ARGMAX_MAX_BLOCKS = 256;  // per row

struct Best {
    float v;
    uint32_t i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
    // b replaces a if greater, or equal with a lower index
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// grid = (blocks per row, rows). part: [rows][gridDim.x] winners; ticket: [rows] counters (zero before the
// first launch; the last block of a row resets its counter, so the buffer is reusable).
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_rows_kernel(const float *__restrict__ x, uint32_t n, size_t stride,
                                                                      Best *__restrict__ part, uint32_t *__restrict__ ticket,
                                                                      uint32_t *__restrict__ out_idx,
                                                                      float *__restrict__ out_val) {
    const uint32_t row = blockIdx.y, nb = gridDim.x, t = threadIdx.x;
    const float *xr = x + (size_t)row * stride;
    // contiguous slice per block, float4 body where the row allows it
    const uint32_t per = (((n + nb - 1) / nb) + 3u) & ~3u;
    const uint32_t lo = min(n, blockIdx.x * per), hi = min(n, lo + per);
    Best b{-3.0e38f, 0u};
    const bool vec = ((reinterpret_cast<uintptr_t>(xr) & 15u) == 0) && (stride % 4u == 0);
    if (vec) {
        const uint32_t hi4 = lo + ((hi - lo) & ~3u);
        for (uint32_t i = lo + 4u * t; i < hi4; i += 4u * ARGMAX_THREADS) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(xr + i));
            if (v.x > b.v) { b.v = v.x; b.i = i; }  // ascending within the thread: lowest index on a tie
            if (v.y > b.v) { b.v = v.y; b.i = i + 1u; }
            if (v.z > b.v) { b.v = v.z; b.i = i + 2u; }
            if (v.w > b.v) { b.v = v.w; b.i = i + 3u; }
        }
        for (uint32_t i = hi4 + t; i < hi; i += ARGMAX_THREADS) {
            const float v = __ldcg(xr + i);
            if (v > b.v) { b.v = v; b.i = i; }
        }
    } else {
        for (uint32_t i = lo + t; i < hi; i += ARGMAX_THREADS) {
            const float v = __ldcg(xr + i);
            if (v > b.v) { b.v = v; b.i = i; }
        }
    }
    __shared__ Best sb[ARGMAX_THREADS / 32];
    __shared__ bool last;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best ob;
        ob.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        ob.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        b = better(b, ob);
    }
    if ((t & 31u) == 0) sb[t >> 5] = b;
    __syncthreads();
    if (t == 0) {
        for (int w = 1; w < ARGMAX_THREADS / 32; w++) b = better(b, sb[w]);
        part[(size_t)row * nb + blockIdx.x] = b;
        __threadfence();
        last = atomicAdd(&ticket[row], 1u) == nb - 1u;
    }
    __syncthreads();
    if (!last) return;
    // the last block of this row: fold the per-block winners
    __threadfence();
    Best f{-3.0e38f, 0u};
    for (uint32_t k = t; k < nb; k += ARGMAX_THREADS) f = better(f, part[(size_t)row * nb + k]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best ob;
        ob.v = __shfl_xor_sync(0xffffffffu, f.v, o);
        ob.i = __shfl_xor_sync(0xffffffffu, f.i, o);
        f = better(f, ob);
    }
    __syncthreads();  // sb is reused
    if ((t & 31u) == 0) sb[t >> 5] = f;
    __syncthreads();
    if (t == 0) {
        for (int w = 1; w < ARGMAX_THREADS / 32; w++) f = better(f, sb[w]);
        out_idx[row] = f.i;
        if (out_val) out_val[row] = f.v;
        ticket[row] = 0u;
    }
}

}  // namespace strix

// ------------------------------------------------------------------ host side
namespace strix {

constexpr size_t ARGMAX_MAX_ROWS = 16;  // the reference's bound on m (decode.rs:3633)

static int ensure_argmax(strix_cuda *h) {
    if (h->am_part) return 0;
    const size_t part_b = ARGMAX_MAX_ROWS * ARGMAX_MAX_BLOCKS * sizeof(Best);
    const size_t total = part_b + 3 * ARGMAX_MAX_ROWS * 4;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, total);
    if (e == cudaSuccess) e = cudaMemset(p, 0, total);
    // (the memset runs on the legacy default stream, the kernels on non-blocking streams: nothing else orders them)
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMallocHost(reinterpret_cast<void **>(&h->am_pin), (ARGMAX_MAX_ROWS + 1) * 4);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        h->err = std::string("argmax: scratch: ") + cudaGetErrorString(e);
        return -1;
    }
    h->am_part = p;
    uint8_t *b = static_cast<uint8_t *>(p) + part_b;
    h->am_ticket = reinterpret_cast<uint32_t *>(b);
    h->am_idx = reinterpret_cast<uint32_t *>(b + ARGMAX_MAX_ROWS * 4);
    h->am_val = reinterpret_cast<float *>(b + 2 * ARGMAX_MAX_ROWS * 4);
    return 0;
}

int argmax_rows_enqueue(strix_cuda *h, const float *d_x, size_t n, size_t stride, size_t rows, cudaStream_t stream) {
    if (rows == 0) return 1;
    if (rows > ARGMAX_MAX_ROWS || n == 0 || n > 0xffffffffull) {
        h->err = "argmax: at most 16 rows of 1 .. 2^32-1 entries";
        return -1;
    }
    if (ensure_argmax(h) < 0) return -1;
    // one block per SM up to the scratch's width; at least 1024 entries per block
    uint32_t nb = (uint32_t)std::min<size_t>((size_t)std::min(h->num_sms, ARGMAX_MAX_BLOCKS), (n + 1023) / 1024);
    if (nb == 0) nb = 1;
    ProfScope prof(h, stream, "argmax");
    argmax_rows_kernel<<<dim3(nb, (unsigned)rows), ARGMAX_THREADS, 0, stream>>>(
        d_x, (uint32_t)n, stride, static_cast<Best *>(h->am_part), h->am_ticket, h->am_idx, h->am_val);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        h->err = std::string("argmax: launch: ") + cudaGetErrorString(e);
        return -1;
    }
    return 1;
}

}  // namespace strix

using namespace strix;

#define CU_TRY(h, expr)                                                    \
    do {                                                                   \
        cudaError_t _e = (expr);                                           \
        if (_e != cudaSuccess) {                                           \
            (h)->err = std::string(#expr) + ": " + cudaGetErrorString(_e); \
            return -1;                                                     \
        }                                                                  \
    } while (0)

extern "C" {

int strix_cuda_argmax_dev(strix_cuda *h, const float *d_x, size_t n, size_t stride, size_t rows, uint32_t *d_ids,
                          float *d_vals, void *stream) {
    if (!h || !d_x) return -1;
    h->err.clear();
    CU_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int rc = argmax_rows_enqueue(h, d_x, n, stride, rows, s);
    if (rc < 0 || rows == 0) return rc;
    if (d_ids) CU_TRY(h, cudaMemcpyAsync(d_ids, h->am_idx, rows * 4, cudaMemcpyDeviceToDevice, s));
    if (d_vals) CU_TRY(h, cudaMemcpyAsync(d_vals, h->am_val, rows * 4, cudaMemcpyDeviceToDevice, s));
    return 1;
}

int strix_cuda_lm_head_argmax_rows(strix_cuda *h, const char *key, const float *xs, size_t xs_len, size_t m, int act,
                                   uint32_t *ids, float *vals) {
    if (!h || !key || !xs || !ids) return -1;
    h->err.clear();
    const Resident *r = find_weight(h, key);
    if (!r) return 0;                                            // not resident: None
    const size_t K = r->L.in_dim;
    if (xs_len != m * K || m > ARGMAX_MAX_ROWS) return 0;        // the reference's guard (decode.rs:3633-3635)
    if (m == 0) return 1;
    if (r->rows == 0) {
        h->err = "lm_head_argmax_rows: this accelerator holds no row of the weight";
        return -1;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    if (ensure_f32(h, h->x, m * K) < 0 || ensure_f32(h, h->y, m * r->rows) < 0) return -1;
    CU_TRY(h, cudaMemcpyAsync(h->x.p, xs, m * K * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    const Resident *w1[1] = {r};
    float *y1[1] = {h->y.p};
    if (gemv_launch_rows(h, 1, w1, h->x.p, nullptr, 0.f, STRIX_PRE_NONE, act, y1, nullptr, (uint32_t)m, (uint32_t)K, 0,
                         h->stream) < 0)
        return -1;
    if (argmax_rows_enqueue(h, h->y.p, r->rows, r->rows, m, h->stream) < 0) return -1;
    CU_TRY(h, cudaMemcpyAsync(h->am_pin, h->am_idx, m * 4, cudaMemcpyDeviceToHost, h->stream));
    if (vals) CU_TRY(h, cudaMemcpyAsync(vals, h->am_val, m * 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaMemcpyAsync(h->am_pin + ARGMAX_MAX_ROWS, h->d_status, 4, cudaMemcpyDeviceToHost, h->stream));
    CU_TRY(h, cudaStreamSynchronize(h->stream));
    if (h->am_pin[ARGMAX_MAX_ROWS] != 0) {
        h->err = "lm_head_argmax_rows: device status " + std::to_string(h->am_pin[ARGMAX_MAX_ROWS]) + " (a bounded wait ran out)";
        cudaMemsetAsync(h->d_status, 0, 4, h->stream);
        return -2;
    }
    // row index within the whole weight (a row shard holds rows [row0, row0 + rows))
    for (size_t t = 0; t < m; t++) ids[t] = h->am_pin[t] + (uint32_t)r->row0;
    return 1;
}

}  // extern "C"

extern "C" void strix_cuda_fold_argmax_shards(size_t n_shards, size_t m, const uint32_t *ids, const float *vals,
                                              uint32_t *out_ids, float *out_vals) {
    if (!ids || !vals || !out_ids) return;
    for (size_t t = 0; t < m; t++) {
        float best_v = -3.0e38f;
        uint32_t best_i = 0;
        for (size_t r = 0; r < n_shards; r++) {
            const float v = vals[r * m + t];
            const uint32_t i = ids[r * m + t];
            if (v > best_v || (v == best_v && i < best_i)) {  // (a NaN compares false both ways: it never wins)
                best_v = v;
                best_i = i;
            }
        }
        out_ids[t] = best_i;
        if (out_vals) out_vals[t] = best_v;
    }
}
