// W8A8 prefill GEMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a
// GEMM: a serving loop that has handed the whole device to its own arena and treats
// any later driver allocation as a bug (or simply has no memory left to give); a
// latency-critical path that cannot afford the implicit device-wide synchronisation
// that cudaMalloc / cudaFree may cause while other streams are busy. The regular entry
// point (strix_cuda_prefill_q8_gemm_dev) grows the handle's scratch buffers on
// demand, so it may allocate on any call whose shape is larger than the last one.
//
// The entry point in this file runs the same kernels but takes every byte of scratch
// (int8 activation codes, per-block scales, code sums and un-bias terms, the transposed
// f32 weight scales, split-K partials) from ONE file-scope device array of fixed size.
// It calls no cudaMalloc / cudaFree and no allocating library routine.
//
// What a caller has to know:
//  * the array is STRIX_NOALLOC_SCRATCH_BYTES (32 MiB) on every GPU that loads the
//    library, for the life of the process; a shape that needs more is refused with
//    an error that names the size;
//  * the driver loads device code lazily: the 32 MiB behind the array and the code of
//    the kernels this path launches are materialised when they are first touched, and
//    that step can allocate (and fail for want of memory). strix_cuda_create touches
//    them all - it looks the array's device address up (cudaGetSymbolAddress, with the
//    handle's device current) and asks for the kernels' attributes - so that happens
//    at handle creation, before a caller's arena takes the device. The entry point
//    falls back to the look-up on its first call only for a device on which no handle
//    was ever created through strix_cuda_create; keep such a first call outside any
//    stream capture;
//  * all calls share the array and it keeps the previous call's contents. Nothing in
//    it has to start at zero (every word that is read is written earlier in the same
//    call), but two calls whose kernels overlap on the GPU (different streams, or
//    different handles on one device) race on it: serialise them.
#include <mutex>
#include <string>

#include "accel.h"

using namespace strix;

#define STRIX_NOALLOC_SCRATCH_BYTES (32u << 20)

// The scratch itself. In host code this name is only a handle for the runtime's symbol
// table, not a device address: it must never be passed to a kernel as a pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[STRIX_NOALLOC_SCRATCH_BYTES];

static std::mutex g_noalloc_mu;
static unsigned char *g_noalloc_ptr[64] = {nullptr};  // device address of the array, per device ordinal

// Device address of g_noalloc_scratch on `device` (which must be current). Looked up once per device.
static cudaError_t noalloc_base(int device, unsigned char **out) {
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        g_noalloc_ptr[device] = static_cast<unsigned char *>(p);
    }
    *out = g_noalloc_ptr[device];
    return cudaSuccess;
}

static inline size_t up256(size_t v) { return (v + 255u) & ~(size_t)255u; }

namespace strix {
// Called by strix_cuda_create with `device` current: the array's backing memory is materialised now.
cudaError_t noalloc_prepare_device(int device) {
    unsigned char *p = nullptr;
    return noalloc_base(device, &p);
}
}  // namespace strix

extern "C" {

size_t strix_cuda_noalloc_scratch_bytes(void) { return STRIX_NOALLOC_SCRATCH_BYTES; }

int strix_cuda_prefill_q8_gemm_noalloc(strix_cuda *h, const char *key, const float *d_xs, size_t m, float *d_y,
                                       void *stream) {
    if (!h || !key || !d_xs || !d_y) return -1;
    h->err.clear();
    const Resident *r = find_weight(h, key);
    if (!r || r->fmt != FMT_Q8_0) return 0;
    if (m == 0 || r->rows == 0) return 1;
    if (m > 0x7fffffffu / r->L.in_dim) {
        h->err = "prefill_q8_gemm_noalloc: m * in_dim does not fit 31 bits";
        return -1;
    }
    cudaError_t e = cudaSetDevice(h->device);
    unsigned char *base = nullptr;
    if (e == cudaSuccess) e = noalloc_base(h->device, &base);
    if (e != cudaSuccess) {
        h->err = std::string("prefill_q8_gemm_noalloc: ") + cudaGetErrorString(e);
        return -1;
    }
    // carve the array: codes | scales | code sums | un-bias terms | transposed weight scales | split-K partials
    const size_t K = r->L.in_dim, nb = r->L.nb, ldm = gemm_x_ld((uint32_t)m), lds = gemm_scales_ld((uint32_t)r->rows);
    const uint32_t splits = gemm_pick_splits((uint32_t)m, (uint32_t)r->rows, (uint32_t)nb, h->num_sms);
    size_t off = 0;
    const size_t o_xq = off;  off += up256(m * K);
    const size_t o_xd = off;  off += up256(nb * ldm * sizeof(float));
    const size_t o_xs = off;  off += up256(nb * ldm * sizeof(int32_t));
    const size_t o_xc = off;  off += up256(nb * ldm * sizeof(float));
    const size_t o_sc = off;  off += up256(nb * lds * sizeof(float));
    const size_t o_pt = off;  off += up256(gemm_workspace_floats((uint32_t)m, (uint32_t)r->rows, splits) * sizeof(float));
    if (off > STRIX_NOALLOC_SCRATCH_BYTES) {
        h->err = "prefill_q8_gemm_noalloc: this shape needs " + std::to_string(off) + " bytes of scratch, the fixed array holds " +
                 std::to_string((size_t)STRIX_NOALLOC_SCRATCH_BYTES);
        return -1;
    }
    int8_t *xq = reinterpret_cast<int8_t *>(base + o_xq);
    float *xd = reinterpret_cast<float *>(base + o_xd);
    int32_t *xs = reinterpret_cast<int32_t *>(base + o_xs);
    float *xc = reinterpret_cast<float *>(base + o_xc);
    float *sc = reinterpret_cast<float *>(base + o_sc);
    float *pt = reinterpret_cast<float *>(base + o_pt);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    e = launch_scales_transpose(r->dev, sc, r->L, (uint32_t)r->rows, st);
    if (e == cudaSuccess) e = launch_xquant8_sum(d_xs, xq, xd, xs, xc, (uint32_t)m, (uint32_t)nb, st);
    if (e == cudaSuccess)
        e = launch_gemm_w8a8(r->gemm_codes, r->L, (uint32_t)r->rows, sc, xq, xd, xs, xc, (uint32_t)m, d_y, pt, splits, 0, nullptr,
                             h->d_status, st);
    if (e != cudaSuccess) {
        h->err = std::string("prefill_q8_gemm_noalloc: ") + cudaGetErrorString(e);
        return -1;
    }
    return 1;
}

}  // extern "C"
