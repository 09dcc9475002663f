/* GGUF container reader (v2 / v3) and the glue that feeds its tensors to the accelerator.
 *
 * Replaces, for the quantized-matmul path, crates/strix-models/src/gguf.rs:104-269 of the reference
 * (GgufFile::open / parse / tensor_bytes / advise_dontneed and the metadata getters): the file is
 * memory-mapped, the metadata and the tensor index are parsed up front, tensor data stays in the map
 * and is handed to strix_cuda_upload_* as borrowed raw block bytes, row-major
 * [out_dim][in_dim / block][block bytes] with in_dim = dims[0], out_dim = dims[1]
 * (crates/strix-backend-cpu/src/qwen3.rs:772-774).
 *
 * Return convention: 1 = ok / found / adopted, 0 = not found / declined, < 0 = error (message from
 * strix_gguf_last_error, thread-local). Plain pointers and sizes only.
 */
#ifndef STRIX_GGUF_H
#define STRIX_GGUF_H

#include <stddef.h>
#include <stdint.h>

#include "strix_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct strix_gguf strix_gguf;

/* ggml_type ids the reference recognises (crates/strix-models/src/ggml_quant.rs:41-64) */
enum {
    STRIX_GGML_F32 = 0, STRIX_GGML_F16 = 1, STRIX_GGML_Q4_0 = 2, STRIX_GGML_Q4_1 = 3, STRIX_GGML_Q5_0 = 6,
    STRIX_GGML_Q5_1 = 7, STRIX_GGML_Q8_0 = 8, STRIX_GGML_Q8_1 = 9, STRIX_GGML_Q2_K = 10, STRIX_GGML_Q3_K = 11,
    STRIX_GGML_Q4_K = 12, STRIX_GGML_Q5_K = 13, STRIX_GGML_Q6_K = 14, STRIX_GGML_Q8_K = 15
};

/* One entry of the tensor index (TensorInfo, gguf.rs:83-101) plus where its bytes are in the map. */
typedef struct strix_gguf_tensor {
    const char *name;     /* owned by the file object */
    uint32_t n_dims;
    uint64_t dims[4];     /* GGUF order, fastest-varying first; unused entries are 1 */
    uint32_t ggml_type;
    uint64_t offset;      /* from the start of the tensor-data section */
    const uint8_t *data;  /* borrowed: valid until strix_gguf_close */
    size_t nbytes;        /* numel / block_elems * block_bytes (gguf.rs:222) */
} strix_gguf_tensor;

/* GgufFile::open (gguf.rs:112-117). Errors: not a GGUF file (magic), version other than 2 / 3,
 * unexpected EOF, nested arrays, unknown metadata or tensor type, data offset past EOF. */
STRIX_API int strix_gguf_open(const char *path, strix_gguf **out);
/* The same parser on a caller-owned buffer (borrowed until close): what the reference's tests do
 * through a temporary file (gguf.rs:433-441). */
STRIX_API int strix_gguf_open_memory(const uint8_t *bytes, size_t len, strix_gguf **out);
STRIX_API void strix_gguf_close(strix_gguf *g);
STRIX_API const char *strix_gguf_last_error(void);

STRIX_API uint32_t strix_gguf_version(const strix_gguf *g);
STRIX_API size_t strix_gguf_alignment(const strix_gguf *g);   /* general.alignment, default 32 (gguf.rs:163-167) */
STRIX_API size_t strix_gguf_data_offset(const strix_gguf *g); /* header end rounded up to the alignment */
STRIX_API size_t strix_gguf_tensor_count(const strix_gguf *g);
STRIX_API size_t strix_gguf_meta_count(const strix_gguf *g);

/* Tensor index, in file order / by name. tensor_bytes' bound check (gguf.rs:224-230) is done here:
 * a tensor whose data runs past EOF gives -1. */
STRIX_API int strix_gguf_tensor_at(const strix_gguf *g, size_t i, strix_gguf_tensor *out);
STRIX_API int strix_gguf_find_tensor(const strix_gguf *g, const char *name, strix_gguf_tensor *out);

/* Metadata getters with the reference's widening rules (MetaValue::as_u64 / as_f32 / as_str,
 * gguf.rs:43-80): any non-negative integer type widens to u64; f32 also accepts f64 and integers.
 * 0 = key missing or of another kind. */
STRIX_API int strix_gguf_meta_u64(const strix_gguf *g, const char *key, uint64_t *out);
STRIX_API int strix_gguf_meta_f32(const strix_gguf *g, const char *key, float *out);
STRIX_API int strix_gguf_meta_str(const strix_gguf *g, const char *key, const char **out, size_t *len);
STRIX_API int strix_gguf_meta_array_len(const strix_gguf *g, const char *key, uint64_t *len, uint32_t *elem_type);
STRIX_API int strix_gguf_meta_key_at(const strix_gguf *g, size_t i, const char **key, uint32_t *value_type);

/* GgufFile::advise_dontneed (gguf.rs:239-258): drop the whole pages inside the tensor from the page
 * cache view of this mapping once the accelerator holds the weight. No-op for an in-memory file. */
STRIX_API void strix_gguf_advise_dontneed(const strix_gguf *g, const char *name);

/* Block geometry of a ggml_type (ggml_quant.rs:88-124); 0 for an unknown id. */
STRIX_API size_t strix_ggml_block_elems(uint32_t ggml_type);
STRIX_API size_t strix_ggml_block_bytes(uint32_t ggml_type);

/* Hand one tensor to the accelerator under its GGUF name, as Model::attach_accel does per weight
 * (qwen3.rs:640-700, 772-774): 2-D Q4_0 / Q4_1 / Q8_0 / Q6_K -> strix_cuda_upload_*, 1-D F32 ->
 * strix_cuda_upload_f32. 1 = adopted, 0 = declined (type or rank the accelerator has no kernel
 * for: the weight stays on the CPU), < 0 = error (strix_cuda_last_error or strix_gguf_last_error). */
STRIX_API int strix_cuda_upload_gguf_tensor(strix_cuda *h, const strix_gguf *g, const char *name, int drop_pages);
/* Every tensor of the file; counts what was adopted and what was declined. */
STRIX_API int strix_cuda_upload_gguf(strix_cuda *h, const strix_gguf *g, int drop_pages, size_t *adopted,
                                     size_t *declined);

#ifdef __cplusplus
}
#endif
#endif
