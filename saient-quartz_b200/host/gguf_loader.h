/*
 * GGUF file reader and device loader: the C++ counterpart of the reference's GgufFile
 * (src/gguf.rs:53-123: header, metadata, tensor table, data section found by general.alignment)
 * and of its upload step (GpuBuf::upload of tensor_data, src/cuda.rs:76-82, 170-172).  The file is
 * mapped read-only; a tensor's bytes are the contiguous range
 *     data_offset + info.offset .. + ggml_type_size(type, n_elems)        (src/gguf.rs:118-123)
 * Uploads go through a pair of page-locked staging buffers so that the copy of chunk i+1 from the
 * mapping overlaps the transfer of chunk i, then through the one-time repack hook
 * (cuda_repack_weights) so that the streaming kernels can serve the tensor.
 *
 * C interface for ctypes / FFI; every function returns 0 / a valid handle on success.
 */
#ifndef QUARTZ_HOST_GGUF_LOADER_H
#define QUARTZ_HOST_GGUF_LOADER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct qg_file qg_file;

/* NULL on failure; qg_last_error() says why (not a GGUF file, unsupported version, truncated ...) */
qg_file *qg_open(const char *path);
void qg_close(qg_file *f);
const char *qg_last_error(void);

uint32_t qg_version(const qg_file *f);
uint64_t qg_data_offset(const qg_file *f);

/* tensor table, in file order */
int qg_n_tensors(const qg_file *f);
int qg_find_tensor(const qg_file *f, const char *name);          /* index or -1 */
const char *qg_tensor_name(const qg_file *f, int i);
uint32_t qg_tensor_type(const qg_file *f, int i);
int qg_tensor_n_dims(const qg_file *f, int i);
uint64_t qg_tensor_dim(const qg_file *f, int i, int d);          /* dims[0] = fastest-varying (in_features) */
uint64_t qg_tensor_bytes(const qg_file *f, int i);               /* 0 for a type this library does not know */
const void *qg_tensor_data(const qg_file *f, int i);             /* pointer into the mapping, NULL if out of range */

/* metadata: 1 if the key exists with a convertible type (u32: UINT32/INT32; u64: UINT64/UINT32;
 * f32: FLOAT32; str: STRING, returned pointer lives as long as the file), else 0 */
int qg_meta_u32(const qg_file *f, const char *key, uint32_t *out);
int qg_meta_u64(const qg_file *f, const char *key, uint64_t *out);
int qg_meta_f32(const qg_file *f, const char *key, float *out);
const char *qg_meta_str(const qg_file *f, const char *key);
int qg_meta_array_len(const qg_file *f, const char *key, uint64_t *out);
int qg_meta_bool(const qg_file *f, const char *key, int *out);

/* Allocate device memory for tensor i (cuda_alloc), stream its bytes in through the staging
 * buffers, and (repack != 0, quantized 2-D/3-D tensors) call cuda_repack_weights with
 * in_dim = dims[0], out_dim = dims[1], n_mats = dims[2] or 1.  Returns the device pointer (the caller
 * owns it: cuda_drop) or NULL.  *repacked_out (optional) receives what the repack hook returned. */
void *qg_upload_tensor(const qg_file *f, int i, int repack, int *repacked_out);

#ifdef __cplusplus
}
#endif
#endif
