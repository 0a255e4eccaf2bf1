/* stage.h - moving tensors between the caller's memory space/dtype and device buffers in the
 * storage type a kernel wants.  Shared by the layers around attention (LayerNorm, dense). */
#ifndef BOAT_STAGE_H
#define BOAT_STAGE_H

#include "boat_internal.h"

int    boat_storage_of(boat_dtype_t dt);                 /* BOAT_CUDA_F32 / BOAT_CUDA_BF16 */
size_t boat_storage_size(int type);
bool   boat_dtype_supported(boat_dtype_t dt);            /* FLOAT32 or BFLOAT16 */
void*  boat_dev_alloc(size_t bytes);                     /* NULL + message on failure */
void   boat_dev_free(void* p);
/* Device buffer with tensor `t` in storage `type`; *owned: caller must boat_dev_free it. */
void*  boat_stage_in(const boat_tensor_t* t, int type, bool* owned);
/* New tensor shaped `shape`, with dtype/device of `like`, filled from device buffer `src`. */
boat_tensor_t* boat_emit_out(const int64_t* shape, size_t ndim, const boat_tensor_t* like, void* src, int type);
/* Like boat_emit_out for a buffer from boat_dev_alloc that the caller is done with: a CUDA result
 * of the same storage type becomes a tensor around *src itself (no copy) and *src is set to NULL,
 * so that the caller's boat_dev_free(*src) is a no-op; every other case copies as boat_emit_out. */
boat_tensor_t* boat_emit_out_take(const int64_t* shape, size_t ndim, const boat_tensor_t* like, void** src, int type);
/* Arithmetic for FP32/BF16 inputs outside the attention layer: BF16 storage -> BF16 tensor
 * cores; FP32 storage -> env BOAT_MMA (tf32 | fp32), default exact FP32. */
int    boat_default_mma(boat_dtype_t dt);

#endif
