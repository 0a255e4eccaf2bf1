/* memory.h - tracked host allocation and host<->HBM byte movement.
 *
 * Mirrors the part of the reference's include/boat/memory.h that the attention path and
 * its callers use (memory.h:25-58, macros :80-90).  Host blocks carry a small header so
 * that boat_memory_free() can keep the global statistics (reference:
 * src/core/memory.c:17-74).  The reference's device variants were host-only stubs
 * (memory.c:174-186, :230-247); here BOAT_DEVICE_CUDA means B200 HBM:
 *   boat_memory_allocate_device(.., BOAT_DEVICE_CUDA, ..) returns a device pointer,
 *   boat_memory_copy() is the H2D / D2H / D2D entry point,
 *   boat_memory_set() fills device memory when given BOAT_DEVICE_CUDA.
 * The pool and arena allocators of the reference (memory.c:292-508) are not used by the
 * attention path and are not provided. */
#ifndef BOAT_MEMORY_H
#define BOAT_MEMORY_H

#include <stddef.h>
#include <stdio.h>
#include "tensor.h"
#include "export.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    size_t allocated_bytes;       /* live host bytes handed out            */
    size_t allocated_blocks;      /* allocations made so far               */
    size_t peak_allocated_bytes;
    size_t freed_bytes;
    size_t freed_blocks;
} boat_memory_stats_t;

/* Host allocation with statistics.  size == 0 returns NULL (memory.c:48-50). */
BOAT_API void* boat_memory_allocate(size_t size, boat_device_t device, const char* file, int line);
BOAT_API void* boat_memory_allocate_zero(size_t size, boat_device_t device, const char* file, int line);
BOAT_API void* boat_memory_reallocate(void* ptr, size_t new_size, boat_device_t device,
                                      const char* file, int line);
BOAT_API void  boat_memory_free(void* ptr);
BOAT_API void  boat_memory_free_safe(void** ptr_ptr);

/* Raw device-aware allocation: CPU -> same as boat_memory_allocate, CUDA -> HBM from the
 * library's stream-ordered pool.  Free with boat_memory_free_device and the same device. */
BOAT_API void* boat_memory_allocate_device(size_t size, boat_device_t device, const char* file, int line);
BOAT_API void  boat_memory_free_device(void* ptr, boat_device_t device);

/* Copy `size` bytes; the two device arguments select memcpy / H2D / D2H / D2D.  The call
 * returns after the bytes have arrived (it synchronises the library stream). */
BOAT_API void boat_memory_copy(void* dest, const void* src, size_t size,
                               boat_device_t dest_device, boat_device_t src_device);
BOAT_API void boat_memory_set(void* dest, int value, size_t size, boat_device_t device);

BOAT_API boat_memory_stats_t boat_memory_get_stats(void);
BOAT_API void boat_memory_reset_stats(void);
BOAT_API void boat_memory_print_stats(FILE* stream);

#ifdef BOAT_MEMORY_DEBUG
#  define boat_malloc(size, device)       boat_memory_allocate(size, device, __FILE__, __LINE__)
#  define boat_calloc(size, device)       boat_memory_allocate_zero(size, device, __FILE__, __LINE__)
#  define boat_realloc(ptr, size, device) boat_memory_reallocate(ptr, size, device, __FILE__, __LINE__)
#else
#  define boat_malloc(size, device)       boat_memory_allocate(size, device, NULL, 0)
#  define boat_calloc(size, device)       boat_memory_allocate_zero(size, device, NULL, 0)
#  define boat_realloc(ptr, size, device) boat_memory_reallocate(ptr, size, device, NULL, 0)
#endif
#define boat_free(ptr) boat_memory_free(ptr)

#ifdef __cplusplus
}
#endif
#endif /* BOAT_MEMORY_H */
