/* memory.c - tracked host allocation plus device-aware allocate / copy / set.
 *
 * Host side follows the reference's scheme (src/core/memory.c:17-74): a header in front of
 * every block remembers the size so that free can maintain the global counters
 * (allocated/peak/freed bytes and blocks).  The device-aware calls, which the reference
 * left as host stubs (memory.c:174-186, :230-247), go to the CUDA runtime layer. */
#include "boat_internal.h"
#include <stdlib.h>
#include <string.h>

typedef struct {
    size_t size;
    boat_device_t device;
    const char* file;
    int line;
    int pinned;              /* block came from the page-locked pool */
    int pad_[3];             /* keeps the payload 16-byte aligned */
} block_header_t;

/* Host blocks of this size and above hold tensor data that will be copied to or from the
 * GPU; they are taken page-locked (and re-used) once the library has been bound to a GPU
 * (boat_cuda_init, or the first compute call).  A host allocation never starts the GPU by
 * itself: before that, and without a GPU, the block is ordinary memory. */
#define BOAT_PINNED_THRESHOLD ((size_t)256 * 1024)

static boat_memory_stats_t g_stats;

int boat_report(const char* what, int rc) {
    if (rc != 0) fprintf(stderr, "boat: %s: %s\n", what, boat_cuda_last_error());
    return rc;
}

static void note_alloc(size_t n) {
    g_stats.allocated_bytes += n;
    g_stats.allocated_blocks += 1;
    if (g_stats.allocated_bytes > g_stats.peak_allocated_bytes)
        g_stats.peak_allocated_bytes = g_stats.allocated_bytes;
}

static void note_free(size_t n) {
    g_stats.allocated_bytes -= n;
    g_stats.freed_bytes += n;
    g_stats.freed_blocks += 1;
}

void* boat_memory_allocate(size_t size, boat_device_t device, const char* file, int line) {
    if (size == 0) return NULL;
    block_header_t* h = NULL;
    int pinned = 0;
    if (size >= BOAT_PINNED_THRESHOLD && boat_cuda_device_count() > 0) {
        h = (block_header_t*)boat_cuda_host_alloc(sizeof(block_header_t) + size);
        pinned = h != NULL;
    }
    if (!h) h = (block_header_t*)malloc(sizeof(block_header_t) + size);
    if (!h) {
        fprintf(stderr, "Memory allocation failed: %zu bytes at %s:%d\n", size, file ? file : "?", line);
        return NULL;
    }
    h->size = size;
    h->device = device;
    h->file = file;
    h->line = line;
    h->pinned = pinned;
    note_alloc(size);
    return h + 1;
}

void* boat_memory_allocate_zero(size_t size, boat_device_t device, const char* file, int line) {
    void* p = boat_memory_allocate(size, device, file, line);
    if (p) memset(p, 0, size);
    return p;
}

void* boat_memory_reallocate(void* ptr, size_t new_size, boat_device_t device, const char* file, int line) {
    if (!ptr) return boat_memory_allocate(new_size, device, file, line);
    if (new_size == 0) {
        boat_memory_free(ptr);
        return NULL;
    }
    block_header_t* old = (block_header_t*)ptr - 1;
    size_t old_size = old->size;
    if (old->pinned || new_size >= BOAT_PINNED_THRESHOLD) {
        /* blocks of the page-locked pool cannot be realloc'ed: allocate, copy, free */
        void* fresh = boat_memory_allocate(new_size, device, file, line);
        if (!fresh) return NULL;
        memcpy(fresh, ptr, old_size < new_size ? old_size : new_size);
        boat_memory_free(ptr);
        return fresh;
    }
    block_header_t* h = (block_header_t*)realloc(old, sizeof(block_header_t) + new_size);
    if (!h) return NULL;
    note_free(old_size);
    note_alloc(new_size);
    h->size = new_size;
    h->device = device;
    h->file = file;
    h->line = line;
    h->pinned = 0;
    return h + 1;
}

void boat_memory_free(void* ptr) {
    if (!ptr) return;
    block_header_t* h = (block_header_t*)ptr - 1;
    note_free(h->size);
    if (h->pinned) boat_cuda_host_free(h);
    else free(h);
}

void boat_memory_free_safe(void** ptr_ptr) {
    if (ptr_ptr && *ptr_ptr) {
        boat_memory_free(*ptr_ptr);
        *ptr_ptr = NULL;
    }
}

void* boat_memory_allocate_device(size_t size, boat_device_t device, const char* file, int line) {
    if (device != BOAT_DEVICE_CUDA) return boat_memory_allocate(size, device, file, line);
    void* p = NULL;
    if (boat_report("device allocation", boat_cuda_malloc(&p, size)) != 0) return NULL;
    return p;
}

void boat_memory_free_device(void* ptr, boat_device_t device) {
    if (!ptr) return;
    if (device != BOAT_DEVICE_CUDA) {
        boat_memory_free(ptr);
        return;
    }
    boat_report("device free", boat_cuda_free(ptr));
}

void boat_memory_copy(void* dest, const void* src, size_t size, boat_device_t dest_device,
                      boat_device_t src_device) {
    if (!dest || !src || size == 0) return;
    bool d = dest_device == BOAT_DEVICE_CUDA, s = src_device == BOAT_DEVICE_CUDA;
    if (!d && !s) {
        memcpy(dest, src, size);
    } else if (d && !s) {
        boat_report("host to device copy", boat_cuda_memcpy_h2d(dest, src, size));
    } else if (!d && s) {
        boat_report("device to host copy", boat_cuda_memcpy_d2h(dest, src, size));
    } else {
        if (boat_report("device copy", boat_cuda_memcpy_d2d(dest, src, size)) == 0)
            boat_report("device copy", boat_cuda_sync());
    }
}

void boat_memory_set(void* dest, int value, size_t size, boat_device_t device) {
    if (!dest || size == 0) return;
    if (device == BOAT_DEVICE_CUDA) boat_report("device fill", boat_cuda_memset(dest, value, size));
    else memset(dest, value, size);
}

boat_memory_stats_t boat_memory_get_stats(void) { return g_stats; }

void boat_memory_reset_stats(void) { memset(&g_stats, 0, sizeof g_stats); }

void boat_memory_print_stats(FILE* stream) {
    if (!stream) stream = stdout;
    fprintf(stream, "host memory: %zu bytes live in %zu allocations (peak %zu bytes), %zu bytes freed in %zu frees\n",
            g_stats.allocated_bytes, g_stats.allocated_blocks - g_stats.freed_blocks,
            g_stats.peak_allocated_bytes, g_stats.freed_bytes, g_stats.freed_blocks);
    fprintf(stream, "device memory: %zu bytes live\n", boat_cuda_bytes_in_use());
}
