/* export.h - symbol visibility and calling-convention macros for the B200 build of
 * Boat's attention path.
 *
 * Replaces the reference's include/boat/export.h (macros BOAT_API, BOAT_CALL,
 * BOAT_NOINLINE at export.h:15-58).  Only the Linux/ELF case exists here: the library is a
 * CUDA shared object, so BOAT_CALL is empty and BOAT_API is default visibility. */
#ifndef BOAT_EXPORT_H
#define BOAT_EXPORT_H

#define BOAT_CALL

#if defined(BOAT_STATIC_BUILD)
#  define BOAT_API
#elif defined(__GNUC__)
#  define BOAT_API __attribute__((visibility("default")))
#else
#  define BOAT_API
#endif

#if defined(__GNUC__)
#  define BOAT_NOINLINE   __attribute__((noinline))
#  define BOAT_DEPRECATED __attribute__((deprecated))
#else
#  define BOAT_NOINLINE
#  define BOAT_DEPRECATED
#endif

#define BOAT_INLINE static inline
#define BOAT_STATIC static

#ifndef BOAT_DEBUG
#  define BOAT_DEBUG 0
#endif

#endif /* BOAT_EXPORT_H */
