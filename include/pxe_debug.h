/* Debug interface of libpxe: the bounds-checked build.
 *
 * libpxe_checked.so is libpxe.so compiled with -DPXE_BOUNDS_CHECK: every access of a kernel to global memory
 * (each load, store and atomic of every kernel family) first looks its address up in a table of the
 * caller's device allocations.  An access that lies outside every allocation, straddles the end of one or is not
 * aligned to its own width is NOT performed: a load yields zeros, a store is dropped, the kernel runs on to its end
 * (no trap, no device assert, the context stays usable) and the first such access is recorded -- address, width,
 * load or store, source file and line of the access.  This is the check a memory checker makes, for boxes where
 * none can run.  It is slow (a binary search per access) and meant for small shapes.
 *
 * The three entry points exist in both builds; the ordinary build answers PXE_ERR_UNSUPPORTED to the last two.
 * One device per process; not thread-safe.
 */
#ifndef PXE_DEBUG_H
#define PXE_DEBUG_H

#include <stddef.h>

#include "pxe.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pxe_bounds_report {
    unsigned int violations;        /* accesses refused since the last reset */
    int bytes;                      /* width of the first one */
    unsigned long long address;     /* its address */
    int line;                       /* source line of the access */
    int is_store;                   /* 1 store or atomic, 0 load */
    int misaligned;                 /* 1 if the address was inside an allocation but not a multiple of its width */
    int reserved;
    char file[48];                  /* base name of the source file */
} pxe_bounds_report;

/* 1 in the bounds-checked build, 0 in the ordinary one. */
PXE_API int pxe_debug_bounds_checked(void);

/* Arms the check with the device allocations the kernels may touch: `count` ranges [starts[i], starts[i] + bytes[i]).
 * Memory the library owns itself (the static scratch of pxe_yolo_decode_static) is added by the library.
 * count = 0 disarms.  Synchronises the device.  Up to 4096 ranges. */
PXE_API int pxe_debug_set_allocations(const void* const* starts, const size_t* bytes, int count);

/* Synchronises the device and copies the record out; reset != 0 clears it afterwards. */
PXE_API int pxe_debug_read_report(pxe_bounds_report* out, int reset);

#ifdef __cplusplus
}
#endif
#endif /* PXE_DEBUG_H */
