/*
 * Static-partition parallel-for used by the CPU oracle (test infrastructure).
 * Mirrors the work split of the reference's thread pool
 * (core/src/system/parallel.zig:154-215): n_items are cut into contiguous
 * ranges of ceil(n/threads) rounded up to a multiple of 16 items, the calling
 * thread runs range 0, and the call returns after a barrier.
 */
#ifndef GAF_POOL_H
#define GAF_POOL_H
#include <stddef.h>

typedef void (*gaf_range_fn)(size_t start, size_t end, void *ctx);

/* nthreads <= 1 runs fn(0, n_items) inline. */
void gaf_parallel_for(size_t n_items, gaf_range_fn fn, void *ctx, int nthreads);

#endif
