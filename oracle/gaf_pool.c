/*
 * Persistent pthread pool with the reference's static partition rule
 * (core/src/system/parallel.zig:154-215).  Test infrastructure only.
 *
 * Workers spin briefly on a generation counter and then sleep on a condition
 * variable; the submitting thread runs range 0 and waits for the others.
 * If the pool is busy (another caller holds it) the call runs single-threaded,
 * like the reference's tryLock fallback (parallel.zig:171-176).
 */
#define _GNU_SOURCE
#include "gaf_pool.h"

#include <pthread.h>
#include <sched.h>
#include <stdatomic.h>
#include <stdlib.h>

#define GAF_MAX_THREADS 256
#define GAF_CHUNK_ROUND 16 /* FLOATS_PER_CACHE_LINE, parallel.zig:16 */
#define GAF_SPINS 20000

typedef struct {
    pthread_t threads[GAF_MAX_THREADS];
    int n_workers; /* spawned workers (excluding the caller) */
    pthread_mutex_t submit;
    pthread_mutex_t mu;
    pthread_cond_t wake;
    pthread_cond_t done_cv;
    atomic_uint generation;
    atomic_int pending;
    /* current task */
    gaf_range_fn fn;
    void *ctx;
    size_t n_items;
    size_t per_thread;
    int active; /* threads participating in this task (including caller) */
} gaf_pool_t;

static gaf_pool_t g_pool = {
    .n_workers = 0,
    .submit = PTHREAD_MUTEX_INITIALIZER,
    .mu = PTHREAD_MUTEX_INITIALIZER,
    .wake = PTHREAD_COND_INITIALIZER,
    .done_cv = PTHREAD_COND_INITIALIZER,
};

static void run_share(gaf_pool_t *p, int idx) {
    if (idx >= p->active) return;
    size_t start = (size_t)idx * p->per_thread;
    if (start >= p->n_items) return;
    size_t end = start + p->per_thread;
    if (end > p->n_items) end = p->n_items;
    p->fn(start, end, p->ctx);
}

static void *worker_main(void *arg) {
    gaf_pool_t *p = &g_pool;
    int idx = (int)(size_t)arg; /* 1-based share index */
    unsigned seen = 0;
    for (;;) {
        int spins = 0;
        while (atomic_load_explicit(&p->generation, memory_order_acquire) == seen) {
            if (++spins < GAF_SPINS) {
#if defined(__x86_64__) || defined(__i386__)
                __builtin_ia32_pause();
#endif
                continue;
            }
            pthread_mutex_lock(&p->mu);
            while (atomic_load_explicit(&p->generation, memory_order_acquire) == seen)
                pthread_cond_wait(&p->wake, &p->mu);
            pthread_mutex_unlock(&p->mu);
        }
        seen = atomic_load_explicit(&p->generation, memory_order_acquire);
        run_share(p, idx);
        if (atomic_fetch_sub_explicit(&p->pending, 1, memory_order_acq_rel) == 1) {
            pthread_mutex_lock(&p->mu);
            pthread_cond_signal(&p->done_cv);
            pthread_mutex_unlock(&p->mu);
        }
    }
    return NULL;
}

static void ensure_workers(gaf_pool_t *p, int want) {
    while (p->n_workers < want && p->n_workers < GAF_MAX_THREADS - 1) {
        int idx = p->n_workers + 1;
        if (pthread_create(&p->threads[p->n_workers], NULL, worker_main,
                           (void *)(size_t)idx) != 0)
            break;
        pthread_detach(p->threads[p->n_workers]);
        p->n_workers++;
    }
}

void gaf_parallel_for(size_t n_items, gaf_range_fn fn, void *ctx, int nthreads) {
    gaf_pool_t *p = &g_pool;
    if (nthreads <= 1 || n_items == 0) {
        fn(0, n_items, ctx);
        return;
    }
    if (nthreads > GAF_MAX_THREADS) nthreads = GAF_MAX_THREADS;
    if (pthread_mutex_trylock(&p->submit) != 0) {
        fn(0, n_items, ctx);
        return;
    }
    ensure_workers(p, nthreads - 1);
    int active = p->n_workers + 1;
    if (active > nthreads) active = nthreads;

    size_t raw = (n_items + (size_t)active - 1) / (size_t)active;
    size_t per = ((raw + GAF_CHUNK_ROUND - 1) / GAF_CHUNK_ROUND) * GAF_CHUNK_ROUND;
    p->fn = fn;
    p->ctx = ctx;
    p->n_items = n_items;
    p->per_thread = per;
    p->active = active;
    /* every spawned worker wakes and decrements, participating or not */
    atomic_store_explicit(&p->pending, p->n_workers, memory_order_release);

    pthread_mutex_lock(&p->mu);
    atomic_fetch_add_explicit(&p->generation, 1, memory_order_release);
    pthread_cond_broadcast(&p->wake);
    pthread_mutex_unlock(&p->mu);

    run_share(p, 0);

    int spins = 0;
    while (atomic_load_explicit(&p->pending, memory_order_acquire) != 0) {
        if (++spins < GAF_SPINS) {
#if defined(__x86_64__) || defined(__i386__)
            __builtin_ia32_pause();
#endif
            continue;
        }
        pthread_mutex_lock(&p->mu);
        while (atomic_load_explicit(&p->pending, memory_order_acquire) != 0)
            pthread_cond_wait(&p->done_cv, &p->mu);
        pthread_mutex_unlock(&p->mu);
    }
    pthread_mutex_unlock(&p->submit);
}
