/* Device-side stand-in for <barrier.h>: a counting barrier over the tasklet threads.
 * TEST INFRASTRUCTURE ONLY (see ../dpu.h). */
#ifndef LUTAMM_SHIM_BARRIER_H
#define LUTAMM_SHIM_BARRIER_H
#include <pthread.h>
typedef struct {
    pthread_mutex_t mu;
    pthread_cond_t cv;
    unsigned count, waiting, generation;
} shim_barrier_t;
#define BARRIER_INIT(name, n) shim_barrier_t name = {PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER, (n), 0, 0}
static inline void barrier_wait(shim_barrier_t* b) {
    pthread_mutex_lock(&b->mu);
    const unsigned gen = b->generation;
    if (++b->waiting == b->count) {
        b->waiting = 0;
        ++b->generation;
        pthread_cond_broadcast(&b->cv);
    } else {
        while (gen == b->generation) pthread_cond_wait(&b->cv, &b->mu);
    }
    pthread_mutex_unlock(&b->mu);
}
#endif
