/* host_backend.c -- TEST INFRASTRUCTURE.  The buffer half of the reference's backend boundary
 * (qwasar_gpu.h:18-37) over plain host memory, so that the reference's engine loader (qwasar.c)
 * and its CPU forward (qwasar_flash_cpu.c) link and run on a machine without any GPU: a "buffer"
 * is a host pointer, qw_buf_wrap keeps the caller's mapping, and no op exists.  Used by
 * flash_toy_cpu.c to reproduce the toy fixture's oracle.json on the CPU. */
#include "qwasar_gpu.h"

#include <stdlib.h>
#include <string.h>

struct qw_buf_s { void *p; size_t len; int own; };

bool qw_gpu_init(char *err, size_t errcap) { (void)err; (void)errcap; return true; }
void qw_gpu_shutdown(void) {}
const char *qw_gpu_name(void) { return "host memory (no device)"; }
uint64_t qw_gpu_working_set_limit(void) { return (uint64_t)1 << 40; }
uint64_t qw_gpu_max_buffer_length(void) { return (uint64_t)1 << 40; }
qw_buf qw_buf_wrap(void *ptr, size_t len) {
    qw_buf b = calloc(1, sizeof *b);
    b->p = ptr; b->len = len;
    return b;
}
qw_buf qw_buf_alloc(size_t len) {
    qw_buf b = calloc(1, sizeof *b);
    b->p = calloc(len ? len : 1, 1); b->len = len; b->own = 1;
    return b;
}
void qw_buf_free(qw_buf b) { if (b) { if (b->own) free(b->p); free(b); } }
void *qw_buf_contents(qw_buf b) { return b ? b->p : NULL; }
size_t qw_buf_length(qw_buf b) { return b ? b->len : 0; }
qw_residency qw_residency_new(qw_buf *bufs, int32_t n) { (void)bufs; (void)n; return NULL; }
void qw_residency_free(qw_residency r) { (void)r; }
