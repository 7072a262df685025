/* Linux stand-in for the part of libdispatch the reference's Flash-Next graph uses
 * (qwasar_flash_graph.c:52, 170-180, 293, 321-327: a group of engram-table gathers run beside the
 * encoding, and a parallel-for).  Here every task runs at once on the calling thread, which keeps
 * the results and drops only the overlap.  TEST INFRASTRUCTURE, see mach-o/dyld.h. */
#ifndef QW_SHIM_DISPATCH_H
#define QW_SHIM_DISPATCH_H
#include <stddef.h>
#include <stdint.h>
typedef void *dispatch_group_t;
typedef void *dispatch_queue_t;
typedef uint64_t dispatch_time_t;
#define DISPATCH_TIME_FOREVER (~(dispatch_time_t)0)
#define QOS_CLASS_USER_INITIATED 0x19
static inline dispatch_queue_t dispatch_get_global_queue(long identifier, unsigned long flags) { (void)identifier; (void)flags; return (dispatch_queue_t)0; }
static inline dispatch_group_t dispatch_group_create(void) { static int one; return &one; }
static inline void dispatch_group_async_f(dispatch_group_t g, dispatch_queue_t q, void *ctx, void (*fn)(void *)) { (void)g; (void)q; fn(ctx); }
static inline long dispatch_group_wait(dispatch_group_t g, dispatch_time_t t) { (void)g; (void)t; return 0; }
static inline void dispatch_apply_f(size_t n, dispatch_queue_t q, void *ctx, void (*fn)(void *, size_t)) { (void)q; for (size_t i = 0; i < n; i++) fn(ctx, i); }
static inline void dispatch_release(void *obj) { (void)obj; }
#endif
