/* Linux stand-in for <sys/sysctl.h> as the reference's engine loader uses it (qwasar.c:605, 615:
 * total memory and memory pressure by name).  Every query answers "not available", which the
 * loader treats as "no reason to refuse the model".  TEST INFRASTRUCTURE, see mach-o/dyld.h. */
#ifndef QW_SHIM_SYS_SYSCTL_H
#define QW_SHIM_SYS_SYSCTL_H
#include <stddef.h>
static inline int sysctlbyname(const char *name, void *oldp, size_t *oldlenp, void *newp, size_t newlen) {
    (void)name; (void)oldp; (void)oldlenp; (void)newp; (void)newlen;
    return -1;
}
#endif
