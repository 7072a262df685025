/* Linux stand-in for the one call the reference's engine loader makes into <mach-o/dyld.h>
 * (qwasar.c:1959, the path of the running executable).  TEST INFRASTRUCTURE: used only when
 * oracle/Makefile builds the reference's loader here; nothing in the product includes it. */
#ifndef QW_SHIM_MACHO_DYLD_H
#define QW_SHIM_MACHO_DYLD_H
#include <stdint.h>
#include <unistd.h>
static inline int _NSGetExecutablePath(char *buf, uint32_t *cap) {
    const ssize_t n = readlink("/proc/self/exe", buf, *cap ? *cap - 1 : 0);
    if (n < 0) return -1;
    buf[n] = 0;
    return 0;
}
#endif
