/* Build stub for the oracle/_ref recipe only: the reference's
 * include/utils/thread_local_allocator.h includes <mimalloc.h>, which is not
 * installed.  Map the three calls it uses onto libc. */
#ifndef OB200_ORACLE_MIMALLOC_STUB_H
#define OB200_ORACLE_MIMALLOC_STUB_H
#include <stdlib.h>
static inline void* mi_malloc(size_t n) { return malloc(n); }
static inline void* mi_aligned_alloc(size_t align, size_t n) {
    void* p = 0; if (align < sizeof(void*)) align = sizeof(void*);
    return posix_memalign(&p, align, n) == 0 ? p : 0;
}
static inline void mi_free(void* p) { free(p); }
#endif
