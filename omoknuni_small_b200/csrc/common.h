// Shared host-side helpers of the C-ABI implementation: thread-local error
// text, status mapping, launch counters.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include "../../include/omoknuni_b200.h"

namespace ob200 {

int set_error(int code, const char* fmt, ...);
int require_device();  // OB200_OK when the current device is compute capability 10.x

struct Counters {
    std::atomic<uint64_t> evals{0}, batches{0}, selections{0}, backups{0}, launches{0};
};
Counters& counters();

inline cudaStream_t as_stream(ob200_stream s) { return reinterpret_cast<cudaStream_t>(s); }

#define OB200_CUDA_OK(expr)                                                              \
    do {                                                                                 \
        cudaError_t _e = (expr);                                                         \
        if (_e != cudaSuccess)                                                           \
            return ::ob200::set_error(OB200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,    \
                                      cudaGetErrorString(_e), __FILE__, __LINE__);       \
    } while (0)

// After a kernel launch: counts it and surfaces a launch error.
#define OB200_LAUNCHED(name)                                                             \
    do {                                                                                 \
        ::ob200::counters().launches.fetch_add(1, std::memory_order_relaxed);            \
        cudaError_t _e = cudaGetLastError();                                             \
        if (_e != cudaSuccess)                                                           \
            return ::ob200::set_error(OB200_ERR_CUDA, "launch of %s failed: %s", name,   \
                                      cudaGetErrorString(_e));                           \
    } while (0)

// Geometry of a board tensor (see the header's "Board tensors" section).
struct BoardGeom {
    int S, GP, slots;
    long long P, Ppad, PT;  // real positions, rounded up to 128, with guards
};
inline BoardGeom board_geom(int S, int B) {
    BoardGeom g;
    g.S = S; g.GP = S + 1; g.slots = g.GP * g.GP;
    g.P = (long long)B * g.slots;
    g.Ppad = (g.P + 127) / 128 * 128;
    g.PT = g.Ppad + 2 * OB200_GUARD;
    return g;
}

}  // namespace ob200
