// Shared host-side helpers of the C-ABI implementation: thread-local error
// text, status mapping, launch counters.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
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

#ifdef __CUDACC__
// Programmatic dependent launch, both ends.  A kernel that starts with OB200_PDL_ENTER() and is launched with
// launch_dependent() may have its CTAs scheduled while the kernel ahead of it in the stream is still running: it
// waits until that kernel has completed and its writes are visible, then lets the kernel behind it be scheduled in
// turn.  Launched any other way the two instructions do nothing.  Every kernel of such a chain must start this way,
// because "completed" is what carries the ordering on to the kernels further ahead.
#define OB200_PDL_ENTER()                                                 \
    do {                                                                  \
        asm volatile("griddepcontrol.wait;" ::: "memory");                \
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   \
    } while (0)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// fp32 -> the 16-bit storage types, round to nearest even (host side: weight packing).
inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
// fp16; magnitudes beyond the largest finite value (65,504) saturate there, as the kernels' stores do.
inline uint16_t f32_to_f16_rne_sat(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);            // NaN
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7BFFu);           // rounds to >= 65,520: saturate
    if (a < 0x33000001u) return sign;                                  // below half the smallest subnormal
    const int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;                          // 24-bit significand
    int shift = e >= -14 ? 13 : 13 + (-14 - e);                        // bits dropped (subnormals drop more)
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    // normal: q has the hidden bit at 1 << 10 (a carry into 1 << 11 bumps the exponent by itself)
    const uint32_t h = e >= -14 ? (((uint32_t)(e + 15) << 10) + (q - 0x400u)) : q;
    return (uint16_t)(sign | h);
}

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
