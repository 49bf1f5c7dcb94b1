// Inline-PTX wrappers shared by the tensor-core kernels of this library (sm_100a):
// mbarriers with bounded waits, bulk / tensor-map copies, tcgen05 matrix and
// instruction descriptors, tcgen05.mma issue / commit, TMEM loads, and the two
// 16-bit storage types of a board tensor (bf16, fp16).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace ob200 {
namespace ptx {

constexpr uint32_t kSpinLimit = 1u << 22;   // polls before a wait gives up (tens of milliseconds)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 255) == 255 && *abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(src) : "memory");
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups
// 1024 bytes apart (stride byte offset); the leading byte offset is not used by swizzled K-major
// layouts and is encoded as 1.  The swizzle is a function of the shared-memory address itself
// (16-byte chunk index XOR address bits 7-9), so a descriptor may start at any 128-byte row of a
// tile that was written with the same swizzle; the base-offset field stays 0 (measured: a non-zero
// base offset on a row-shifted start gives wrong products).  Split in two words so that the
// issuing thread only adds to the low one.
constexpr uint32_t kDescHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1u << 16); }

// kind::f16 instruction descriptor: fp32 accumulate (bit 4), operand format of A (bits 7-9) and B
// (bits 10-12): 0 = fp16, 1 = bf16; both operands K-major; N >> 3 at bit 17, M >> 4 at bit 24.
// Both formats run at the same rate.
__host__ __device__ constexpr uint32_t make_idesc(bool f16, int M, int N) {
    return (1u << 4) | (f16 ? 0u : ((1u << 7) | (1u << 10))) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\n"
        "mov.b64 da, {%1, %3};\nmov.b64 db, {%2, %3};\n"
        "setp.ne.b32 p, %5, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

// ---- the 16-bit storage type of a board tensor: bf16 (F16 = false) or fp16 (F16 = true) ----
// Two stored values (low half first) -> fp32.
template <bool F16>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
    if (F16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        lo = f.x; hi = f.y;
    } else {
        lo = __uint_as_float(w << 16); hi = __uint_as_float(w & 0xFFFF0000u);   // bf16 -> fp32 is a 16-bit shift
    }
}
// fp32 -> two stored values, round to nearest even.  fp16 saturates to the largest finite value
// (65,504) instead of overflowing to infinity, so an activation that outgrows the format clamps.
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t d;
    if (F16) asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    else { const __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi); d = *reinterpret_cast<const uint32_t*>(&h2); }
    return d;
}
// relu, then as pack2
template <bool F16>
__device__ __forceinline__ uint32_t pack2_relu(float lo, float hi) {
    uint32_t d;
    if (F16) asm("cvt.rn.relu.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    else asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
// One value of a board tensor from fp32 (encoders; not a hot path): runtime choice of the type.
__device__ __forceinline__ uint16_t store16(float v, int f16) {
    if (f16) { const __half h = __float2half_rn(v); return *reinterpret_cast<const uint16_t*>(&h); }
    const __nv_bfloat16 h = __float2bfloat16(v);
    return *reinterpret_cast<const uint16_t*>(&h);
}

}  // namespace ptx
}  // namespace ob200
