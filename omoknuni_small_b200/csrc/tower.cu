// 3x3 convolution layer of the residual tower as an implicit GEMM on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), sm_100a.
//
// GEMM view: M = board positions (128 per tile), N = 64 output channels,
// K = 9 taps x C_in.  Activations are board tensors (channels blocked by 8,
// positions on a padded (S+1)x(S+1) grid, see omoknuni_b200.h), so that
//   * a tile plus its halo is, per channel block, ONE contiguous run of
//     16-byte position records: the producer warp fetches it with a handful
//     of 1-D bulk async copies (cp.async.bulk, completion on an mbarrier);
//   * in shared memory the run is already the tensor core's no-swizzle
//     K-major layout (8 positions x 16 bytes = one 128-byte core matrix,
//     next 8 positions 128 bytes further, next channel block one run
//     further), so every tap of the 3x3 stencil is the SAME buffer read
//     through a matrix descriptor whose start address is shifted by
//     (dy*(S+1)+dx) records.  The tile is brought on chip once and used by
//     all 9 taps; zero columns/rows/guards in the tensor are the padding.
// Weights (BatchNorm folded, bf16) stay resident in shared memory for the
// whole launch.  Warp 0 produces (bulk copies), warp 1 issues the MMAs, warps
// 2-9 (two warpgroups on alternate tiles) run the epilogue (TMEM -> registers, + bias, + residual, ReLU, zero the
// padding positions, bf16, 16-byte coalesced stores).  Four shared-memory
// stages and four TMEM accumulators decouple the three roles.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises the
// error word, leaves its loops, frees its TMEM and returns.
#include "common.h"
#include <cuda_bf16.h>
#include <cstring>
#include <vector>

namespace ob200 {
namespace {

constexpr int kTileM = 128;             // positions per tile
constexpr int kCout = 64;               // output channels (GEMM N)
constexpr int kHaloMax = OB200_GUARD;   // smem rows kept before / after a tile
constexpr int kTileRows = kTileM + 2 * kHaloMax;       // 192 records per channel block
constexpr int kChunkBytes = kTileRows * 16;             // 3072
constexpr int kStages = 4;
constexpr int kAccStages = 4;
constexpr int kTmemCols = kAccStages * kCout;           // 256 (power of two)
constexpr int kEpiGroups = 2;           // epilogue warpgroups, alternating tiles
constexpr int kThreads = 64 + 128 * kEpiGroups;
constexpr uint32_t kSpinLimit = 1u << 22;

struct ConvParams {
    const uint8_t* in;        // board tensor, cin channels
    const uint8_t* w;         // packed weights
    const float* bias;        // [64]
    const uint8_t* residual;  // board tensor, 64 channels, or null
    uint8_t* out;             // board tensor, 64 channels
    int* error;               // device error word (0 = fine)
    long long PT;             // positions per channel block incl. guards
    long long P;              // real positions = B * slots
    int num_tiles;
    int S, GP, slots;
    int relu;
};

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
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) {
            __nanosleep(32);
            if ((i & 1023) == 0 && *abort_flag) return false;
        }
    }
    return false;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor, no swizzle, K-major: core matrices of
// 8 rows x 16 bytes stored as 128 contiguous bytes; `lbo` = bytes between the
// two K-adjacent core matrices of one MMA (K = 16), `sbo` = bytes between
// 8-row groups along M / N.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, M = 128, N = 64.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kCout >> 3) << 17) |
                            ((uint32_t)(kTileM >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate) : "memory");
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

struct alignas(16) Pack8 { __nv_bfloat162 v[4]; };

template <int CC>  // input channel blocks of 8 (8 for 64 channels, 4 for the 32-channel stem)
__global__ void __launch_bounds__(kThreads, 1) conv3x3_kernel(const ConvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kWBytes = 9 * CC * kCout * 16;
    constexpr int kStageBytes = CC * kChunkBytes;
    uint8_t* w_s = smem;
    uint8_t* a_s = smem + kWBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(a_s + kStages * kStageBytes);
    // bars: [0,4) full, [4,8) empty, [8,12) accumulator full, [12,16) accumulator empty, 16 weights
    float* bias_s = reinterpret_cast<float*>(bars + 17);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bias_s + kCout);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (4 + s); };
    auto accfull_bar = [&](int a) { return bar0 + 8u * (8 + a); };
    auto accempty_bar = [&](int a) { return bar0 + 8u * (12 + a); };
    const uint32_t w_bar = bar0 + 8u * 16;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < kAccStages; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), 4); }
        mbar_init(w_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < kCout) bias_s[threadIdx.x] = p.bias[threadIdx.x];
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int halo = p.GP + 1;
    const uint32_t chunk_copy_bytes = (uint32_t)(kTileM + 2 * halo) * 16u;

    if (warp == 0) {
        // ---------------- producer: bulk copies global -> shared ----------------
        if (lane == 0) {
            mbar_arrive_expect_tx(w_bar, (uint32_t)kWBytes);
            bulk_g2s(smem_u32(w_s), p.w, (uint32_t)kWBytes, w_bar);
            int it = 0;
            for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
                const int s = it % kStages;
                const uint32_t ph = (uint32_t)(it / kStages) & 1u;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) {
                    *abort_flag = 1; atomicExch(p.error, 1); break;
                }
                mbar_arrive_expect_tx(full_bar(s), chunk_copy_bytes * CC);
                const long long first = (long long)OB200_GUARD + (long long)tile * kTileM - halo;
                const uint32_t dst0 = smem_u32(a_s + s * kStageBytes) + (uint32_t)(kHaloMax - halo) * 16u;
#pragma unroll
                for (int c = 0; c < CC; ++c)
                    bulk_g2s(dst0 + c * kChunkBytes, p.in + ((long long)c * p.PT + first) * 16, chunk_copy_bytes,
                             full_bar(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(w_bar, 0, abort_flag);
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 2); }
            int it = 0;
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
                const int s = it % kStages, a = it % kAccStages;
                const uint32_t ph = (uint32_t)(it / kStages) & 1u, pa = (uint32_t)(it / kAccStages) & 1u;
                if (!mbar_wait(accempty_bar(a), pa ^ 1u, abort_flag) || !mbar_wait(full_bar(s), ph, abort_flag)) {
                    *abort_flag = 1; atomicExch(p.error, 2); break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_base = smem_u32(a_s + s * kStageBytes) + (uint32_t)kHaloMax * 16u;
                const uint32_t w_base = smem_u32(w_s);
                const uint32_t d_tmem = tmem_base + (uint32_t)a * kCout;
                uint32_t acc = 0;
#pragma unroll
                for (int tap = 0; tap < 9; ++tap) {
                    const int shift = (tap / 3 - 1) * p.GP + (tap % 3 - 1);
#pragma unroll
                    for (int ks = 0; ks < CC / 2; ++ks) {
                        const uint64_t ad = make_desc(a_base + (uint32_t)(2 * ks) * kChunkBytes + (uint32_t)(shift * 16),
                                                      kChunkBytes, 128);
                        const uint64_t bd = make_desc(w_base + (uint32_t)((tap * CC + 2 * ks) * kCout * 16),
                                                      kCout * 16, 128);
                        umma(d_tmem, ad, bd, acc);
                        acc = 1;
                    }
                }
                umma_commit(empty_bar(s));      // smem stage free once these MMAs have read it
                umma_commit(accfull_bar(a));    // accumulator ready for the epilogue
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> global ----------------
        // Two warpgroups take alternate tiles.  A thread owns one position (TMEM lane) and
        // all 64 channels; the residual is fetched before the wait on the accumulator so
        // that its latency hides behind the MMAs of the tile.
        const int q = warp & 3;                 // TMEM lane quadrant this warp may read
        const int group = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const uint8_t* __restrict__ resid = p.residual;
        uint8_t* __restrict__ outp = p.out;
        const int P = (int)p.P;
        int it = group;
        for (int tile = blockIdx.x + group * gridDim.x; tile < p.num_tiles; tile += kEpiGroups * gridDim.x, it += kEpiGroups) {
            const int a = it % kAccStages;
            const uint32_t pa = (uint32_t)(it / kAccStages) & 1u;
            const int pos = tile * kTileM + row;
            bool valid = pos < P;
            if (valid) {
                const int rr = pos % p.slots;
                valid = (rr / p.GP < p.S) && (rr % p.GP < p.S);
            }
            const long long rec = (long long)OB200_GUARD + pos;
            uint4 rs[kCout / 8];
            if (resid != nullptr && valid) {
#pragma unroll
                for (int c = 0; c < kCout / 8; ++c)
                    rs[c] = __ldg(reinterpret_cast<const uint4*>(resid + ((long long)c * p.PT + rec) * 16));
            } else {
#pragma unroll
                for (int c = 0; c < kCout / 8; ++c) rs[c] = make_uint4(0u, 0u, 0u, 0u);
            }
            if (!mbar_wait(accfull_bar(a), pa, abort_flag)) {
                *abort_flag = 1; atomicExch(p.error, 3); break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[64];
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)a * kCout;
            tmem_ld32(taddr, r);
            tmem_ld32(taddr + 32, r + 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accempty_bar(a));
#pragma unroll
            for (int c = 0; c < kCout / 8; ++c) {
                uint4 o = make_uint4(0u, 0u, 0u, 0u);
                if (valid) {
                    const uint32_t rw[4] = {rs[c].x, rs[c].y, rs[c].z, rs[c].w};
                    uint32_t ow[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // bf16 -> fp32 is a 16-bit shift
                        float v0 = __uint_as_float(r[c * 8 + 2 * j]) + bias_s[c * 8 + 2 * j] + __uint_as_float(rw[j] << 16);
                        float v1 = __uint_as_float(r[c * 8 + 2 * j + 1]) + bias_s[c * 8 + 2 * j + 1] + __uint_as_float(rw[j] & 0xFFFF0000u);
                        if (p.relu) { v0 = fmaxf(v0, 0.0f); v1 = fmaxf(v1, 0.0f); }
                        const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                        ow[j] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                }
                *reinterpret_cast<uint4*>(outp + ((long long)c * p.PT + rec) * 16) = o;
            }
        }
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        // give bulk copies that may still be in flight time to land before the CTA's
        // shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

template <int CC>
constexpr int conv_smem_bytes() {
    return 9 * CC * kCout * 16 + kStages * CC * kChunkBytes + 17 * 8 + kCout * 4 + 16;
}

inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

}  // namespace
}  // namespace ob200

namespace ob200 {

// One error word per device, raised by kernels whose bounded waits run out.
__device__ int g_device_error;

int* device_error_word() {
    static int* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cached[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_device_error) != cudaSuccess) return nullptr;
        cached[dev] = static_cast<int*>(ptr);
    }
    return cached[dev];
}

template <int CC>
static int launch_conv(const ConvParams& p, cudaStream_t st) {
    static bool configured[64] = {false};
    int dev = 0;
    OB200_CUDA_OK(cudaGetDevice(&dev));
    constexpr int smem = conv_smem_bytes<CC>();
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        OB200_CUDA_OK(cudaFuncSetAttribute(conv3x3_kernel<CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    int sms = 0;
    OB200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int grid = p.num_tiles < sms ? p.num_tiles : sms;   // one persistent CTA per SM
    conv3x3_kernel<CC><<<grid, kThreads, smem, st>>>(p);
    OB200_LAUNCHED("conv3x3_kernel");
    return OB200_OK;
}

// stride_positions: positions between channel blocks of all three tensors; 0 = the
// compact tensors for exactly B boards.
int launch_conv3x3(const void* in, const void* packed_w, const float* bias, const void* residual, void* out,
                   int B, int S, int cin, int cout, int relu, long long stride_positions, cudaStream_t st) {
    if (!in || !packed_w || !bias || !out || B <= 0)
        return set_error(OB200_ERR_INVALID, "conv3x3: null pointer or empty batch");
    if (cout != kCout || (cin != 32 && cin != 64))
        return set_error(OB200_ERR_UNSUPPORTED, "conv3x3: this build covers cout = 64 and cin in {32, 64}; got cin %d cout %d",
                         cin, cout);
    if (S < 1 || S + 2 > kHaloMax)
        return set_error(OB200_ERR_UNSUPPORTED, "conv3x3: board_size %d outside [1, %d]", S, kHaloMax - 2);
    if (((uintptr_t)in | (uintptr_t)packed_w | (uintptr_t)out | (uintptr_t)residual) & 15)
        return set_error(OB200_ERR_INVALID, "conv3x3: tensors must be 16-byte aligned");
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(S, B);
    ConvParams p;
    p.in = static_cast<const uint8_t*>(in); p.w = static_cast<const uint8_t*>(packed_w); p.bias = bias;
    p.residual = static_cast<const uint8_t*>(residual); p.out = static_cast<uint8_t*>(out);
    p.error = device_error_word();
    if (!p.error) return set_error(OB200_ERR_CUDA, "conv3x3: cannot resolve the device error word");
    if (stride_positions && stride_positions < g.PT)
        return set_error(OB200_ERR_INVALID, "conv3x3: tensor stride smaller than the batch needs");
    p.PT = stride_positions ? stride_positions : g.PT; p.P = g.P; p.num_tiles = (int)(g.Ppad / kTileM); p.S = S; p.GP = g.GP; p.slots = g.slots; p.relu = relu;
    return cin == 64 ? launch_conv<8>(p, st) : launch_conv<4>(p, st);
}

}  // namespace ob200

using namespace ob200;

extern "C" {

int ob200_launch_conv3x3(const void* in, const void* packed_w, const float* bias, const void* residual,
                         void* out, int32_t B, int32_t board_size, int32_t cin, int32_t cout, int32_t relu,
                         ob200_stream stream) {
    return launch_conv3x3(in, packed_w, bias, residual, out, B, board_size, cin, cout, relu, 0, as_stream(stream));
}

int64_t ob200_packed_conv3x3_bytes(int32_t cin, int32_t cout) {
    if (cin <= 0 || cout <= 0 || (cin & 7)) return 0;
    return (int64_t)9 * cin * cout * 2;
}

// Packed image: [tap = ky*3+kx][cin/8][cout][8] bf16 — per tap and per block
// of 8 input channels, `cout` rows of 16 bytes: the K-major no-swizzle
// operand layout of the tensor core with the output channel as the row.
int ob200_pack_conv3x3_weights(const float* w_oihw, const float* scale, int32_t cout, int32_t cin_real,
                               int32_t cin, void* packed_out) {
    if (!w_oihw || !packed_out || cout <= 0 || cin_real <= 0 || cin < cin_real || (cin & 7))
        return set_error(OB200_ERR_INVALID, "ob200_pack_conv3x3_weights: bad arguments (cout %d, cin_real %d, cin %d)",
                         cout, cin_real, cin);
    uint16_t* o = static_cast<uint16_t*>(packed_out);
    const int chunks = cin / 8;
    for (int tap = 0; tap < 9; ++tap)
        for (int cb = 0; cb < chunks; ++cb)
            for (int co = 0; co < cout; ++co)
                for (int j = 0; j < 8; ++j) {
                    const int ci = cb * 8 + j;
                    float v = 0.0f;
                    if (ci < cin_real) v = w_oihw[((size_t)co * cin_real + ci) * 9 + tap] * (scale ? scale[co] : 1.0f);
                    o[(((size_t)tap * chunks + cb) * cout + co) * 8 + j] = f32_to_bf16_rne(v);
                }
    return OB200_OK;
}

/* Reads and clears the device error word of the current device (synchronises
 * the device).  0 = no kernel gave up on a wait. */
int ob200_device_error_code(int32_t* code_out) {
    if (!code_out) return set_error(OB200_ERR_INVALID, "ob200_device_error_code: null output");
    if (int rc = require_device()) return rc;
    int* w = device_error_word();
    if (!w) return set_error(OB200_ERR_CUDA, "cannot resolve the device error word");
    int v = 0;
    OB200_CUDA_OK(cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) { int z = 0; OB200_CUDA_OK(cudaMemcpy(w, &z, sizeof(int), cudaMemcpyHostToDevice)); }
    *code_out = v;
    return OB200_OK;
}

}  // extern "C"
