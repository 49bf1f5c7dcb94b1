// 3x3 convolution layer of the residual tower as an implicit GEMM on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), sm_100a.
//
// GEMM view: M = board positions (128 per tile), N = 64 output channels,
// K = 9 taps x 64 input channels.  Activations are bf16 NHWC board tensors
// (see omoknuni_b200.h): one position = 64 channels = one 128-byte row, boards
// laid on a padded (S+1) x (S+1) grid whose extra column / row and the guard
// rows are zero, so that
//   * a tile plus its halo is one 2-D TMA box (64 channels x rows) that lands
//     in shared memory in the tensor core's 128-byte-swizzled K-major layout;
//   * every tap of the stencil is the SAME shared-memory tile read through a
//     matrix descriptor whose start address is moved by (dy*(S+1)+dx) rows
//     (the 128-byte swizzle is a function of the shared-memory address, so a
//     row-shifted start reads the same bytes TMA wrote).  A tile is fetched
//     once and used by all 9 taps; the zero rows / columns of the tensor are
//     the convolution's padding.
// Weights (BatchNorm folded, bf16, pre-swizzled on the host) stay resident in
// shared memory for the whole launch.  Warp 0 produces (TMA loads), warp 1
// issues the MMAs, warps 2-9 (two groups of 4 warps on alternate tiles) run the
// epilogue: TMEM -> registers, + bias, + residual (brought into the staging tile
// by TMA), ReLU, zero the padding positions, bf16, swizzled staging tile in
// shared memory, one TMA store.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises the
// device error word, leaves its loops, frees its TMEM and returns.
#include "internal.h"
#include "sm100_ptx.cuh"
#include <cstdlib>
#include <cstring>
#include <vector>

namespace ob200 {
namespace {

constexpr int kTileM = 128;             // positions per tile
constexpr int kC = 64;                  // channels in and out (GEMM N and K per tap)
constexpr int kRowBytes = kC * 2;       // one position
constexpr int kHaloMax = OB200_GUARD;   // halo rows kept before / after a tile, at most
constexpr int kStageBytes = (kTileM + 2 * kHaloMax) * kRowBytes;   // 24,576
constexpr int kWBytes = 9 * kC * kRowBytes;                        // 73,728
constexpr int kOutBytes = kTileM * kRowBytes;                      // 16,384
constexpr int kStages = 3;
constexpr int kAccStages = 4;
constexpr int kTmemCols = kAccStages * kC;                         // 256 (power of two)
constexpr int kEpiGroups = 2;
constexpr int kEpiWarps = 4;             // per group: 4 TMEM lane quadrants x (kEpiWarps / 4) slices of the 64 channels
constexpr int kChPerThread = kC / (kEpiWarps / 4);   // channels one epilogue thread handles
constexpr int kThreads = 64 + 32 * kEpiWarps * kEpiGroups;
constexpr int kNumBars = 2 * kStages + 2 * kAccStages + 1 + kEpiGroups;
constexpr int kSmemBytes = kWBytes + kStages * kStageBytes + kEpiGroups * kOutBytes + kNumBars * 8 + kC * 4 + 16 + 1024;

struct ConvParams {
    const uint8_t* w;         // packed, pre-swizzled weights
    const float* bias;        // [64]
    int has_residual;         // the residual tensor map is live
    int* error;               // device error word (0 = fine)
    int P;                    // real positions = B * slots
    int num_tiles;
    int S, GP, slots;
    int halo;                 // halo rows of the TMA box (GP + 1)
    int relu;
};

using namespace ptx;
__device__ __forceinline__ void group_bar(int id) {   // the threads of one epilogue group
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(32 * kEpiWarps) : "memory");
}
// Barrier of one epilogue group that also tells every thread whether any of them reports `bad`:
// the group gives up on a wait as a whole, so no thread is ever left at a barrier its siblings
// have walked away from.
__device__ __forceinline__ bool group_any(int id, bool bad) {
    uint32_t r;
    asm volatile(
        "{\n.reg .pred p, q;\nsetp.ne.b32 q, %2, 0;\nbar.red.or.pred p, %1, %3, q;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(r) : "r"(id), "r"((uint32_t)bad), "r"(32 * kEpiWarps) : "memory");
    return r != 0;
}

// F16: activations and weights are fp16 instead of bf16.
template <bool F16>
__global__ void __launch_bounds__(kThreads, 1)
conv3x3_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
               const __grid_constant__ CUtensorMap res_map, const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    // swizzled tiles need 1024-byte aligned bases
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* w_s = smem;
    uint8_t* a_s = w_s + kWBytes;
    uint8_t* o_s = a_s + kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(o_s + kEpiGroups * kOutBytes);
    float* bias_s = reinterpret_cast<float*>(bars + kNumBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bias_s + kC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kIdesc = make_idesc(F16, kTileM, kC);
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto accfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
    auto accempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + kAccStages + a); };
    const uint32_t w_bar = bar0 + 8u * (2 * kStages + 2 * kAccStages);
    auto res_bar = [&](int g) { return bar0 + 8u * (2 * kStages + 2 * kAccStages + 1 + g); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < kAccStages; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), kEpiWarps); }
        mbar_init(w_bar, 1);
        for (int g = 0; g < kEpiGroups; ++g) mbar_init(res_bar(g), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&in_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&out_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&res_map) : "memory");
    }
    if (threadIdx.x < kC) bias_s[threadIdx.x] = p.bias[threadIdx.x];
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: the next layer's CTAs may start their own prologue
    // (barriers, TMEM, weights) as soon as SMs free up; what depends on the previous
    // kernel's output (activation loads, residual loads, output stores) sits behind
    // griddepcontrol.wait below.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ---------------- producer: TMA loads global -> shared ----------------
        if (lane == 0) {
            mbar_arrive_expect_tx(w_bar, (uint32_t)kWBytes);
            bulk_g2s(smem_u32(w_s), p.w, (uint32_t)kWBytes, w_bar);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            const uint32_t box_bytes = (uint32_t)(kTileM + 2 * p.halo) * kRowBytes;
            int it = 0;
            for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
                const int s = it % kStages;
                const uint32_t ph = (uint32_t)(it / kStages) & 1u;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) {
                    *abort_flag = 1; atomicExch(p.error, 1); break;
                }
                mbar_arrive_expect_tx(full_bar(s), box_bytes);
                tma_load_2d(smem_u32(a_s + s * kStageBytes), &in_map, 0, OB200_GUARD + tile * kTileM - p.halo, full_bar(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(w_bar, 0, abort_flag);
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 2); }
            // Everything that does not change from tile to tile is prepared once: the issuing
            // thread is a single warp lane, so each MMA must cost it a handful of integer
            // instructions, not a descriptor rebuild.
            const uint32_t w_lo = desc_lo(smem_u32(w_s));
            int tap_off[9];
#pragma unroll
            for (int tap = 0; tap < 9; ++tap)
                tap_off[tap] = (p.halo + (tap / 3 - 1) * p.GP + (tap % 3 - 1)) * (kRowBytes >> 4);
            const uint32_t a_base = desc_lo(smem_u32(a_s));
            int s = 0, a = 0;
            uint32_t ph = 0, pa = 0;
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                if (!mbar_wait(accempty_bar(a), pa ^ 1u, abort_flag) || !mbar_wait(full_bar(s), ph, abort_flag)) {
                    *abort_flag = 1; atomicExch(p.error, 2); break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_lo = a_base + (uint32_t)(s * (kStageBytes >> 4));
                const uint32_t d_tmem = tmem_base + (uint32_t)a * kC;
#pragma unroll
                for (int tap = 0; tap < 9; ++tap) {
#pragma unroll
                    for (int ks = 0; ks < kC / 16; ++ks)
                        umma(d_tmem, a_lo + (uint32_t)(tap_off[tap] + ks * 2),
                             w_lo + (uint32_t)(tap * (kC * kRowBytes >> 4) + ks * 2), kIdesc, (tap | ks) ? 1u : 0u);
                }
                umma_commit(empty_bar(s));      // smem stage free once these MMAs have read it
                umma_commit(accfull_bar(a));    // accumulator ready for the epilogue
                if (++s == kStages) { s = 0; ph ^= 1u; }
                if (++a == kAccStages) { a = 0; pa ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> shared -> TMA store ----------------
        // Groups of kEpiWarps warps take alternate tiles.  Within a group a warp owns one TMEM
        // lane quadrant (32 positions; fixed by warp id % 4) and one slice of the 64 channels.
        // With a residual, TMA loads the residual's tile into the group's staging tile while the
        // tile's MMAs run; a thread then reads its own row, adds, and writes the result back in
        // place before the TMA store.
        const int ew = warp - 2;
        const int group = ew / kEpiWarps;
        const int slice = (ew % kEpiWarps) >> 2;     // channels [kChPerThread*slice, +kChPerThread)
        const int q = warp & 3;                      // TMEM lane quadrant this warp may read
        const int row = q * 32 + lane;
        const bool leader = (ew % kEpiWarps) == 0 && lane == 0;
        constexpr int kChunks = kChPerThread / 8;    // 16-byte chunks per thread
        const bool has_res = p.has_residual != 0;
        uint8_t* stage_out = o_s + group * kOutBytes;
        const uint32_t stage_out_u32 = smem_u32(stage_out);
        const float* bias_t = bias_s + slice * kChPerThread;
        uint32_t res_phase = 0;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        int it = group;
        for (int tile = blockIdx.x + group * gridDim.x; tile < p.num_tiles; tile += kEpiGroups * gridDim.x, it += kEpiGroups) {
            const int a = it % kAccStages;
            const uint32_t pa = (uint32_t)(it / kAccStages) & 1u;
            const int pos = tile * kTileM + row;
            bool valid = pos < p.P;
            if (valid) {
                const int rr = pos % p.slots;
                valid = (rr / p.GP < p.S) && (rr % p.GP < p.S);
            }
            if (leader) {
                // the previous store of this group must have finished reading the staging tile
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                if (has_res) {
                    mbar_arrive_expect_tx(res_bar(group), (uint32_t)kOutBytes);
                    tma_load_2d(stage_out_u32, &res_map, 0, OB200_GUARD + tile * kTileM, res_bar(group));
                }
            }
            // Both waits of the tile first, then one vote of the whole group on their outcome (which is also
            // the barrier behind the leader's wait above: the staging tile is free).
            bool good = mbar_wait(accfull_bar(a), pa, abort_flag);
            if (good && has_res) good = mbar_wait(res_bar(group), res_phase, abort_flag);
            if (group_any(1 + 2 * group, !good)) {
                *abort_flag = 1; atomicExch(p.error, 3); break;
            }
            if (has_res) res_phase ^= 1u;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[kChPerThread];
#pragma unroll
            for (int h = 0; h < kChPerThread / 32; ++h)
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kC + slice * kChPerThread + h * 32), r + h * 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accempty_bar(a));
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                // 128-byte swizzle of the staging tile: 16-byte chunk k of row r sits at chunk k ^ (r % 8)
                uint4* slot = reinterpret_cast<uint4*>(stage_out + row * kRowBytes + (((slice * kChunks + c) ^ (row & 7)) << 4));
                uint4 o = make_uint4(0u, 0u, 0u, 0u);
                if (valid) {
                    const uint4 rv = has_res ? *slot : make_uint4(0u, 0u, 0u, 0u);
                    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
                    uint32_t ow[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float r0, r1;
                        unpack2<F16>(rw[j], r0, r1);      // an absent residual reads as +0 in either type
                        float v0 = __uint_as_float(r[c * 8 + 2 * j]) + bias_t[c * 8 + 2 * j] + r0;
                        float v1 = __uint_as_float(r[c * 8 + 2 * j + 1]) + bias_t[c * 8 + 2 * j + 1] + r1;
                        if (p.relu) { v0 = fmaxf(v0, 0.0f); v1 = fmaxf(v1, 0.0f); }
                        ow[j] = pack2<F16>(v0, v1);
                    }
                    o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                }
                *slot = o;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            group_bar(2 + 2 * group);
            if (leader) {
                tma_store_2d(&out_map, 0, OB200_GUARD + tile * kTileM, stage_out_u32);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        // give copies that may still be in flight time to land before the shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
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

// 2-D tensor map over a board tensor: inner dimension the `channels` channels of a position,
// outer dimension `rows` positions; boxes of 64 channels (128 bytes) x box_rows, 128-byte swizzle.
int make_board_tensor_map(const void* base, long long rows, int box_rows, BoardTensorMap* out, int channels) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn)
            return set_error(OB200_ERR_CUDA, "cannot resolve cuTensorMapEncodeTiled from the driver");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    static_assert(sizeof(BoardTensorMap) == sizeof(CUtensorMap), "tensor map size");
    if (((uintptr_t)base & 15) || rows <= 0 || box_rows <= 0 || box_rows > 256 || channels < kC || channels % kC)
        return set_error(OB200_ERR_INVALID,
                         "board tensor map: base must be 16-byte aligned, box rows in [1,256], channels a multiple of 64");
    const cuuint64_t dims[2] = {(cuuint64_t)channels, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)channels * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kC, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(OB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return OB200_OK;
}

int conv_halo_rows(int S) { return S + 2; }   // |dy*(S+1)+dx| <= S+2 rows before / after a tile

int launch_conv3x3_maps(const BoardTensorMap& in_map, const BoardTensorMap& out_map, const BoardTensorMap* res_map,
                        const void* packed_w, const float* bias, int B, int S, int relu, cudaStream_t st, int dtype) {
    if (!packed_w || !bias || B <= 0) return set_error(OB200_ERR_INVALID, "conv3x3: null pointer or empty batch");
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "conv3x3: bad dtype %d", dtype);
    if (S < 1 || conv_halo_rows(S) > kHaloMax)
        return set_error(OB200_ERR_UNSUPPORTED, "conv3x3: board_size %d outside [1, %d]", S, kHaloMax - 2);
    if ((uintptr_t)packed_w & 15) return set_error(OB200_ERR_INVALID, "conv3x3: weights must be 16-byte aligned");
    if (int rc = require_device()) return rc;
    static bool configured[64][2] = {{false, false}};
    int dev = 0;
    OB200_CUDA_OK(cudaGetDevice(&dev));
    auto kernel = dtype == OB200_DTYPE_F16 ? conv3x3_kernel<true> : conv3x3_kernel<false>;
    if (dev < 0 || dev >= 64 || !configured[dev][dtype]) {
        OB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        if (dev >= 0 && dev < 64) configured[dev][dtype] = true;
    }
    int sms = 0;
    OB200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const BoardGeom g = board_geom(S, B);
    ConvParams p;
    p.w = static_cast<const uint8_t*>(packed_w); p.bias = bias; p.has_residual = res_map != nullptr;
    p.error = device_error_word();
    if (!p.error) return set_error(OB200_ERR_CUDA, "conv3x3: cannot resolve the device error word");
    p.P = (int)g.P; p.num_tiles = (int)(g.Ppad / kTileM); p.S = S; p.GP = g.GP; p.slots = g.slots;
    p.halo = conv_halo_rows(S); p.relu = relu;
    const int grid = p.num_tiles < sms ? p.num_tiles : sms;   // one persistent CTA per SM
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, *reinterpret_cast<const CUtensorMap*>(&in_map),
                                     *reinterpret_cast<const CUtensorMap*>(&out_map),
                                     *reinterpret_cast<const CUtensorMap*>(res_map ? res_map : &out_map), p));
    OB200_LAUNCHED("conv3x3_kernel");
    return OB200_OK;
}

}  // namespace ob200

using namespace ob200;

extern "C" {

int ob200_launch_conv3x3(const void* in, const void* packed_w, const float* bias, const void* residual,
                         void* out, int32_t B, int32_t board_size, int32_t cin, int32_t cout, int32_t relu,
                         ob200_stream stream) {
    return ob200_launch_conv3x3_dt(in, packed_w, bias, residual, out, B, board_size, cin, cout, relu, OB200_DTYPE_BF16, stream);
}

int ob200_launch_conv3x3_dt(const void* in, const void* packed_w, const float* bias, const void* residual,
                            void* out, int32_t B, int32_t board_size, int32_t cin, int32_t cout, int32_t relu,
                            int32_t dtype, ob200_stream stream) {
    if (!in || !out || B <= 0) return set_error(OB200_ERR_INVALID, "ob200_launch_conv3x3: null pointer or empty batch");
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "ob200_launch_conv3x3: bad dtype %d", dtype);
    if (conv_wide_covers(cin, cout)) {
        if (board_size < 1 || conv_halo_rows(board_size) > kHaloMax)
            return set_error(OB200_ERR_UNSUPPORTED, "ob200_launch_conv3x3: board_size %d outside [1, %d]", board_size, kHaloMax - 2);
        const BoardGeom gw = board_geom(board_size, B);
        BoardTensorMap wim, wom;
        if (int rc = make_board_tensor_map(in, gw.PT, conv_wide_box_rows(), &wim, cin)) return rc;
        if (int rc = make_board_tensor_map(out, gw.PT, kTileM, &wom, cout)) return rc;
        BoardTensorMap wrm;
        if (residual)
            if (int rc = make_board_tensor_map(residual, gw.PT, kTileM, &wrm, cout)) return rc;
        return launch_conv_wide_maps(wim, wom, residual ? &wrm : nullptr, packed_w, bias, B, board_size, cin, cout, 9, relu,
                                     as_stream(stream), nullptr, dtype);
    }
    if (cin != kC || cout != kC)
        return set_error(OB200_ERR_UNSUPPORTED,
                         "ob200_launch_conv3x3: covered shapes are 64 -> 64 and {64,128,192,256} -> {128,256}; got %d -> %d", cin, cout);
    if (board_size < 1 || conv_halo_rows(board_size) > kHaloMax)
        return set_error(OB200_ERR_UNSUPPORTED, "ob200_launch_conv3x3: board_size %d outside [1, %d]", board_size, kHaloMax - 2);
    const BoardGeom g = board_geom(board_size, B);
    BoardTensorMap im, om;
    if (int rc = make_board_tensor_map(in, g.PT, kTileM + 2 * conv_halo_rows(board_size), &im)) return rc;
    if (int rc = make_board_tensor_map(out, g.PT, kTileM, &om)) return rc;
    BoardTensorMap rm;
    if (residual)
        if (int rc = make_board_tensor_map(residual, g.PT, kTileM, &rm)) return rc;
    return launch_conv3x3_maps(im, om, residual ? &rm : nullptr, packed_w, bias, B, board_size, relu, as_stream(stream), dtype);
}

int64_t ob200_packed_conv3x3_bytes(int32_t cin, int32_t cout) {
    if (conv_wide_covers(cin, cout)) return (int64_t)conv_wide_packed_bytes(cin, cout, 9);
    if (cin != kC || cout != kC) return 0;
    return (int64_t)kWBytes;
}

// Packed image: [tap = ky*3+kx][cout][cin] bf16 (or fp16), one 128-byte row per output channel and
// tap, its 16-byte chunks (8 input channels) permuted by the 128-byte swizzle
// (chunk j of row r stored at chunk j ^ (r % 8)) — the K-major shared-memory operand
// layout of the tensor core, ready for a plain bulk copy.
int ob200_pack_conv3x3_weights(const float* w_oihw, const float* scale, int32_t cout, int32_t cin_real,
                               int32_t cin, void* packed_out) {
    return ob200_pack_conv3x3_weights_dt(w_oihw, scale, cout, cin_real, cin, OB200_DTYPE_BF16, packed_out);
}

int ob200_pack_conv3x3_weights_dt(const float* w_oihw, const float* scale, int32_t cout, int32_t cin_real,
                                  int32_t cin, int32_t dtype, void* packed_out) {
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16)
        return set_error(OB200_ERR_INVALID, "ob200_pack_conv3x3_weights: bad dtype %d", dtype);
    if (conv_wide_covers(cin, cout)) return conv_wide_pack(w_oihw, scale, cout, cin_real, cin, 9, packed_out, dtype);
    if (!w_oihw || !packed_out || cout != kC || cin != kC || cin_real <= 0 || cin_real > cin)
        return set_error(OB200_ERR_INVALID, "ob200_pack_conv3x3_weights: covered shapes are 64 -> 64 and {64,128,192,256} -> {128,256}; got cout %d, cin_real %d, cin %d",
                         cout, cin_real, cin);
    uint16_t* o = static_cast<uint16_t*>(packed_out);
    for (int tap = 0; tap < 9; ++tap)
        for (int co = 0; co < kC; ++co)
            for (int ci = 0; ci < kC; ++ci) {
                float v = 0.0f;
                if (ci < cin_real) v = w_oihw[((size_t)co * cin_real + ci) * 9 + tap] * (scale ? scale[co] : 1.0f);
                const size_t byte = (size_t)tap * kC * kRowBytes + (size_t)co * kRowBytes + ((((ci >> 3) ^ (co & 7))) << 4) + (ci & 7) * 2;
                o[byte / 2] = dtype == OB200_DTYPE_F16 ? f32_to_f16_rne_sat(v) : f32_to_bf16_rne(v);
            }
    return OB200_OK;
}

// A wait that nothing will ever satisfy, with a small limit: the same bounded-wait-then-report
// path the kernels take when a copy or a tensor-core completion never arrives.
__global__ void bounded_wait_probe_kernel(int* error_word, int limit) {
    __shared__ __align__(8) uint64_t bar;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    bool done = false;
    for (int i = 0; i < limit && !done; ++i) done = mbar_test(smem_u32(&bar), 0);
    if (!done) atomicExch(error_word, 9);
}

int ob200_debug_bounded_wait(int32_t spin_limit, ob200_stream stream) {
    if (spin_limit < 1 || spin_limit > (1 << 20))
        return set_error(OB200_ERR_INVALID, "ob200_debug_bounded_wait: spin_limit %d outside [1, 2^20]", spin_limit);
    if (int rc = require_device()) return rc;
    int* w = device_error_word();
    if (!w) return set_error(OB200_ERR_CUDA, "cannot resolve the device error word");
    bounded_wait_probe_kernel<<<1, 1, 0, as_stream(stream)>>>(w, spin_limit);
    OB200_LAUNCHED("bounded_wait_probe_kernel");
    return OB200_OK;
}

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
