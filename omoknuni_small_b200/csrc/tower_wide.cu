// 3x3 (or 1x1) convolution for towers of 128 / 256 channels as an implicit GEMM
// on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), sm_100a.
//
// GEMM view of one work unit: M = 256 board positions (two 128-row MMA tiles),
// N = 128 output channels, K = taps x C_in.  Activations are bf16 NHWC board
// tensors (see omoknuni_b200.h) read in 64-channel slices: a slice of a position
// is one 128-byte row, so a unit's positions plus the stencil halo arrive as two
// 2-D TMA boxes (64 channels x 160 rows) in the tensor core's 128-byte-swizzled
// K-major layout, and every tap is the same shared-memory tile read through a
// matrix descriptor whose start is moved by (dy*(S+1)+dx) rows.  With 128 or 256
// channels a layer's weights (288 KB / 1.1 MB) do not fit in shared memory: they
// stream from L2 as 16 KB blocks (128 output channels x 64 input channels of one
// tap, pre-swizzled on the host) through a 6-deep ring; each block feeds the MMAs
// of both tiles of the unit, which halves the weight traffic per position, and
// N = 128 keeps the shared-memory operand reads of an MMA (8 KB) within what the
// tensor core consumes per instruction.
//
// Warp 0 loads activations, warp 2 loads weights, warp 1 issues the MMAs, warps
// 4-11 (one group of 4 per tile of the unit) run the epilogue: TMEM -> registers,
// + bias, + residual (brought into the staging tile by TMA), ReLU, zero the
// padding positions, bf16, swizzled staging tile, TMA store - 64 channels at a
// time.  Accumulators are double-buffered (2 units x 2 tiles x 128 columns = all
// 512 TMEM columns), so the epilogue of a unit overlaps the MMAs of the next.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises the
// device error word, leaves its loops, frees its TMEM and returns.
#include "internal.h"
#include "sm100_ptx.cuh"
#include <cstring>

namespace ob200 {
namespace {

constexpr int kTileM = 128;              // positions per MMA tile
constexpr int kUnitTiles = 2;            // tiles per work unit
constexpr int kN = 128;                  // output channels per work unit
constexpr int kSlice = 64;               // input channels per K slice
constexpr int kRowBytes = kSlice * 2;    // one position of one slice
constexpr int kBoxRows = 160;            // rows per activation TMA box; two boxes per stage
constexpr int kAStageBytes = 2 * kBoxRows * kRowBytes;   // 40,960: 256 positions + 2 x 32 halo rows
constexpr int kAStages = 2;
constexpr int kBStageBytes = kN * kRowBytes;              // 16,384
constexpr int kBStages = 6;
constexpr int kOutBytes = kTileM * kRowBytes;             // 16,384: 64 output channels of a tile
constexpr int kEpiGroups = kUnitTiles;
constexpr int kAccStages = 2;
constexpr int kTmemCols = kAccStages * kUnitTiles * kN;   // 512
constexpr int kThreads = 128 + 128 * kEpiGroups;          // warps 0-3 roles, 4-11 epilogue
constexpr int kNumBars = 2 * kAStages + 2 * kBStages + 2 * kAccStages + kEpiGroups;
constexpr int kMaxCout = 256;
constexpr int kSmemBytes = kAStages * kAStageBytes + kBStages * kBStageBytes + kEpiGroups * kOutBytes +
                           kNumBars * 8 + kMaxCout * 4 + 16 + 1024;

struct WideParams {
    const uint8_t* w;         // packed weights: [n_half][k_slice][tap] blocks of 128 x 64, pre-swizzled
    const float* bias;        // [cout]
    int has_residual;         // the residual tensor map is live
    float* out_f32;           // when set: results as fp32 [positions][cout] by plain stores, no bf16 tensor
    int* error;               // device error word (0 = fine)
    int P;                    // real positions = B * slots
    int num_tiles;            // 128-position tiles
    int m_units;              // ceil(num_tiles / 2)
    int n_halves;             // cout / 128
    int k_slices;             // cin / 64
    int cout;
    int S, GP, slots;
    int halo;                 // rows before the unit's first position in a stage
    int relu;
};

using namespace ptx;
__device__ __forceinline__ void group_bar(int id) {   // the 128 threads of one epilogue group
    asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}
// Barrier of one epilogue group that also tells every thread whether any of them reports `bad`:
// the group gives up on a wait as a whole, so no thread is left at a barrier its siblings have left.
__device__ __forceinline__ bool group_any(int id, bool bad) {
    uint32_t r;
    asm volatile(
        "{\n.reg .pred p, q;\nsetp.ne.b32 q, %2, 0;\nbar.red.or.pred p, %1, 128, q;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(r) : "r"(id), "r"((uint32_t)bad) : "memory");
    return r != 0;
}

// F16: activations and weights are fp16 instead of bf16.
template <int TAPS, bool F16>
__global__ void __launch_bounds__(kThreads, 1)
conv_wide_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                 const __grid_constant__ CUtensorMap res_map, const WideParams p) {
    constexpr uint32_t kIdesc = make_idesc(F16, kTileM, kN);
    extern __shared__ uint8_t smem_raw[];
    // swizzled tiles need 1024-byte aligned bases
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_s = smem;
    uint8_t* b_s = a_s + kAStages * kAStageBytes;
    uint8_t* o_s = b_s + kBStages * kBStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(o_s + kEpiGroups * kOutBytes);
    float* bias_s = reinterpret_cast<float*>(bars + kNumBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bias_s + kMaxCout);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto afull_bar = [&](int s) { return bar0 + 8u * s; };
    auto aempty_bar = [&](int s) { return bar0 + 8u * (kAStages + s); };
    auto bfull_bar = [&](int s) { return bar0 + 8u * (2 * kAStages + s); };
    auto bempty_bar = [&](int s) { return bar0 + 8u * (2 * kAStages + kBStages + s); };
    auto accfull_bar = [&](int a) { return bar0 + 8u * (2 * kAStages + 2 * kBStages + a); };
    auto accempty_bar = [&](int a) { return bar0 + 8u * (2 * kAStages + 2 * kBStages + kAccStages + a); };
    auto res_bar = [&](int g) { return bar0 + 8u * (2 * kAStages + 2 * kBStages + 2 * kAccStages + g); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kAStages; ++s) { mbar_init(afull_bar(s), 1); mbar_init(aempty_bar(s), 1); }
        for (int s = 0; s < kBStages; ++s) { mbar_init(bfull_bar(s), 1); mbar_init(bempty_bar(s), 1); }
        for (int a = 0; a < kAccStages; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), 4 * kEpiGroups); }
        for (int g = 0; g < kEpiGroups; ++g) mbar_init(res_bar(g), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&in_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&out_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&res_map) : "memory");
    }
    for (int i = threadIdx.x; i < p.cout; i += kThreads) bias_s[i] = p.bias[i];
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: what reads or writes activations sits behind
    // griddepcontrol.wait; the weight ring may fill while the previous layer drains.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int num_units = p.m_units * p.n_halves;

    if (warp == 0) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int it = 0;
            for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
                const int mu = u / p.n_halves;
                const int row0 = OB200_GUARD + mu * (kUnitTiles * kTileM) - p.halo;
                bool ok = true;
                for (int kc = 0; kc < p.k_slices; ++kc, ++it) {
                    const int s = it % kAStages;
                    const uint32_t ph = (uint32_t)(it / kAStages) & 1u;
                    if (!mbar_wait(aempty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(afull_bar(s), (uint32_t)kAStageBytes);
                    const uint32_t dst = smem_u32(a_s + s * kAStageBytes);
                    tma_load_2d(dst, &in_map, kc * kSlice, row0, afull_bar(s));
                    tma_load_2d(dst + kBoxRows * kRowBytes, &in_map, kc * kSlice, row0 + kBoxRows, afull_bar(s));
                }
                if (!ok) { *abort_flag = 1; atomicExch(p.error, 1); break; }
            }
        }
    } else if (warp == 2) {
        // ---------------- weight producer ----------------
        if (lane == 0) {
            int jt = 0;
            for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
                const int nh = u % p.n_halves;
                const uint8_t* src = p.w + (size_t)nh * p.k_slices * TAPS * kBStageBytes;
                const int blocks = p.k_slices * TAPS;
                bool ok = true;
                for (int j = 0; j < blocks; ++j, ++jt) {
                    const int s = jt % kBStages;
                    const uint32_t ph = (uint32_t)(jt / kBStages) & 1u;
                    if (!mbar_wait(bempty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(bfull_bar(s), (uint32_t)kBStageBytes);
                    bulk_g2s(smem_u32(b_s + s * kBStageBytes), src + (size_t)j * kBStageBytes, (uint32_t)kBStageBytes,
                             bfull_bar(s));
                }
                if (!ok) { *abort_flag = 1; atomicExch(p.error, 4); break; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // One thread issues; the loop over taps, tiles and 16-channel steps is unrolled with
        // compile-time offsets and ring positions are kept as counters, because every integer
        // instruction between two MMAs of this thread is time the tensor core waits.
        if (lane == 0) {
            int tap_off[TAPS];
#pragma unroll
            for (int tap = 0; tap < TAPS; ++tap) {
                const int dy = TAPS == 9 ? tap / 3 - 1 : 0, dx = TAPS == 9 ? tap % 3 - 1 : 0;
                tap_off[tap] = (p.halo + dy * p.GP + dx) * (kRowBytes >> 4);
            }
            const uint32_t a_base = desc_lo(smem_u32(a_s)), b_base = desc_lo(smem_u32(b_s));
            int sa = 0, sb = 0, acc = 0;
            uint32_t pha = 0, phb = 0, phacc = 0;
            bool ok = true;
            for (int u = blockIdx.x; ok && u < num_units; u += gridDim.x) {
                const int mu = u / p.n_halves;
                const bool two = p.num_tiles - mu * kUnitTiles >= kUnitTiles;
                if (!mbar_wait(accempty_bar(acc), phacc ^ 1u, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kUnitTiles * kN);
                for (int kc = 0; ok && kc < p.k_slices; ++kc) {
                    if (!mbar_wait(afull_bar(sa), pha, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_lo = a_base + (uint32_t)(sa * (kAStageBytes >> 4));
#pragma unroll
                    for (int tap = 0; tap < TAPS; ++tap) {
                        if (!mbar_wait(bfull_bar(sb), phb, abort_flag)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t b_lo = b_base + (uint32_t)(sb * (kBStageBytes >> 4));
                        const uint32_t at = a_lo + (uint32_t)tap_off[tap];
#pragma unroll
                        for (int ks = 0; ks < kSlice / 16; ++ks)
                            umma(d_tmem, at + (uint32_t)(ks * 2), b_lo + (uint32_t)(ks * 2), kIdesc, (tap | ks) ? 1u : (uint32_t)(kc != 0));
                        if (two) {
#pragma unroll
                            for (int ks = 0; ks < kSlice / 16; ++ks)
                                umma(d_tmem + (uint32_t)kN, at + (uint32_t)(kTileM * (kRowBytes >> 4) + ks * 2),
                                     b_lo + (uint32_t)(ks * 2), kIdesc, (tap | ks) ? 1u : (uint32_t)(kc != 0));
                        }
                        umma_commit(bempty_bar(sb));    // weight block free once these MMAs have read it
                        if (++sb == kBStages) { sb = 0; phb ^= 1u; }
                    }
                    if (ok) umma_commit(aempty_bar(sa));   // activation stage free
                    if (++sa == kAStages) { sa = 0; pha ^= 1u; }
                }
                if (ok) umma_commit(accfull_bar(acc));     // accumulators ready for the epilogue
                if (++acc == kAccStages) { acc = 0; phacc ^= 1u; }
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 2); }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue: TMEM -> registers -> shared -> TMA store ----------------
        // Group g (4 warps) owns tile g of every unit; a warp owns one TMEM lane quadrant
        // (fixed by warp id % 4), a thread one position and all 128 output channels, 64 at a time.
        // The group has one staging tile (128 positions x 64 channels).  With a residual, TMA loads
        // the residual's 64-channel half into the staging tile (the first half while the unit's
        // MMAs run); a thread then reads its own row, adds, and writes the result back in place
        // before the TMA store.
        const int ew = warp - 4;
        const int group = ew >> 2;
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool leader = (ew & 3) == 0 && lane == 0;
        const bool has_res = p.has_residual != 0;
        uint8_t* stage_out = o_s + group * kOutBytes;
        const uint32_t stage_out_u32 = smem_u32(stage_out);
        uint32_t res_phase = 0;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        int ut = 0;
        for (int u = blockIdx.x; u < num_units; u += gridDim.x, ++ut) {
            const int mu = u / p.n_halves, nh = u % p.n_halves;
            const int a = ut % kAccStages;
            const uint32_t pa = (uint32_t)(ut / kAccStages) & 1u;
            const int tile = mu * kUnitTiles + group;
            const bool active = tile < p.num_tiles;
            const int pos = tile * kTileM + row;
            bool valid = active && pos < p.P;
            if (valid) {
                const int rr = pos % p.slots;
                valid = (rr / p.GP < p.S) && (rr % p.GP < p.S);
            }
            if (active && leader) {
                // the previous store of this group must have finished reading the staging tile
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                if (has_res) {
                    mbar_arrive_expect_tx(res_bar(group), (uint32_t)kOutBytes);
                    tma_load_2d(stage_out_u32, &res_map, nh * kN, OB200_GUARD + tile * kTileM, res_bar(group));
                }
            }
            if (group_any(1 + 2 * group, !mbar_wait(accfull_bar(a), pa, abort_flag))) {
                *abort_flag = 1; atomicExch(p.error, 3); break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!active) {   // a unit with one tile: nothing to read, release the accumulator
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(accempty_bar(a));
                continue;
            }
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kUnitTiles * kN + group * kN);
            bool ok = true;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (half == 1 && leader) {
                    // second half: the store of the first must have read the staging tile
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    if (has_res) {
                        mbar_arrive_expect_tx(res_bar(group), (uint32_t)kOutBytes);
                        tma_load_2d(stage_out_u32, &res_map, nh * kN + 64, OB200_GUARD + tile * kTileM, res_bar(group));
                    }
                }
                uint32_t r[64];
                tmem_ld32(t_acc + (uint32_t)(half * 64), r);
                tmem_ld32(t_acc + (uint32_t)(half * 64 + 32), r + 32);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (half == 1) {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(accempty_bar(a));
                }
                if (p.out_f32 != nullptr) {
                    // fp32 output (policy planes): the thread's 64 channels are 256 contiguous bytes
                    float4* dst = reinterpret_cast<float4*>(p.out_f32 + (size_t)(OB200_GUARD + pos) * p.cout + nh * kN + half * 64);
                    const float* bias_f = bias_s + nh * kN + half * 64;
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        if (valid) {
                            o.x = __uint_as_float(r[4 * c]) + bias_f[4 * c];
                            o.y = __uint_as_float(r[4 * c + 1]) + bias_f[4 * c + 1];
                            o.z = __uint_as_float(r[4 * c + 2]) + bias_f[4 * c + 2];
                            o.w = __uint_as_float(r[4 * c + 3]) + bias_f[4 * c + 3];
                            if (p.relu) { o.x = fmaxf(o.x, 0.0f); o.y = fmaxf(o.y, 0.0f); o.z = fmaxf(o.z, 0.0f); o.w = fmaxf(o.w, 0.0f); }
                        }
                        dst[c] = o;
                    }
                    continue;
                }
                // the vote is also the barrier behind the leader's wait: the staging tile is free
                if (group_any(1 + 2 * group, has_res && !mbar_wait(res_bar(group), res_phase, abort_flag))) { ok = false; break; }
                if (has_res) res_phase ^= 1u;
                const float* bias_t = bias_s + nh * kN + half * 64;
                uint8_t* my_row = stage_out + row * kRowBytes;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    // 128-byte swizzle of the staging tile: 16-byte chunk k of row r sits at chunk k ^ (r % 8)
                    uint4* slot = reinterpret_cast<uint4*>(my_row + ((c ^ (row & 7)) << 4));
                    uint4 o = make_uint4(0u, 0u, 0u, 0u);
                    if (valid) {
                        const uint4 rv = has_res ? *slot : make_uint4(0u, 0u, 0u, 0u);
                        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
                        uint32_t ow[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float r0, r1;
                            unpack2<F16>(rw[j], r0, r1);
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
                    tma_store_2d(&out_map, nh * kN + half * 64, OB200_GUARD + tile * kTileM, stage_out_u32);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 5); break; }
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

bool conv_wide_covers(int cin, int cout) {
    return cin >= kSlice && cin <= 256 && cin % kSlice == 0 && (cout == 128 || cout == 256);
}
int conv_wide_box_rows() { return kBoxRows; }

int launch_conv_wide_maps(const BoardTensorMap& in_map, const BoardTensorMap& out_map, const BoardTensorMap* res_map,
                          const void* packed_w, const float* bias, int B, int S, int cin, int cout, int taps, int relu,
                          cudaStream_t st, float* out_f32, int dtype) {
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "conv (wide): bad dtype %d", dtype);
    if (!packed_w || !bias || B <= 0) return set_error(OB200_ERR_INVALID, "conv (wide): null pointer or empty batch");
    if (!conv_wide_covers(cin, cout) || (taps != 9 && taps != 1))
        return set_error(OB200_ERR_UNSUPPORTED, "conv (wide): %d -> %d channels with %d taps is not covered", cin, cout, taps);
    if (S < 1 || S + 2 > OB200_GUARD)
        return set_error(OB200_ERR_UNSUPPORTED, "conv (wide): board_size %d outside [1, %d]", S, OB200_GUARD - 2);
    if ((uintptr_t)packed_w & 15) return set_error(OB200_ERR_INVALID, "conv (wide): weights must be 16-byte aligned");
    if (int rc = require_device()) return rc;
    static bool configured[64] = {false};
    int dev = 0;
    OB200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        OB200_CUDA_OK(cudaFuncSetAttribute(conv_wide_kernel<9, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        OB200_CUDA_OK(cudaFuncSetAttribute(conv_wide_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        OB200_CUDA_OK(cudaFuncSetAttribute(conv_wide_kernel<9, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        OB200_CUDA_OK(cudaFuncSetAttribute(conv_wide_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    int sms = 0;
    OB200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const BoardGeom g = board_geom(S, B);
    WideParams p;
    p.w = static_cast<const uint8_t*>(packed_w); p.bias = bias; p.has_residual = res_map != nullptr;
    p.out_f32 = out_f32;
    if (out_f32 && res_map) return set_error(OB200_ERR_INVALID, "conv (wide): fp32 output takes no residual");
    p.error = device_error_word();
    if (!p.error) return set_error(OB200_ERR_CUDA, "conv (wide): cannot resolve the device error word");
    p.P = (int)g.P; p.num_tiles = (int)(g.Ppad / kTileM); p.m_units = (p.num_tiles + kUnitTiles - 1) / kUnitTiles;
    p.n_halves = cout / kN; p.k_slices = cin / kSlice; p.cout = cout;
    p.S = S; p.GP = g.GP; p.slots = g.slots;
    p.halo = taps == 9 ? S + 2 : 0; p.relu = relu;   // |dy*(S+1)+dx| <= S+2 rows before / after a unit
    const int units = p.m_units * p.n_halves;
    const int grid = units < sms ? units : sms;   // one persistent CTA per SM
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const CUtensorMap& im = *reinterpret_cast<const CUtensorMap*>(&in_map);
    const CUtensorMap& om = *reinterpret_cast<const CUtensorMap*>(&out_map);
    const CUtensorMap& rm = *reinterpret_cast<const CUtensorMap*>(res_map ? res_map : &out_map);
    auto kernel = dtype == OB200_DTYPE_F16 ? (taps == 9 ? conv_wide_kernel<9, true> : conv_wide_kernel<1, true>)
                                           : (taps == 9 ? conv_wide_kernel<9, false> : conv_wide_kernel<1, false>);
    OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, im, om, rm, p));
    OB200_LAUNCHED("conv_wide_kernel");
    return OB200_OK;
}

size_t conv_wide_packed_bytes(int cin, int cout, int taps) { return (size_t)taps * cin * cout * 2; }

// Packed image: blocks [n_half][k_slice][tap] of 128 output channels x 64 input channels, bf16 (or fp16),
// one 128-byte row per output channel, its 16-byte chunks (8 input channels) permuted by the
// 128-byte swizzle (chunk j of row r stored at chunk j ^ (r % 8)): the K-major shared-memory
// operand layout of the tensor core, ready for plain bulk copies in the order the kernel
// consumes them.  w: [cout][cin_real][taps] fp32 (OIHW), scale: per output channel or null.
int conv_wide_pack(const float* w, const float* scale, int cout, int cin_real, int cin, int taps, void* packed_out, int dtype) {
    if (!w || !packed_out || !conv_wide_covers(cin, cout) || cin_real <= 0 || cin_real > cin || (taps != 9 && taps != 1))
        return set_error(OB200_ERR_INVALID, "conv (wide) pack: cout %d, cin_real %d, cin %d, taps %d not covered", cout,
                         cin_real, cin, taps);
    uint16_t* o = static_cast<uint16_t*>(packed_out);
    const int KS = cin / kSlice;
    for (int co = 0; co < cout; ++co)
        for (int ci = 0; ci < cin; ++ci)
            for (int tap = 0; tap < taps; ++tap) {
                float v = 0.0f;
                if (ci < cin_real) v = w[((size_t)co * cin_real + ci) * taps + tap] * (scale ? scale[co] : 1.0f);
                const int nh = co / kN, col = co % kN, kc = ci / kSlice, cil = ci % kSlice;
                const size_t block = ((size_t)nh * KS + kc) * taps + tap;
                const size_t byte = block * kBStageBytes + (size_t)col * kRowBytes + ((((cil >> 3) ^ (col & 7))) << 4) + (cil & 7) * 2;
                o[byte / 2] = dtype == OB200_DTYPE_F16 ? f32_to_f16_rne_sat(v) : f32_to_bf16_rne(v);
            }
    return OB200_OK;
}

}  // namespace ob200
