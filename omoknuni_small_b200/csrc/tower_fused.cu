// The whole 64-filter residual tower as ONE persistent kernel (sm_100a).
//
// Same tile arithmetic as conv3x3_kernel (tower.cu): M = 128 positions per tile,
// N = 64, K = 9 taps x 64, taps as row-shifted shared-memory descriptors, TMEM
// accumulators, residual by TMA into the staging tile.  What changes is what
// happens between layers.  A launch per layer pays the pipeline's fill and drain,
// the 72 KB weight load and the launch gap 21 times (about 4 us of a 22 us layer
// at batch 1024).  Here every CTA walks the layers itself:
//   * tile t of layer l only needs tiles t-1, t, t+1 of layer l-1 (its halo).  Each
//     finished tile publishes a flag (store complete -> fence -> release store); the
//     producer warp acquires the three flags before it issues the tile's TMA load.
//     With the static tile -> CTA assignment all CTAs move through the layers in
//     near lock step, so the waits are short and the MMA pipeline never drains at a
//     layer boundary;
//   * weights are double-buffered in shared memory: a loader warp brings layer l+1
//     in while layer l computes (the buffer is handed back by a tcgen05.commit after
//     the last MMA of layer l-1).
//   * one thread per epilogue group issues the TMA store, hands the staging tile back
//     (with the next tile's residual already loading into it), waits for the store to
//     complete and publishes the flag, so that this latency and the fences stay off the
//     128 threads that do the arithmetic; the producer polls the halo flags of two tiles
//     at a time and stops polling once the previous layer's published-tile count is
//     complete (a poll with its two fences costs about 1.6 us).
// Measured at batch 1024 (15x15, 21 layers): 19.6 us per layer instead of 22.2 us as separate
// launches; the MMA issue period (36 MMAs, 2,440 cycles per tile) is the same in both and is
// what bounds the kernel.
// The three activation buffers rotate exactly as in the per-layer path, so the
// write-after-read hazards are covered by the same flags (a tile is overwritten
// only by a layer whose loads already waited for every reader of that tile).
// CTAs wait on one another, so the kernel is launched cooperatively (all CTAs
// resident), every wait is bounded, and a CTA that gives up raises the device
// error word and stops publishing, which makes its neighbours give up in turn.
#include "internal.h"
#include <cooperative_groups.h>
#include "sm100_ptx.cuh"

namespace ob200 {
namespace {

constexpr int kTileM = 128;
constexpr int kC = 64;
constexpr int kRowBytes = kC * 2;
constexpr int kWBytes = 9 * kC * kRowBytes;          // 73,728 per layer
constexpr int kOutBytes = kTileM * kRowBytes;        // 16,384
constexpr int kStages = 2;                           // activation tiles in flight
constexpr int kAccStages = 4;
constexpr int kTmemCols = kAccStages * kC;           // 256
constexpr int kEpiGroups = 2;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 96 + 32 * kEpiWarps * kEpiGroups + 32 * kEpiGroups;   // warps: 0 loads, 1 MMA, 2 weights, 3-10 epilogue, 11-12 store / publish
constexpr int kNumBars = 2 * kStages + 2 * kAccStages + 4 + 2 * kEpiGroups;
constexpr uint32_t kFlagSpin = 1u << 20;

struct alignas(128) TowerLayerDev {
    CUtensorMap in_map;       // load boxes over the layer's input (unused for layer 0)
    CUtensorMap out_map;      // 128-row store boxes over the layer's output
    CUtensorMap res_map;      // 128-row boxes over the residual tensor (when has_res)
    const uint8_t* w;         // packed weights (ob200_pack_conv3x3_weights)
    const float* bias;        // [64]
    int has_res;
    int pad_[27];
};
static_assert(sizeof(TowerLayerDev) % 128 == 0, "layer descriptor must keep the tensor maps 64-byte aligned");

struct TowerParams {
    const TowerLayerDev* layers;
    int n_layers;
    int* flags;               // [n_layers][tiles_pitch], value == epoch when the tile is stored
    int* done;                // [n_layers] tiles of the layer published in this epoch (zeroed by the host before the launch)
    int tiles_pitch;
    int epoch;
    int* error;
    int P, num_tiles, S, GP, slots, halo;
    int stage_bytes;          // (128 + 2 * halo) rows, rounded up to 1024
};

using namespace ptx;
// The halo flags of a tile (f[0..2]) and of the CTA's next tile (f[3..5]) in one poll: relaxed
// loads in flight together (plus the layer's count of published tiles), one acquire fence when
// the first three are up.  *next_ok tells whether the next tile's three were up as well.
__device__ __forceinline__ bool flags_wait(const int* const (&f)[6], const int* done, int epoch, int* finished,
                                           bool* next_ok, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kFlagSpin; ++i) {
        int v[6], d;
#pragma unroll
        for (int j = 0; j < 6; ++j) asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v[j]) : "l"(f[j]) : "memory");
        asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(d) : "l"(done) : "memory");
        if (v[0] == epoch && v[1] == epoch && v[2] == epoch) {
            asm volatile("fence.acq_rel.gpu;" ::: "memory");
            *finished = d;
            *next_ok = v[3] == epoch && v[4] == epoch && v[5] == epoch;
            return true;
        }
        if ((i & 15) == 15) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    return false;
}
// F16: activations and weights are fp16 instead of bf16.
template <bool F16>
__global__ void __launch_bounds__(kThreads, 1)
conv_tower_kernel(const __grid_constant__ CUtensorMap stem_in_map, const TowerParams p) {
    constexpr uint32_t kIdesc = make_idesc(F16, kTileM, kC);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* w_s = smem;                                   // two weight buffers
    uint8_t* a_s = w_s + 2 * kWBytes;                      // kStages activation tiles
    uint8_t* o_s = a_s + kStages * p.stage_bytes;          // one staging tile per epilogue group
    float* bias_s = reinterpret_cast<float*>(o_s + kEpiGroups * kOutBytes);   // [n_layers][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(bias_s + p.n_layers * kC);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto accfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
    auto accempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + kAccStages + a); };
    auto wfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 * kAccStages + b); };
    auto wempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 * kAccStages + 2 + b); };
    // per epilogue group: "staging tile ready for the threads" (residual landed, or simply free) and
    // "staging tile written" (4 warps)
    auto ready_bar = [&](int g) { return bar0 + 8u * (2 * kStages + 2 * kAccStages + 4 + g); };
    auto written_bar = [&](int g) { return bar0 + 8u * (2 * kStages + 2 * kAccStages + 4 + kEpiGroups + g); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < kAccStages; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), kEpiWarps); }
        for (int b = 0; b < 2; ++b) { mbar_init(wfull_bar(b), 1); mbar_init(wempty_bar(b), 1); }
        for (int g = 0; g < kEpiGroups; ++g) { mbar_init(ready_bar(g), 1); mbar_init(written_bar(g), kEpiWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&stem_in_map) : "memory");
    }
    for (int i = threadIdx.x; i < p.n_layers * kC; i += kThreads) bias_s[i] = p.layers[i / kC].bias[i % kC];
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            const uint32_t box_bytes = (uint32_t)(kTileM + 2 * p.halo) * kRowBytes;
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            for (int l = 0; ok && l < p.n_layers; ++l) {
                const CUtensorMap* map = l == 0 ? &stem_in_map : &p.layers[l].in_map;
                const int* prev = p.flags + (size_t)(l - 1) * p.tiles_pitch;
                bool prev_done = l == 0;     // every tile of the previous layer is published
                bool checked = false;        // this tile's halo was seen complete by the previous poll
                for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                    if (!prev_done && !checked) {
                        // the tile's halo: tiles tile-1, tile, tile+1 of the previous layer; the next tile's
                        // halo rides along in the same poll
                        const int t2 = tile + (int)gridDim.x < p.num_tiles ? tile + (int)gridDim.x : tile;
                        const int* const f[6] = {prev + (tile > 0 ? tile - 1 : tile), prev + tile,
                                                 prev + (tile + 1 < p.num_tiles ? tile + 1 : tile),
                                                 prev + (t2 > 0 ? t2 - 1 : t2), prev + t2,
                                                 prev + (t2 + 1 < p.num_tiles ? t2 + 1 : t2)};
                        int finished = 0;
                        if (!flags_wait(f, p.done + (l - 1), p.epoch, &finished, &checked, abort_flag)) { ok = false; break; }
                        prev_done = finished == p.num_tiles;
                        asm volatile("fence.proxy.async;" ::: "memory");   // acquired data -> reads by the copy engine
                    } else {
                        checked = false;
                    }
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(full_bar(s), box_bytes);
                    tma_load_2d(smem_u32(a_s + s * p.stage_bytes), map, 0, OB200_GUARD + tile * kTileM - p.halo, full_bar(s));
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 1); }
        }
    } else if (warp == 2) {
        // ---------------- weight loader ----------------
        if (lane == 0) {
            for (int l = 0; l < p.n_layers; ++l) {
                const int b = l & 1;
                if (l >= 2 && !mbar_wait(wempty_bar(b), (uint32_t)((l - 2) >> 1) & 1u, abort_flag)) {
                    *abort_flag = 1; atomicExch(p.error, 4); break;
                }
                mbar_arrive_expect_tx(wfull_bar(b), (uint32_t)kWBytes);
                bulk_g2s(smem_u32(w_s + b * kWBytes), p.layers[l].w, (uint32_t)kWBytes, wfull_bar(b));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int tap_off[9];
#pragma unroll
            for (int tap = 0; tap < 9; ++tap)
                tap_off[tap] = (p.halo + (tap / 3 - 1) * p.GP + (tap % 3 - 1)) * (kRowBytes >> 4);
            const uint32_t a_base = desc_lo(smem_u32(a_s)), w_base = desc_lo(smem_u32(w_s));
            int s = 0, a = 0;
            uint32_t ph = 0, pa = 0;
            bool ok = true;
            for (int l = 0; ok && l < p.n_layers; ++l) {
                const int b = l & 1;
                if (!mbar_wait(wfull_bar(b), (uint32_t)(l >> 1) & 1u, abort_flag)) { ok = false; break; }
                const uint32_t w_lo = w_base + (uint32_t)(b * (kWBytes >> 4));
                for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                    if (!mbar_wait(accempty_bar(a), pa ^ 1u, abort_flag) || !mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_lo = a_base + (uint32_t)(s * (p.stage_bytes >> 4));
                    const uint32_t d_tmem = tmem_base + (uint32_t)a * kC;
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
#pragma unroll
                        for (int ks = 0; ks < kC / 16; ++ks)
                            umma(d_tmem, a_lo + (uint32_t)(tap_off[tap] + ks * 2),
                                 w_lo + (uint32_t)(tap * (kC * kRowBytes >> 4) + ks * 2), kIdesc, (tap | ks) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));
                    umma_commit(accfull_bar(a));
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                    if (++a == kAccStages) { a = 0; pa ^= 1u; }
                }
                if (ok) umma_commit(wempty_bar(b));     // this layer's MMAs have read the weight buffer
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 2); }
        }
    } else if (warp >= 3 && warp < 3 + kEpiWarps * kEpiGroups) {
        // ---------------- epilogue: TMEM -> registers -> staging tile ----------------
        // Group g takes this CTA's tiles k = g, g + 2, ... of every layer (k counts the CTA's tiles
        // within the layer, so a given tile belongs to the same group in every layer).  The group's
        // store / publish warp hands it the staging tile (with the residual in it when the layer
        // has one) and takes it back when the four warps have written their rows.
        const int ew = warp - 3;
        const int group = ew / kEpiWarps;
        const int q = warp & 3;                      // TMEM lane quadrant this warp may read
        const int row = q * 32 + lane;
        uint8_t* stage_out = o_s + group * kOutBytes;
        uint32_t ready_phase = 0;
        int it = 0;
        bool ok = true;
        for (int l = 0; ok && l < p.n_layers; ++l) {
            const bool has_res = p.layers[l].has_res != 0;
            const float* bias_t = bias_s + l * kC;
            int k = 0;
            for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it, ++k) {
                if ((k & 1) != group) continue;
                const int a = it % kAccStages;
                const uint32_t pa = (uint32_t)(it / kAccStages) & 1u;
                const int pos = tile * kTileM + row;
                bool valid = pos < p.P;
                if (valid) {
                    const int rr = pos % p.slots;
                    valid = (rr / p.GP < p.S) && (rr % p.GP < p.S);
                }
                // a warp gives up as a whole (the TMEM loads below need all 32 lanes)
                if (!__all_sync(0xffffffffu, mbar_wait(accfull_bar(a), pa, abort_flag))) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t r[kC];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kC), r);
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kC + 32), r + 32);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(accempty_bar(a));
                if (!__all_sync(0xffffffffu, mbar_wait(ready_bar(group), ready_phase, abort_flag))) { ok = false; break; }
                ready_phase ^= 1u;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    // 128-byte swizzle of the staging tile: 16-byte chunk k of row r sits at chunk k ^ (r % 8)
                    uint4* slot = reinterpret_cast<uint4*>(stage_out + row * kRowBytes + ((c ^ (row & 7)) << 4));
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
                            v0 = fmaxf(v0, 0.0f); v1 = fmaxf(v1, 0.0f);
                            ow[j] = pack2<F16>(v0, v1);
                        }
                        o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                    *slot = o;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // rows -> the TMA store's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(written_bar(group));
            }
        }
        if (!ok) { *abort_flag = 1; atomicExch(p.error, 3); }
    } else if (warp >= 3 + kEpiWarps * kEpiGroups) {
        // ---------------- store / publish (one thread per epilogue group) ----------------
        // Keeps the latency of "store complete -> fence -> flag" off the epilogue threads.  Per tile:
        // make the staging tile ready (TMA load of the residual, which is this tile of layer l-2 and
        // was stored by this same thread, or a plain arrive), wait for the four warps, TMA store, wait
        // until the store has read the tile (it can be handed out again), later wait for the store to
        // complete and publish the tile's flag.
        const int group = warp - (3 + kEpiWarps * kEpiGroups);
        if (lane == 0) {
            const uint32_t stage_out_u32 = smem_u32(o_s + group * kOutBytes);
            uint32_t written_phase = 0;
            int* pending = nullptr;       // flag of the tile whose store is in flight
            int* pending_done = nullptr;
            bool first = true;
            bool ok = true;
            auto publish = [&]() {
                if (pending != nullptr) {
                    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the store is complete
                    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(pending), "r"(p.epoch) : "memory");
                    asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(pending_done) : "memory");
                    pending = nullptr;
                }
            };
            for (int l = 0; ok && l < p.n_layers; ++l) {
                const TowerLayerDev* L = p.layers + l;
                int k = 0;
                for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++k) {
                    if ((k & 1) != group) continue;
                    if (first) {
                        // the group's first tile (layer 0, no residual): the staging tile is simply free; every
                        // later hand-over happens right after the previous tile's store (below)
                        mbar_arrive(ready_bar(group));
                        first = false;
                    }
                    if (!mbar_wait(written_bar(group), written_phase, abort_flag)) { ok = false; break; }
                    written_phase ^= 1u;
                    tma_store_2d(&L->out_map, 0, OB200_GUARD + tile * kTileM, stage_out_u32);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // staging tile reusable
                    pending = p.flags + (size_t)l * p.tiles_pitch + tile;
                    pending_done = p.done + l;
                    // hand the staging tile to the threads for the group's next tile first, then see this
                    // tile's store through and publish it (neighbours wait for the flag at layer boundaries)
                    int ntile = tile + 2 * (int)gridDim.x, nl = l;
                    if (ntile >= p.num_tiles) { nl = l + 1; ntile = (int)blockIdx.x + group * (int)gridDim.x; }
                    if (nl < p.n_layers && ntile < p.num_tiles) {
                        const TowerLayerDev* NL = p.layers + nl;
                        if (NL->has_res) {
                            mbar_arrive_expect_tx(ready_bar(group), (uint32_t)kOutBytes);
                            tma_load_2d(stage_out_u32, &NL->res_map, 0, OB200_GUARD + ntile * kTileM, ready_bar(group));
                        } else {
                            mbar_arrive(ready_bar(group));
                        }
                    }
                    publish();
                }
            }
            publish();
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 5); }
        }
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

}  // namespace

size_t tower_fused_layer_bytes() { return sizeof(TowerLayerDev); }

// Fills one layer descriptor (host memory; the caller uploads the array).
void tower_fused_fill_layer(void* dst, const BoardTensorMap* in_map, const BoardTensorMap& out_map,
                            const BoardTensorMap* res_map, const void* w, const float* bias) {
    TowerLayerDev d;
    std::memset(&d, 0, sizeof(d));
    if (in_map) std::memcpy(&d.in_map, in_map, sizeof(CUtensorMap));
    std::memcpy(&d.out_map, &out_map, sizeof(CUtensorMap));
    if (res_map) std::memcpy(&d.res_map, res_map, sizeof(CUtensorMap));
    d.w = static_cast<const uint8_t*>(w); d.bias = bias; d.has_res = res_map != nullptr;
    std::memcpy(dst, &d, sizeof(d));
}

// Shared memory the fused tower needs for a board size / depth, or 0 when it does not fit.
size_t tower_fused_smem_bytes(int S, int n_layers) {
    const int halo = conv_halo_rows(S);
    const size_t stage = ((size_t)(kTileM + 2 * halo) * kRowBytes + 1023) / 1024 * 1024;
    const size_t total = 2 * (size_t)kWBytes + kStages * stage + kEpiGroups * (size_t)kOutBytes + (size_t)n_layers * kC * 4 +
                         kNumBars * 8 + 16 + 1024;
    return total <= 232448 ? total : 0;
}

// One launch for the whole tower.  layers_dev: n_layers descriptors on the device; flags:
// n_layers x tiles_pitch ints that only ever hold earlier epochs; done: n_layers ints (zeroed here).  Returns OB200_ERR_UNSUPPORTED
// when the cooperative launch is not possible (the caller then runs layer by layer).
int launch_conv_tower(const BoardTensorMap& stem_in_map, const void* layers_dev, int n_layers, int* flags, int tiles_pitch,
                      int* done, int epoch, int B, int S, cudaStream_t st, int dtype) {
    if (!layers_dev || !flags || !done || n_layers < 1 || B <= 0) return set_error(OB200_ERR_INVALID, "conv tower: bad arguments");
    const size_t smem = tower_fused_smem_bytes(S, n_layers);
    if (!smem) return set_error(OB200_ERR_UNSUPPORTED, "conv tower: board size %d / %d layers do not fit shared memory", S, n_layers);
    if (int rc = require_device()) return rc;
    int dev = 0, sms = 0, coop = 0;
    OB200_CUDA_OK(cudaGetDevice(&dev));
    OB200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    OB200_CUDA_OK(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) return set_error(OB200_ERR_UNSUPPORTED, "conv tower: the device does not support cooperative launches");
    const bool f16 = dtype == OB200_DTYPE_F16;
    auto kernel = f16 ? conv_tower_kernel<true> : conv_tower_kernel<false>;
    static size_t configured[64][2] = {{0, 0}};
    if (dev >= 0 && dev < 64 && configured[dev][f16] < smem) {
        OB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][f16] = smem;
    }
    const BoardGeom g = board_geom(S, B);
    TowerParams p;
    p.layers = static_cast<const TowerLayerDev*>(layers_dev); p.n_layers = n_layers; p.flags = flags; p.tiles_pitch = tiles_pitch;
    p.done = done; p.epoch = epoch; p.error = device_error_word();
    if (!p.error) return set_error(OB200_ERR_CUDA, "conv tower: cannot resolve the device error word");
    p.P = (int)g.P; p.num_tiles = (int)(g.Ppad / kTileM); p.S = S; p.GP = g.GP; p.slots = g.slots; p.halo = conv_halo_rows(S);
    p.stage_bytes = (int)(((size_t)(kTileM + 2 * p.halo) * kRowBytes + 1023) / 1024 * 1024);
    if (p.num_tiles > tiles_pitch) return set_error(OB200_ERR_TOO_LARGE, "conv tower: %d tiles exceed the flag pitch %d", p.num_tiles, tiles_pitch);
    const int grid = p.num_tiles < sms ? p.num_tiles : sms;
    int per_sm = 0;
    OB200_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem));
    if (per_sm < 1 || grid > per_sm * sms)
        return set_error(OB200_ERR_UNSUPPORTED, "conv tower: %d CTAs cannot all be resident", grid);
    OB200_CUDA_OK(cudaMemsetAsync(done, 0, (size_t)n_layers * sizeof(int), st));
    CUtensorMap stem = *reinterpret_cast<const CUtensorMap*>(&stem_in_map);
    void* args[] = {&stem, &p};
    OB200_CUDA_OK(cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(kThreads), args, smem, st));
    OB200_LAUNCHED("conv_tower_kernel");
    return OB200_OK;
}

}  // namespace ob200
