// The 64-filter residual tower with the boards RESIDENT in shared memory (sm_100a).
//
// A board of up to 15x15 cells is at most 256 padded positions x 64 channels = 32 KB in bf16 or fp16, and a
// 3x3 convolution never looks outside its own board (the padded row / column around every board is
// zero).  So a CTA can take a board through ALL the layers without the activations ever leaving the
// SM: two buffers per board (x: block input / residual / block output, y: the middle of a block),
// the layer's output written by the epilogue threads straight into the 128-byte-swizzled layout the
// next layer's MMA descriptors read.  Per tile that removes the TMA load of the input box, the TMA
// load of the residual, the staging tile and the TMA store - 85 KB of shared-memory traffic that
// otherwise competes with the tensor cores' operand reads - and every hand-over through global
// memory.  What is left is the MMA issue rate (128x64x16 tcgen05.mma: 48 cycles each, 36 per tile).
//
//   * Two boards are in flight per CTA, and every 128-row TILE of a board has its own MMA-issuing warp
//     (four issuers for two 15x15 boards): while board 0's layer-l accumulators are drained and written
//     back as layer l+1's input, the tensor cores run board 1's layer l (board 1 runs two thirds of a
//     layer behind board 0).  The thread that issues tcgen05.mma is held by every MMA and pays for every
//     instruction between two of them (descriptor arithmetic, the waits for weights, the commits:
//     56-59 cycles per MMA for one thread, measured, against 48 for the instruction itself) and waits at
//     every layer boundary; with an issuer per tile the tensor cores take the next MMA from whichever
//     thread has one ready.  MMAs of one tile stay in one thread, so their order - and with it every
//     bit of the result - does not depend on the interleaving.  TMEM holds both boards' accumulators
//     for two consecutive layers (2 x 2 boards x 2 tiles x 64 columns = 512).
//   * Weights stream from L2 through a one-layer ring of three 24 KB blocks (three taps each): the
//     MMAs of a tile go tap by tap, a block is handed back by a tcgen05.commit of every issuer, and
//     the loader refills it with the same taps of the next layer when all have come in (it stands in
//     for the issuers of an absent second board).
//   * Boards are assigned statically: CTA c takes boards c, c + grid, c + 2 grid, ... two at a time.
//     The first input of a board arrives by TMA into y, the tower's output leaves by TMA from x.
//   * The last layer's epilogue has a position's 64 output channels at hand and, when asked to, also
//     computes the policy / value heads' 1x1 convolutions (up to four head channels) for it.
//   * Given Gomoku move histories instead of an input tensor, the epilogue threads write a board's
//     input planes straight into its buffer (a position's row is 17 ones or zeros): no encoder launch,
//     no input tensor in HBM.
// There is no communication between CTAs, so this is an ordinary launch (and may be captured in a
// graph).  Every wait is bounded; a thread that gives up raises the device error word.
// Measured (15x15, 21 layers, B200): about 7,400 cycles per layer for a pair of boards (four tiles), against
// 6,912 for the MMAs alone, and about 5,450 for a lone board; 320-332 us for 1,024 boards (1,037-1,074 TFLOP/s)
// and 1,174 us for 4,096 (1,173 TFLOP/s) where a launch per layer takes 466 / 1,650 us; 74-79 us for 1 to
// 148 boards (93-140 us as a launch per layer).
#include "internal.h"
#include "sm100_ptx.cuh"
#include <cstring>

namespace ob200 {
namespace {

constexpr int kTileM = 128;
constexpr int kC = 64;
constexpr int kRowBytes = kC * 2;
constexpr int kTapBytes = kC * kRowBytes;            // 8,192: one tap of one layer
constexpr int kSlotRows = 256;                       // rows reserved per board
constexpr int kGuardRows = 24;                       // zero rows before / between / after the two boards (>= S + 2)
constexpr int kBufRows = 3 * kGuardRows + 2 * kSlotRows;     // 584
constexpr int kBufBytes = kBufRows * kRowBytes;      // 74,752
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 8;                         // two groups of four: group g drains tile g of the board
constexpr int kIssuers = 4;                          // warp w < 4 issues the MMAs of board w / 2, tile w % 2
constexpr int kThreads = 32 * kIssuers + 32 * kEpiWarps + 32;   // warps 0-3: MMA issue, warps 4-11: epilogue, warp 12: weight loader
constexpr int kStaggerTap = 6;                       // board 1 starts a layer when board 0 has issued this tap of it
constexpr int kWGroups = 3;                          // the weight ring is handed over in groups of three taps
constexpr int kWGroupBytes = 3 * kTapBytes;          // 24,576
constexpr int kNumBars = 2 + 2 + 4 + kWGroups + kWGroups + 2 + 2 + 1;

struct alignas(32) ResidentLayer {
    const uint8_t* w;         // packed weights (ob200_pack_conv3x3_weights): 9 taps x 8 KB
    const float* bias;        // [64]
    int has_res;
    int pad_[3];
};

constexpr int kHeadMax = 4;                          // head channels the last epilogue can take along

struct ResidentParams {
    const ResidentLayer* layers;
    int n_layers;
    int B, S, GP, slots;
    int* error;
    // optional: the heads' 1x1 convolutions (+ folded BatchNorm, ReLU) on the tower's output, done by the last
    // layer's epilogue while the row is at hand.  head_ch == 0: none.
    const float* head_w;      // [head_ch][64]
    const float* head_b;      // [head_ch]
    int head_ch, head_pc;     // channels in all, and how many of them belong to the policy head
    float* hp;                // [B][head_pc][S*S]
    float* hv;                // [B][head_ch - head_pc][S*S]
    // optional: the tower's input comes from Gomoku move histories instead of an input tensor - the epilogue
    // threads write each board's input rows themselves (the planes of ob200_launch_encode_gomoku).  enc_hist == null: off.
    const int16_t* enc_hist;  // [B][16] k-th most recent move
    const uint8_t* enc_nh;    // [B]
    const uint8_t* enc_tm;    // [B] 1 BLACK, 2 WHITE
    int enc_planes;           // 17 or 19
};

using namespace ptx;

// One 128-byte row of a layer's output: relu(accumulator + bias [+ residual]).
// 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r % 8).
// The residual is the row's old content; res holds it (chunk c in res[c]), read by load_row before the layer's
// accumulators were waited for: the row has held the block's input since this very thread wrote it two layers ago.
__device__ __forceinline__ void load_row(const uint8_t* src_row, int row, uint4 (&res)[8]) {
#pragma unroll
    for (int c = 0; c < 8; ++c) res[c] = *reinterpret_cast<const uint4*>(src_row + ((c ^ (row & 7)) << 4));
}
// C0: the first of the four chunks (32 channels) covered, r holding their accumulators.
template <bool RES, bool F16, int C0>
__device__ __forceinline__ void store_half_row(uint8_t* dst_row, int row, const uint32_t* r_in, const float* bias_t, const uint4 (&res)[8]) {
    const uint32_t* r = r_in - C0 * 8;
#pragma unroll
    for (int c = C0; c < C0 + 4; ++c) {
        uint4* slot = reinterpret_cast<uint4*>(dst_row + ((c ^ (row & 7)) << 4));
        const float4 b0 = *reinterpret_cast<const float4*>(bias_t + c * 8), b1 = *reinterpret_cast<const float4*>(bias_t + c * 8 + 4);
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint32_t rw[4] = {0u, 0u, 0u, 0u};
        if (RES) { rw[0] = res[c].x; rw[1] = res[c].y; rw[2] = res[c].z; rw[3] = res[c].w; }
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v0 = __uint_as_float(r[c * 8 + 2 * j]) + bb[2 * j];
            float v1 = __uint_as_float(r[c * 8 + 2 * j + 1]) + bb[2 * j + 1];
            if (RES) { float r0, r1; unpack2<F16>(rw[j], r0, r1); v0 += r0; v1 += r1; }
            ow[j] = pack2_relu<F16>(v0, v1);
        }
        *slot = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}
// The input row of one position from the board's move history, as encode_gomoku_board_kernel writes it
// (GomokuState::getEnhancedTensorRepresentation, reference src/games/gomoku/gomoku_state.cpp:223-262): plane p < 16
// is one where move k = p + 1 (p even) / p - 1 (p odd) of the history was played, plane 16 is one everywhere iff
// BLACK is to move, planes 17 / 18 (attack / defense) are zero as the reference's CPU code computes them.
template <bool F16>
__device__ __forceinline__ void write_input_row(uint8_t* dst_row, int row, bool valid, int cell, const int16_t* hist, int nh, int tm, int planes) {
    uint32_t w[12] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};     // channels 0-23, two per word
    if (valid) {
        const uint4 ha = __ldg(reinterpret_cast<const uint4*>(hist)), hb = __ldg(reinterpret_cast<const uint4*>(hist) + 1);
        const uint32_t hw[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
        const uint32_t one = F16 ? 0x3C00u : 0x3F80u;
#pragma unroll
        for (int pl = 0; pl < 16; ++pl) {
            const int k = (pl & 1) ? pl - 1 : pl + 1;
            const int hk = (int)(int16_t)((k & 1) ? (hw[k >> 1] >> 16) : (hw[k >> 1] & 0xffffu));
            if (k < nh && hk == cell) w[pl >> 1] |= one << ((pl & 1) * 16);
        }
        if (planes > 16 && tm == 1) w[8] = one;
    }
#pragma unroll
    for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(dst_row + ((c ^ (row & 7)) << 4)) =
            c < 3 ? make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]) : make_uint4(0u, 0u, 0u, 0u);
}
// The heads' 1x1 convolutions for one position, from the row just written (16-bit, as the head kernel would
// read it from the tower's output tensor).  Same order of additions as head_conv_kernel: eight partial sums
// over eight consecutive channels each, added as ((0+1)+(2+3))+((4+5)+(6+7)), then the bias, then ReLU.
template <bool F16>
__device__ __noinline__ void head_row(const uint8_t* row_ptr, int row, const float* head_s, int head_ch, int head_pc,
                                      int board, int S, int GP, float* hp, float* hv) {
    float a[kC];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(row_ptr + ((c ^ (row & 7)) << 4));
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            unpack2<F16>(w4[j], a[c * 8 + 2 * j], a[c * 8 + 2 * j + 1]);
        }
    }
    const int y = row / GP, x = row - y * GP, S2 = S * S, cell = y * S + x;
    for (int h = 0; h < head_ch; ++h) {
        const float* wh = head_s + h * kC;
        float part[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) acc = fmaf(a[j * 8 + k], wh[j * 8 + k], acc);
            part[j] = acc;
        }
        const float sum = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
        const float o = fmaxf(sum + head_s[kHeadMax * kC + h], 0.0f);
        if (h < head_pc) hp[((size_t)board * head_pc + h) * S2 + cell] = o;
        else hv[((size_t)board * (head_ch - head_pc) + (h - head_pc)) * S2 + cell] = o;
    }
}
__device__ __forceinline__ void store_zero_row(uint8_t* dst_row) {
#pragma unroll
    for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(dst_row)[c] = make_uint4(0u, 0u, 0u, 0u);
}

// T: 128-row tiles per board (1 for boards up to 10x10, 2 up to 15x15).
// PAIR: CTAs take their boards two at a time (the general case).  When no CTA has more than one board
// (batches up to the SM count) the barriers count the issuers of one board only.
// F16: the boards and weights are fp16 instead of bf16 (same instruction, other operand-format bits).
template <int T, bool PAIR, bool F16>
__global__ void __launch_bounds__(kThreads, 1)
conv_tower_resident_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                           const ResidentParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* x_s = smem;                                   // [guard][board 0][guard][board 1][guard]
    uint8_t* y_s = x_s + kBufBytes;
    uint8_t* w_s = y_s + kBufBytes;                        // nine tap blocks of the current / next layer
    float* bias_s = reinterpret_cast<float*>(w_s + 9 * kTapBytes);   // [n_layers][64]
    float* head_s = bias_s + p.n_layers * kC;                        // [kHeadMax][64] weights, [kHeadMax] biases
    uint64_t* bars = reinterpret_cast<uint64_t*>(head_s + kHeadMax * kC + kHeadMax);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kIdesc = make_idesc(F16, kTileM, kC);
    const uint32_t bar0 = smem_u32(bars);
    auto in_full = [&](int bd) { return bar0 + 8u * bd; };               // the board's first input has landed in y
    auto act_ready = [&](int bd) { return bar0 + 8u * (2 + bd); };       // the previous layer's output is written
    auto acc_full = [&](int bd, int tile) { return bar0 + 8u * (4 + 2 * bd + tile); };   // the tile's MMAs of this layer are complete
    auto w_full = [&](int g) { return bar0 + 8u * (8 + g); };
    auto w_empty = [&](int g) { return bar0 + 8u * (8 + kWGroups + g); };
    auto out_written = [&](int bd) { return bar0 + 8u * (8 + 2 * kWGroups + bd); };    // the tower's output is complete in x
    auto x_free = [&](int bd) { return bar0 + 8u * (10 + 2 * kWGroups + bd); };        // the output store has read x
    const uint32_t stagger = bar0 + 8u * (12 + 2 * kWGroups);                          // board 0 is far enough into the layer

    if (threadIdx.x == 0) {
        for (int bd = 0; bd < 2; ++bd) {
            mbar_init(in_full(bd), p.enc_hist ? 4 * T : 1); mbar_init(act_ready(bd), 4 * T);
            mbar_init(acc_full(bd, 0), 1); mbar_init(acc_full(bd, 1), 1);
            mbar_init(out_written(bd), 4 * T); mbar_init(x_free(bd), 1);
        }
        // a weight block comes back from every issuer of a full round
        for (int g = 0; g < kWGroups; ++g) { mbar_init(w_full(g), 1); mbar_init(w_empty(g), (PAIR ? 2 : 1) * T); }
        mbar_init(stagger, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&in_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&out_map) : "memory");
    }
    // guards, and the rows of a slot beyond the board, are zero for the kernel's lifetime
    for (int i = threadIdx.x; i < 2 * kBufBytes / 16; i += kThreads) reinterpret_cast<uint4*>(x_s)[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < p.n_layers * kC; i += kThreads) bias_s[i] = p.layers[i / kC].bias[i % kC];
    for (int i = threadIdx.x; i < p.head_ch * kC; i += kThreads) head_s[i] = p.head_w[i];
    if ((int)threadIdx.x < p.head_ch) head_s[kHeadMax * kC + threadIdx.x] = p.head_b[threadIdx.x];
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the zeros -> reads by the tensor cores / TMA
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // this CTA's boards: blockIdx.x, + gridDim.x, ...; two per round
    const int n_my = ((int)blockIdx.x < p.B) ? (p.B - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int rounds = (n_my + 1) / 2;
    const int L = p.n_layers;
    auto board_of = [&](int round, int bd) { return (int)blockIdx.x + (2 * round + bd) * (int)gridDim.x; };
    auto slot_off = [&](int bd) { return (uint32_t)((kGuardRows + bd * (kSlotRows + kGuardRows)) * kRowBytes); };

    if (warp == kIssuers + kEpiWarps) {
        // ---------------- weight loader ----------------
        // constants of the network: may start before the kernels ahead of this one in the stream are complete
        if (lane == 0) {
            const int total = rounds * L;
            bool ok = true;
            for (int it = 0; ok && it < total; ++it) {
                const uint8_t* src = p.layers[it % L].w;
                // a block comes back from every issuer; in a round with a single board (the last one, when the
                // CTA's board count is odd) the loader stands in for the issuers of the missing board
                const bool prev_alone = PAIR && it > 0 && (n_my & 1) && (it - 1) / L == rounds - 1;
                for (int g = 0; g < kWGroups; ++g) {
                    if (prev_alone)
                        for (int k = 0; k < T; ++k) mbar_arrive(w_empty(g));
                    if (it > 0 && !mbar_wait(w_empty(g), (uint32_t)(it - 1) & 1u, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(w_full(g), (uint32_t)kWGroupBytes);
                    bulk_g2s(smem_u32(w_s + g * kWGroupBytes), src + (size_t)g * kWGroupBytes, (uint32_t)kWGroupBytes, w_full(g));
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 4); }
        }
    } else if (warp < kIssuers) {
        // ---------------- MMA issuers: warp w for board w / 2, tile w % 2 ----------------
        // Board 1 runs two thirds of a layer behind board 0 (its issuers start a layer when board 0's first
        // issuer has issued tap kStaggerTap), so that one board's MMAs cover the other's epilogue; every
        // issuer hands the weight blocks back, and the loader waits for all of them.
        const int bd = warp >> 1, tile = warp & 1;
        if (lane == 0 && tile < T && (PAIR || bd == 0)) {
            int tap_off[9];
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) tap_off[tap] = ((tap / 3) * p.GP + (tap % 3)) * (kRowBytes >> 4);
            // descriptor of the row GP + 1 rows above the tile's first row (tap 0 of its position 0), per buffer
            const uint32_t tile_off = (uint32_t)(tile * kTileM * kRowBytes) - (uint32_t)((p.GP + 1) * kRowBytes);
            const uint32_t a_base_x = desc_lo(smem_u32(x_s) + slot_off(bd) + tile_off);
            const uint32_t a_base_y = desc_lo(smem_u32(y_s) + slot_off(bd) + tile_off);
            const uint32_t w_lo = desc_lo(smem_u32(w_s));
            uint32_t ready_cnt = 0u, stagger_cnt = 0u;
            bool ok = true;
            int it = 0;
            for (int round = 0; ok && round < rounds; ++round) {
                const int nb = n_my - 2 * round >= 2 ? 2 : 1;
                if (bd >= nb) break;                    // a single board in the last round: board 1's issuers are done
                for (int l = 0; ok && l < L; ++l, ++it) {
                    const uint32_t a_lo = (l == 0 || !(l & 1)) ? a_base_y : a_base_x;   // stem and second convolutions read y, first ones x
                    if (l == 0) {
                        if (!mbar_wait(in_full(bd), (uint32_t)round & 1u, abort_flag)) { ok = false; break; }
                    } else {
                        if (!mbar_wait(act_ready(bd), ready_cnt & 1u, abort_flag)) { ok = false; break; }
                        ++ready_cnt;
                    }
                    if (bd == 1) {
                        if (!mbar_wait(stagger, stagger_cnt & 1u, abort_flag)) { ok = false; break; }
                        ++stagger_cnt;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_tmem = tmem_base + (uint32_t)((it & 1) * 256 + bd * 128 + tile * kC);
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        // weights are waited for and handed back three taps at a time (a wait costs the issuing
                        // thread about 50 cycles, a commit 25)
                        if (tap % 3 == 0) {
                            if (!mbar_wait(w_full(tap / 3), (uint32_t)it & 1u, abort_flag)) { ok = false; break; }
                        }
#pragma unroll
                        for (int ks = 0; ks < kC / 16; ++ks)
                            umma(d_tmem, a_lo + (uint32_t)(tap_off[tap] + ks * 2),
                                 w_lo + (uint32_t)(tap * (kTapBytes >> 4) + ks * 2), kIdesc, (tap | ks) ? 1u : 0u);
                        if (tap % 3 == 2) umma_commit(w_empty(tap / 3));
                        if (PAIR && tap == kStaggerTap && warp == 0) mbar_arrive(stagger);
                    }
                    if (!ok) break;
                    umma_commit(acc_full(bd, tile));
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.error, 2); }
        }
    } else if (warp - kIssuers < 4 * T) {
        // ---------------- epilogue: TMEM -> registers -> the next layer's input rows ----------------
        // group g (four warps, one per TMEM lane quadrant) drains tile g as soon as that tile's MMAs are complete
        asm volatile("griddepcontrol.wait;" ::: "memory");   // inputs come from the kernels ahead in the stream
        const int group = (warp - kIssuers) >> 2;
        const int q = warp & 3;                          // TMEM lane quadrant this warp may read
        const int row = group * kTileM + q * 32 + lane;  // row within the board's slot
        const bool valid = row < p.slots && (row / p.GP < p.S) && (row % p.GP < p.S);
        const bool elected = warp == kIssuers && lane == 0;     // issues the boards' loads and stores
        const uint32_t in_bytes = (uint32_t)p.slots * kRowBytes;
        bool ok = true;
        const bool encode = p.enc_hist != nullptr;
        const int cell = (row / p.GP) * p.S + row % p.GP;
        // a board's input: by TMA from the input tensor, or written here from its move history
        auto encode_board = [&](int board, int bd) {
            write_input_row<F16>(y_s + slot_off(bd) + row * kRowBytes, row, valid, cell, p.enc_hist + (size_t)board * 16,
                                 p.enc_nh[board], p.enc_tm[board], p.enc_planes);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // rows -> the tensor cores' reads
            __syncwarp();
            if (lane == 0) mbar_arrive(in_full(bd));
        };
        if (encode) {
            for (int bd = 0; bd < 2 && bd < n_my; ++bd) encode_board(board_of(0, bd), bd);
        } else if (elected) {
            for (int bd = 0; bd < 2 && bd < n_my; ++bd) {
                mbar_arrive_expect_tx(in_full(bd), in_bytes);
                tma_load_2d(smem_u32(y_s) + slot_off(bd), &in_map, 0, OB200_GUARD + board_of(0, bd) * p.slots, in_full(bd));
            }
        }
        uint32_t full_cnt0 = 0u, full_cnt1 = 0u;
        int it = 0;
        for (int round = 0; ok && round < rounds; ++round) {
            const int nb = n_my - 2 * round >= 2 ? 2 : 1;
            for (int l = 0; ok && l < L; ++l, ++it) {
                const bool has_res = p.layers[l].has_res != 0;
                const bool to_x = l == 0 || !(l & 1);
                const float* bias_t = bias_s + l * kC;
                for (int bd = 0; bd < nb; ++bd) {
                    uint8_t* dst_row = (to_x ? x_s : y_s) + slot_off(bd) + row * kRowBytes;
                    uint4 res[8];
                    if (has_res && valid) load_row(dst_row, row, res);      // while the tile's MMAs still run
                    // every wait's outcome is voted on, so that a warp gives up as a whole (the TMEM loads below
                    // need all 32 lanes; the elected lane may come late from its store)
                    bool good = mbar_wait(acc_full(bd, group), (bd ? full_cnt1 : full_cnt0) & 1u, abort_flag);
                    if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
                    if (bd) ++full_cnt1; else ++full_cnt0;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // the row goes in two halves of 32 channels: half the accumulators in registers at a time
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((it & 1) * 256 + bd * 128 + group * kC);
                    tmem_ld32(taddr, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (l == 0 && round > 0) {
                        // x still holds the previous round's output until its store has read it
                        if (elected) {
                            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            mbar_arrive(x_free(bd));
                        }
                        good = mbar_wait(x_free(bd), (uint32_t)(round - 1) & 1u, abort_flag);
                        if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
                    }
                    if (!valid) store_zero_row(dst_row);
                    else if (has_res) store_half_row<true, F16, 0>(dst_row, row, r, bias_t, res);
                    else store_half_row<false, F16, 0>(dst_row, row, r, bias_t, res);
                    tmem_ld32(taddr + 32, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (!valid) {}
                    else if (has_res) store_half_row<true, F16, 4>(dst_row, row, r, bias_t, res);
                    else store_half_row<false, F16, 4>(dst_row, row, r, bias_t, res);
                    if (l + 1 == L && p.head_ch > 0 && valid)
                        head_row<F16>(dst_row, row, head_s, p.head_ch, p.head_pc, board_of(round, bd), p.S, p.GP, p.hp, p.hv);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // rows -> the tensor cores' / the store's reads
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (l + 1 < L) {
                        if (lane == 0) mbar_arrive(act_ready(bd));
                    } else {
                        if (lane == 0) mbar_arrive(out_written(bd));
                        const bool successor = 2 * (round + 1) + bd < n_my;
                        // the board is through when every warp has drained its tile: y is free then (both tiles' last MMAs
                        // are complete) and the successor may come in
                        if (elected || (encode && successor)) good = mbar_wait(out_written(bd), (uint32_t)round & 1u, abort_flag);
                        if (elected && good) {
                            tma_store_2d(&out_map, 0, OB200_GUARD + board_of(round, bd) * p.slots, smem_u32(x_s) + slot_off(bd));
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            if (successor && !encode) {
                                mbar_arrive_expect_tx(in_full(bd), in_bytes);
                                tma_load_2d(smem_u32(y_s) + slot_off(bd), &in_map, 0, OB200_GUARD + board_of(round + 1, bd) * p.slots,
                                            in_full(bd));
                            }
                        }
                        if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
                        if (encode && successor) encode_board(board_of(round + 1, bd), bd);
                    }
                }
            }
        }
        if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the output stores are complete
        if (!ok) { *abort_flag = 1; atomicExch(p.error, 3); }
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);    // copies in flight into shared memory land first
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

}  // namespace

size_t tower_resident_layer_bytes() { return sizeof(ResidentLayer); }

void tower_resident_fill_layer(void* dst, const void* w, const float* bias, int has_res) {
    ResidentLayer d;
    std::memset(&d, 0, sizeof(d));
    d.w = static_cast<const uint8_t*>(w); d.bias = bias; d.has_res = has_res;
    std::memcpy(dst, &d, sizeof(d));
}

// Rows of the load / store boxes: one whole board.
int tower_resident_box_rows(int S) { return (S + 1) * (S + 1); }

// Shared memory the kernel needs, or 0 when the board or the depth does not fit.
size_t tower_resident_smem_bytes(int S, int n_layers) {
    if (S < 1 || (S + 1) * (S + 1) > kSlotRows || S + 2 > kGuardRows || n_layers < 1) return 0;
    const size_t total = 2 * (size_t)kBufBytes + 9 * (size_t)kTapBytes + (size_t)n_layers * kC * 4 + (kHeadMax * kC + kHeadMax) * 4 +
                         kNumBars * 8 + 16 + 1024;
    return total <= 232448 ? total : 0;
}

// The whole tower in one ordinary launch.  in_map / out_map: boxes of tower_resident_box_rows(S)
// rows over the 64-channel input tensor and the output tensor; layers_dev: n_layers descriptors on
// the device.
int tower_resident_head_channels_max() { return kHeadMax; }

// heads (optional, head_ch in 1..tower_resident_head_channels_max()): the heads' 1x1 convolutions on the
// tower's output ride along in the last epilogue; results as launch_head_conv writes them.
int launch_conv_tower_resident(const BoardTensorMap& in_map, const BoardTensorMap& out_map, const void* layers_dev,
                               int n_layers, int B, int S, cudaStream_t st, const float* head_w, const float* head_b,
                               int head_ch, int head_pc, float* hp, float* hv, int dtype, const int16_t* enc_hist,
                               const uint8_t* enc_nh, const uint8_t* enc_tm, int enc_planes) {
    if (enc_hist && (!enc_nh || !enc_tm || (enc_planes != 17 && enc_planes != 19) || ((uintptr_t)enc_hist & 15)))
        return set_error(OB200_ERR_INVALID, "resident tower: bad move-history arguments (17 or 19 planes, histories 16-byte aligned)");
    if (!layers_dev || n_layers < 1 || B <= 0) return set_error(OB200_ERR_INVALID, "resident tower: bad arguments");
    if (head_ch < 0 || head_ch > kHeadMax || head_pc < 0 || head_pc > head_ch ||
        (head_ch > 0 && (!head_w || !head_b || (head_pc > 0 && !hp) || (head_pc < head_ch && !hv))))
        return set_error(OB200_ERR_INVALID, "resident tower: bad head arguments");
    const size_t smem = tower_resident_smem_bytes(S, n_layers);
    if (!smem) return set_error(OB200_ERR_UNSUPPORTED, "resident tower: board size %d / %d layers do not fit shared memory", S, n_layers);
    if (int rc = require_device()) return rc;
    int dev = 0, sms = 0;
    OB200_CUDA_OK(cudaGetDevice(&dev));
    OB200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int slots = (S + 1) * (S + 1);
    const bool two_tiles = slots > kTileM;
    const bool pair = B > sms;          // some CTA has two boards or more
    const bool f16 = dtype == OB200_DTYPE_F16;
    auto kernel = f16 ? (two_tiles ? (pair ? conv_tower_resident_kernel<2, true, true> : conv_tower_resident_kernel<2, false, true>)
                                   : (pair ? conv_tower_resident_kernel<1, true, true> : conv_tower_resident_kernel<1, false, true>))
                      : (two_tiles ? (pair ? conv_tower_resident_kernel<2, true, false> : conv_tower_resident_kernel<2, false, false>)
                                   : (pair ? conv_tower_resident_kernel<1, true, false> : conv_tower_resident_kernel<1, false, false>));
    static size_t configured[64][8] = {{0}};
    const int variant = f16 * 4 + two_tiles * 2 + pair;
    if (dev >= 0 && dev < 64 && configured[dev][variant] < smem) {
        OB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][variant] = smem;
    }
    ResidentParams p;
    p.layers = static_cast<const ResidentLayer*>(layers_dev); p.n_layers = n_layers; p.B = B; p.S = S; p.GP = S + 1; p.slots = slots;
    p.error = device_error_word();
    if (!p.error) return set_error(OB200_ERR_CUDA, "resident tower: cannot resolve the device error word");
    p.head_w = head_w; p.head_b = head_b; p.head_ch = head_ch; p.head_pc = head_pc; p.hp = hp; p.hv = hv;
    p.enc_hist = enc_hist; p.enc_nh = enc_nh; p.enc_tm = enc_tm; p.enc_planes = enc_planes;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(B < sms ? B : sms); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const CUtensorMap& im = *reinterpret_cast<const CUtensorMap*>(&in_map);
    const CUtensorMap& om = *reinterpret_cast<const CUtensorMap*>(&out_map);
    OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, im, om, p));
    OB200_LAUNCHED("conv_tower_resident_kernel");
    return OB200_OK;
}

}  // namespace ob200
