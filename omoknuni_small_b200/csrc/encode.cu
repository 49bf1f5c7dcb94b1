// Leaf state -> 16-bit board tensor (bf16, or fp16 when the launcher is given that type; sm_100a).
//
// Output format (see "Board tensors" in omoknuni_b200.h): NHWC, positions on a
// (S+1) x (S+1) grid per board whose last column / row are zero, guard
// positions before and after.  Stores are 16 bytes wide, consecutive threads
// consecutive addresses; the kernels also write the zero padding, so the output
// needs no memset.
#include "internal.h"
#include "sm100_ptx.cuh"
#include <mutex>

namespace ob200 {
namespace {

struct alignas(16) Pack8 { uint16_t v[8]; };
using ptx::store16;
constexpr size_t kMaxBoardSmem = 200 * 1024;   // a board's block must fit a CTA's shared memory
constexpr int kMaxDevices = 64;

// Gomoku planes from the move history; reference semantics in
// GomokuState::getEnhancedTensorRepresentation
// (src/games/gomoku/gomoku_state.cpp:223-262): the k-th most recent move is
// the opponent's for even k and the side to move's for odd k; plane 2i holds
// the side to move's i-th most recent stone, plane 2i+1 the opponent's.
// Hence plane p takes move k = p + 1 (p even) or p - 1 (p odd).
constexpr int kEncThreads = 128;
__global__ void __launch_bounds__(kEncThreads)
encode_gomoku_kernel(const int16_t* __restrict__ history, const uint8_t* __restrict__ n_hist,
                     const uint8_t* __restrict__ to_move, int B, int S, int planes, int chunks,
                     int chunk_shift, int cover, int f16, Pack8* __restrict__ out) {
    // cover = positions written (guards included); chunks = channels / 8 (chunk_shift = log2 when it
    // is a power of two, else -1).  Phase 1: a thread works out the 24 plane channels of one
    // position.  Phase 2: the block writes its 128 positions as 16-byte stores, consecutive threads
    // consecutive addresses; channels past 24 are zero.
    __shared__ Pack8 stage[kEncThreads][3];
    const int base = blockIdx.x * kEncThreads;
    const int pidx = base + threadIdx.x;
    Pack8 o[3];
#pragma unroll
    for (int c = 0; c < 3; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j) o[c].v[j] = (uint16_t)0;
    const int p = pidx - OB200_GUARD;
    const int GP = S + 1, slots = GP * GP;
    if (p >= 0 && p < B * slots) {
        const int b = p / slots, r = p - b * slots;
        const int y = r / GP, x = r - y * GP;
        if (y < S && x < S) {
            const int cell = y * S + x;
            const int nh = n_hist[b];
            // the board's 16 history entries as two 16-byte loads (the launcher checks alignment)
            const uint4* h4 = reinterpret_cast<const uint4*>(history + (size_t)b * 16);
            const uint4 ha = __ldg(h4), hb = __ldg(h4 + 1);
            const uint32_t hw[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
            for (int plane = 0; plane < 16; ++plane) {
                const int k = (plane & 1) ? plane - 1 : plane + 1;
                const int hk = (int)(int16_t)((k & 1) ? (hw[k >> 1] >> 16) : (hw[k >> 1] & 0xffffu));
                if (k < nh && hk == cell) o[plane >> 3].v[plane & 7] = store16(1.0f, f16);
            }
            // plane 16: colour.  Planes 17 / 18 (attack / defense): zero, as the reference's CPU
            // code yields for every legal move (src/utils/attack_defense_module.cpp:96-154).
            if (planes > 16 && to_move[b] == 1) o[2].v[0] = store16(1.0f, f16);
        }
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) stage[threadIdx.x][c] = o[c];
    __syncthreads();
    const int n_pos = min(kEncThreads, cover - base);
    const int n = n_pos * chunks;
    Pack8 zero;
#pragma unroll
    for (int j = 0; j < 8; ++j) zero.v[j] = (uint16_t)0;
    Pack8* dst = out + (size_t)base * chunks;
    for (int idx = threadIdx.x; idx < n; idx += kEncThreads) {
        const int pl = chunk_shift >= 0 ? idx >> chunk_shift : idx / chunks;
        const int ch = idx - pl * chunks;
        dst[idx] = ch < 3 ? stage[pl][ch] : zero;
    }
}

// The same planes, a CTA per board: the board's (S+1)^2 x C block of the tensor is built in
// shared memory (zero fill, then one 2-byte store per history stone and per cell of the colour
// plane) and leaves as one bulk copy.  Blocks B and B + 1 zero the guard positions before the
// first and after the last board.
__global__ void __launch_bounds__(256)
encode_gomoku_board_kernel(const int16_t* __restrict__ history, const uint8_t* __restrict__ n_hist,
                           const uint8_t* __restrict__ to_move, int B, int S, int planes, int C, int cover, int f16,
                           uint8_t* __restrict__ out) {
    extern __shared__ __align__(128) uint8_t board_s[];
    const int GP = S + 1, slots = GP * GP, S2 = S * S;
    const int row_bytes = C * 2;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    if ((int)blockIdx.x >= B) {
        const long long first = (int)blockIdx.x == B ? 0 : (long long)OB200_GUARD + (long long)B * slots;
        const long long last = (int)blockIdx.x == B ? OB200_GUARD : cover;
        uint4* o16 = reinterpret_cast<uint4*>(out);
        for (long long i = first * row_bytes / 16 + threadIdx.x; i < last * row_bytes / 16; i += blockDim.x) o16[i] = z;
        return;
    }
    const int bytes = slots * row_bytes;
    uint4* s16 = reinterpret_cast<uint4*>(board_s);
    for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) s16[i] = z;
    __syncthreads();
    const int b = blockIdx.x;
    uint16_t* sb = reinterpret_cast<uint16_t*>(board_s);
    const uint16_t one = store16(1.0f, f16);
    if (threadIdx.x < 16) {
        const int plane = threadIdx.x;
        const int k = (plane & 1) ? plane - 1 : plane + 1;
        if (k < (int)n_hist[b]) {
            const int cell = history[(size_t)b * 16 + k];
            if (cell >= 0 && cell < S2) {
                const int y = cell / S, x = cell - y * S;
                sb[(y * GP + x) * C + plane] = one;
            }
        }
    }
    // plane 16: colour.  Planes 17 / 18 (attack / defense) stay zero, as the reference's CPU code
    // yields for every legal move (src/utils/attack_defense_module.cpp:96-154).
    if (planes > 16 && to_move[b] == 1) {
        for (int cell = threadIdx.x; cell < S2; cell += blockDim.x) {
            const int y = cell / S, x = cell - y * S;
            sb[(y * GP + x) * C + 16] = one;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> bulk copy engine
    __syncthreads();
    if (threadIdx.x == 0) {
        uint8_t* dst = out + ((size_t)OB200_GUARD + (size_t)b * slots) * row_bytes;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                     "r"((uint32_t)__cvta_generic_to_shared(board_s)), "r"((uint32_t)bytes)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory read before the CTA ends
    }
}

// Go planes (GoState::getEnhancedTensorRepresentation, src/games/go/go_state.cpp:596-704, with the
// CPU code of computeAttackDefensePlanes, :1306-1476), a CTA per board:
//   0 black stones, 1 white stones, 2 all ones iff black is to move, 3 / 4 min(1, liberties / 10) of
//   the black / white group on its stones, 5 ko point, 6 / 7 distance to the nearer edge over S/2,
//   8 min(1, capture / 5), 9 min(1, defense) on the legal cells.
// Groups: every stone starts as its own label; labels fall to the minimum over same-coloured
// neighbours and are compressed (label = label[label]) until nothing changes, which takes a few
// rounds per board rather than one per stone of the longest chain.  Liberties: every empty cell
// adds one to each distinct group beside it.  The board's (S+1)^2 x C block of the tensor is built
// in shared memory and leaves as one bulk copy, as in encode_gomoku_board_kernel.
constexpr int kGoThreads = 256;
constexpr int kGoMaxCells = 31 * 31;
__global__ void __launch_bounds__(kGoThreads)
encode_go_kernel(const int8_t* __restrict__ stones, const int32_t* __restrict__ ko_point,
                 const uint8_t* __restrict__ to_move, const uint32_t* __restrict__ legal_bits, int legal_words,
                 int B, int S, int C, int cover, int f16, uint8_t* __restrict__ out) {
    extern __shared__ __align__(128) uint8_t board_s[];
    __shared__ int label[kGoMaxCells];
    __shared__ int gsize[kGoMaxCells];
    __shared__ int glibs[kGoMaxCells];
    __shared__ int8_t st[kGoMaxCells];
    const int GP = S + 1, slots = GP * GP, S2 = S * S;
    const int row_bytes = C * 2;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    if ((int)blockIdx.x >= B) {
        const long long first = (int)blockIdx.x == B ? 0 : (long long)OB200_GUARD + (long long)B * slots;
        const long long last = (int)blockIdx.x == B ? OB200_GUARD : cover;
        uint4* o16 = reinterpret_cast<uint4*>(out);
        for (long long i = first * row_bytes / 16 + threadIdx.x; i < last * row_bytes / 16; i += blockDim.x) o16[i] = z;
        return;
    }
    const int b = blockIdx.x;
    const int bytes = slots * row_bytes;
    uint4* s16 = reinterpret_cast<uint4*>(board_s);
    for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) s16[i] = z;
    for (int p = threadIdx.x; p < S2; p += blockDim.x) {
        const int8_t v = stones[(size_t)b * S2 + p];
        st[p] = v; label[p] = v ? p : -1; gsize[p] = 0; glibs[p] = 0;
    }
    __syncthreads();
    // ---- groups ----
    for (int round = 0; round < S2; ++round) {
        int changed = 0;
        for (int p = threadIdx.x; p < S2; p += blockDim.x) {
            if (!st[p]) continue;
            const int x = p % S, y = p / S;
            int m = label[p];
            if (y > 0 && st[p - S] == st[p]) m = min(m, label[p - S]);
            if (x + 1 < S && st[p + 1] == st[p]) m = min(m, label[p + 1]);
            if (y + 1 < S && st[p + S] == st[p]) m = min(m, label[p + S]);
            if (x > 0 && st[p - 1] == st[p]) m = min(m, label[p - 1]);
            m = min(m, label[m]);                        // compress: labels only ever decrease, a stale read is still valid
            if (m < label[p]) { label[p] = m; changed = 1; }
        }
        if (!__syncthreads_or(changed)) break;
    }
    // every label now names the lowest cell of its group (a fixed point of the rule above)
    for (int p = threadIdx.x; p < S2; p += blockDim.x)
        if (st[p]) atomicAdd(&gsize[label[p]], 1);
    for (int e = threadIdx.x; e < S2; e += blockDim.x) {
        if (st[e]) continue;
        const int x = e % S, y = e / S;
        int seen[4], ns = 0;
        const int nb[4] = {y > 0 ? e - S : -1, x + 1 < S ? e + 1 : -1, y + 1 < S ? e + S : -1, x > 0 ? e - 1 : -1};
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            if (nb[d] < 0 || !st[nb[d]]) continue;
            const int g = label[nb[d]];
            bool dup = false;
            for (int k = 0; k < ns; ++k) dup |= seen[k] == g;
            if (!dup) { seen[ns++] = g; atomicAdd(&glibs[g], 1); }
        }
    }
    __syncthreads();
    // ---- planes ----
    uint16_t* sb = reinterpret_cast<uint16_t*>(board_s);
    const uint16_t one = store16(1.0f, f16);
    const int mover = to_move[b];
    const int ko = ko_point[b];
    const float half = fmaxf(1.0f, __fdiv_rn((float)S, 2.0f));
    for (int p = threadIdx.x; p < S2; p += blockDim.x) {
        const int x = p % S, y = p / S;
        uint16_t* o = sb + (size_t)(y * GP + x) * C;
        const int s = st[p];
        if (s == 1) o[0] = one;
        if (s == 2) o[1] = one;
        if (mover == 1) o[2] = one;
        if (s) o[s == 1 ? 3 : 4] = store16(fminf(1.0f, __fdiv_rn((float)glibs[label[p]], 10.0f)), f16);
        if (p == ko) o[5] = one;
        o[6] = store16(fminf(1.0f, fmaxf(0.0f, __fdiv_rn((float)min(x, S - 1 - x), half))), f16);
        o[7] = store16(fminf(1.0f, fmaxf(0.0f, __fdiv_rn((float)min(y, S - 1 - y), half))), f16);
        if ((legal_bits[(size_t)b * legal_words + (p >> 5)] >> (p & 31)) & 1u) {
            const int nb[4] = {y > 0 ? p - S : -1, x + 1 < S ? p + 1 : -1, y + 1 < S ? p + S : -1, x > 0 ? p - 1 : -1};
            float capture = 0.0f, defense = 0.0f;
            int empty_adj = 0, friendly_adj = 0;
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                if (nb[d] < 0) continue;
                const int q = nb[d], sq = st[q];
                if (!sq) { ++empty_adj; continue; }
                const int g = label[q];
                if (sq != mover) {
                    const int left = glibs[g] - (s == 0 ? 1 : 0);   // liberties other than the move itself
                    if (left == 0) capture = __fadd_rn(capture, (float)gsize[g]);
                    else if (left == 1) capture = __fadd_rn(capture, __fmul_rn((float)gsize[g], 0.5f));
                } else {
                    ++friendly_adj;
                    if (glibs[g] <= 2) defense = __fadd_rn(defense, __fmul_rn(__fsub_rn(3.0f, (float)glibs[g]), 0.5f));
                }
            }
            if (friendly_adj >= 2 && empty_adj <= 1) defense = __fadd_rn(defense, 0.3f);
            o[8] = store16(fminf(1.0f, __fdiv_rn(capture, 5.0f)), f16);
            o[9] = store16(fminf(1.0f, defense), f16);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        uint8_t* dst = out + ((size_t)OB200_GUARD + (size_t)b * slots) * row_bytes;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                     "r"((uint32_t)__cvta_generic_to_shared(board_s)), "r"((uint32_t)bytes)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
}

// Chess planes (ChessState::getEnhancedTensorRepresentation, src/games/chess/chess_state.cpp:745-826,
// with the CPU code of computeAttackDefensePlanes, :1753-1803), a CTA of 64 threads per board, one
// thread per square (square = rank * 8 + file): 0-5 white P N B R Q K, 6-11 black, 12 ones iff white
// to move, 13 0.25 per castling right, 14 en passant square, 15 min(1, halfmove / 100), 16 chess960,
// 17 clamp(occurrences / 3, 0, 1), 18 / 19 on every legal destination min(1, sum / 10) of the values
// (1, 3, 3, 5, 9, 100) of the enemy / own pieces on the 8 squares around it.
__global__ void __launch_bounds__(64)
encode_chess_kernel(const int8_t* __restrict__ pieces, const int32_t* __restrict__ meta,
                    const uint32_t* __restrict__ legal_to, int B, int C, int cover, int f16,
                    uint8_t* __restrict__ out) {
    extern __shared__ __align__(128) uint8_t board_s[];
    __shared__ int8_t pc_s[64];
    constexpr int S = 8, GP = 9, slots = 81;
    const int row_bytes = C * 2;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    if ((int)blockIdx.x >= B) {
        const long long first = (int)blockIdx.x == B ? 0 : (long long)OB200_GUARD + (long long)B * slots;
        const long long last = (int)blockIdx.x == B ? OB200_GUARD : cover;
        uint4* o16 = reinterpret_cast<uint4*>(out);
        for (long long i = first * row_bytes / 16 + threadIdx.x; i < last * row_bytes / 16; i += blockDim.x) o16[i] = z;
        return;
    }
    const int b = blockIdx.x, sq = threadIdx.x;
    const int bytes = slots * row_bytes;
    uint4* s16 = reinterpret_cast<uint4*>(board_s);
    for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) s16[i] = z;
    const int pc = pieces[(size_t)b * 64 + sq];
    pc_s[sq] = (int8_t)pc;
    const int32_t* m = meta + (size_t)b * 6;
    const int mover = m[0], castling_bits = m[1], ep = m[2], halfmove = m[3], chess960 = m[4], reps = m[5];
    __syncthreads();
    const int r0 = sq >> 3, c0 = sq & 7;
    uint16_t* o = reinterpret_cast<uint16_t*>(board_s) + (size_t)(r0 * GP + c0) * C;
    const uint16_t one = store16(1.0f, f16);
    if (pc) o[(pc & 7) - 1 + ((pc & 8) ? 6 : 0)] = one;
    if (mover == 1) o[12] = one;
    o[13] = store16(0.25f * (float)__popc(castling_bits & 15), f16);
    if (sq == ep) o[14] = one;
    o[15] = store16(fminf(1.0f, __fdiv_rn((float)halfmove, 100.0f)), f16);
    if (chess960) o[16] = one;
    o[17] = store16(fminf(1.0f, fmaxf(0.0f, __fdiv_rn((float)reps, 3.0f))), f16);
    if ((legal_to[(size_t)b * 2 + (sq >> 5)] >> (sq & 31)) & 1u) {
        float attack = 0.0f, defense = 0.0f;
#pragma unroll
        for (int dr = -1; dr <= 1; ++dr)
#pragma unroll
            for (int dc = -1; dc <= 1; ++dc) {
                if (!dr && !dc) continue;
                const int r = r0 + dr, c = c0 + dc;
                if (r < 0 || r >= S || c < 0 || c >= S) continue;
                const int q = pc_s[r * 8 + c];
                if (!q) continue;
                const int t = q & 7;
                const float v = t == 1 ? 1.0f : t <= 3 ? 3.0f : t == 4 ? 5.0f : t == 5 ? 9.0f : 100.0f;
                if (((q & 8) ? 2 : 1) != mover) attack = __fadd_rn(attack, v); else defense = __fadd_rn(defense, v);
            }
        o[18] = store16(fminf(1.0f, __fdiv_rn(attack, 10.0f)), f16);
        o[19] = store16(fminf(1.0f, __fdiv_rn(defense, 10.0f)), f16);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        uint8_t* dst = out + ((size_t)OB200_GUARD + (size_t)b * slots) * row_bytes;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                     "r"((uint32_t)__cvta_generic_to_shared(board_s)), "r"((uint32_t)bytes)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
}

// The 3-plane Gomoku representation (GomokuState::getTensorRepresentation,
// src/games/gomoku/gomoku_state.cpp:184-208): channel 0 the stones of the side to move, 1 the
// opponent's, 2 ones iff BLACK is to move.  One thread per (position, 8-channel block).
__global__ void __launch_bounds__(256)
encode_gomoku3_kernel(const int8_t* __restrict__ stones, const uint8_t* __restrict__ to_move, int B, int S, int chunks,
                      long long cover, int f16, Pack8* __restrict__ out) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= cover * chunks) return;
    const long long pidx = gid / chunks;
    const int chunk = (int)(gid - pidx * chunks);
    Pack8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = (uint16_t)0;
    const long long p = pidx - OB200_GUARD;
    const int GP = S + 1, slots = GP * GP;
    if (chunk == 0 && p >= 0 && p < (long long)B * slots) {
        const int b = (int)(p / slots), r = (int)(p - (long long)b * slots);
        const int y = r / GP, x = r - y * GP;
        if (y < S && x < S) {
            const int st = stones[(size_t)b * S * S + y * S + x], me = to_move[b];
            if (st == me) o.v[0] = store16(1.0f, f16);
            else if (st != 0) o.v[1] = store16(1.0f, f16);
            if (me == 1) o.v[2] = store16(1.0f, f16);
        }
    }
    out[gid] = o;
}

__global__ void __launch_bounds__(256)
planes_to_board_tensor_kernel(const float* __restrict__ planes, int B, int C, int S, int chunks,
                              long long cover, int f16, Pack8* __restrict__ out) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= cover * chunks) return;
    const int chunk = (int)(gid % chunks);
    const long long p = gid / chunks - OB200_GUARD;
    const int GP = S + 1, slots = GP * GP;
    Pack8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = (uint16_t)0;
    if (p >= 0 && p < (long long)B * slots) {
        const int b = (int)(p / slots), r = (int)(p % slots);
        const int y = r / GP, x = r % GP;
        if (y < S && x < S) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = chunk * 8 + j;
                if (c < C) o.v[j] = store16(__ldg(planes + (((size_t)b * C + c) * S + y) * S + x), f16);
            }
        }
    }
    out[gid] = o;
}

}  // namespace

int launch_encode_gomoku(const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                         int32_t B, int32_t board_size, int32_t planes, int32_t out_channels,
                         void* board_tensor_out, cudaStream_t stream, int dtype) {
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "encode: bad dtype %d", dtype);
    const int f16 = dtype == OB200_DTYPE_F16;
    if (!history || !n_hist || !to_move || !board_tensor_out || B < 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_gomoku: null pointer or negative batch");
    if (planes != 17 && planes != 19)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_gomoku: planes must be 17 or 19, got %d", planes);
    if (board_size < 5 || board_size > 31 || out_channels < planes || (out_channels & 7))
        return set_error(OB200_ERR_INVALID,
                         "ob200_launch_encode_gomoku: board_size %d must be in [5,31] and out_channels %d a multiple of 8 >= planes",
                         board_size, out_channels);
    if (reinterpret_cast<uintptr_t>(history) & 15)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_gomoku: history must be 16-byte aligned");
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(board_size, B);
    const int chunks = out_channels / 8;
    if (g.PT * chunks > 0x7fffffffLL) return set_error(OB200_ERR_TOO_LARGE, "encode: batch too large");
    const size_t board_bytes = (size_t)(board_size + 1) * (board_size + 1) * out_channels * 2;
    if (board_bytes <= kMaxBoardSmem) {
        // one CTA per board, the board's block staged in shared memory
        static std::once_flag once[kMaxDevices];
        int dev = 0;
        OB200_CUDA_OK(cudaGetDevice(&dev));
        if (dev >= 0 && dev < kMaxDevices)
            std::call_once(once[dev], [] {
                cudaFuncSetAttribute(encode_gomoku_board_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kMaxBoardSmem);
            });
        else if (board_bytes > 48 * 1024)
            OB200_CUDA_OK(cudaFuncSetAttribute(encode_gomoku_board_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)kMaxBoardSmem));
        encode_gomoku_board_kernel<<<(unsigned)(B + 2), 256, board_bytes, stream>>>(
            history, n_hist, to_move, B, board_size, planes, out_channels, (int)g.PT, f16,
            static_cast<uint8_t*>(board_tensor_out));
        OB200_LAUNCHED("encode_gomoku_board_kernel");
        return OB200_OK;
    }
    int chunk_shift = -1;
    for (int sft = 0; sft < 8; ++sft)
        if ((1 << sft) == chunks) chunk_shift = sft;
    encode_gomoku_kernel<<<(unsigned)((g.PT + kEncThreads - 1) / kEncThreads), kEncThreads, 0, stream>>>(
        history, n_hist, to_move, B, board_size, planes, chunks, chunk_shift, (int)g.PT, f16,
        reinterpret_cast<Pack8*>(board_tensor_out));
    OB200_LAUNCHED("encode_gomoku_kernel");
    return OB200_OK;
}

int launch_encode_go(const int8_t* stones, const int32_t* ko_point, const uint8_t* to_move, const uint32_t* legal_bits,
                     int32_t B, int32_t board_size, int32_t out_channels, void* board_tensor_out, cudaStream_t stream, int dtype) {
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "encode: bad dtype %d", dtype);
    const int f16 = dtype == OB200_DTYPE_F16;
    if (!stones || !ko_point || !to_move || !legal_bits || !board_tensor_out || B < 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_go: null pointer or negative batch");
    if (board_size < 2 || board_size > 30 || out_channels < 10 || (out_channels & 7))
        return set_error(OB200_ERR_INVALID,
                         "ob200_launch_encode_go: board_size %d must be in [2,30] and out_channels %d a multiple of 8 >= 10",
                         board_size, out_channels);
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(board_size, B);
    const size_t board_bytes = (size_t)(board_size + 1) * (board_size + 1) * out_channels * 2;
    if (board_bytes > kMaxBoardSmem - 16 * 1024)
        return set_error(OB200_ERR_UNSUPPORTED, "ob200_launch_encode_go: a %dx%d board with %d channels does not fit shared memory",
                         board_size, board_size, out_channels);
    if (board_bytes > 32 * 1024)
        OB200_CUDA_OK(cudaFuncSetAttribute(encode_go_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)board_bytes));
    const int legal_words = (board_size * board_size + 31) / 32;
    encode_go_kernel<<<(unsigned)(B + 2), kGoThreads, board_bytes, stream>>>(
        stones, ko_point, to_move, legal_bits, legal_words, B, board_size, out_channels, (int)g.PT, f16,
        static_cast<uint8_t*>(board_tensor_out));
    OB200_LAUNCHED("encode_go_kernel");
    return OB200_OK;
}

int launch_encode_chess(const int8_t* pieces, const int32_t* meta, const uint32_t* legal_to, int32_t B,
                        int32_t out_channels, void* board_tensor_out, cudaStream_t stream, int dtype) {
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "encode: bad dtype %d", dtype);
    const int f16 = dtype == OB200_DTYPE_F16;
    if (!pieces || !meta || !legal_to || !board_tensor_out || B < 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_chess: null pointer or negative batch");
    if (out_channels < 20 || (out_channels & 7) || out_channels > 256)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_chess: out_channels %d must be a multiple of 8 in [24, 256]", out_channels);
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(8, B);
    const size_t board_bytes = (size_t)81 * out_channels * 2;
    encode_chess_kernel<<<(unsigned)(B + 2), 64, board_bytes, stream>>>(pieces, meta, legal_to, B, out_channels, (int)g.PT, f16,
                                                                         static_cast<uint8_t*>(board_tensor_out));
    OB200_LAUNCHED("encode_chess_kernel");
    return OB200_OK;
}

int launch_encode_gomoku3(const int8_t* stones, const uint8_t* to_move, int32_t B, int32_t board_size, int32_t out_channels,
                          void* board_tensor_out, cudaStream_t stream, int dtype) {
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "encode: bad dtype %d", dtype);
    const int f16 = dtype == OB200_DTYPE_F16;
    if (!stones || !to_move || !board_tensor_out || B < 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_gomoku3: null pointer or negative batch");
    if (board_size < 1 || board_size > 31 || out_channels < 8 || (out_channels & 7))
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_gomoku3: bad board_size %d / out_channels %d", board_size,
                         out_channels);
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(board_size, B);
    const int chunks = out_channels / 8;
    const long long total = g.PT * chunks;
    encode_gomoku3_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(stones, to_move, B, board_size, chunks, g.PT, f16,
                                                                              reinterpret_cast<Pack8*>(board_tensor_out));
    OB200_LAUNCHED("encode_gomoku3_kernel");
    return OB200_OK;
}

int launch_planes_to_board_tensor(const float* planes_nchw, int32_t B, int32_t C, int32_t board_size,
                                  int32_t out_channels, void* board_tensor_out, cudaStream_t stream, int dtype) {
    if (dtype != OB200_DTYPE_BF16 && dtype != OB200_DTYPE_F16) return set_error(OB200_ERR_INVALID, "encode: bad dtype %d", dtype);
    const int f16 = dtype == OB200_DTYPE_F16;
    if (!planes_nchw || !board_tensor_out || B < 0 || C <= 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_planes_to_board_tensor: bad arguments");
    if (board_size < 1 || board_size > 31 || out_channels <= 0 || (out_channels & 7))
        return set_error(OB200_ERR_INVALID, "ob200_launch_planes_to_board_tensor: bad board_size %d / out_channels %d",
                         board_size, out_channels);
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(board_size, B);
    const int chunks = out_channels / 8;
    const long long total = g.PT * chunks;
    planes_to_board_tensor_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        planes_nchw, B, C, board_size, chunks, g.PT, f16, reinterpret_cast<Pack8*>(board_tensor_out));
    OB200_LAUNCHED("planes_to_board_tensor_kernel");
    return OB200_OK;
}

// ---------------------------------------------------------------------------
// Gomoku attack / defense planes (GomokuAttackDefenseModule, src/utils/attack_defense_module.cpp).
// A colour's threat count (:205-222) is the number of windows, over the four line directions, of 5 cells with
// both end cells empty and 3 or 2 of its stones among the 3 between them, plus windows of 6 with 4 or 3 among
// the 4 between (:333-392 rows and columns, :394-487 diagonals; whatever else lies between does not matter).
// For an empty cell m and the side to move p (:61-111, :113-203):
//   attack[m]  = threats(after, p) - threats(before, p),  defense[m] = threats(before, o) - threats(after, o),
// `before` being the board with m empty and `after` the board the module is handed.  compute_planes hands it the
// position itself (m still empty), so both planes come out zero for every cell: stone_placed == 0.  With
// stone_placed != 0 `after` carries p's stone on m, the way the module's own tests call compute_bonuses.
// Only the windows through m differ between the two boards, so a thread visits those: 4 directions x (5 + 6).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gomoku_attack_defense_kernel(const int8_t* __restrict__ stones, const uint8_t* __restrict__ to_move, int B, int S,
                             int stone_placed, float* __restrict__ attack, float* __restrict__ defense) {
    extern __shared__ int8_t board[];
    const int b = blockIdx.x;
    if (b >= B) return;
    const int cells = S * S;
    for (int i = threadIdx.x; i < cells; i += blockDim.x) board[i] = stones[(size_t)b * cells + i];
    __syncthreads();
    const int p = to_move[b], o = p == 1 ? 2 : 1;
    for (int m = threadIdx.x; m < cells; m += blockDim.x) {
        float att = 0.0f, def = 0.0f;
        if (board[m] == 0) {
            const int r = m / S, c = m - r * S;
            const int after_m = stone_placed ? p : 0;
            int att_after = 0, att_before = 0, def_after = 0, def_before = 0;
            const int dr[4] = {0, 1, 1, 1}, dc[4] = {1, 0, 1, -1};
#pragma unroll
            for (int d = 0; d < 4; ++d) {
#pragma unroll
                for (int len = 5; len <= 6; ++len) {
                    const int need = len - 2;                     // stones asked for between the end cells
                    for (int k = 0; k < len; ++k) {               // m is the k-th cell of the window
                        const int r0 = r - k * dr[d], c0 = c - k * dc[d];
                        const int r1 = r0 + (len - 1) * dr[d], c1 = c0 + (len - 1) * dc[d];
                        if (r0 < 0 || r1 >= S || c0 < 0 || c0 >= S || c1 < 0 || c1 >= S) continue;
                        int mine = 0, theirs = 0;
                        bool ends_empty = true;
                        for (int j = 0; j < len; ++j) {
                            if (j == k) continue;
                            const int v = board[(r0 + j * dr[d]) * S + c0 + j * dc[d]];
                            if (j == 0 || j == len - 1) ends_empty = ends_empty && v == 0;
                            else { mine += v == p; theirs += v == o; }
                        }
                        if (!ends_empty) continue;
                        const bool m_is_end = k == 0 || k == len - 1;
                        // before: m empty.  after: m holds after_m.
                        const bool open_before = true, open_after = !m_is_end || after_m == 0;
                        const int mine_after = mine + ((!m_is_end && after_m == p) ? 1 : 0);
                        att_before += open_before && (mine == need || mine == need - 1);
                        att_after += open_after && (mine_after == need || mine_after == need - 1);
                        def_before += open_before && (theirs == need || theirs == need - 1);
                        def_after += open_after && (theirs == need || theirs == need - 1);
                    }
                }
            }
            att = (float)(att_after - att_before);
            def = (float)(def_before - def_after);
        }
        attack[(size_t)b * cells + m] = att;
        defense[(size_t)b * cells + m] = def;
    }
}

int launch_gomoku_attack_defense(const int8_t* stones, const uint8_t* to_move, int B, int S, int stone_placed,
                                 float* attack, float* defense, cudaStream_t st) {
    if (!stones || !to_move || !attack || !defense) return set_error(OB200_ERR_INVALID, "attack/defense planes: null pointer");
    if (B < 0 || S < 6 || S > 32) return set_error(OB200_ERR_INVALID, "attack/defense planes: need B >= 0 and board_size in [6, 32]");
    if (B == 0) return OB200_OK;
    gomoku_attack_defense_kernel<<<B, 256, S * S, st>>>(stones, to_move, B, S, stone_placed, attack, defense);
    OB200_LAUNCHED("gomoku_attack_defense_kernel");
    return OB200_OK;
}

}  // namespace ob200

using namespace ob200;

extern "C" {

int ob200_launch_encode_gomoku(const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                               int32_t B, int32_t board_size, int32_t planes, int32_t out_channels,
                               void* board_tensor_out, ob200_stream stream) {
    return launch_encode_gomoku(history, n_hist, to_move, B, board_size, planes, out_channels, board_tensor_out,
                                as_stream(stream));
}

int ob200_launch_encode_gomoku_dt(const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                                  int32_t B, int32_t board_size, int32_t planes, int32_t out_channels, int32_t dtype,
                                  void* board_tensor_out, ob200_stream stream) {
    return launch_encode_gomoku(history, n_hist, to_move, B, board_size, planes, out_channels, board_tensor_out,
                                as_stream(stream), dtype);
}

int ob200_launch_encode_go(const int8_t* stones, const int32_t* ko_point, const uint8_t* to_move,
                           const uint32_t* legal_bits, int32_t B, int32_t board_size, int32_t out_channels,
                           void* board_tensor_out, ob200_stream stream) {
    return launch_encode_go(stones, ko_point, to_move, legal_bits, B, board_size, out_channels, board_tensor_out,
                            as_stream(stream));
}

int ob200_launch_encode_gomoku3(const int8_t* stones, const uint8_t* to_move, int32_t B, int32_t board_size,
                                int32_t out_channels, void* board_tensor_out, ob200_stream stream) {
    return launch_encode_gomoku3(stones, to_move, B, board_size, out_channels, board_tensor_out, as_stream(stream));
}

int ob200_launch_gomoku_attack_defense(const int8_t* stones, const uint8_t* to_move, int32_t B, int32_t board_size,
                                       int32_t stone_placed, float* attack_out, float* defense_out, ob200_stream stream) {
    return launch_gomoku_attack_defense(stones, to_move, B, board_size, stone_placed, attack_out, defense_out, as_stream(stream));
}

int ob200_launch_encode_chess(const int8_t* pieces, const int32_t* meta, const uint32_t* legal_to, int32_t B,
                              int32_t out_channels, void* board_tensor_out, ob200_stream stream) {
    return launch_encode_chess(pieces, meta, legal_to, B, out_channels, board_tensor_out, as_stream(stream));
}

int ob200_launch_planes_to_board_tensor(const float* planes_nchw, int32_t B, int32_t C, int32_t board_size,
                                        int32_t out_channels, void* board_tensor_out, ob200_stream stream) {
    return launch_planes_to_board_tensor(planes_nchw, B, C, board_size, out_channels, board_tensor_out,
                                         as_stream(stream));
}

int ob200_launch_planes_to_board_tensor_dt(const float* planes_nchw, int32_t B, int32_t C, int32_t board_size,
                                           int32_t out_channels, int32_t dtype, void* board_tensor_out, ob200_stream stream) {
    return launch_planes_to_board_tensor(planes_nchw, B, C, board_size, out_channels, board_tensor_out,
                                         as_stream(stream), dtype);
}

}  // extern "C"
