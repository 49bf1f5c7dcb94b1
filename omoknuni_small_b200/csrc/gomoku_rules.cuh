// Which cells of a Gomoku position become children of a search node: the moves the rule set leaves the side to move
// (freestyle, Omok, Renju: GomokuRules, src/games/gomoku/gomoku_rules.cpp) and the limits MCTSNode::expand puts on
// the number of children (the cap and progressive widening, src/mcts/mcts_node.cpp:283-340).  Device code for one
// warp per node on bitmaps of at most 256 cells.
#pragma once
#include "internal.h"
#include <cuda_runtime.h>
#include <cstdint>

namespace ob200 {
namespace rules {

// Which of a new node's legal moves become children (MCTSNode::expand, src/mcts/mcts_node.cpp:283-340): at most
// max_children of them, the first in move order (the reference's cap of 1,000), and with progressive widening a
// random subset of `target` of those.  The reference draws the subset with a generator seeded from the operating
// system's entropy source; here a move's rank is the 64-bit mix of (seed, node id, move), so the same seed gives
// the same subset, and the `target` lowest ranks are kept.
struct Widening {
    uint32_t* empty;            // [max_nodes][mask_words] empty cells of every node's position; null: every empty cell is a child
    int max_children;           // <= 0: no cap
    int target;                 // <= 0: no widening
    unsigned long long seed;
    int rules;                  // OB200_RULES_*: which empty cells BLACK may not play
};

// Omok: BLACK may not make six or more in a row, nor open threes in two directions at once
// (GomokuRules::is_black_omok_forbidden, src/games/gomoku/gomoku_rules.cpp:118-198).  black / empty: bitmaps of the
// position (the cell itself is empty); S the board size.  An "open three in a direction" is the reference's: three
// consecutive black stones containing the cell, with the cell before and the cell after them on the board and empty.
__host__ __device__ inline bool omok_forbidden(const uint32_t* black, const uint32_t* empty, int S, int cell) {
    const int r = cell / S, c = cell - r * S;
    auto is_black = [&](int rr, int cc) {
        if (rr < 0 || rr >= S || cc < 0 || cc >= S) return false;
        const int a = rr * S + cc;
        return a == cell || ((black[a >> 5] >> (a & 31)) & 1u);
    };
    auto is_empty = [&](int rr, int cc) {
        if (rr < 0 || rr >= S || cc < 0 || cc >= S) return false;
        const int a = rr * S + cc;
        return a != cell && ((empty[a >> 5] >> (a & 31)) & 1u);
    };
    const int dr[4] = {1, 0, 1, 1}, dc[4] = {0, 1, 1, -1};
    int open_threes = 0;
    for (int d = 0; d < 4; ++d) {
        int run = 1;
        for (int k = 1; k < S && is_black(r + k * dr[d], c + k * dc[d]); ++k) ++run;
        for (int k = 1; k < S && is_black(r - k * dr[d], c - k * dc[d]); ++k) ++run;
        if (run >= 6) return true;
        bool open = false;
        for (int i = 0; i < 3 && !open; ++i) {
            const int r0 = r - i * dr[d], c0 = c - i * dc[d];
            if (is_black(r0, c0) && is_black(r0 + dr[d], c0 + dc[d]) && is_black(r0 + 2 * dr[d], c0 + 2 * dc[d]))
                open = is_empty(r0 - dr[d], c0 - dc[d]) && is_empty(r0 + 3 * dr[d], c0 + 3 * dc[d]);
        }
        open_threes += open;
    }
    return open_threes >= 2;
}
// Renju: BLACK's forbidden moves - overline, double four, double three
// (GomokuRules::is_black_renju_forbidden and what it calls, src/games/gomoku/gomoku_rules.cpp:200-879).
// A thread tests one cell on its own copy of BLACK's stones (hypothetical stones are set and cleared in it);
// empty0 is the position's empty-cell bitmap, so a cell is empty when it is in empty0 and not in the copy.
// The reference's double-three test recurses through the cell that would complete each three to a straight
// four; the recursion is unrolled at compile time to kRenjuDepth levels (the deepest seen on 600 dense
// boards is 3), beyond which a test answers "not a double three", as the CPU restatement does.
constexpr int kRenjuDepth = 4;
struct RjBoard {
    uint32_t bk[8];
    const uint32_t* empty0;
    int S;
    __device__ bool in(int r, int c) const { return r >= 0 && r < S && c >= 0 && c < S; }
    __device__ bool black(int r, int c) const { return in(r, c) && ((bk[(r * S + c) >> 5] >> ((r * S + c) & 31)) & 1u); }
    __device__ bool empty(int r, int c) const {
        if (!in(r, c)) return false;
        const int a = r * S + c;
        return ((empty0[a >> 5] >> (a & 31)) & 1u) && !((bk[a >> 5] >> (a & 31)) & 1u);
    }
    __device__ void set(int a) { bk[a >> 5] |= 1u << (a & 31); }
    __device__ void clear(int a) { bk[a >> 5] &= ~(1u << (a & 31)); }
};
static __device__ __constant__ int kRjDr[4] = {1, 0, 1, 1};
static __device__ __constant__ int kRjDc[4] = {0, 1, 1, -1};
// get_line_length_at_action (:38-69): BLACK's run through a cell that holds a black stone
static __device__ __noinline__ int rj_len(const RjBoard& b, int a, int d) {
    const int r = a / b.S, c = a - r * b.S;
    if (!b.black(r, c)) return 0;
    int n = 1;
    for (int i = 1; i < b.S && b.black(r + i * kRjDr[d], c + i * kRjDc[d]); ++i) ++n;
    for (int i = 1; i < b.S && b.black(r - i * kRjDr[d], c - i * kRjDc[d]); ++i) ++n;
    return n;
}
static __device__ __noinline__ int rj_len_if_filled(RjBoard& b, int cell, int d) {     // `cell` is empty
    b.set(cell);
    const int n = rj_len(b, cell, d);
    b.clear(cell);
    return n;
}
static __device__ __noinline__ bool rj_overline(const RjBoard& b, int a) {              // renju_is_overline :251-258
    for (int d = 0; d < 4; ++d) if (rj_len(b, a, d) > 5) return true;
    return false;
}
// count_renju_fours_at_action :260-436: per direction at most one four - a solid four that one more stone makes
// exactly five, else four stones and a gap in a window of five whose gap makes exactly five, else a stone one gap
// away (at distance 2-4) whose gap would join a run of three or more with room to extend.
static __device__ __noinline__ int rj_fours(RjBoard& b, int a) {
    const int S = b.S, r = a / S, c = a - r * S;
    int count = 0;
    for (int d = 0; d < 4; ++d) {
        const int dr = kRjDr[d], dc = kRjDc[d];
        bool found = false;
        for (int off = 0; off < 4 && !found; ++off) {
            const int r0 = r - off * dr, c0 = c - off * dc;
            bool solid = true;
            for (int i = 0; i < 4; ++i) solid = solid && b.black(r0 + i * dr, c0 + i * dc);
            if (!solid) continue;
            const int rb = r0 - dr, cb = c0 - dc, ra = r0 + 4 * dr, ca = c0 + 4 * dc;
            bool five = false;
            if (b.empty(rb, cb) && rj_len_if_filled(b, rb * S + cb, d) == 5) five = true;
            if (!five && b.empty(ra, ca) && rj_len_if_filled(b, ra * S + ca, d) == 5) five = true;
            found = five;
        }
        for (int off = 0; off < 5 && !found; ++off) {
            const int r0 = r - off * dr, c0 = c - off * dc;
            int stones = 0, empties = 0, gap = -1;
            bool valid = true;
            for (int i = 0; i < 5 && valid; ++i) {
                const int rk = r0 + i * dr, ck = c0 + i * dc;
                if (!b.in(rk, ck)) { valid = false; break; }
                if (b.black(rk, ck)) ++stones;
                else if (b.empty(rk, ck)) { ++empties; gap = rk * S + ck; }
                else valid = false;
            }
            if (valid && stones == 4 && empties == 1 && rj_len_if_filled(b, gap, d) == 5) found = true;
        }
        for (int dist = 2; dist <= 4 && !found; ++dist) {
            const int rf = r + dist * dr, cf = c + dist * dc;
            if (b.black(rf, cf)) {
                const int rg = r + (dist - 1) * dr, cg = c + (dist - 1) * dc;
                if (b.empty(rg, cg) && rj_len_if_filled(b, rg * S + cg, d) >= 3 &&
                    (b.empty(r - dr, c - dc) || b.empty(rf + dr, cf + dc))) { found = true; break; }
            }
            const int rk = r - dist * dr, ck = c - dist * dc;
            if (b.black(rk, ck)) {
                const int rg = r - (dist - 1) * dr, cg = c - (dist - 1) * dc;
                if (b.empty(rg, cg) && rj_len_if_filled(b, rg * S + cg, d) >= 3 &&
                    (b.empty(rk - dr, ck - dc) || b.empty(r + dr, c + dc))) { found = true; break; }
            }
        }
        count += found;
    }
    return count;
}
template <int DEPTH> __device__ bool rj_double_three(RjBoard& b, int a);
// A triple of consecutive black stones from (r0, c0) along d is a "three" (is_renju_three_definition :580-635) when
// a stone on one of its two empty end extensions gives a straight four (both ends empty, :637-676) that is itself
// allowed (no overline, no double four, no double three) and makes no five or more.
template <int DEPTH>
__device__ bool rj_three(RjBoard& b, int r0, int c0, int d) {
    const int dr = kRjDr[d], dc = kRjDc[d], S = b.S;
    for (int e = 0; e < 2; ++e) {
        const int rs = e == 0 ? r0 - dr : r0 + 3 * dr, cs = e == 0 ? c0 - dc : c0 + 3 * dc;
        if (!b.empty(rs, cs)) continue;
        const int spot = rs * S + cs;
        b.set(spot);
        const int rf = e == 0 ? rs : r0, cf = e == 0 ? cs : c0;       // first stone of the four
        bool ok = b.empty(rf - dr, cf - dc) && b.empty(rf + 4 * dr, cf + 4 * dc);
        if (ok && (rj_overline(b, spot) || rj_fours(b, spot) >= 2 || rj_double_three<DEPTH + 1>(b, spot))) ok = false;
        if (ok)
            for (int d2 = 0; d2 < 4; ++d2)
                if (rj_len(b, spot, d2) >= 5) { ok = false; break; }
        b.clear(spot);
        if (ok) return true;
    }
    return false;
}
// check_renju_double_three_recursive :460-578: two or more threes through the stone on `a`.  (The reference then
// counts how many of them can be taken to an allowed straight four and lets the move pass when at most one can;
// that count repeats the test that made each of them a three, so it equals the number of threes.)
template <int DEPTH>
__device__ bool rj_double_three(RjBoard& b, int a) {
    if constexpr (DEPTH > kRenjuDepth) {
        return false;
    } else {
        const int S = b.S, r = a / S, c = a - r * S;
        int threes = 0;
        for (int d = 0; d < 4; ++d)
            for (int off = 0; off < 3; ++off) {
                const int r0 = r - off * kRjDr[d], c0 = c - off * kRjDc[d];
                bool all = true;
                for (int k = 0; k < 3; ++k) all = all && b.black(r0 + k * kRjDr[d], c0 + k * kRjDc[d]);
                if (all && rj_three<DEPTH>(b, r0, c0, d)) ++threes;
            }
        return threes >= 2;
    }
}
// is_black_renju_forbidden :200-249 for an empty cell
static __device__ bool renju_forbidden(const uint32_t* black, const uint32_t* empty0, int S, int cell) {
    RjBoard b;
    for (int w = 0; w < 8; ++w) b.bk[w] = black[w];
    b.empty0 = empty0; b.S = S;
    b.set(cell);
    bool exact_five = false, over = false;
    for (int d = 0; d < 4; ++d) {
        const int n = rj_len(b, cell, d);
        exact_five = exact_five || n == 5;
        over = over || n > 5;
    }
    if (exact_five && !over) return false;
    if (over) return true;
    if (rj_fours(b, cell) >= 2) return true;
    return rj_double_three<0>(b, cell);
}
// One warp: legal <- empty minus the cells the rules deny the side to move (8 words, shared memory).
static __device__ void legal_moves_warp(const uint32_t* black, const uint32_t* empty, uint32_t* legal, int S, int mask_words,
                                 int rules, bool black_to_move, int lane) {
    if (lane < 8) legal[lane] = lane < mask_words ? empty[lane] : 0u;
    __syncwarp();
    if (rules != OB200_RULES_FREESTYLE && black_to_move)
        for (int cell = lane; cell < S * S; cell += 32)
            if (((empty[cell >> 5] >> (cell & 31)) & 1u) &&
                (rules == OB200_RULES_OMOK ? omok_forbidden(black, empty, S, cell) : renju_forbidden(black, empty, S, cell)))
                atomicAnd(&legal[cell >> 5], ~(1u << (cell & 31)));
    __syncwarp();
}
__host__ __device__ __forceinline__ unsigned long long widen_key(unsigned long long seed, int id, int s) {
    unsigned long long z = seed ^ ((unsigned long long)(id + 1) * 0x9E3779B97F4A7C15ull) ^ ((unsigned long long)(s + 1) * 0xC2B2AE3D27D4EB4Full);
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull; z ^= z >> 27; z *= 0x94D049BB133111EBull; z ^= z >> 31;
    return z;
}
// One warp, rows of at most 256 slots (8 mask words): exists <- the chosen subset of `empty`.
static __device__ void widen_mask_warp(const uint32_t* empty, uint32_t* exists, int mask_words, const Widening& wd, int id, int lane) {
    uint32_t w[8];
    int total = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        w[k] = k < mask_words ? empty[k] : 0u;
        if (wd.max_children > 0) {                      // the cap: the first max_children legal moves in move order
            int keep = wd.max_children - total;
            if (keep < 0) keep = 0;
            while (__popc(w[k]) > keep) w[k] &= ~(1u << (31 - __clz(w[k])));
        }
        total += __popc(w[k]);
    }
    if (wd.target > 0 && total > wd.target) {
        // lane l owns slots 8 l .. 8 l + 7; a slot stays when fewer than `target` legal slots rank below it
        uint32_t mine = (w[lane >> 2] >> ((lane & 3) * 8)) & 0xFFu;
        unsigned long long key[8];
        int rank[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { key[j] = widen_key(wd.seed, id, lane * 8 + j); rank[j] = 0; }
        for (int l = 0; l < 32; ++l) {
            const uint32_t theirs = __shfl_sync(0xffffffffu, mine, l);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const unsigned long long k = __shfl_sync(0xffffffffu, key[jj], l);
                if (!((theirs >> jj) & 1u)) continue;
                const int s2 = l * 8 + jj;
#pragma unroll
                for (int j = 0; j < 8; ++j) rank[j] += (k < key[j] || (k == key[j] && s2 < lane * 8 + j)) ? 1 : 0;
            }
        }
        uint32_t keep = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) keep |= (uint32_t)(((mine >> j) & 1u) && rank[j] < wd.target) << j;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) word |= __shfl_sync(0xffffffffu, keep, 4 * k + b) << (8 * b);
            w[k] = word;
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (k < mask_words && lane == 0) exists[k] = w[k];
}

}  // namespace rules
}  // namespace ob200
