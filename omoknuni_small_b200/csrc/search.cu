// Leaf-parallel MCTS for Gomoku with device-resident trees: the search loop
// around the selection, encoder and network kernels.  Host code only enqueues;
// nothing inside a move waits for the GPU.
//
// Takes the place of MCTSEngine::executeBatchedTreeSearch (reference
// src/mcts/mcts_engine_batch_tree_simple.cpp:14-301) for a group of independent
// games, of MCTSNode::expand (src/mcts/mcts_node.cpp:238-436: one child per
// legal move), addDirichletNoise (src/mcts/mcts_engine_eval.cpp:83-110) and
// getActionProbabilities (src/mcts/mcts_engine_tree.cpp:389-465).
//
// Tree layout: one ob200_tree_view over a pool of nodes shared by all trees;
// node t (< n_trees) is the root of tree t; a node's child slot is the board
// cell of the move (slot == action), its existence bit says the cell is a child:
// an empty cell that the rule set allows the side to move (gomoku_rules.cuh) and
// that survived the limits on children, when those are on.
#include "internal.h"
#include "gomoku_rules.cuh"
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <random>
#include <utility>
#include <vector>

struct ob200_search {
    ob200_search_config cfg{};
    ob200_net* net = nullptr;
    int S = 15, A = 225, pitch = 228, mask_words = 8;
    int max_nodes = 0, sims_per_round = 0;     // per tree
    ob200_tree_view tv{};                      // device arrays
    int32_t* n_used = nullptr;                 // device node counter
    int32_t* term_count = nullptr;             // device counter of terminal leaves
    uint32_t* root_stones = nullptr;           // [n_trees][2][8]: BLACK, WHITE bitmaps
    int16_t* root_hist = nullptr;              // [n_trees][16] k-th most recent move
    uint8_t *root_nh = nullptr, *root_tm = nullptr;
    int32_t* root_count = nullptr;             // stones on the board at the root
    int32_t *roots = nullptr, *paths = nullptr, *path_len = nullptr;
    int16_t* leaf_hist = nullptr; uint8_t *leaf_nh = nullptr, *leaf_tm = nullptr;
    float *leaf_value = nullptr, *term_value = nullptr;   // term_value: NaN = not terminal
    float *policy = nullptr, *value = nullptr, *noise = nullptr;
    // transposition table: Zobrist keys of positions -> node id (open addressing)
    unsigned long long *zobrist = nullptr, *node_hash = nullptr, *tt_key = nullptr;
    int32_t* tt_val = nullptr;
    int tt_size = 0;                           // power of two; 0 = table off
    std::vector<unsigned long long> zobrist_host;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    uint64_t moves_done = 0;
    // Gamma(alpha, 1) variates for the root noise of move number gamma_for (counted from 1): [n_trees][A]
    std::vector<float> gamma_host, noise_host;
    uint64_t gamma_for = 0;
    uint32_t* empty_bits = nullptr;            // [max_nodes][mask_words], only when a node's children can be fewer than its legal moves
    int max_children = 1000, widen_target = 0;
    // expansion plan of a round (per simulation)
    int32_t *plan_status = nullptr, *plan_aux = nullptr, *plan_new_id = nullptr;
    unsigned long long* plan_hash = nullptr;
    // test hooks: leaf values rounded to multiples of 1 / value_quantum (0 = off); a record of what every network
    // call of a move returned
    float value_quantum = 0.0f;
    float *rec_policy = nullptr, *rec_value = nullptr;   // [rec_rounds + 1][leaf_batch][A], [rec_rounds + 1][leaf_batch]
    int rec_rounds = 0;
    double wall_ms = 0.0;                                // host time of the last ob200_search_run
    // test / measurement hook: events around the five phases of every round of the next run
    bool phase_timing = false;
    std::vector<cudaEvent_t> phase_ev;                   // [rounds][6]
    double phase_ms[5] = {0, 0, 0, 0, 0};                // descent, leaf positions, network, expansion, backup
    std::vector<void*> owned;
};

namespace ob200 {
namespace {

using namespace rules;
constexpr int kMaxDepth = 64;

__device__ __forceinline__ bool bit(const uint32_t* m, int i) { return (m[i >> 5] >> (i & 31)) & 1u; }

// Roots: existence mask = empty cells (or the widened subset of them), statistics zero, no children yet.
__global__ void init_roots_kernel(ob200_tree_view t, const uint32_t* __restrict__ stones, int n_trees,
                                  int32_t* n_used, int32_t* term_count, Widening wd, const uint8_t* __restrict__ root_tm, int S) {
    __shared__ uint32_t legal_s[8];
    const int tree = blockIdx.x;
    const uint32_t* st = stones + (size_t)tree * 16;
    const size_t row = (size_t)tree * t.pitch;
    for (int s = threadIdx.x; s < t.pitch; s += blockDim.x) {
        t.N[row + s] = 0; t.W[row + s] = 0.0f; t.VL[row + s] = 0; t.P[row + s] = 0.0f;
        t.child_node[row + s] = -1;
    }
    uint32_t* own = (wd.empty ? wd.empty : t.legal_bits) + (size_t)tree * t.mask_words;
    for (int w = threadIdx.x; w < t.mask_words; w += blockDim.x) {
        uint32_t occupied = st[w] | st[8 + w];
        uint32_t valid = 0xFFFFFFFFu;
        if ((w + 1) * 32 > t.n_children) valid = (w * 32 >= t.n_children) ? 0u : ((1u << (t.n_children - w * 32)) - 1u);
        own[w] = ~occupied & valid;
    }
    if (wd.empty) {
        __syncthreads();
        if (threadIdx.x < 32) {
            legal_moves_warp(st, own, legal_s, S, t.mask_words, wd.rules, root_tm[tree] == 1, threadIdx.x);
            widen_mask_warp(legal_s, t.legal_bits + (size_t)tree * t.mask_words, t.mask_words, wd, tree, threadIdx.x);
        }
    }
    if (threadIdx.x == 0) {
        t.node_visits[tree] = 0;
        if (tree == 0) { *n_used = n_trees; *term_count = 0; }
    }
}

// P = (1 - eps) * P + eps * noise on the existing root children
// (MCTSEngine::addDirichletNoise, src/mcts/mcts_engine_eval.cpp:83-110).
__global__ void mix_noise_kernel(ob200_tree_view t, const float* __restrict__ noise, float eps) {
    const int tree = blockIdx.x;
    const size_t row = (size_t)tree * t.pitch;
    const uint32_t* m = t.legal_bits + (size_t)tree * t.mask_words;
    for (int s = threadIdx.x; s < t.n_children; s += blockDim.x)
        if (bit(m, s))   // (1 - eps) * prior + eps * noise, each operation rounded as the reference's C++ does (no fused multiply-add)
            t.P[row + s] = __fadd_rn(__fmul_rn(__fsub_rn(1.0f, eps), t.P[row + s]), __fmul_rn(eps, noise[(size_t)tree * t.pitch + s]));
}

// One thread per simulation: the leaf position from root + path.
//   history (k-th most recent move), side to move, and whether the game is over:
//   five or more in a row through the last move for the player who made it
//   (freestyle rules), or a full board.
__global__ void leaf_prepare_kernel(const int32_t* __restrict__ paths, const int32_t* __restrict__ path_len,
                                    int n_sims, int sims_per_tree, int max_depth, int S,
                                    const uint32_t* __restrict__ root_stones, const int16_t* __restrict__ root_hist,
                                    const uint8_t* __restrict__ root_nh, const uint8_t* __restrict__ root_tm,
                                    const int32_t* __restrict__ root_count, int16_t* __restrict__ leaf_hist,
                                    uint8_t* __restrict__ leaf_nh, uint8_t* __restrict__ leaf_tm,
                                    float* __restrict__ term_value, int32_t* term_count, int rules) {
    OB200_PDL_ENTER();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_sims) return;
    const int tree = i / sims_per_tree;
    int len = path_len[i];
    if (len > max_depth) len = max_depth;
    const int32_t* p = paths + (size_t)i * max_depth * 2;
    const int rtm = root_tm[tree], rnh = root_nh[tree];
    const int tm = (len & 1) ? 3 - rtm : rtm;
    int nh = 0;
    for (int k = 0; k < 16; ++k) {
        int mv = -1;
        if (k < len) mv = p[2 * (len - 1 - k) + 1];
        else if (k - len < rnh) mv = root_hist[(size_t)tree * 16 + (k - len)];
        leaf_hist[(size_t)i * 16 + k] = (int16_t)mv;
        if (mv >= 0) nh = k + 1;
    }
    leaf_nh[i] = (uint8_t)nh;
    leaf_tm[i] = (uint8_t)tm;
    float tv = nanf("");
    if (len > 0) {
        const int mover = 3 - tm;                              // who made the last move
        const uint32_t* st = root_stones + (size_t)tree * 16 + (mover - 1) * 8;
        const int last = p[2 * (len - 1) + 1];
        const int r0 = last / S, c0 = last % S;
        auto has = [&](int r, int c) {
            if (r < 0 || r >= S || c < 0 || c >= S) return false;
            const int cell = r * S + c;
            if (bit(st, cell)) return true;
            for (int d = len - 1; d >= 0; d -= 2)              // the mover's moves on the path
                if (p[2 * d + 1] == cell) return true;
            return false;
        };
        const int dr[4] = {0, 1, 1, 1}, dc[4] = {1, 0, 1, -1};
        // five or more wins; under Renju BLACK needs exactly five and no longer line through the stone
        // (GomokuState::refresh_winner_cache, src/games/gomoku/gomoku_state.cpp:812-860)
        bool five_up = false, exact = false, over = false;
        for (int dir = 0; dir < 4; ++dir) {
            int run = 1;
            for (int k = 1; k < 6 && has(r0 + k * dr[dir], c0 + k * dc[dir]); ++k) ++run;
            for (int k = 1; k < 6 && has(r0 - k * dr[dir], c0 - k * dc[dir]); ++k) ++run;
            five_up = five_up || run >= 5; exact = exact || run == 5; over = over || run > 5;
        }
        const bool win = (rules == OB200_RULES_RENJU && mover == 1) ? (exact && !over) : five_up;
        if (win) tv = -1.0f;                                    // the side to move has lost
        else if (root_count[tree] + len >= S * S) tv = 0.0f;    // full board
    }
    term_value[i] = tv;
    if (tv == tv) atomicAdd(term_count, 1);
}

// Expansion of a round's leaf edges, in two kernels.  The outcome is a function of the inputs alone
// (no dependence on which thread runs first), and it is the outcome of taking the round's simulations
// one after another in index order:
//   * an edge reached by several simulations of the round is expanded by the one with the lowest index;
//   * new nodes get consecutive ids in the order of the simulations that create them;
//   * with the transposition table, the position behind an edge (Zobrist key: stones + side to move, as
//     GomokuState::compute_hash_signature_internal, src/games/gomoku/gomoku_state.cpp:947-958) is looked
//     up first; if this game already has a node for it - from an earlier round, or from a simulation of
//     this round with a lower index - the edge is pointed at that node (the reference re-points the
//     parent's child reference, src/mcts/mcts_engine_batch_tree_simple.cpp:117-162) and nothing is created.
//
// expand_plan_kernel is ONE CTA that walks the simulations in phases separated by __syncthreads:
//   A  leaf value (game result for finished games, else the network's); lowest index claims the edge
//      (atomicMin of a code that orders by index);
//   B  winners look their position up in the table as it was before the round;
//   C  the others enter their key (or find the slot a sibling of this round took) and the lowest index
//      per key becomes its owner;
//   D  owners are counted in index order (block scan) -> node ids;
//   E  edges and table entries are pointed at the ids.
// expand_rows_kernel (a warp per simulation) then fills the rows of the nodes created.
constexpr int kPlanThreads = 1024;
enum : int32_t { kPlanNone = 0, kPlanCandidate = 1, kPlanNew = 2, kPlanShareOld = 3, kPlanShareNew = 4, kPlanOwner = 5 };

struct PlanScratch {
    int32_t* status;            // [L] one of kPlan*
    int32_t* aux;               // [L] table slot (candidate / owner), node id (share old), owner's index (share new)
    int32_t* new_id;            // [L] id of the node this simulation creates, or -1
    unsigned long long* hash;   // [L] key of the position behind the edge
};

__device__ __forceinline__ float quantized(float v, float q) { return q > 0.0f ? __fdiv_rn(rintf(__fmul_rn(v, q)), q) : v; }

__global__ void __launch_bounds__(kPlanThreads)
expand_plan_kernel(ob200_tree_view t, const int32_t* __restrict__ paths, const int32_t* __restrict__ path_len,
                   int n_sims, int max_depth, const float* __restrict__ value, const float* __restrict__ term_value,
                   float value_sign, float value_quantum, int max_nodes, int32_t* n_used, float* __restrict__ leaf_value,
                   int sims_per_tree, const uint8_t* __restrict__ root_tm, const unsigned long long* __restrict__ zobrist,
                   const unsigned long long* __restrict__ node_hash, unsigned long long* tt_key, int32_t* tt_val, int tt_size,
                   PlanScratch ps) {
    __shared__ int warp_sums[kPlanThreads / 32];
    __shared__ int carry_s;
    OB200_PDL_ENTER();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    auto code = [&](int i) { return -2 - (n_sims - 1 - i); };            // lower index -> smaller code; all below -1
    auto edge = [&](int i, int len) {
        const int32_t* p = paths + (size_t)i * max_depth * 2;
        return (size_t)p[2 * (len - 1)] * t.pitch + p[2 * (len - 1) + 1];
    };
    auto length = [&](int i) { const int len = path_len[i]; return len > max_depth ? max_depth : len; };
    // ---- A: values, claims ----
    for (int i = tid; i < n_sims; i += kPlanThreads) {
        const int len = length(i);
        const float tv = term_value[i];
        const bool terminal = tv == tv;
        leaf_value[i] = value_sign * (terminal ? tv : quantized(value[i], value_quantum));
        int st = kPlanNone;
        if (len > 0 && !terminal) {
            const size_t e = edge(i, len);
            if (*reinterpret_cast<volatile int32_t*>(t.child_node + e) < 0) { atomicMin(t.child_node + e, code(i)); st = kPlanCandidate; }
        }
        ps.status[i] = st; ps.aux[i] = -1; ps.new_id[i] = -1;
    }
    __syncthreads();
    // ---- B: winners; table lookup against the state before this round ----
    for (int i = tid; i < n_sims; i += kPlanThreads) {
        if (ps.status[i] != kPlanCandidate) continue;
        const int len = length(i);
        const size_t e = edge(i, len);
        if (*reinterpret_cast<volatile int32_t*>(t.child_node + e) != code(i)) { ps.status[i] = kPlanNone; continue; }
        if (tt_size <= 0) { ps.status[i] = kPlanNew; continue; }
        const int32_t* p = paths + (size_t)i * max_depth * 2;
        const int parent = p[2 * (len - 1)], slot = p[2 * (len - 1) + 1];
        const int rtm = root_tm[i / sims_per_tree];
        const int mover = ((len - 1) & 1) ? 3 - rtm : rtm;
        unsigned long long h = node_hash[parent] ^ zobrist[(mover - 1) * 225 + slot] ^ zobrist[450];
        if (h == 0) h = 1;
        ps.hash[i] = h;
        int st = kPlanNew;                                                // probe limit reached: a node outside the table
        unsigned idx = (unsigned)(h >> 17) & (unsigned)(tt_size - 1);
        for (int tries = 0; tries < 64; ++tries, idx = (idx + 1) & (unsigned)(tt_size - 1)) {
            const unsigned long long k = *reinterpret_cast<volatile unsigned long long*>(tt_key + idx);
            if (k == 0) { st = kPlanCandidate; break; }
            if (k == h) {
                const int other = *reinterpret_cast<volatile int32_t*>(tt_val + idx);
                if (other >= 0) { st = kPlanShareOld; ps.aux[i] = other; } else st = kPlanCandidate;
                break;
            }
        }
        ps.status[i] = st;
    }
    __syncthreads();
    // ---- C: candidates enter their key; the lowest index per key owns it ----
    for (int i = tid; i < n_sims; i += kPlanThreads) {
        if (ps.status[i] != kPlanCandidate) continue;
        const unsigned long long h = ps.hash[i];
        int found = -1;
        unsigned idx = (unsigned)(h >> 17) & (unsigned)(tt_size - 1);
        for (int tries = 0; tries < 64 && found < 0; ++tries, idx = (idx + 1) & (unsigned)(tt_size - 1)) {
            unsigned long long k = *reinterpret_cast<volatile unsigned long long*>(tt_key + idx);
            if (k == 0) { k = atomicCAS(tt_key + idx, 0ull, h); if (k == 0) k = h; }
            if (k == h) found = (int)idx;
        }
        if (found < 0) { ps.status[i] = kPlanNew; continue; }
        atomicMin(tt_val + found, code(i));
        ps.aux[i] = found;
    }
    __syncthreads();
    for (int i = tid; i < n_sims; i += kPlanThreads) {
        if (ps.status[i] != kPlanCandidate) continue;
        const int v = *reinterpret_cast<volatile int32_t*>(tt_val + ps.aux[i]);
        if (v == code(i)) ps.status[i] = kPlanOwner;
        else { ps.status[i] = kPlanShareNew; ps.aux[i] = n_sims - 1 - (-2 - v); }
    }
    // ---- D: ids in index order ----
    if (tid == 0) carry_s = *n_used;
    __syncthreads();
    for (int base = 0; base < n_sims; base += kPlanThreads) {
        const int i = base + tid;
        const int st = i < n_sims ? ps.status[i] : kPlanNone;
        const int flag = (st == kPlanOwner || st == kPlanNew) ? 1 : 0;
        int incl = flag;
        for (int off = 1; off < 32; off <<= 1) { const int o = __shfl_up_sync(0xffffffffu, incl, off); if (lane >= off) incl += o; }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
            for (int off = 1; off < 32; off <<= 1) { const int o = __shfl_up_sync(0xffffffffu, w, off); if (lane >= off) w += o; }
            warp_sums[lane] = w;                                          // inclusive sums over the warps
        }
        __syncthreads();
        const int before = carry_s + (warp ? warp_sums[warp - 1] : 0) + incl - flag;
        if (flag) ps.new_id[i] = before < max_nodes ? before : -1;       // pool exhausted: the edge stays a leaf
        __syncthreads();
        if (tid == 0) carry_s += warp_sums[kPlanThreads / 32 - 1];
        __syncthreads();
    }
    if (tid == 0) *n_used = carry_s < max_nodes ? carry_s : max_nodes;
    // ---- E: point edges and table entries at the nodes ----
    for (int i = tid; i < n_sims; i += kPlanThreads) {
        const int st = ps.status[i];
        if (st == kPlanNone) continue;
        const size_t e = edge(i, length(i));
        int child = -1;
        if (st == kPlanOwner) { child = ps.new_id[i]; tt_val[ps.aux[i]] = child; }
        else if (st == kPlanNew) child = ps.new_id[i];
        else if (st == kPlanShareOld) child = ps.aux[i];
        else if (st == kPlanShareNew) child = ps.new_id[ps.aux[i]];
        t.child_node[e] = child;
    }
}

// One warp per simulation that creates a node: existence mask = the parent's minus the move, priors =
// clamp(policy, 0, 1) on the existing slots with no renormalisation (MCTSNode::expand +
// setPriorProbabilities, src/mcts/mcts_node.cpp:238-436,546-553), statistics zero.
__global__ void __launch_bounds__(256)
expand_rows_kernel(ob200_tree_view t, const int32_t* __restrict__ paths, const int32_t* __restrict__ path_len,
                   int n_sims, int max_depth, const float* __restrict__ policy, int policy_size,
                   unsigned long long* node_hash, int tt_size, PlanScratch ps, Widening wd,
                   const uint32_t* __restrict__ root_stones, const uint8_t* __restrict__ root_tm, int sims_per_tree, int S) {
    __shared__ uint32_t black_s[8][8], legal_s[8][8];
    OB200_PDL_ENTER();
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    if (i >= n_sims) return;
    const int st = ps.status[i];
    const int id = ps.new_id[i];
    if ((st != kPlanOwner && st != kPlanNew) || id < 0) return;
    int len = path_len[i];
    if (len > max_depth) len = max_depth;
    const int32_t* p = paths + (size_t)i * max_depth * 2;
    const int parent = p[2 * (len - 1)], slot = p[2 * (len - 1) + 1];
    const size_t row = (size_t)id * t.pitch;
    // the position's empty cells: the parent's minus the move; they are the children unless the node is widened
    const uint32_t* pm = (wd.empty ? wd.empty : t.legal_bits) + (size_t)parent * t.mask_words;
    uint32_t* own = (wd.empty ? wd.empty : t.legal_bits) + (size_t)id * t.mask_words;
    uint32_t* cm = t.legal_bits + (size_t)id * t.mask_words;
    for (int w = lane; w < t.mask_words; w += 32) own[w] = pm[w] & ~((w == (slot >> 5)) ? (1u << (slot & 31)) : 0u);
    __syncwarp();
    if (wd.empty) {
        const int tree = i / sims_per_tree;
        const bool black_to_move = (root_tm[tree] == 1) == ((len & 1) == 0);     // the root's side moves at even depths
        if (wd.rules != OB200_RULES_FREESTYLE && black_to_move) {
            // BLACK's stones at the new node: the root's, and the path's moves made by BLACK
            if (lane < 8) black_s[wi][lane] = root_stones[(size_t)tree * 16 + lane];
            __syncwarp();
            for (int d = lane; d < len; d += 32) {
                const bool black_moved = (root_tm[tree] == 1) == ((d & 1) == 0);
                const int a = p[2 * d + 1];
                if (black_moved) atomicOr(&black_s[wi][a >> 5], 1u << (a & 31));
            }
            __syncwarp();
        }
        legal_moves_warp(black_s[wi], own, legal_s[wi], S, t.mask_words, wd.rules, black_to_move, lane);
        widen_mask_warp(legal_s[wi], cm, t.mask_words, wd, id, lane);
        __syncwarp();
    }
    const float* pol = policy + (size_t)i * policy_size;
    for (int s = lane; s < t.pitch; s += 32) {
        float pr = 0.0f;
        if (s < t.n_children && bit(cm, s)) pr = fminf(1.0f, fmaxf(0.0f, pol[s]));
        t.N[row + s] = 0; t.W[row + s] = 0.0f; t.VL[row + s] = 0; t.P[row + s] = pr;
        t.child_node[row + s] = -1;
    }
    if (lane == 0) {
        t.node_visits[id] = 0;
        if (tt_size > 0) node_hash[id] = ps.hash[i];
    }
}

}  // namespace
}  // namespace ob200

// Accessors of the network handle that the search needs (defined in net.cu).
namespace ob200 {
int net_forward_gomoku_for_search(ob200_net* n, const int16_t* hist, const uint8_t* nh, const uint8_t* tm, int B, float* policy,
                                  float* value, cudaStream_t st);
const ob200_net_config* net_config(ob200_net* n);
}

using namespace ob200;

namespace {

template <typename T>
int salloc(ob200_search* s, T** out, size_t count) {
    void* p = nullptr;
    OB200_CUDA_OK(cudaMalloc(&p, count * sizeof(T)));
    s->owned.push_back(p);
    *out = static_cast<T*>(p);
    return OB200_OK;
}

}  // namespace

namespace {
// One Gamma(alpha, 1) variate per (tree, cell) for move number `move`; a function of (seed, move) alone.
void draw_gammas(ob200_search* s, uint64_t move) {
    std::mt19937_64 rng(s->cfg.seed + 0x9E3779B97F4A7C15ull * move);
    std::gamma_distribution<float> gamma(s->cfg.dirichlet_alpha, 1.0f);
    s->gamma_host.resize((size_t)s->cfg.n_trees * s->A);
    for (float& g : s->gamma_host) g = gamma(rng);
    s->gamma_for = move;
}
}  // namespace

extern "C" {

int ob200_search_create(ob200_net* net, const ob200_search_config* cfg, ob200_search** out) {
    if (!net || !cfg || !out) return set_error(OB200_ERR_INVALID, "ob200_search_create: null argument");
    *out = nullptr;
    const ob200_net_config* nc = net_config(net);
    if (!nc) return set_error(OB200_ERR_STATE, "ob200_search_create: the network is not finalised");
    if (nc->board_size != 15 || nc->policy_size != 225 || (nc->input_channels != 17 && nc->input_channels != 19))
        return set_error(OB200_ERR_UNSUPPORTED, "ob200_search_create: the search is built for 15x15 Gomoku networks (17 or 19 planes, 225 moves)");
    if (cfg->n_trees < 1 || cfg->sims_per_move < 1 || cfg->leaf_batch < cfg->n_trees || cfg->leaf_batch % cfg->n_trees ||
        cfg->leaf_batch > nc->max_batch || cfg->max_depth < 1 || cfg->max_depth > kMaxDepth || cfg->virtual_loss < 0 ||
        (cfg->value_sign != 1 && cfg->value_sign != -1) || cfg->dirichlet_epsilon < 0 || cfg->dirichlet_epsilon > 1 ||
        cfg->max_children < 0 || (cfg->use_progressive_widening && !(cfg->progressive_widening_c >= 0.0f)) ||
        cfg->rules < 0 || cfg->rules > OB200_RULES_RENJU)
        return set_error(OB200_ERR_INVALID,
                         "ob200_search_create: need leaf_batch a multiple of n_trees and <= the network's max_batch (%d), max_depth in [1,%d], value_sign +-1",
                         nc->max_batch, kMaxDepth);
    OB200_CUDA_OK(cudaSetDevice(nc->device));
    if (int rc = require_device()) return rc;
    ob200_search* s = new ob200_search;
    s->cfg = *cfg; s->net = net;
    s->sims_per_round = cfg->leaf_batch / cfg->n_trees;
    const int rounds = (cfg->sims_per_move + s->sims_per_round - 1) / s->sims_per_round;
    s->max_nodes = cfg->n_trees * (1 + rounds * s->sims_per_round);     // every simulation adds at most one node
    const size_t edges = (size_t)s->max_nodes * s->pitch;
    const int T = cfg->n_trees, L = cfg->leaf_batch;
    int rc = OB200_OK;
    auto A_ = [&](int r) { if (!rc) rc = r; };
    A_(salloc(s, &s->tv.N, edges)); A_(salloc(s, &s->tv.W, edges)); A_(salloc(s, &s->tv.P, edges));
    A_(salloc(s, &s->tv.VL, edges)); A_(salloc(s, &s->tv.child_node, edges));
    A_(salloc(s, &s->tv.legal_bits, (size_t)s->max_nodes * s->mask_words));
    A_(salloc(s, &s->tv.node_visits, (size_t)s->max_nodes));
    s->max_children = cfg->max_children > 0 ? cfg->max_children : 1000;
    if (cfg->use_progressive_widening)       // the reference's count for a node without visits: (visits + 1)^k = 1
        s->widen_target = (int)std::max(8.0f, (float)((double)cfg->progressive_widening_c * std::pow(1.0, (double)cfg->progressive_widening_k)));
    if (s->widen_target > 0 || s->max_children < s->A || cfg->rules != OB200_RULES_FREESTYLE)
        A_(salloc(s, &s->empty_bits, (size_t)s->max_nodes * s->mask_words));
    A_(salloc(s, &s->n_used, 1)); A_(salloc(s, &s->term_count, 1));
    A_(salloc(s, &s->root_stones, (size_t)T * 16)); A_(salloc(s, &s->root_hist, (size_t)T * 16));
    A_(salloc(s, &s->root_nh, (size_t)T)); A_(salloc(s, &s->root_tm, (size_t)T)); A_(salloc(s, &s->root_count, (size_t)T));
    A_(salloc(s, &s->roots, (size_t)T));
    A_(salloc(s, &s->paths, (size_t)L * cfg->max_depth * 2)); A_(salloc(s, &s->path_len, (size_t)L));
    A_(salloc(s, &s->leaf_hist, (size_t)L * 16)); A_(salloc(s, &s->leaf_nh, (size_t)L)); A_(salloc(s, &s->leaf_tm, (size_t)L));
    A_(salloc(s, &s->leaf_value, (size_t)L)); A_(salloc(s, &s->term_value, (size_t)L));
    A_(salloc(s, &s->policy, (size_t)L * s->A)); A_(salloc(s, &s->value, (size_t)L));
    A_(salloc(s, &s->noise, (size_t)T * s->pitch));
    A_(salloc(s, &s->plan_status, (size_t)L)); A_(salloc(s, &s->plan_aux, (size_t)L)); A_(salloc(s, &s->plan_new_id, (size_t)L));
    A_(salloc(s, &s->plan_hash, (size_t)L));
    if (cfg->use_transposition_table) {
        s->tt_size = 1;
        while (s->tt_size < 2 * s->max_nodes) s->tt_size <<= 1;
        A_(salloc(s, &s->zobrist, 451)); A_(salloc(s, &s->node_hash, (size_t)s->max_nodes));
        A_(salloc(s, &s->tt_key, (size_t)s->tt_size)); A_(salloc(s, &s->tt_val, (size_t)s->tt_size));
    }
    if (rc) { ob200_search_destroy(s); return rc; }
    s->tv.n_nodes = s->max_nodes; s->tv.n_children = s->A; s->tv.pitch = s->pitch; s->tv.mask_words = s->mask_words;
    std::vector<int32_t> roots(T);
    for (int t = 0; t < T; ++t) roots[t] = t;
    OB200_CUDA_OK(cudaMemcpy(s->roots, roots.data(), T * sizeof(int32_t), cudaMemcpyHostToDevice));
    if (s->tt_size) {
        // Zobrist keys: splitmix64 stream from the seed; [0,225) BLACK stones, [225,450) WHITE, [450] side to move
        s->zobrist_host.resize(451);
        unsigned long long x = cfg->seed ^ 0xD1B54A32D192ED03ull;
        for (auto& z : s->zobrist_host) {
            x += 0x9E3779B97F4A7C15ull;
            unsigned long long v = x;
            v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull; v = (v ^ (v >> 27)) * 0x94D049BB133111EBull; z = v ^ (v >> 31);
        }
        OB200_CUDA_OK(cudaMemcpy(s->zobrist, s->zobrist_host.data(), 451 * 8, cudaMemcpyHostToDevice));
    }
    OB200_CUDA_OK(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
    OB200_CUDA_OK(cudaEventCreate(&s->ev0)); OB200_CUDA_OK(cudaEventCreate(&s->ev1));
    *out = s;
    return OB200_OK;
}

void ob200_search_destroy(ob200_search* s) {
    if (!s) return;
    if (s->stream) { cudaStreamSynchronize(s->stream); cudaStreamDestroy(s->stream); }
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    for (cudaEvent_t e : s->phase_ev) if (e) cudaEventDestroy(e);
    for (void* p : s->owned) cudaFree(p);
    delete s;
}

int ob200_search_debug_tree(ob200_search* s, ob200_tree_view* view_out, int32_t* nodes_used_out) {
    if (!s || !view_out) return set_error(OB200_ERR_INVALID, "ob200_search_debug_tree: null argument");
    *view_out = s->tv;
    if (nodes_used_out) OB200_CUDA_OK(cudaMemcpy(nodes_used_out, s->n_used, sizeof(int32_t), cudaMemcpyDeviceToHost));
    return OB200_OK;
}

int ob200_search_debug_hooks(ob200_search* s, float value_quantum, int32_t record_rounds) {
    if (!s || value_quantum < 0.0f || record_rounds < 0) return set_error(OB200_ERR_INVALID, "ob200_search_debug_hooks: bad argument");
    const ob200_net_config* nc = net_config(s->net);
    OB200_CUDA_OK(cudaSetDevice(nc->device));
    s->value_quantum = value_quantum;
    if (record_rounds > 0 && !s->rec_policy) {
        const size_t L = (size_t)s->cfg.leaf_batch;
        if (int rc = salloc(s, &s->rec_policy, (size_t)(record_rounds + 1) * L * s->A)) return rc;
        if (int rc = salloc(s, &s->rec_value, (size_t)(record_rounds + 1) * L)) return rc;
        s->rec_rounds = record_rounds;
    }
    return OB200_OK;
}

int ob200_search_debug_phases(ob200_search* s, int32_t enable, double* phase_ms_out) {
    if (!s) return set_error(OB200_ERR_INVALID, "ob200_search_debug_phases: null argument");
    if (phase_ms_out)
        for (int k = 0; k < 5; ++k) phase_ms_out[k] = s->phase_ms[k];
    s->phase_timing = enable != 0;
    return OB200_OK;
}

int ob200_search_debug_record(ob200_search* s, const float** policy_out, const float** value_out, const float** noise_out) {
    if (!s) return set_error(OB200_ERR_INVALID, "ob200_search_debug_record: null argument");
    if (policy_out) *policy_out = s->rec_policy;
    if (value_out) *value_out = s->rec_value;
    if (noise_out) *noise_out = s->noise;
    return OB200_OK;
}

int ob200_copy_to_host(void* dst_host, const void* src_device, int64_t bytes) {
    if (!dst_host || !src_device || bytes < 0) return set_error(OB200_ERR_INVALID, "ob200_copy_to_host: bad argument");
    OB200_CUDA_OK(cudaMemcpy(dst_host, src_device, (size_t)bytes, cudaMemcpyDeviceToHost));
    return OB200_OK;
}

int ob200_search_run(ob200_search* s, const int16_t* moves, const int32_t* n_moves, int32_t moves_stride,
                     float temperature, float* pi_out, int32_t* visits_out, ob200_search_stats* stats) {
    if (!s || !moves || !n_moves || !pi_out || moves_stride < 0)
        return set_error(OB200_ERR_INVALID, "ob200_search_run: null argument");
    const ob200_search_config& c = s->cfg;
    const int T = c.n_trees, L = c.leaf_batch, S = s->S, A = s->A;
    const ob200_net_config* nc = net_config(s->net);
    const auto wall0 = std::chrono::steady_clock::now();
    OB200_CUDA_OK(cudaSetDevice(nc->device));
    // ---- roots from the move lists (host) ----
    std::vector<uint32_t> stones((size_t)T * 16, 0u);
    std::vector<int16_t> hist((size_t)T * 16, (int16_t)-1);
    std::vector<uint8_t> nh(T), tm(T);
    std::vector<int32_t> count(T);
    for (int t = 0; t < T; ++t) {
        const int n = n_moves[t];
        if (n < 0 || n > moves_stride || n >= A)
            return set_error(OB200_ERR_INVALID, "ob200_search_run: tree %d has %d moves (stride %d, board %d cells)", t, n, moves_stride, A);
        for (int i = 0; i < n; ++i) {
            const int mv = moves[(size_t)t * moves_stride + i];
            if (mv < 0 || mv >= A) return set_error(OB200_ERR_INVALID, "ob200_search_run: tree %d move %d out of range", t, mv);
            uint32_t& w = stones[(size_t)t * 16 + (i & 1) * 8 + (mv >> 5)];
            if (((stones[(size_t)t * 16 + (mv >> 5)] | stones[(size_t)t * 16 + 8 + (mv >> 5)]) >> (mv & 31)) & 1u)
                return set_error(OB200_ERR_INVALID, "ob200_search_run: tree %d plays cell %d twice", t, mv);
            w |= 1u << (mv & 31);
        }
        const int k = n < 16 ? n : 16;
        for (int i = 0; i < k; ++i) hist[(size_t)t * 16 + i] = moves[(size_t)t * moves_stride + n - 1 - i];
        nh[t] = (uint8_t)k; tm[t] = (uint8_t)((n & 1) ? 2 : 1); count[t] = n;
    }
    cudaStream_t st = s->stream;
    OB200_CUDA_OK(cudaMemcpyAsync(s->root_stones, stones.data(), stones.size() * 4, cudaMemcpyHostToDevice, st));
    OB200_CUDA_OK(cudaMemcpyAsync(s->root_hist, hist.data(), hist.size() * 2, cudaMemcpyHostToDevice, st));
    OB200_CUDA_OK(cudaMemcpyAsync(s->root_nh, nh.data(), T, cudaMemcpyHostToDevice, st));
    OB200_CUDA_OK(cudaMemcpyAsync(s->root_tm, tm.data(), T, cudaMemcpyHostToDevice, st));
    OB200_CUDA_OK(cudaMemcpyAsync(s->root_count, count.data(), T * 4, cudaMemcpyHostToDevice, st));
    // the widening ranks change from move to move
    unsigned long long wseed = c.seed + 0x632BE59BD9B4E019ull * (s->moves_done + 1);
    wseed ^= wseed >> 31; wseed *= 0xD6E8FEB86659FD93ull; wseed ^= wseed >> 32;
    if (s->tt_size) {
        std::vector<unsigned long long> rh(T, 0ull);
        for (int t = 0; t < T; ++t) {
            for (int i = 0; i < n_moves[t]; ++i) rh[t] ^= s->zobrist_host[(i & 1) * 225 + moves[(size_t)t * moves_stride + i]];
            if (n_moves[t] & 1) rh[t] ^= s->zobrist_host[450];
            rh[t] ^= 0x9E3779B97F4A7C15ull * (unsigned long long)(t + 1);   // per-game salt: games do not share nodes
        }
        OB200_CUDA_OK(cudaMemcpyAsync(s->node_hash, rh.data(), (size_t)T * 8, cudaMemcpyHostToDevice, st));
        OB200_CUDA_OK(cudaMemsetAsync(s->tt_key, 0, (size_t)s->tt_size * 8, st));
        OB200_CUDA_OK(cudaMemsetAsync(s->tt_val, 0xFF, (size_t)s->tt_size * 4, st));
    }
    OB200_CUDA_OK(cudaEventRecord(s->ev0, st));
    // ---- roots: create, evaluate, priors (+ noise) ----
    const Widening wd{s->empty_bits, s->empty_bits ? s->max_children : 0, s->empty_bits ? s->widen_target : 0, wseed, c.rules};
    init_roots_kernel<<<T, 128, 0, st>>>(s->tv, s->root_stones, T, s->n_used, s->term_count, wd, s->root_tm, s->S);
    OB200_LAUNCHED("init_roots_kernel");
    // root noise: Gamma(alpha, 1) per existing child, normalised (addDirichletNoise, :83-110).  The children are what
    // the kernel above made of the rules and the limits on children, so their masks are read back (2 KB, the GPU has
    // nothing else to do yet); the Gamma variates of this move were drawn while the previous move ran on the GPU.
    if (c.dirichlet_epsilon > 0.0f) {
        std::vector<uint32_t> root_mask((size_t)T * s->mask_words);
        OB200_CUDA_OK(cudaMemcpyAsync(root_mask.data(), s->tv.legal_bits, root_mask.size() * 4, cudaMemcpyDeviceToHost, st));
        if (s->gamma_for != s->moves_done + 1) draw_gammas(s, s->moves_done + 1);
        OB200_CUDA_OK(cudaStreamSynchronize(st));
        std::vector<float>& noise = s->noise_host;
        noise.assign((size_t)T * s->pitch, 0.0f);
        for (int t = 0; t < T; ++t) {
            // one variate per child in child order, summed and divided in fp32; a zero sum gives uniform noise (:83-100)
            float* row = noise.data() + (size_t)t * s->pitch;
            const float* g = s->gamma_host.data() + (size_t)t * A;
            const uint32_t* child = root_mask.data() + (size_t)t * s->mask_words;
            float sum = 0.0f;
            int children = 0;
            auto is_child = [&](int a) { return (child[a >> 5] >> (a & 31)) & 1u; };
            for (int a = 0; a < A; ++a)
                if (is_child(a)) { row[a] = g[a]; sum += row[a]; ++children; }
            for (int a = 0; a < A; ++a)
                if (is_child(a)) row[a] = sum > 0.0f ? row[a] / sum : 1.0f / (float)children;
        }
        OB200_CUDA_OK(cudaMemcpyAsync(s->noise, noise.data(), noise.size() * 4, cudaMemcpyHostToDevice, st));
    }
    if (int rc = net_forward_gomoku_for_search(s->net, s->root_hist, s->root_nh, s->root_tm, T, s->policy, s->value, st)) return rc;
    if (int rc = ob200_launch_set_priors(&s->tv, s->roots, T, s->policy, A, nullptr, st)) return rc;
    if (s->rec_policy) {
        OB200_CUDA_OK(cudaMemcpyAsync(s->rec_policy, s->policy, (size_t)T * A * 4, cudaMemcpyDeviceToDevice, st));
        OB200_CUDA_OK(cudaMemcpyAsync(s->rec_value, s->value, (size_t)T * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (c.dirichlet_epsilon > 0.0f) {
        mix_noise_kernel<<<T, 128, 0, st>>>(s->tv, s->noise, c.dirichlet_epsilon);
        OB200_LAUNCHED("mix_noise_kernel");
    }
    // ---- rounds ----
    const int rounds = (c.sims_per_move + s->sims_per_round - 1) / s->sims_per_round;
    if (s->phase_timing && (int)s->phase_ev.size() < rounds * 6) {
        const size_t have = s->phase_ev.size();
        s->phase_ev.resize((size_t)rounds * 6, nullptr);
        for (size_t i = have; i < s->phase_ev.size(); ++i) OB200_CUDA_OK(cudaEventCreate(&s->phase_ev[i]));
    }
    auto mark = [&](int r, int k) { return s->phase_timing ? cudaEventRecord(s->phase_ev[(size_t)r * 6 + k], st) : cudaSuccess; };
    for (int r = 0; r < rounds; ++r) {
        OB200_CUDA_OK(mark(r, 0));
        if (int rc = ob200_launch_traverse(&s->tv, s->roots, T, s->sims_per_round, c.c_puct, c.virtual_loss, c.max_depth,
                                           s->paths, s->path_len, st)) return rc;
        OB200_CUDA_OK(mark(r, 1));
        OB200_CUDA_OK(launch_dependent(leaf_prepare_kernel, dim3((L + 127) / 128), dim3(128), 0, st, s->paths, s->path_len, L,
                                       s->sims_per_round, c.max_depth, S, s->root_stones, s->root_hist, s->root_nh, s->root_tm,
                                       s->root_count, s->leaf_hist, s->leaf_nh, s->leaf_tm, s->term_value, s->term_count, c.rules));
        counters().launches.fetch_add(1, std::memory_order_relaxed);
        OB200_CUDA_OK(mark(r, 2));
        if (int rc = net_forward_gomoku_for_search(s->net, s->leaf_hist, s->leaf_nh, s->leaf_tm, L, s->policy, s->value, st)) return rc;
        OB200_CUDA_OK(mark(r, 3));
        if (s->rec_policy && r < s->rec_rounds) {
            OB200_CUDA_OK(cudaMemcpyAsync(s->rec_policy + (size_t)(r + 1) * L * A, s->policy, (size_t)L * A * 4, cudaMemcpyDeviceToDevice, st));
            OB200_CUDA_OK(cudaMemcpyAsync(s->rec_value + (size_t)(r + 1) * L, s->value, (size_t)L * 4, cudaMemcpyDeviceToDevice, st));
        }
        const PlanScratch ps{s->plan_status, s->plan_aux, s->plan_new_id, s->plan_hash};
        OB200_CUDA_OK(launch_dependent(expand_plan_kernel, dim3(1), dim3(kPlanThreads), 0, st, s->tv, s->paths, s->path_len, L, c.max_depth,
                                       s->value, s->term_value, (float)c.value_sign, s->value_quantum, s->max_nodes, s->n_used,
                                       s->leaf_value, s->sims_per_round, s->root_tm, s->zobrist, s->node_hash, s->tt_key, s->tt_val,
                                       s->tt_size, ps));
        OB200_CUDA_OK(launch_dependent(expand_rows_kernel, dim3((L * 32 + 255) / 256), dim3(256), 0, st, s->tv, s->paths, s->path_len, L,
                                       c.max_depth, s->policy, A, s->node_hash, s->tt_size, ps, wd, s->root_stones, s->root_tm,
                                       s->sims_per_round, s->S));
        counters().launches.fetch_add(2, std::memory_order_relaxed);
        OB200_CUDA_OK(mark(r, 4));
        if (int rc = ob200_launch_backup(&s->tv, s->paths, s->path_len, s->leaf_value, L, c.max_depth, c.virtual_loss, st)) return rc;
        OB200_CUDA_OK(mark(r, 5));
    }
    OB200_CUDA_OK(cudaEventRecord(s->ev1, st));
    // the next move's Gamma variates, while this one runs on the GPU (the copies into pageable memory below return only
    // when the stream has drained)
    if (c.dirichlet_epsilon > 0.0f) draw_gammas(s, s->moves_done + 2);
    // ---- results: root visit counts -> pi (getActionProbabilities, src/mcts/mcts_engine_tree.cpp:389-465) ----
    std::vector<int32_t> rootN((size_t)T * s->pitch);
    int32_t used = 0, terms = 0;
    OB200_CUDA_OK(cudaMemcpyAsync(rootN.data(), s->tv.N, rootN.size() * 4, cudaMemcpyDeviceToHost, st));
    OB200_CUDA_OK(cudaMemcpyAsync(&used, s->n_used, 4, cudaMemcpyDeviceToHost, st));
    OB200_CUDA_OK(cudaMemcpyAsync(&terms, s->term_count, 4, cudaMemcpyDeviceToHost, st));
    int err = 0;
    int* errw = device_error_word();
    if (errw) OB200_CUDA_OK(cudaMemcpyAsync(&err, errw, 4, cudaMemcpyDeviceToHost, st));
    OB200_CUDA_OK(cudaStreamSynchronize(st));
    if (err) {
        cudaMemsetAsync(errw, 0, 4, st); cudaStreamSynchronize(st);
        return set_error(OB200_ERR_TIMEOUT, "a kernel gave up on a bounded wait (code %d) during the search", err);
    }
    for (int t = 0; t < T; ++t) {
        const int32_t* n = rootN.data() + (size_t)t * s->pitch;
        float* pi = pi_out + (size_t)t * A;
        int nmax = 0, amax = -1;
        for (int a = 0; a < A; ++a) { if (visits_out) visits_out[(size_t)t * A + a] = n[a]; if (n[a] > nmax) { nmax = n[a]; amax = a; } }
        std::memset(pi, 0, sizeof(float) * A);
        if (nmax <= 0) continue;
        if (temperature < 0.01f) { pi[amax] = 1.0f; continue; }
        double sum = 0.0;
        for (int a = 0; a < A; ++a) if (n[a] > 0) { pi[a] = std::pow((float)n[a] / (float)nmax, 1.0f / temperature); sum += pi[a]; }
        for (int a = 0; a < A; ++a) pi[a] = (float)(pi[a] / sum);
    }
    s->moves_done++;
    if (s->phase_timing) {
        for (double& v : s->phase_ms) v = 0.0;
        for (int r = 0; r < rounds; ++r)
            for (int k = 0; k < 5; ++k) {
                float ms = 0.0f;
                cudaEventElapsedTime(&ms, s->phase_ev[(size_t)r * 6 + k], s->phase_ev[(size_t)r * 6 + k + 1]);
                s->phase_ms[k] += ms;
            }
    }
    if (stats) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, s->ev0, s->ev1);
        stats->simulations = (int64_t)rounds * L;
        stats->evaluations = (int64_t)rounds * L + T;
        stats->nodes = used; stats->terminal_leaves = terms; stats->device_ms = ms;
        stats->wall_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - wall0).count();
    }
    return OB200_OK;
}

}  // extern "C"
