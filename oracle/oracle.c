/* TEST INFRASTRUCTURE — not part of the product.
 *
 * Plain-C CPU restatement of the reference project's algorithms for the
 * leaf-parallel evaluation path (cosmosapjw-quantum/omoknuni_small; file:line
 * below are paths inside that project).  Only tests/, the smoke check and the
 * benchmark's CPU-baseline leg load this library; the product never does.
 *
 * Pinned against the reference's own classes compiled from its sources
 * (oracle/_ref, see oracle/Makefile) by tests/golden/make_golden.py and
 * tests/test_oracle.py, and against the known-answer cases of
 * the reference's unit tests (tests/mcts/mcts_node_test.cpp:237-298,
 * tests/mcts/virtual_loss_test.cpp:160-224,282-308).
 *
 * Compile with -ffp-contract=off: the reference is built without FMA
 * contraction (x86-64 baseline, -O3), and selection compares fp32 scores.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <limits.h>
#include <omp.h>

/* MCTSNode::selectChild, src/mcts/mcts_node.cpp:90-236 (RAVE off, no child
 * pending evaluation), over flat arrays.  Child slots whose legal bit is 0 do
 * not exist.  Returns the slot, or -1 for a node without children.  The
 * reference runs its scan twice with identical results; once is enough. */
static int select_row(const int32_t* N, const float* W, const float* P, const int32_t* VL,
                      const uint32_t* legal, int n_children, int n_parent, float c_puct) {
    float best = -INFINITY;
    int best_i = -1;
    /* :94-95  exploration_param = c * sqrt((float)visit_count) */
    const float explore = c_puct * sqrtf((float)n_parent);
    int have = 0, min_n = INT_MAX, min_i = -1;
    for (int i = 0; i < n_children; ++i) {
        if (!((legal[i >> 5] >> (i & 31)) & 1u)) continue;
        have = 1;
        const int ev = N[i] + VL[i];                          /* :147 */
        const float val = W[i] - (float)VL[i];                /* :148 */
        const float q = ev > 0 ? val / (float)ev : 0.0f;      /* :151-152 */
        const float u = P[i] * explore / (1.0f + (float)ev);  /* :154-155 */
        const float s = q + u;                                /* :157 */
        if (s > best) { best = s; best_i = i; }               /* :160 strict */
        if (N[i] < min_n) { min_n = N[i]; min_i = i; }        /* :173-181 fallback */
    }
    if (best_i < 0 && have) return min_i;
    return best_i;
}

void oracle_puct_select(const int32_t* N, const float* W, const float* P, int32_t* VL,
                        const uint32_t* legal, const int32_t* node_visits, int n_children,
                        int pitch, int mask_words, const int32_t* node_ids, int n, float c_puct,
                        int vl_value, int apply_vl, int32_t* sel_out, int threads) {
    if (threads > 0) omp_set_num_threads(threads);
#pragma omp parallel for schedule(static) if (!apply_vl || !node_ids)
    for (int i = 0; i < n; ++i) {
        const int node = node_ids ? node_ids[i] : i;
        const size_t r = (size_t)node * pitch;
        const int s = select_row(N + r, W + r, P + r, VL + r, legal + (size_t)node * mask_words,
                                 n_children, node_visits[node], c_puct);
        sel_out[i] = s;
        /* applyVirtualLoss on the selected child, mcts_engine_batch_tree_simple.cpp:111;
         * addVirtualLoss ignores amount <= 0, mcts_node_virtual_loss.cpp:15-20 */
        if (s >= 0 && apply_vl && vl_value > 0) VL[r + s] += vl_value;
    }
}

/* MCTSNode::addVirtualLoss(int), src/mcts/mcts_node_virtual_loss.cpp:15-20 */
void oracle_vl_apply(int32_t* VL, int pitch, const int32_t* node_ids, const int32_t* sel, int n,
                     int vl_value) {
    if (vl_value <= 0) return;
    for (int i = 0; i < n; ++i) {
        const int node = node_ids ? node_ids[i] : i;
        if (sel[i] >= 0) VL[(size_t)node * pitch + sel[i]] += vl_value;
    }
}

/* MCTSNode::removeVirtualLoss(int), src/mcts/mcts_node_virtual_loss.cpp:32-42 */
static void remove_vl(int32_t* vl, int amount) {
    if (amount <= 0) return;
    const int cur = *vl;
    *vl = cur - amount;
    if (cur < amount) *vl = 0;
}
/* MCTSNode::removeVirtualLoss(), :22-30 */
static void remove_vl_one(int32_t* vl) {
    const int cur = *vl;
    *vl = cur - 1;
    if (cur <= 0) *vl = 0;
}

void oracle_vl_revert(int32_t* VL, int pitch, const int32_t* node_ids, const int32_t* sel, int n,
                      int vl_value) {
    for (int i = 0; i < n; ++i) {
        const int node = node_ids ? node_ids[i] : i;
        if (sel[i] >= 0) remove_vl(&VL[(size_t)node * pitch + sel[i]], vl_value);
    }
}

/* A sequence of operations on one counter (op > 0 add, op < 0 remove(-op),
 * op == 0 the argument-less remove); out[i] = counter after operation i. */
void oracle_vl_ops(int initial, const int32_t* ops, int n_ops, int32_t* out) {
    int32_t vl = 0;
    if (initial > 0) vl += initial;
    for (int i = 0; i < n_ops; ++i) {
        if (ops[i] > 0) vl += ops[i];
        else if (ops[i] < 0) remove_vl(&vl, -ops[i]);
        else remove_vl_one(&vl);
        out[i] = vl;
    }
}

/* Backup: MCTSNode::update (src/mcts/mcts_node_virtual_loss.cpp:54-71) followed
 * by revertVirtualLoss and the sign flip, per path node from leaf to root
 * (src/mcts/mcts_engine_batch_tree_simple.cpp:276-281), on edge statistics.
 * paths[i][d] = (node, slot), root first.  Paths are applied in index order. */
void oracle_backup(int32_t* N, float* W, int32_t* VL, int32_t* node_visits,
                   const int32_t* child_node, int pitch, const int32_t* paths,
                   const int32_t* path_len, const float* leaf_values, int n, int max_depth,
                   int vl_value) {
    for (int i = 0; i < n; ++i) {
        int len = path_len[i] > max_depth ? max_depth : path_len[i];
        float v = leaf_values[i];
        const int32_t* p = paths + (size_t)i * max_depth * 2;
        for (int d = len - 1; d >= 0; --d) {
            const size_t e = (size_t)p[2 * d] * pitch + p[2 * d + 1];
            N[e] += 1;                         /* visit_count_.fetch_add(1) */
            W[e] = W[e] + v;                   /* value_sum_ CAS loop       */
            if (VL[e] > 0) remove_vl_one(&VL[e]);
            remove_vl(&VL[e], vl_value);       /* revertVirtualLoss(vl)     */
            if (d == len - 1 && child_node && child_node[e] >= 0) node_visits[child_node[e]] += 1;
            node_visits[p[2 * d]] += 1;
            v = -v;
        }
    }
}

/* MCTSNode::setPriorProbabilities, src/mcts/mcts_node.cpp:512-593: the prior of
 * a child is the policy entry of its action clamped to [0, 1] (:546-553), 0.01
 * for an action outside the policy (:559), no renormalisation. */
void oracle_set_priors(float* P, const uint32_t* legal, int n_children, int pitch, int mask_words,
                       const int32_t* node_ids, int n, const float* policy, int policy_size,
                       const int32_t* slot_action) {
    for (int i = 0; i < n; ++i) {
        const int node = node_ids ? node_ids[i] : i;
        const size_t r = (size_t)node * pitch;
        const uint32_t* m = legal + (size_t)node * mask_words;
        for (int s = 0; s < pitch; ++s) {
            float p = 0.0f;
            if (s < n_children && ((m[s >> 5] >> (s & 31)) & 1u)) {
                const int a = slot_action ? slot_action[r + s] : s;
                if (a >= 0 && a < policy_size) {
                    p = policy[(size_t)i * policy_size + a];
                    p = fminf(1.0f, fmaxf(0.0f, p));
                } else {
                    p = 0.01f;
                }
            }
            P[r + s] = p;
        }
    }
}

/* Phase 1 of MCTSEngine::executeBatchedTreeSearch
 * (src/mcts/mcts_engine_batch_tree_simple.cpp:85-166) with a defined order:
 * the simulations of one tree run one after another, each selecting with the
 * virtual loss left by the earlier ones and adding vl_value to the edge it
 * takes; the descent ends at an unexpanded edge (child_node < 0), at a node
 * without children, or after max_depth steps. */
void oracle_traverse(const int32_t* N, const float* W, const float* P, int32_t* VL,
                     const uint32_t* legal, const int32_t* node_visits, const int32_t* child_node,
                     int n_nodes, int n_children, int pitch, int mask_words, const int32_t* roots,
                     int n_trees, int sims_per_tree, float c_puct, int vl_value, int max_depth,
                     int32_t* paths_out, int32_t* path_len_out) {
    for (int t = 0; t < n_trees; ++t) {
        for (int k = 0; k < sims_per_tree; ++k) {
            const size_t sim = (size_t)t * sims_per_tree + k;
            int32_t* path = paths_out + sim * max_depth * 2;
            int node = roots[t], depth = 0;
            while (depth < max_depth && node >= 0 && node < n_nodes) {
                const size_t r = (size_t)node * pitch;
                const int s = select_row(N + r, W + r, P + r, VL + r,
                                         legal + (size_t)node * mask_words, n_children,
                                         node_visits[node], c_puct);
                if (s < 0) break;
                if (vl_value > 0) VL[r + s] += vl_value;
                path[2 * depth] = node;
                path[2 * depth + 1] = s;
                ++depth;
                node = child_node ? child_node[r + s] : -1;
            }
            path_len_out[sim] = depth;
        }
    }
}

/* GomokuState::getEnhancedTensorRepresentation,
 * src/games/gomoku/gomoku_state.cpp:210-372, from the move history.
 * history[k] = k-th most recent move (k = 0 newest).  Move k is the
 * opponent's when k is even (:228-230) and the side to move's when k is odd
 * (:231-233); the side to move's i-th most recent move sets plane 2i
 * (:238-245), the opponent's sets plane 2i+1 (:247-254), i < 8.  Plane 16 is
 * 1.0 everywhere iff BLACK (1) is to move (:257-262).  Planes 17/18 come from
 * GomokuAttackDefenseModule::compute_planes
 * (src/utils/attack_defense_module.cpp:61-111): for every legal (empty) cell
 * the "before" board of compute_attack_bonus/compute_defense_bonus (:113-154,
 * :156-203) only clears an already empty cell, so after == before and both
 * planes are zero.  out: [planes][S][S] fp32, planes = 17 or 19. */
void oracle_gomoku_encode(const int16_t* history, int n_hist, int to_move, int S, int planes,
                          float* out) {
    memset(out, 0, sizeof(float) * (size_t)planes * S * S);
    for (int k = 0; k < n_hist && k < 16; ++k) {
        const int a = history[k];
        const int r = a / S, c = a % S;
        if (a < 0 || r >= S) continue;
        const int i = k / 2;
        const int plane = (k & 1) ? 2 * i : 2 * i + 1;
        if (plane < 16) out[((size_t)plane * S + r) * S + c] = 1.0f;
    }
    if (planes > 16 && to_move == 1)
        for (int j = 0; j < S * S; ++j) out[(size_t)16 * S * S + j] = 1.0f;
}

void oracle_gomoku_encode_batch(const int16_t* history, const uint8_t* n_hist,
                                const uint8_t* to_move, int B, int S, int planes, float* out,
                                int threads) {
    if (threads > 0) omp_set_num_threads(threads);
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b)
        oracle_gomoku_encode(history + (size_t)b * 16, n_hist[b], to_move[b], S, planes,
                             out + (size_t)b * planes * S * S);
}

/* Game result after a move list on an S x S freestyle Gomoku board (BLACK first):
 * 0 = ongoing, 1 = BLACK won, 2 = WHITE won, 3 = draw (full board).
 * GomokuState::refresh_winner_cache (src/games/gomoku/gomoku_state.cpp:792-860) checks
 * only the last move, for the player who made it, with
 * GomokuRules::is_five_in_a_row(action, player, allow_overline = true) for freestyle
 * (src/games/gomoku/gomoku_rules.cpp:71-100: a line of length >= 5 through the stone in
 * any of 4 directions); isTerminal (:131-156) adds the stalemate of a full board. */
/* rules 2 (Renju): BLACK wins only with a line of exactly five through the stone and no longer one
 * (refresh_winner_cache :812-843); WHITE, and both sides under the other rules, with five or more. */
int oracle_gomoku_result_rules(const int16_t* moves, int n, int S, int rules) {
    signed char board[32 * 32];
    memset(board, 0, sizeof(board));
    for (int i = 0; i < n; ++i) board[moves[i]] = (signed char)(1 + (i & 1));
    if (n == 0) return 0;
    const int last = moves[n - 1], who = board[last];
    const int r0 = last / S, c0 = last % S;
    static const int DR[4] = {1, 0, 1, 1}, DC[4] = {0, 1, 1, -1};
    int five_up = 0, exact = 0, over = 0;
    for (int d = 0; d < 4; ++d) {
        int len = 1;
        for (int k = 1;; ++k) {
            const int r = r0 + k * DR[d], c = c0 + k * DC[d];
            if (r < 0 || r >= S || c < 0 || c >= S || board[r * S + c] != who) break;
            ++len;
        }
        for (int k = 1;; ++k) {
            const int r = r0 - k * DR[d], c = c0 - k * DC[d];
            if (r < 0 || r >= S || c < 0 || c >= S || board[r * S + c] != who) break;
            ++len;
        }
        five_up = five_up || len >= 5; exact = exact || len == 5; over = over || len > 5;
    }
    if ((rules == 2 && who == 1) ? (exact && !over) : five_up) return who;
    return n >= S * S ? 3 : 0;
}
int oracle_gomoku_result(const int16_t* moves, int n, int S) { return oracle_gomoku_result_rules(moves, n, S, 0); }

/* Go planes, as GoState::getEnhancedTensorRepresentation (src/games/go/go_state.cpp:596-704)
 * with the CPU code of computeAttackDefensePlanes (:1306-1476).  Inputs are what the state
 * holds: stones (0 empty, 1 black, 2 white), the ko point (or -1), the side to move and the
 * legal cells (GoState::getLegalMoves, :227-265: not suicide, not the ko point, no superko
 * repetition - rule logic that stays with the caller).  planes: [10][S][S]
 *   0 black stones, 1 white stones (getTensorRepresentation, :557-594), 2 all ones iff black is
 *   to move; 3 / 4 min(1, liberties / 10) of the black / white group on its stones (:608-660);
 *   5 ko point (:666-674); 6 / 7 min(x, S-1-x) / (S/2), the same for y (:677-694);
 *   8 min(1, capture / 5), 9 min(1, defense) on the legal cells (:1349-1471):
 *     capture += size (group left without liberty other than the move) or 0.5 * size (one left),
 *       once per adjacent enemy STONE (a group touching the move twice counts twice);
 *     defense += (3 - liberties) * 0.5 for each adjacent friendly stone whose group has <= 2
 *       liberties; += 0.3 when >= 2 adjacent cells are friendly and <= 1 is empty.
 * Adjacent cells in the order of getAdjacentPositions (:1170-1186): up, right, down, left. */
void oracle_go_encode(const signed char* stones, int ko_point, int to_move, const unsigned char* legal, int S,
                      float* planes) {
    const int S2 = S * S;
    static const int DX[4] = {0, 1, 0, -1}, DY[4] = {-1, 0, 1, 0};
    int label[32 * 32], gsize[32 * 32], glibs[32 * 32], stack[32 * 32];
    memset(planes, 0, sizeof(float) * 10 * S2);
    for (int p = 0; p < S2; ++p) { label[p] = -1; gsize[p] = 0; glibs[p] = 0; }
    /* groups: flood fill, label = lowest cell of the group */
    for (int p = 0; p < S2; ++p) {
        if (stones[p] == 0 || label[p] >= 0) continue;
        int top = 0, n = 0;
        stack[top++] = p; label[p] = p;
        while (top) {
            const int c = stack[--top];
            ++n;
            const int x = c % S, y = c / S;
            for (int d = 0; d < 4; ++d) {
                const int nx = x + DX[d], ny = y + DY[d];
                if (nx < 0 || nx >= S || ny < 0 || ny >= S) continue;
                const int q = ny * S + nx;
                if (stones[q] == stones[p] && label[q] < 0) { label[q] = p; stack[top++] = q; }
            }
        }
        gsize[p] = n;
    }
    /* liberties: an empty cell counts once for every distinct group beside it */
    for (int e = 0; e < S2; ++e) {
        if (stones[e] != 0) continue;
        int seen[4], ns = 0;
        const int x = e % S, y = e / S;
        for (int d = 0; d < 4; ++d) {
            const int nx = x + DX[d], ny = y + DY[d];
            if (nx < 0 || nx >= S || ny < 0 || ny >= S) continue;
            const int q = ny * S + nx;
            if (stones[q] == 0) continue;
            int dup = 0;
            for (int k = 0; k < ns; ++k) dup |= seen[k] == label[q];
            if (!dup) { seen[ns++] = label[q]; ++glibs[label[q]]; }
        }
    }
    const float half = (float)S / 2.0f > 1.0f ? (float)S / 2.0f : 1.0f;
    for (int p = 0; p < S2; ++p) {
        const int x = p % S, y = p / S;
        if (stones[p] == 1) planes[0 * S2 + p] = 1.0f;
        if (stones[p] == 2) planes[1 * S2 + p] = 1.0f;
        planes[2 * S2 + p] = to_move == 1 ? 1.0f : 0.0f;
        if (stones[p] != 0) {
            const float v = (float)glibs[label[p]] / 10.0f;
            planes[(stones[p] == 1 ? 3 : 4) * S2 + p] = v < 1.0f ? v : 1.0f;
        }
        float dx = (float)(x < S - 1 - x ? x : S - 1 - x) / half, dy = (float)(y < S - 1 - y ? y : S - 1 - y) / half;
        planes[6 * S2 + p] = dx < 0.0f ? 0.0f : dx > 1.0f ? 1.0f : dx;
        planes[7 * S2 + p] = dy < 0.0f ? 0.0f : dy > 1.0f ? 1.0f : dy;
    }
    if (ko_point >= 0 && ko_point < S2) planes[5 * S2 + ko_point] = 1.0f;
    for (int m = 0; m < S2; ++m) {
        if (!legal[m]) continue;
        const int x = m % S, y = m / S;
        float capture = 0.0f, defense = 0.0f;
        int empty_adj = 0, friendly_adj = 0;
        for (int d = 0; d < 4; ++d) {
            const int nx = x + DX[d], ny = y + DY[d];
            if (nx < 0 || nx >= S || ny < 0 || ny >= S) continue;
            const int q = ny * S + nx, st = stones[q];
            if (st == 0) { ++empty_adj; continue; }
            const int g = label[q];
            if (st != to_move) {
                /* liberties of the group other than the move itself (the move is empty and adjacent) */
                const int left = glibs[g] - (stones[m] == 0 ? 1 : 0);
                if (left == 0) capture += (float)gsize[g] * 1.0f;
                else if (left == 1) capture += (float)gsize[g] * 0.5f;
            } else {
                ++friendly_adj;
                if (glibs[g] <= 2) defense += (3.0f - (float)glibs[g]) * 0.5f;
            }
        }
        if (friendly_adj >= 2 && empty_adj <= 1) defense += 0.3f;
        const float a = capture / 5.0f;
        planes[8 * S2 + m] = a < 1.0f ? a : 1.0f;
        planes[9 * S2 + m] = defense < 1.0f ? defense : 1.0f;
    }
}

void oracle_go_encode_batch(const signed char* stones, const int* ko_point, const unsigned char* to_move,
                            const unsigned char* legal, int B, int S, float* planes) {
    for (int b = 0; b < B; ++b)
        oracle_go_encode(stones + (size_t)b * S * S, ko_point[b], to_move[b], legal + (size_t)b * S * S, S,
                         planes + (size_t)b * 10 * S * S);
}

/* Chess planes, as ChessState::getEnhancedTensorRepresentation (src/games/chess/chess_state.cpp:
 * 745-826) with the CPU code of computeAttackDefensePlanes (:1753-1803).  Square = rank * 8 + file
 * (:408-410).  pieces[64]: 0 empty, else type 1..6 (pawn, knight, bishop, rook, queen, king), + 8 for
 * black.  meta: {side to move (1 white, 2 black), castling bits (1 WK, 2 WQ, 4 BK, 8 BQ), en passant
 * square or -1, halfmove clock, chess960, times the position has occurred}.  legal_to: the 64-bit set
 * of destination squares of the legal moves (move generation stays with the caller).
 * planes [20][8][8]: 0-5 white P N B R Q K, 6-11 black (getTensorRepresentation, :692-740);
 *   12 ones iff white to move; 13 0.25 per castling right; 14 en passant square; 15 min(1,
 *   halfmove / 100); 16 chess960; 17 clamp(occurrences / 3, 0, 1); 18 / 19 on every legal
 *   destination: min(1, sum / 10) of the values (1, 3, 3, 5, 9, 100) of the enemy / own pieces on the
 *   8 squares around it. */
void oracle_chess_encode(const signed char* pieces, const int* meta, const unsigned int* legal_to, float* planes) {
    static const float VAL[7] = {0.0f, 1.0f, 3.0f, 3.0f, 5.0f, 9.0f, 100.0f};
    memset(planes, 0, sizeof(float) * 20 * 64);
    const int mover = meta[0];
    float castling = 0.0f;
    for (int k = 0; k < 4; ++k) if (meta[1] & (1 << k)) castling += 0.25f;
    float half = (float)meta[3] / 100.0f; if (half > 1.0f) half = 1.0f;
    float rep = (float)meta[5] / 3.0f; rep = rep < 0.0f ? 0.0f : rep > 1.0f ? 1.0f : rep;
    for (int sq = 0; sq < 64; ++sq) {
        const int pc = pieces[sq];
        if (pc) planes[((pc & 7) - 1 + (pc & 8 ? 6 : 0)) * 64 + sq] = 1.0f;
        planes[12 * 64 + sq] = mover == 1 ? 1.0f : 0.0f;
        planes[13 * 64 + sq] = castling;
        planes[15 * 64 + sq] = half;
        planes[16 * 64 + sq] = meta[4] ? 1.0f : 0.0f;
        planes[17 * 64 + sq] = rep;
    }
    if (meta[2] >= 0 && meta[2] < 64) planes[14 * 64 + meta[2]] = 1.0f;
    for (int sq = 0; sq < 64; ++sq) {
        if (!((legal_to[sq >> 5] >> (sq & 31)) & 1u)) continue;
        const int r0 = sq / 8, c0 = sq % 8;
        float attack = 0.0f, defense = 0.0f;
        for (int dr = -1; dr <= 1; ++dr)
            for (int dc = -1; dc <= 1; ++dc) {
                if (!dr && !dc) continue;
                const int r = r0 + dr, c = c0 + dc;
                if (r < 0 || r >= 8 || c < 0 || c >= 8) continue;
                const int pc = pieces[r * 8 + c];
                if (!pc) continue;
                const int color = pc & 8 ? 2 : 1;
                if (color != mover) attack += VAL[pc & 7]; else defense += VAL[pc & 7];
            }
        const float a = attack / 10.0f, d = defense / 10.0f;
        planes[18 * 64 + sq] = a < 1.0f ? a : 1.0f;
        planes[19 * 64 + sq] = d < 1.0f ? d : 1.0f;
    }
}

void oracle_chess_encode_batch(const signed char* pieces, const int* meta, const unsigned int* legal_to, int B,
                               float* planes) {
    for (int b = 0; b < B; ++b)
        oracle_chess_encode(pieces + (size_t)b * 64, meta + (size_t)b * 6, legal_to + (size_t)b * 2,
                            planes + (size_t)b * 20 * 64);
}

/* The 3-plane Gomoku representation, GomokuState::getTensorRepresentation
 * (src/games/gomoku/gomoku_state.cpp:184-208), used when the network takes 3 input channels
 * (src/nn/resnet_model.cpp:258-260): plane 0 the stones of the side to move, plane 1 the
 * opponent's, plane 2 all ones iff BLACK (1) is to move.  stones: 0 empty, 1 black, 2 white. */
void oracle_gomoku_planes3_batch(const signed char* stones, const unsigned char* to_move, int B, int S, float* planes) {
    const int S2 = S * S;
    for (int b = 0; b < B; ++b)
        for (int p = 0; p < S2; ++p) {
            const int st = stones[(size_t)b * S2 + p], me = to_move[b];
            planes[((size_t)b * 3 + 0) * S2 + p] = st == me ? 1.0f : 0.0f;
            planes[((size_t)b * 3 + 1) * S2 + p] = (st != 0 && st != me) ? 1.0f : 0.0f;
            planes[((size_t)b * 3 + 2) * S2 + p] = me == 1 ? 1.0f : 0.0f;
        }
}

/* ---------------------------------------------------------------------------
 * One round of the leaf-parallel search on edge arrays: what happens between the
 * descent (oracle_traverse) and the backup (oracle_backup).
 *
 * The reference's pieces: MCTSNode::expand creates one child per legal move
 * (src/mcts/mcts_node.cpp:238-436; for Gomoku legal = empty cell, so the child
 * set of a new node is its parent's minus the move just made);
 * setPriorProbabilities gives child a the prior clamp(policy[a], 0, 1) with no
 * renormalisation (:546-553); the batched loop backs up the network value of
 * the leaf with the sign it has there (mcts_engine_batch_tree_simple.cpp:276-281),
 * the serial loop uses the game result for a finished game
 * (mcts_engine_search.cpp:588-610); the transposition table maps the Zobrist
 * key of a position (stones + side to move,
 * GomokuState::compute_hash_signature_internal, gomoku_state.cpp:947-958) to its
 * node and the parent's child reference is pointed at a node found there
 * (mcts_engine_batch_tree_simple.cpp:117-162).
 *
 * Order: the simulations of the round are taken one after another in index
 * order (the reference leaves the order to its thread scheduler).  A leaf edge
 * that an earlier simulation of the round already expanded is left alone; new
 * nodes get consecutive ids; with the table on (node_hash != NULL), a position
 * that already has a node in this game (node_hash equal; every node but the
 * roots is in the table) is shared instead of created.
 *
 * root_moves[t * moves_stride + i]: the game so far (BLACK first).  zobrist: 451
 * keys ([0,225) BLACK stones, [225,450) WHITE, [450] side to move).
 * terminal_out[i]: 0 not terminal, 1 the side to move has lost, 2 draw. */
static float quantized(float v, float q) { return q > 0.0f ? rintf(v * q) / q : v; }

/* GomokuRules::is_black_omok_forbidden, src/games/gomoku/gomoku_rules.cpp:176-198: with BLACK's stone on `action`
 * (an empty cell), a line of six or more through it (omok_is_six_in_a_row :118-127 over get_line_length_at_action
 * :38-69), or an open three in two or more of the four directions (omok_makes_double_three :161-174).  An open
 * three in a direction (check_omok_open_three_in_direction :129-159): one of the three placements of three
 * consecutive cells containing the action is all BLACK, and the cell before and the cell after it are on the board
 * and empty.  board: 0 empty, 1 black, 2 white. */
int oracle_omok_forbidden(const int8_t* board, int S, int action) {
    static const int dr[4] = {1, 0, 1, 1}, dc[4] = {0, 1, 1, -1};
    const int r = action / S, c = action % S;
#define OB_BLACK(rr, cc) ((rr) >= 0 && (rr) < S && (cc) >= 0 && (cc) < S && (((rr) * S + (cc)) == action || board[(rr) * S + (cc)] == 1))
#define OB_EMPTY(rr, cc) ((rr) >= 0 && (rr) < S && (cc) >= 0 && (cc) < S && ((rr) * S + (cc)) != action && board[(rr) * S + (cc)] == 0)
    int open_threes = 0;
    for (int d = 0; d < 4; ++d) {
        int run = 1;
        for (int k = 1; k < S && OB_BLACK(r + k * dr[d], c + k * dc[d]); ++k) ++run;
        for (int k = 1; k < S && OB_BLACK(r - k * dr[d], c - k * dc[d]); ++k) ++run;
        if (run >= 6) return 1;
    }
    for (int d = 0; d < 4; ++d) {
        int open = 0;
        for (int i = 0; i < 3 && !open; ++i) {
            const int r0 = r - i * dr[d], c0 = c - i * dc[d];
            int three = 1;
            for (int k = 0; k < 3; ++k) three = three && OB_BLACK(r0 + k * dr[d], c0 + k * dc[d]);
            if (three && OB_EMPTY(r0 - dr[d], c0 - dc[d]) && OB_EMPTY(r0 + 3 * dr[d], c0 + 3 * dc[d])) open = 1;
        }
        open_threes += open;
    }
#undef OB_BLACK
#undef OB_EMPTY
    return open_threes >= 2;
}
/* ---------------------------------------------------------------------------------------------
 * Renju: BLACK's forbidden moves.  GomokuRules::is_black_renju_forbidden and what it calls,
 * src/games/gomoku/gomoku_rules.cpp:200-879, restated on a board array (0 empty, 1 black, 2 white) that
 * already holds BLACK's stone on the cell under test; hypothetical further stones are set and cleared in
 * place where the reference wraps its board accessor in another lambda.
 * ------------------------------------------------------------------------------------------- */
static const int RJ_DR[4] = {1, 0, 1, 1}, RJ_DC[4] = {0, 1, 1, -1};
#define RJ_IN(S, r, c) ((r) >= 0 && (r) < (S) && (c) >= 0 && (c) < (S))
static int rj_black(const int8_t* b, int S, int r, int c) { return RJ_IN(S, r, c) && b[r * S + c] == 1; }
static int rj_empty(const int8_t* b, int S, int r, int c) { return RJ_IN(S, r, c) && b[r * S + c] == 0; }
/* get_line_length_at_action (:38-69): BLACK's run through a cell that holds a black stone, else 0 */
static int rj_len(const int8_t* b, int S, int a, int d) {
    const int r = a / S, c = a % S;
    if (b[a] != 1) return 0;
    int n = 1;
    for (int i = 1; i < S && rj_black(b, S, r + i * RJ_DR[d], c + i * RJ_DC[d]); ++i) ++n;
    for (int i = 1; i < S && rj_black(b, S, r - i * RJ_DR[d], c - i * RJ_DC[d]); ++i) ++n;
    return n;
}
static int rj_len_if_filled(int8_t* b, int S, int cell, int d) {      /* the run through `cell` with a black stone put there */
    const int8_t keep = b[cell];
    b[cell] = 1;
    const int n = rj_len(b, S, cell, d);
    b[cell] = keep;
    return n;
}
static int rj_overline(const int8_t* b, int S, int a) {               /* renju_is_overline :251-258 */
    for (int d = 0; d < 4; ++d) if (rj_len(b, S, a, d) > 5) return 1;
    return 0;
}
/* count_renju_fours_at_action :260-436: per direction at most one four - a solid four that one more stone makes
 * exactly five, else four stones and a gap in a window of five whose gap makes exactly five, else a stone one
 * gap away (at distance 2-4) whose gap would join a run of three or more with room to extend. */
static int rj_fours(int8_t* b, int S, int a) {
    const int r = a / S, c = a % S;
    int count = 0;
    for (int d = 0; d < 4; ++d) {
        const int dr = RJ_DR[d], dc = RJ_DC[d];
        int found = 0;
        for (int off = 0; off < 4 && !found; ++off) {
            const int r0 = r - off * dr, c0 = c - off * dc;
            int solid = 1;
            for (int i = 0; i < 4; ++i) solid = solid && rj_black(b, S, r0 + i * dr, c0 + i * dc);
            if (!solid) continue;
            const int rb = r0 - dr, cb = c0 - dc, ra = r0 + 4 * dr, ca = c0 + 4 * dc;
            const int open_before = rj_empty(b, S, rb, cb), open_after = rj_empty(b, S, ra, ca);
            int five = 0;
            if (open_before && rj_len_if_filled(b, S, rb * S + cb, d) == 5) five = 1;
            if (!five && open_after && rj_len_if_filled(b, S, ra * S + ca, d) == 5) five = 1;
            if (five) found = 1;
        }
        for (int off = 0; off < 5 && !found; ++off) {
            const int r0 = r - off * dr, c0 = c - off * dc;
            int stones = 0, empties = 0, gap = -1, valid = 1;
            for (int i = 0; i < 5 && valid; ++i) {
                const int rk = r0 + i * dr, ck = c0 + i * dc;
                if (!RJ_IN(S, rk, ck)) { valid = 0; break; }
                if (b[rk * S + ck] == 1) ++stones;
                else if (b[rk * S + ck] == 0) { ++empties; gap = rk * S + ck; }
                else valid = 0;
            }
            if (valid && stones == 4 && empties == 1 && rj_len_if_filled(b, S, gap, d) == 5) found = 1;
        }
        for (int dist = 2; dist <= 4 && !found; ++dist) {
            const int rf = r + dist * dr, cf = c + dist * dc;
            if (rj_black(b, S, rf, cf)) {
                const int rg = r + (dist - 1) * dr, cg = c + (dist - 1) * dc;
                if (rj_empty(b, S, rg, cg) && rj_len_if_filled(b, S, rg * S + cg, d) >= 3 &&
                    (rj_empty(b, S, r - dr, c - dc) || rj_empty(b, S, rf + dr, cf + dc))) { found = 1; break; }
            }
            const int rk = r - dist * dr, ck = c - dist * dc;
            if (rj_black(b, S, rk, ck)) {
                const int rg = r - (dist - 1) * dr, cg = c - (dist - 1) * dc;
                if (rj_empty(b, S, rg, cg) && rj_len_if_filled(b, S, rg * S + cg, d) >= 3 &&
                    (rj_empty(b, S, rk - dr, ck - dc) || rj_empty(b, S, r + dr, c + dc))) { found = 1; break; }
            }
        }
        count += found;
    }
    return count;
}
static int rj_depth_hits = 0;                                        /* how often the depth limit below cut a recursion */
static int rj_depth_seen = 0;                                        /* deepest recursion so far */
int oracle_renju_depth_hits(void) { return rj_depth_hits; }
int oracle_renju_depth_seen(void) { return rj_depth_seen; }
enum { RJ_MAX_DEPTH = 6 };
static int rj_double_three(int8_t* b, int S, int a, int depth);
/* A triple of consecutive black stones starting at (r0, c0) along d is a "three" (is_renju_three_definition
 * :580-635) when one of its two end extensions is empty and putting a stone there gives a straight four (four in
 * a row with both ends empty, :637-676) that is itself allowed (no overline, no double four, no double three -
 * check_s4_forbidden_primary :472-484 and the checker it is given, :449-456) and makes no five or more. */
static int rj_three(int8_t* b, int S, int r0, int c0, int d, int depth) {
    const int dr = RJ_DR[d], dc = RJ_DC[d];
    const int ext[2][2] = {{r0 - dr, c0 - dc}, {r0 + 3 * dr, c0 + 3 * dc}};
    for (int e = 0; e < 2; ++e) {
        const int rs = ext[e][0], cs = ext[e][1];
        if (!rj_empty(b, S, rs, cs)) continue;
        const int spot = rs * S + cs;
        b[spot] = 1;
        /* the four: the triple plus the spot */
        const int rf = e == 0 ? rs : r0, cf = e == 0 ? cs : c0;      /* first stone of the four */
        int ok = rj_empty(b, S, rf - dr, cf - dc) && rj_empty(b, S, rf + 4 * dr, cf + 4 * dc);
        if (ok && (rj_overline(b, S, spot) || rj_fours(b, S, spot) >= 2 || rj_double_three(b, S, spot, depth + 1))) ok = 0;
        if (ok)
            for (int d2 = 0; d2 < 4; ++d2)
                if (rj_len(b, S, spot, d2) >= 5) { ok = 0; break; }
        b[spot] = 0;
        if (ok) return 1;
    }
    return 0;
}
/* check_renju_double_three_recursive :460-578: the threes through the stone on `a`; fewer than two: allowed.  With
 * two or more the reference then asks how many of them can be taken to an allowed straight four
 * (check_renju_double_three_exception_recursive :678-745) and lets the move pass when at most one can - which is
 * the very test that made each of them a three, so the count equals the number of threes; it is restated as the
 * reference states it all the same. */
static int rj_double_three(int8_t* b, int S, int a, int depth) {
    if (depth > RJ_MAX_DEPTH) { ++rj_depth_hits; return 0; }
    if (depth > rj_depth_seen) rj_depth_seen = depth;
    const int r = a / S, c = a % S;
    int threes = 0, resolvable = 0;
    int tr[12], tc[12], td[12];
    for (int d = 0; d < 4; ++d)
        for (int off = 0; off < 3; ++off) {
            const int r0 = r - off * RJ_DR[d], c0 = c - off * RJ_DC[d];
            int all = 1;
            for (int k = 0; k < 3; ++k) all = all && rj_black(b, S, r0 + k * RJ_DR[d], c0 + k * RJ_DC[d]);
            if (all && rj_three(b, S, r0, c0, d, depth)) { tr[threes] = r0; tc[threes] = c0; td[threes] = d; ++threes; }
        }
    if (threes < 2) return 0;
    for (int t = 0; t < threes; ++t) resolvable += rj_three(b, S, tr[t], tc[t], td[t], depth);
    return resolvable <= 1 ? 0 : 1;
}
/* is_black_renju_forbidden :200-249 for an empty cell of `board` */
int oracle_renju_forbidden(const int8_t* board, int S, int action) {
    int8_t b[32 * 32];
    memcpy(b, board, (size_t)S * S);
    b[action] = 1;
    int exact_five = 0, over = 0;
    for (int d = 0; d < 4; ++d) {
        const int n = rj_len(b, S, action, d);
        exact_five = exact_five || n == 5;
        over = over || n > 5;
    }
    if (exact_five && !over) return 0;
    if (over) return 1;
    if (rj_fours(b, S, action) >= 2) return 1;
    return rj_double_three(b, S, action, 0);
}

/* The legal moves of a Gomoku position (GomokuState::is_move_valid_internal, src/games/gomoku/gomoku_state.cpp:
 * 915-943, without the opening restriction): the empty cells, minus BLACK's forbidden ones under Omok (rules 1)
 * or Renju (rules 2) when BLACK is to move.  legal_out: one bit per cell, mask_words words. */
void oracle_gomoku_legal_mask(const int16_t* moves, int n_moves, int S, int rules, uint32_t* legal_out, int mask_words) {
    int8_t board[32 * 32];
    memset(board, 0, sizeof board);
    for (int i = 0; i < n_moves; ++i) board[moves[i]] = (int8_t)(1 + (i & 1));
    for (int w = 0; w < mask_words; ++w) legal_out[w] = 0;
    const int black_to_move = (n_moves & 1) == 0;
    for (int a = 0; a < S * S; ++a) {
        if (board[a]) continue;
        if (rules == 1 && black_to_move && oracle_omok_forbidden(board, S, a)) continue;
        if (rules == 2 && black_to_move && oracle_renju_forbidden(board, S, a)) continue;
        legal_out[a >> 5] |= 1u << (a & 31);
    }
}

/* The children a new node gets out of its legal moves (MCTSNode::expand,
 * src/mcts/mcts_node.cpp:283-340): at most max_children, the first in move order (:287-291, 1,000 in the
 * reference), and with progressive widening `target` of those chosen at random (:297-340 with the shuffle at
 * :356).  The reference seeds its shuffle from the operating system, so its subset cannot be reproduced; the
 * choice restated here is the library's: a move's rank is a 64-bit mix of (seed, node id, move) and the `target`
 * lowest ranks stay.  max_children <= 0: no cap; target <= 0: no widening. */
static uint64_t widen_key(uint64_t seed, int id, int s) {
    uint64_t z = seed ^ ((uint64_t)(id + 1) * 0x9E3779B97F4A7C15ull) ^ ((uint64_t)(s + 1) * 0xC2B2AE3D27D4EB4Full);
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull; z ^= z >> 27; z *= 0x94D049BB133111EBull; z ^= z >> 31;
    return z;
}
void oracle_widen_mask(const uint32_t* empty, uint32_t* exists, int n_children, int mask_words,
                       int max_children, int target, uint64_t seed, int id) {
    int total = 0;
    for (int w = 0; w < mask_words; ++w) exists[w] = 0;
    for (int s = 0; s < n_children; ++s)
        if (((empty[s >> 5] >> (s & 31)) & 1u) && (max_children <= 0 || total < max_children)) {
            exists[s >> 5] |= 1u << (s & 31);
            ++total;
        }
    if (target <= 0 || total <= target) return;
    uint32_t capped[64];                       /* the moves that survived the cap: ranks are taken among them */
    for (int w = 0; w < mask_words && w < 64; ++w) capped[w] = exists[w];
    for (int s = 0; s < n_children; ++s) {
        if (!((capped[s >> 5] >> (s & 31)) & 1u)) continue;
        const uint64_t k = widen_key(seed, id, s);
        int rank = 0;
        for (int s2 = 0; s2 < n_children; ++s2) {
            if (s2 == s || !((capped[s2 >> 5] >> (s2 & 31)) & 1u)) continue;
            const uint64_t k2 = widen_key(seed, id, s2);
            if (k2 < k || (k2 == k && s2 < s)) ++rank;
        }
        if (rank >= target) exists[s >> 5] &= ~(1u << (s & 31));
    }
}
/* The count progressive widening asks for at a node with `visits` visits (:305-308):
 * max(8, c * (visits + 1)^k), computed in double and compared as float as the reference's expression does. */
int oracle_widen_target(float cpw, float kpw, int visits) {
    const float want = (float)((double)cpw * pow((double)(visits + 1), (double)kpw));
    return (int)(want > 8.0f ? want : 8.0f);
}

void oracle_search_expand_widen(int32_t* N, float* W, float* P, int32_t* VL, uint32_t* legal,
                          int32_t* node_visits, int32_t* child_node, uint64_t* node_hash,
                          int32_t* n_used, int max_nodes, int n_children, int pitch, int mask_words,
                          const int32_t* paths, const int32_t* path_len, int n_sims, int max_depth,
                          int sims_per_tree, const int16_t* root_moves, const int32_t* root_n_moves,
                          int moves_stride, int S, const float* policy, int policy_size,
                          const float* value, float value_sign, float value_quantum,
                          const uint64_t* zobrist, int n_trees, float* leaf_value_out,
                          int32_t* terminal_out, uint32_t* empty, int max_children, int widen_target,
                          uint64_t widen_seed, int rules) {
    int16_t game[32 * 32];
    for (int i = 0; i < n_sims; ++i) {
        const int tree = i / sims_per_tree;
        const int len = path_len[i] > max_depth ? max_depth : path_len[i];
        const int32_t* p = paths + (size_t)i * max_depth * 2;
        const int n0 = root_n_moves[tree];
        /* the leaf position: the root's moves, then the path's */
        for (int k = 0; k < n0; ++k) game[k] = root_moves[(size_t)tree * moves_stride + k];
        for (int d = 0; d < len; ++d) game[n0 + d] = (int16_t)p[2 * d + 1];
        int term = 0;
        float tv = 0.0f;
        if (len > 0) {
            const int res = oracle_gomoku_result_rules(game, n0 + len, S, rules);
            if (res == 1 || res == 2) { term = 1; tv = -1.0f; }   /* the last mover won: the side to move has lost */
            else if (res == 3) { term = 2; tv = 0.0f; }
        }
        terminal_out[i] = term;
        leaf_value_out[i] = value_sign * (term ? tv : quantized(value[i], value_quantum));
        if (len == 0 || term) continue;
        const int parent = p[2 * (len - 1)], slot = p[2 * (len - 1) + 1];
        const size_t e = (size_t)parent * pitch + slot;
        if (child_node[e] >= 0) continue;                         /* expanded before, or earlier in this round */
        uint64_t h = 0;
        if (node_hash) {
            const int mover = 1 + ((n0 + len - 1) & 1);           /* who made the move behind the edge */
            h = node_hash[parent] ^ zobrist[(mover - 1) * 225 + slot] ^ zobrist[450];
            if (h == 0) h = 1;
            int found = -1;
            for (int k = n_trees; k < *n_used && found < 0; ++k)
                if (node_hash[k] == h) found = k;
            if (found >= 0) { child_node[e] = found; continue; }  /* transposition: share the node */
        }
        if (*n_used >= max_nodes) continue;                       /* pool exhausted: the edge stays a leaf */
        const int id = (*n_used)++;
        const size_t row = (size_t)id * pitch;
        /* empty != NULL: the positions' empty cells are kept apart from the children a node was given */
        const uint32_t* pm = (empty ? empty : legal) + (size_t)parent * mask_words;
        uint32_t* own = (empty ? empty : legal) + (size_t)id * mask_words;
        uint32_t* cm = legal + (size_t)id * mask_words;
        for (int w = 0; w < mask_words; ++w) own[w] = pm[w] & ~((w == (slot >> 5)) ? (1u << (slot & 31)) : 0u);
        if (empty) {
            /* the moves the rules leave the side to move, then the limits on children */
            uint32_t legal_now[64];
            oracle_gomoku_legal_mask(game, n0 + len, S, rules, legal_now, mask_words);
            oracle_widen_mask(legal_now, cm, n_children, mask_words, max_children, widen_target, widen_seed, id);
        }
        for (int s = 0; s < pitch; ++s) {
            float pr = 0.0f;
            if (s < n_children && ((cm[s >> 5] >> (s & 31)) & 1u) && s < policy_size)
                pr = fminf(1.0f, fmaxf(0.0f, policy[(size_t)i * policy_size + s]));
            N[row + s] = 0; W[row + s] = 0.0f; VL[row + s] = 0; P[row + s] = pr; child_node[row + s] = -1;
        }
        node_visits[id] = 0;
        if (node_hash) node_hash[id] = h;
        child_node[e] = id;
    }
}

void oracle_search_expand(int32_t* N, float* W, float* P, int32_t* VL, uint32_t* legal,
                          int32_t* node_visits, int32_t* child_node, uint64_t* node_hash,
                          int32_t* n_used, int max_nodes, int n_children, int pitch, int mask_words,
                          const int32_t* paths, const int32_t* path_len, int n_sims, int max_depth,
                          int sims_per_tree, const int16_t* root_moves, const int32_t* root_n_moves,
                          int moves_stride, int S, const float* policy, int policy_size,
                          const float* value, float value_sign, float value_quantum,
                          const uint64_t* zobrist, int n_trees, float* leaf_value_out,
                          int32_t* terminal_out) {
    oracle_search_expand_widen(N, W, P, VL, legal, node_visits, child_node, node_hash, n_used, max_nodes, n_children,
                               pitch, mask_words, paths, path_len, n_sims, max_depth, sims_per_tree, root_moves,
                               root_n_moves, moves_stride, S, policy, policy_size, value, value_sign, value_quantum,
                               zobrist, n_trees, leaf_value_out, terminal_out, NULL, 0, 0, 0, 0);
}

/* MCTSEngine::addDirichletNoise, src/mcts/mcts_engine_eval.cpp:83-110.  The noise
 * part (:83-100): one Gamma(alpha, 1) draw per child (`gammas`, in child order),
 * summed in fp32 and each divided by the sum; a zero sum gives uniform noise. */
void oracle_dirichlet_normalize(float* gammas, int n) {
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += gammas[i];
    for (int i = 0; i < n; ++i) gammas[i] = sum > 0.0f ? gammas[i] / sum : 1.0f / (float)n;
}
/* The mix (:102-109): prior = (1 - eps) * prior + eps * noise on every child of the
 * root.  noise: [n][pitch], indexed by child slot. */
void oracle_mix_noise(float* P, const uint32_t* legal, int n_children, int pitch, int mask_words,
                      const int32_t* node_ids, int n, const float* noise, float eps) {
    for (int i = 0; i < n; ++i) {
        const int node = node_ids ? node_ids[i] : i;
        const uint32_t* m = legal + (size_t)node * mask_words;
        for (int s = 0; s < n_children; ++s)
            if ((m[s >> 5] >> (s & 31)) & 1u) {
                float* p = P + (size_t)node * pitch + s;
                *p = (1.0f - eps) * *p + eps * noise[(size_t)i * pitch + s];
            }
    }
}

/* GomokuAttackDefenseModule, src/utils/attack_defense_module.cpp.
 * count_threats_for_color (:205-222): windows of 5 asking for 3 stones and windows of 6 asking for 4, along rows
 * and columns (:333-392, count_1d_patterns on the mask and on its transpose) and along both diagonals (:394-487).
 * A window counts when both end cells are empty and the cells between them hold exactly `need` or `need - 1`
 * stones of the colour ("perfect" and "broken" are added up, :375-390). */
static int threat_windows(const int8_t* board, int S, int color, int len, int need) {
    static const int dr[4] = {0, 1, 1, 1}, dc[4] = {1, 0, 1, -1};
    int count = 0;
    for (int d = 0; d < 4; ++d)
        for (int r = 0; r < S; ++r)
            for (int c = 0; c < S; ++c) {
                const int r1 = r + (len - 1) * dr[d], c1 = c + (len - 1) * dc[d];
                if (r1 >= S || c1 < 0 || c1 >= S) continue;
                int inside = 0;
                for (int k = 1; k < len - 1; ++k) inside += board[(r + k * dr[d]) * S + c + k * dc[d]] == color;
                const int ends_empty = board[r * S + c] == 0 && board[r1 * S + c1] == 0;
                if (ends_empty && (inside == need || inside == need - 1)) ++count;
            }
    return count;
}
int oracle_gomoku_threats(const int8_t* board, int S, int color) {
    return threat_windows(board, S, color, 5, 3) + threat_windows(board, S, color, 6, 4);
}
/* compute_planes (:61-111) with compute_attack_bonus / compute_defense_bonus (:113-203) for every empty cell m of
 * every board: `after` is the board handed to the module - the position itself (stone_placed == 0, what
 * compute_planes does) or the position with the mover's stone on m (stone_placed != 0) - and `before` is `after`
 * with m cleared when it is empty or the mover's (:123-139).  attack = threats(after, mover) - threats(before,
 * mover); defense = threats(before, opponent) - threats(after, opponent).  Occupied cells stay zero. */
void oracle_gomoku_attack_defense(const int8_t* stones, const uint8_t* to_move, int B, int S, int stone_placed,
                                  float* attack, float* defense) {
    int8_t after[32 * 32], before[32 * 32];
    const int cells = S * S;
    for (int b = 0; b < B; ++b) {
        const int p = to_move[b], o = p == 1 ? 2 : 1;
        for (int m = 0; m < cells; ++m) {
            attack[(size_t)b * cells + m] = 0.0f;
            defense[(size_t)b * cells + m] = 0.0f;
            if (stones[(size_t)b * cells + m] != 0) continue;
            memcpy(after, stones + (size_t)b * cells, (size_t)cells);
            if (stone_placed) after[m] = (int8_t)p;
            memcpy(before, after, (size_t)cells);
            if (before[m] == 0 || before[m] == p) before[m] = 0;
            attack[(size_t)b * cells + m] = (float)oracle_gomoku_threats(after, S, p) - (float)oracle_gomoku_threats(before, S, p);
            defense[(size_t)b * cells + m] = (float)oracle_gomoku_threats(before, S, o) - (float)oracle_gomoku_threats(after, S, o);
        }
    }
}
