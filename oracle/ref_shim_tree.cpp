// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points that drive the reference project's *own* classes, compiled
// from the reference's source files where they lie (see oracle/Makefile).  The
// resulting library (oracle/_ref/libref_tree.so) is used only to pin the CPU
// restatement in oracle/oracle.c and as the timed CPU baseline.
//
// Reference classes exercised:
//   alphazero::mcts::MCTSNode::selectChild        src/mcts/mcts_node.cpp:90
//   MCTSNode::addVirtualLoss/removeVirtualLoss    src/mcts/mcts_node_virtual_loss.cpp:15,32
//   MCTSNode::update                              src/mcts/mcts_node_virtual_loss.cpp:54
//   MCTSNode::expand                              src/mcts/mcts_node.cpp:238
//   GomokuAttackDefenseModule::compute_planes     src/utils/attack_defense_module.cpp:61
//   GomokuAttackDefenseModule::compute_bonuses    src/utils/attack_defense_module.cpp:50
//   GomokuState::getEnhancedTensorRepresentation  src/games/gomoku/gomoku_state.cpp:210
//   GomokuState::getTensorRepresentation          src/games/gomoku/gomoku_state.cpp:184
#include <cstdint>
#include <cstring>
#include <memory>
#include <optional>
#include <string>
#include <vector>
#include <chrono>
#include <omp.h>

#include "core/igamestate.h"
#include "mcts/mcts_node.h"
#include "games/gomoku/gomoku_state.h"
#include "games/go/go_state.h"
#include "games/chess/chess_state.h"
#include "games/chess/chess_types.h"
#include "utils/attack_defense_module.h"
#include "ref_tiny_state.h"

using alphazero::core::GameResult;
using alphazero::mcts::MCTSNode;
using ref_tiny::Family;
using ref_tiny::TinyState;
using ref_tiny::index_of;
using ref_tiny::load_stats;
using ref_tiny::make_family;

extern "C" {

// selectChild on one parent whose children carry the given statistics
// (children listed in index order; only existing == legal children are given).
// Returns the selected child's index or -1 when there are no children.
int ref_select_child(int n_children, const int32_t* N, const float* W, const float* P,
                     const int32_t* VL, int n_parent, float c_puct) {
    Family f = make_family(n_children, N, W, P, VL, n_parent);
    return index_of(f, f.parent->selectChild(c_puct, false, 3000.0f));
}

// Batched form over CSR-compacted parents, OpenMP over parents, followed by
// applyVirtualLoss(vl) and revertVirtualLoss(vl) on the selected child, as the
// search loop does (src/mcts/mcts_engine_batch_tree_simple.cpp:102-111,279).
// vl_after_apply / vl_after_revert may be null.  Returns seconds spent inside
// the select+apply+revert calls only (tree construction excluded), summed over
// the repeat count, measured as wall time of the parallel region.
double ref_select_batch(int n_parents, const int64_t* row_ptr, const int32_t* N, const float* W,
                        const float* P, const int32_t* VL, const int32_t* n_parent, float c_puct,
                        int vl_amount, int32_t* sel_out, int32_t* vl_after_apply,
                        int32_t* vl_after_revert, int repeats, int threads) {
    if (threads > 0) omp_set_num_threads(threads);
    std::vector<Family> fam(n_parents);
#pragma omp parallel for schedule(dynamic, 16)
    for (int p = 0; p < n_parents; ++p) {
        int64_t a = row_ptr[p], b = row_ptr[p + 1];
        fam[p] = make_family((int)(b - a), N + a, W + a, P + a, VL + a, n_parent[p]);
    }
    double total = 0.0;
    for (int r = 0; r < (repeats < 1 ? 1 : repeats); ++r) {
        auto t0 = std::chrono::steady_clock::now();
#pragma omp parallel for schedule(static)
        for (int p = 0; p < n_parents; ++p) {
            auto best = fam[p].parent->selectChild(c_puct, false, 3000.0f);
            int idx = index_of(fam[p], best);
            sel_out[p] = idx;
            if (best) {
                best->applyVirtualLoss(vl_amount);
                if (vl_after_apply) vl_after_apply[p] = best->getVirtualLoss();
                best->revertVirtualLoss(vl_amount);
                if (vl_after_revert) vl_after_revert[p] = best->getVirtualLoss();
            }
        }
        total += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    }
    return total;
}

// A sequence of virtual-loss operations on one node: op > 0 addVirtualLoss(op),
// op < 0 removeVirtualLoss(-op), op == 0 the argument-less removeVirtualLoss().
// out[i] = getVirtualLoss() after operation i.
void ref_vl_ops(int initial, const int32_t* ops, int n_ops, int32_t* out) {
    auto node = MCTSNode::create(std::make_unique<TinyState>());
    if (initial > 0) node->addVirtualLoss(initial);
    for (int i = 0; i < n_ops; ++i) {
        if (ops[i] > 0) node->addVirtualLoss(ops[i]);
        else if (ops[i] < 0) node->removeVirtualLoss(-ops[i]);
        else node->removeVirtualLoss();
        out[i] = node->getVirtualLoss();
    }
}

// The backup loop of the batched search (mcts_engine_batch_tree_simple.cpp:
// 276-281) on a path of real nodes given root->leaf; walks leaf->root doing
// update(v); revertVirtualLoss(vl); v = -v.  In/out: N, VL; W in, and
// mean_out[i] = getValue() (= W/N in fp32) after the walk.
void ref_backup_path(int depth, int32_t* N, const float* W, int32_t* VL, float leaf_value,
                     int vl_amount, float* mean_out) {
    std::vector<std::shared_ptr<MCTSNode>> path;
    for (int i = 0; i < depth; ++i) {
        auto n = MCTSNode::create(std::make_unique<TinyState>());
        load_stats(*n, N[i], W[i], VL[i], 0.0f);
        path.push_back(n);
    }
    float v = leaf_value;
    for (auto it = path.rbegin(); it != path.rend(); ++it) {
        (*it)->update(v);
        (*it)->revertVirtualLoss(vl_amount);
        v = -v;
    }
    for (int i = 0; i < depth; ++i) {
        N[i] = path[i]->getVisitCount();
        VL[i] = path[i]->getVirtualLoss();
        mean_out[i] = path[i]->getValue();
    }
}

// Real GomokuState: play `n_moves` actions from the empty board, then write
// getEnhancedTensorRepresentation() (19 planes) into planes19[19*S*S] and
// getTensorRepresentation() (3 planes) into planes3[3*S*S] (either may be
// null).  Returns the side to move (1 = BLACK, 2 = WHITE), or -1 on an
// illegal move.
int ref_gomoku_encode(int board_size, const int32_t* moves, int n_moves, float* planes19,
                      float* planes3) {
    alphazero::games::gomoku::GomokuState st(board_size, false, false, 0, false);
    for (int i = 0; i < n_moves; ++i) {
        if (!st.isLegalMove(moves[i])) return -1;
        st.makeMove(moves[i]);
    }
    const int S = board_size;
    if (planes19) {
        auto t = st.getEnhancedTensorRepresentation();
        for (size_t c = 0; c < t.size(); ++c)
            for (int r = 0; r < S; ++r)
                std::memcpy(planes19 + (c * S + r) * S, t[c][r].data(), sizeof(float) * S);
    }
    if (planes3) {
        auto t = st.getTensorRepresentation();
        for (size_t c = 0; c < t.size(); ++c)
            for (int r = 0; r < S; ++r)
                std::memcpy(planes3 + (c * S + r) * S, t[c][r].data(), sizeof(float) * S);
    }
    return st.getCurrentPlayer();
}

// Encoder CPU baseline: encode `n_states` positions (CSR move lists) with
// OpenMP over states as src/nn/resnet_model.cpp:410 does.  Returns seconds
// (-1 when a move list is illegal).
double ref_gomoku_encode_batch(int board_size, int n_states, const int64_t* row_ptr,
                               const int32_t* moves, float* planes19, int threads) {
    if (threads > 0) omp_set_num_threads(threads);
    const int S = board_size;
    std::vector<std::unique_ptr<alphazero::games::gomoku::GomokuState>> st(n_states);
    for (int s = 0; s < n_states; ++s) {
        st[s] = std::make_unique<alphazero::games::gomoku::GomokuState>(S, false, false, 0, false);
        for (int64_t i = row_ptr[s]; i < row_ptr[s + 1]; ++i) {
            if (!st[s]->isLegalMove(moves[i])) return -1.0;  // caller must pass legal, unfinished games
            st[s]->makeMove(moves[i]);
        }
    }
    auto t0 = std::chrono::steady_clock::now();
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < n_states; ++s) {
        auto t = st[s]->getEnhancedTensorRepresentation();
        float* dst = planes19 + (size_t)s * 19 * S * S;
        for (size_t c = 0; c < t.size(); ++c)
            for (int r = 0; r < S; ++r)
                std::memcpy(dst + (c * S + r) * S, t[c][r].data(), sizeof(float) * S);
    }
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

// Game result the reference reports after playing `moves` (all but the last must leave the
// game unfinished): 0 ongoing, 1 BLACK won, 2 WHITE won, 3 draw, -1 illegal move list.
int ref_gomoku_result(int board_size, const int32_t* moves, int n_moves) {
    alphazero::games::gomoku::GomokuState st(board_size, false, false, 0, false);
    for (int i = 0; i < n_moves; ++i) {
        if (st.isTerminal() || !st.isLegalMove(moves[i])) return -1;
        st.makeMove(moves[i]);
    }
    if (!st.isTerminal()) return 0;
    switch (st.getGameResult()) {
        case GameResult::WIN_PLAYER1: return 1;
        case GameResult::WIN_PLAYER2: return 2;
        case GameResult::DRAW: return 3;
        default: return 0;
    }
}

// The same on a state constructed with the variant flags; the moves are played without asking isLegalMove, so that
// a line longer than five by BLACK can be put on the board.
int ref_gomoku_result_variant(int board_size, const int32_t* moves, int n_moves, int use_renju, int use_omok) {
    alphazero::games::gomoku::GomokuState st(board_size, use_renju != 0, use_omok != 0, 0, false);
    for (int i = 0; i < n_moves; ++i) {
        try { st.makeMove(moves[i]); } catch (...) { return -1; }
    }
    if (!st.isTerminal()) return 0;
    switch (st.getGameResult()) {
        case GameResult::WIN_PLAYER1: return 1;
        case GameResult::WIN_PLAYER2: return 2;
        case GameResult::DRAW: return 3;
        default: return 0;
    }
}

// Real GoState (Chinese rules, positional superko as the constructor's defaults): play
// `n_moves` actions (cell index y*S+x, or -1 for a pass) from the empty board, then export what a
// device encoder takes (stones 0/1/2, ko point or -1, side to move, legal cells as bytes; the
// pass move is always legal and not listed) and getEnhancedTensorRepresentation()
// (src/games/go/go_state.cpp:596-704: 10 planes) into planes10[10*S*S].  Any output may be
// null.  Returns the number of planes, or -1 on an illegal move / finished game.
int ref_go_encode(int board_size, const int32_t* moves, int n_moves, int8_t* stones, int32_t* ko_point,
                  int32_t* to_move, uint8_t* legal, float* planes10) {
    alphazero::games::go::GoState st(board_size);
    for (int i = 0; i < n_moves; ++i) {
        if (st.isTerminal() || !st.isLegalMove(moves[i])) return -1;
        st.makeMove(moves[i]);
    }
    const int S = board_size, S2 = S * S;
    if (stones) for (int p = 0; p < S2; ++p) stones[p] = (int8_t)st.getStone(p);
    if (ko_point) *ko_point = st.getKoPoint();
    if (to_move) *to_move = st.getCurrentPlayer();
    if (legal) {
        std::memset(legal, 0, S2);
        for (int m : st.getLegalMoves()) if (m >= 0 && m < S2) legal[m] = 1;
    }
    int planes = 0;
    if (planes10) {
        // a fresh copy, as the engine encodes node states it has just cloned: the copy constructor
        // starts with empty group / tensor caches (src/games/go/go_state.cpp:140-178); the state that
        // played the moves can hold groups cached before its last captures
        alphazero::games::go::GoState fresh(st);
        auto t = fresh.getEnhancedTensorRepresentation();
        planes = (int)t.size();
        for (size_t c = 0; c < t.size() && c < 10; ++c)
            for (int r = 0; r < S; ++r)
                std::memcpy(planes10 + (c * S + r) * S, t[c][r].data(), sizeof(float) * S);
    }
    return planes;
}

// Real ChessState: `n_plies` random legal moves (LCG on `seed`) from the start position, then
// export what a device encoder takes - pieces[64] (0 empty, else type 1..6 = P N B R Q K, + 8 for
// black), meta[6] = {side to move (1 white, 2 black), castling bits (1 WK, 2 WQ, 4 BK, 8 BQ),
// en passant square or -1, halfmove clock, chess960, 0}, legal_to[2] = the 64-bit set of
// destination squares of the legal moves - and getEnhancedTensorRepresentation()
// (src/games/chess/chess_state.cpp:745-826: 20 planes) of a fresh copy into planes20[20*64].
// Returns the number of plies actually played (the game may end early), or -1 on error.
int ref_chess_random_encode(uint64_t seed, int n_plies, int8_t* pieces, int32_t* meta, uint32_t* legal_to,
                            float* planes20) {
    using namespace alphazero::games::chess;
    ChessState st;
    uint64_t x = seed * 6364136223846793005ULL + 1442695040888963407ULL;
    int played = 0;
    for (; played < n_plies; ++played) {
        if (st.isTerminal()) break;
        auto legal = st.getLegalMoves();
        if (legal.empty()) break;
        x = x * 6364136223846793005ULL + 1442695040888963407ULL;
        st.makeMove(legal[(x >> 33) % legal.size()]);
    }
    ChessState fresh(st);
    for (int sq = 0; sq < 64; ++sq) {
        const Piece p = fresh.getPiece(sq);
        pieces[sq] = p.type == PieceType::NONE ? 0 : (int8_t)((int)p.type + (p.color == PieceColor::BLACK ? 8 : 0));
    }
    const CastlingRights cr = fresh.getCastlingRights();
    meta[0] = fresh.getCurrentPlayer();
    meta[1] = (cr.white_kingside ? 1 : 0) | (cr.white_queenside ? 2 : 0) | (cr.black_kingside ? 4 : 0) | (cr.black_queenside ? 8 : 0);
    meta[2] = fresh.getEnPassantSquare();
    meta[3] = fresh.getHalfmoveClock();
    meta[4] = fresh.isChess960() ? 1 : 0;
    meta[5] = 0;
    legal_to[0] = legal_to[1] = 0;
    for (const auto& m : fresh.generateLegalMoves())
        if (m.to_square >= 0 && m.to_square < 64) legal_to[m.to_square >> 5] |= 1u << (m.to_square & 31);
    auto t = fresh.getEnhancedTensorRepresentation();
    if (t.size() != 20) return -1;
    for (size_t c = 0; c < 20; ++c)
        for (int r = 0; r < 8; ++r)
            std::memcpy(planes20 + (c * 8 + r) * 8, t[c][r].data(), sizeof(float) * 8);
    return played;
}

// MCTSNode::expand (src/mcts/mcts_node.cpp:238-436) on a Gomoku position reached by `moves`: the actions of the
// children it creates, in the node's own (shuffled) order.  Returns their number, or -1 when more than `cap`.
int ref_expand_gomoku(const int16_t* moves, int n_moves, int board_size, int use_progressive_widening, float cpw,
                      float kpw, int32_t* actions_out, int cap) {
    auto st = std::make_unique<alphazero::games::gomoku::GomokuState>(board_size, false, false, 0, false);
    for (int i = 0; i < n_moves; ++i) st->makeMove(moves[i]);
    auto node = MCTSNode::create(std::move(st), nullptr);
    node->expand(use_progressive_widening != 0, cpw, kpw);
    const std::vector<int>& acts = node->getActions();
    if ((int)acts.size() > cap) return -1;
    for (size_t i = 0; i < acts.size(); ++i) actions_out[i] = acts[i];
    return (int)acts.size();
}

// GomokuAttackDefenseModule::compute_planes (src/utils/attack_defense_module.cpp:61-111) on the GomokuState reached
// by `moves`.
int ref_attack_defense_planes(const int16_t* moves, int n_moves, int board_size, float* attack, float* defense) {
    std::vector<std::unique_ptr<alphazero::core::IGameState>> states;
    auto st = std::make_unique<alphazero::games::gomoku::GomokuState>(board_size, false, false, 0, false);
    for (int i = 0; i < n_moves; ++i) st->makeMove(moves[i]);
    states.push_back(std::move(st));
    alphazero::GomokuAttackDefenseModule module(board_size);
    auto planes = module.compute_planes(states);
    for (int r = 0; r < board_size; ++r)
        for (int c = 0; c < board_size; ++c) {
            attack[r * board_size + c] = planes.first[0][r][c];
            defense[r * board_size + c] = planes.second[0][r][c];
        }
    return 0;
}

// compute_bonuses (:50-59, :113-203) for every empty cell of a board, called the way the module's own tests call
// it: the board handed over already holds the player's stone on the chosen cell.
int ref_attack_defense_bonuses(const int8_t* board, int board_size, int player, float* attack, float* defense) {
    alphazero::GomokuAttackDefenseModule module(board_size);
    std::vector<std::vector<std::vector<int>>> batch(1, std::vector<std::vector<int>>(board_size, std::vector<int>(board_size, 0)));
    for (int r = 0; r < board_size; ++r)
        for (int c = 0; c < board_size; ++c) batch[0][r][c] = board[r * board_size + c];
    for (int m = 0; m < board_size * board_size; ++m) {
        attack[m] = defense[m] = 0.0f;
        const int r = m / board_size, c = m % board_size;
        if (batch[0][r][c] != 0) continue;
        batch[0][r][c] = player;
        auto [a, d] = module.compute_bonuses(batch, std::vector<int>{m}, std::vector<int>{player});
        batch[0][r][c] = 0;
        attack[m] = a[0];
        defense[m] = d[0];
    }
    return 0;
}

// GomokuState::getLegalMoves (through is_move_valid_internal, src/games/gomoku/gomoku_state.cpp:915-943) on a state
// constructed with the variant flags, after `moves`.  legal_out: one byte per cell.  -1 when a move was not legal.
int ref_gomoku_legal_moves(const int16_t* moves, int n_moves, int board_size, int use_renju, int use_omok, uint8_t* legal_out) {
    alphazero::games::gomoku::GomokuState st(board_size, use_renju != 0, use_omok != 0, 0, false);
    for (int i = 0; i < n_moves; ++i) {
        if (!st.isLegalMove(moves[i])) return -1;
        st.makeMove(moves[i]);
    }
    std::memset(legal_out, 0, (size_t)board_size * board_size);
    for (int a : st.getLegalMoves()) legal_out[a] = 1;
    return 0;
}

}  // extern "C"
