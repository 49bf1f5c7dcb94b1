// MCTSEngine::search for a group of Gomoku games at once, on the device-resident search of
// include/omoknuni_b200.h, behind the reference's own types: settings come in as
// alphazero::mcts::MCTSSettings (reference include/mcts/mcts_engine.h:55-152), results go out as
// alphazero::mcts::SearchResult with its MCTSStats filled (:154-211) - what
// SelfPlayManager::generateGame reads after engine.search(state)
// (src/selfplay/self_play_manager.cpp:711-760): action, probabilities over the whole action space,
// value, stats.total_nodes / search_time / avg_batch_size / total_evaluations /
// total_batches_processed / nodes_per_second.
// Header-only; compile inside the reference project (needs its headers) and link
// libomoknuni_b200.so.
#pragma once

#include <chrono>
#include <cstdio>
#include <memory>
#include <random>
#include <vector>

#include "mcts/mcts_engine.h"    // reference header: MCTSSettings, MCTSStats, SearchResult
#include "b200_network.h"

namespace omoknuni_b200 {

class B200GomokuSearch {
public:
    // n_games: games searched together (the reference runs one engine per game thread,
    // src/selfplay/self_play_manager.cpp:366-376).  settings.batch_size is the leaf batch of one
    // network call (rounded up to a multiple of n_games).
    B200GomokuSearch(std::shared_ptr<B200Network> net, const alphazero::mcts::MCTSSettings& settings, int n_games,
                     uint64_t seed = 0, int rules = OB200_RULES_FREESTYLE)
        : net_(std::move(net)), settings_(settings), n_games_(n_games), rng_(seed) {
        ob200_search_config c{};
        c.n_trees = n_games;
        c.sims_per_move = settings.num_simulations;
        const int per_tree = std::max(1, settings.batch_size / std::max(1, n_games));
        c.leaf_batch = per_tree * n_games;
        c.max_depth = std::min(64, std::max(1, settings.tensor_max_depth));
        c.c_puct = settings.exploration_constant;
        c.virtual_loss = settings.virtual_loss;
        c.dirichlet_alpha = settings.dirichlet_alpha;
        c.dirichlet_epsilon = settings.add_dirichlet_noise ? settings.dirichlet_epsilon : 0.0f;
        c.value_sign = 1;                                    // the reference's batched loop
        c.use_transposition_table = settings.use_transposition_table ? 1 : 0;
        c.seed = seed;
        c.max_children = 0;                                  // MCTSNode::expand's own cap of 1,000
        c.use_progressive_widening = settings.use_progressive_widening ? 1 : 0;
        c.progressive_widening_c = settings.progressive_widening_c;
        c.progressive_widening_k = settings.progressive_widening_k;
        c.rules = rules;                                     // the variant the GomokuStates were constructed with
        cfg_ = c;
        if (!net_ || !net_->handle() || ob200_search_create(net_->handle(), &c, &search_) != OB200_OK) {
            std::fprintf(stderr, "[B200GomokuSearch] %s\n", ob200_last_error());
            search_ = nullptr;
        }
    }
    ~B200GomokuSearch() { ob200_search_destroy(search_); }
    B200GomokuSearch(const B200GomokuSearch&) = delete;
    B200GomokuSearch& operator=(const B200GomokuSearch&) = delete;
    bool ok() const { return search_ != nullptr; }

    // One move for every game.  states[g]: the game's current state (unfinished); only its move history is
    // read.  On failure every result has action -1 and empty probabilities, as MCTSEngine::search returns
    // when it cannot search (src/mcts/mcts_engine_main.cpp:256-330).
    std::vector<alphazero::mcts::SearchResult> search(const std::vector<const alphazero::core::IGameState*>& states) {
        std::vector<alphazero::mcts::SearchResult> out(states.size());
        if (!search_ || (int)states.size() != n_games_) return out;
        size_t stride = 1;
        std::vector<std::vector<int>> hist(states.size());
        for (size_t g = 0; g < states.size(); ++g) {
            if (!states[g]) return out;
            hist[g] = states[g]->getMoveHistory();
            stride = std::max(stride, hist[g].size());
        }
        std::vector<int16_t> moves(states.size() * stride, (int16_t)-1);
        std::vector<int32_t> n_moves(states.size());
        for (size_t g = 0; g < states.size(); ++g) {
            n_moves[g] = (int32_t)hist[g].size();
            for (size_t i = 0; i < hist[g].size(); ++i) moves[g * stride + i] = (int16_t)hist[g][i];
        }
        const int A = 225;
        std::vector<float> pi(states.size() * A);
        std::vector<int32_t> visits(states.size() * A);
        ob200_search_stats st{};
        ob200_counters before{}, after{};
        ob200_get_counters(&before);
        if (ob200_search_run(search_, moves.data(), n_moves.data(), (int32_t)stride, settings_.temperature, pi.data(),
                             visits.data(), &st) != OB200_OK) {
            std::fprintf(stderr, "[B200GomokuSearch] %s\n", ob200_last_error());
            return out;
        }
        ob200_get_counters(&after);
        const uint64_t batches = after.batches - before.batches, evals = after.evals - before.evals;
        for (size_t g = 0; g < states.size(); ++g) {
            auto& r = out[g];
            r.probabilities.assign(pi.begin() + g * A, pi.begin() + (g + 1) * A);
            // the move: argmax for temperature ~ 0, else sampled from the visit distribution
            // (src/mcts/mcts_engine_main.cpp:380-405)
            int best = 0;
            for (int a = 1; a < A; ++a) if (r.probabilities[a] > r.probabilities[best]) best = a;
            if (settings_.temperature >= 0.01f) {
                std::discrete_distribution<int> d(r.probabilities.begin(), r.probabilities.end());
                best = d(rng_);
            }
            r.action = best;
            r.value = 0.0f;                                   // root value: not tracked per game by the device search
            auto& s = r.stats;
            s.total_nodes = (size_t)(st.nodes / (int64_t)states.size());
            s.search_time = std::chrono::milliseconds((long long)(st.wall_ms + 0.5));
            s.total_evaluations = (size_t)evals;
            s.total_batches_processed = (size_t)batches;
            s.avg_batch_size = batches ? (float)((double)evals / (double)batches) : 0.0f;
            s.avg_batch_latency = std::chrono::milliseconds(batches ? (long long)(st.device_ms / (double)batches + 0.5) : 0);
            s.nodes_per_second = st.wall_ms > 0 ? (float)(st.simulations / (double)states.size() / (st.wall_ms * 1e-3)) : 0.0f;
            s.total_requests_processed = (size_t)st.simulations;
            s.tt_size = settings_.use_transposition_table ? (size_t)st.nodes : 0;
        }
        return out;
    }

    const ob200_search_config& config() const { return cfg_; }

private:
    std::shared_ptr<B200Network> net_;
    alphazero::mcts::MCTSSettings settings_;
    int n_games_ = 0;
    ob200_search_config cfg_{};
    ob200_search* search_ = nullptr;
    std::mt19937_64 rng_;
};

}  // namespace omoknuni_b200
