// TEST INFRASTRUCTURE — not part of the product.
//
// Proves the drop-in boundary with the reference's own types and code, compiled from the
// reference's sources where they lie (see oracle/Makefile).  Four checks:
//
//   adapter_check direct <weights> <games> <out> <cin> <blocks> <pc> <vc> [f16]
//       real alphazero::games::gomoku::GomokuState objects handed, as
//       std::vector<std::unique_ptr<core::IGameState>>, to omoknuni_b200::B200Network::inference
//       through a NeuralNetwork pointer — the call the reference's SharedInferenceQueue /
//       MCTSEngine make (src/mcts/shared_inference_queue.cpp:355, mcts_engine_main.cpp:163-165).
//   adapter_check queue <weights> <games> <out> <cin> <blocks> <pc> <vc> <producers>
//       the reference's own batch collector, alphazero::mcts::SharedInferenceQueue
//       (src/mcts/shared_inference_queue.cpp, compiled unchanged), with B200Network behind it:
//       several producer threads call submitBatch (include/mcts/shared_inference_queue.h:43-45)
//       with requests of different sizes; every request's results must equal direct inference on
//       the same states; a network that is not ready must come back as the reference's default
//       outputs (uniform policy, value 0: src/nn/resnet_model.cpp:610-623) and a network that
//       throws must arrive as an exception at future.get() (shared_inference_queue.cpp:401-408).
//   adapter_check tree <seed>
//       omoknuni_b200::B200Tree against real alphazero::mcts::MCTSNode families: selectChild +
//       applyVirtualLoss, revertVirtualLoss, the update / revertVirtualLoss backup loop,
//       setPriorProbabilities after expand on a real GomokuState.
//   adapter_check engine <weights> <cin> <blocks> <pc> <vc>
//       omoknuni_b200::B200GomokuSearch: settings in as the reference's MCTSSettings, results out
//       as its SearchResult / MCTSStats; the assertions of the reference's own engine tests
//       (tests/mcts/mcts_engine_test.cpp:143-157, tests/integration/mcts_with_nn_test.cpp:79-93).
//
// games file: int32 n_games, then per game int32 n_moves + moves (n_moves = -1: a null state).
// out file: float policy[n][225], value[n].
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <future>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "games/gomoku/gomoku_state.h"
#include "mcts/shared_inference_queue.h"
#include "ref_tiny_state.h"
#include "../omoknuni_small_b200/adapter/b200_network.h"
#include "../omoknuni_small_b200/adapter/b200_search.h"
#include "../omoknuni_small_b200/adapter/b200_tree.h"

using alphazero::core::IGameState;
using alphazero::games::gomoku::GomokuState;
using alphazero::mcts::NetworkOutput;
using States = std::vector<std::unique_ptr<IGameState>>;

namespace {

bool read_games(const char* path, std::vector<std::vector<int>>* games) {
    std::FILE* g = std::fopen(path, "rb");
    if (!g) return false;
    int32_t n = 0;
    if (std::fread(&n, 4, 1, g) != 1) return false;
    for (int i = 0; i < n; ++i) {
        int32_t k = 0;
        if (std::fread(&k, 4, 1, g) != 1) return false;
        std::vector<int> mv;
        if (k < 0) { mv.push_back(-1); games->push_back(mv); continue; }     // marker of a null state
        for (int j = 0; j < k; ++j) {
            int32_t m = 0;
            if (std::fread(&m, 4, 1, g) != 1) return false;
            mv.push_back(m);
        }
        games->push_back(mv);
    }
    std::fclose(g);
    return true;
}

std::unique_ptr<IGameState> make_state(const std::vector<int>& mv) {
    if (mv.size() == 1 && mv[0] == -1) return nullptr;
    auto st = std::make_unique<GomokuState>(15, false, false, 0, false);
    for (int m : mv) st->makeMove(m);
    return st;
}

bool write_out(const char* path, const std::vector<NetworkOutput>& out) {
    std::FILE* o = std::fopen(path, "wb");
    if (!o) return false;
    for (const auto& r : out) std::fwrite(r.policy.data(), sizeof(float), r.policy.size(), o);
    for (const auto& r : out) std::fwrite(&r.value, sizeof(float), 1, o);
    std::fclose(o);
    return true;
}

bool same(const NetworkOutput& a, const NetworkOutput& b) {
    return a.policy.size() == b.policy.size() && a.value == b.value &&
           std::memcmp(a.policy.data(), b.policy.data(), a.policy.size() * sizeof(float)) == 0;
}

#define REQUIRE(cond, ...)                                                  \
    do {                                                                    \
        if (!(cond)) { std::fprintf(stderr, "adapter_check: " __VA_ARGS__); std::fprintf(stderr, "\n"); return 10; } \
    } while (0)

int run_direct(int argc, char** argv) {
    if (argc < 9) return 2;
    const int cin = std::atoi(argv[5]), blocks = std::atoi(argv[6]), pc = std::atoi(argv[7]), vc = std::atoi(argv[8]);
    const int dtype = (argc > 9 && std::string(argv[9]) == "f16") ? OB200_DTYPE_F16 : OB200_DTYPE_BF16;
    std::vector<std::vector<int>> games;
    if (!read_games(argv[3], &games)) return 3;
    States states;
    for (const auto& g : games) states.push_back(make_state(g));
    // through the base-class pointer, as the reference's callers hold it
    std::shared_ptr<alphazero::nn::NeuralNetwork> net = std::make_shared<omoknuni_b200::B200Network>(
        cin, 15, blocks, 64, 225, pc, vc, /*max_batch=*/64, /*device=*/0, /*keep_weights=*/false, dtype);
    net->load(argv[2]);
    const auto out = net->inference(states);     // more states than max_batch: the adapter slices
    REQUIRE(out.size() == states.size() && net->getPolicySize() == 225 && net->getInputShape()[0] == cin, "shapes");
    // the same network as the std::function the engine's other constructor takes (include/mcts/mcts_engine.h:230-231)
    {
        const auto fn = omoknuni_b200::makeInferenceFunction(std::static_pointer_cast<omoknuni_b200::B200Network>(net));
        const auto again = fn(states);
        REQUIRE(again.size() == out.size(), "inference function: size");
        REQUIRE(net->supportsEvaluateBatch() && net->isDeterministic() && net->getGPUOptimizationStatus().model_is_deterministic,
                "optional interface");
        const auto one = net->evaluate(*states[0]);
        REQUIRE(one.value == out[0].value && one.policy == out[0].policy, "evaluate(state) differs from inference()");
        for (size_t i = 0; i < out.size(); ++i)
            REQUIRE(again[i].value == out[i].value && again[i].policy == out[i].policy, "inference function: state %zu differs", i);
    }
    // several engine threads calling inference() on the same network at once, as the reference's engines do when no
    // global queue is set up (src/mcts/mcts_engine_batch_tree_simple.cpp:231-233): every thread's results equal the
    // single-threaded ones
    {
        const int n_threads = 4, rounds = 6;
        std::atomic<int> mismatches{0};
        std::vector<std::thread> threads;
        for (int th = 0; th < n_threads; ++th)
            threads.emplace_back([&, th] {
                for (int r = 0; r < rounds; ++r) {
                    // a different slice of the states per thread and round, sizes on both sides of max_batch
                    const size_t first = (size_t)((th * 7 + r * 13) % (int)games.size());
                    const size_t count = std::min(games.size() - first, (size_t)(1 + (th * 31 + r * 17) % 100));
                    States mine;
                    for (size_t i = 0; i < count; ++i) mine.push_back(make_state(games[first + i]));
                    const auto got = net->inference(mine);
                    if (got.size() != count) { mismatches++; continue; }
                    for (size_t i = 0; i < count; ++i)
                        if (got[i].value != out[first + i].value || got[i].policy != out[first + i].policy) mismatches++;
                }
            });
        for (auto& t : threads) t.join();
        REQUIRE(mismatches.load() == 0, "%d results of concurrent inference() calls differ from the single-threaded ones", mismatches.load());
    }
    if (!write_out(argv[4], out)) return 5;
    std::printf("adapter_check direct: %zu states evaluated; 4 threads x 6 concurrent calls equal\n", out.size());
    return 0;
}

// A network whose inference throws: what the collector must turn into an exception at future.get().
class ThrowingNetwork : public alphazero::nn::NeuralNetwork {
public:
    std::vector<NetworkOutput> inference(const States&) override { throw std::runtime_error("injected failure"); }
    void save(const std::string&) override {}
    void load(const std::string&) override {}
    std::vector<int64_t> getInputShape() const override { return {17, 15, 15}; }
    int64_t getPolicySize() const override { return 225; }
};

int run_queue(int argc, char** argv) {
    if (argc < 10) return 2;
    const int cin = std::atoi(argv[5]), blocks = std::atoi(argv[6]), pc = std::atoi(argv[7]), vc = std::atoi(argv[8]);
    const int producers = std::atoi(argv[9]);
    std::vector<std::vector<int>> games;
    if (!read_games(argv[3], &games)) return 3;
    auto b200 = std::make_shared<omoknuni_b200::B200Network>(cin, 15, blocks, 64, 225, pc, vc, /*max_batch=*/64, 0);
    b200->load(argv[2]);
    REQUIRE(b200->ok() && b200->handle(), "the network did not load");
    std::shared_ptr<alphazero::nn::NeuralNetwork> net = b200;

    // direct inference on every game: the expected values
    States all;
    for (const auto& g : games) all.push_back(make_state(g));
    const auto want = net->inference(all);

    // requests of 1..9 states, dealt round-robin to the producer threads
    struct Request { size_t first, count; };
    std::vector<Request> reqs;
    for (size_t at = 0, k = 0; at < games.size(); ++k) {
        const size_t c = std::min(games.size() - at, (size_t)(1 + (k * 5) % 9));
        reqs.push_back({at, c});
        at += c;
    }
    ob200_counters c0{}, c1{};
    ob200_get_counters(&c0);
    std::vector<NetworkOutput> got(games.size());
    std::atomic<int> failures{0};
    {
        alphazero::mcts::SharedInferenceQueue queue(net, /*max_batch_size=*/48, /*batch_timeout_ms=*/5);
        queue.start();
        std::vector<std::thread> threads;
        for (int p = 0; p < producers; ++p)
            threads.emplace_back([&, p] {
                for (size_t r = p; r < reqs.size(); r += producers) {
                    States states;
                    for (size_t i = 0; i < reqs[r].count; ++i) states.push_back(make_state(games[reqs[r].first + i]));
                    try {
                        auto fut = queue.submitBatch(std::move(states));     // ownership moves in, as in the engine
                        auto res = fut.get();
                        if (res.size() != reqs[r].count) { ++failures; continue; }
                        for (size_t i = 0; i < res.size(); ++i) got[reqs[r].first + i] = std::move(res[i]);
                    } catch (...) { ++failures; }
                }
            });
        for (auto& t : threads) t.join();
        const auto& st = queue.getStats();
        std::printf("adapter_check queue: %llu requests, %llu states, %llu batches, average batch %.1f\n",
                    (unsigned long long)st.total_requests.load(), (unsigned long long)st.total_states.load(),
                    (unsigned long long)st.total_batches.load(), st.average_batch_size.load());
        REQUIRE(st.total_requests.load() == reqs.size() && st.total_states.load() == games.size(), "queue statistics");
        REQUIRE(st.total_batches.load() <= reqs.size(), "batches");
        queue.stop();
    }
    ob200_get_counters(&c1);
    REQUIRE(failures.load() == 0, "%d requests failed", failures.load());
    for (size_t i = 0; i < games.size(); ++i) REQUIRE(same(got[i], want[i]), "state %zu differs between the queue and direct inference", i);
    REQUIRE(c1.evals - c0.evals == games.size(), "the library evaluated %llu states for %zu submitted",
            (unsigned long long)(c1.evals - c0.evals), games.size());

    // a network that is not ready behind the same collector: default outputs, no exception
    {
        std::shared_ptr<alphazero::nn::NeuralNetwork> raw =
            std::make_shared<omoknuni_b200::B200Network>(cin, 15, blocks, 64, 225, pc, vc, 64, 0);   // never finalised
        alphazero::mcts::SharedInferenceQueue queue(raw, 16, 5);
        queue.start();
        States states;
        for (int i = 0; i < 3; ++i) states.push_back(make_state(games[i]));
        auto res = queue.submitBatch(std::move(states)).get();
        REQUIRE(res.size() == 3, "default outputs: size");
        for (const auto& r : res) {
            REQUIRE(r.value == 0.0f && r.policy.size() == 225, "default outputs: value / size");
            for (float p : r.policy) REQUIRE(std::fabs(p - 1.0f / 225.0f) < 1e-7f, "default outputs: not uniform");
        }
        queue.stop();
    }
    // a configuration the library refuses (no such tower width): the adapter holds no handle, still no throw
    {
        omoknuni_b200::B200Network bad(cin, 15, blocks, /*num_filters=*/65, 225, pc, vc, 64, 0);
        REQUIRE(!bad.ok(), "a 65-filter tower must be refused");
        States states;
        states.push_back(make_state(games[0]));
        const auto res = bad.inference(states);
        REQUIRE(res.size() == 1 && res[0].value == 0.0f && std::fabs(res[0].policy[7] - 1.0f / 225.0f) < 1e-7f, "refused configuration: defaults");
    }
    // a network that throws: the collector hands the exception to every request of the batch
    {
        std::shared_ptr<alphazero::nn::NeuralNetwork> thrower = std::make_shared<ThrowingNetwork>();
        alphazero::mcts::SharedInferenceQueue queue(thrower, 16, 5);
        queue.start();
        States states;
        states.push_back(make_state(games[0]));
        auto fut = queue.submitBatch(std::move(states));
        bool threw = false;
        try { fut.get(); } catch (const std::exception&) { threw = true; }
        REQUIRE(threw, "an exception inside inference must reach future.get()");
        queue.stop();
    }
    if (!write_out(argv[4], got)) return 5;
    std::printf("adapter_check queue: %zu states through SharedInferenceQueue::submitBatch from %d threads, equal to direct inference\n",
                games.size(), producers);
    return 0;
}

int run_tree(int argc, char** argv) {
    using alphazero::mcts::MCTSNode;
    const unsigned seed = argc > 2 ? (unsigned)std::atoi(argv[2]) : 1u;
    std::mt19937 rng(seed);
    const int P = 300, C = 225, vl = 3;
    const float c_puct = 1.5f;
    omoknuni_b200::B200Tree tree(P + 64, C);
    REQUIRE(tree.ok(), "tree handle");
    std::vector<ref_tiny::Family> fam(P);
    std::vector<std::vector<int>> slot_of(P);            // child index -> slot (children exist on a random subset of slots)
    std::vector<int> nodes(P);
    std::uniform_real_distribution<float> U(-1.0f, 1.0f);
    for (int p = 0; p < P; ++p) {
        std::vector<int> slots;
        const int want = 1 + (int)(rng() % C);
        for (int s = 0; s < C; ++s) if ((int)(rng() % C) < want) slots.push_back(s);
        if (slots.empty()) slots.push_back((int)(rng() % C));
        if (p == 0) slots.clear();                        // a node without children
        const int n = (int)slots.size();
        std::vector<int32_t> N(n), VL(n);
        std::vector<float> W(n), Pr(n);
        int parent_visits = 0;
        for (int i = 0; i < n; ++i) {
            N[i] = (int)(rng() % 12); VL[i] = (int)(rng() % 4);
            W[i] = (float)N[i] * U(rng); Pr[i] = std::fabs(U(rng));
            parent_visits += N[i];
        }
        fam[p] = ref_tiny::make_family(n, N.data(), W.data(), Pr.data(), VL.data(), parent_visits);
        slot_of[p] = slots;
        nodes[p] = tree.addNode(slots);
        REQUIRE(nodes[p] == p, "node ids are dense");
        omoknuni_b200::B200Tree::ChildStats st;
        st.visits.assign(C, 0); st.virtual_loss.assign(C, 0); st.value_sum.assign(C, 0.0f); st.prior.assign(C, 0.0f);
        for (int i = 0; i < n; ++i) { st.visits[slots[i]] = N[i]; st.virtual_loss[slots[i]] = VL[i]; st.value_sum[slots[i]] = W[i]; st.prior[slots[i]] = Pr[i]; }
        REQUIRE(tree.loadChildStats(p, st, parent_visits), "load statistics");
    }
    // ---- selectChild + applyVirtualLoss ----
    const std::vector<int> sel = tree.selectChildBatch(nodes, c_puct, vl);
    std::vector<int> sel_slots(P, -1);
    std::vector<std::shared_ptr<MCTSNode>> best(P);
    for (int p = 0; p < P; ++p) {
        best[p] = fam[p].parent->selectChild(c_puct, false, 3000.0f);
        const int idx = ref_tiny::index_of(fam[p], best[p]);
        sel_slots[p] = idx < 0 ? -1 : slot_of[p][idx];
        REQUIRE(sel[p] == sel_slots[p], "parent %d: selectChild gives slot %d, the device %d", p, sel_slots[p], sel[p]);
        if (best[p]) best[p]->applyVirtualLoss(vl);
    }
    auto compare_vl = [&](const char* when) -> int {
        for (int p = 0; p < P; ++p) {
            omoknuni_b200::B200Tree::ChildStats st;
            REQUIRE(tree.childStats(p, &st), "read statistics");
            auto& kids = fam[p].parent->getChildren();
            for (size_t i = 0; i < kids.size(); ++i)
                REQUIRE(kids[i]->getVirtualLoss() == st.virtual_loss[slot_of[p][i]], "%s: parent %d child %zu virtual loss %d vs %d", when, p, i,
                        kids[i]->getVirtualLoss(), st.virtual_loss[slot_of[p][i]]);
        }
        return 0;
    };
    if (int rc = compare_vl("after applyVirtualLoss")) return rc;
    // ---- revertVirtualLoss, twice: the second one runs into the clamp at zero for small counters ----
    for (int round = 0; round < 2; ++round) {
        REQUIRE(tree.revertVirtualLoss(nodes, sel, vl), "revert");
        for (int p = 0; p < P; ++p) if (best[p]) best[p]->revertVirtualLoss(vl);
        if (int rc = compare_vl("after revertVirtualLoss")) return rc;
    }
    // ---- backup: update(v); revertVirtualLoss(vl); v = -v from the leaf up, on chains of real nodes ----
    {
        const int depth = 6, n_paths = 40;
        std::vector<std::vector<std::pair<int, int>>> paths(n_paths);
        std::vector<float> leaf(n_paths);
        std::vector<std::vector<std::shared_ptr<MCTSNode>>> chain(n_paths);
        for (int i = 0; i < n_paths; ++i) {
            leaf[i] = (float)((int)(rng() % 513) - 256) / 256.0f;
            for (int d = 0; d < depth; ++d) {
                const int p = 1 + (int)(rng() % (P - 1));
                const int idx = (int)(rng() % slot_of[p].size());
                paths[i].push_back({p, slot_of[p][idx]});
                chain[i].push_back(fam[p].parent->getChildren()[idx]);
            }
        }
        // virtual loss as a descent would have left it
        for (int i = 0; i < n_paths; ++i)
            for (int d = 0; d < depth; ++d) {
                chain[i][d]->applyVirtualLoss(vl);
                REQUIRE(tree.applyVirtualLoss({paths[i][d].first}, {paths[i][d].second}, vl), "apply");
            }
        REQUIRE(tree.backup(paths, leaf, vl), "backup");
        for (int i = 0; i < n_paths; ++i) {
            float v = leaf[i];
            for (int d = depth - 1; d >= 0; --d) { chain[i][d]->update(v); chain[i][d]->revertVirtualLoss(vl); v = -v; }
        }
        for (int p = 0; p < P; ++p) {
            omoknuni_b200::B200Tree::ChildStats st;
            REQUIRE(tree.childStats(p, &st), "read statistics");
            auto& kids = fam[p].parent->getChildren();
            for (size_t i = 0; i < kids.size(); ++i) {
                const int s = slot_of[p][i];
                REQUIRE(kids[i]->getVisitCount() == st.visits[s] && kids[i]->getVirtualLoss() == st.virtual_loss[s],
                        "backup: parent %d child %zu visits %d / %d, virtual loss %d / %d", p, i, kids[i]->getVisitCount(), st.visits[s],
                        kids[i]->getVirtualLoss(), st.virtual_loss[s]);
                // value sums: leaf values are multiples of 1/256 and the loaded sums take part in few additions; compare the means
                const float mean = st.visits[s] ? st.value_sum[s] / (float)st.visits[s] : 0.0f;
                REQUIRE(std::fabs(kids[i]->getValue() - mean) <= 1e-5f, "backup: parent %d child %zu value %g vs %g", p, i, kids[i]->getValue(), mean);
            }
        }
    }
    // ---- expand + setPriorProbabilities on a real Gomoku position ----
    {
        auto st = std::make_unique<GomokuState>(15, false, false, 0, false);
        for (int m : {112, 113, 97, 127, 98}) st->makeMove(m);
        const std::vector<int> legal = st->getLegalMoves();
        auto node = MCTSNode::create(st->clone());
        node->expand(false, 2.0f, 0.5f);                            // children in shuffled order; getAction() names them
        std::vector<float> policy(225);
        for (auto& x : policy) x = U(rng) * 1.3f;                    // values below 0 and above 1: the clamp matters
        node->setPriorProbabilities(policy);
        const int id = tree.addNode(legal);
        REQUIRE(id >= 0 && tree.setPriorProbabilities(id, policy), "set priors");
        omoknuni_b200::B200Tree::ChildStats cs;
        REQUIRE(tree.childStats(id, &cs), "read priors");
        REQUIRE(node->getChildren().size() == legal.size(), "expand creates one child per legal move");
        std::vector<char> seen(225, 0);
        for (auto& child : node->getChildren()) {
            const int a = child->getAction();
            seen[a] = 1;
            REQUIRE(child->getPriorProbability() == cs.prior[a], "prior of move %d: %g vs %g", a, child->getPriorProbability(), cs.prior[a]);
        }
        for (int a = 0; a < 225; ++a) if (!seen[a]) REQUIRE(cs.prior[a] == 0.0f, "occupied cell %d has a prior", a);
    }
    std::printf("adapter_check tree: %d parents; selection, virtual loss, backup and priors equal to MCTSNode\n", P);
    return 0;
}

int run_engine(int argc, char** argv) {
    if (argc < 7) return 2;
    const int cin = std::atoi(argv[3]), blocks = std::atoi(argv[4]), pc = std::atoi(argv[5]), vc = std::atoi(argv[6]);
    auto net = std::make_shared<omoknuni_b200::B200Network>(cin, 15, blocks, 64, 225, pc, vc, /*max_batch=*/128, 0);
    net->load(argv[2]);
    REQUIRE(net->handle(), "the network did not load");
    alphazero::mcts::MCTSSettings settings;
    settings.num_simulations = 96;
    settings.batch_size = 64;
    settings.exploration_constant = 1.5f;
    settings.virtual_loss = 3;
    settings.add_dirichlet_noise = true;
    settings.temperature = 1.0f;
    settings.use_transposition_table = true;
    const int G = 4;
    omoknuni_b200::B200GomokuSearch engine(net, settings, G, /*seed=*/5);
    REQUIRE(engine.ok(), "search handle");
    std::vector<std::unique_ptr<GomokuState>> games;
    for (int g = 0; g < G; ++g) {
        games.push_back(std::make_unique<GomokuState>(15, false, false, 0, false));
        for (int k = 0; k < g; ++k) games.back()->makeMove(112 + k);
    }
    // a few moves of play, as tests/integration/mcts_with_nn_test.cpp:95-130 does with the reference engine
    for (int move = 0; move < 3; ++move) {
        std::vector<const IGameState*> view;
        for (auto& s : games) view.push_back(s.get());
        const auto results = engine.search(view);
        REQUIRE((int)results.size() == G, "one result per game");
        for (int g = 0; g < G; ++g) {
            const alphazero::mcts::SearchResult& r = results[g];
            REQUIRE(r.action >= 0 && games[g]->isLegalMove(r.action), "game %d: action %d is not legal", g, r.action);
            REQUIRE(r.probabilities.size() == 225, "probabilities over the whole action space");
            double sum = 0;
            for (float p : r.probabilities) { REQUIRE(p >= 0.0f, "negative probability"); sum += p; }
            REQUIRE(std::fabs(sum - 1.0) < 1e-4, "probabilities sum to %g", sum);
            // MCTSSettings' defaults switch progressive widening on with c = 2: a node gets max(8, 2) = 8 children
            int moves_tried = 0;
            for (float p : r.probabilities) moves_tried += p > 0.0f;
            REQUIRE(settings.use_progressive_widening && moves_tried >= 1 && moves_tried <= 8, "game %d: %d root moves visited under widening", g, moves_tried);
            REQUIRE(r.stats.total_nodes > 1 && r.stats.total_evaluations > 0, "stats: nodes %zu evaluations %zu", r.stats.total_nodes, r.stats.total_evaluations);
            REQUIRE(r.stats.avg_batch_size > 1.0f && r.stats.total_batches_processed > 0, "stats: batches");
            REQUIRE(r.stats.nodes_per_second > 0.0f, "stats: rate");
            games[g]->makeMove(r.action);
        }
    }
    alphazero::mcts::MCTSStats totals;
    omoknuni_b200::B200Tree::fillStats(totals);
    REQUIRE(totals.total_evaluations > 0 && totals.total_batches_processed > 0 && totals.avg_batch_size > 1.0f, "process-wide stats");
    std::printf("adapter_check engine: %d games x 3 moves through MCTSSettings -> SearchResult; evaluations %zu, batches %zu, average batch %.1f\n",
                G, totals.total_evaluations, totals.total_batches_processed, totals.avg_batch_size);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: adapter_check direct|queue|tree|engine ...\n"); return 2; }
    const std::string mode = argv[1];
    if (mode == "direct") return run_direct(argc, argv);
    if (mode == "queue") return run_queue(argc, argv);
    if (mode == "tree") return run_tree(argc, argv);
    if (mode == "engine") return run_engine(argc, argv);
    std::fprintf(stderr, "adapter_check: unknown mode %s\n", mode.c_str());
    return 2;
}
