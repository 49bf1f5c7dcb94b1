// TEST INFRASTRUCTURE — not part of the product.
//
// Proves the drop-in boundary with the reference's own types: real
// alphazero::games::gomoku::GomokuState objects (compiled from the reference's
// sources) are handed, as std::vector<std::unique_ptr<core::IGameState>>, to
// omoknuni_b200::B200Network::inference — the call the reference's
// SharedInferenceQueue / MCTSEngine make on a NeuralNetwork
// (src/mcts/shared_inference_queue.cpp:355, mcts_engine_main.cpp:163-165).
//
//   adapter_check <weights.bin> <games.bin> <out.bin> <input_channels> <blocks> <policy_ch> <value_ch>
// games.bin: int32 n_games, then per game int32 n_moves + moves.  A game with
// n_moves = -1 stands for a null state.  out.bin: float policy[n][225], value[n].
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <vector>

#include "games/gomoku/gomoku_state.h"
#include "../omoknuni_small_b200/adapter/b200_network.h"

int main(int argc, char** argv) {
    if (argc < 8) { std::fprintf(stderr, "usage: adapter_check weights games out cin blocks pc vc\n"); return 2; }
    const int cin = std::atoi(argv[4]), blocks = std::atoi(argv[5]), pc = std::atoi(argv[6]), vc = std::atoi(argv[7]);
    std::FILE* g = std::fopen(argv[2], "rb");
    if (!g) return 3;
    int32_t n = 0;
    if (std::fread(&n, 4, 1, g) != 1) return 3;
    std::vector<std::unique_ptr<alphazero::core::IGameState>> states;
    for (int i = 0; i < n; ++i) {
        int32_t k = 0;
        if (std::fread(&k, 4, 1, g) != 1) return 3;
        if (k < 0) { states.emplace_back(nullptr); continue; }
        auto st = std::make_unique<alphazero::games::gomoku::GomokuState>(15, false, false, 0, false);
        for (int j = 0; j < k; ++j) {
            int32_t mv = 0;
            if (std::fread(&mv, 4, 1, g) != 1) return 3;
            st->makeMove(mv);
        }
        states.push_back(std::move(st));
    }
    std::fclose(g);

    // through the base-class pointer, as the reference's callers hold it
    std::shared_ptr<alphazero::nn::NeuralNetwork> net =
        std::make_shared<omoknuni_b200::B200Network>(cin, 15, blocks, 64, 225, pc, vc, /*max_batch=*/64, /*device=*/0);
    net->load(argv[1]);
    const auto out = net->inference(states);     // more states than max_batch: the adapter slices
    if ((int)out.size() != n || net->getPolicySize() != 225 || net->getInputShape()[0] != cin) return 4;

    std::FILE* o = std::fopen(argv[3], "wb");
    if (!o) return 5;
    for (const auto& r : out) std::fwrite(r.policy.data(), sizeof(float), r.policy.size(), o);
    for (const auto& r : out) std::fwrite(&r.value, sizeof(float), 1, o);
    std::fclose(o);
    std::printf("adapter_check: %d states evaluated\n", n);
    return 0;
}
