// Drop-in for the reference project's network class: implements
// alphazero::nn::NeuralNetwork (reference include/nn/neural_network.h:20-147)
// on top of the C ABI in include/omoknuni_b200.h.  Header-only; compile it
// inside the reference project (it needs the reference's own headers) and link
// libomoknuni_b200.so.  No libtorch.
//
// Behaviour kept from alphazero::nn::ResNetModel (reference
// src/nn/resnet_model.cpp):
//   * constructor arguments in the same order (:51-53), plus the two head
//     widths the reference hard-codes as 32 (:81,:90);
//   * inference() returns one NetworkOutput per state, policy = softmax
//     probabilities over the whole action space, value in [-1, 1] (:752-763);
//   * a null state contributes all-zero planes (:412-416);
//   * any failure returns a uniform policy and value 0 for every state
//     (:610-623, :801-810) — inference() never throws;
//   * getInputShape() = {channels, board, board}, getPolicySize() (:866-873).
// Weights enter by the reference's parameter names (setTensor) or from a flat
// file written by save().  save() needs the fp32 tensors as they were given: a
// network that will be saved is constructed with keep_weights = true (a second
// host copy of every tensor for the object's lifetime); without it the copies
// are dropped when finalize() has uploaded the weights and save() writes nothing.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "nn/neural_network.h"   // reference header
#include "omoknuni_b200.h"

namespace omoknuni_b200 {

class B200Network : public alphazero::nn::NeuralNetwork {
public:
    B200Network(int64_t input_channels, int64_t board_size, int64_t num_res_blocks = 10, int64_t num_filters = 64,
                int64_t policy_size = 0, int policy_head_ch = 32, int value_head_ch = 32, int max_batch = 1024,
                int device = 0, bool keep_weights = false, int tower_dtype = OB200_DTYPE_BF16)
        : keep_weights_(keep_weights) {
        cfg_.board_size = (int32_t)board_size;
        cfg_.input_channels = (int32_t)input_channels;
        cfg_.filters = (int32_t)num_filters;
        cfg_.blocks = (int32_t)num_res_blocks;
        cfg_.policy_size = (int32_t)(policy_size ? policy_size : board_size * board_size);
        cfg_.policy_head_ch = policy_head_ch;
        cfg_.value_head_ch = value_head_ch;
        cfg_.value_hidden = 256;
        cfg_.max_batch = max_batch;
        cfg_.device = device;
        cfg_.policy_kind = OB200_POLICY_FC;
        cfg_.tower_dtype = tower_dtype;
        if (ob200_net_create(&cfg_, &net_) != OB200_OK) {
            std::fprintf(stderr, "[B200Network] %s\n", ob200_last_error());
            net_ = nullptr;
        }
    }
    ~B200Network() override { ob200_net_destroy(net_); }
    B200Network(const B200Network&) = delete;
    B200Network& operator=(const B200Network&) = delete;

    bool ok() const { return net_ != nullptr; }
    ob200_net* handle() const { return ready_ ? net_ : nullptr; }   // for the search adapter; null until finalised

    // One tensor under the reference module's name, e.g. "res_blocks.3.bn1.running_var".
    bool setTensor(const std::string& name, const float* data, int64_t numel) {
        if (!net_) return false;
        if (keep_weights_) kept_.push_back({name, std::vector<float>(data, data + numel)});
        return report(ob200_net_set_tensor(net_, name.c_str(), data, numel));
    }
    bool finalize() { return net_ && report(ob200_net_finalize(net_)) && (ready_ = true); }

    std::vector<alphazero::mcts::NetworkOutput> inference(
        const std::vector<std::unique_ptr<alphazero::core::IGameState>>& states) override {
        const size_t n = states.size();
        const int A = cfg_.policy_size;
        std::vector<alphazero::mcts::NetworkOutput> out(n);
        for (auto& o : out) { o.policy.assign(A, 1.0f / (float)A); o.value = 0.0f; }   // the reference's default outputs
        if (n == 0 || !net_ || !ready_) return out;
        // Requests larger than max_batch go slice by slice with two slices in flight: while the results of one
        // travel back to the host, the next one's kernels run (ob200_net_submit_gomoku / ob200_net_wait).
        struct Slice {
            std::vector<float> policy, value;
            std::vector<int16_t> hist; std::vector<uint8_t> nh, tm;
            size_t first = 0; int B = 0; int32_t ticket = -1;
        } slice[2];
        try {
            for (auto& sl : slice) { sl.policy.resize((size_t)cfg_.max_batch * A); sl.value.resize(cfg_.max_batch); }
            auto collect = [&](Slice& sl) {
                if (sl.ticket < 0) return;
                const int rc = ob200_net_wait(net_, sl.ticket);
                sl.ticket = -1;
                if (rc != OB200_OK) { report(rc); return; }                  // this slice keeps the default outputs
                for (int b = 0; b < sl.B; ++b) {
                    out[sl.first + b].policy.assign(sl.policy.begin() + (size_t)b * A, sl.policy.begin() + (size_t)(b + 1) * A);
                    out[sl.first + b].value = sl.value[b];
                }
            };
            int turn = 0;
            for (size_t first = 0; first < n; first += (size_t)cfg_.max_batch, turn ^= 1) {
                Slice& sl = slice[turn];
                collect(sl);                                                 // the slice submitted two turns ago
                const int B = (int)std::min(n - first, (size_t)cfg_.max_batch);
                sl.first = first; sl.B = B;
                const bool gomoku = allGomoku(states, first, B) && (cfg_.input_channels == 17 || cfg_.input_channels == 19);
                int rc;
                if (gomoku) {
                    // Gomoku: the device encoder needs only the last 16 moves and the side to move
                    sl.hist.assign((size_t)B * 16, (int16_t)-1);
                    sl.nh.assign(B, 0); sl.tm.assign(B, 2);
                    for (int b = 0; b < B; ++b) {
                        const auto& st = states[first + b];
                        if (!st) continue;                                  // null state: zero planes
                        const std::vector<int> mv = st->getMoveHistory();
                        const int k = (int)std::min<size_t>(16, mv.size());
                        for (int i = 0; i < k; ++i) sl.hist[(size_t)b * 16 + i] = (int16_t)mv[mv.size() - 1 - i];
                        sl.nh[b] = (uint8_t)k;
                        sl.tm[b] = (uint8_t)st->getCurrentPlayer();
                    }
                    rc = ob200_net_submit_gomoku(net_, sl.hist.data(), sl.nh.data(), sl.tm.data(), B, sl.policy.data(), sl.value.data(),
                                                 OB200_OUT_PROBS, &sl.ticket);
                    if (rc == OB200_OK) continue;
                    sl.ticket = -1;
                    if (rc != OB200_ERR_STATE) { report(rc); continue; }
                    // both of the handle's slots are taken (other threads are calling inference() too): finish our other
                    // slice, then take this one through the one-call form, which waits its turn
                    collect(slice[turn ^ 1]);
                    rc = ob200_net_infer_gomoku(net_, sl.hist.data(), sl.nh.data(), sl.tm.data(), B, sl.policy.data(), sl.value.data(),
                                                OB200_OUT_PROBS);
                } else {
                    // any other game: the state's own planes, as prepareInputTensor gathers them (:258-260, :410-494)
                    const int S = cfg_.board_size, C = cfg_.input_channels;
                    std::vector<float> planes((size_t)B * C * S * S, 0.0f);
                    for (int b = 0; b < B; ++b) {
                        const auto& st = states[first + b];
                        if (!st) continue;
                        const auto t = (C == 3) ? st->getTensorRepresentation() : st->getEnhancedTensorRepresentation();
                        for (int c = 0; c < C && c < (int)t.size(); ++c)
                            for (int r = 0; r < S && r < (int)t[c].size(); ++r)
                                std::memcpy(&planes[(((size_t)b * C + c) * S + r) * S], t[c][r].data(),
                                            sizeof(float) * std::min<size_t>(S, t[c][r].size()));
                    }
                    rc = ob200_net_infer_planes(net_, planes.data(), B, C, sl.policy.data(), sl.value.data(), OB200_OUT_PROBS);
                }
                if (rc != OB200_OK) { report(rc); continue; }               // this slice keeps the default outputs
                for (int b = 0; b < B; ++b) {
                    out[first + b].policy.assign(sl.policy.begin() + (size_t)b * A, sl.policy.begin() + (size_t)(b + 1) * A);
                    out[first + b].value = sl.value[b];
                }
            }
            collect(slice[turn]);
            collect(slice[turn ^ 1]);
        } catch (...) {
            // as the reference: swallow and keep the defaults (a slice still in flight writes into buffers of
            // this frame: wait for it before they go away)
            for (auto& sl : slice) if (sl.ticket >= 0) { ob200_net_wait(net_, sl.ticket); sl.ticket = -1; }
        }
        return out;
    }

    // Flat weight file: repeated { uint32 name_len, name, uint64 numel, float data[numel] }.
    void save(const std::string& path) override {
        std::FILE* f = std::fopen(path.c_str(), "wb");
        if (!f) return;
        for (const auto& t : kept_) {
            const uint32_t len = (uint32_t)t.name.size();
            const uint64_t numel = t.data.size();
            std::fwrite(&len, 4, 1, f); std::fwrite(t.name.data(), 1, len, f);
            std::fwrite(&numel, 8, 1, f); std::fwrite(t.data.data(), 4, numel, f);
        }
        std::fclose(f);
    }
    void load(const std::string& path) override {
        std::FILE* f = std::fopen(path.c_str(), "rb");
        if (!f) return;
        std::fseek(f, 0, SEEK_END);
        const long file_size = std::ftell(f);
        std::fseek(f, 0, SEEK_SET);
        uint32_t len; uint64_t numel;
        while (std::fread(&len, 4, 1, f) == 1 && len < 4096) {
            std::string name(len, '\0');
            if (std::fread(&name[0], 1, len, f) != len || std::fread(&numel, 8, 1, f) != 1) break;
            // a truncated or corrupt file must not turn into an allocation of whatever its bytes say
            const long here = std::ftell(f);
            if (here < 0 || file_size < here || numel > (uint64_t)(file_size - here) / 4) break;
            std::vector<float> data(numel);
            if (std::fread(data.data(), 4, numel, f) != numel) break;
            setTensor(name, data.data(), (int64_t)numel);
        }
        std::fclose(f);
        finalize();
    }
    std::vector<int64_t> getInputShape() const override { return {cfg_.input_channels, cfg_.board_size, cfg_.board_size}; }
    int64_t getPolicySize() const override { return cfg_.policy_size; }
    // The optional part of the interface (include/nn/neural_network.h:60-119): inference() is the batch path; the
    // same weights give the same bits on every call; what the reference's optimisation switches ask for is how the
    // library works anyway (one launch per tower that can be captured in a graph, activations resident on the GPU).
    bool supportsEvaluateBatch() const override { return true; }
    std::vector<alphazero::mcts::NetworkOutput> evaluateBatch(
        const std::vector<std::unique_ptr<alphazero::core::IGameState>>& states) override { return inference(states); }
    bool isDeterministic() const override { return true; }
    GPUOptimizationStatus getGPUOptimizationStatus() const override {
        GPUOptimizationStatus st;
        st.cuda_graphs_supported = true;
        st.persistent_kernels_enabled = ready_;
        st.model_is_deterministic = true;
        return st;
    }

private:
    struct Kept { std::string name; std::vector<float> data; };

    static bool allGomoku(const std::vector<std::unique_ptr<alphazero::core::IGameState>>& s, size_t first, int B) {
        for (int b = 0; b < B; ++b)
            if (s[first + b] && s[first + b]->getGameType() != alphazero::core::GameType::GOMOKU) return false;
        return true;
    }
    bool report(int rc) {
        if (rc != OB200_OK) std::fprintf(stderr, "[B200Network] %s\n", ob200_last_error());
        return rc == OB200_OK;
    }

    ob200_net_config cfg_{};
    ob200_net* net_ = nullptr;
    bool ready_ = false;
    bool keep_weights_ = false;
    std::vector<Kept> kept_;
};

// The engine's other injection point: MCTSEngine(InferenceFunction, const MCTSSettings&)
// (include/mcts/mcts_engine.h:230-231, :247), which every engine test of the reference uses.  The function keeps the
// network alive.
inline std::function<std::vector<alphazero::mcts::NetworkOutput>(const std::vector<std::unique_ptr<alphazero::core::IGameState>>&)>
makeInferenceFunction(std::shared_ptr<B200Network> net) {
    return [net](const std::vector<std::unique_ptr<alphazero::core::IGameState>>& states) { return net->inference(states); };
}

}  // namespace omoknuni_b200
