// TEST INFRASTRUCTURE.  The smallest IGameState the reference's MCTSNode constructor accepts, and
// helpers that build real MCTSNode parents whose children carry given statistics through the
// node's public API only.  Shared by ref_shim_tree.cpp and adapter_check.cpp.
#pragma once
#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "core/igamestate.h"
#include "mcts/mcts_node.h"

namespace ref_tiny {

using alphazero::core::GameResult;
using alphazero::core::GameType;
using alphazero::core::IGameState;
using alphazero::mcts::MCTSNode;

// MCTSNode's constructor calls validate(), getGameResult(), getCurrentPlayer(), getLegalMoves() and getHash().
class TinyState final : public IGameState {
public:
    TinyState() : IGameState(GameType::UNKNOWN) {}
    std::vector<int> getLegalMoves() const override { return {0}; }
    bool isLegalMove(int a) const override { return a == 0; }
    void makeMove(int) override {}
    bool undoMove() override { return false; }
    bool isTerminal() const override { return false; }
    GameResult getGameResult() const override { return GameResult::ONGOING; }
    int getCurrentPlayer() const override { return 1; }
    int getBoardSize() const override { return 1; }
    int getActionSpaceSize() const override { return 1; }
    std::vector<std::vector<std::vector<float>>> getTensorRepresentation() const override { return {}; }
    std::vector<std::vector<std::vector<float>>> getEnhancedTensorRepresentation() const override { return {}; }
    uint64_t getHash() const override { return 0; }
    std::unique_ptr<IGameState> clone() const override { return std::make_unique<TinyState>(); }
    void copyFrom(const IGameState&) override {}
    std::string actionToString(int a) const override { return std::to_string(a); }
    std::optional<int> stringToAction(const std::string&) const override { return 0; }
    std::string toString() const override { return "tiny"; }
    bool equals(const IGameState&) const override { return true; }
    std::vector<int> getMoveHistory() const override { return {}; }
    bool validate() const override { return true; }
};

// Give a freshly created node the statistics (N, W, VL, P) through its public API only.  update(w)
// once then update(0) leaves value_sum_ == w exactly; update() removes one unit of virtual loss when
// present, so VL goes last.
inline void load_stats(MCTSNode& node, int n, float w, int vl, float p) {
    if (n > 0) {
        node.update(w);
        for (int i = 1; i < n; ++i) node.update(0.0f);
    }
    if (vl > 0) node.addVirtualLoss(vl);
    node.setPriorProbability(p);
}

struct Family {
    std::shared_ptr<MCTSNode> parent;
};

inline Family make_family(int n_children, const int32_t* N, const float* W, const float* P, const int32_t* VL, int n_parent) {
    Family f;
    f.parent = MCTSNode::create(std::make_unique<TinyState>());
    for (int i = 0; i < n_parent; ++i) f.parent->update(0.0f);
    auto& kids = f.parent->getChildren();
    kids.reserve(n_children);
    for (int i = 0; i < n_children; ++i) {
        auto c = MCTSNode::create(std::make_unique<TinyState>(), f.parent);
        load_stats(*c, N[i], W[i], VL[i], P[i]);
        c->setAction(i);
        kids.push_back(std::move(c));
    }
    return f;
}

inline int index_of(const Family& f, const std::shared_ptr<MCTSNode>& c) {
    if (!c) return -1;
    auto& kids = f.parent->getChildren();
    for (size_t i = 0; i < kids.size(); ++i) if (kids[i].get() == c.get()) return (int)i;
    return -1;
}

}  // namespace ref_tiny
