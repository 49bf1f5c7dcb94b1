// Drop-in for the per-node calls MCTSEngine makes on alphazero::mcts::MCTSNode
// (reference include/mcts/mcts_node.h:39-101): selectChild, applyVirtualLoss,
// revertVirtualLoss, update, expand, setPriorProbabilities - the same meanings,
// over a device-resident tree, many nodes per call.  Where the reference's batched
// loop does, one simulation at a time inside an OpenMP region
// (src/mcts/mcts_engine_batch_tree_simple.cpp:100-111),
//     best = current->selectChild(c_puct, ...);  best->applyVirtualLoss(vl);
// a loop built on this class collects the current node of every simulation and calls
// selectChildBatch once per tree level; where it does (:276-281)
//     for node in reverse(path): node->update(v); node->revertVirtualLoss(vl); v = -v;
// it hands all paths to backup().
//
// A node is an integer id; its children are slots (the reference's child index: slot
// s of node n stands for n->getChildren()[s]); statistics belong to the edge
// (node, slot), which is where the reference keeps them too (in the child object).
// Header-only, plain C++17 over the C ABI of include/omoknuni_b200.h; no CUDA
// headers, no libtorch.  Errors: methods return false (or -1) after printing the
// library's message, as the reference's callers swallow and log
// (src/mcts/mcts_engine_search.cpp:668-670); nothing throws.
#pragma once

#include <cstdint>
#include <cstdio>
#include <vector>

#include "omoknuni_b200.h"

namespace omoknuni_b200 {

class B200Tree {
public:
    // max_nodes: capacity of the node pool; max_children: child slots per node (225 for 15x15 Gomoku:
    // slot == action; any enumeration of legal moves works as long as the caller keeps it)
    B200Tree(int max_nodes, int max_children, int device = 0) : children_(max_children) {
        if (ob200_tree_create(device, max_nodes, max_children, &tree_) != OB200_OK) { report(); tree_ = nullptr; }
        words_ = (max_children + 31) / 32;
    }
    ~B200Tree() { ob200_tree_destroy(tree_); }
    B200Tree(const B200Tree&) = delete;
    B200Tree& operator=(const B200Tree&) = delete;

    bool ok() const { return tree_ != nullptr; }
    int size() const { return ob200_tree_node_count(tree_); }
    bool clear() { return tree_ && check(ob200_tree_clear(tree_)); }

    // MCTSNode::create + expand (src/mcts/mcts_node.cpp:238-436): a node whose children are the given
    // slots (for a game state: its legal moves), all unvisited and not yet expanded.  Returns the id.
    int addNode(const std::vector<int>& child_slots) {
        if (!tree_) return -1;
        std::vector<uint32_t> bits(words_, 0u);
        for (int s : child_slots)
            if (s >= 0 && s < children_) bits[s >> 5] |= 1u << (s & 31);
        int32_t id = -1;
        return check(ob200_tree_add_nodes(tree_, 1, bits.data(), words_, &id)) ? id : -1;
    }
    // The child behind edge (parent, slot) is node `child`: expand's children_ entry, or the
    // transposition redirect of MCTSNode::updateChildReference.
    bool setChild(int parent, int slot, int child) {
        const int32_t p = parent, s = slot, c = child;
        return tree_ && check(ob200_tree_link(tree_, 1, &p, &s, &c));
    }

    // selectChild(c_puct) for every node of `nodes` (RAVE off; -1 for a node without children), and when
    // virtual_loss > 0 applyVirtualLoss(virtual_loss) on each selected child, as the search loop does right
    // after the selection.  Entries of one call do not see each other's virtual loss.
    std::vector<int> selectChildBatch(const std::vector<int>& nodes, float c_puct, int virtual_loss = 0) {
        std::vector<int32_t> sel(nodes.size(), -1);
        if (!tree_ || nodes.empty()) return std::vector<int>(sel.begin(), sel.end());
        const std::vector<int32_t> ids(nodes.begin(), nodes.end());
        if (!check(ob200_tree_select(tree_, ids.data(), (int32_t)ids.size(), c_puct, virtual_loss, virtual_loss > 0, sel.data())))
            std::fill(sel.begin(), sel.end(), -1);
        return std::vector<int>(sel.begin(), sel.end());
    }
    // MCTSNode::applyVirtualLoss / addVirtualLoss(amount) on the children (nodes[i], slots[i]).
    bool applyVirtualLoss(const std::vector<int>& nodes, const std::vector<int>& slots, int amount) {
        return amount <= 0 || virtualLoss(nodes, slots, amount);
    }
    // MCTSNode::revertVirtualLoss / removeVirtualLoss(amount): subtract, clamp at zero.
    bool revertVirtualLoss(const std::vector<int>& nodes, const std::vector<int>& slots, int amount) {
        return amount <= 0 || virtualLoss(nodes, slots, -amount);
    }
    // The backup loop: paths[i] = edges (node, slot) from the root down; leaf to root each edge gets
    // update(v) (visits + 1, value sum + v, one unit of virtual loss off), revertVirtualLoss(virtual_loss),
    // and v changes sign per ply.
    bool backup(const std::vector<std::vector<std::pair<int, int>>>& paths, const std::vector<float>& leaf_values, int virtual_loss) {
        if (!tree_ || paths.size() != leaf_values.size()) return false;
        size_t depth = 1;
        for (const auto& p : paths) depth = p.size() > depth ? p.size() : depth;
        std::vector<int32_t> flat(paths.size() * depth * 2, 0), len(paths.size());
        for (size_t i = 0; i < paths.size(); ++i) {
            len[i] = (int32_t)paths[i].size();
            for (size_t d = 0; d < paths[i].size(); ++d) {
                flat[(i * depth + d) * 2] = paths[i][d].first;
                flat[(i * depth + d) * 2 + 1] = paths[i][d].second;
            }
        }
        return check(ob200_tree_backup(tree_, flat.data(), len.data(), leaf_values.data(), (int32_t)paths.size(), (int32_t)depth, virtual_loss));
    }
    // MCTSNode::setPriorProbabilities (src/mcts/mcts_node.cpp:512-593) with slot == action:
    // prior of child s = clamp(policy[s], 0, 1), no renormalisation.
    bool setPriorProbabilities(int node, const std::vector<float>& policy) {
        const int32_t id = node;
        return tree_ && check(ob200_tree_set_priors(tree_, &id, 1, policy.data(), (int32_t)policy.size()));
    }

    // Per-child statistics of one node, as MCTSNode's getters give them for each child:
    // getVisitCount, value sum (getValue() * visits), getVirtualLoss, getPriorProbability.
    struct ChildStats { std::vector<int> visits, virtual_loss; std::vector<float> value_sum, prior; };
    bool childStats(int node, ChildStats* out) {
        if (!tree_ || !out) return false;
        ob200_tree_view v;
        if (!check(ob200_tree_view_of(tree_, &v))) return false;
        std::vector<int32_t> n(v.pitch), vl(v.pitch);
        std::vector<float> w(v.pitch), p(v.pitch);
        if (!check(ob200_tree_read(tree_, OB200_TREE_N, node, 1, n.data())) || !check(ob200_tree_read(tree_, OB200_TREE_VL, node, 1, vl.data())) ||
            !check(ob200_tree_read(tree_, OB200_TREE_W, node, 1, w.data())) || !check(ob200_tree_read(tree_, OB200_TREE_P, node, 1, p.data())))
            return false;
        out->visits.assign(n.begin(), n.begin() + children_); out->virtual_loss.assign(vl.begin(), vl.begin() + children_);
        out->value_sum.assign(w.begin(), w.begin() + children_); out->prior.assign(p.begin(), p.begin() + children_);
        return true;
    }
    // Load the statistics of one node's children (tests, tree reuse from a host-side tree).
    bool loadChildStats(int node, const ChildStats& s, int node_visits) {
        if (!tree_) return false;
        ob200_tree_view v;
        if (!check(ob200_tree_view_of(tree_, &v))) return false;
        std::vector<int32_t> n(v.pitch, 0), vl(v.pitch, 0);
        std::vector<float> w(v.pitch, 0.0f), p(v.pitch, 0.0f);
        for (int i = 0; i < children_; ++i) {
            if (i < (int)s.visits.size()) n[i] = s.visits[i];
            if (i < (int)s.virtual_loss.size()) vl[i] = s.virtual_loss[i];
            if (i < (int)s.value_sum.size()) w[i] = s.value_sum[i];
            if (i < (int)s.prior.size()) p[i] = s.prior[i];
        }
        const int32_t nv = node_visits;
        return check(ob200_tree_write(tree_, OB200_TREE_N, node, 1, n.data())) && check(ob200_tree_write(tree_, OB200_TREE_VL, node, 1, vl.data())) &&
               check(ob200_tree_write(tree_, OB200_TREE_W, node, 1, w.data())) && check(ob200_tree_write(tree_, OB200_TREE_P, node, 1, p.data())) &&
               check(ob200_tree_write(tree_, OB200_TREE_VISITS, node, 1, &nv));
    }
    int nodeVisits(int node) {
        int32_t v = -1;
        return tree_ && check(ob200_tree_read(tree_, OB200_TREE_VISITS, node, 1, &v)) ? v : -1;
    }

    // The fields of the reference's MCTSStats (include/mcts/mcts_engine.h:154-197) that this path produces, from
    // the library's per-process counters: total_evaluations, total_batches_processed, avg_batch_size.  A template
    // so that this header does not need the engine header; any struct with those members works.
    template <class Stats>
    static void fillStats(Stats& s) {
        ob200_counters c;
        if (ob200_get_counters(&c) != OB200_OK) return;
        s.total_evaluations = (decltype(s.total_evaluations))c.evals;
        s.total_batches_processed = (decltype(s.total_batches_processed))c.batches;
        s.avg_batch_size = c.batches ? (float)((double)c.evals / (double)c.batches) : 0.0f;
    }

    ob200_tree* handle() const { return tree_; }

private:
    bool virtualLoss(const std::vector<int>& nodes, const std::vector<int>& slots, int amount) {
        if (!tree_ || nodes.size() != slots.size()) return false;
        if (nodes.empty()) return true;
        const std::vector<int32_t> n(nodes.begin(), nodes.end()), s(slots.begin(), slots.end());
        return check(ob200_tree_virtual_loss(tree_, n.data(), s.data(), (int32_t)n.size(), amount));
    }
    bool check(int rc) { if (rc != OB200_OK) report(); return rc == OB200_OK; }
    static void report() { std::fprintf(stderr, "[B200Tree] %s\n", ob200_last_error()); }

    ob200_tree* tree_ = nullptr;
    int children_ = 0, words_ = 0;
};

}  // namespace omoknuni_b200
