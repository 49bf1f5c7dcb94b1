// Tree handle with HOST buffers at the boundary: the calls a C++ search loop makes where the
// reference calls MCTSNode::selectChild / applyVirtualLoss / revertVirtualLoss / update /
// setPriorProbabilities / expand (reference include/mcts/mcts_node.h:39-101, call sites
// src/mcts/mcts_engine_batch_tree_simple.cpp:100-111,249-281), batched.  The edge statistics
// live on the device as the structure of arrays of ob200_tree_view; arguments and results
// cross the boundary through page-locked staging buffers owned by the handle, on its own
// stream, one call at a time (internal mutex).
#include "internal.h"
#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

struct ob200_tree {
    int device = 0;
    int max_nodes = 0, n_nodes = 0;            // capacity, nodes in use
    ob200_tree_view view{};                    // device arrays; view.n_nodes = capacity
    cudaStream_t stream = nullptr;
    std::mutex mu;
    // staging: one page-locked block and its device twin, grown on demand
    unsigned char *h_stage = nullptr, *d_stage = nullptr;
    size_t stage_bytes = 0;
    std::vector<void*> owned;
};

namespace ob200 {
namespace {

constexpr size_t kAlign = 256;
size_t round_up(size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

int ensure_stage(ob200_tree* t, size_t bytes) {
    if (bytes <= t->stage_bytes) return OB200_OK;
    size_t want = std::max<size_t>(bytes, 1 << 16);
    want = round_up(want + want / 2);
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    if (t->h_stage) cudaFreeHost(t->h_stage);
    if (t->d_stage) cudaFree(t->d_stage);
    t->h_stage = t->d_stage = nullptr; t->stage_bytes = 0;
    OB200_CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&t->h_stage), want));
    OB200_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&t->d_stage), want));
    t->stage_bytes = want;
    return OB200_OK;
}

// Lays host arrays out in the staging block (256-byte aligned pieces), copies the block to the
// device in one transfer and returns the device addresses.
struct Stager {
    ob200_tree* t;
    size_t used = 0;
    explicit Stager(ob200_tree* tree) : t(tree) {}
    size_t reserve(size_t bytes) { const size_t at = used; used = round_up(used + bytes); return at; }
};

template <typename T>
int dev_array(ob200_tree* t, T** out, size_t count, int fill_byte) {
    void* p = nullptr;
    OB200_CUDA_OK(cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)));
    t->owned.push_back(p);
    OB200_CUDA_OK(cudaMemset(p, fill_byte, std::max<size_t>(count, 1) * sizeof(T)));
    *out = static_cast<T*>(p);
    return OB200_OK;
}

int enter(ob200_tree* t, const char* who) {
    if (!t) return set_error(OB200_ERR_INVALID, "%s: null tree", who);
    OB200_CUDA_OK(cudaSetDevice(t->device));
    return require_device();
}

int check_nodes(ob200_tree* t, const int32_t* ids, int n, const char* who) {
    for (int i = 0; i < n; ++i)
        if (ids[i] < 0 || ids[i] >= t->n_nodes)
            return set_error(OB200_ERR_INVALID, "%s: node id %d (entry %d) outside [0, %d)", who, ids[i], i, t->n_nodes);
    return OB200_OK;
}

__global__ void link_kernel(ob200_tree_view v, const int32_t* parent, const int32_t* slot, const int32_t* child, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v.child_node[(size_t)parent[i] * v.pitch + slot[i]] = child[i];
}

}  // namespace
}  // namespace ob200

using namespace ob200;

extern "C" {

int ob200_tree_create(int32_t device, int32_t max_nodes, int32_t n_children, ob200_tree** out) {
    if (!out || max_nodes < 1 || n_children < 1)
        return set_error(OB200_ERR_INVALID, "ob200_tree_create: need max_nodes >= 1, n_children >= 1 and an output pointer");
    *out = nullptr;
    if (cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();
        return set_error(OB200_ERR_NO_DEVICE, "ob200_tree_create: CUDA device %d is not available (there is no CPU path)", device);
    }
    if (int rc = require_device()) return rc;
    ob200_tree* t = new ob200_tree;
    t->device = device; t->max_nodes = max_nodes;
    ob200_tree_view& v = t->view;
    v.n_nodes = max_nodes; v.n_children = n_children;
    v.pitch = ob200_tree_pitch(n_children);
    v.mask_words = (ob200_tree_mask_words(n_children) + 3) / 4 * 4;     // 16-byte rows: the staged selection kernel applies
    const size_t edges = (size_t)max_nodes * v.pitch;
    int rc = OB200_OK;
    auto A = [&](int r) { if (!rc) rc = r; };
    A(dev_array(t, &v.N, edges, 0)); A(dev_array(t, &v.W, edges, 0)); A(dev_array(t, &v.P, edges, 0));
    A(dev_array(t, &v.VL, edges, 0)); A(dev_array(t, &v.child_node, edges, 0xFF));
    A(dev_array(t, &v.legal_bits, (size_t)max_nodes * v.mask_words, 0)); A(dev_array(t, &v.node_visits, (size_t)max_nodes, 0));
    if (!rc && cudaStreamCreateWithFlags(&t->stream, cudaStreamNonBlocking) != cudaSuccess)
        rc = set_error(OB200_ERR_CUDA, "ob200_tree_create: cannot create a stream");
    if (rc) { ob200_tree_destroy(t); return rc; }
    *out = t;
    return OB200_OK;
}

void ob200_tree_destroy(ob200_tree* t) {
    if (!t) return;
    cudaSetDevice(t->device);
    if (t->stream) { cudaStreamSynchronize(t->stream); cudaStreamDestroy(t->stream); }
    for (void* p : t->owned) cudaFree(p);
    if (t->h_stage) cudaFreeHost(t->h_stage);
    if (t->d_stage) cudaFree(t->d_stage);
    delete t;
}

int ob200_tree_view_of(ob200_tree* t, ob200_tree_view* view_out) {
    if (!t || !view_out) return set_error(OB200_ERR_INVALID, "ob200_tree_view_of: null argument");
    *view_out = t->view;
    return OB200_OK;
}

int32_t ob200_tree_node_count(ob200_tree* t) { return t ? t->n_nodes : 0; }

int ob200_tree_clear(ob200_tree* t) {
    if (int rc = enter(t, "ob200_tree_clear")) return rc;
    std::lock_guard<std::mutex> lk(t->mu);
    const ob200_tree_view& v = t->view;
    const size_t edges = (size_t)t->n_nodes * v.pitch;
    OB200_CUDA_OK(cudaMemsetAsync(v.N, 0, edges * 4, t->stream)); OB200_CUDA_OK(cudaMemsetAsync(v.W, 0, edges * 4, t->stream));
    OB200_CUDA_OK(cudaMemsetAsync(v.P, 0, edges * 4, t->stream)); OB200_CUDA_OK(cudaMemsetAsync(v.VL, 0, edges * 4, t->stream));
    OB200_CUDA_OK(cudaMemsetAsync(v.child_node, 0xFF, edges * 4, t->stream));
    OB200_CUDA_OK(cudaMemsetAsync(v.legal_bits, 0, (size_t)t->n_nodes * v.mask_words * 4, t->stream));
    OB200_CUDA_OK(cudaMemsetAsync(v.node_visits, 0, (size_t)t->n_nodes * 4, t->stream));
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    t->n_nodes = 0;
    return OB200_OK;
}

int ob200_tree_add_nodes(ob200_tree* t, int32_t n, const uint32_t* exists_bits, int32_t words_per_node, int32_t* first_id_out) {
    if (int rc = enter(t, "ob200_tree_add_nodes")) return rc;
    const ob200_tree_view& v = t->view;
    if (n < 0 || !exists_bits || words_per_node < ob200_tree_mask_words(v.n_children) || words_per_node > v.mask_words)
        return set_error(OB200_ERR_INVALID, "ob200_tree_add_nodes: need exists_bits with %d to %d words per node", ob200_tree_mask_words(v.n_children), v.mask_words);
    std::lock_guard<std::mutex> lk(t->mu);
    if (t->n_nodes + (long long)n > t->max_nodes)
        return set_error(OB200_ERR_TOO_LARGE, "ob200_tree_add_nodes: %d + %d nodes exceed the tree's capacity %d", t->n_nodes, n, t->max_nodes);
    if (first_id_out) *first_id_out = t->n_nodes;
    if (n == 0) return OB200_OK;
    const size_t bytes = (size_t)n * v.mask_words * 4;
    if (int rc = ensure_stage(t, bytes)) return rc;
    uint32_t* h = reinterpret_cast<uint32_t*>(t->h_stage);
    std::memset(h, 0, bytes);
    const int real_words = ob200_tree_mask_words(v.n_children);
    for (int i = 0; i < n; ++i)
        for (int w = 0; w < real_words; ++w) {
            uint32_t m = exists_bits[(size_t)i * words_per_node + w];
            if ((w + 1) * 32 > v.n_children) m &= (v.n_children - w * 32 >= 32) ? 0xFFFFFFFFu : ((1u << (v.n_children - w * 32)) - 1u);
            h[(size_t)i * v.mask_words + w] = m;
        }
    // rows of new nodes are zero / -1 already: the arrays start that way and ob200_tree_clear restores it
    OB200_CUDA_OK(cudaMemcpyAsync(v.legal_bits + (size_t)t->n_nodes * v.mask_words, h, bytes, cudaMemcpyHostToDevice, t->stream));
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    t->n_nodes += n;
    return OB200_OK;
}

int ob200_tree_link(ob200_tree* t, int32_t n, const int32_t* parent, const int32_t* slot, const int32_t* child) {
    if (int rc = enter(t, "ob200_tree_link")) return rc;
    if (n < 0 || !parent || !slot || !child) return set_error(OB200_ERR_INVALID, "ob200_tree_link: null argument");
    std::lock_guard<std::mutex> lk(t->mu);
    if (int rc = check_nodes(t, parent, n, "ob200_tree_link")) return rc;
    for (int i = 0; i < n; ++i)
        if (slot[i] < 0 || slot[i] >= t->view.n_children || child[i] < -1 || child[i] >= t->n_nodes)
            return set_error(OB200_ERR_INVALID, "ob200_tree_link: entry %d: slot %d / child %d out of range", i, slot[i], child[i]);
    if (n == 0) return OB200_OK;
    Stager s(t);
    const size_t a = s.reserve((size_t)n * 4), b = s.reserve((size_t)n * 4), c = s.reserve((size_t)n * 4);
    if (int rc = ensure_stage(t, s.used)) return rc;
    std::memcpy(t->h_stage + a, parent, (size_t)n * 4); std::memcpy(t->h_stage + b, slot, (size_t)n * 4);
    std::memcpy(t->h_stage + c, child, (size_t)n * 4);
    OB200_CUDA_OK(cudaMemcpyAsync(t->d_stage, t->h_stage, s.used, cudaMemcpyHostToDevice, t->stream));
    link_kernel<<<(n + 255) / 256, 256, 0, t->stream>>>(t->view, reinterpret_cast<int32_t*>(t->d_stage + a),
                                                        reinterpret_cast<int32_t*>(t->d_stage + b),
                                                        reinterpret_cast<int32_t*>(t->d_stage + c), n);
    OB200_LAUNCHED("link_kernel");
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    return OB200_OK;
}

int ob200_tree_select(ob200_tree* t, const int32_t* node_ids, int32_t n, float c_puct, int32_t vl_value, int32_t apply_vl,
                      int32_t* sel_out) {
    if (int rc = enter(t, "ob200_tree_select")) return rc;
    if (n < 0 || !node_ids || !sel_out) return set_error(OB200_ERR_INVALID, "ob200_tree_select: null argument");
    std::lock_guard<std::mutex> lk(t->mu);
    if (int rc = check_nodes(t, node_ids, n, "ob200_tree_select")) return rc;
    if (n == 0) return OB200_OK;
    Stager s(t);
    const size_t a = s.reserve((size_t)n * 4), b = s.reserve((size_t)n * 4);
    if (int rc = ensure_stage(t, s.used)) return rc;
    std::memcpy(t->h_stage + a, node_ids, (size_t)n * 4);
    OB200_CUDA_OK(cudaMemcpyAsync(t->d_stage + a, t->h_stage + a, (size_t)n * 4, cudaMemcpyHostToDevice, t->stream));
    if (int rc = ob200_launch_puct_select(&t->view, reinterpret_cast<int32_t*>(t->d_stage + a), n, c_puct, vl_value, apply_vl,
                                          reinterpret_cast<int32_t*>(t->d_stage + b), t->stream)) return rc;
    OB200_CUDA_OK(cudaMemcpyAsync(t->h_stage + b, t->d_stage + b, (size_t)n * 4, cudaMemcpyDeviceToHost, t->stream));
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    std::memcpy(sel_out, t->h_stage + b, (size_t)n * 4);
    return OB200_OK;
}

int ob200_tree_virtual_loss(ob200_tree* t, const int32_t* node_ids, const int32_t* slots, int32_t n, int32_t amount) {
    if (int rc = enter(t, "ob200_tree_virtual_loss")) return rc;
    if (n < 0 || !node_ids || !slots) return set_error(OB200_ERR_INVALID, "ob200_tree_virtual_loss: null argument");
    std::lock_guard<std::mutex> lk(t->mu);
    if (int rc = check_nodes(t, node_ids, n, "ob200_tree_virtual_loss")) return rc;
    for (int i = 0; i < n; ++i)
        if (slots[i] >= t->view.n_children) return set_error(OB200_ERR_INVALID, "ob200_tree_virtual_loss: slot %d out of range", slots[i]);
    if (n == 0 || amount == 0) return OB200_OK;
    Stager s(t);
    const size_t a = s.reserve((size_t)n * 4), b = s.reserve((size_t)n * 4);
    if (int rc = ensure_stage(t, s.used)) return rc;
    std::memcpy(t->h_stage + a, node_ids, (size_t)n * 4); std::memcpy(t->h_stage + b, slots, (size_t)n * 4);
    OB200_CUDA_OK(cudaMemcpyAsync(t->d_stage, t->h_stage, s.used, cudaMemcpyHostToDevice, t->stream));
    const int32_t* dn = reinterpret_cast<int32_t*>(t->d_stage + a);
    const int32_t* ds = reinterpret_cast<int32_t*>(t->d_stage + b);
    const int rc = amount > 0 ? ob200_launch_vl_apply(&t->view, dn, ds, n, amount, t->stream)
                              : ob200_launch_vl_revert(&t->view, dn, ds, n, -amount, t->stream);
    if (rc) return rc;
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    return OB200_OK;
}

int ob200_tree_backup(ob200_tree* t, const int32_t* paths, const int32_t* path_len, const float* leaf_values, int32_t n,
                      int32_t max_depth, int32_t vl_value) {
    if (int rc = enter(t, "ob200_tree_backup")) return rc;
    if (n < 0 || max_depth < 1 || !paths || !path_len || !leaf_values) return set_error(OB200_ERR_INVALID, "ob200_tree_backup: bad argument");
    std::lock_guard<std::mutex> lk(t->mu);
    for (int i = 0; i < n; ++i) {
        const int len = std::min(path_len[i], max_depth);
        for (int d = 0; d < len; ++d) {
            const int node = paths[((size_t)i * max_depth + d) * 2], slot = paths[((size_t)i * max_depth + d) * 2 + 1];
            if (node < 0 || node >= t->n_nodes || slot < 0 || slot >= t->view.n_children)
                return set_error(OB200_ERR_INVALID, "ob200_tree_backup: path %d step %d names edge (%d, %d)", i, d, node, slot);
        }
    }
    if (n == 0) return OB200_OK;
    Stager s(t);
    const size_t pb = (size_t)n * max_depth * 2 * 4;
    const size_t a = s.reserve(pb), b = s.reserve((size_t)n * 4), c = s.reserve((size_t)n * 4);
    if (int rc = ensure_stage(t, s.used)) return rc;
    std::memcpy(t->h_stage + a, paths, pb); std::memcpy(t->h_stage + b, path_len, (size_t)n * 4);
    std::memcpy(t->h_stage + c, leaf_values, (size_t)n * 4);
    OB200_CUDA_OK(cudaMemcpyAsync(t->d_stage, t->h_stage, s.used, cudaMemcpyHostToDevice, t->stream));
    if (int rc = ob200_launch_backup(&t->view, reinterpret_cast<int32_t*>(t->d_stage + a), reinterpret_cast<int32_t*>(t->d_stage + b),
                                     reinterpret_cast<float*>(t->d_stage + c), n, max_depth, vl_value, t->stream)) return rc;
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    return OB200_OK;
}

int ob200_tree_set_priors(ob200_tree* t, const int32_t* node_ids, int32_t n, const float* policy, int32_t policy_size) {
    if (int rc = enter(t, "ob200_tree_set_priors")) return rc;
    if (n < 0 || !node_ids || !policy || policy_size < 1) return set_error(OB200_ERR_INVALID, "ob200_tree_set_priors: bad argument");
    std::lock_guard<std::mutex> lk(t->mu);
    if (int rc = check_nodes(t, node_ids, n, "ob200_tree_set_priors")) return rc;
    if (n == 0) return OB200_OK;
    Stager s(t);
    const size_t a = s.reserve((size_t)n * 4), b = s.reserve((size_t)n * policy_size * 4);
    if (int rc = ensure_stage(t, s.used)) return rc;
    std::memcpy(t->h_stage + a, node_ids, (size_t)n * 4); std::memcpy(t->h_stage + b, policy, (size_t)n * policy_size * 4);
    OB200_CUDA_OK(cudaMemcpyAsync(t->d_stage, t->h_stage, s.used, cudaMemcpyHostToDevice, t->stream));
    if (int rc = ob200_launch_set_priors(&t->view, reinterpret_cast<int32_t*>(t->d_stage + a), n, reinterpret_cast<float*>(t->d_stage + b),
                                         policy_size, nullptr, t->stream)) return rc;
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    return OB200_OK;
}

static int field_ptr(ob200_tree* t, int32_t field, unsigned char** base, size_t* row_bytes) {
    const ob200_tree_view& v = t->view;
    switch (field) {
        case OB200_TREE_N: *base = reinterpret_cast<unsigned char*>(v.N); *row_bytes = (size_t)v.pitch * 4; break;
        case OB200_TREE_W: *base = reinterpret_cast<unsigned char*>(v.W); *row_bytes = (size_t)v.pitch * 4; break;
        case OB200_TREE_P: *base = reinterpret_cast<unsigned char*>(v.P); *row_bytes = (size_t)v.pitch * 4; break;
        case OB200_TREE_VL: *base = reinterpret_cast<unsigned char*>(v.VL); *row_bytes = (size_t)v.pitch * 4; break;
        case OB200_TREE_CHILD: *base = reinterpret_cast<unsigned char*>(v.child_node); *row_bytes = (size_t)v.pitch * 4; break;
        case OB200_TREE_EXISTS: *base = reinterpret_cast<unsigned char*>(v.legal_bits); *row_bytes = (size_t)v.mask_words * 4; break;
        case OB200_TREE_VISITS: *base = reinterpret_cast<unsigned char*>(v.node_visits); *row_bytes = 4; break;
        default: return set_error(OB200_ERR_INVALID, "tree field %d unknown", field);
    }
    return OB200_OK;
}

int ob200_tree_read(ob200_tree* t, int32_t field, int32_t first_node, int32_t n_nodes, void* host_out) {
    if (int rc = enter(t, "ob200_tree_read")) return rc;
    std::lock_guard<std::mutex> lk(t->mu);
    if (!host_out || first_node < 0 || n_nodes < 0 || first_node + (long long)n_nodes > t->n_nodes)
        return set_error(OB200_ERR_INVALID, "ob200_tree_read: nodes [%d, %d) outside the %d in use", first_node, first_node + n_nodes, t->n_nodes);
    unsigned char* base; size_t row;
    if (int rc = field_ptr(t, field, &base, &row)) return rc;
    if (n_nodes == 0) return OB200_OK;
    OB200_CUDA_OK(cudaMemcpyAsync(host_out, base + (size_t)first_node * row, (size_t)n_nodes * row, cudaMemcpyDeviceToHost, t->stream));
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    return OB200_OK;
}

int ob200_tree_write(ob200_tree* t, int32_t field, int32_t first_node, int32_t n_nodes, const void* host_in) {
    if (int rc = enter(t, "ob200_tree_write")) return rc;
    std::lock_guard<std::mutex> lk(t->mu);
    if (!host_in || first_node < 0 || n_nodes < 0 || first_node + (long long)n_nodes > t->n_nodes)
        return set_error(OB200_ERR_INVALID, "ob200_tree_write: nodes [%d, %d) outside the %d in use", first_node, first_node + n_nodes, t->n_nodes);
    if (field == OB200_TREE_EXISTS) return set_error(OB200_ERR_INVALID, "ob200_tree_write: existence masks are set by ob200_tree_add_nodes");
    unsigned char* base; size_t row;
    if (int rc = field_ptr(t, field, &base, &row)) return rc;
    if (n_nodes == 0) return OB200_OK;
    OB200_CUDA_OK(cudaMemcpyAsync(base + (size_t)first_node * row, host_in, (size_t)n_nodes * row, cudaMemcpyHostToDevice, t->stream));
    OB200_CUDA_OK(cudaStreamSynchronize(t->stream));
    return OB200_OK;
}

}  // extern "C"
