// Batched PUCT selection, virtual loss, backup and prior scatter over
// structure-of-arrays edge statistics (sm_100a).
//
// One warp owns one node row.  Rows are `pitch` (multiple of 4) elements, so
// every lane issues 128-bit loads of N, W, P and VL; a 225-slot row is 57
// vectors = two fully independent load rounds per lane.  Scores use IEEE
// round-to-nearest intrinsics in the operation order of
// MCTSNode::selectChild (reference src/mcts/mcts_node.cpp:143-167), so no
// FMA contraction or fast-math can change a comparison.  The argmax is a
// shuffle butterfly whose combine rule keeps the lowest slot on equal scores.
#include "common.h"
#include <cfloat>

namespace ob200 {
namespace {

constexpr int kWarpsPerBlock = 8;

struct Best {
    float score;   // best score seen with strict '>' starting from -inf
    int idx;       // its slot, -1 when nothing compared greater than -inf
    int min_n;     // fewest visits among existing slots (fallback)
    int min_idx;   // its slot, -1 when the row has no slot
};

__device__ __forceinline__ float puct_score(int n, float w, float p, int vl, float explore) {
    const int ev = n + vl;
    const float evf = (float)ev;
    const float q = ev > 0 ? __fdiv_rn(__fsub_rn(w, (float)vl), evf) : 0.0f;
    const float u = __fdiv_rn(__fmul_rn(p, explore), __fadd_rn(1.0f, evf));
    return __fadd_rn(q, u);
}

__device__ __forceinline__ void consider(Best& b, int slot, int n, float w, float p, int vl,
                                         float explore) {
    const float s = puct_score(n, w, p, vl, explore);
    if (s > b.score) { b.score = s; b.idx = slot; }
    if (n < b.min_n) { b.min_n = n; b.min_idx = slot; }
}

__device__ __forceinline__ Best warp_combine(Best b) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, b.score, off);
        const int oi = __shfl_xor_sync(0xffffffffu, b.idx, off);
        const int on = __shfl_xor_sync(0xffffffffu, b.min_n, off);
        const int om = __shfl_xor_sync(0xffffffffu, b.min_idx, off);
        if (oi >= 0 && (b.idx < 0 || os > b.score || (os == b.score && oi < b.idx))) {
            b.score = os; b.idx = oi;
        }
        if (om >= 0 && (b.min_idx < 0 || on < b.min_n || (on == b.min_n && om < b.min_idx))) {
            b.min_n = on; b.min_idx = om;
        }
    }
    return b;
}

// Scans one row with the whole warp.  kStream: N/W/P are read with streaming
// loads (each byte is used once per pass); VL always comes from L2 because
// other warps change it with atomics.
template <bool kStream>
__device__ __forceinline__ int select_row(const ob200_tree_view& t, int node, float c_puct, int lane) {
    const int nvec = t.pitch >> 2;
    const size_t row = (size_t)node * t.pitch;
    const int4* __restrict__ N4 = reinterpret_cast<const int4*>(t.N + row);
    const float4* __restrict__ W4 = reinterpret_cast<const float4*>(t.W + row);
    const float4* __restrict__ P4 = reinterpret_cast<const float4*>(t.P + row);
    const int4* V4 = reinterpret_cast<const int4*>(t.VL + row);
    const uint32_t* __restrict__ mask = t.legal_bits + (size_t)node * t.mask_words;
    const float explore = __fmul_rn(c_puct, __fsqrt_rn((float)t.node_visits[node]));

    Best b{-INFINITY, -1, INT_MAX, -1};
    for (int v0 = 0; v0 < nvec; v0 += 64) {
        // two independent load rounds in flight per lane
        const int va = v0 + lane, vb = v0 + 32 + lane;
        const bool ha = va < nvec, hb = vb < nvec;
        int4 na, nb, la, lb; float4 wa, wb, pa, pb; uint32_t ma = 0, mb = 0;
        if (ha) {
            na = kStream ? __ldcs(N4 + va) : __ldcg(N4 + va);
            wa = kStream ? __ldcs(W4 + va) : __ldcg(W4 + va);
            pa = kStream ? __ldcs(P4 + va) : __ldcg(P4 + va);
            la = __ldcg(V4 + va);
            ma = (__ldg(mask + (va >> 3)) >> ((va & 7) * 4)) & 0xFu;
        }
        if (hb) {
            nb = kStream ? __ldcs(N4 + vb) : __ldcg(N4 + vb);
            wb = kStream ? __ldcs(W4 + vb) : __ldcg(W4 + vb);
            pb = kStream ? __ldcs(P4 + vb) : __ldcg(P4 + vb);
            lb = __ldcg(V4 + vb);
            mb = (__ldg(mask + (vb >> 3)) >> ((vb & 7) * 4)) & 0xFu;
        }
        if (ha && ma) {
            const int s = va * 4;
            if (ma & 1u) consider(b, s + 0, na.x, wa.x, pa.x, la.x, explore);
            if (ma & 2u) consider(b, s + 1, na.y, wa.y, pa.y, la.y, explore);
            if (ma & 4u) consider(b, s + 2, na.z, wa.z, pa.z, la.z, explore);
            if (ma & 8u) consider(b, s + 3, na.w, wa.w, pa.w, la.w, explore);
        }
        if (hb && mb) {
            const int s = vb * 4;
            if (mb & 1u) consider(b, s + 0, nb.x, wb.x, pb.x, lb.x, explore);
            if (mb & 2u) consider(b, s + 1, nb.y, wb.y, pb.y, lb.y, explore);
            if (mb & 4u) consider(b, s + 2, nb.z, wb.z, pb.z, lb.z, explore);
            if (mb & 8u) consider(b, s + 3, nb.w, wb.w, pb.w, lb.w, explore);
        }
    }
    b = warp_combine(b);
    return b.idx >= 0 ? b.idx : b.min_idx;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
puct_select_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids, int n, float c_puct,
                   int vl_value, int apply_vl, int32_t* __restrict__ sel_out) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n) return;
    const int node = node_ids ? node_ids[warp] : warp;
    int sel = -1;
    if (node >= 0 && node < t.n_nodes) sel = select_row<true>(t, node, c_puct, lane);
    if (lane == 0) {
        sel_out[warp] = sel;
        if (sel >= 0 && apply_vl && vl_value > 0) atomicAdd(t.VL + (size_t)node * t.pitch + sel, vl_value);
    }
}

// max(old - amount, 0) as one atomic step (sequentially the same result as
// the reference's fetch_sub followed by the store of zero).
__device__ __forceinline__ void vl_sub_clamped(int32_t* addr, int amount, bool one_first) {
    int old = *reinterpret_cast<volatile int32_t*>(addr);
    while (true) {
        int v = old;
        if (one_first && v > 0) v -= 1;           // MCTSNode::update removes one unit when present
        if (amount > 0) v = (v < amount) ? 0 : v - amount;
        const int seen = atomicCAS(addr, old, v);
        if (seen == old) break;
        old = seen;
    }
}

__global__ void vl_apply_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids,
                                const int32_t* __restrict__ sel, int n, int vl_value) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int node = node_ids ? node_ids[i] : i;
    const int s = sel[i];
    if (node < 0 || node >= t.n_nodes || s < 0 || s >= t.n_children) return;
    atomicAdd(t.VL + (size_t)node * t.pitch + s, vl_value);
}

__global__ void vl_revert_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids,
                                 const int32_t* __restrict__ sel, int n, int vl_value) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int node = node_ids ? node_ids[i] : i;
    const int s = sel[i];
    if (node < 0 || node >= t.n_nodes || s < 0 || s >= t.n_children) return;
    vl_sub_clamped(t.VL + (size_t)node * t.pitch + s, vl_value, false);
}

__global__ void backup_kernel(ob200_tree_view t, const int32_t* __restrict__ paths,
                              const int32_t* __restrict__ path_len,
                              const float* __restrict__ leaf_values, int n, int max_depth,
                              int vl_value) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int len = path_len[i];
    if (len > max_depth) len = max_depth;
    float v = leaf_values[i];
    const int32_t* p = paths + (size_t)i * max_depth * 2;
    for (int d = len - 1; d >= 0; --d) {
        const int node = p[2 * d], s = p[2 * d + 1];
        if (node < 0 || node >= t.n_nodes || s < 0 || s >= t.n_children) { v = -v; continue; }
        const size_t e = (size_t)node * t.pitch + s;
        atomicAdd(t.N + e, 1);
        atomicAdd(t.W + e, v);
        vl_sub_clamped(t.VL + e, vl_value, true);
        if (d == len - 1 && t.child_node) {
            const int child = t.child_node[e];
            if (child >= 0 && child < t.n_nodes) atomicAdd(t.node_visits + child, 1);
        }
        atomicAdd(t.node_visits + node, 1);
        v = -v;
    }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
set_priors_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids, int n,
                  const float* __restrict__ policy, int policy_size,
                  const int32_t* __restrict__ slot_action) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n) return;
    const int node = node_ids ? node_ids[warp] : warp;
    if (node < 0 || node >= t.n_nodes) return;
    const size_t row = (size_t)node * t.pitch;
    const uint32_t* mask = t.legal_bits + (size_t)node * t.mask_words;
    const float* pol = policy + (size_t)warp * policy_size;
    for (int s = lane; s < t.pitch; s += 32) {
        float p = 0.0f;
        if (s < t.n_children && ((mask[s >> 5] >> (s & 31)) & 1u)) {
            const int a = slot_action ? slot_action[row + s] : s;
            // out-of-range actions get the reference's small default
            p = (a >= 0 && a < policy_size) ? fminf(1.0f, fmaxf(0.0f, pol[a])) : 0.01f;
        }
        t.P[row + s] = p;
    }
}

// One warp per tree, simulations of a tree in sequence so that each sees the
// virtual loss left by the ones before it.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
traverse_kernel(ob200_tree_view t, const int32_t* __restrict__ roots, int n_trees,
                int sims_per_tree, float c_puct, int vl_value, int max_depth,
                int32_t* __restrict__ paths_out, int32_t* __restrict__ path_len_out) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_trees) return;
    const int root = roots[warp];
    for (int k = 0; k < sims_per_tree; ++k) {
        const size_t sim = (size_t)warp * sims_per_tree + k;
        int32_t* path = paths_out + sim * max_depth * 2;
        int node = root, depth = 0;
        while (depth < max_depth && node >= 0 && node < t.n_nodes) {
            const int sel = select_row<false>(t, node, c_puct, lane);
            if (sel < 0) break;
            int next = -1;
            if (lane == 0) {
                const size_t e = (size_t)node * t.pitch + sel;
                if (vl_value > 0) atomicAdd(t.VL + e, vl_value);
                path[2 * depth] = node;
                path[2 * depth + 1] = sel;
                next = t.child_node ? __ldcg(t.child_node + e) : -1;
            }
            __threadfence();
            next = __shfl_sync(0xffffffffu, next, 0);
            ++depth;
            node = next;
        }
        if (lane == 0) path_len_out[sim] = depth;
        __syncwarp();
    }
}

int check_view(const ob200_tree_view* t, const char* who) {
    if (!t) return set_error(OB200_ERR_INVALID, "%s: null tree view", who);
    if (!t->N || !t->W || !t->P || !t->VL || !t->legal_bits || !t->node_visits)
        return set_error(OB200_ERR_INVALID, "%s: null array in tree view", who);
    if (t->n_nodes < 0 || t->n_children <= 0 || t->pitch < t->n_children || (t->pitch & 3) ||
        t->mask_words * 32 < t->pitch)
        return set_error(OB200_ERR_INVALID,
                         "%s: bad geometry (n_nodes %d, n_children %d, pitch %d must be a multiple of 4 and >= n_children, mask_words %d must cover pitch)",
                         who, t->n_nodes, t->n_children, t->pitch, t->mask_words);
    if (((uintptr_t)t->N | (uintptr_t)t->W | (uintptr_t)t->P | (uintptr_t)t->VL) & 15)
        return set_error(OB200_ERR_INVALID, "%s: N/W/P/VL must be 16-byte aligned", who);
    return OB200_OK;
}

}  // namespace
}  // namespace ob200

using namespace ob200;

extern "C" {

int ob200_launch_puct_select(const ob200_tree_view* tree, const int32_t* node_ids, int32_t n,
                             float c_puct, int32_t vl_value, int32_t apply_vl, int32_t* sel_out,
                             ob200_stream stream) {
    if (int rc = check_view(tree, "ob200_launch_puct_select")) return rc;
    if (n == 0) return OB200_OK;
    if (n < 0 || (!node_ids && n > tree->n_nodes) || !sel_out)
        return set_error(OB200_ERR_INVALID, "ob200_launch_puct_select: bad n (%d) or null output", n);
    if (int rc = require_device()) return rc;
    const int blocks = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
    puct_select_kernel<<<blocks, kWarpsPerBlock * 32, 0, as_stream(stream)>>>(*tree, node_ids, n, c_puct, vl_value,
                                                                             apply_vl, sel_out);
    OB200_LAUNCHED("puct_select_kernel");
    counters().selections.fetch_add((uint64_t)n, std::memory_order_relaxed);
    return OB200_OK;
}

int ob200_launch_vl_apply(const ob200_tree_view* tree, const int32_t* node_ids, const int32_t* sel,
                          int32_t n, int32_t vl_value, ob200_stream stream) {
    if (int rc = check_view(tree, "ob200_launch_vl_apply")) return rc;
    if (n < 0 || !sel) return set_error(OB200_ERR_INVALID, "ob200_launch_vl_apply: bad arguments");
    if (int rc = require_device()) return rc;
    if (n == 0 || vl_value <= 0) return OB200_OK;   // the reference ignores amount <= 0
    vl_apply_kernel<<<(n + 255) / 256, 256, 0, as_stream(stream)>>>(*tree, node_ids, sel, n, vl_value);
    OB200_LAUNCHED("vl_apply_kernel");
    return OB200_OK;
}

int ob200_launch_vl_revert(const ob200_tree_view* tree, const int32_t* node_ids, const int32_t* sel,
                           int32_t n, int32_t vl_value, ob200_stream stream) {
    if (int rc = check_view(tree, "ob200_launch_vl_revert")) return rc;
    if (n < 0 || !sel) return set_error(OB200_ERR_INVALID, "ob200_launch_vl_revert: bad arguments");
    if (int rc = require_device()) return rc;
    if (n == 0 || vl_value <= 0) return OB200_OK;
    vl_revert_kernel<<<(n + 255) / 256, 256, 0, as_stream(stream)>>>(*tree, node_ids, sel, n, vl_value);
    OB200_LAUNCHED("vl_revert_kernel");
    return OB200_OK;
}

int ob200_launch_backup(const ob200_tree_view* tree, const int32_t* paths, const int32_t* path_len,
                        const float* leaf_values, int32_t n, int32_t max_depth, int32_t vl_value,
                        ob200_stream stream) {
    if (int rc = check_view(tree, "ob200_launch_backup")) return rc;
    if (n < 0 || max_depth <= 0 || !paths || !path_len || !leaf_values)
        return set_error(OB200_ERR_INVALID, "ob200_launch_backup: bad arguments");
    if (int rc = require_device()) return rc;
    if (n == 0) return OB200_OK;
    backup_kernel<<<(n + 127) / 128, 128, 0, as_stream(stream)>>>(*tree, paths, path_len, leaf_values, n, max_depth,
                                                                  vl_value);
    OB200_LAUNCHED("backup_kernel");
    counters().backups.fetch_add((uint64_t)n, std::memory_order_relaxed);
    return OB200_OK;
}

int ob200_launch_set_priors(const ob200_tree_view* tree, const int32_t* node_ids, int32_t n,
                            const float* policy, int32_t policy_size, const int32_t* slot_action,
                            ob200_stream stream) {
    if (int rc = check_view(tree, "ob200_launch_set_priors")) return rc;
    if (n < 0 || !policy || policy_size <= 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_set_priors: bad arguments");
    if (int rc = require_device()) return rc;
    if (n == 0) return OB200_OK;
    const int blocks = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
    set_priors_kernel<<<blocks, kWarpsPerBlock * 32, 0, as_stream(stream)>>>(*tree, node_ids, n, policy, policy_size,
                                                                            slot_action);
    OB200_LAUNCHED("set_priors_kernel");
    return OB200_OK;
}

int ob200_launch_traverse(const ob200_tree_view* tree, const int32_t* roots, int32_t n_trees,
                          int32_t sims_per_tree, float c_puct, int32_t vl_value, int32_t max_depth,
                          int32_t* paths_out, int32_t* path_len_out, ob200_stream stream) {
    if (int rc = check_view(tree, "ob200_launch_traverse")) return rc;
    if (n_trees < 0 || sims_per_tree <= 0 || max_depth <= 0 || !roots || !paths_out || !path_len_out)
        return set_error(OB200_ERR_INVALID, "ob200_launch_traverse: bad arguments");
    if (int rc = require_device()) return rc;
    if (n_trees == 0) return OB200_OK;
    // one warp per block: trees are few and latency-bound, so spread them over the SMs
    traverse_kernel<<<n_trees, 32, 0, as_stream(stream)>>>(*tree, roots, n_trees, sims_per_tree, c_puct,
                                                                          vl_value, max_depth, paths_out, path_len_out);
    OB200_LAUNCHED("traverse_kernel");
    counters().selections.fetch_add((uint64_t)n_trees * sims_per_tree, std::memory_order_relaxed);
    return OB200_OK;
}

}  // extern "C"
