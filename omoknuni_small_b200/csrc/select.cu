// Batched PUCT selection, virtual loss, backup and prior scatter over
// structure-of-arrays edge statistics (sm_100a).
//
// Rows are `pitch` (multiple of 4) elements.  Scores use IEEE round-to-nearest
// intrinsics in the operation order of MCTSNode::selectChild (reference
// src/mcts/mcts_node.cpp:143-167), so no FMA contraction or fast-math can
// change a comparison; the kernels that bracket scores with reciprocals first
// evaluate that expression for every slot that can hold the maximum, and the
// combine rule keeps the lowest slot on equal scores.  Three selection kernels:
//   puct_select_kernel            a warp per row, 128-bit loads (small launches, any width);
//   puct_select_staged_kernel     a warp per row of up to 256 slots, rows staged in shared
//                                 memory through per-warp rings of bulk async copies;
//   puct_select_segmented_kernel  wider rows cut into 256-slot segments through the same rings,
//                                 a 64-bit atomic maximum per row, puct_select_finish_kernel.
// Then the virtual-loss kernels, backup, prior scatter, and the wavefront descent (traverse_kernel).
#include "internal.h"
#include <cfloat>
#include <map>
#include <mutex>
#include <type_traits>
#include <utility>

namespace ob200 {
namespace {

constexpr int kWarpsPerBlock = 8;

struct Best {
    float score;   // best score seen with strict '>' starting from -inf
    int idx;       // its slot, -1 when nothing compared greater than -inf
};

__device__ __forceinline__ float puct_score(int n, float w, float p, int vl, float explore) {
    const int ev = n + vl;
    const float evf = (float)ev;
    const float q = ev > 0 ? __fdiv_rn(__fsub_rn(w, (float)vl), evf) : 0.0f;
    const float u = __fdiv_rn(__fmul_rn(p, explore), __fadd_rn(1.0f, evf));
    return __fadd_rn(q, u);
}

// Branch-free per slot: a slot that does not exist scores -inf, which the strict
// '>' never takes (the reference never sees such a slot at all).
__device__ __forceinline__ void consider(Best& b, int slot, bool legal, int n, float w, float p, int vl,
                                         float explore) {
    float s = puct_score(n, w, p, vl, explore);
    s = legal ? s : -INFINITY;
    if (s > b.score) { b.score = s; b.idx = slot; }
}

__device__ __forceinline__ Best warp_combine(Best b) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, b.score, off);
        const int oi = __shfl_xor_sync(0xffffffffu, b.idx, off);
        if (oi >= 0 && (b.idx < 0 || os > b.score || (os == b.score && oi < b.idx))) {
            b.score = os; b.idx = oi;
        }
    }
    return b;
}

// The reference's fallback when no score compared greater than -inf (all NaN or
// -inf): the least-visited existing child, first one on ties
// (src/mcts/mcts_node.cpp:173-181).  Rare, so it is a second scan of N only.
__device__ __noinline__ int least_visited_row(const int32_t* N, const uint32_t* mask, int n_children, int lane) {
    int mn = INT_MAX, mi = -1;
    for (int s = lane; s < n_children; s += 32)
        if ((mask[s >> 5] >> (s & 31)) & 1u) {
            const int n = N[s];
            if (n < mn) { mn = n; mi = s; }
        }
    for (int off = 16; off > 0; off >>= 1) {
        const int on = __shfl_xor_sync(0xffffffffu, mn, off);
        const int om = __shfl_xor_sync(0xffffffffu, mi, off);
        if (om >= 0 && (mi < 0 || on < mn || (on == mn && om < mi))) { mn = on; mi = om; }
    }
    return mi;
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

    Best b{-INFINITY, -1};
    for (int v0 = 0; v0 < nvec; v0 += 64) {
        // two independent load rounds in flight per lane; out-of-range lanes re-read vector 0
        // with an empty mask, so that the arithmetic below has no branches
        const int va = v0 + lane, vb = v0 + 32 + lane;
        const bool ha = va < nvec, hb = vb < nvec;
        const int ia = ha ? va : 0, ib = hb ? vb : 0;
        const int4 na = kStream ? __ldcs(N4 + ia) : __ldcg(N4 + ia);
        const float4 wa = kStream ? __ldcs(W4 + ia) : __ldcg(W4 + ia);
        const float4 pa = kStream ? __ldcs(P4 + ia) : __ldcg(P4 + ia);
        const int4 la = __ldcg(V4 + ia);
        const int4 nb = kStream ? __ldcs(N4 + ib) : __ldcg(N4 + ib);
        const float4 wb = kStream ? __ldcs(W4 + ib) : __ldcg(W4 + ib);
        const float4 pb = kStream ? __ldcs(P4 + ib) : __ldcg(P4 + ib);
        const int4 lb = __ldcg(V4 + ib);
        const uint32_t ma = ha ? (__ldg(mask + (ia >> 3)) >> ((ia & 7) * 4)) & 0xFu : 0u;
        const uint32_t mb = hb ? (__ldg(mask + (ib >> 3)) >> ((ib & 7) * 4)) & 0xFu : 0u;
        const int sa = va * 4, sb = vb * 4;
        consider(b, sa + 0, ma & 1u, na.x, wa.x, pa.x, la.x, explore);
        consider(b, sa + 1, ma & 2u, na.y, wa.y, pa.y, la.y, explore);
        consider(b, sa + 2, ma & 4u, na.z, wa.z, pa.z, la.z, explore);
        consider(b, sa + 3, ma & 8u, na.w, wa.w, pa.w, la.w, explore);
        consider(b, sb + 0, mb & 1u, nb.x, wb.x, pb.x, lb.x, explore);
        consider(b, sb + 1, mb & 2u, nb.y, wb.y, pb.y, lb.y, explore);
        consider(b, sb + 2, mb & 4u, nb.z, wb.z, pb.z, lb.z, explore);
        consider(b, sb + 3, mb & 8u, nb.w, wb.w, pb.w, lb.w, explore);
    }
    b = warp_combine(b);
    if (b.idx < 0)
        return least_visited_row(t.N + (size_t)node * t.pitch, t.legal_bits + (size_t)node * t.mask_words, t.n_children, lane);
    return b.idx;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32, 4)
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

// Cheap bracket of the score: one MUFU reciprocal per division instead of an IEEE
// divide.  rcp.approx is within 1 ulp, so with q~ = val * rcp(ev), u~ = (p*explore) *
// rcp(1 + ev) and m = |q~| + |u~| the exact score s (the reference's fp32 expression)
// satisfies |s - s~| < 2^-21 * m; kBracket = 2^-19 leaves a factor 4.  The staged kernel
// uses the bracket to find the few slots that can hold the maximum and evaluates only
// those with the exact expression, so the selected index is still bit-exact:
//   T = max over slots of (s~ - kBracket*m) <= max s,   and the reference's choice i*
//   (first slot attaining max s) has s~ + kBracket*m >= s_i* >= T, as has every slot tied
//   with it; the exact pass over { s~ + kBracket*m >= T } in slot order therefore sees
//   i* and everything that could beat or tie it.  NaN brackets compare false (never a
//   candidate, as NaN scores are never selected) and are ignored by the maximum.
constexpr float kBracket = 1.9073486328125e-06f;   // 2^-19

__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void bracket(int n, float w, float p, int vl, float explore, bool legal, float& lo,
                                        float& hi) {
    const int ev = n + vl;
    const float evf = (float)ev;
    const float q = ev > 0 ? __fmul_rn(__fsub_rn(w, (float)vl), rcp_approx(evf)) : 0.0f;
    const float u = __fmul_rn(__fmul_rn(p, explore), rcp_approx(__fadd_rn(1.0f, evf)));
    const float s = __fadd_rn(q, u);
    const float m = __fadd_rn(fabsf(q), fabsf(u));
    lo = legal ? fmaf(-kBracket, m, s) : -INFINITY;
    hi = legal ? fmaf(kBracket, m, s) : -INFINITY;
}

constexpr int kWideMinPitch = 1024;          // rows at least this wide always take the segmented kernel
constexpr long long kSegMinItems = 24576;    // narrower rows (257-1,023 slots) take it from this many segments on

// ---------------------------------------------------------------------------
// Staged variant for rows of up to 256 slots: a persistent grid, every warp
// walks its own list of nodes and keeps a three-deep ring of rows in shared
// memory, filled by 1-D bulk async copies (one per array row, completion on an
// mbarrier).  The copies of the next two nodes are in flight while the current one
// is scored from shared memory, so HBM latency is hidden by the ring instead of
// by occupancy, and the registers are free for the arithmetic.
// ---------------------------------------------------------------------------
constexpr int kStagedWarps = 20;
constexpr int kStagedDepth = 3;
constexpr int kStagedMaxPitch = 256;
constexpr uint32_t kStagedSpin = 1u << 24;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kStagedSpin; ++i) {
        uint32_t ok;
        // the hint lets the hardware park the thread for up to ~1 us instead of spinning
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 1000;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void row_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(kStagedWarps * 32, 1)
puct_select_staged_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids, int n, float c_puct,
                          int vl_value, int apply_vl, int32_t* __restrict__ sel_out, int* error_word) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_bytes = t.pitch * 4, mask_bytes = t.mask_words * 4;
    const int stage_bytes = (4 * row_bytes + mask_bytes + 127) & ~127;
    uint8_t* ring = smem + (size_t)warp * kStagedDepth * stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStagedWarps * kStagedDepth * stage_bytes) + warp * kStagedDepth;
    if (lane == 0) {
        for (int d = 0; d < kStagedDepth; ++d)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(bars + d)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // launched as a programmatic dependent: the set-up above may run while the kernel ahead in the stream (the
    // previous pass's revert) finishes; its writes are visible from here on
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // a kernel launched behind this one with programmatic stream serialization (the virtual-loss revert) may be
    // scheduled from now on; it waits for this grid's completion before it reads anything
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int total_warps = gridDim.x * kStagedWarps;
    const int first = blockIdx.x * kStagedWarps + warp;
    const int nvec = t.pitch >> 2;

    // Lanes 0-4 each issue one of the five row copies of a node; lane 0 also posts the byte
    // count (a copy that completes before the count is posted only drives the pending byte
    // count negative; the phase cannot complete before lane 0's arrival).
    auto fetch = [&](int i, int stage) {       // call with lanes 0-4
        const int node = node_ids ? node_ids[i] : i;
        if (node < 0 || node >= t.n_nodes) return;     // nothing to copy; the consumer skips it too
        const uint32_t bar = s_u32(bars + stage);
        const uint32_t dst = s_u32(ring + (size_t)stage * stage_bytes);
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(4 * row_bytes + mask_bytes)) : "memory");
        const size_t off = (size_t)node * t.pitch;
        const void* src = lane == 0 ? (const void*)(t.N + off) : lane == 1 ? (const void*)(t.W + off)
                        : lane == 2 ? (const void*)(t.P + off) : lane == 3 ? (const void*)(t.VL + off)
                                    : (const void*)(t.legal_bits + (size_t)node * t.mask_words);
        row_copy(dst + lane * row_bytes, src, lane == 4 ? mask_bytes : row_bytes, bar);
    };

    // node id and node visit count travel in a small register queue, loaded when the
    // node's rows are requested, so that no global load sits between a full barrier and
    // the arithmetic
    int q_node[kStagedDepth - 1], q_visits[kStagedDepth - 1];
    auto lookup = [&](int i, int& node, int& visits) {
        node = -1; visits = 0;
        if (i < n) {
            node = node_ids ? __ldg(node_ids + i) : i;
            if (node < 0 || node >= t.n_nodes) node = -1;
            else visits = __ldg(t.node_visits + node);
        }
    };
#pragma unroll
    for (int d = 0; d < kStagedDepth - 1; ++d) {
        lookup(first + d * total_warps, q_node[d], q_visits[d]);
        if (first + d * total_warps < n && lane < 5) fetch(first + d * total_warps, d);
    }
    uint32_t phase_bits = 0;                   // one parity bit per stage
    int k = 0;
    for (int i = first; i < n; i += total_warps, ++k) {
        const int stage = k % kStagedDepth;
        const int nxt = i + (kStagedDepth - 1) * total_warps;
        __syncwarp();                           // every lane is done reading the stage about to be refilled
        if (nxt < n && lane < 5) fetch(nxt, (k + kStagedDepth - 1) % kStagedDepth);
        const int node = q_node[0];
        const int visits = q_visits[0];
#pragma unroll
        for (int d = 0; d + 1 < kStagedDepth - 1; ++d) { q_node[d] = q_node[d + 1]; q_visits[d] = q_visits[d + 1]; }
        lookup(nxt, q_node[kStagedDepth - 2], q_visits[kStagedDepth - 2]);
        int sel = -1;
        if (node >= 0) {
            const float explore = __fmul_rn(c_puct, __fsqrt_rn((float)visits));
            if (!bar_wait(s_u32(bars + stage), (phase_bits >> stage) & 1u)) {
                if (lane == 0) atomicExch(error_word, 4);
                break;
            }
            phase_bits ^= 1u << stage;
            const uint8_t* st = ring + (size_t)stage * stage_bytes;
            const int4* N4 = reinterpret_cast<const int4*>(st);
            const float4* W4 = reinterpret_cast<const float4*>(st + row_bytes);
            const float4* P4 = reinterpret_cast<const float4*>(st + 2 * row_bytes);
            const int4* V4 = reinterpret_cast<const int4*>(st + 3 * row_bytes);
            const uint32_t* mask = reinterpret_cast<const uint32_t*>(st + 4 * row_bytes);
            // pass 1: brackets of this lane's slots (rows of <= 256 slots: two vectors a lane)
            float hi[8];
            float lane_lo = -INFINITY;
            uint32_t legal8 = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int v = lane + 32 * h;
                const bool in = v < nvec;
                const int vi = in ? v : 0;
                const int4 nn = N4[vi]; const float4 ww = W4[vi]; const float4 pp = P4[vi]; const int4 ll = V4[vi];
                const uint32_t m = in ? (mask[vi >> 3] >> ((vi & 7) * 4)) & 0xFu : 0u;
                legal8 |= m << (4 * h);
                float lo;
                bracket(nn.x, ww.x, pp.x, ll.x, explore, m & 1u, lo, hi[4 * h + 0]); lane_lo = fmaxf(lane_lo, lo);
                bracket(nn.y, ww.y, pp.y, ll.y, explore, m & 2u, lo, hi[4 * h + 1]); lane_lo = fmaxf(lane_lo, lo);
                bracket(nn.z, ww.z, pp.z, ll.z, explore, m & 4u, lo, hi[4 * h + 2]); lane_lo = fmaxf(lane_lo, lo);
                bracket(nn.w, ww.w, pp.w, ll.w, explore, m & 8u, lo, hi[4 * h + 3]); lane_lo = fmaxf(lane_lo, lo);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) lane_lo = fmaxf(lane_lo, __shfl_xor_sync(0xffffffffu, lane_lo, off));
            // pass 2: the slots whose bracket reaches the best lower bound.  Usually there is
            // exactly one, and with a finite bound it is the answer without any exact score.
            uint32_t cand = 0;
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) cand |= (uint32_t)(((legal8 >> k2) & 1u) && hi[k2] >= lane_lo) << k2;
            const uint32_t lanes_with = __ballot_sync(0xffffffffu, cand != 0);
            const uint32_t lanes_multi = __ballot_sync(0xffffffffu, (cand & (cand - 1)) != 0);
            Best b{-INFINITY, -1};
            if (__popc(lanes_with) == 1 && lanes_multi == 0 && lane_lo > -INFINITY) {
                const int k2 = __ffs(cand) - 1;                       // valid on the owning lane only
                const int slot = (lane + 32 * (k2 >> 2)) * 4 + (k2 & 3);
                b.idx = __shfl_sync(0xffffffffu, slot, __ffs(lanes_with) - 1);
            } else {
                const int32_t* Ns = reinterpret_cast<const int32_t*>(N4);
                const float* Ws = reinterpret_cast<const float*>(W4);
                const float* Ps = reinterpret_cast<const float*>(P4);
                const int32_t* Vs = reinterpret_cast<const int32_t*>(V4);
#pragma unroll
                for (int k2 = 0; k2 < 8; ++k2) {
                    if ((cand >> k2) & 1u) {
                        const int slot = (lane + 32 * (k2 >> 2)) * 4 + (k2 & 3);
                        const float sc = puct_score(Ns[slot], Ws[slot], Ps[slot], Vs[slot], explore);
                        if (sc > b.score) { b.score = sc; b.idx = slot; }
                    }
                }
                b = warp_combine(b);
            }
            sel = b.idx >= 0 ? b.idx
                             : least_visited_row(t.N + (size_t)node * t.pitch, t.legal_bits + (size_t)node * t.mask_words,
                                                 t.n_children, lane);
        }
        if (lane == 0) {
            sel_out[i] = sel;
            if (sel >= 0 && apply_vl && vl_value > 0) atomicAdd(t.VL + (size_t)node * t.pitch + sel, vl_value);
        }
    }
}

// ---------------------------------------------------------------------------
// Wide rows (chess: 4,672 children = 75 KB of statistics per node), segmented: a node's row is cut into segments
// of 256 slots and every (node, segment) pair is one work item of the staged design above - a warp per item, a
// three-deep ring of 4 KB segments per warp filled by bulk async copies - so the bytes stream at the rate of the
// narrow-row kernel.  A segment yields its exact maximum (score, lowest slot) and folds it into the node's 64-bit
// word of scratch with one atomic maximum: order-preserving bits of the score above the complemented slot, so the
// largest word is the largest score and, among equals, the lowest slot.  A second small kernel (one thread per
// node, started as a programmatic dependent) turns the word into the selection, applies the virtual loss and
// zeroes the word for the next launch.  The maximum of the segments' exact maxima is the row's exact maximum, so
// the choice is the reference's bit for bit.
// ---------------------------------------------------------------------------
// The approximate score of one slot (see bracket() for the error bound), folded into the lane's running maximum
// of the existing slots' scores and of the error scale m.  A NaN score is never a candidate and fmaxf ignores it.
// MAGIC converts the two counts to fp32 with an integer add and a subtraction of 2^23 (exact for 0 <= x < 2^23)
// instead of two conversion instructions, which share the quarter-rate unit with the reciprocals; `range`
// collects the bits of every count so that the caller can tell when a count was outside that range.
template <bool MAGIC>
__device__ __forceinline__ void approx_score(int n, float w, float p, int vl, float explore, bool exists, float& s_out,
                                             float& lane_s, float& lane_m, uint32_t& range) {
    const int ev = n + vl;
    float evf, vlf, d2;
    if (MAGIC) {
        evf = __fsub_rn(__int_as_float(ev + 0x4B000000), 8388608.0f);
        vlf = __fsub_rn(__int_as_float(vl + 0x4B000000), 8388608.0f);
        d2 = __fsub_rn(__int_as_float(ev + 0x4B000001), 8388608.0f);
        range |= (uint32_t)ev | (uint32_t)vl;
    } else {
        evf = (float)ev; vlf = (float)vl; d2 = __fadd_rn(1.0f, evf);
    }
    const float q = ev > 0 ? __fmul_rn(__fsub_rn(w, vlf), rcp_approx(evf)) : 0.0f;
    const float u = __fmul_rn(__fmul_rn(p, explore), rcp_approx(d2));
    const float s = __fadd_rn(q, u);
    s_out = s;
    if (exists) { lane_s = fmaxf(lane_s, s); lane_m = fmaxf(lane_m, __fadd_rn(fabsf(q), fabsf(u))); }
}
constexpr int kSegSlots = 256;
#ifndef OB200_SEG_WARPS
#define OB200_SEG_WARPS 27
#define OB200_SEG_DEPTH 2
#endif
constexpr int kSegWarps = OB200_SEG_WARPS;   // warps x stages x 4 KB <= 216 KB of shared memory
constexpr int kSegDepth = OB200_SEG_DEPTH;
// fp32 -> unsigned bits with the same order (-0 < +0, which no comparison here depends on)
__device__ __forceinline__ uint32_t order_bits(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__global__ void __launch_bounds__(kSegWarps * 32, 1)
puct_select_segmented_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids, int n, int segs, float c_puct,
                             unsigned long long* __restrict__ best_word, int* error_word) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kRowBytes = kSegSlots * 4;
    constexpr int kStageBytes = 4 * kRowBytes;
    uint8_t* ring = smem + (size_t)warp * kSegDepth * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kSegWarps * kSegDepth * kStageBytes) + warp * kSegDepth;
    if (lane == 0) {
        for (int d = 0; d < kSegDepth; ++d)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(bars + d)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // launched as a programmatic dependent: the set-up above may run while the kernel ahead in the stream (the
    // previous pass's revert) finishes; its writes are visible from here on
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // A warp takes a contiguous run of (entry, segment) pairs, so most steps stay on the same node: its id and visit
    // count are looked up once per node, and the best of the node's segments seen by this warp is folded into the
    // node's word once.  (Handing the runs out through a counter instead measured slower: 38.6 to 44.9 us against
    // 34.2 us for 2,048 rows of 4,672, the fewer the runs per warp the worse.)
    const int total_warps = gridDim.x * kSegWarps;
    const int w_index = blockIdx.x * kSegWarps + warp;
    const long long items = (long long)n * segs;
    const int base_items = (int)(items / total_warps), extra = (int)(items - (long long)base_items * total_warps);
    const long long first = (long long)w_index * base_items + min(w_index, extra);
    int to_look_up = base_items + (w_index < extra ? 1 : 0);
    struct Item { int entry, seg, node, slots, visits; uint32_t bits; };
    int nx_entry = (int)(first / segs), nx_seg = (int)(first - (long long)nx_entry * segs);      // the next pair to look up
    int c_entry = -1, c_node = -1, c_visits = 0;
    int ahead_node = node_ids && nx_entry < n ? __ldg(node_ids + nx_entry) : nx_entry;      // node id of entry nx_entry
    const int mask_lane = lane >> 3, mask_shift = (lane & 7) * 4;
    auto lookup = [&]() {
        Item a{n, 0, -1, 0, 0, 0u};
        if (to_look_up <= 0) return a;
        --to_look_up;
        a.entry = nx_entry; a.seg = nx_seg;
        if (++nx_seg == segs) { nx_seg = 0; ++nx_entry; }
        if (a.entry != c_entry) {                 // a new node: its id was requested one node ahead, its visit count
            c_entry = a.entry;                    // is not needed before the segment is scored
            const int node = ahead_node;
            ahead_node = node_ids && a.entry + 1 < n ? __ldg(node_ids + a.entry + 1) : a.entry + 1;
            c_node = (node >= 0 && node < t.n_nodes) ? node : -1;
            if (c_node >= 0) c_visits = __ldg(t.node_visits + c_node);
        }
        if (c_node < 0) return a;
        a.node = c_node; a.visits = c_visits;
        a.slots = min(kSegSlots, t.pitch - a.seg * kSegSlots);
        // vectors lane and lane + 32 of the segment: four existence bits each, from the node's mask row (eight
        // vectors a word, so the two words of a lane are four apart)
        const uint32_t* mask = t.legal_bits + (size_t)c_node * t.mask_words + a.seg * (kSegSlots / 32) + mask_lane;
        if (lane * 4 < a.slots) a.bits = (__ldg(mask) >> mask_shift) & 0xFu;
        if (lane * 4 + 128 < a.slots) a.bits |= ((__ldg(mask + 4) >> mask_shift) & 0xFu) << 4;
        return a;
    };
    auto fetch = [&](const Item& a, int stage) {       // call with lanes 0-3
        if (a.node < 0) return;
        const uint32_t bar = s_u32(bars + stage);
        const uint32_t dst = s_u32(ring + (size_t)stage * kStageBytes);
        const uint32_t bytes = (uint32_t)a.slots * 4;
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(4 * bytes) : "memory");
        const size_t off = (size_t)a.node * t.pitch + (size_t)a.seg * kSegSlots;
        const void* src = lane == 0 ? (const void*)(t.N + off) : lane == 1 ? (const void*)(t.W + off)
                        : lane == 2 ? (const void*)(t.P + off) : (const void*)(t.VL + off);
        row_copy(dst + lane * kRowBytes, src, bytes, bar);
    };
    Best nb{-INFINITY, -1};                       // best of the current entry's segments so far (slot within the row)
    int nb_entry = -1;
    float explore = 0.0f;                         // c_puct * sqrt(visits) of that entry's node
    auto flush = [&]() {
        // + 0.0f turns -0 into +0: the two compare equal in the reference and must not be ordered by their bits
        if (lane == 0 && nb.idx >= 0)
            atomicMax(best_word + nb_entry, ((unsigned long long)order_bits(__fadd_rn(nb.score, 0.0f)) << 32) | (uint32_t)~(uint32_t)nb.idx);
        nb.score = -INFINITY; nb.idx = -1;
    };
    Item q[kSegDepth - 1];
#pragma unroll
    for (int d = 0; d < kSegDepth - 1; ++d) {
        q[d] = lookup();
        if (lane < 4) fetch(q[d], d);
    }
    uint32_t phase_bits = 0;
    for (int k = 0;; ++k) {
        const int stage = k % kSegDepth;
        __syncwarp();                           // every lane is done reading the stage about to be refilled
        const Item cur = q[0];
        if (cur.entry >= n) break;
#pragma unroll
        for (int d = 0; d + 1 < kSegDepth - 1; ++d) q[d] = q[d + 1];
        q[kSegDepth - 2] = lookup();
        if (lane < 4) fetch(q[kSegDepth - 2], (k + kSegDepth - 1) % kSegDepth);
        if (cur.node < 0) continue;               // the finishing kernel reports -1 for an entry that names no node
        if (cur.entry != nb_entry) {
            flush();
            nb_entry = cur.entry;
            explore = __fmul_rn(c_puct, __fsqrt_rn((float)cur.visits));
        }
        if (!bar_wait(s_u32(bars + stage), (phase_bits >> stage) & 1u)) {
            if (lane == 0) atomicExch(error_word, 4);
            break;
        }
        phase_bits ^= 1u << stage;
        const uint8_t* st = ring + (size_t)stage * kStageBytes;
        const int4* N4 = reinterpret_cast<const int4*>(st);
        const float4* W4 = reinterpret_cast<const float4*>(st + kRowBytes);
        const float4* P4 = reinterpret_cast<const float4*>(st + 2 * kRowBytes);
        const int4* V4 = reinterpret_cast<const int4*>(st + 3 * kRowBytes);
        // Approximate scores s~ (one MUFU reciprocal per division) with |s - s~| < kBracket * m, m = |q~| + |u~|;
        // M = the largest m of the segment bounds every slot's error, so the segment's exact maximum is attained
        // among the slots with s~ >= max s~ - 2 kBracket M.
        float sc[8];
        float lane_s = -INFINITY, lane_m = 0.0f;
        uint32_t range = 0;
        auto scores = [&](auto magic) {
            constexpr bool kMagic = decltype(magic)::value;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t m = (cur.bits >> (4 * h)) & 0xFu;
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[4 * h + j] = -INFINITY;
                if (m) {                          // a vector without an existing child (most of a chess row) costs nothing
                    const int v = lane + 32 * h;
                    const int4 nn = N4[v]; const float4 ww = W4[v]; const float4 pp = P4[v]; const int4 ll = V4[v];
                    approx_score<kMagic>(nn.x, ww.x, pp.x, ll.x, explore, m & 1u, sc[4 * h + 0], lane_s, lane_m, range);
                    approx_score<kMagic>(nn.y, ww.y, pp.y, ll.y, explore, m & 2u, sc[4 * h + 1], lane_s, lane_m, range);
                    approx_score<kMagic>(nn.z, ww.z, pp.z, ll.z, explore, m & 4u, sc[4 * h + 2], lane_s, lane_m, range);
                    approx_score<kMagic>(nn.w, ww.w, pp.w, ll.w, explore, m & 8u, sc[4 * h + 3], lane_s, lane_m, range);
                }
            }
        };
        scores(std::true_type{});
        if (__any_sync(0xffffffffu, range >> 23)) {       // a count beyond 2^23 or negative: the conversions proper
            lane_s = -INFINITY; lane_m = 0.0f;
            scores(std::false_type{});
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            lane_s = fmaxf(lane_s, __shfl_xor_sync(0xffffffffu, lane_s, off));
            lane_m = fmaxf(lane_m, __shfl_xor_sync(0xffffffffu, lane_m, off));
        }
        float thr = fmaf(-2.0f * kBracket, lane_m, lane_s);
        thr = thr == thr ? thr : -INFINITY;       // inf - inf: no usable bound, every existing slot is a candidate
        uint32_t cand = 0;
#pragma unroll
        for (int k2 = 0; k2 < 8; ++k2) cand |= (uint32_t)(sc[k2] >= thr) << k2;
        cand &= cur.bits;
        const int32_t* Ns = reinterpret_cast<const int32_t*>(N4);
        const float* Ws = reinterpret_cast<const float*>(W4);
        const float* Ps = reinterpret_cast<const float*>(P4);
        const int32_t* Vs = reinterpret_cast<const int32_t*>(V4);
        // the exact expression for the candidates (usually one or two of the 256), by the whole warp at once
        uint32_t lanes = __ballot_sync(0xffffffffu, cand != 0);
        while (lanes) {
            const int l = __ffs(lanes) - 1;
            lanes &= lanes - 1;
            uint32_t c = __shfl_sync(0xffffffffu, cand, l);
            while (c) {
                const int k2 = __ffs(c) - 1;
                c &= c - 1;
                const int slot = (l + 32 * (k2 >> 2)) * 4 + (k2 & 3);
                const float e = puct_score(Ns[slot], Ws[slot], Ps[slot], Vs[slot], explore);
                const int row_slot = cur.seg * kSegSlots + slot;
                if (e > nb.score || (e == nb.score && row_slot < nb.idx)) { nb.score = e; nb.idx = row_slot; }
            }
        }
    }
    flush();
}

// One thread per entry of the launch: the node's word -> selection (lowest-visited existing child when no score
// was comparable, as the narrow-row kernels; rare, so it is a plain scan), virtual loss, word back to zero.
__global__ void __launch_bounds__(256)
puct_select_finish_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids, int n, int vl_value, int apply_vl,
                          int32_t* __restrict__ sel_out, unsigned long long* __restrict__ best_word) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int entry = (int)(blockIdx.x * (unsigned)blockDim.x + threadIdx.x);
    if (entry >= n) return;
    const int node = node_ids ? __ldg(node_ids + entry) : entry;
    const unsigned long long w = __ldcg(best_word + entry);
    int sel = -1;
    if (node >= 0 && node < t.n_nodes) {
        if (w) {
            sel = (int)~(uint32_t)w;
        } else {
            const int32_t* N = t.N + (size_t)node * t.pitch;
            const uint32_t* mask = t.legal_bits + (size_t)node * t.mask_words;
            int mn = INT_MAX;
            for (int s = 0; s < t.n_children; ++s)
                if (((mask[s >> 5] >> (s & 31)) & 1u) && N[s] < mn) { mn = N[s]; sel = s; }
        }
    }
    sel_out[entry] = sel;
    if (sel >= 0 && apply_vl && vl_value > 0) atomicAdd(t.VL + (size_t)node * t.pitch + sel, vl_value);
    if (w) best_word[entry] = 0ull;
}

// One 64-bit word per entry of a wide-row launch, zero between launches.  Launches on one stream are ordered, so
// the words are kept per (device, stream) and grown on demand; a stream's words are never freed (a few KB each).
static unsigned long long* wide_scratch(int dev, cudaStream_t stream, int n) {
    struct Slot { unsigned long long* p; int cap; };
    static std::mutex mu;
    static std::map<std::pair<int, cudaStream_t>, Slot> slots;
    std::lock_guard<std::mutex> lock(mu);
    Slot& s = slots[{dev, stream}];
    if (s.cap >= n) return s.p;
    // the old words may still be in use by launches in flight on this stream: release them in stream order
    if (s.p && cudaFreeAsync(s.p, stream) != cudaSuccess) return nullptr;
    s.p = nullptr; s.cap = 0;
    const int cap = n < 1024 ? 1024 : n;
    unsigned long long* p = nullptr;
    if (cudaMallocAsync(reinterpret_cast<void**>(&p), (size_t)cap * 8, stream) != cudaSuccess) return nullptr;
    if (cudaMemsetAsync(p, 0, (size_t)cap * 8, stream) != cudaSuccess) { cudaFreeAsync(p, stream); return nullptr; }
    s.p = p; s.cap = cap;
    return p;
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

// MCTSNode::removeVirtualLoss(int) as the reference writes it (src/mcts/mcts_node_virtual_loss.cpp:32-42, and its
// kernel src/mcts/gpu_virtual_loss_kernels.cu:123-129): subtract, and if the counter held less than the amount, put it
// back to zero.  One atomic round trip in the common case; reverts that meet on one counter end at the same value
// as in any sequential order (all of them subtract the same amount, and the zero is written last).
// Launched with programmatic stream serialization: its CTAs may be scheduled while the kernel ahead of it in the
// stream (the selection that produces `sel`) is still running, and wait here until that kernel's writes are visible.
__global__ void vl_revert_kernel(ob200_tree_view t, const int32_t* __restrict__ node_ids,
                                 const int32_t* __restrict__ sel, int n, int vl_value) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // the next selection may set itself up
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int node = node_ids ? node_ids[i] : i;
    const int s = sel[i];
    if (node < 0 || node >= t.n_nodes || s < 0 || s >= t.n_children) return;
    int32_t* addr = t.VL + (size_t)node * t.pitch + s;
    const int old = atomicSub(addr, vl_value);
    if (old < vl_value) atomicMax(addr, 0);
}

__global__ void backup_kernel(ob200_tree_view t, const int32_t* __restrict__ paths,
                              const int32_t* __restrict__ path_len,
                              const float* __restrict__ leaf_values, int n, int max_depth,
                              int vl_value) {
    OB200_PDL_ENTER();
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

// select_row for rows of at most 256 slots (two vectors a lane), as the descent uses it: approximate scores with one
// error scale for the row, the exact expression only for the slots that can hold the maximum (see approx_score and
// the segmented kernel above; the choice is the reference's bit for bit), instead of two IEEE divisions per slot.
__device__ __forceinline__ int select_row_narrow(const ob200_tree_view& t, int node, float c_puct, int lane) {
    const int nvec = t.pitch >> 2;
    const size_t row = (size_t)node * t.pitch;
    const int4* N4 = reinterpret_cast<const int4*>(t.N + row);
    const float4* W4 = reinterpret_cast<const float4*>(t.W + row);
    const float4* P4 = reinterpret_cast<const float4*>(t.P + row);
    const int4* V4 = reinterpret_cast<const int4*>(t.VL + row);
    const uint32_t* mask = t.legal_bits + (size_t)node * t.mask_words;
    const float explore = __fmul_rn(c_puct, __fsqrt_rn((float)t.node_visits[node]));
    int n8[8], l8[8];
    float w8[8], p8[8];
    uint32_t bits = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int v = lane + 32 * h;
        const bool have = v < nvec;
        const int vi = have ? v : 0;
        const int4 nn = __ldcg(N4 + vi);
        const float4 ww = __ldcg(W4 + vi);
        const float4 pp = __ldcg(P4 + vi);
        const int4 ll = __ldcg(V4 + vi);
        if (have) bits |= ((__ldg(mask + (vi >> 3)) >> ((vi & 7) * 4)) & 0xFu) << (4 * h);
        n8[4 * h] = nn.x; n8[4 * h + 1] = nn.y; n8[4 * h + 2] = nn.z; n8[4 * h + 3] = nn.w;
        w8[4 * h] = ww.x; w8[4 * h + 1] = ww.y; w8[4 * h + 2] = ww.z; w8[4 * h + 3] = ww.w;
        p8[4 * h] = pp.x; p8[4 * h + 1] = pp.y; p8[4 * h + 2] = pp.z; p8[4 * h + 3] = pp.w;
        l8[4 * h] = ll.x; l8[4 * h + 1] = ll.y; l8[4 * h + 2] = ll.z; l8[4 * h + 3] = ll.w;
    }
    float sc[8];
    float lane_s = -INFINITY, lane_m = 0.0f;
    uint32_t range = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) approx_score<true>(n8[k], w8[k], p8[k], l8[k], explore, (bits >> k) & 1u, sc[k], lane_s, lane_m, range);
    if (__any_sync(0xffffffffu, range >> 23)) {               // a count beyond 2^23 or negative: the conversions proper
        lane_s = -INFINITY; lane_m = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) approx_score<false>(n8[k], w8[k], p8[k], l8[k], explore, (bits >> k) & 1u, sc[k], lane_s, lane_m, range);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        lane_s = fmaxf(lane_s, __shfl_xor_sync(0xffffffffu, lane_s, off));
        lane_m = fmaxf(lane_m, __shfl_xor_sync(0xffffffffu, lane_m, off));
    }
    float thr = fmaf(-2.0f * kBracket, lane_m, lane_s);
    thr = thr == thr ? thr : -INFINITY;
    Best b{-INFINITY, -1};
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (((bits >> k) & 1u) && sc[k] >= thr) {
            const float e = puct_score(n8[k], w8[k], p8[k], l8[k], explore);
            if (e > b.score) { b.score = e; b.idx = (lane + 32 * (k >> 2)) * 4 + (k & 3); }
        }
    b = warp_combine(b);
    if (b.idx < 0)
        return least_visited_row(t.N + row, mask, t.n_children, lane);
    return b.idx;
}

// One CTA per tree.  Simulations of a tree are ordered: simulation k must see the virtual loss
// that simulations < k left on every edge it scores.  They still overlap as a wavefront: the CTA
// advances in steps, a simulation takes one level per step, and simulation k starts at least one
// step after simulation k - 1, so when k scores the edges at depth d, every earlier simulation
// has already passed depth d (virtual loss is per edge, and edges below depth d do not enter the
// scores at depth d).  sims + depth steps instead of sims x depth.  The order is the sequential
// one as long as a node is reached at one depth only (a tree; a game in which every move adds a
// stone): two simulations can then never be at the same node in the same step.
constexpr int kTravWarps = 16;
__global__ void __launch_bounds__(kTravWarps * 32)
traverse_kernel(ob200_tree_view t, const int32_t* __restrict__ roots, int n_trees,
                int sims_per_tree, float c_puct, int vl_value, int max_depth,
                int32_t* __restrict__ paths_out, int32_t* __restrict__ path_len_out) {
    __shared__ int n_started, n_finished;
    const int tree = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) { n_started = 0; n_finished = 0; }
    OB200_PDL_ENTER();
    __syncthreads();
    const int root = roots[tree];
    int k = -1;            // simulation this warp is running, -1 = idle
    int my_next = warp;    // next simulation this warp owns (k = warp mod kTravWarps)
    int depth = 0, node = -1;
    while (true) {
        const int started = n_started, finished = n_finished;
        if (finished >= sims_per_tree) break;
        bool start_now = false;
        if (k < 0 && my_next == started && my_next < sims_per_tree) {
            k = my_next; my_next += kTravWarps; depth = 0; node = root; start_now = true;
        }
        __syncthreads();   // every warp has read the counters before any warp updates them
        if (k >= 0) {
            const size_t sim = (size_t)tree * sims_per_tree + k;
            bool done = true;
            if (depth < max_depth && node >= 0 && node < t.n_nodes) {
                // the row of child links rides along with the statistics (rows of up to 256 slots: two 16-byte
                // vectors per lane), so that the descent does not pay a second trip to L2 once the slot is known
                const bool links_in_regs = t.child_node != nullptr && t.pitch <= 256 && ((uintptr_t)t.child_node & 15) == 0;
                int4 ca = make_int4(-1, -1, -1, -1), cb = ca;
                if (links_in_regs) {
                    const int4* C4 = reinterpret_cast<const int4*>(t.child_node + (size_t)node * t.pitch);
                    const int nvec = t.pitch >> 2;
                    if (lane < nvec) ca = __ldcg(C4 + lane);
                    if (lane + 32 < nvec) cb = __ldcg(C4 + 32 + lane);
                }
                const int sel = t.pitch <= 256 ? select_row_narrow(t, node, c_puct, lane) : select_row<false>(t, node, c_puct, lane);
                if (sel >= 0) {
                    int next = -1;
                    if (links_in_regs) {
                        const int4 c = (sel >> 7) ? cb : ca;          // vector sel / 4 sits in lane (sel / 4) % 32
                        const int e4 = sel & 3;
                        const int mine = e4 == 0 ? c.x : e4 == 1 ? c.y : e4 == 2 ? c.z : c.w;
                        next = __shfl_sync(0xffffffffu, mine, (sel >> 2) & 31);
                    }
                    if (lane == 0) {
                        const size_t e = (size_t)node * t.pitch + sel;
                        // the next reader of this counter is a warp of this CTA, after the barrier below
                        if (vl_value > 0) atomicAdd(t.VL + e, vl_value);
                        int32_t* path = paths_out + sim * max_depth * 2;
                        path[2 * depth] = node;
                        path[2 * depth + 1] = sel;
                        if (!links_in_regs) next = t.child_node ? __ldcg(t.child_node + e) : -1;
                    }
                    if (!links_in_regs) next = __shfl_sync(0xffffffffu, next, 0);
                    ++depth;
                    node = next;
                    done = !(depth < max_depth && node >= 0 && node < t.n_nodes);
                }
            }
            if (lane == 0) {
                if (done) { path_len_out[sim] = depth; atomicAdd(&n_finished, 1); }
                if (start_now) atomicAdd(&n_started, 1);
            }
            if (done) k = -1;
        }
        __syncthreads();
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
    const int stage_bytes = (4 * tree->pitch * 4 + tree->mask_words * 4 + 127) & ~127;
    const int staged_smem = kStagedWarps * kStagedDepth * stage_bytes + kStagedWarps * kStagedDepth * 8;
    // the staged kernel fetches every row, the mask row included, with 16-byte-granular bulk copies: a mask array
    // that is not 16-byte aligned (a slice of a larger buffer) takes the direct kernel instead
    const bool mask_aligned = ((uintptr_t)tree->legal_bits & 15) == 0;
    if (tree->pitch <= kStagedMaxPitch && (tree->mask_words & 3) == 0 && mask_aligned && n >= 1024 && staged_smem <= 227 * 1024) {
        // rows small enough to ring-buffer in shared memory: persistent staged kernel
        int dev = 0, sms = 0;
        OB200_CUDA_OK(cudaGetDevice(&dev));
        OB200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        const int smem = staged_smem;
        static int configured[64] = {0};
        if (dev >= 0 && dev < 64 && configured[dev] < smem) {
            OB200_CUDA_OK(cudaFuncSetAttribute(puct_select_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            configured[dev] = smem;
        }
        int* errw = device_error_word();
        if (!errw) return set_error(OB200_ERR_CUDA, "ob200_launch_puct_select: cannot resolve the device error word");
        const int want = (n + kStagedWarps - 1) / kStagedWarps;
        cudaLaunchAttribute pdl[1];
        pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pdl[0].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3((unsigned)(want < sms ? want : sms));
        lc.blockDim = dim3(kStagedWarps * 32);
        lc.dynamicSmemBytes = (size_t)smem;
        lc.stream = as_stream(stream);
        lc.attrs = pdl;
        lc.numAttrs = 1;
        OB200_CUDA_OK(cudaLaunchKernelEx(&lc, puct_select_staged_kernel, *tree, node_ids, n, c_puct, vl_value, apply_vl, sel_out, errw));
        counters().launches.fetch_add(1, std::memory_order_relaxed);
    } else if (tree->pitch >= kWideMinPitch ||
               (tree->pitch > kStagedMaxPitch && (long long)n * ((tree->pitch + kSegSlots - 1) / kSegSlots) >= kSegMinItems)) {
        // wide rows (chess: 4,672; Go's 362 in large launches: 16,384 x 362 takes 28.4 us against 33.9 us with a
        // warp per node, 4,096 x 512 17.5 us against 13.5 us): segments of 256 slots through the staged design, a (score, slot) word per
        // segment as scratch, allocated and freed in stream order
        int dev = 0, sms = 0;
        OB200_CUDA_OK(cudaGetDevice(&dev));
        OB200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        const int segs = (tree->pitch + kSegSlots - 1) / kSegSlots;
        const int smem = kSegWarps * kSegDepth * 4 * kSegSlots * 4 + kSegWarps * kSegDepth * 8;
        static bool configured_w[64] = {false};
        if (dev < 0 || dev >= 64 || !configured_w[dev]) {
            OB200_CUDA_OK(cudaFuncSetAttribute(puct_select_segmented_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            if (dev >= 0 && dev < 64) configured_w[dev] = true;
        }
        int* errw = device_error_word();
        if (!errw) return set_error(OB200_ERR_CUDA, "ob200_launch_puct_select: cannot resolve the device error word");
        unsigned long long* words = wide_scratch(dev, as_stream(stream), n);
        if (!words) return set_error(OB200_ERR_CUDA, "ob200_launch_puct_select: cannot allocate %d selection words", n);
        const long long items = (long long)n * segs;
        const long long want = (items + kSegWarps - 1) / kSegWarps;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(want < sms ? want : sms));
        cfg.blockDim = dim3(kSegWarps * 32);
        cfg.dynamicSmemBytes = (size_t)smem;
        cfg.stream = as_stream(stream);
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, puct_select_segmented_kernel, *tree, node_ids, n, segs, c_puct, words, errw));
        cfg = cudaLaunchConfig_t{};
        cfg.gridDim = dim3((unsigned)((n + 255) / 256));
        cfg.blockDim = dim3(256);
        cfg.stream = as_stream(stream);
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, puct_select_finish_kernel, *tree, node_ids, n, vl_value, apply_vl, sel_out, words));
        counters().launches.fetch_add(2, std::memory_order_relaxed);
    } else {
        const int blocks = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
        puct_select_kernel<<<blocks, kWarpsPerBlock * 32, 0, as_stream(stream)>>>(*tree, node_ids, n, c_puct, vl_value,
                                                                                 apply_vl, sel_out);
        OB200_LAUNCHED("puct_select_kernel");
    }
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n + 255) / 256)); cfg.blockDim = dim3(256); cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, vl_revert_kernel, *tree, node_ids, sel, (int)n, (int)vl_value));
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
    OB200_CUDA_OK(launch_dependent(backup_kernel, dim3((n + 127) / 128), dim3(128), 0, as_stream(stream), *tree, paths, path_len,
                                   leaf_values, n, max_depth, vl_value));
    counters().launches.fetch_add(1, std::memory_order_relaxed);
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
    // one CTA per tree: trees are few and latency-bound, so spread them over the SMs
    OB200_CUDA_OK(launch_dependent(traverse_kernel, dim3(n_trees), dim3(kTravWarps * 32), 0, as_stream(stream), *tree, roots, n_trees,
                                   sims_per_tree, c_puct, vl_value, max_depth, paths_out, path_len_out));
    counters().launches.fetch_add(1, std::memory_order_relaxed);
    counters().selections.fetch_add((uint64_t)n_trees * sims_per_tree, std::memory_order_relaxed);
    return OB200_OK;
}

}  // extern "C"
