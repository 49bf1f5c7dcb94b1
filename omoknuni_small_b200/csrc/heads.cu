// Policy and value heads (sm_100a, fp32 CUDA cores; < 1 % of the network's
// arithmetic with the 2-channel / 1-channel heads).
//
//   head_conv_kernel   1x1 convolution (+ folded BatchNorm, ReLU) of both heads
//                      from the tower's board tensor; writes fp32 activations
//                      in the reference's flatten order c * S*S + y * S + x
//                      (src/nn/resnet_model.cpp:183,209 view({B,-1}) on NCHW).
//   fc_kernel          out[b][j] = act(sum_i in[b][i] * WT[i][j] + bias[j]);
//                      register-tiled (32 boards x 64 outputs per CTA, 4 x 4 per
//                      thread, cp.async pipeline), weight matrix stored transposed.
//   fc_pair_kernel     the policy FC and the value head's first FC as one launch.
//   head_tails_kernel  in-place softmax over the rows of logits, and value_fc2 + tanh, as one launch.
//   value_out_kernel   value_fc2 + tanh (one warp per board), for the value head on its own.
#include "internal.h"
#include "sm100_ptx.cuh"
#include <mutex>

namespace ob200 {
namespace {

struct alignas(16) Pack8 { uint32_t v[4]; };

// A warp takes 32 consecutive positions of the board tensor (pad positions included, their
// results are dropped).  Eight lanes share a position: lane = 8 * (position within a group of 4)
// + channel block, so a warp-wide 16-byte load covers 4 positions x 128 contiguous bytes of one
// 64-channel slice and the 8 loads of a warp are issued back to back.  Each lane multiplies its
// 8 channels (per slice) into a head channel's partial sum, three shuffle steps add the 8 lanes,
// and lane (sub, blk) keeps the sum of group blk: after 8 groups every lane owns one position and
// stores once per head channel.  C = tower channels (a multiple of 64).
// HCT > 0: that many head channels, partial sums of all of them held in registers while the
// slices stream by; HCT == 0: any number, weights in shared memory, one head channel at a time.
constexpr int kHeadThreads = 128;
template <int HCT>
__global__ void __launch_bounds__(kHeadThreads)
head_conv_kernel(const uint8_t* __restrict__ tower, const float* __restrict__ w,
                 const float* __restrict__ bias, int HC, int pc, float* __restrict__ hp,
                 float* __restrict__ hv, int B, int S, int C, int f16) {
    extern __shared__ float w_s[];  // HCT == 0: [HC][C] folded weights then [HC] biases
    const int lane = threadIdx.x & 31, sub = lane >> 3, blk = lane & 7;
    if (HCT == 0) {
        for (int i = threadIdx.x; i < HC * C; i += blockDim.x) w_s[i] = w[i];
        for (int i = threadIdx.x; i < HC; i += blockDim.x) w_s[HC * C + i] = bias[i];
        __syncthreads();
    }
    const int hc = HCT > 0 ? HCT : HC;
    const int S2 = S * S, GP = S + 1, slots = GP * GP, vc = hc - pc;
    const int total = B * slots;
    const int slices = C >> 6;
    const size_t row_bytes = (size_t)C * 2;
    const int p0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * 32;
    if (p0 >= total) return;
    // the tensor's trailing guard positions make the (at most 31) positions past the end readable
    const uint8_t* src = tower + ((size_t)OB200_GUARD + p0 + sub) * row_bytes + blk * 16;
    float a[8][8];
    auto load_slice = [&](int sl) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const Pack8 v = *reinterpret_cast<const Pack8*>(src + (size_t)it * 4 * row_bytes + (size_t)sl * 128);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // the tower's storage type: both conversions are exact
                if (f16) ptx::unpack2<true>(v.v[j], a[it][2 * j], a[it][2 * j + 1]);
                else ptx::unpack2<false>(v.v[j], a[it][2 * j], a[it][2 * j + 1]);
            }
        }
    };
    // this lane's own position: group blk, member sub
    const int p = p0 + blk * 4 + sub;
    const int b = p / slots, r = p - b * slots;
    const int y = r / GP, x = r - y * GP;
    const bool real = p < total && y < S && x < S;
    const int cell = y * S + x;
    auto finish = [&](int h, const float (&part)[8], float bh) {
        float keep = 0.0f;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            float s = part[it];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            keep = (it == blk) ? s : keep;
        }
        if (real) {
            const float o = fmaxf(keep + bh, 0.0f);
            if (h < pc) hp[((size_t)b * pc + h) * S2 + cell] = o;
            else hv[((size_t)b * vc + (h - pc)) * S2 + cell] = o;
        }
    };
    if (HCT > 0) {
        constexpr int kRegCh = HCT > 0 ? HCT : 1;
        float part[kRegCh][8];
#pragma unroll
        for (int h = 0; h < kRegCh; ++h)
#pragma unroll
            for (int it = 0; it < 8; ++it) part[h][it] = 0.0f;
        for (int sl = 0; sl < slices; ++sl) {
            load_slice(sl);
#pragma unroll
            for (int h = 0; h < kRegCh; ++h) {
                const float4* wr = reinterpret_cast<const float4*>(w + (size_t)h * C + sl * 64 + blk * 8);
                const float4 w0 = __ldg(wr), w1 = __ldg(wr + 1);
                const float wk[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int it = 0; it < 8; ++it)
#pragma unroll
                    for (int k = 0; k < 8; ++k) part[h][it] = fmaf(a[it][k], wk[k], part[h][it]);
            }
        }
#pragma unroll
        for (int h = 0; h < kRegCh; ++h) finish(h, part[h], __ldg(bias + h));
    } else {
        if (slices == 1) load_slice(0);
        for (int h = 0; h < hc; ++h) {
            float part[8];
#pragma unroll
            for (int it = 0; it < 8; ++it) part[it] = 0.0f;
            for (int sl = 0; sl < slices; ++sl) {
                if (slices > 1) load_slice(sl);   // re-read per head channel (L1 / L2 hits)
                const float4* wr = reinterpret_cast<const float4*>(w_s + (size_t)h * C + sl * 64 + blk * 8);
                const float4 w0 = wr[0], w1 = wr[1];
                const float wk[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int it = 0; it < 8; ++it)
#pragma unroll
                    for (int k = 0; k < 8; ++k) part[it] = fmaf(a[it][k], wk[k], part[it]);
            }
            finish(h, part, w_s[hc * C + h]);
        }
    }
}

// out[b][j] = act(sum_i in[b][i] * WT[i][j] + bias[j]).  Register-tiled: a CTA owns 32 boards x
// 64 outputs, a thread 4 boards x 4 outputs.  The 256 threads form two groups of 128 that each
// take half of the inner dimension and run their own 3-stage cp.async pipeline of 16-deep tiles
// (operands read back from shared memory as float4: 2 shared loads feed 16 multiply-adds); the
// second group's sums pass through shared memory to the first, which applies bias / ReLU.
constexpr int kFcTileB = 32, kFcTileN = 64, kFcTileK = 16, kFcStages = 3, kFcAPitch = kFcTileB + 4;
struct FcStage {
    float a[kFcTileK][kFcAPitch];   // inputs, k-major; the pad spreads the staging writes over banks
    float b[kFcTileK][kFcTileN];    // weights
};
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
struct FcProblem {
    const float* in;     // [B][K]
    const float* WT;     // [K][Nout]
    const float* bias;   // [Nout]
    float* out;          // [B][Nout]
    int K, Nout, relu;
};
__device__ __forceinline__ void fc_tile(FcStage (*st)[kFcStages], const float* __restrict__ in, const float* __restrict__ WT,
                                        const float* __restrict__ bias, float* __restrict__ out, int B, int K, int Nout,
                                        int relu, int tile_b, int tile_n) {
    const int half = threadIdx.x >> 7, t = threadIdx.x & 127;
    const int b0 = tile_b * kFcTileB, n0 = tile_n * kFcTileN;
    const int tb = (t >> 4) * 4, tn = (t & 15) * 4;   // 8 x 16 threads
    const int tiles = (K + kFcTileK - 1) / kFcTileK, split = (tiles + 1) / 2;
    const int first = half ? split : 0, last = half ? tiles : split;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    auto issue = [&](int tile, int slot) {
        if (tile < last) {
            FcStage& s = st[half][slot];
            const int k0 = tile * kFcTileK;
#pragma unroll
            for (int r = 0; r < (kFcTileK * kFcTileB) / 128; ++r) {
                const int idx = t + r * 128;
                const int bb = idx / kFcTileK, kk = idx - bb * kFcTileK;   // threads walk k: rows of `in`
                const int gb = b0 + bb, gk = k0 + kk;
                if (gb < B && gk < K) cp_async4(&s.a[kk][bb], in + (size_t)gb * K + gk);
                else s.a[kk][bb] = 0.0f;
            }
#pragma unroll
            for (int r = 0; r < (kFcTileK * kFcTileN) / 128; ++r) {
                const int idx = t + r * 128;
                const int kk = idx / kFcTileN, nn = idx - kk * kFcTileN;
                const int gk = k0 + kk, gn = n0 + nn;
                if (gk < K && gn < Nout) cp_async4(&s.b[kk][nn], WT + (size_t)gk * Nout + gn);
                else s.b[kk][nn] = 0.0f;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int s = 0; s < kFcStages - 1; ++s) issue(first + s, s);
    for (int tile = first; tile < last; ++tile) {
        const int slot = (tile - first) % kFcStages;
        asm volatile("cp.async.wait_group %0;" ::"n"(kFcStages - 2) : "memory");
        asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");   // tile landed; previous slot free
        issue(tile + kFcStages - 1, (slot + kFcStages - 1) % kFcStages);
        const FcStage& s = st[half][slot];
#pragma unroll
        for (int kk = 0; kk < kFcTileK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&s.a[kk][tb]);
            const float4 bv = *reinterpret_cast<const float4*>(&s.b[kk][tn]);
            const float aa[4] = {av.x, av.y, av.z, av.w}, bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], bb[j], acc[i][j]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float* red = reinterpret_cast<float*>(&st[0][0]);   // 128 x 16 floats, reusing the stages
    if (half) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) red[(i * 4 + j) * 128 + t] = acc[i][j];
    }
    __syncthreads();
    if (half) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gb = b0 + tb + i;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tn + j;
            if (gb >= B || gn >= Nout) continue;
            float v = acc[i][j] + red[(i * 4 + j) * 128 + t] + bias[gn];
            if (relu) v = fmaxf(v, 0.0f);
            out[(size_t)gb * Nout + gn] = v;
        }
    }
}

__global__ void __launch_bounds__(256)
fc_kernel(const float* __restrict__ in, const float* __restrict__ WT, const float* __restrict__ bias,
          float* __restrict__ out, int B, int K, int Nout, int relu) {
    __shared__ __align__(16) FcStage st[2][kFcStages];
    fc_tile(st, in, WT, bias, out, B, K, Nout, relu, blockIdx.x, blockIdx.y);
}

// Two independent layers over the same boards in one launch (the policy FC and the value head's first FC): the
// first tiles_n0 values of blockIdx.y are output tiles of problem 0, the rest of problem 1.  Each output is
// computed exactly as fc_kernel computes it.
__global__ void __launch_bounds__(256)
fc_pair_kernel(FcProblem p0, FcProblem p1, int B, int tiles_n0) {
    __shared__ __align__(16) FcStage st[2][kFcStages];
    asm volatile("griddepcontrol.wait;" ::: "memory");               // the inputs come from the kernel ahead in the stream
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const bool first = (int)blockIdx.y < tiles_n0;
    const FcProblem& p = first ? p0 : p1;
    fc_tile(st, p.in, p.WT, p.bias, p.out, B, p.K, p.Nout, p.relu, blockIdx.x, first ? blockIdx.y : blockIdx.y - tiles_n0);
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
    for (int off = 16; off > 0; off >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, off);
        v = is_max ? fmaxf(v, o) : v + o;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    v = red[0];
    for (int i = 1; i < nw; ++i) v = is_max ? fmaxf(v, red[i]) : v + red[i];
    return v;
}

__global__ void __launch_bounds__(256)
value_out_kernel(const float* __restrict__ hidden, const float* __restrict__ w2, float b2, int H, int B,
                 float* __restrict__ value) {
    const int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (b >= B) return;
    float s = 0.0f;
    for (int i = lane; i < H; i += 32) s = fmaf(hidden[(size_t)b * H + i], w2[i], s);
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) value[b] = tanhf(s + b2);
}

// The tails of both heads in one launch, started as a programmatic dependent of fc_pair_kernel: CTAs
// [0, softmax_rows) normalise one row of logits each (maximum, sum of exponentials, division), the rest finish four boards' values
// each as value_out_kernel does (a warp per board).
__global__ void __launch_bounds__(128)
head_tails_kernel(float* __restrict__ logits, int A, int softmax_rows, const float* __restrict__ hidden,
                  const float* __restrict__ w2, float b2, int H, int B, float* __restrict__ value) {
    __shared__ float red[4];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if ((int)blockIdx.x < softmax_rows) {
        float* row = logits + (size_t)blockIdx.x * A;
        float m = -INFINITY;
        for (int i = threadIdx.x; i < A; i += blockDim.x) m = fmaxf(m, row[i]);
        m = block_reduce(m, true, red);
        float s = 0.0f;
        for (int i = threadIdx.x; i < A; i += blockDim.x) s += expf(row[i] - m);
        s = block_reduce(s, false, red);
        const float inv = 1.0f / s;
        for (int i = threadIdx.x; i < A; i += blockDim.x) row[i] = expf(row[i] - m) * inv;
    } else {
        const int b = ((int)blockIdx.x - softmax_rows) * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
        if (b >= B) return;
        float s = 0.0f;
        for (int i = lane; i < H; i += 32) s = fmaf(hidden[(size_t)b * H + i], w2[i], s);
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) value[b] = tanhf(s + b2);
    }
}

}  // namespace

// The FC part of both heads in two launches: {policy FC (when policy_in is given), value FC1 + ReLU}, then
// {softmax over the logits (when asked), value FC2 + tanh}.  The FC results equal launch_fc / launch_value_out on
// the same buffers bit for bit.
int launch_head_fcs(const float* policy_in, const float* WpT, const float* bp, float* policy_out, int policy_k, int policy_size,
                    int softmax, const float* value_in, const float* W1T, const float* b1, float* hidden, int value_k, int H,
                    const float* w2, float b2, float* value_out, int B, cudaStream_t st) {
    const FcProblem p0{policy_in, WpT, bp, policy_out, policy_k, policy_size, 0};
    const FcProblem p1{value_in, W1T, b1, hidden, value_k, H, 1};
    const int tiles0 = policy_in ? (policy_size + kFcTileN - 1) / kFcTileN : 0, tiles1 = (H + kFcTileN - 1) / kFcTileN;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((B + kFcTileB - 1) / kFcTileB, tiles0 + tiles1);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, fc_pair_kernel, p0, p1, B, tiles0));
    counters().launches.fetch_add(1, std::memory_order_relaxed);
    const int rows = softmax ? B : 0;
    cfg.gridDim = dim3((unsigned)(rows + (B + 3) / 4));
    cfg.blockDim = dim3(128);
    OB200_CUDA_OK(cudaLaunchKernelEx(&cfg, head_tails_kernel, policy_out, policy_size, rows, (const float*)hidden, w2, b2, H, B, value_out));
    counters().launches.fetch_add(1, std::memory_order_relaxed);
    return OB200_OK;
}

int launch_head_conv(const void* tower, const float* w, const float* bias, int HC, int pc,
                     float* hp, float* hv, int B, int S, cudaStream_t st, int C, int dtype) {
    const int f16 = dtype == OB200_DTYPE_F16;
    if (C < 64 || C % 64) return set_error(OB200_ERR_INVALID, "head conv: tower channels %d not a multiple of 64", C);
    const long long total = (long long)B * (S + 1) * (S + 1);   // positions, one warp per 32
    const unsigned grid = (unsigned)((total + kHeadThreads - 1) / kHeadThreads);
    const uint8_t* t = static_cast<const uint8_t*>(tower);
    switch (HC) {
        case 1: head_conv_kernel<1><<<grid, kHeadThreads, 0, st>>>(t, w, bias, HC, pc, hp, hv, B, S, C, f16); break;
        case 2: head_conv_kernel<2><<<grid, kHeadThreads, 0, st>>>(t, w, bias, HC, pc, hp, hv, B, S, C, f16); break;
        case 3: head_conv_kernel<3><<<grid, kHeadThreads, 0, st>>>(t, w, bias, HC, pc, hp, hv, B, S, C, f16); break;
        case 4: head_conv_kernel<4><<<grid, kHeadThreads, 0, st>>>(t, w, bias, HC, pc, hp, hv, B, S, C, f16); break;
        default: {
            const size_t smem = (size_t)(HC * C + HC) * sizeof(float);
            if (smem > 200 * 1024)
                return set_error(OB200_ERR_UNSUPPORTED, "head conv: %d head channels x %d tower channels exceed shared memory", HC, C);
            if (smem > 48 * 1024)
                OB200_CUDA_OK(cudaFuncSetAttribute(head_conv_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            head_conv_kernel<0><<<grid, kHeadThreads, smem, st>>>(t, w, bias, HC, pc, hp, hv, B, S, C, f16);
        }
    }
    OB200_LAUNCHED("head_conv_kernel");
    return OB200_OK;
}

int launch_fc(const float* in, const float* WT, const float* bias, float* out, int B, int K, int Nout, int relu,
              cudaStream_t st) {
    dim3 grid((B + kFcTileB - 1) / kFcTileB, (Nout + kFcTileN - 1) / kFcTileN);
    fc_kernel<<<grid, 256, 0, st>>>(in, WT, bias, out, B, K, Nout, relu);
    OB200_LAUNCHED("fc_kernel");
    return OB200_OK;
}

int launch_value_out(const float* hidden, const float* w2, float b2, int H, int B, float* value, cudaStream_t st) {
    value_out_kernel<<<(B * 32 + 255) / 256, 256, 0, st>>>(hidden, w2, b2, H, B, value);
    OB200_LAUNCHED("value_out_kernel");
    return OB200_OK;
}

// ---------------------------------------------------------------------------
// Value head without any allocation.  The two intermediates of the value head
// (the 1x1-convolution activations and the hidden layer) live in this
// file-scope device array instead of buffers obtained from cudaMalloc.  Every
// GPU that loads the library holds the 2 MiB until the process exits.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchFloats = size_t(1) << 19;
static __device__ __align__(256) float g_value_head_scratch[kStaticScratchFloats];

size_t value_head_static_capacity() { return kStaticScratchFloats; }

// In host code the array's name is only a stand-in for the symbol: its device address
// is asked from the runtime once per device, with that device current.
static int value_head_scratch_ptr(float** out) {
    static std::mutex mu;
    static float* cached[64] = {nullptr};
    int dev = 0;
    OB200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(OB200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (!cached[dev]) {
        void* ptr = nullptr;
        OB200_CUDA_OK(cudaGetSymbolAddress(&ptr, g_value_head_scratch));
        cached[dev] = static_cast<float*>(ptr);
    }
    *out = cached[dev];
    return OB200_OK;
}

int launch_value_head_static(const void* tower, const float* vw, const float* vb, int vc, const float* W1T,
                             const float* b1, const float* w2, float b2, int H, int B, int S, float* value_out,
                             cudaStream_t st, int dtype) {
    const size_t need = (size_t)B * ((size_t)vc * S * S + (size_t)H);
    if (need > kStaticScratchFloats)
        return set_error(OB200_ERR_TOO_LARGE,
                         "value head without allocation: batch %d needs %zu scratch floats (%d x %d x %d + %d per board), the static array holds %zu",
                         B, need, vc, S, S, H, kStaticScratchFloats);
    float* scratch = nullptr;
    if (int rc = value_head_scratch_ptr(&scratch)) return rc;
    float* hv = scratch;                                  // [B][vc * S * S]
    float* hidden = scratch + (size_t)B * vc * S * S;     // [B][H]
    // every element read below is written first by the launch before it: nothing needs clearing
    if (int rc = launch_head_conv(tower, vw, vb, vc, 0, hv, hv, B, S, st, 64, dtype)) return rc;
    if (int rc = launch_fc(hv, W1T, b1, hidden, B, vc * S * S, H, 1, st)) return rc;
    return launch_value_out(hidden, w2, b2, H, B, value_out, st);
}

}  // namespace ob200
