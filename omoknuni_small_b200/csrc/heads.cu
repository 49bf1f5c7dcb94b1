// Policy and value heads (sm_100a, fp32 CUDA cores; < 1 % of the network's
// arithmetic with the 2-channel / 1-channel heads).
//
//   head_conv_kernel   1x1 convolution (+ folded BatchNorm, ReLU) of both heads
//                      from the tower's board tensor; writes fp32 activations
//                      in the reference's flatten order c * S*S + y * S + x
//                      (src/nn/resnet_model.cpp:183,209 view({B,-1}) on NCHW).
//   fc_kernel          out[b][j] = act(sum_i in[b][i] * WT[i][j] + bias[j]);
//                      a CTA owns 8 boards x 64 outputs split in 4 K-slices, the
//                      weight matrix is stored transposed so that threads read
//                      it coalesced and each weight is used for 8 boards.
//   softmax_kernel     in-place softmax over a row.
//   value_out_kernel   value_fc2 + tanh (one warp per board).
#include "internal.h"
#include <cuda_bf16.h>
#include <mutex>

namespace ob200 {
namespace {

constexpr int kFcBoards = 8;
constexpr int kFcThreads = 256;
constexpr int kFcKTile = 512;

struct alignas(16) Pack8 { __nv_bfloat162 v[4]; };

// One thread per real board cell; w_s holds [HC][64] folded weights.
__global__ void __launch_bounds__(128)
head_conv_kernel(const uint8_t* __restrict__ tower, const float* __restrict__ w,
                 const float* __restrict__ bias, int HC, int pc, float* __restrict__ hp,
                 float* __restrict__ hv, int B, int S) {
    extern __shared__ float w_s[];  // HC*64 weights then HC biases
    for (int i = threadIdx.x; i < HC * 64; i += blockDim.x) w_s[i] = w[i];
    for (int i = threadIdx.x; i < HC; i += blockDim.x) w_s[HC * 64 + i] = bias[i];
    __syncthreads();
    const int S2 = S * S, GP = S + 1;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (long long)B * S2) return;
    const int b = (int)(gid / S2), cell = (int)(gid % S2);
    const int y = cell / S, x = cell % S;
    const long long rec = (long long)OB200_GUARD + (long long)b * GP * GP + y * GP + x;
    float a[64];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const Pack8 v = *reinterpret_cast<const Pack8*>(tower + rec * 128 + c * 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(v.v[j]);
            a[c * 8 + 2 * j] = f.x; a[c * 8 + 2 * j + 1] = f.y;
        }
    }
    const int vc = HC - pc;
    for (int h = 0; h < HC; ++h) {
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < 64; ++k) s = fmaf(a[k], w_s[h * 64 + k], s);
        s = fmaxf(s + w_s[HC * 64 + h], 0.0f);
        if (h < pc) hp[((size_t)b * pc + h) * S2 + cell] = s;
        else hv[((size_t)b * vc + (h - pc)) * S2 + cell] = s;
    }
}

// A CTA owns 8 boards x 64 outputs; its 256 threads are 4 K-slices x 64 outputs, so a
// thread walks a quarter of the inner dimension with 8 accumulators (one weight load
// feeds 8 boards) and the slices are summed through shared memory.  Small tiles give a
// grid of several CTAs per SM, which is what hides the L2 latency of the weight reads.
__global__ void __launch_bounds__(kFcThreads)
fc_kernel(const float* __restrict__ in, const float* __restrict__ WT, const float* __restrict__ bias,
          float* __restrict__ out, int B, int K, int Nout, int relu) {
    __shared__ __align__(16) float in_s[kFcBoards][kFcKTile];
    __shared__ float red[3][kFcBoards][64];
    const int b0 = blockIdx.x * kFcBoards;
    const int jl = threadIdx.x & 63, slice = threadIdx.x >> 6;
    const int j = blockIdx.y * 64 + jl;
    float acc[kFcBoards];
#pragma unroll
    for (int g = 0; g < kFcBoards; ++g) acc[g] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += kFcKTile) {
        const int kt = min(kFcKTile, K - k0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < kFcBoards * kt; idx += kFcThreads) {
            const int g = idx / kt, i = idx % kt;
            in_s[g][i] = (b0 + g < B) ? in[(size_t)(b0 + g) * K + k0 + i] : 0.0f;
        }
        __syncthreads();
        if (j < Nout) {
            // slices are multiples of 4 wide so that the staged inputs are read as float4:
            // one shared-memory load feeds 4 multiply-adds (the loop is otherwise bound by
            // shared-memory instruction issue)
            const int per = ((kt + 3) / 4 + 3) & ~3;
            const int i0 = slice * per, i1 = min(kt, i0 + per);
            const float* wp = WT + (size_t)k0 * Nout + j;
            int i = i0;
            for (; i + 4 <= i1; i += 4) {
                const float w0 = __ldg(wp + (size_t)i * Nout), w1 = __ldg(wp + (size_t)(i + 1) * Nout);
                const float w2 = __ldg(wp + (size_t)(i + 2) * Nout), w3 = __ldg(wp + (size_t)(i + 3) * Nout);
#pragma unroll
                for (int g = 0; g < kFcBoards; ++g) {
                    const float4 x = *reinterpret_cast<const float4*>(&in_s[g][i]);
                    acc[g] = fmaf(x.x, w0, acc[g]); acc[g] = fmaf(x.y, w1, acc[g]);
                    acc[g] = fmaf(x.z, w2, acc[g]); acc[g] = fmaf(x.w, w3, acc[g]);
                }
            }
            for (; i < i1; ++i) {
                const float wv = __ldg(wp + (size_t)i * Nout);
#pragma unroll
                for (int g = 0; g < kFcBoards; ++g) acc[g] = fmaf(in_s[g][i], wv, acc[g]);
            }
        }
    }
    if (slice > 0) {
#pragma unroll
        for (int g = 0; g < kFcBoards; ++g) red[slice - 1][g][jl] = acc[g];
    }
    __syncthreads();
    if (slice == 0 && j < Nout) {
        const float bj = bias[j];
#pragma unroll
        for (int g = 0; g < kFcBoards; ++g)
            if (b0 + g < B) {
                float v = acc[g] + red[0][g][jl] + red[1][g][jl] + red[2][g][jl] + bj;
                if (relu) v = fmaxf(v, 0.0f);
                out[(size_t)(b0 + g) * Nout + j] = v;
            }
    }
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

__global__ void __launch_bounds__(128) softmax_kernel(float* __restrict__ x, int A) {
    __shared__ float red[4];
    float* row = x + (size_t)blockIdx.x * A;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < A; i += blockDim.x) m = fmaxf(m, row[i]);
    m = block_reduce(m, true, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < A; i += blockDim.x) s += expf(row[i] - m);
    s = block_reduce(s, false, red);
    const float inv = 1.0f / s;
    for (int i = threadIdx.x; i < A; i += blockDim.x) row[i] = expf(row[i] - m) * inv;
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

}  // namespace

int launch_head_conv(const void* tower, const float* w, const float* bias, int HC, int pc,
                     float* hp, float* hv, int B, int S, cudaStream_t st) {
    const long long total = (long long)B * S * S;
    const size_t smem = (size_t)(HC * 64 + HC) * sizeof(float);
    head_conv_kernel<<<(unsigned)((total + 127) / 128), 128, smem, st>>>(static_cast<const uint8_t*>(tower), w, bias,
                                                                        HC, pc, hp, hv, B, S);
    OB200_LAUNCHED("head_conv_kernel");
    return OB200_OK;
}

int launch_fc(const float* in, const float* WT, const float* bias, float* out, int B, int K, int Nout, int relu,
              cudaStream_t st) {
    dim3 grid((B + kFcBoards - 1) / kFcBoards, (Nout + 63) / 64);
    fc_kernel<<<grid, kFcThreads, 0, st>>>(in, WT, bias, out, B, K, Nout, relu);
    OB200_LAUNCHED("fc_kernel");
    return OB200_OK;
}

int launch_softmax(float* x, int B, int A, cudaStream_t st) {
    softmax_kernel<<<B, 128, 0, st>>>(x, A);
    OB200_LAUNCHED("softmax_kernel");
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
                             cudaStream_t st) {
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
    if (int rc = launch_head_conv(tower, vw, vb, vc, 0, hv, hv, B, S, st)) return rc;
    if (int rc = launch_fc(hv, W1T, b1, hidden, B, vc * S * S, H, 1, st)) return rc;
    return launch_value_out(hidden, w2, b2, H, B, value_out, st);
}

}  // namespace ob200
