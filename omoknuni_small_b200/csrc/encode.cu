// Leaf state -> bf16 board tensor (sm_100a).
//
// Output format (see "Board tensors" in omoknuni_b200.h): NHWC, positions on a
// (S+1) x (S+1) grid per board whose last column / row are zero, guard
// positions before and after.  A thread produces one position (its 16-byte
// channel blocks one after the other); the kernels also write the zero
// padding, so the output needs no memset.
#include "internal.h"
#include <cuda_bf16.h>

namespace ob200 {
namespace {

struct alignas(16) Pack8 { __nv_bfloat16 v[8]; };

// Gomoku planes from the move history; reference semantics in
// GomokuState::getEnhancedTensorRepresentation
// (src/games/gomoku/gomoku_state.cpp:223-262): the k-th most recent move is
// the opponent's for even k and the side to move's for odd k; plane 2i holds
// the side to move's i-th most recent stone, plane 2i+1 the opponent's.
// Hence plane p takes move k = p + 1 (p even) or p - 1 (p odd).
__global__ void __launch_bounds__(256)
encode_gomoku_kernel(const int16_t* __restrict__ history, const uint8_t* __restrict__ n_hist,
                     const uint8_t* __restrict__ to_move, int B, int S, int planes, int chunks,
                     int cover, Pack8* __restrict__ out) {
    // cover = positions written (guards included); chunks = channels / 8.
    // One thread per position writes all its chunks; only the first three can be non-zero.
    const int pidx = blockIdx.x * blockDim.x + threadIdx.x;
    if (pidx >= cover) return;
    const int p = pidx - OB200_GUARD;
    const int GP = S + 1, slots = GP * GP;
    int cell = -1, b = 0;
    if (p >= 0 && p < B * slots) {
        b = p / slots;
        const int r = p - b * slots;
        const int y = r / GP, x = r - y * GP;
        if (y < S && x < S) cell = y * S + x;
    }
    Pack8 zero;
#pragma unroll
    for (int j = 0; j < 8; ++j) zero.v[j] = __float2bfloat16(0.0f);
    Pack8* dst = out + (size_t)pidx * chunks;
    if (cell < 0) {
        for (int c = 0; c < chunks; ++c) dst[c] = zero;
        return;
    }
    const int nh = n_hist[b];
    const int16_t* h = history + (size_t)b * 16;
    const float colour = (planes > 16 && to_move[b] == 1) ? 1.0f : 0.0f;
    for (int c = 0; c < chunks; ++c) {
        Pack8 o = zero;
        if (c < 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int plane = c * 8 + j;
                const int k = (plane & 1) ? plane - 1 : plane + 1;
                if (k < nh && h[k] == cell) o.v[j] = __float2bfloat16(1.0f);
            }
        } else if (c == 2) {
            // plane 16: colour.  Planes 17 / 18 (attack / defense): zero, as the reference's CPU
            // code yields for every legal move (src/utils/attack_defense_module.cpp:96-154).
            o.v[0] = __float2bfloat16(colour);
        }
        dst[c] = o;
    }
}

__global__ void __launch_bounds__(256)
planes_to_board_tensor_kernel(const float* __restrict__ planes, int B, int C, int S, int chunks,
                              long long cover, Pack8* __restrict__ out) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= cover * chunks) return;
    const int chunk = (int)(gid % chunks);
    const long long p = gid / chunks - OB200_GUARD;
    const int GP = S + 1, slots = GP * GP;
    Pack8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(0.0f);
    if (p >= 0 && p < (long long)B * slots) {
        const int b = (int)(p / slots), r = (int)(p % slots);
        const int y = r / GP, x = r % GP;
        if (y < S && x < S) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = chunk * 8 + j;
                if (c < C) o.v[j] = __float2bfloat16(__ldg(planes + (((size_t)b * C + c) * S + y) * S + x));
            }
        }
    }
    out[gid] = o;
}

}  // namespace

int launch_encode_gomoku(const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                         int32_t B, int32_t board_size, int32_t planes, int32_t out_channels,
                         void* board_tensor_out, cudaStream_t stream) {
    if (!history || !n_hist || !to_move || !board_tensor_out || B < 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_gomoku: null pointer or negative batch");
    if (planes != 17 && planes != 19)
        return set_error(OB200_ERR_INVALID, "ob200_launch_encode_gomoku: planes must be 17 or 19, got %d", planes);
    if (board_size < 5 || board_size > 31 || out_channels < planes || (out_channels & 7))
        return set_error(OB200_ERR_INVALID,
                         "ob200_launch_encode_gomoku: board_size %d must be in [5,31] and out_channels %d a multiple of 8 >= planes",
                         board_size, out_channels);
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(board_size, B);
    const int chunks = out_channels / 8;
    if (g.PT > 0x7fffffffLL / 2) return set_error(OB200_ERR_TOO_LARGE, "encode: batch too large");
    encode_gomoku_kernel<<<(unsigned)((g.PT + 255) / 256), 256, 0, stream>>>(
        history, n_hist, to_move, B, board_size, planes, chunks, (int)g.PT, reinterpret_cast<Pack8*>(board_tensor_out));
    OB200_LAUNCHED("encode_gomoku_kernel");
    return OB200_OK;
}

int launch_planes_to_board_tensor(const float* planes_nchw, int32_t B, int32_t C, int32_t board_size,
                                  int32_t out_channels, void* board_tensor_out, cudaStream_t stream) {
    if (!planes_nchw || !board_tensor_out || B < 0 || C <= 0)
        return set_error(OB200_ERR_INVALID, "ob200_launch_planes_to_board_tensor: bad arguments");
    if (board_size < 1 || board_size > 31 || out_channels <= 0 || (out_channels & 7))
        return set_error(OB200_ERR_INVALID, "ob200_launch_planes_to_board_tensor: bad board_size %d / out_channels %d",
                         board_size, out_channels);
    if (int rc = require_device()) return rc;
    const BoardGeom g = board_geom(board_size, B);
    const int chunks = out_channels / 8;
    const long long total = g.PT * chunks;
    planes_to_board_tensor_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        planes_nchw, B, C, board_size, chunks, g.PT, reinterpret_cast<Pack8*>(board_tensor_out));
    OB200_LAUNCHED("planes_to_board_tensor_kernel");
    return OB200_OK;
}

}  // namespace ob200

using namespace ob200;

extern "C" {

int ob200_launch_encode_gomoku(const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                               int32_t B, int32_t board_size, int32_t planes, int32_t out_channels,
                               void* board_tensor_out, ob200_stream stream) {
    return launch_encode_gomoku(history, n_hist, to_move, B, board_size, planes, out_channels, board_tensor_out,
                                as_stream(stream));
}

int ob200_launch_planes_to_board_tensor(const float* planes_nchw, int32_t B, int32_t C, int32_t board_size,
                                        int32_t out_channels, void* board_tensor_out, ob200_stream stream) {
    return launch_planes_to_board_tensor(planes_nchw, B, C, board_size, out_channels, board_tensor_out,
                                         as_stream(stream));
}

}  // extern "C"
