// Launchers shared between the translation units of the library (C++ linkage).
#pragma once
#include "common.h"

namespace ob200 {

int launch_encode_gomoku(const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move, int32_t B,
                         int32_t board_size, int32_t planes, int32_t out_channels, void* board_tensor_out,
                         cudaStream_t stream, int dtype = 0);
int launch_encode_go(const int8_t* stones, const int32_t* ko_point, const uint8_t* to_move, const uint32_t* legal_bits,
                     int32_t B, int32_t board_size, int32_t out_channels, void* board_tensor_out, cudaStream_t stream,
                     int dtype = 0);
int launch_encode_gomoku3(const int8_t* stones, const uint8_t* to_move, int32_t B, int32_t board_size, int32_t out_channels,
                          void* board_tensor_out, cudaStream_t stream, int dtype = 0);
int launch_encode_chess(const int8_t* pieces, const int32_t* meta, const uint32_t* legal_to, int32_t B,
                        int32_t out_channels, void* board_tensor_out, cudaStream_t stream, int dtype = 0);
int launch_planes_to_board_tensor(const float* planes_nchw, int32_t B, int32_t C, int32_t board_size,
                                  int32_t out_channels, void* board_tensor_out, cudaStream_t stream, int dtype = 0);
// Opaque storage of a CUtensorMap (128 bytes, 64-byte aligned) so that only the convolution's
// translation unit needs the driver API header.
struct alignas(64) BoardTensorMap { unsigned char opaque[128]; };
int make_board_tensor_map(const void* base, long long rows, int box_rows, BoardTensorMap* out, int channels = 64);
int conv_halo_rows(int S);   // 64-channel kernel: load boxes have 128 + 2 * conv_halo_rows(S) rows
// res_map: the residual tensor through a 128-row-box map (a store map of that buffer), or null
int launch_conv3x3_maps(const BoardTensorMap& in_map, const BoardTensorMap& out_map, const BoardTensorMap* res_map,
                        const void* packed_w, const float* bias, int B, int S, int relu, cudaStream_t st, int dtype = 0);
int* device_error_word();
// The whole 64-filter tower as one cooperative launch (tower_fused.cu).
size_t tower_fused_layer_bytes();
void tower_fused_fill_layer(void* dst, const BoardTensorMap* in_map, const BoardTensorMap& out_map,
                            const BoardTensorMap* res_map, const void* w, const float* bias);
size_t tower_fused_smem_bytes(int S, int n_layers);   // 0: does not fit
int launch_conv_tower(const BoardTensorMap& stem_in_map, const void* layers_dev, int n_layers, int* flags, int tiles_pitch,
                      int* done, int epoch, int B, int S, cudaStream_t st, int dtype = 0);
// The 64-filter tower with the boards resident in shared memory (tower_resident.cu): boards up to
// 15x15, one ordinary launch.  in_map / out_map: boxes of tower_resident_box_rows(S) rows.
size_t tower_resident_layer_bytes();
void tower_resident_fill_layer(void* dst, const void* w, const float* bias, int has_res);
int tower_resident_box_rows(int S);
size_t tower_resident_smem_bytes(int S, int n_layers);   // 0: does not fit
int tower_resident_head_channels_max();
// head_ch > 0: the heads' 1x1 convolutions ride along in the last epilogue (results as launch_head_conv's).
// enc_hist != null: the input is not read through in_map but written by the kernel from Gomoku move histories
// ([B][16] int16, 16-byte aligned; history lengths and sides to move [B]; 17 or 19 planes), as launch_encode_gomoku would.
int launch_conv_tower_resident(const BoardTensorMap& in_map, const BoardTensorMap& out_map, const void* layers_dev,
                               int n_layers, int B, int S, cudaStream_t st, const float* head_w = nullptr,
                               const float* head_b = nullptr, int head_ch = 0, int head_pc = 0, float* hp = nullptr,
                               float* hv = nullptr, int dtype = 0, const int16_t* enc_hist = nullptr,
                               const uint8_t* enc_nh = nullptr, const uint8_t* enc_tm = nullptr, int enc_planes = 0);
// Towers of 128 / 256 channels (tower_wide.cu): cin a multiple of 64 up to 256, cout 128 or 256,
// taps 9 (3x3) or 1 (1x1).  in_map: boxes of conv_wide_box_rows() rows over a cin-channel tensor;
// out_map / res_map (residual, or null): boxes of 128 rows over a cout-channel tensor.
// out_f32 (optional): fp32 [positions][cout] output by plain stores instead of the bf16 tensor.
bool conv_wide_covers(int cin, int cout);
int conv_wide_box_rows();
size_t conv_wide_packed_bytes(int cin, int cout, int taps);
int conv_wide_pack(const float* w, const float* scale, int cout, int cin_real, int cin, int taps, void* packed_out, int dtype = 0);
int launch_conv_wide_maps(const BoardTensorMap& in_map, const BoardTensorMap& out_map, const BoardTensorMap* res_map,
                          const void* packed_w, const float* bias, int B, int S, int cin, int cout, int taps, int relu,
                          cudaStream_t st, float* out_f32 = nullptr, int dtype = 0);

// C: channels of the tower board tensor (a multiple of 64); w: [HC][C]
int launch_head_conv(const void* tower, const float* w, const float* bias, int HC, int pc, float* hp,
                     float* hv, int B, int S, cudaStream_t st, int C = 64, int dtype = 0);
int launch_fc(const float* in, const float* WT, const float* bias, float* out, int B, int K, int Nout, int relu,
              cudaStream_t st);
// Both heads' FC layers in two launches ({policy FC, value FC1}, {softmax, value FC2 + tanh}); policy_in may be
// null (a policy that is already in policy_out); results as the single-layer launchers give them.
int launch_head_fcs(const float* policy_in, const float* WpT, const float* bp, float* policy_out, int policy_k, int policy_size,
                    int softmax, const float* value_in, const float* W1T, const float* b1, float* hidden, int value_k, int H,
                    const float* w2, float b2, float* value_out, int B, cudaStream_t st);
int launch_value_out(const float* hidden, const float* w2, float b2, int H, int B, float* value, cudaStream_t st);
int launch_value_head_static(const void* tower, const float* vw, const float* vb, int vc, const float* W1T,
                             const float* b1, const float* w2, float b2, int H, int B, int S, float* value_out,
                             cudaStream_t st, int dtype = 0);
size_t value_head_static_capacity();

}  // namespace ob200
