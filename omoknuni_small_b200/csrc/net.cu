// Network handle: weights under the reference module's names, BatchNorm
// folding, device buffers, and the forward pass as a sequence of launches on
// one stream (stem conv, 2 x blocks residual convs, heads).
//
// Takes the place of alphazero::nn::ResNetModel (reference
// src/nn/resnet_model.cpp:51-237 construction + forward, :594-811 inference).
#include "internal.h"
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <condition_variable>
#include <map>
#include <mutex>
#include <string>
#include <vector>

struct ob200_net {
    ob200_net_config cfg{};
    int cin_pad = 64;               // channels of the input board tensor (input_channels rounded up to 64)
    bool wide = false;              // filters 128 / 256: the streamed-weight kernel; 64: the resident-weight kernel
    int box_in = 0;                 // rows of a load box of the tower kernel in use
    long long rows = 0;             // positions per board tensor (sized for max_batch)
    ob200::BoardTensorMap in_map_load{}, act_load[3]{}, act_store[3]{};
    std::map<std::string, std::vector<float>> host;  // tensors as given
    bool finalized = false;
    std::mutex mu;                  // calls on one handle are serialised
    cudaStream_t stream = nullptr;  // used by the host-buffer calls
    // device: tower
    std::vector<void*> conv_w;      // packed bf16, 1 + 2 * blocks
    std::vector<float*> conv_b;
    void* act_in = nullptr;         // cin_pad channels
    void* act[3] = {nullptr, nullptr, nullptr};      // filters channels each
    const void* tower_out = nullptr;
    int tower_path = -1;            // path of the last forward: 0 per layer, 1 cooperative launch, 2 board-resident
    // the fused tower (64 filters): per-layer descriptors and tile flags on the device
    void* fused_layers = nullptr; int *fused_flags = nullptr, *fused_done = nullptr; int fused_pitch = 0, fused_epoch = 0, fused_final = 0;
    bool fused = false, fused_forced = false;   // forced: OB200_TOWER_FUSED=2 (tests: every batch size)
    // the board-resident tower (64 filters, boards up to 15x15): layer descriptors, whole-board boxes
    void* resident_layers = nullptr; bool resident = false;
    ob200::BoardTensorMap in_map_board{}, out_map_board{};
    int sm_count = 148;
    // device: heads
    float *head_w = nullptr, *head_b = nullptr;      // [pc+vc][64], [pc+vc]
    float *WpT = nullptr, *bp = nullptr, *W1T = nullptr, *b1 = nullptr, *w2 = nullptr;
    float b2 = 0.0f;
    float *hp = nullptr, *hv = nullptr, *hidden = nullptr;
    // device: policy as convolution planes (policy_kind 1): 1x1 convolution on the tensor cores
    void* pol_w = nullptr; float* pol_b = nullptr; float* pol_planes = nullptr; int pol_cout = 0;
    // device + pinned host staging of the host-buffer calls.  Two calls may be in flight per handle: while the
    // results of one travel back to the host on the copy stream, the next one's kernels run.  What the two must
    // not share is doubled (a "slot"): the device output arrays, their pinned landing buffers, the input staging.
    struct Slot {
        bool busy = false;
        int B = 0;
        float *d_policy = nullptr, *d_value = nullptr;
        float *h_policy = nullptr, *h_value = nullptr;
        int16_t* h_hist = nullptr;
        int16_t* d_hist = nullptr;  // [histories | history lengths | sides to move] of the batch in this slot
        int* h_err = nullptr;       // pinned landing word for the device error code
        float *user_policy = nullptr, *user_value = nullptr;
        bool direct = false;        // results are copied straight into the caller's page-locked buffers
        cudaEvent_t computed = nullptr, done = nullptr, hist_ready = nullptr;
    } slot[2];
    std::condition_variable slot_cv;
    cudaStream_t copy_stream = nullptr;   // device -> host copies of results
    cudaStream_t in_stream = nullptr;     // host -> device copies of move histories, ahead of the batch that reads them
    cudaEvent_t planes_copied = nullptr;  // the planes staging buffer has been read by its host -> device copy
    float *d_planes = nullptr;
    float *h_planes = nullptr;
    size_t planes_capacity = 0;     // floats per staging buffer
    std::vector<void*> owned_dev, owned_host;
};

namespace ob200 {
namespace {

constexpr float kBnEps = 1e-5f;     // torch BatchNorm2d default, unchanged by the reference

template <typename T>
int dev_alloc(ob200_net* n, T** out, size_t count, bool zero) {
    void* p = nullptr;
    OB200_CUDA_OK(cudaMalloc(&p, count * sizeof(T)));
    n->owned_dev.push_back(p);
    if (zero) OB200_CUDA_OK(cudaMemset(p, 0, count * sizeof(T)));
    *out = static_cast<T*>(p);
    return OB200_OK;
}
template <typename T>
int host_alloc(ob200_net* n, T** out, size_t count) {
    void* p = nullptr;
    OB200_CUDA_OK(cudaMallocHost(&p, count * sizeof(T)));
    n->owned_host.push_back(p);
    *out = static_cast<T*>(p);
    return OB200_OK;
}
template <typename T>
int upload(ob200_net* n, T** out, const std::vector<T>& v) {
    if (int rc = dev_alloc(n, out, v.size(), false)) return rc;
    OB200_CUDA_OK(cudaMemcpy(*out, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return OB200_OK;
}

// scale = gamma / sqrt(var + eps), shift = beta - mean * scale
int bn_fold(ob200_net* n, const std::string& prefix, int c, std::vector<float>& scale, std::vector<float>& shift) {
    const char* leaves[4] = {".weight", ".bias", ".running_mean", ".running_var"};
    const std::vector<float>* t[4];
    for (int i = 0; i < 4; ++i) {
        auto it = n->host.find(prefix + leaves[i]);
        if (it == n->host.end() || (int)it->second.size() != c)
            return set_error(OB200_ERR_STATE, "ob200_net_finalize: tensor %s%s missing or not of %d elements",
                             prefix.c_str(), leaves[i], c);
        t[i] = &it->second;
    }
    scale.resize(c); shift.resize(c);
    for (int i = 0; i < c; ++i) {
        const float s = (*t[0])[i] / std::sqrt((*t[3])[i] + kBnEps);
        scale[i] = s;
        shift[i] = (*t[1])[i] - (*t[2])[i] * s;
    }
    return OB200_OK;
}

int need(ob200_net* n, const std::string& name, size_t numel, const std::vector<float>** out) {
    auto it = n->host.find(name);
    if (it == n->host.end() || it->second.size() != numel)
        return set_error(OB200_ERR_STATE, "ob200_net_finalize: tensor %s missing or not of %zu elements", name.c_str(),
                         numel);
    *out = &it->second;
    return OB200_OK;
}

int add_conv(ob200_net* n, const std::string& conv, const std::string& bn, int cin_real, int cin) {
    const int F = n->cfg.filters;
    const std::vector<float>* w;
    if (int rc = need(n, conv + ".weight", (size_t)F * cin_real * 9, &w)) return rc;
    std::vector<float> scale, shift;
    if (int rc = bn_fold(n, bn, F, scale, shift)) return rc;
    std::vector<uint16_t> packed((size_t)9 * cin * F);
    if (int rc = ob200_pack_conv3x3_weights_dt(w->data(), scale.data(), F, cin_real, cin, n->cfg.tower_dtype, packed.data())) return rc;
    uint16_t* dw = nullptr; float* db = nullptr;
    if (int rc = upload(n, &dw, packed)) return rc;
    if (int rc = upload(n, &db, shift)) return rc;
    n->conv_w.push_back(dw); n->conv_b.push_back(db);
    return OB200_OK;
}

// One tower layer on the kernel that covers the handle's width.
int tower_conv(ob200_net* n, const BoardTensorMap& in_map, int cin, const BoardTensorMap& out_map,
               const BoardTensorMap* res_map, int layer, int B, cudaStream_t st) {
    const ob200_net_config& c = n->cfg;
    if (n->wide)
        return launch_conv_wide_maps(in_map, out_map, res_map, n->conv_w[layer], n->conv_b[layer], B, c.board_size, cin,
                                     c.filters, 9, 1, st, nullptr, c.tower_dtype);
    return launch_conv3x3_maps(in_map, out_map, res_map, n->conv_w[layer], n->conv_b[layer], B, c.board_size, 1, st, c.tower_dtype);
}

// Load map over a caller's input board tensor holding B boards.
int input_map(ob200_net* n, const void* input_bt, int B, int box_rows, BoardTensorMap* out) {
    return make_board_tensor_map(input_bt, board_geom(n->cfg.board_size, B).PT, box_rows, out, n->cin_pad);
}

// logits[b][plane * S2 + cell] = planes[(G + b * slots + y * GP + x)][plane]: the fp32 output of the
// policy 1x1 convolution, gathered into the NCHW-flattened order of a convolutional policy head.
__global__ void __launch_bounds__(256)
policy_planes_gather_kernel(const float* __restrict__ planes, int pitch, int n_planes, int B, int S,
                            float* __restrict__ logits) {
    const int S2 = S * S, GP = S + 1;
    const long long total = (long long)B * n_planes * S2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int cell = (int)(i % S2);
        const long long t = i / S2;
        const int plane = (int)(t % n_planes), b = (int)(t / n_planes);
        const int y = cell / S, x = cell - y * S;
        logits[i] = planes[((size_t)OB200_GUARD + (size_t)b * GP * GP + y * GP + x) * pitch + plane];
    }
}

}  // namespace
}  // namespace ob200

using namespace ob200;

extern "C" {

int ob200_net_create(const ob200_net_config* cfg, ob200_net** out) {
    if (!cfg || !out) return set_error(OB200_ERR_INVALID, "ob200_net_create: null argument");
    *out = nullptr;
    if (cfg->board_size < 1 || cfg->board_size > OB200_GUARD - 2 || cfg->input_channels < 1 || cfg->blocks < 0 ||
        cfg->policy_size < 1 || cfg->policy_head_ch < 1 || cfg->value_head_ch < 1 || cfg->value_hidden < 1 ||
        cfg->max_batch < 1)
        return set_error(OB200_ERR_INVALID, "ob200_net_create: bad configuration value");
    if (cfg->filters != 64 && cfg->filters != 128 && cfg->filters != 256)
        return set_error(OB200_ERR_UNSUPPORTED, "ob200_net_create: the tower kernels cover filters = 64, 128, 256; got %d",
                         cfg->filters);
    if (cfg->input_channels > (cfg->filters == 64 ? 64 : 256))
        return set_error(OB200_ERR_UNSUPPORTED, "ob200_net_create: input_channels %d too many for filters %d",
                         cfg->input_channels, cfg->filters);
    if (cfg->policy_kind != OB200_POLICY_FC && cfg->policy_kind != OB200_POLICY_CONV_PLANES)
        return set_error(OB200_ERR_INVALID, "ob200_net_create: bad policy_kind %d", cfg->policy_kind);
    if (cfg->tower_dtype != OB200_DTYPE_BF16 && cfg->tower_dtype != OB200_DTYPE_F16)
        return set_error(OB200_ERR_INVALID, "ob200_net_create: bad tower_dtype %d", cfg->tower_dtype);
    if (cfg->policy_kind == OB200_POLICY_CONV_PLANES) {
        if (cfg->filters == 64)
            return set_error(OB200_ERR_UNSUPPORTED, "ob200_net_create: the convolutional policy head needs filters 128 or 256");
        if (cfg->policy_size != cfg->policy_head_ch * cfg->board_size * cfg->board_size || cfg->policy_head_ch > 256)
            return set_error(OB200_ERR_INVALID,
                             "ob200_net_create: convolutional policy head: policy_size must be policy_head_ch * board_size^2, at most 256 planes");
    }
    if (cudaSetDevice(cfg->device) != cudaSuccess) {
        cudaGetLastError();
        return set_error(OB200_ERR_NO_DEVICE, "ob200_net_create: CUDA device %d is not available (there is no CPU path)", cfg->device);
    }
    if (int rc = require_device()) return rc;
    ob200_net* n = new ob200_net;
    n->cfg = *cfg;
    n->cin_pad = (cfg->input_channels + 63) / 64 * 64;
    n->wide = cfg->filters != 64;
    n->box_in = n->wide ? conv_wide_box_rows() : 128 + 2 * conv_halo_rows(cfg->board_size);
    n->rows = board_geom(cfg->board_size, cfg->max_batch).PT;
    *out = n;
    return OB200_OK;
}

void ob200_net_destroy(ob200_net* n) {
    if (!n) return;
    cudaSetDevice(n->cfg.device);
    if (n->stream) { cudaStreamSynchronize(n->stream); cudaStreamDestroy(n->stream); }
    if (n->copy_stream) { cudaStreamSynchronize(n->copy_stream); cudaStreamDestroy(n->copy_stream); }
    if (n->planes_copied) cudaEventDestroy(n->planes_copied);
    if (n->in_stream) { cudaStreamSynchronize(n->in_stream); cudaStreamDestroy(n->in_stream); }
    for (auto& sl : n->slot) {
        if (sl.computed) cudaEventDestroy(sl.computed);
        if (sl.done) cudaEventDestroy(sl.done);
        if (sl.hist_ready) cudaEventDestroy(sl.hist_ready);
    }
    for (void* p : n->owned_dev) cudaFree(p);
    for (void* p : n->owned_host) cudaFreeHost(p);
    delete n;
}

int ob200_net_set_tensor(ob200_net* n, const char* name, const float* data, int64_t numel) {
    if (!n || !name || !data || numel < 0) return set_error(OB200_ERR_INVALID, "ob200_net_set_tensor: bad argument");
    std::lock_guard<std::mutex> lk(n->mu);
    if (n->finalized) return set_error(OB200_ERR_STATE, "ob200_net_set_tensor: weights already finalised");
    const std::string s(name);
    if (s.size() > 19 && s.compare(s.size() - 19, 19, "num_batches_tracked") == 0) return OB200_OK;
    n->host[s].assign(data, data + numel);
    return OB200_OK;
}

int ob200_net_finalize(ob200_net* n) {
    if (!n) return set_error(OB200_ERR_INVALID, "ob200_net_finalize: null handle");
    std::lock_guard<std::mutex> lk(n->mu);
    if (n->finalized) return set_error(OB200_ERR_STATE, "ob200_net_finalize: already finalised");
    const ob200_net_config& c = n->cfg;
    OB200_CUDA_OK(cudaSetDevice(c.device));
    const int F = c.filters, S2 = c.board_size * c.board_size, pc = c.policy_head_ch, vc = c.value_head_ch;
    // tower
    if (int rc = add_conv(n, "input_conv", "input_bn", c.input_channels, n->cin_pad)) return rc;
    for (int i = 0; i < c.blocks; ++i) {
        const std::string p = "res_blocks." + std::to_string(i) + ".";
        if (int rc = add_conv(n, p + "conv1", p + "bn1", F, F)) return rc;
        if (int rc = add_conv(n, p + "conv2", p + "bn2", F, F)) return rc;
    }
    // heads: 1x1 convolutions with BatchNorm folded, policy rows first
    const bool planes_policy = c.policy_kind == OB200_POLICY_CONV_PLANES;
    const int pch = planes_policy ? 0 : pc;        // policy channels that go through the small head kernel
    const std::vector<float>*pw = nullptr, *vw, *fcw, *fcb, *f1w, *f1b, *f2w, *f2b;
    if (!planes_policy)
        if (int rc = need(n, "policy_conv.weight", (size_t)pc * F, &pw)) return rc;
    if (int rc = need(n, "value_conv.weight", (size_t)vc * F, &vw)) return rc;
    std::vector<float> ps, pb, vs, vb;
    if (!planes_policy)
        if (int rc = bn_fold(n, "policy_bn", pc, ps, pb)) return rc;
    if (int rc = bn_fold(n, "value_bn", vc, vs, vb)) return rc;
    std::vector<float> hw((size_t)(pch + vc) * F), hb(pch + vc);
    for (int h = 0; h < pch; ++h) { for (int k = 0; k < F; ++k) hw[(size_t)h * F + k] = (*pw)[(size_t)h * F + k] * ps[h]; hb[h] = pb[h]; }
    for (int h = 0; h < vc; ++h) { for (int k = 0; k < F; ++k) hw[(size_t)(pch + h) * F + k] = (*vw)[(size_t)h * F + k] * vs[h]; hb[pch + h] = vb[h]; }
    if (int rc = upload(n, &n->head_w, hw)) return rc;
    if (int rc = upload(n, &n->head_b, hb)) return rc;
    // fully connected layers, stored transposed ([in][out]) for coalesced reads
    const int Kp = pc * S2, Kv = vc * S2, A = c.policy_size, H = c.value_hidden;
    if (planes_policy) {
        // policy planes: 1x1 convolution with bias, no BatchNorm, no ReLU, run on the tensor cores with the
        // plane count padded to 128 / 256 output channels
        const std::vector<float>*cw, *cb;
        if (int rc = need(n, "policy_conv.weight", (size_t)pc * F, &cw)) return rc;
        if (int rc = need(n, "policy_conv.bias", (size_t)pc, &cb)) return rc;
        n->pol_cout = pc <= 128 ? 128 : 256;
        std::vector<float> wpad((size_t)n->pol_cout * F, 0.0f), bpad(n->pol_cout, 0.0f);
        std::copy(cw->begin(), cw->end(), wpad.begin());
        std::copy(cb->begin(), cb->end(), bpad.begin());
        std::vector<uint16_t> packed(conv_wide_packed_bytes(F, n->pol_cout, 1) / 2);
        if (int rc = conv_wide_pack(wpad.data(), nullptr, n->pol_cout, F, F, 1, packed.data(), c.tower_dtype)) return rc;
        uint16_t* dw = nullptr;
        if (int rc = upload(n, &dw, packed)) return rc;
        n->pol_w = dw;
        if (int rc = upload(n, &n->pol_b, bpad)) return rc;
        if (int rc = dev_alloc(n, &n->pol_planes, (size_t)n->rows * n->pol_cout, false)) return rc;
    } else {
        if (int rc = need(n, "policy_fc.weight", (size_t)A * Kp, &fcw)) return rc;
        if (int rc = need(n, "policy_fc.bias", (size_t)A, &fcb)) return rc;
        std::vector<float> wpt((size_t)Kp * A);
        for (int j = 0; j < A; ++j) for (int i = 0; i < Kp; ++i) wpt[(size_t)i * A + j] = (*fcw)[(size_t)j * Kp + i];
        if (int rc = upload(n, &n->WpT, wpt)) return rc;
        if (int rc = upload(n, &n->bp, *fcb)) return rc;
    }
    if (int rc = need(n, "value_fc1.weight", (size_t)H * Kv, &f1w)) return rc;
    if (int rc = need(n, "value_fc1.bias", (size_t)H, &f1b)) return rc;
    if (int rc = need(n, "value_fc2.weight", (size_t)H, &f2w)) return rc;
    if (int rc = need(n, "value_fc2.bias", 1, &f2b)) return rc;
    std::vector<float> w1t((size_t)Kv * H);
    for (int j = 0; j < H; ++j) for (int i = 0; i < Kv; ++i) w1t[(size_t)i * H + j] = (*f1w)[(size_t)j * Kv + i];
    if (int rc = upload(n, &n->W1T, w1t)) return rc;
    if (int rc = upload(n, &n->b1, *f1b)) return rc;
    if (int rc = upload(n, &n->w2, *f2w)) return rc;
    n->b2 = (*f2b)[0];
    // activations (zeroed once: guards and padding stay zero for the handle's lifetime)
    const int box_store = 128;
    uint8_t* p8 = nullptr;
    if (int rc = dev_alloc(n, &p8, (size_t)n->rows * n->cin_pad * 2, true)) return rc;
    n->act_in = p8;
    if (int rc = make_board_tensor_map(p8, n->rows, n->box_in, &n->in_map_load, n->cin_pad)) return rc;
    for (int i = 0; i < 3; ++i) {
        if (int rc = dev_alloc(n, &p8, (size_t)n->rows * F * 2, true)) return rc;
        n->act[i] = p8;
        if (int rc = make_board_tensor_map(p8, n->rows, n->box_in, &n->act_load[i], F)) return rc;
        if (int rc = make_board_tensor_map(p8, n->rows, box_store, &n->act_store[i], F)) return rc;
    }
    if (!n->wide && tower_fused_smem_bytes(c.board_size, 1 + 2 * c.blocks) != 0) {
        // one cooperative launch for the whole tower: layer descriptors with the buffer rotation of
        // forward_device baked in, and one "tile stored" flag per layer and tile
        const char* env = std::getenv("OB200_TOWER_FUSED");
        const int L = 1 + 2 * c.blocks;
        std::vector<unsigned char> host(tower_fused_layer_bytes() * L);
        int x = 0, y = 1, z = 2;
        tower_fused_fill_layer(host.data(), nullptr, n->act_store[x], nullptr, n->conv_w[0], n->conv_b[0]);
        for (int i = 0; i < c.blocks; ++i) {
            tower_fused_fill_layer(host.data() + tower_fused_layer_bytes() * (1 + 2 * i), &n->act_load[x], n->act_store[y], nullptr,
                                   n->conv_w[1 + 2 * i], n->conv_b[1 + 2 * i]);
            tower_fused_fill_layer(host.data() + tower_fused_layer_bytes() * (2 + 2 * i), &n->act_load[y], n->act_store[z],
                                   &n->act_store[x], n->conv_w[2 + 2 * i], n->conv_b[2 + 2 * i]);
            std::swap(x, z);
        }
        n->fused_final = x;
        unsigned char* dl = nullptr;
        if (int rc = upload(n, &dl, host)) return rc;
        n->fused_layers = dl;
        n->fused_pitch = (int)(board_geom(c.board_size, c.max_batch).Ppad / 128);
        if (int rc = dev_alloc(n, &n->fused_flags, (size_t)L * n->fused_pitch, true)) return rc;
        if (int rc = dev_alloc(n, &n->fused_done, (size_t)L, true)) return rc;
        n->fused = !(env && env[0] == '0');
        n->fused_forced = env && env[0] == '2';
        int dev = 0;
        OB200_CUDA_OK(cudaGetDevice(&dev));
        OB200_CUDA_OK(cudaDeviceGetAttribute(&n->sm_count, cudaDevAttrMultiProcessorCount, dev));
    }
    if (!n->wide && n->cin_pad == 64 && tower_resident_smem_bytes(c.board_size, 1 + 2 * c.blocks) != 0) {
        // boards stay in shared memory through all the layers: one ordinary launch, whole-board boxes
        const char* env = std::getenv("OB200_TOWER_RESIDENT");
        const int L = 1 + 2 * c.blocks;
        std::vector<unsigned char> host(tower_resident_layer_bytes() * L);
        for (int l = 0; l < L; ++l)
            tower_resident_fill_layer(host.data() + tower_resident_layer_bytes() * l, n->conv_w[l], n->conv_b[l], l >= 2 && !(l & 1));
        unsigned char* dl = nullptr;
        if (int rc = upload(n, &dl, host)) return rc;
        n->resident_layers = dl;
        const int box = tower_resident_box_rows(c.board_size);
        if (int rc = make_board_tensor_map(n->act_in, n->rows, box, &n->in_map_board, n->cin_pad)) return rc;
        if (int rc = make_board_tensor_map(n->act[0], n->rows, box, &n->out_map_board, F)) return rc;
        // on unless switched off; an explicit choice about the single-launch tower (OB200_TOWER_FUSED, used by
        // tests and comparisons to pick one of the other two paths) also switches it off unless it is asked for
        n->resident = env ? env[0] != '0' : std::getenv("OB200_TOWER_FUSED") == nullptr;
    }
    const size_t MB = c.max_batch;
    if (int rc = dev_alloc(n, &n->hp, MB * (planes_policy ? 1 : Kp), false)) return rc;
    if (int rc = dev_alloc(n, &n->hv, MB * Kv, false)) return rc;
    if (int rc = dev_alloc(n, &n->hidden, MB * H, false)) return rc;
    for (auto& sl : n->slot) {
        if (int rc = dev_alloc(n, &sl.d_policy, MB * A, false)) return rc;
        if (int rc = dev_alloc(n, &sl.d_value, MB, false)) return rc;
        if (int rc = host_alloc(n, &sl.h_policy, MB * A)) return rc;
        if (int rc = host_alloc(n, &sl.h_value, MB)) return rc;
        // move histories, history lengths and sides to move of a batch share one staging block (34 bytes per board,
        // packed for the batch's size), so that they reach the device in one copy
        if (int rc = host_alloc(n, &sl.h_hist, MB * 17)) return rc;
        if (int rc = dev_alloc(n, &sl.d_hist, MB * 17, false)) return rc;
        OB200_CUDA_OK(cudaEventCreateWithFlags(&sl.hist_ready, cudaEventDisableTiming));
        if (int rc = host_alloc(n, &sl.h_err, 1)) return rc;
        *sl.h_err = 0;
        OB200_CUDA_OK(cudaEventCreateWithFlags(&sl.computed, cudaEventDisableTiming));
        OB200_CUDA_OK(cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming));
    }
    n->planes_capacity = MB * (size_t)std::max(c.input_channels, 19) * S2;
    if (int rc = dev_alloc(n, &n->d_planes, n->planes_capacity, false)) return rc;
    if (int rc = host_alloc(n, &n->h_planes, n->planes_capacity)) return rc;
    OB200_CUDA_OK(cudaStreamCreateWithFlags(&n->stream, cudaStreamNonBlocking));
    OB200_CUDA_OK(cudaStreamCreateWithFlags(&n->copy_stream, cudaStreamNonBlocking));
    OB200_CUDA_OK(cudaStreamCreateWithFlags(&n->in_stream, cudaStreamNonBlocking));
    OB200_CUDA_OK(cudaEventCreateWithFlags(&n->planes_copied, cudaEventDisableTiming));
    OB200_CUDA_OK(cudaEventRecord(n->planes_copied, n->stream));
    OB200_CUDA_OK(cudaDeviceSynchronize());
    n->host.clear();
    n->finalized = true;
    return OB200_OK;
}

}  // extern "C"

namespace ob200 {
namespace {

// The tower alone; returns the index of the activation buffer that holds its output in *out_buf.
// `input_bt`: a board tensor of cin_pad channels holding the B input boards (the handle's own staging
// tensor or a caller's).
// heads_done (optional): the caller wants the heads' 1x1 convolutions too; set when the tower kernel took them along.
// gomoku (optional): the input is given as Gomoku move histories on the device instead of a board tensor; the
// board-resident tower writes its own input rows from them, the other paths run the encoder kernel first.
struct GomokuInput { const int16_t* hist; const uint8_t* nh; const uint8_t* tm; };
int tower_device(ob200_net* n, const void* input_bt, int B, int* out_buf, cudaStream_t st, bool* heads_done = nullptr,
                 const GomokuInput* gomoku = nullptr) {
    const ob200_net_config& c = n->cfg;
    if (gomoku) input_bt = n->act_in;
    const int S = c.board_size;
    const int F = c.filters;
    int x = 0, y = 1, z = 2;
    bool done = false;
    const bool own_input = input_bt == n->act_in;
    if (n->resident) {
        BoardTensorMap board_map;
        if (!own_input)
            if (int rc = input_map(n, input_bt, B, tower_resident_box_rows(S), &board_map)) return rc;
        // the heads' 1x1 convolutions ride along when they are few (FC policy head: policy + value channels)
        const int hc = c.policy_head_ch + c.value_head_ch;
        const bool with_heads = heads_done && c.policy_kind != OB200_POLICY_CONV_PLANES && hc <= tower_resident_head_channels_max();
        const int rc = launch_conv_tower_resident(own_input ? n->in_map_board : board_map, n->out_map_board, n->resident_layers,
                                                  1 + 2 * c.blocks, B, S, st, n->head_w, n->head_b, with_heads ? hc : 0,
                                                  with_heads ? c.policy_head_ch : 0, n->hp, n->hv, c.tower_dtype,
                                                  gomoku ? gomoku->hist : nullptr, gomoku ? gomoku->nh : nullptr,
                                                  gomoku ? gomoku->tm : nullptr, c.input_channels);
        if (rc == OB200_OK) { done = true; x = 0; n->tower_path = 2; if (heads_done) *heads_done = with_heads; }
        else if (rc == OB200_ERR_UNSUPPORTED) n->resident = false;
        else return rc;
    }
    if (!done && gomoku)       // the other tower paths read an input tensor: encode into the handle's own
        if (int rc = launch_encode_gomoku(gomoku->hist, gomoku->nh, gomoku->tm, B, S, c.input_channels, n->cin_pad, n->act_in, st,
                                          c.tower_dtype)) return rc;
    BoardTensorMap conv_map;
    if (!done && !own_input)
        if (int rc = input_map(n, input_bt, B, n->box_in, &conv_map)) return rc;
    const BoardTensorMap& in_map = own_input ? n->in_map_load : conv_map;
    // The fused tower pays off in a window of batch sizes (measured, 15x15: 4.5 % faster at 1,024 boards,
    // equal at 512, 45 % slower at 64, 19 % slower at 4,096).  Below about 8 tiles per CTA and layer the
    // hand-over of tiles through flags in global memory (store complete -> flag -> poll, about 3 us per
    // layer on the critical path) costs more than a kernel boundary; and it keeps two activation tiles
    // in flight per CTA, which covers L2 latency but not DRAM latency, so the three rotating
    // activation tensors must stay resident in L2 (40 MB each at most; 15x15 boards: 1,220 per batch).
    const BoardGeom bg = board_geom(S, B);
    const bool l2_resident = (size_t)bg.PT * 128 <= ((size_t)40 << 20);
    const bool enough_tiles = bg.Ppad / 128 >= 8LL * n->sm_count;
    // The tile flags carry a per-launch epoch kept on the host: a launch replayed from a captured
    // graph would see its own earlier flags, so a capturing stream gets the per-layer kernels.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &capturing) != cudaSuccess) { cudaGetLastError(); capturing = cudaStreamCaptureStatusNone; }
    if (!done && n->fused && capturing == cudaStreamCaptureStatusNone && (n->fused_forced || (l2_resident && enough_tiles))) {
        if (++n->fused_epoch == 0) ++n->fused_epoch;   // flags start at zero: epoch 0 is never used
        const int rc = launch_conv_tower(in_map, n->fused_layers, 1 + 2 * c.blocks, n->fused_flags, n->fused_pitch,
                                         n->fused_done, n->fused_epoch, B, S, st, c.tower_dtype);
        if (rc == OB200_OK) { done = true; x = n->fused_final; n->tower_path = 1; }
        else if (rc == OB200_ERR_UNSUPPORTED) n->fused = false;   // not launchable here: layer by layer from now on
        else return rc;
    }
    if (!done) {
        n->tower_path = 0;
        if (int rc = tower_conv(n, in_map, n->cin_pad, n->act_store[x], nullptr, 0, B, st)) return rc;
        for (int i = 0; i < c.blocks; ++i) {
            if (int rc = tower_conv(n, n->act_load[x], F, n->act_store[y], nullptr, 1 + 2 * i, B, st)) return rc;
            if (int rc = tower_conv(n, n->act_load[y], F, n->act_store[z], &n->act_store[x], 2 + 2 * i, B, st)) return rc;
            std::swap(x, z);
        }
    }
    n->tower_out = n->act[x];
    *out_buf = x;
    return OB200_OK;
}

int forward_device(ob200_net* n, const void* input_bt, int B, float* policy_out, float* value_out,
                   int out_kind, cudaStream_t st, const GomokuInput* gomoku = nullptr) {
    const ob200_net_config& c = n->cfg;
    const int S = c.board_size;
    const int F = c.filters;
    int x = 0;
    bool heads_done = false;
    if (int rc = tower_device(n, input_bt, B, &x, st, &heads_done, gomoku)) return rc;
    const int S2 = S * S, pc = c.policy_head_ch, vc = c.value_head_ch;
    if (c.policy_kind == OB200_POLICY_CONV_PLANES) {
        if (int rc = launch_conv_wide_maps(n->act_load[x], n->act_load[x], nullptr, n->pol_w, n->pol_b, B, S, F, n->pol_cout, 1, 0,
                                           st, n->pol_planes, c.tower_dtype)) return rc;
        const long long total = (long long)B * pc * S2;
        policy_planes_gather_kernel<<<(unsigned)std::min<long long>((total + 255) / 256, 148 * 16), 256, 0, st>>>(
            n->pol_planes, n->pol_cout, pc, B, S, policy_out);
        OB200_LAUNCHED("policy_planes_gather_kernel");
        if (int rc = launch_head_conv(n->act[x], n->head_w, n->head_b, vc, 0, n->hv, n->hv, B, S, st, F, c.tower_dtype)) return rc;
    } else if (!heads_done) {
        if (int rc = launch_head_conv(n->act[x], n->head_w, n->head_b, pc + vc, pc, n->hp, n->hv, B, S, st, F, c.tower_dtype)) return rc;
    }
    // the FC layers of both heads: {policy FC, value FC1} in one launch, {softmax, value FC2 + tanh} in the next
    const bool fc_policy = c.policy_kind != OB200_POLICY_CONV_PLANES;
    if (int rc = launch_head_fcs(fc_policy ? n->hp : nullptr, n->WpT, n->bp, policy_out, pc * S2, c.policy_size,
                                 out_kind == OB200_OUT_PROBS, n->hv, n->W1T, n->b1, n->hidden, vc * S2, c.value_hidden, n->w2,
                                 n->b2, value_out, B, st)) return rc;
    counters().evals.fetch_add((uint64_t)B, std::memory_order_relaxed);
    counters().batches.fetch_add(1, std::memory_order_relaxed);
    return OB200_OK;
}

int check_call(ob200_net* n, int B, const void* a, const void* b, const void* c, int out_kind, const char* who) {
    if (!n || !a || !b || !c) return set_error(OB200_ERR_INVALID, "%s: null argument", who);
    if (!n->finalized) return set_error(OB200_ERR_STATE, "%s: weights not finalised", who);
    if (B < 1 || B > n->cfg.max_batch)
        return set_error(OB200_ERR_TOO_LARGE, "%s: batch %d outside [1, max_batch %d]", who, B, n->cfg.max_batch);
    if (out_kind != OB200_OUT_PROBS && out_kind != OB200_OUT_LOGITS)
        return set_error(OB200_ERR_INVALID, "%s: bad out_kind %d", who, out_kind);
    return OB200_OK;
}

bool is_pinned_host(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeHost;
}

// A free slot for a host-buffer call; with `wait` the caller sleeps until one of the two is handed back.
// The handle's mutex is held (lk).  Returns the slot index, or -1 when both are pending and !wait.
int acquire_slot(ob200_net* n, std::unique_lock<std::mutex>& lk, bool wait) {
    for (;;) {
        for (int i = 0; i < 2; ++i)
            if (!n->slot[i].busy) { n->slot[i].busy = true; return i; }
        if (!wait) return -1;
        n->slot_cv.wait(lk);
    }
}
void release_slot(ob200_net* n, int i) {
    { std::lock_guard<std::mutex> lk(n->mu); n->slot[i].busy = false; }
    n->slot_cv.notify_one();
}

// After the forward has been enqueued on the handle's stream: results travel back on the copy stream, so the
// next call's kernels can run meanwhile.  Outputs the caller keeps in page-locked memory are written by the
// copy engine directly; pageable ones go through the slot's pinned buffers (copied out in wait_slot).
int enqueue_results(ob200_net* n, int si, int B, float* policy_out, float* value_out) {
    ob200_net::Slot& sl = n->slot[si];
    const size_t A = n->cfg.policy_size;
    sl.B = B; sl.user_policy = policy_out; sl.user_value = value_out;
    sl.direct = is_pinned_host(policy_out) && is_pinned_host(value_out);
    OB200_CUDA_OK(cudaEventRecord(sl.computed, n->stream));
    OB200_CUDA_OK(cudaStreamWaitEvent(n->copy_stream, sl.computed, 0));
    OB200_CUDA_OK(cudaMemcpyAsync(sl.direct ? policy_out : sl.h_policy, sl.d_policy, (size_t)B * A * sizeof(float), cudaMemcpyDeviceToHost, n->copy_stream));
    OB200_CUDA_OK(cudaMemcpyAsync(sl.direct ? value_out : sl.h_value, sl.d_value, (size_t)B * sizeof(float), cudaMemcpyDeviceToHost, n->copy_stream));
    int* errw = device_error_word();
    if (errw) OB200_CUDA_OK(cudaMemcpyAsync(sl.h_err, errw, sizeof(int), cudaMemcpyDeviceToHost, n->copy_stream));
    OB200_CUDA_OK(cudaEventRecord(sl.done, n->copy_stream));
    return OB200_OK;
}

// Waits for a slot's results, reports a kernel that gave up on a bounded wait, hands the slot back.
int wait_slot(ob200_net* n, int si) {
    ob200_net::Slot& sl = n->slot[si];
    const size_t A = n->cfg.policy_size;
    const cudaError_t e = cudaEventSynchronize(sl.done);
    int rc = OB200_OK;
    if (e != cudaSuccess) rc = set_error(OB200_ERR_CUDA, "waiting for the results failed: %s", cudaGetErrorString(e));
    else if (*sl.h_err) {
        const int err = *sl.h_err;
        *sl.h_err = 0;
        int* errw = device_error_word();
        if (errw) { cudaMemsetAsync(errw, 0, sizeof(int), n->copy_stream); cudaStreamSynchronize(n->copy_stream); }
        rc = set_error(OB200_ERR_TIMEOUT, "a tower kernel gave up on a bounded wait (role code %d); outputs are not valid", err);
    } else if (!sl.direct) {
        std::memcpy(sl.user_policy, sl.h_policy, (size_t)sl.B * A * sizeof(float));
        std::memcpy(sl.user_value, sl.h_value, (size_t)sl.B * sizeof(float));
    }
    release_slot(n, si);
    return rc;
}

// Gomoku histories -> staging -> device -> encoder -> forward -> results on their way back.  Handle mutex held.
int enqueue_gomoku(ob200_net* n, int si, const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move, int32_t B,
                   float* policy_out, float* value_out, int32_t out_kind) {
    ob200_net::Slot& sl = n->slot[si];
    const size_t hist_bytes = (size_t)B * 16 * sizeof(int16_t);
    uint8_t* h8 = reinterpret_cast<uint8_t*>(sl.h_hist);
    uint8_t* d8 = reinterpret_cast<uint8_t*>(sl.d_hist);
    std::memcpy(h8, history, hist_bytes);
    std::memcpy(h8 + hist_bytes, n_hist, (size_t)B);
    std::memcpy(h8 + hist_bytes + B, to_move, (size_t)B);
    // the copy goes on a stream of its own, so that it runs while the batch ahead still computes; the slot's device
    // block is free: its previous batch was waited for before the slot was handed out again
    OB200_CUDA_OK(cudaMemcpyAsync(d8, h8, hist_bytes + 2 * (size_t)B, cudaMemcpyHostToDevice, n->in_stream));
    OB200_CUDA_OK(cudaEventRecord(sl.hist_ready, n->in_stream));
    OB200_CUDA_OK(cudaStreamWaitEvent(n->stream, sl.hist_ready, 0));
    const GomokuInput g{sl.d_hist, d8 + hist_bytes, d8 + hist_bytes + B};
    if (int rc = forward_device(n, nullptr, B, sl.d_policy, sl.d_value, out_kind, n->stream, &g)) return rc;
    return enqueue_results(n, si, B, policy_out, value_out);
}

}  // namespace
}  // namespace ob200

namespace ob200 {
// For the search loop: forward on device move histories, probabilities out, no locking
// beyond the handle's (the search is the handle's only user while it runs).
int net_forward_gomoku_for_search(ob200_net* n, const int16_t* hist, const uint8_t* nh, const uint8_t* tm, int B, float* policy,
                                  float* value, cudaStream_t st) {
    if (!n || !n->finalized) return set_error(OB200_ERR_STATE, "search: the network is not finalised");
    std::lock_guard<std::mutex> lk(n->mu);
    const GomokuInput g{hist, nh, tm};
    return forward_device(n, nullptr, B, policy, value, OB200_OUT_PROBS, st, &g);
}
const ob200_net_config* net_config(ob200_net* n) { return (n && n->finalized) ? &n->cfg : nullptr; }
}  // namespace ob200

extern "C" {

int ob200_net_infer_planes(ob200_net* n, const float* planes, int32_t B, int32_t C, float* policy_out,
                           float* value_out, int32_t out_kind) {
    if (int rc = check_call(n, B, planes, policy_out, value_out, out_kind, "ob200_net_infer_planes")) return rc;
    std::unique_lock<std::mutex> lk(n->mu);
    const ob200_net_config& c = n->cfg;
    const size_t S2 = (size_t)c.board_size * c.board_size;
    if (C < 1 || (size_t)B * C * S2 > n->planes_capacity)
        return set_error(OB200_ERR_TOO_LARGE, "ob200_net_infer_planes: %d planes x batch %d exceeds the staging buffer", C, B);
    OB200_CUDA_OK(cudaSetDevice(c.device));
    // as ResNetModel::forward: the first min(C, input_channels) planes are used (:117-147);
    // planes beyond input_channels are dropped while staging
    const int used = C < c.input_channels ? C : c.input_channels;
    const int si = acquire_slot(n, lk, true);
    OB200_CUDA_OK(cudaEventSynchronize(n->planes_copied));      // the previous call's copy has read the staging buffer
    for (int b = 0; b < B; ++b)
        std::memcpy(n->h_planes + (size_t)b * used * S2, planes + (size_t)b * C * S2, (size_t)used * S2 * sizeof(float));
    int rc = OB200_OK;
    auto step = [&](int r) { if (!rc) rc = r; };
    if (cudaMemcpyAsync(n->d_planes, n->h_planes, (size_t)B * used * S2 * sizeof(float), cudaMemcpyHostToDevice, n->stream) != cudaSuccess ||
        cudaEventRecord(n->planes_copied, n->stream) != cudaSuccess)
        rc = set_error(OB200_ERR_CUDA, "ob200_net_infer_planes: copying the planes to the device failed");
    step(rc ? rc : launch_planes_to_board_tensor(n->d_planes, B, used, c.board_size, n->cin_pad, n->act_in, n->stream, c.tower_dtype));
    step(rc ? rc : forward_device(n, n->act_in, B, n->slot[si].d_policy, n->slot[si].d_value, out_kind, n->stream));
    step(rc ? rc : enqueue_results(n, si, B, policy_out, value_out));
    lk.unlock();
    if (rc) { release_slot(n, si); return rc; }
    return wait_slot(n, si);
}

static int check_gomoku(ob200_net* n, const uint8_t* n_hist, const uint8_t* to_move, const char* who) {
    if (!n_hist || !to_move) return set_error(OB200_ERR_INVALID, "%s: null argument", who);
    const ob200_net_config& c = n->cfg;
    if (c.input_channels != 17 && c.input_channels != 19)
        return set_error(OB200_ERR_UNSUPPORTED, "%s: the Gomoku encoder makes 17 or 19 planes; the network takes %d", who, c.input_channels);
    return OB200_OK;
}

int ob200_net_infer_gomoku(ob200_net* n, const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                           int32_t B, float* policy_out, float* value_out, int32_t out_kind) {
    if (int rc = check_call(n, B, history, policy_out, value_out, out_kind, "ob200_net_infer_gomoku")) return rc;
    if (int rc = check_gomoku(n, n_hist, to_move, "ob200_net_infer_gomoku")) return rc;
    std::unique_lock<std::mutex> lk(n->mu);
    OB200_CUDA_OK(cudaSetDevice(n->cfg.device));
    const int si = acquire_slot(n, lk, true);
    const int rc = enqueue_gomoku(n, si, history, n_hist, to_move, B, policy_out, value_out, out_kind);
    lk.unlock();
    if (rc) { release_slot(n, si); return rc; }
    return wait_slot(n, si);      // without the handle's mutex: another thread's call is enqueued meanwhile
}

int ob200_net_submit_gomoku(ob200_net* n, const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                            int32_t B, float* policy_out, float* value_out, int32_t out_kind, int32_t* ticket_out) {
    if (!ticket_out) return set_error(OB200_ERR_INVALID, "ob200_net_submit_gomoku: null ticket");
    *ticket_out = -1;
    if (int rc = check_call(n, B, history, policy_out, value_out, out_kind, "ob200_net_submit_gomoku")) return rc;
    if (int rc = check_gomoku(n, n_hist, to_move, "ob200_net_submit_gomoku")) return rc;
    std::unique_lock<std::mutex> lk(n->mu);
    OB200_CUDA_OK(cudaSetDevice(n->cfg.device));
    const int si = acquire_slot(n, lk, false);
    if (si < 0) return set_error(OB200_ERR_STATE, "ob200_net_submit_gomoku: two calls are pending on this handle already; wait for one first");
    const int rc = enqueue_gomoku(n, si, history, n_hist, to_move, B, policy_out, value_out, out_kind);
    lk.unlock();
    if (rc) { release_slot(n, si); return rc; }
    *ticket_out = si;
    return OB200_OK;
}

int ob200_net_wait(ob200_net* n, int32_t ticket) {
    if (!n || ticket < 0 || ticket > 1) return set_error(OB200_ERR_INVALID, "ob200_net_wait: bad handle or ticket %d", ticket);
    {
        std::lock_guard<std::mutex> lk(n->mu);
        if (!n->slot[ticket].busy) return set_error(OB200_ERR_STATE, "ob200_net_wait: ticket %d is not pending", ticket);
    }
    if (cudaSetDevice(n->cfg.device) != cudaSuccess) { cudaGetLastError(); return set_error(OB200_ERR_CUDA, "ob200_net_wait: cannot select the device"); }
    return wait_slot(n, ticket);
}

int ob200_net_forward_device(ob200_net* n, const void* input_board_tensor, int32_t B, float* policy_out,
                             float* value_out, int32_t out_kind, ob200_stream stream) {
    if (int rc = check_call(n, B, input_board_tensor, policy_out, value_out, out_kind, "ob200_net_forward_device")) return rc;
    std::lock_guard<std::mutex> lk(n->mu);
    OB200_CUDA_OK(cudaSetDevice(n->cfg.device));
    return forward_device(n, input_board_tensor, B, policy_out, value_out, out_kind, as_stream(stream));
}

int ob200_net_forward_gomoku_device(ob200_net* n, const int16_t* history, const uint8_t* n_hist, const uint8_t* to_move,
                                    int32_t B, float* policy_out, float* value_out, int32_t out_kind, ob200_stream stream) {
    if (int rc = check_call(n, B, history, policy_out, value_out, out_kind, "ob200_net_forward_gomoku_device")) return rc;
    if (int rc = check_gomoku(n, n_hist, to_move, "ob200_net_forward_gomoku_device")) return rc;
    if ((uintptr_t)history & 15) return set_error(OB200_ERR_INVALID, "ob200_net_forward_gomoku_device: history must be 16-byte aligned");
    std::lock_guard<std::mutex> lk(n->mu);
    OB200_CUDA_OK(cudaSetDevice(n->cfg.device));
    const GomokuInput g{history, n_hist, to_move};
    return forward_device(n, nullptr, B, policy_out, value_out, out_kind, as_stream(stream), &g);
}

const void* ob200_net_debug_tower_output(ob200_net* n) { return n ? n->tower_out : nullptr; }
int32_t ob200_net_debug_tower_path(ob200_net* n) { return n ? n->tower_path : -1; }

int ob200_net_tower_device(ob200_net* n, const void* input_board_tensor, int32_t B, ob200_stream stream) {
    if (!n || !input_board_tensor) return set_error(OB200_ERR_INVALID, "ob200_net_tower_device: null argument");
    if (!n->finalized) return set_error(OB200_ERR_STATE, "ob200_net_tower_device: weights not finalised");
    if (B < 1 || B > n->cfg.max_batch)
        return set_error(OB200_ERR_TOO_LARGE, "ob200_net_tower_device: batch %d outside [1, max_batch %d]", B, n->cfg.max_batch);
    std::lock_guard<std::mutex> lk(n->mu);
    OB200_CUDA_OK(cudaSetDevice(n->cfg.device));
    int x = 0;
    return tower_device(n, input_board_tensor, B, &x, as_stream(stream));
}

int ob200_net_value_head_noalloc(ob200_net* n, const void* tower_board_tensor, int32_t B, float* value_out,
                                 ob200_stream stream) {
    if (!n || !tower_board_tensor || !value_out)
        return set_error(OB200_ERR_INVALID, "ob200_net_value_head_noalloc: null argument");
    if (!n->finalized) return set_error(OB200_ERR_STATE, "ob200_net_value_head_noalloc: weights not finalised");
    if (B < 1) return set_error(OB200_ERR_INVALID, "ob200_net_value_head_noalloc: batch %d", B);
    // like every other call on a handle: one call at a time, on the handle's own device (the scratch array
    // is looked up per device, and the weights live on this one)
    std::lock_guard<std::mutex> lk(n->mu);
    const ob200_net_config& c = n->cfg;
    OB200_CUDA_OK(cudaSetDevice(c.device));
    if (int rc = require_device()) return rc;
    const int pc = c.policy_kind == OB200_POLICY_CONV_PLANES ? 0 : c.policy_head_ch;
    if (c.filters != 64)
        return set_error(OB200_ERR_UNSUPPORTED, "ob200_net_value_head_noalloc: covers towers of 64 filters");
    return launch_value_head_static(tower_board_tensor, n->head_w + (size_t)pc * c.filters, n->head_b + pc,
                                    c.value_head_ch, n->W1T, n->b1, n->w2, n->b2, c.value_hidden, B, c.board_size,
                                    value_out, as_stream(stream), c.tower_dtype);
}

int64_t ob200_value_head_noalloc_capacity(void) { return (int64_t)value_head_static_capacity(); }
int32_t ob200_net_input_tensor_channels(ob200_net* n) { return n ? n->cin_pad : 0; }

}  // extern "C"
