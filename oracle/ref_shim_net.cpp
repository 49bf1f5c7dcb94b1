// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points around the reference's own network class
// alphazero::nn::ResNetModel (src/nn/resnet_model.cpp:51-237), compiled from
// the reference's source files against the libtorch that ships inside the
// Python torch wheel (see oracle/Makefile, target ref_net).  Used to pin the
// Python restatement oracle/net_ref.py, to generate tests/golden fixtures,
// and as the timed CPU baseline of the network forward.
#include <torch/torch.h>
#include <chrono>
#include <cstring>
#include <memory>
#include <sstream>
#include <string>

#include "nn/resnet_model.h"

namespace {
struct Net {
    std::shared_ptr<alphazero::nn::ResNetModel> m;
    int64_t in_ch, board, policy;
};
torch::Tensor* find(Net* n, const std::string& name, torch::Tensor& slot) {
    for (auto& kv : n->m->named_parameters(true)) if (kv.key() == name) { slot = kv.value(); return &slot; }
    for (auto& kv : n->m->named_buffers(true)) if (kv.key() == name) { slot = kv.value(); return &slot; }
    return nullptr;
}
}  // namespace

extern "C" {

// Constructs the reference model after torch::manual_seed(seed), so that its
// libtorch default initialisation is reproducible.
void* ref_net_create(int in_ch, int board, int blocks, int filters, int policy, uint64_t seed) {
    try {
        torch::manual_seed(seed);
        auto* n = new Net{std::make_shared<alphazero::nn::ResNetModel>(in_ch, board, blocks, filters, policy),
                          in_ch, board, policy ? policy : board * board};
        n->m->eval();
        return n;
    } catch (const std::exception& e) {
        fprintf(stderr, "ref_net_create: %s\n", e.what());
        return nullptr;
    }
}
void ref_net_destroy(void* h) { delete static_cast<Net*>(h); }

// "name numel\n" for every parameter then every buffer, in module order.
int64_t ref_net_names(void* h, char* buf, int64_t cap) {
    auto* n = static_cast<Net*>(h);
    std::ostringstream os;
    for (auto& kv : n->m->named_parameters(true)) os << kv.key() << ' ' << kv.value().numel() << '\n';
    for (auto& kv : n->m->named_buffers(true)) os << kv.key() << ' ' << kv.value().numel() << '\n';
    std::string s = os.str();
    if ((int64_t)s.size() + 1 <= cap) std::memcpy(buf, s.c_str(), s.size() + 1);
    return (int64_t)s.size() + 1;
}
// Copy a parameter/buffer out as fp32 (int64 buffers are converted). Returns numel or -1.
int64_t ref_net_get(void* h, const char* name, float* out, int64_t cap) {
    torch::NoGradGuard g; torch::Tensor t;
    if (!find(static_cast<Net*>(h), name, t)) return -1;
    auto f = t.detach().to(torch::kFloat32).contiguous();
    if (f.numel() > cap) return f.numel();
    std::memcpy(out, f.data_ptr<float>(), sizeof(float) * f.numel());
    return f.numel();
}
// Overwrite a parameter/buffer from fp32 data. Returns numel or -1.
int64_t ref_net_set(void* h, const char* name, const float* data, int64_t numel) {
    torch::NoGradGuard g; torch::Tensor t;
    if (!find(static_cast<Net*>(h), name, t) || t.numel() != numel) return -1;
    auto src = torch::from_blob(const_cast<float*>(data), t.sizes(), torch::kFloat32);
    t.copy_(src.to(t.dtype()));
    return numel;
}
// ResNetModel::forward on x[B, C, S, S] fp32 (CPU). logp_out[B, policy] is the
// log-softmax the reference returns, value_out[B] the tanh value.  Runs
// `repeats` forwards and returns the mean seconds per forward (-1 on error).
double ref_net_forward(void* h, const float* x, int B, int C, float* logp_out, float* value_out,
                       int threads, int repeats) {
    auto* n = static_cast<Net*>(h);
    try {
        torch::NoGradGuard g;
        if (threads > 0) at::set_num_threads(threads);
        auto xt = torch::from_blob(const_cast<float*>(x), {B, C, n->board, n->board}, torch::kFloat32);
        torch::Tensor p, v; double total = 0;
        for (int r = 0; r < (repeats < 1 ? 1 : repeats); ++r) {
            auto t0 = std::chrono::steady_clock::now();
            std::tie(p, v) = n->m->forward(xt);
            total += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        }
        p = p.contiguous(); v = v.contiguous();
        if (logp_out) std::memcpy(logp_out, p.data_ptr<float>(), sizeof(float) * p.numel());
        if (value_out) std::memcpy(value_out, v.data_ptr<float>(), sizeof(float) * v.numel());
        return total / (repeats < 1 ? 1 : repeats);
    } catch (const std::exception& e) {
        fprintf(stderr, "ref_net_forward: %s\n", e.what());
        return -1.0;
    }
}
int ref_net_threads() { return at::get_num_threads(); }
// ResNetModel::save (src/nn/resnet_model.cpp:813-828): the checkpoint format of the reference.
int ref_net_save(void* h, const char* path) {
    try { static_cast<Net*>(h)->m->save(path); return 0; } catch (const std::exception& e) {
        fprintf(stderr, "ref_net_save: %s\n", e.what()); return -1; }
}

}  // extern "C"
