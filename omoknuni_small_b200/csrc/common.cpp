#include "common.h"
#include <mutex>

namespace ob200 {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

Counters& counters() {
    static Counters c;
    return c;
}

int require_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(OB200_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    }
    static std::mutex mu;
    static int cached[64];
    static bool have[64];
    std::lock_guard<std::mutex> lk(mu);
    if (dev >= 0 && dev < 64 && have[dev])
        return cached[dev] == 10 ? OB200_OK
                                 : set_error(OB200_ERR_NO_DEVICE, "device %d is sm_%d, need sm_100", dev, cached[dev] * 10);
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return set_error(OB200_ERR_NO_DEVICE, "cannot query device %d", dev);
    if (dev >= 0 && dev < 64) { cached[dev] = major; have[dev] = true; }
    if (major != 10)
        return set_error(OB200_ERR_NO_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
    return OB200_OK;
}

}  // namespace ob200

extern "C" {

const char* ob200_last_error(void) { return ob200::g_err; }
int ob200_version(void) { return OB200_VERSION; }

int ob200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    int ok = 0;
    for (int d = 0; d < n; ++d) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess && major == 10) ++ok;
    }
    return ok;
}

int ob200_get_counters(ob200_counters* out) {
    if (!out) return ob200::set_error(OB200_ERR_INVALID, "ob200_get_counters: null output");
    auto& c = ob200::counters();
    out->evals = c.evals.load(); out->batches = c.batches.load();
    out->selections = c.selections.load(); out->backups = c.backups.load();
    out->kernel_launches = c.launches.load();
    return OB200_OK;
}
void ob200_reset_counters(void) {
    auto& c = ob200::counters();
    c.evals = 0; c.batches = 0; c.selections = 0; c.backups = 0; c.launches = 0;
}

int32_t ob200_tree_pitch(int32_t n_children) { return n_children <= 0 ? 0 : (n_children + 3) / 4 * 4; }
int32_t ob200_tree_mask_words(int32_t n_children) { return n_children <= 0 ? 0 : (n_children + 31) / 32; }

int64_t ob200_board_tensor_positions(int32_t board_size, int32_t B) {
    if (board_size <= 0 || B < 0) return 0;
    return ob200::board_geom(board_size, B).PT;
}
int64_t ob200_board_tensor_bytes(int32_t board_size, int32_t B, int32_t channels) {
    if (board_size <= 0 || B < 0 || channels <= 0) return 0;
    return ob200::board_geom(board_size, B).PT * (int64_t)((channels + 7) / 8 * 8) * 2;
}

}  // extern "C"
