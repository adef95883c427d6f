// Process-wide status plumbing of the library: last-error text, launch counter, version queries and the pinned
// host allocation helpers the engine's generated library also exports.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace mynn {

static std::mutex g_err_mu;
static char g_err[1024] = "";
std::atomic<long long> g_launches{0};

// Setters of the per-translation-unit copies of the wait budget (see tcgen05.cuh).
static std::vector<int (*)(unsigned long long)> &wait_budget_setters() {
    static std::vector<int (*)(unsigned long long)> v;
    return v;
}
void register_wait_budget_setter(int (*fn)(unsigned long long)) { wait_budget_setters().push_back(fn); }

// Option state read by the launchers (defaults: automatic K split, tensor-core prefill attention, no injected stall).
int g_ksplit_override = 0;
int g_prefill_attention_mode = 1;
int g_fuse_rope = 1;
int g_decode_ring = 1;
std::atomic<int> g_inject_stall{0};

void set_error(const char *fmt, ...) {
    std::lock_guard<std::mutex> lk(g_err_mu);
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

}  // namespace mynn

extern "C" const char *mynn_b200_last_error(void) {
    static thread_local char copy[1024];
    std::lock_guard<std::mutex> lk(mynn::g_err_mu);
    std::memcpy(copy, mynn::g_err, sizeof copy);
    return copy;
}

extern "C" int mynn_b200_abi_version(void) { return 1; }

extern "C" int mynn_b200_compiled_arch(void) {
#ifdef MYNN_COMPILED_ARCH
    return MYNN_COMPILED_ARCH;
#else
    return 0;
#endif
}

extern "C" int mynn_b200_set_option(int option, long long value) {
    using namespace mynn;
    switch (option) {
        case MYNN_OPT_WAIT_BUDGET_US: {
            if (value < 1 || value > 60LL * 1000 * 1000) return fail(MYNN_E_ARG, "set_option: wait budget of %lld us outside [1, 60e6]", value);
            for (auto fn : wait_budget_setters())
                if (fn((unsigned long long)value * 1000ull)) return fail(MYNN_E_CUDA, "set_option: could not update the wait budget on this device");
            return MYNN_OK;
        }
        case MYNN_OPT_KSPLIT:
            if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8) return fail(MYNN_E_ARG, "set_option: K split must be 0, 1, 2, 4 or 8");
            g_ksplit_override = (int)value;
            return MYNN_OK;
        case MYNN_OPT_PREFILL_ATTENTION:
            if (value < -1 || value > 3) return fail(MYNN_E_ARG, "set_option: prefill attention mode %lld outside [-1, 3]", value);
            g_prefill_attention_mode = (int)value;
            return MYNN_OK;
        case MYNN_OPT_INJECT_STALL:
            if (value < 0 || value > 2) return fail(MYNN_E_ARG, "set_option: stall injection %lld outside [0, 2]", value);
            g_inject_stall.store((int)value);
            return MYNN_OK;
        case MYNN_OPT_FUSE_ROPE:
            if (value != 0 && value != 1) return fail(MYNN_E_ARG, "set_option: fused RoPE must be 0 or 1");
            g_fuse_rope = (int)value;
            return MYNN_OK;
        case MYNN_OPT_DECODE_RING:
            if (value != 0 && value != 1) return fail(MYNN_E_ARG, "set_option: decode ring must be 0 or 1");
            g_decode_ring = (int)value;
            return MYNN_OK;
        default:
            return fail(MYNN_E_ARG, "set_option: unknown option %d", option);
    }
}

extern "C" int64_t mynn_b200_launch_count(void) { return mynn::g_launches.load(); }

// Same contract as the engine's helpers (src/codegen/cuda/cpp/common.cu:4-13) except that failure returns NULL
// instead of exiting the process.
extern "C" void *alloc_pinned(size_t bytes) {
    void *p = nullptr;
    cudaError_t e = cudaMallocHost(&p, bytes);
    if (e != cudaSuccess) {
        mynn::set_error("cudaMallocHost(%zu) failed: %s", bytes, cudaGetErrorString(e));
        return nullptr;
    }
    return p;
}

extern "C" void free_pinned(void *p) {
    if (p) cudaFreeHost(p);
}
