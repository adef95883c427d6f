// Process-wide status plumbing of the library: last-error text, launch counter, version queries and the pinned
// host allocation helpers the engine's generated library also exports.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace mynn {

static std::mutex g_err_mu;
static char g_err[1024] = "";
std::atomic<long long> g_launches{0};
int g_pdl_level = [] { const char *e = getenv("MYNN_PDL_LEVEL"); return e ? atoi(e) : 0; }();

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
