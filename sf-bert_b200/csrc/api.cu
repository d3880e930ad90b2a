// Error reporting and version of libsfbert_b200.
#include "common.cuh"
#include <string.h>

namespace sfb {

char *error_buffer()
{
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return 1;
}

void clear_error() { error_buffer()[0] = 0; }

int check_launch(const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    clear_error();
    return 0;
}

int current_device()
{
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

int device_sm_count(int dev)
{
    static std::atomic<int> cache[64];
    if (dev < 0 || dev >= 64) return 0;
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v > 0) return v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 0;
    cache[dev].store(v, std::memory_order_relaxed);
    return v;
}

}  // namespace sfb

extern "C" const char *sfb_last_error(void) { return sfb::error_buffer(); }
extern "C" int sfb_version(void) { return 100; }
