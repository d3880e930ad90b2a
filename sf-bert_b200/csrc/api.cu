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

}  // namespace sfb

extern "C" const char *sfb_last_error(void) { return sfb::error_buffer(); }
extern "C" int sfb_version(void) { return 100; }
