// Shared helpers of libsfbert_b200: error reporting, element conversion, LUT access.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>

#include "../../include/sfbert_b200.h"

namespace sfb {

// ---- host: error string (thread local) -----------------------------------------------------
char *error_buffer();
int fail(const char *fmt, ...);
void clear_error();
int check_launch(const char *what);

#define SFB_REQUIRE(cond, ...)                 \
    do {                                       \
        if (!(cond)) return sfb::fail(__VA_ARGS__); \
    } while (0)

static inline cudaStream_t as_stream(sfb_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- host: set-up that is per DEVICE (function attributes, SM count), not per process ----------
// A launcher keeps one DeviceOnce per kernel family:  if (!once.done(dev)) { ...set attributes...; once.mark(dev); }
// Two threads may both run the set-up of a device; setting an attribute twice is harmless.
int current_device();                 // ordinal of the calling thread's current device, -1 on failure
int device_sm_count(int dev);         // cached per device, 0 on failure
struct DeviceOnce {
    std::atomic<uint64_t> mask{0};
    bool done(int dev) const { return dev >= 0 && dev < 64 && ((mask.load(std::memory_order_acquire) >> dev) & 1u); }
    void mark(int dev) { if (dev >= 0 && dev < 64) mask.fetch_or(1ull << dev, std::memory_order_release); }
};

// ---- launches that may overlap the end of the kernel before them ---------------------------------
// A kernel launched with launch_overlapped() may have its CTAs placed while the previous kernel of the stream is
// still draining (programmatic dependent launch): its launch latency and set-up then hide under that tail.  Such a
// kernel calls grid_dependency_wait() before it touches global memory -- the call returns once the previous kernel has
// completed and its writes are visible -- and grid_launch_dependents() right after, which lets the kernel after IT be
// placed as soon as SMs become free.  Both are no-ops in a kernel launched the plain way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) {
        // a driver or a capture mode that refuses the attribute: the same launch, fully serialised
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    }
    return e;
}

// ---- device: element conversion -------------------------------------------------------------
// fp32 -> bf16 bits the way the reference stores S and P (ew_op_gpu.h:241-253): add half a bf16
// ulp of the magnitude, round toward zero, keep the upper 16 bits.
__device__ __forceinline__ uint16_t to_bhalf_bits(float v)
{
    uint32_t u = __float_as_uint(v);
    float e = __uint_as_float(u & 0xff800000u);
    float f;
    asm("fma.rz.ftz.f32 %0, %1, 0f3b800000, %2;" : "=f"(f) : "f"(e), "f"(v));
    return (uint16_t)(__float_as_uint(f) >> 16);
}
__device__ __forceinline__ float from_bhalf_bits(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

template <int DT> struct Elem;
template <> struct Elem<SFB_F32> {
    typedef float type;
    static __device__ __forceinline__ float load(const void *p, size_t i) { return ((const float *)p)[i]; }
    static __device__ __forceinline__ void store(void *p, size_t i, float v) { ((float *)p)[i] = v; }
    static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct Elem<SFB_BF16> {
    typedef uint16_t type;
    static __device__ __forceinline__ float load(const void *p, size_t i) { return from_bhalf_bits(((const uint16_t *)p)[i]); }
    static __device__ __forceinline__ void store(void *p, size_t i, float v) { ((uint16_t *)p)[i] = to_bhalf_bits(v); }
    static __device__ __forceinline__ float round(float v) { return from_bhalf_bits(to_bhalf_bits(v)); }
};
template <> struct Elem<SFB_F16> {
    typedef __half type;
    static __device__ __forceinline__ float load(const void *p, size_t i) { return __half2float(((const __half *)p)[i]); }
    static __device__ __forceinline__ void store(void *p, size_t i, float v) { ((__half *)p)[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};

static inline size_t elem_size(int dt) { return dt == SFB_F32 ? 4 : 2; }
static inline bool valid_dtype(int dt) { return dt == SFB_F32 || dt == SFB_BF16 || dt == SFB_F16; }

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace sfb
