/*
 * Storage types and constants the reference's call sites use (gpu_types.h:48-58,135-137,213 of
 * HeyHaoh/SF-Bert), so that a driver written against the reference compiles unchanged against
 * this library's headers.
 */
#ifndef SFB_DROPIN_GPU_TYPES_H
#define SFB_DROPIN_GPU_TYPES_H

#include <cuda.h>
#include <vector_types.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef unsigned int uint;
typedef unsigned short ushort;
typedef unsigned char uchar;
typedef unsigned long long uint64;

/* bf16 storage: 1 sign, 8 exponent, 7 mantissa bits (gpu_types.h:48-58) */
typedef struct __align__(2) bhalf {
    __host__ __device__ bhalf() {}
    __host__ __device__ bhalf(ushort v) : x(v) {}
    ushort x;
} bhalf;

typedef struct __align__(4) bhalf2 {
    __host__ __device__ bhalf2() {}
    __host__ __device__ bhalf2(uint v) : x(v) {}
    uint x;
} bhalf2;

/* fp16 storage (the OpenAI code the reference derives from calls it ehalf): an ADDITION, used only by the 16-bit
 * overloads below the reference's own signatures */
typedef struct __align__(2) ehalf {
    __host__ __device__ ehalf() {}
    __host__ __device__ ehalf(ushort v) : x(v) {}
    ushort x;
} ehalf;

#define NT_OP 0
#define NN_OP 1
#define TN_OP 2

#ifndef CEIL_DIV
#define CEIL_DIV(x, y) (((x) + (y) - 1) / (y))
#endif

#endif
