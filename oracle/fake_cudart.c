/*
 * A stand-in for the CUDA runtime that lets the reference's own test programs
 * (stride/local/fixed/big_bird/no_fusion *_test.cu, compiled unmodified where they lie)
 * run on a machine WITHOUT a GPU: "device" memory is host memory, kernels are never
 * launched, and every host->device upload is written to $SFB_CAPTURE_DIR.  The uploads
 * are the LUT and mask arrays those programs build, which is what pins the oracle's
 * LUT / mask builders.  TEST INFRASTRUCTURE ONLY; never linked into the product.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { unsigned x, y, z; } dim3_t;

static const char *g_names[256];
static const void *g_funcs[256];
static int g_nfuncs = 0;
static int g_copy_idx = 0;
static dim3_t g_grid, g_block;
static size_t g_smem;
static void *g_stream;
static char g_seen[256];

static FILE *cap_log(void)
{
    static FILE *f = NULL;
    if (!f) {
        const char *dir = getenv("SFB_CAPTURE_DIR");
        char path[1024];
        snprintf(path, sizeof path, "%s/capture.log", dir ? dir : ".");
        f = fopen(path, "w");
        if (!f) f = stderr;
    }
    return f;
}

void **__cudaRegisterFatBinary(void *fatCubin) { (void)fatCubin; static void *h; return &h; }
void __cudaRegisterFatBinaryEnd(void **h) { (void)h; }
void __cudaUnregisterFatBinary(void **h) { (void)h; }
char __cudaInitModule(void **h) { (void)h; return 1; }
void __cudaRegisterFunction(void **h, const char *hostFun, char *deviceFun, const char *deviceName,
                            int thread_limit, void *tid, void *bid, void *bDim, void *gDim, int *wSize)
{
    (void)h; (void)deviceFun; (void)thread_limit; (void)tid; (void)bid; (void)bDim; (void)gDim; (void)wSize;
    if (g_nfuncs < 256) { g_funcs[g_nfuncs] = hostFun; g_names[g_nfuncs] = deviceName; g_nfuncs++; }
}
unsigned __cudaPushCallConfiguration(dim3_t grid, dim3_t block, size_t smem, void *stream)
{
    g_grid = grid; g_block = block; g_smem = smem; g_stream = stream;
    return 0;
}
int __cudaPopCallConfiguration(dim3_t *grid, dim3_t *block, size_t *smem, void **stream)
{
    *grid = g_grid; *block = g_block; *smem = g_smem; *stream = g_stream;
    return 0;
}
int cudaLaunchKernel(const void *func, dim3_t grid, dim3_t block, void **args, size_t smem, void *stream)
{
    (void)args; (void)stream;
    for (int i = 0; i < g_nfuncs; i++)
        if (g_funcs[i] == func && !g_seen[i]) {
            g_seen[i] = 1;
            fprintf(cap_log(), "launch %s grid %u %u %u block %u %u %u smem %zu\n", g_names[i],
                    grid.x, grid.y, grid.z, block.x, block.y, block.z, smem);
            fflush(cap_log());
        }
    return 0;
}
int cudaMalloc(void **p, size_t n) { *p = calloc(1, n ? n : 1); return *p ? 0 : 2; }
int cudaFree(void *p) { free(p); return 0; }
int cudaMemset(void *p, int v, size_t n) { memset(p, v, n); return 0; }
int cudaStreamCreate(void **s) { *s = NULL; return 0; }
int cudaDeviceSynchronize(void) { return 0; }
int cudaMemcpy(void *dst, const void *src, size_t n, int kind)
{
    if (kind == 1 /* host to device */) {
        const char *dir = getenv("SFB_CAPTURE_DIR");
        fprintf(cap_log(), "h2d %d bytes %zu\n", g_copy_idx, n);
        fflush(cap_log());
        if (n <= (8u << 20)) {
            char path[1024];
            snprintf(path, sizeof path, "%s/h2d_%02d.bin", dir ? dir : ".", g_copy_idx);
            FILE *f = fopen(path, "wb");
            if (f) { fwrite(src, 1, n, f); fclose(f); }
        }
        g_copy_idx++;
    }
    memcpy(dst, src, n);
    return 0;
}
