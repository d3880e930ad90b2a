// Fused bias + residual + LayerNorm: one pass over HBM (read x and resid, write out and,
// optionally, the pre-norm sum), one warp per row with 16-byte accesses and the row held in
// registers.  Replaces three launches of the reference (cuda_kernels.h:334-372,449-469).
#include "attn.cuh"

namespace sfb {

template <int DT> struct Vec8;
template <> struct Vec8<SFB_F32> {
    static constexpr int N = 4;  // elements per 16-byte access
    static __device__ __forceinline__ void decode(float (&v)[4], const uint4 &u)
    {
        v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
    }
    static __device__ __forceinline__ uint4 encode(const float (&v)[4])
    {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
    static __device__ __forceinline__ void load(float (&v)[4], const void *p, size_t i)
    {
        float4 t = *(const float4 *)((const float *)p + i);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(void *p, size_t i, const float (&v)[4])
    {
        *(float4 *)((float *)p + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec8<SFB_BF16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void decode(float (&v)[8], const uint4 &u)
    {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; t++) {
            v[2 * t] = __uint_as_float(w[t] << 16);
            v[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 encode(const float (&v)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; t++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
            w[t] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ void load(float (&v)[8], const void *p, size_t i)
    {
        uint4 u = *(const uint4 *)((const uint16_t *)p + i);
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; t++) {
            v[2 * t] = __uint_as_float(w[t] << 16);
            v[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(void *p, size_t i, const float (&v)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; t++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
            w[t] = *reinterpret_cast<uint32_t *>(&h);
        }
        *(uint4 *)((uint16_t *)p + i) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Vec8<SFB_F16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void decode(float (&v)[8], const uint4 &u)
    {
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; t++) {
            float2 f = __half22float2(*reinterpret_cast<__half2 *>(&w[t]));
            v[2 * t] = f.x;
            v[2 * t + 1] = f.y;
        }
    }
    static __device__ __forceinline__ uint4 encode(const float (&v)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; t++) {
            __half2 h = __floats2half2_rn(v[2 * t], v[2 * t + 1]);
            w[t] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ void load(float (&v)[8], const void *p, size_t i)
    {
        uint4 u = *(const uint4 *)((const uint16_t *)p + i);
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; t++) {
            float2 f = __half22float2(*reinterpret_cast<__half2 *>(&w[t]));
            v[2 * t] = f.x;
            v[2 * t + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(void *p, size_t i, const float (&v)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; t++) {
            __half2 h = __floats2half2_rn(v[2 * t], v[2 * t + 1]);
            w[t] = *reinterpret_cast<uint32_t *>(&h);
        }
        *(uint4 *)((uint16_t *)p + i) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// streamed once: 16 bytes that bypass L1 on the way in, and leave L2 first on the way out
__device__ __forceinline__ uint4 ld_stream16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_stream16(void *p, const uint4 &v)
{
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// CHUNKS 16-byte accesses per lane: hidden <= 32 * CHUNKS * N.  One warp per row, 8 warps per CTA, a fixed grid of
// warps striding over the rows.  bias, gain and beta sit in shared memory as fp32 (read once per CTA; from global
// memory they were three times the row's own bytes through L1 for every row).  All of a row's loads are issued before
// anything waits for one of them; with PREFETCH the next row's loads are issued before this row's arithmetic.
// A row is read once, by the warp that later writes it, so out (or sum_out) may be x or resid themselves.
template <int DT, int CHUNKS, bool HAS_RESID, bool PREFETCH>
__global__ void __launch_bounds__(256) bias_residual_layernorm_kernel(void *out, void *sum_out,
                                                                     float *__restrict__ mean, float *__restrict__ rstd,
                                                                     const void *x, const float *__restrict__ bias,
                                                                     const void *resid, const float *__restrict__ gain,
                                                                     const float *__restrict__ beta, uint32_t m, uint32_t hidden)
{
    constexpr int N = Vec8<DT>::N;
    constexpr int ESZ = 16 / N;
    extern __shared__ __align__(16) float prm[];           // [bias | gain | beta][hidden]
    grid_dependency_wait();
    grid_launch_dependents();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps = gridDim.x * (blockDim.x >> 5);
    const uint8_t *xb = (const uint8_t *)x, *rb = (const uint8_t *)resid;
    uint4 xr[CHUNKS], rr[CHUNKS];
    auto issue = [&](uint32_t row) {
        const size_t base = (size_t)row * hidden;
#pragma unroll
        for (int c = 0; c < CHUNKS; c++) {
            const uint32_t col = (c * 32 + lane) * N;
            if (col < hidden) {
                xr[c] = ld_stream16(xb + (base + col) * ESZ);
                if (HAS_RESID) rr[c] = ld_stream16(rb + (base + col) * ESZ);
            }
        }
    };
    uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (PREFETCH && row < m) issue(row);                   // the first row is on its way while the parameters are staged
    for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        prm[i] = bias ? bias[i] : 0.f;
        prm[hidden + i] = gain[i];
        prm[2 * hidden + i] = beta[i];
    }
    __syncthreads();
    for (; row < m; row += warps) {
        const size_t base = (size_t)row * hidden;
        if (!PREFETCH) issue(row);
        float v[CHUNKS][N];
        float s = 0.f, s2 = 0.f;
#pragma unroll
        for (int c = 0; c < CHUNKS; c++) {
            const uint32_t col = (c * 32 + lane) * N;
            if (col < hidden) {
                Vec8<DT>::decode(v[c], xr[c]);
#pragma unroll
                for (int t = 0; t < N; t += 4) {
                    const float4 bb = *(const float4 *)(prm + col + t);
                    v[c][t] += bb.x; v[c][t + 1] += bb.y; v[c][t + 2] += bb.z; v[c][t + 3] += bb.w;
                }
                if (HAS_RESID) {
                    float r[N];
                    Vec8<DT>::decode(r, rr[c]);
#pragma unroll
                    for (int t = 0; t < N; t++) v[c][t] = r[t] + v[c][t];
                }
            }
        }
        if (PREFETCH && row + warps < m) issue(row + warps);     // the raw words are decoded: their registers take the next row
#pragma unroll
        for (int c = 0; c < CHUNKS; c++) {
            const uint32_t col = (c * 32 + lane) * N;
            if (col < hidden) {
                if (sum_out) st_stream16((uint8_t *)sum_out + (base + col) * ESZ, Vec8<DT>::encode(v[c]));
#pragma unroll
                for (int t = 0; t < N; t++) {
                    s += v[c][t];
                    s2 = fmaf(v[c][t], v[c][t], s2);
                }
            }
        }
        s = warp_sum(s);
        s2 = warp_sum(s2);
        const float mu = s / (float)hidden;
        // var = E[x^2] - mean^2 with eps inside the root (layernorm.h:28-30)
        const float rs = rsqrtf(fmaxf(s2 / (float)hidden - mu * mu, 0.f) + 1e-5f);
        if (lane == 0) {
            if (mean) mean[row] = mu;
            if (rstd) rstd[row] = rs;
        }
#pragma unroll
        for (int c = 0; c < CHUNKS; c++) {
            const uint32_t col = (c * 32 + lane) * N;
            if (col < hidden) {
                float y[N];
#pragma unroll
                for (int t = 0; t < N; t += 4) {
                    const float4 g = *(const float4 *)(prm + hidden + col + t);
                    const float4 be = *(const float4 *)(prm + 2 * hidden + col + t);
                    y[t] = (v[c][t] - mu) * rs * g.x + be.x;
                    y[t + 1] = (v[c][t + 1] - mu) * rs * g.y + be.y;
                    y[t + 2] = (v[c][t + 2] - mu) * rs * g.z + be.z;
                    y[t + 3] = (v[c][t + 3] - mu) * rs * g.w + be.w;
                }
                st_stream16((uint8_t *)out + (base + col) * ESZ, Vec8<DT>::encode(y));
            }
        }
    }
}

// Few rows (every row can be in flight at once): two warps per row, each holding half of it, four rows per CTA, one
// pass and no loop.  Half the registers per thread of the kernel above, so twice the rows are resident; the two halves'
// sums meet in shared memory.  bias, gain and beta come through L1 (the streamed rows bypass it).
template <int DT, int HCHUNKS, bool HAS_RESID>
__global__ void __launch_bounds__(256) bias_residual_layernorm_split_kernel(void *out, void *sum_out, float *__restrict__ mean,
                                                                           float *__restrict__ rstd, const void *x,
                                                                           const float *__restrict__ bias, const void *resid,
                                                                           const float *__restrict__ gain, const float *__restrict__ beta,
                                                                           uint32_t m, uint32_t hidden)
{
    constexpr int N = Vec8<DT>::N;
    constexpr int ESZ = 16 / N;
    __shared__ float2 part[8];
    grid_dependency_wait();
    grid_launch_dependents();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * 4 + (warp >> 1), half = warp & 1;
    const bool live = row < m;
    const size_t base = (size_t)row * hidden;
    const uint8_t *xb = (const uint8_t *)x, *rb = (const uint8_t *)resid;
    uint4 xr[HCHUNKS], rr[HCHUNKS];
#pragma unroll
    for (int c = 0; c < HCHUNKS; c++) {
        const uint32_t col = ((half * HCHUNKS + c) * 32 + lane) * N;
        if (live && col < hidden) {
            xr[c] = ld_stream16(xb + (base + col) * ESZ);
            if (HAS_RESID) rr[c] = ld_stream16(rb + (base + col) * ESZ);
        }
    }
    float v[HCHUNKS][N];
    float s = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < HCHUNKS; c++) {
        const uint32_t col = ((half * HCHUNKS + c) * 32 + lane) * N;
        if (live && col < hidden) {
            Vec8<DT>::decode(v[c], xr[c]);
            if (bias) {
#pragma unroll
                for (int t = 0; t < N; t += 4) {
                    const float4 bb = __ldg((const float4 *)(bias + col + t));
                    v[c][t] += bb.x; v[c][t + 1] += bb.y; v[c][t + 2] += bb.z; v[c][t + 3] += bb.w;
                }
            }
            if (HAS_RESID) {
                float r[N];
                Vec8<DT>::decode(r, rr[c]);
#pragma unroll
                for (int t = 0; t < N; t++) v[c][t] = r[t] + v[c][t];
            }
            if (sum_out) st_stream16((uint8_t *)sum_out + (base + col) * ESZ, Vec8<DT>::encode(v[c]));
#pragma unroll
            for (int t = 0; t < N; t++) {
                s += v[c][t];
                s2 = fmaf(v[c][t], v[c][t], s2);
            }
        }
    }
    s = warp_sum(s);
    s2 = warp_sum(s2);
    if (lane == 0) part[warp] = make_float2(s, s2);
    __syncthreads();
    const float2 other = part[warp ^ 1];
    s += other.x;
    s2 += other.y;
    const float mu = s / (float)hidden;
    const float rs = rsqrtf(fmaxf(s2 / (float)hidden - mu * mu, 0.f) + 1e-5f);
    if (live && lane == 0 && half == 0) {
        if (mean) mean[row] = mu;
        if (rstd) rstd[row] = rs;
    }
#pragma unroll
    for (int c = 0; c < HCHUNKS; c++) {
        const uint32_t col = ((half * HCHUNKS + c) * 32 + lane) * N;
        if (live && col < hidden) {
            float y[N];
#pragma unroll
            for (int t = 0; t < N; t += 4) {
                const float4 g = __ldg((const float4 *)(gain + col + t));
                const float4 be = __ldg((const float4 *)(beta + col + t));
                y[t] = (v[c][t] - mu) * rs * g.x + be.x;
                y[t + 1] = (v[c][t + 1] - mu) * rs * g.y + be.y;
                y[t + 2] = (v[c][t + 2] - mu) * rs * g.z + be.z;
                y[t + 3] = (v[c][t + 3] - mu) * rs * g.w + be.w;
            }
            st_stream16((uint8_t *)out + (base + col) * ESZ, Vec8<DT>::encode(y));
        }
    }
}

#ifndef SFB_LN_SPLIT
#define SFB_LN_SPLIT 1
#endif
constexpr bool kLnSplit = SFB_LN_SPLIT != 0;
#ifndef SFB_LN_SPLIT_ROWS
#define SFB_LN_SPLIT_ROWS 64
#endif
constexpr uint64_t kLnSplitRows = SFB_LN_SPLIT_ROWS;   // rows per SM up to which a launch takes the two-warps-per-row kernel

template <int DT>
static int launch_ln(cudaStream_t s, void *out, void *sum_out, float *mean, float *rstd, const void *x, const float *bias,
                     const void *resid, const float *gain, const float *beta, uint32_t m, uint32_t hidden)
{
    constexpr int N = Vec8<DT>::N;
    const uint32_t per_chunk = 32 * N;
    const uint32_t chunks = (hidden + per_chunk - 1) / per_chunk;
    const uint32_t rows_per_cta = 8;
    // the grid is the CTAs that are resident at once (a second wave of CTAs would start while the first one's warps
    // are still striding: measured 0.62 against 0.66 of copy bandwidth); the warps loop over the remaining rows
    const uint32_t want = (m + rows_per_cta - 1) / rows_per_cta;
    const size_t smem = 3 * (size_t)hidden * sizeof(float);
    const int sms = device_sm_count(current_device());
    SFB_REQUIRE(sms > 0, "sfb_bias_residual_layernorm: cannot query the device");
#ifndef SFB_LN_PREFETCH
#define SFB_LN_PREFETCH true
#endif
#define LN_LAUNCH(C, R)                                                                                                        \
    do {                                                                                                                       \
        auto kern = bias_residual_layernorm_kernel<DT, C, R, SFB_LN_PREFETCH>;                                                 \
        int per_sm = 0;                                                                                                        \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 32 * rows_per_cta, smem) != cudaSuccess || per_sm < 1) \
            per_sm = 1;                                                                                                        \
        const uint32_t resident = (uint32_t)per_sm * (uint32_t)sms;                                                            \
        launch_overlapped(kern, dim3(want < resident ? want : resident), dim3(32 * rows_per_cta), smem, s, out, sum_out, mean, rstd, x, \
                          bias, resid, gain, beta, m, hidden);                                                                 \
    } while (0)
#define LN_CASE(C)                                                                                                             \
    do {                                                                                                                       \
        if (resid) LN_LAUNCH(C, true);                                                                                         \
        else LN_LAUNCH(C, false);                                                                                              \
    } while (0)
    // few rows (at most two waves of these CTAs): every row at once, two warps each, four rows per CTA
#define LN_SPLIT(H, R)                                                                                                         \
    do {                                                                                                                       \
        auto kern = bias_residual_layernorm_split_kernel<DT, H, R>;                                                            \
        launch_overlapped(kern, dim3((m + 3) / 4), dim3(256), 0, s, out, sum_out, mean, rstd, x, bias, resid, gain, beta, m, hidden); \
        return check_launch("sfb_bias_residual_layernorm");                                                                    \
    } while (0)
#define LN_SPLIT_CASE(H)                                                                                                       \
    do {                                                                                                                       \
        if (resid) LN_SPLIT(H, true);                                                                                          \
        else LN_SPLIT(H, false);                                                                                               \
    } while (0)
    if (kLnSplit && chunks >= 2 && chunks <= 8 && (uint64_t)m <= kLnSplitRows * (uint64_t)sms) {
        const uint32_t hc = (chunks + 1) / 2;
        if (hc == 1) LN_SPLIT_CASE(1);
        else if (hc == 2) LN_SPLIT_CASE(2);
        else if (hc == 3) LN_SPLIT_CASE(3);
        else LN_SPLIT_CASE(4);
    }
#undef LN_SPLIT_CASE
#undef LN_SPLIT
    if (chunks <= 1) LN_CASE(1);
    else if (chunks <= 2) LN_CASE(2);
    else if (chunks <= 3) LN_CASE(3);
    else if (chunks <= 4) LN_CASE(4);
    else if (chunks <= 6) LN_CASE(6);
    else if (chunks <= 8) LN_CASE(8);
    else if (chunks <= 16) LN_CASE(16);
    else return fail("sfb_bias_residual_layernorm: hidden %u too large (max %u)", hidden, 16 * per_chunk);
#undef LN_LAUNCH
#undef LN_CASE
    return check_launch("sfb_bias_residual_layernorm");
}

}  // namespace sfb

using namespace sfb;

extern "C" int sfb_bias_residual_layernorm(sfb_stream_t stream, void *out, void *sum_out, float *mean, float *rstd,
                                           const void *x, const float *bias, const void *resid, const float *gain,
                                           const float *beta, uint32_t m, uint32_t hidden, int dtype)
{
    SFB_REQUIRE(out && x && gain && beta, "sfb_bias_residual_layernorm: NULL pointer");
    SFB_REQUIRE(valid_dtype(dtype), "sfb_bias_residual_layernorm: unknown dtype %d", dtype);
    SFB_REQUIRE(hidden >= 8 && hidden % 8 == 0, "sfb_bias_residual_layernorm: hidden %u must be a multiple of 8", hidden);
    const uintptr_t al = (uintptr_t)out | (uintptr_t)x | (uintptr_t)sum_out | (uintptr_t)resid | (uintptr_t)bias |
                         (uintptr_t)gain | (uintptr_t)beta;
    SFB_REQUIRE((al & 15) == 0, "sfb_bias_residual_layernorm: pointers must be 16-byte aligned");
    if (m == 0) { clear_error(); return 0; }
    cudaStream_t s = as_stream(stream);
    if (dtype == SFB_F32) return launch_ln<SFB_F32>(s, out, sum_out, mean, rstd, x, bias, resid, gain, beta, m, hidden);
    if (dtype == SFB_BF16) return launch_ln<SFB_BF16>(s, out, sum_out, mean, rstd, x, bias, resid, gain, beta, m, hidden);
    return launch_ln<SFB_F16>(s, out, sum_out, mean, rstd, x, bias, resid, gain, beta, m, hidden);
}

// ---- bias + GELU ------------------------------------------------------------------------------------
// y = t * sigmoid(1.702 t), t = x + bias  (the reference's GELU, ewops.h:32-43 / cuda_kernels.h:561-581,
// with the bias add of cuda_kernels.h:471-489 folded in).  One 16-byte access per thread and step.
namespace sfb {

template <int DT>
// out may be x itself (the header allows the call in place), so neither carries __restrict__
__global__ void __launch_bounds__(256) bias_gelu_kernel(void *out, const void *x,
                                                       const float *__restrict__ bias, size_t total, uint32_t n)
{
    constexpr int N = Vec8<DT>::N;
    const size_t stride = (size_t)gridDim.x * blockDim.x * N;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * N; i < total; i += stride) {
        float v[N];
        Vec8<DT>::load(v, x, i);
        const uint32_t col = (uint32_t)(i % n);
#pragma unroll
        for (int t = 0; t < N; t++) {
            const float a = v[t] + (bias ? __ldg(bias + col + t) : 0.f);
            v[t] = a / (1.f + __expf(-1.702f * a));
        }
        Vec8<DT>::store(out, i, v);
    }
}

// Embedding lookup + positional add: out[b, l, :] = table[ids[b, l], :] + pos[l, :].  A thread owns one 16-byte piece
// (l, col) of the position table for a run of batch elements: the position piece is read once and stays in registers,
// so per output row only the table row comes in and the output row goes out (with a piece per token the positions
// crossed from L2 to the SMs once per token: a third of all the bytes the kernel moved).  kEmbUnroll batch elements are
// in flight per step, their ids requested one step ahead.  A warp covers 512 contiguous bytes of a row.  An id outside
// [0, vocab) gives a row of zeros (plus pos) and is counted in *bad_ids -- no out-of-bounds read.
constexpr int kEmbUnroll = 4;
template <int DT>
__global__ void __launch_bounds__(256) embedding_kernel(void *__restrict__ out, const void *__restrict__ table,
                                                       const int32_t *__restrict__ ids, const void *__restrict__ pos, uint32_t batch,
                                                       uint32_t per_cta_y, uint32_t seq_len, uint32_t hidden, uint32_t vocab,
                                                       uint32_t *bad_ids)
{
    constexpr int N = Vec8<DT>::N, U = kEmbUnroll;
    constexpr int ESZ = 16 / N;
    const uint32_t per_row = hidden / N;                                   // 16-byte pieces per row
    const uint32_t piece = blockIdx.x * blockDim.x + threadIdx.x;          // < seq_len * per_row < 2^32 (checked by the host)
    if (piece >= seq_len * per_row) return;
    const uint32_t l = piece / per_row, col = (piece - l * per_row) * N;
    const uint32_t b_begin = blockIdx.y * per_cta_y, b_end = min(batch, b_begin + per_cta_y);
    const uint8_t *tb = (const uint8_t *)table;
    float q[N];
#pragma unroll
    for (int t = 0; t < N; t++) q[t] = 0.f;
    if (pos) Vec8<DT>::decode(q, __ldg((const uint4 *)((const uint8_t *)pos + ((size_t)l * hidden + col) * ESZ)));
    auto fetch_ids = [&](uint32_t b0, int32_t (&id)[U]) {
#pragma unroll
        for (int u = 0; u < U; u++) id[u] = b0 + u < b_end ? __ldg(ids + (size_t)(b0 + u) * seq_len + l) : -1;
    };
    int32_t id[U], id_next[U];
    if (b_begin < b_end) fetch_ids(b_begin, id);
    for (uint32_t b0 = b_begin; b0 < b_end; b0 += U) {
        uint4 tv[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            ok[u] = id[u] >= 0 && (uint32_t)id[u] < vocab;
            tv[u] = make_uint4(0u, 0u, 0u, 0u);                            // all-zero bits decode to 0 in every type
            if (ok[u]) tv[u] = __ldg((const uint4 *)(tb + ((size_t)id[u] * hidden + col) * ESZ));
        }
        if (b0 + U < b_end) fetch_ids(b0 + U, id_next);
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (b0 + u < b_end) {
                if (!ok[u] && col == 0 && bad_ids) atomicAdd(bad_ids, 1u);
                float v[N];
                Vec8<DT>::decode(v, tv[u]);
#pragma unroll
                for (int t = 0; t < N; t++) v[t] += q[t];
                st_stream16((uint8_t *)out + (((size_t)(b0 + u) * seq_len + l) * hidden + col) * ESZ, Vec8<DT>::encode(v));
            }
            id[u] = id_next[u];
        }
    }
}

// out[row] = sum over the row of a * b: rows of d elements, 8 lanes per row (16-byte accesses, shuffle reduction).
// delta = rowdot(dO, O) is the row constant of the softmax gradient.
template <int DT>
__global__ void __launch_bounds__(256) rowdot_kernel(float *__restrict__ out, const void *__restrict__ a, const void *__restrict__ b,
                                                    size_t rows, uint32_t d)
{
    constexpr int N = Vec8<DT>::N;
    const size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 8;
    const uint32_t part = threadIdx.x & 7;
    float sum = 0.f;
    if (row < rows)
        for (uint32_t c = part * N; c < d; c += 8 * N) {
            float x[N], y[N];
            Vec8<DT>::load(x, a, row * d + c);
            Vec8<DT>::load(y, b, row * d + c);
#pragma unroll
            for (int t = 0; t < N; t++) sum = fmaf(x[t], y[t], sum);
        }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (row < rows && part == 0) out[row] = sum;
}

int rowdot(cudaStream_t s, float *out, const void *a, const void *b, size_t rows, uint32_t d, int dtype)
{
    const unsigned ctas = (unsigned)((rows * 8 + 255) / 256);
    if (dtype == SFB_F32) rowdot_kernel<SFB_F32><<<ctas, 256, 0, s>>>(out, a, b, rows, d);
    else if (dtype == SFB_BF16) rowdot_kernel<SFB_BF16><<<ctas, 256, 0, s>>>(out, a, b, rows, d);
    else rowdot_kernel<SFB_F16><<<ctas, 256, 0, s>>>(out, a, b, rows, d);
    return check_launch("sfb_rowdot");
}

int embedding_lookup(cudaStream_t s, void *out, const void *table, const int32_t *ids, const void *pos, uint32_t batch,
                     uint32_t seq_len, uint32_t hidden, uint32_t vocab, int dtype, uint32_t *bad_ids)
{
    const int per = dtype == SFB_F32 ? 4 : 8;
    if (hidden % per) return fail("sfb_embedding: hidden=%u must be a multiple of %d for this type", hidden, per);
    if (bad_ids) cudaMemsetAsync(bad_ids, 0, sizeof(uint32_t), s);
    const size_t pieces = (size_t)seq_len * (hidden / per);                 // one thread per 16-byte piece of a position row
    if (pieces >= (1ull << 32)) return fail("sfb_embedding: seq_len * hidden too large");
    const int sms = device_sm_count(current_device());
    if (sms <= 0) return fail("sfb_embedding: cannot query the device");
    // short sequences: the batch is split over gridDim.y until the grid has about eight CTAs per SM
    const size_t ctas_x = (pieces + 255) / 256;
    uint32_t split = (uint32_t)(((size_t)sms * 8 + ctas_x - 1) / ctas_x);
    if (split > batch) split = batch;
    if (split > 65535u) split = 65535u;
    if (split < 1) split = 1;
    const uint32_t per_y = (batch + split - 1) / split;
    const dim3 grid((unsigned)ctas_x, (batch + per_y - 1) / per_y);
    if (dtype == SFB_F32) embedding_kernel<SFB_F32><<<grid, 256, 0, s>>>(out, table, ids, pos, batch, per_y, seq_len, hidden, vocab, bad_ids);
    else if (dtype == SFB_BF16) embedding_kernel<SFB_BF16><<<grid, 256, 0, s>>>(out, table, ids, pos, batch, per_y, seq_len, hidden, vocab, bad_ids);
    else embedding_kernel<SFB_F16><<<grid, 256, 0, s>>>(out, table, ids, pos, batch, per_y, seq_len, hidden, vocab, bad_ids);
    return check_launch("sfb_embedding");
}

}  // namespace sfb

extern "C" int sfb_bias_gelu(sfb_stream_t stream, void *out, const void *x, const float *bias, uint32_t m, uint32_t n, int dtype)
{
    SFB_REQUIRE(out && x, "sfb_bias_gelu: NULL pointer");
    SFB_REQUIRE(valid_dtype(dtype), "sfb_bias_gelu: unknown dtype %d", dtype);
    SFB_REQUIRE(n >= 8 && n % 8 == 0, "sfb_bias_gelu: row length %u must be a multiple of 8", n);
    SFB_REQUIRE((((uintptr_t)out | (uintptr_t)x | (uintptr_t)bias) & 15) == 0, "sfb_bias_gelu: pointers must be 16-byte aligned");
    const size_t total = (size_t)m * n;
    if (total == 0) { clear_error(); return 0; }
    cudaStream_t s = as_stream(stream);
    const int per = dtype == SFB_F32 ? 4 : 8;
    size_t ctas = (total / per + 255) / 256;
    if (ctas > 148 * 16) ctas = 148 * 16;
    if (dtype == SFB_F32) bias_gelu_kernel<SFB_F32><<<(unsigned)ctas, 256, 0, s>>>(out, x, bias, total, n);
    else if (dtype == SFB_BF16) bias_gelu_kernel<SFB_BF16><<<(unsigned)ctas, 256, 0, s>>>(out, x, bias, total, n);
    else bias_gelu_kernel<SFB_F16><<<(unsigned)ctas, 256, 0, s>>>(out, x, bias, total, n);
    return check_launch("sfb_bias_gelu");
}
