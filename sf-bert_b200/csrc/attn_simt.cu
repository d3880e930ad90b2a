// FP32-arithmetic (CUDA-core) kernels of the block-sparse attention path: SDDMM, masked softmax,
// SpMM and the two block-row-owned fusions.  They serve fp32 operands (1e-5 parity with the CPU
// reference cannot be met on tensor cores) and every shape the tcgen05 kernels do not cover.
//
// Thread layout shared by all matmul kernels: 256 threads as a 16x16 grid; thread (ty,tx) owns
// rows ty+16m and columns tx+16n of a tile, so the 16 lanes of a half-warp own one set of rows
// and row reductions are four shuffles.
#include "attn.cuh"
#include <float.h>
#include <math.h>

namespace sfb {

#define LOG2E_F 1.4426950408889634f


template <int BS>
struct MaskWord { typedef uint32_t type; };
template <>
struct MaskWord<64> { typedef uint64_t type; };

// loads rows [row0, row0+BS) x columns [k0, k0+KC) of a [*, HD] row-major operand into smem as
// dst[k][r] (k-major, row stride BS+1), zero beyond d
template <int DT, int BS, int KC>
__device__ __forceinline__ void load_tile_kmajor(float (*dst)[BS + 1], const void *src, size_t base, size_t HD,
                                                 uint32_t k0, uint32_t d)
{
    for (uint32_t e = threadIdx.x; e < BS * KC; e += 256) {
        uint32_t r = e / KC, k = e % KC;
        float v = 0.f;
        if (k0 + k < d) v = Elem<DT>::load(src, base + (size_t)r * HD + k0 + k);
        dst[k][r] = v;
    }
}

// ------------------------------------------------------------------------------------------------
// SDDMM: one CTA per non-zero block
template <int BS, int AB_DT, int C_DT>
__global__ void __launch_bounds__(256) sddmm_nt_kernel(const uint2 *__restrict__ lut, const void *__restrict__ A,
                                                      const void *__restrict__ Bm, void *__restrict__ C, AttnDims p)
{
    constexpr int KC = 32, T = BS / 16;
    __shared__ float As[KC][BS + 1];
    __shared__ float Bs[KC][BS + 1];
    const uint32_t bid = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const uint2 e = lut[(size_t)h * p.lut_stride + bid];
    const size_t HD = (size_t)p.H * p.d;
    const size_t baseA = ((size_t)b * p.nb_a * BS + (size_t)e.x * BS) * HD + (size_t)h * p.d;
    const size_t baseB = ((size_t)b * p.nb_b * BS + (size_t)e.y * BS) * HD + (size_t)h * p.d;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    float acc[T][T];
#pragma unroll
    for (int m = 0; m < T; m++)
#pragma unroll
        for (int n = 0; n < T; n++) acc[m][n] = 0.f;

    for (uint32_t k0 = 0; k0 < p.d; k0 += KC) {
        load_tile_kmajor<AB_DT, BS, KC>(As, A, baseA, HD, k0, p.d);
        load_tile_kmajor<AB_DT, BS, KC>(Bs, Bm, baseB, HD, k0, p.d);
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < KC; k++) {
            float a[T], bb[T];
#pragma unroll
            for (int m = 0; m < T; m++) a[m] = As[k][ty + 16 * m];
#pragma unroll
            for (int n = 0; n < T; n++) bb[n] = Bs[k][tx + 16 * n];
#pragma unroll
            for (int m = 0; m < T; m++)
#pragma unroll
                for (int n = 0; n < T; n++) acc[m][n] = fmaf(a[m], bb[n], acc[m][n]);
        }
        __syncthreads();
    }
    const size_t baseC = (((size_t)b * p.H + h) * p.blocks + bid) * BS * BS;
#pragma unroll
    for (int m = 0; m < T; m++)
#pragma unroll
        for (int n = 0; n < T; n++) Elem<C_DT>::store(C, baseC + (size_t)(ty + 16 * m) * BS + tx + 16 * n, acc[m][n]);
}

// ------------------------------------------------------------------------------------------------
template <int Y_DT>
__device__ __forceinline__ void store8(void *y, size_t idx, const float (&v)[8])
{
    if (Y_DT == SFB_F32) {
        float4 *p = (float4 *)((float *)y + idx);
        p[0] = make_float4(v[0], v[1], v[2], v[3]);
        p[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (Y_DT == SFB_BF16) {
                // probabilities: the hardware's round-to-nearest-even pack (one instruction per pair); it differs
                // from the reference's add-half-and-truncate rounding (ew_op_gpu.h:241-253) on exact ties only
                __nv_bfloat162 hb = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&hb);
            } else {
                __half2 hh = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&hh);
            }
        }
        *(uint4 *)((uint16_t *)y + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// raw 16-byte (16-bit types) or 32-byte (fp32) load of 8 scores, kept unconverted so that many can be in flight
template <int X_DT> struct Raw8 { uint4 a; };
template <> struct Raw8<SFB_F32> { uint4 a, b; };

template <int X_DT>
__device__ __forceinline__ Raw8<X_DT> load_raw8(const void *x, size_t idx)
{
    Raw8<X_DT> r;
    if (X_DT == SFB_F32) {
        const uint4 *p = (const uint4 *)((const float *)x + idx);
        r.a = __ldg(p);
        ((Raw8<SFB_F32> &)r).b = __ldg(p + 1);
    } else {
        r.a = __ldg((const uint4 *)((const uint16_t *)x + idx));
    }
    return r;
}

template <int X_DT>
__device__ __forceinline__ void unpack8(float (&v)[8], const Raw8<X_DT> &r)
{
    if (X_DT == SFB_F32) {
        const Raw8<SFB_F32> &q = (const Raw8<SFB_F32> &)r;
        v[0] = __uint_as_float(q.a.x); v[1] = __uint_as_float(q.a.y); v[2] = __uint_as_float(q.a.z); v[3] = __uint_as_float(q.a.w);
        v[4] = __uint_as_float(q.b.x); v[5] = __uint_as_float(q.b.y); v[6] = __uint_as_float(q.b.z); v[7] = __uint_as_float(q.b.w);
    } else {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (X_DT == SFB_BF16) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            } else {
                float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                v[2 * i] = f.x;
                v[2 * i + 1] = f.y;
            }
        }
    }
}

__device__ __forceinline__ float ex2_fast(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Masked softmax: one CTA per block-row.  A lane owns 8 consecutive keys of one query row of one block
// (16 bytes of bf16), so a warp reads 512 contiguous bytes per block; the lanes of a row (BS/8 of them)
// combine with shuffles.
//
// NB > 0: the row has at most NB blocks.  All of them are loaded up front (NB independent 16-byte loads per
// lane in flight) and stay in registers: one pass over HBM, one exponential per element.
// NB == 0: rows of any length.  Pass 1 finds the row maximum, pass 2 the sum of exponentials, pass 3 writes;
// passes 2 and 3 re-read scores this CTA has just pulled through L2.
// SPLIT > 1: the block-row is shared by SPLIT CTAs of BS/SPLIT query rows each.  Registers decide how many of the
// register-resident CTAs an SM holds, and small CTAs fill what the register file leaves: with loads of some CTAs in
// flight while others compute and store, the 12- and 16-block rows run at the speed of a copy (0.98 of it; a CTA per
// whole block-row, one per SM, reached 0.6-0.7).
// The second launch bound asks for the number of CTAs per SM that the variant's registers allow anyway (it keeps the
// compiler from spending registers the occupancy needs).
template <int BS, int X_DT, int Y_DT, int NB, int SPLIT>
__global__ void __launch_bounds__(BS * BS / 8 / SPLIT, (NB > 0 && SPLIT > 1 && BS == 64 && X_DT != SFB_F32) ? (NB <= 12 ? 6 : NB <= 18 ? 5 : 4) : 1) softmax_kernel(const uint2 *__restrict__ lut,
                                                                const typename MaskWord<BS>::type *__restrict__ mask,
                                                                const void *__restrict__ X, void *__restrict__ Y, AttnDims p,
                                                                float scale_log2e, int rescale_in_place)
{
    typedef typename MaskWord<BS>::type W;
    constexpr int LPR = BS / 8;  // lanes per query row
    const uint32_t i = blockIdx.x / SPLIT, b = blockIdx.y, h = blockIdx.z;
    const uint2 *nn = lut + (size_t)h * p.lut_stride;
    const uint2 head = nn[i];
    const uint32_t off = head.x, cnt = head.y;
    if (cnt == 0) return;
    const uint32_t r = (blockIdx.x % SPLIT) * (BS / SPLIT) + threadIdx.x / LPR;        // query row inside the block
    const uint32_t c0 = (threadIdx.x % LPR) * 8;  // first key of this lane
    const size_t base = ((size_t)b * p.H + h) * p.blocks * BS * BS + (size_t)r * BS + c0;
    const W *mrow = mask ? mask + (size_t)h * p.mask_stride + (size_t)r * p.blocks : nullptr;

    if (NB > 0) {
        constexpr int N = NB > 0 ? NB : 1;
        Raw8<X_DT> raw[N];
        uint32_t blks[N], bits[N];
#pragma unroll
        for (int j = 0; j < N; j++) {
            blks[j] = 0;
            bits[j] = 0;
            if (j < (int)cnt) {
                blks[j] = nn[off + j].x;
                raw[j] = load_raw8<X_DT>(X, base + (size_t)blks[j] * BS * BS);
                bits[j] = mrow ? (uint32_t)((__ldg(mrow + blks[j]) >> c0) & 0xffu) : 0xffu;
            }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < N; j++) {
            if (j < (int)cnt) {
                float v[8];
                unpack8<X_DT>(v, raw[j]);
#pragma unroll
                for (int t = 0; t < 8; t++)
                    if ((bits[j] >> t) & 1u) mx = fmaxf(mx, v[t]);
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float mxs = mx > -INFINITY ? mx * scale_log2e : 0.f;
        // second sweep: one exponential per score; the results replace the raw scores in their registers as
        // packed fp16 pairs (e is in (0, 1], 11 bits are more than the 16-bit output keeps)
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < N; j++) {
            if (j < (int)cnt) {
                float v[8];
                unpack8<X_DT>(v, raw[j]);
#pragma unroll
                for (int t = 0; t < 8; t++) {
                    v[t] = ((bits[j] >> t) & 1u) ? ex2_fast(fmaf(v[t], scale_log2e, -mxs)) : 0.f;
                    sum += v[t];
                }
                if (Y_DT != SFB_F32) {   // fp32 outputs recompute the exponential below instead: fp16 would cost them bits
                    __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                    __half2 h2 = __floats2half2_rn(v[4], v[5]), h3 = __floats2half2_rn(v[6], v[7]);
                    raw[j].a = make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                                          *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
                }
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
        for (int j = 0; j < N; j++) {
            if (j < (int)cnt) {
                float v[8];
                if (Y_DT != SFB_F32) {
                    const uint32_t w[4] = {raw[j].a.x, raw[j].a.y, raw[j].a.z, raw[j].a.w};
#pragma unroll
                    for (int t = 0; t < 4; t++) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[t]));
                        v[2 * t] = f.x * inv;
                        v[2 * t + 1] = f.y * inv;
                    }
                } else {
                    unpack8<X_DT>(v, raw[j]);
#pragma unroll
                    for (int t = 0; t < 8; t++)
                        v[t] = ((bits[j] >> t) & 1u) ? ex2_fast(fmaf(v[t], scale_log2e, -mxs)) * inv : 0.f;
                }
                store8<Y_DT>(Y, base + (size_t)blks[j] * BS * BS, v);
            }
        }
        return;
    }

    // pass 1: the row maximum (packed bf16 max when there is no mask: 4 instructions per 8 scores)
    float mx = -INFINITY;
    if (X_DT == SFB_BF16 && !mrow) {
        uint32_t acc[4] = {0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u};   // pairs of -inf
        for (uint32_t e = 0; e < cnt; e++) {
            const uint32_t blk = nn[off + e].x;
            const Raw8<X_DT> r8 = load_raw8<X_DT>(X, base + (size_t)blk * BS * BS);
            const uint32_t w[4] = {r8.a.x, r8.a.y, r8.a.z, r8.a.w};
#pragma unroll
            for (int t = 0; t < 4; t++) {
                __nv_bfloat162 m2 = __hmax2(*reinterpret_cast<__nv_bfloat162 *>(&acc[t]), *reinterpret_cast<const __nv_bfloat162 *>(&w[t]));
                acc[t] = *reinterpret_cast<uint32_t *>(&m2);
            }
        }
#pragma unroll
        for (int t = 0; t < 4; t++)
            mx = fmaxf(mx, fmaxf(__uint_as_float(acc[t] << 16), __uint_as_float(acc[t] & 0xffff0000u)));
    } else {
        for (uint32_t e = 0; e < cnt; e++) {
            const uint32_t blk = nn[off + e].x;
            float v[8];
            unpack8<X_DT>(v, load_raw8<X_DT>(X, base + (size_t)blk * BS * BS));
            const uint32_t bits = mrow ? (uint32_t)((__ldg(mrow + blk) >> c0) & 0xffu) : 0xffu;
#pragma unroll
            for (int t = 0; t < 8; t++)
                if ((bits >> t) & 1u) mx = fmaxf(mx, v[t]);
        }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float mxs = mx > -INFINITY ? mx * scale_log2e : 0.f;
    // pass 2: one exponential per score; the unnormalised value goes to Y in the output type
    float sum = 0.f;
    for (uint32_t e = 0; e < cnt; e++) {
        const uint32_t blk = nn[off + e].x;
        float v[8];
        unpack8<X_DT>(v, load_raw8<X_DT>(X, base + (size_t)blk * BS * BS));
        if (mrow) {
            const uint32_t bits = (uint32_t)((__ldg(mrow + blk) >> c0) & 0xffu);
#pragma unroll
            for (int t = 0; t < 8; t++) v[t] = ((bits >> t) & 1u) ? ex2_fast(fmaf(v[t], scale_log2e, -mxs)) : 0.f;
        } else {
#pragma unroll
            for (int t = 0; t < 8; t++) v[t] = ex2_fast(fmaf(v[t], scale_log2e, -mxs));
        }
#pragma unroll
        for (int t = 0; t < 8; t++) sum += v[t];
        if (rescale_in_place) store8<Y_DT>(Y, base + (size_t)blk * BS * BS, v);
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    if (!rescale_in_place) {
        // pass 3 for long rows (their Y would not stay in L2 between two passes): exponentials again, from X
        for (uint32_t e = 0; e < cnt; e++) {
            const uint32_t blk = nn[off + e].x;
            float v[8];
            unpack8<X_DT>(v, load_raw8<X_DT>(X, base + (size_t)blk * BS * BS));
            const uint32_t bits = mrow ? (uint32_t)((__ldg(mrow + blk) >> c0) & 0xffu) : 0xffu;
#pragma unroll
            for (int t = 0; t < 8; t++) v[t] = ((bits >> t) & 1u) ? ex2_fast(fmaf(v[t], scale_log2e, -mxs)) * inv : 0.f;
            store8<Y_DT>(Y, base + (size_t)blk * BS * BS, v);
        }
        return;
    }
    // pass 3: every thread rescales the values it wrote itself (they are still in L2): packed multiplies
    for (uint32_t e = 0; e < cnt; e++) {
        const uint32_t blk = nn[off + e].x;
        const size_t idx = base + (size_t)blk * BS * BS;
        if (Y_DT == SFB_F32) {
            float4 *py = (float4 *)((float *)Y + idx);
            float4 y0 = py[0], y1 = py[1];
            py[0] = make_float4(y0.x * inv, y0.y * inv, y0.z * inv, y0.w * inv);
            py[1] = make_float4(y1.x * inv, y1.y * inv, y1.z * inv, y1.w * inv);
        } else {
            uint4 *py = (uint4 *)((uint16_t *)Y + idx);
            uint4 u = *py;
            uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int t = 0; t < 4; t++) {
                if (Y_DT == SFB_BF16) {
                    __nv_bfloat162 r2 = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&w[t]), __float2bfloat162_rn(inv));
                    w[t] = *reinterpret_cast<uint32_t *>(&r2);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<__half2 *>(&w[t]));
                    __half2 r2 = __floats2half2_rn(f.x * inv, f.y * inv);
                    w[t] = *reinterpret_cast<uint32_t *>(&r2);
                }
            }
            *py = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Softmax gradient: dx = (dy - sum over the query row of dy*y) * y * scale.  Same decomposition as the forward
// softmax: one CTA per block-row, a lane owns 8 consecutive keys of one query row of one block.
// NB > 0: the row has at most NB blocks; dy and y of all of them are loaded up front and stay in registers
// (one pass over HBM).  NB == 0: any length; the second sweep re-reads what the first pulled through L2.
// SPLIT > 1: the block-row is shared by SPLIT CTAs of BS/SPLIT query rows each -- fewer threads per CTA leave more
// registers per thread, which is what lets longer rows stay register-resident.
template <int BS, int DT, int NB, int SPLIT>
__global__ void __launch_bounds__(BS * BS / 8 / SPLIT) softmax_grad_kernel(const uint2 *__restrict__ lut, const void *__restrict__ DY,
                                                                     const void *__restrict__ Y, void *__restrict__ DX, AttnDims p,
                                                                     float scale)
{
    constexpr int LPR = BS / 8;  // lanes per query row
    const uint32_t i = blockIdx.x / SPLIT, b = blockIdx.y, h = blockIdx.z;
    const uint2 *nn = lut + (size_t)h * p.lut_stride;
    const uint2 head = nn[i];
    const uint32_t off = head.x, cnt = head.y;
    if (cnt == 0) return;
    const uint32_t r = (blockIdx.x % SPLIT) * (BS / SPLIT) + threadIdx.x / LPR;
    const uint32_t c0 = (threadIdx.x % LPR) * 8;
    const size_t base = ((size_t)b * p.H + h) * p.blocks * BS * BS + (size_t)r * BS + c0;

    if (NB > 0) {
        constexpr int N = NB > 0 ? NB : 1;
        Raw8<DT> rdy[N], ry[N];
        uint32_t blks[N];
#pragma unroll
        for (int j = 0; j < N; j++) {
            blks[j] = 0;
            if (j < (int)cnt) {
                blks[j] = nn[off + j].x;
                rdy[j] = load_raw8<DT>(DY, base + (size_t)blks[j] * BS * BS);
                ry[j] = load_raw8<DT>(Y, base + (size_t)blks[j] * BS * BS);
            }
        }
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < N; j++)
            if (j < (int)cnt) {
                float a[8], c[8];
                unpack8<DT>(a, rdy[j]);
                unpack8<DT>(c, ry[j]);
#pragma unroll
                for (int t = 0; t < 8; t++) sum = fmaf(a[t], c[t], sum);
            }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
        for (int j = 0; j < N; j++)
            if (j < (int)cnt) {
                float a[8], c[8];
                unpack8<DT>(a, rdy[j]);
                unpack8<DT>(c, ry[j]);
#pragma unroll
                for (int t = 0; t < 8; t++) a[t] = (a[t] - sum) * c[t] * scale;
                store8<DT>(DX, base + (size_t)blks[j] * BS * BS, a);
            }
        return;
    }
    float sum = 0.f;
    for (uint32_t e = 0; e < cnt; e++) {
        const size_t at = base + (size_t)nn[off + e].x * BS * BS;
        float a[8], c[8];
        unpack8<DT>(a, load_raw8<DT>(DY, at));
        unpack8<DT>(c, load_raw8<DT>(Y, at));
#pragma unroll
        for (int t = 0; t < 8; t++) sum = fmaf(a[t], c[t], sum);
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (uint32_t e = 0; e < cnt; e++) {
        const size_t at = base + (size_t)nn[off + e].x * BS * BS;
        float a[8], c[8];
        unpack8<DT>(a, load_raw8<DT>(DY, at));
        unpack8<DT>(c, load_raw8<DT>(Y, at));
#pragma unroll
        for (int t = 0; t < 8; t++) a[t] = (a[t] - sum) * c[t] * scale;
        store8<DT>(DX, at, a);
    }
}

// ------------------------------------------------------------------------------------------------
// SpMM: one CTA per (block-row, 64-wide slice of d).  TRANS = false: O = sum over the row's blocks of P . V (NN, the
// lut is the nn_lut).  TRANS = true: the backward products dV = P^T dO and dK = dS^T Q -- the lut is the tn_lut,
// "row" i is a block COLUMN, an entry names a block of that column and the block-row its B rows come from, and
// the block is used transposed.
template <int BS, int A_DT, int BC_DT, bool TRANS>
__global__ void __launch_bounds__(256) spmm_nn_kernel(const uint2 *__restrict__ lut, const void *__restrict__ Pm,
                                                     const void *__restrict__ V, void *__restrict__ O, AttnDims p)
{
    constexpr int TM = BS / 16, TN = 4;
    __shared__ float Ps[BS][BS + 16];
    __shared__ float Vs[BS][64];
    const uint32_t nslice = (p.d + 63) / 64;
    const uint32_t i = blockIdx.x / nslice, n0 = (blockIdx.x % nslice) * 64;
    const uint32_t b = blockIdx.y, h = blockIdx.z;
    const uint2 *nn = lut + (size_t)h * p.lut_stride;
    const uint2 head = nn[i];
    const size_t HD = (size_t)p.H * p.d;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    float acc[TM][TN];
#pragma unroll
    for (int m = 0; m < TM; m++)
#pragma unroll
        for (int n = 0; n < TN; n++) acc[m][n] = 0.f;

    for (uint32_t e = 0; e < head.y; e++) {
        const uint2 ent = nn[head.x + e];
        const size_t baseP = (((size_t)b * p.H + h) * p.blocks + ent.x) * BS * BS;
        const size_t baseV = ((size_t)b * p.nb_b * BS + (size_t)ent.y * BS) * HD + (size_t)h * p.d + n0;
        for (uint32_t t = threadIdx.x; t < BS * BS; t += 256) Ps[t / BS][t % BS] = Elem<A_DT>::load(Pm, baseP + t);
        for (uint32_t t = threadIdx.x; t < BS * 64; t += 256) {
            uint32_t c = t / 64, n = t % 64;
            Vs[c][n] = (n0 + n < p.d) ? Elem<BC_DT>::load(V, baseV + (size_t)c * HD + n) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int c = 0; c < BS; c++) {
            float a[TM], bb[TN];
#pragma unroll
            for (int m = 0; m < TM; m++) a[m] = TRANS ? Ps[c][ty + 16 * m] : Ps[ty + 16 * m][c];
#pragma unroll
            for (int n = 0; n < TN; n++) bb[n] = Vs[c][tx + 16 * n];
#pragma unroll
            for (int m = 0; m < TM; m++)
#pragma unroll
                for (int n = 0; n < TN; n++) acc[m][n] = fmaf(a[m], bb[n], acc[m][n]);
        }
        __syncthreads();
    }
    // rows without blocks are written as zeros (blocksparse.h:949-962)
    const size_t baseO = ((size_t)b * p.nb_a * BS + (size_t)i * BS) * HD + (size_t)h * p.d + n0;
#pragma unroll
    for (int m = 0; m < TM; m++)
#pragma unroll
        for (int n = 0; n < TN; n++)
            if (n0 + tx + 16 * n < p.d) Elem<BC_DT>::store(O, baseO + (size_t)(ty + 16 * m) * HD + tx + 16 * n, acc[m][n]);
}

// ------------------------------------------------------------------------------------------------
// Block-row-owned fusions.  Dynamic smem: Qs[DMAX][BS+1] | Ks[DMAX][BS+1] | (attention only)
// Vs[BS][DMAX] | Ps[BS][BS+16].
template <int BS>
__device__ __forceinline__ void score_tile(float (&s)[BS / 16][BS / 16], const float (*Qs)[BS + 1],
                                           const float (*Ks)[BS + 1], uint32_t d, int tx, int ty)
{
    constexpr int T = BS / 16;
#pragma unroll
    for (int m = 0; m < T; m++)
#pragma unroll
        for (int n = 0; n < T; n++) s[m][n] = 0.f;
#pragma unroll 4
    for (uint32_t k = 0; k < d; k++) {
        float a[T], bb[T];
#pragma unroll
        for (int m = 0; m < T; m++) a[m] = Qs[k][ty + 16 * m];
#pragma unroll
        for (int n = 0; n < T; n++) bb[n] = Ks[k][tx + 16 * n];
#pragma unroll
        for (int m = 0; m < T; m++)
#pragma unroll
            for (int n = 0; n < T; n++) s[m][n] = fmaf(a[m], bb[n], s[m][n]);
    }
}

__device__ __forceinline__ float half_warp_max(float v)
{
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float half_warp_sum(float v)
{
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// SDDMM + softmax, probabilities out.  Pass 1 stores the raw scores (in the output type) into Y and
// tracks the row max / sum; pass 2 lets every thread turn the scores it wrote itself into
// probabilities, so no thread ever reads another thread's global writes.
template <int BS, int DMAX, int AB_DT, int Y_DT>
__global__ void __launch_bounds__(256) fused_sddmm_softmax_kernel(const uint2 *__restrict__ lut, const void *__restrict__ A,
                                                                 const void *__restrict__ Bm,
                                                                 const typename MaskWord<BS>::type *__restrict__ mask,
                                                                 void *__restrict__ Y, AttnDims p, float scale_log2e)
{
    typedef typename MaskWord<BS>::type W;
    constexpr int T = BS / 16;
    extern __shared__ float smem[];
    float (*Qs)[BS + 1] = (float (*)[BS + 1])smem;
    float (*Ks)[BS + 1] = (float (*)[BS + 1])(smem + DMAX * (BS + 1));
    const uint32_t i = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const uint2 *nn = lut + (size_t)h * p.lut_stride;
    const uint2 head = nn[i];
    if (head.y == 0) return;
    const size_t HD = (size_t)p.H * p.d;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const W *mh = mask ? mask + (size_t)h * p.mask_stride : nullptr;

    for (uint32_t k0 = 0; k0 < p.d; k0 += 32)
        load_tile_kmajor<AB_DT, BS, 32>(Qs + k0, A, ((size_t)b * p.nb_a * BS + (size_t)i * BS) * HD + (size_t)h * p.d, HD, k0, p.d);

    float mx[T], sum[T];
#pragma unroll
    for (int m = 0; m < T; m++) { mx[m] = -INFINITY; sum[m] = 0.f; }

    for (uint32_t e = 0; e < head.y; e++) {
        const uint2 ent = nn[head.x + e];
        __syncthreads();
        for (uint32_t k0 = 0; k0 < p.d; k0 += 32)
            load_tile_kmajor<AB_DT, BS, 32>(Ks + k0, Bm, ((size_t)b * p.nb_b * BS + (size_t)ent.y * BS) * HD + (size_t)h * p.d, HD, k0, p.d);
        __syncthreads();
        float s[T][T];
        score_tile<BS>(s, Qs, Ks, p.d, tx, ty);
        const size_t baseY = (((size_t)b * p.H + h) * p.blocks + ent.x) * BS * BS;
#pragma unroll
        for (int m = 0; m < T; m++) {
            const uint32_t r = ty + 16 * m;
            const W w = mh ? __ldg(mh + (size_t)ent.x * BS + r) : ~(W)0;
            float bm = -INFINITY, t[T];
#pragma unroll
            for (int n = 0; n < T; n++) {
                const uint32_t c = tx + 16 * n;
                // the stored (possibly 16-bit) score is what pass 2 will read: use it for the statistics too
                Elem<Y_DT>::store(Y, baseY + (size_t)r * BS + c, s[m][n]);
                float sv = Elem<Y_DT>::round(s[m][n]);
                t[n] = ((w >> c) & 1) ? sv * scale_log2e : -INFINITY;
                bm = fmaxf(bm, t[n]);
            }
            bm = half_warp_max(bm);
            if (bm > mx[m]) {
                sum[m] *= exp2f(mx[m] - bm);
                mx[m] = bm;
            }
            float ps = 0.f;
            if (mx[m] > -INFINITY) {
#pragma unroll
                for (int n = 0; n < T; n++) ps += exp2f(t[n] - mx[m]);
            }
            sum[m] += half_warp_sum(ps);
        }
    }
    for (uint32_t e = 0; e < head.y; e++) {
        const uint2 ent = nn[head.x + e];
        const size_t baseY = (((size_t)b * p.H + h) * p.blocks + ent.x) * BS * BS;
#pragma unroll
        for (int m = 0; m < T; m++) {
            const uint32_t r = ty + 16 * m;
            const W w = mh ? __ldg(mh + (size_t)ent.x * BS + r) : ~(W)0;
            const float inv = sum[m] > 0.f ? 1.f / sum[m] : 0.f;
#pragma unroll
            for (int n = 0; n < T; n++) {
                const uint32_t c = tx + 16 * n;
                float sv = Elem<Y_DT>::load(Y, baseY + (size_t)r * BS + c);
                float pv = (((w >> c) & 1) && inv > 0.f) ? exp2f(sv * scale_log2e - mx[m]) * inv : 0.f;
                Elem<Y_DT>::store(Y, baseY + (size_t)r * BS + c, pv);
            }
        }
    }
}

// SDDMM + softmax + SpMM with an online softmax; S and P never leave the SM.
template <int BS, int DMAX, int DT>
__global__ void __launch_bounds__(256) fused_attention_kernel(const uint2 *__restrict__ lut, const void *__restrict__ Q,
                                                             const void *__restrict__ K, const void *__restrict__ V,
                                                             void *__restrict__ O,
                                                             const typename MaskWord<BS>::type *__restrict__ mask,
                                                             AttnDims p, float scale_log2e)
{
    typedef typename MaskWord<BS>::type W;
    constexpr int T = BS / 16, TD = DMAX / 16;
    extern __shared__ float smem[];
    float (*Qs)[BS + 1] = (float (*)[BS + 1])smem;
    float (*Ks)[BS + 1] = (float (*)[BS + 1])(smem + DMAX * (BS + 1));
    float (*Vs)[DMAX] = (float (*)[DMAX])(smem + 2 * DMAX * (BS + 1));
    float (*Ps)[BS + 16] = (float (*)[BS + 16])(smem + 2 * DMAX * (BS + 1) + BS * DMAX);
    const uint32_t i = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const uint2 *nn = lut + (size_t)h * p.lut_stride;
    const uint2 head = nn[i];
    const size_t HD = p.in_pitch ? (size_t)p.in_pitch : (size_t)p.H * p.d;      // row pitch of q, k, v
    const size_t HDo = p.out_pitch ? (size_t)p.out_pitch : (size_t)p.H * p.d;   // row pitch of o
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const W *mh = mask ? mask + (size_t)h * p.mask_stride : nullptr;

    if (head.y)
        for (uint32_t k0 = 0; k0 < p.d; k0 += 32)
            load_tile_kmajor<DT, BS, 32>(Qs + k0, Q, ((size_t)b * p.nb_a * BS + (size_t)i * BS) * HD + (size_t)h * p.d, HD, k0, p.d);

    float mx[T], sum[T], acc[T][TD];
#pragma unroll
    for (int m = 0; m < T; m++) {
        mx[m] = -INFINITY;
        sum[m] = 0.f;
#pragma unroll
        for (int n = 0; n < TD; n++) acc[m][n] = 0.f;
    }

    for (uint32_t e = 0; e < head.y; e++) {
        const uint2 ent = nn[head.x + e];
        const size_t baseKV = ((size_t)b * p.nb_b * BS + (size_t)ent.y * BS) * HD + (size_t)h * p.d;
        __syncthreads();
        for (uint32_t k0 = 0; k0 < p.d; k0 += 32) load_tile_kmajor<DT, BS, 32>(Ks + k0, K, baseKV, HD, k0, p.d);
        for (uint32_t t = threadIdx.x; t < BS * DMAX; t += 256) {
            uint32_t c = t / DMAX, n = t % DMAX;
            Vs[c][n] = n < p.d ? Elem<DT>::load(V, baseKV + (size_t)c * HD + n) : 0.f;
        }
        __syncthreads();
        float s[T][T];
        score_tile<BS>(s, Qs, Ks, p.d, tx, ty);
#pragma unroll
        for (int m = 0; m < T; m++) {
            const uint32_t r = ty + 16 * m;
            const W w = mh ? __ldg(mh + (size_t)ent.x * BS + r) : ~(W)0;
            float bm = -INFINITY;
#pragma unroll
            for (int n = 0; n < T; n++) {
                const uint32_t c = tx + 16 * n;
                s[m][n] = ((w >> c) & 1) ? s[m][n] * scale_log2e : -INFINITY;
                bm = fmaxf(bm, s[m][n]);
            }
            bm = half_warp_max(bm);
            float alpha = 1.f;
            if (bm > mx[m]) {
                alpha = exp2f(mx[m] - bm);
                mx[m] = bm;
            }
            float ps = 0.f;
#pragma unroll
            for (int n = 0; n < T; n++) {
                float pv = mx[m] > -INFINITY ? exp2f(s[m][n] - mx[m]) : 0.f;
                Ps[r][tx + 16 * n] = pv;
                ps += pv;
            }
            sum[m] = sum[m] * alpha + half_warp_sum(ps);
#pragma unroll
            for (int n = 0; n < TD; n++) acc[m][n] *= alpha;
        }
        __syncthreads();
#pragma unroll 4
        for (int c = 0; c < BS; c++) {
            float a[T], bb[TD];
#pragma unroll
            for (int m = 0; m < T; m++) a[m] = Ps[ty + 16 * m][c];
#pragma unroll
            for (int n = 0; n < TD; n++) bb[n] = Vs[c][tx + 16 * n];
#pragma unroll
            for (int m = 0; m < T; m++)
#pragma unroll
                for (int n = 0; n < TD; n++) acc[m][n] = fmaf(a[m], bb[n], acc[m][n]);
        }
    }
    const size_t baseO = ((size_t)b * p.nb_a * BS + (size_t)i * BS) * HDo + (size_t)h * p.d;
#pragma unroll
    for (int m = 0; m < T; m++) {
        const float inv = sum[m] > 0.f ? 1.f / sum[m] : 0.f;
#pragma unroll
        for (int n = 0; n < TD; n++)
            if ((uint32_t)(tx + 16 * n) < p.d)
                Elem<DT>::store(O, baseO + (size_t)(ty + 16 * m) * HDo + tx + 16 * n, acc[m][n] * inv);
    }
}

// ------------------------------------------------------------------------------------------------
// host-side dispatch
#define DISPATCH_BS(bs, ...)            \
    if (bs == 32) { constexpr int BS = 32; __VA_ARGS__ } else { constexpr int BS = 64; __VA_ARGS__ }
#define DISPATCH_DT(dt, NAME, ...)                                         \
    if (dt == SFB_F32) { constexpr int NAME = SFB_F32; __VA_ARGS__ }        \
    else if (dt == SFB_BF16) { constexpr int NAME = SFB_BF16; __VA_ARGS__ } \
    else { constexpr int NAME = SFB_F16; __VA_ARGS__ }

int simt_sddmm_nt(cudaStream_t s, const void *lut, const void *a, const void *b, void *c, int ab_dtype, int c_dtype,
                  uint32_t bs, const AttnDims &p)
{
    dim3 grid(p.blocks, p.B, p.H);
    DISPATCH_BS(bs, DISPATCH_DT(ab_dtype, AB, {
        if (c_dtype == SFB_F32) sddmm_nt_kernel<BS, AB, SFB_F32><<<grid, 256, 0, s>>>((const uint2 *)lut, a, b, c, p);
        else if (c_dtype == SFB_BF16) sddmm_nt_kernel<BS, AB, SFB_BF16><<<grid, 256, 0, s>>>((const uint2 *)lut, a, b, c, p);
        else sddmm_nt_kernel<BS, AB, SFB_F16><<<grid, 256, 0, s>>>((const uint2 *)lut, a, b, c, p);
    }))
    return check_launch("sfb_bst_sgemm_nt");
}

int simt_softmax(cudaStream_t s, const void *lut, const void *mask, const void *x, void *y, int x_dtype, int y_dtype,
                 uint32_t bs, const AttnDims &p, float scale, uint32_t max_lut)
{
    const float sl = scale * LOG2E_F;
    // The caller's max_lut (0 = unknown) picks the variant.  16-bit scores: rows of up to 20 blocks stay in registers,
    // one pass over HBM; from 9 blocks up a CTA takes a quarter of the block-row's query rows.  Longer or unknown rows
    // are streamed: three sweeps, the second and third over lines the CTA has just pulled through L2.  Measured and not
    // kept for rows of 17-32 blocks: two groups of lanes per query row, each holding every other block (0.68 of copy
    // bandwidth on 17-block rows against 0.77 with 20 slots per lane).
    const int inplace = max_lut != 0 && max_lut <= 12;   // streamed short rows: unnormalised values wait in L2 for the rescale
    int nb = 0;   // block slots of the register tile, 0 = stream
    if (x_dtype == SFB_BF16)
        nb = max_lut == 0 ? 0 : max_lut <= 4 ? 4 : max_lut <= 8 ? 8 : max_lut <= 12 ? 12 : max_lut <= 16 ? 16 : max_lut <= 18 ? 18 : max_lut <= 20 ? 20 : 0;
    else
        nb = (max_lut >= 3 && max_lut <= 4) ? 4 : (max_lut >= 7 && max_lut <= 8) ? 8 : (max_lut >= 14 && max_lut <= 16) ? 16 : 0;
#define SM_LAUNCH(XD, NBV, SPL)                                                                                        \
    DISPATCH_DT(y_dtype, YD, {                                                                                         \
        softmax_kernel<BS, XD, YD, NBV, SPL><<<dim3(p.nb_a * SPL, p.B, p.H), BS * BS / 8 / SPL, 0, s>>>(             \
            (const uint2 *)lut, (const W *)mask, x, y, p, sl, inplace);                                                \
    })
    DISPATCH_BS(bs, {
        typedef typename MaskWord<BS>::type W;
        if (x_dtype == SFB_BF16) {
            if (nb == 4) { SM_LAUNCH(SFB_BF16, 4, 1) }
            else if (nb == 8) { SM_LAUNCH(SFB_BF16, 8, 1) }
            else if (nb == 12) { SM_LAUNCH(SFB_BF16, 12, 4) }
            else if (nb == 16) { SM_LAUNCH(SFB_BF16, 16, 4) }
            else if (nb == 18) { SM_LAUNCH(SFB_BF16, 18, 4) }
            else if (nb == 20) { SM_LAUNCH(SFB_BF16, 20, 4) }
            else { SM_LAUNCH(SFB_BF16, 0, 1) }
        } else {
            if (nb == 4) { SM_LAUNCH(SFB_F32, 4, 1) }
            else if (nb == 8) { SM_LAUNCH(SFB_F32, 8, 1) }
            else if (nb == 16) { SM_LAUNCH(SFB_F32, 16, 1) }
            else { SM_LAUNCH(SFB_F32, 0, 1) }
        }
    })
#undef SM_LAUNCH
    return check_launch("sfb_masked_softmax");
}

int simt_spmm_nn(cudaStream_t s, const void *lut, const void *a, const void *b, void *c, int a_dtype, int bc_dtype,
                 uint32_t bs, const AttnDims &p, bool trans)
{
    dim3 grid(p.nb_a * ((p.d + 63) / 64), p.B, p.H);
    DISPATCH_BS(bs, DISPATCH_DT(a_dtype, AD, DISPATCH_DT(bc_dtype, BD, {
        if (trans) spmm_nn_kernel<BS, AD, BD, true><<<grid, 256, 0, s>>>((const uint2 *)lut, a, b, c, p);
        else spmm_nn_kernel<BS, AD, BD, false><<<grid, 256, 0, s>>>((const uint2 *)lut, a, b, c, p);
    })))
    return check_launch("sfb_bst_sgemm_xn");
}

int simt_softmax_grad(cudaStream_t s, const void *lut, const void *dy, const void *y, void *dx, int dtype, uint32_t bs,
                      const AttnDims &p, float scale, uint32_t max_lut)
{
    // rows of up to 8 blocks (24 for 16-bit types; the caller's max_lut says so) stay in registers: one pass over
    // HBM; 0 = unknown, stream.  The streamed variant re-reads dy and y, and at full size those re-reads miss L2.
    const bool wide = dtype != SFB_F32;
    const int nb = (max_lut >= 1 && max_lut <= 4) ? 4 : (max_lut >= 5 && max_lut <= 8) ? 8
                   : (max_lut >= 9 && max_lut <= 12 && wide) ? 12 : (max_lut >= 13 && max_lut <= 16 && wide) ? 16
                   : (max_lut >= 17 && max_lut <= 24 && wide) ? 24 : 0;
#define SG_LAUNCH(NBV, SPL)                                                                                            \
    DISPATCH_DT(dtype, DT, {                                                                                           \
        softmax_grad_kernel<BS, DT, NBV, SPL><<<dim3(p.nb_a * SPL, p.B, p.H), BS * BS / 8 / SPL, 0, s>>>((const uint2 *)lut, dy, y, dx, p, scale); \
    })
    DISPATCH_BS(bs, {
        if (nb == 4) { SG_LAUNCH(4, 1) } else if (nb == 8) { SG_LAUNCH(8, 1) } else if (nb == 12) { SG_LAUNCH(12, 1) }
        else if (nb == 16) { SG_LAUNCH(16, 1) } else if (nb == 24) { SG_LAUNCH(24, 2) } else { SG_LAUNCH(0, 1) }
    })
#undef SG_LAUNCH
    return check_launch("sfb_masked_softmax_grad");
}

template <typename K>
static int set_smem(K kernel, size_t bytes)
{
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(%zu bytes): %s", bytes, cudaGetErrorString(e));
    }
    return 0;
}

int simt_fused_sddmm_softmax(cudaStream_t s, const void *nn_lut, const void *a, const void *b, const void *mask, void *y,
                             int ab_dtype, int y_dtype, uint32_t bs, const AttnDims &p, float scale)
{
    SFB_REQUIRE(p.d <= 128, "sfb_fused_sddmm_softmax: state_dim %u > 128 not supported", p.d);
    dim3 grid(p.nb_a, p.B, p.H);
    const float sl = scale * LOG2E_F;
#define LAUNCH_FSS(DMAX)                                                                                         \
    {                                                                                                            \
        typedef typename MaskWord<BS>::type W;                                                                   \
        size_t bytes = sizeof(float) * 2 * DMAX * (BS + 1);                                                      \
        auto kern = fused_sddmm_softmax_kernel<BS, DMAX, AB, YD>;                                                \
        if (set_smem(kern, bytes)) return 1;                                                                     \
        kern<<<grid, 256, bytes, s>>>((const uint2 *)nn_lut, a, b, (const W *)mask, y, p, sl);                   \
    }
    DISPATCH_BS(bs, DISPATCH_DT(ab_dtype, AB, DISPATCH_DT(y_dtype, YD, {
        if (p.d <= 64) LAUNCH_FSS(64) else LAUNCH_FSS(128)
    })))
#undef LAUNCH_FSS
    return check_launch("sfb_fused_sddmm_softmax");
}

int simt_fused_attention(cudaStream_t s, const void *nn_lut, const void *q, const void *k, const void *v, void *o,
                         const void *mask, int dtype, uint32_t bs, const AttnDims &p, float scale)
{
    SFB_REQUIRE(p.d <= 128, "sfb_fused_attention: state_dim %u > 128 not supported", p.d);
    dim3 grid(p.nb_a, p.B, p.H);
    const float sl = scale * LOG2E_F;
#define LAUNCH_FA(DMAX)                                                                                          \
    {                                                                                                            \
        typedef typename MaskWord<BS>::type W;                                                                   \
        size_t bytes = sizeof(float) * (2 * DMAX * (BS + 1) + BS * DMAX + BS * (BS + 16));                       \
        auto kern = fused_attention_kernel<BS, DMAX, DT>;                                                        \
        if (set_smem(kern, bytes)) return 1;                                                                     \
        kern<<<grid, 256, bytes, s>>>((const uint2 *)nn_lut, q, k, v, o, (const W *)mask, p, sl);                \
    }
    DISPATCH_BS(bs, DISPATCH_DT(dtype, DT, {
        if (p.d <= 64) LAUNCH_FA(64) else LAUNCH_FA(128)
    }))
#undef LAUNCH_FA
    return check_launch("sfb_fused_attention");
}

}  // namespace sfb
