// Shared pieces of the tcgen05 kernels: PTX wrappers (mbarrier, TMA, tcgen05.mma / ld / st), the bounded
// waits with the library's status word, the union of two block-rows' key blocks, and the host-side
// tensor-map encoder.
#pragma once
#include "attn.cuh"
#include <cuda.h>

namespace sfb {
namespace tc {

constexpr int kMaxUnion = 512;                  // key blocks a row pair may touch
constexpr uint32_t kTileBytes = 64 * 64 * 2;    // one 64x64 16-bit tile
constexpr uint32_t kQBytes = 128 * 64 * 2;
#ifndef SFB_WAIT_LIMIT_LOG2
#define SFB_WAIT_LIMIT_LOG2 24
#endif
constexpr uint32_t kWaitLimit = 1u << SFB_WAIT_LIMIT_LOG2;   // polls before a bounded wait gives up

struct UnionEntry {
    uint32_t col;      // key block column
    uint32_t flags;    // bit 0: upper block-row has it, bit 1: lower block-row has it
    uint32_t blk[2];   // block ids
};

// 0 = ok; otherwise (code << 24 | CTA index) of the first CTA that gave up on a bounded wait.  One copy per
// translation unit (no relocatable device code); each .cu that includes this header exports a reader.
static __device__ uint32_t g_status = 0;

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// one look at the barrier that never suspends the thread (for a thread that watches several barriers)
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// the same with a suspend-time hint: the thread sleeps in the barrier unit until the phase completes or about
// `ns` nanoseconds have passed, instead of coming back at once and polling again (polling warps take issue slots
// and shared-memory bandwidth from the warps that do the work)
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t *bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// bounded wait: false when the limit ran out or another role already gave up
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
{
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(&g_status, 0u, (code << 24) | (blockIdx.x & 0xffffffu));
    return false;
}

// the same wait for a whole warp: one outcome for all lanes, and the warp is converged afterwards
// (the tcgen05.ld / tcgen05.st that follow are .sync.aligned)
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
{
    const bool ok = mbar_wait(bar, parity, abort_flag, code);
    return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint64_t *bar, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// same, with the A operand read from TMEM (lane = row, one 32-bit column = two 16-bit elements along K)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart.  lbo_bytes only matters
// for an MN-major operand wider than 64 elements: it is the distance to the next group of 64 columns.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes = 16)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);   // start address
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;   // leading byte offset
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
    d |= (uint64_t)1 << 46;                    // descriptor version
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}

// instruction descriptor of kind::f16: fp32 accumulator, M x N tile, 16-bit A and B (0 = fp16, 1 = bf16)
__device__ __forceinline__ uint32_t instr_desc(uint32_t a_fmt, uint32_t b_fmt, uint32_t M, uint32_t N, uint32_t b_mn_major)
{
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (b_mn_major << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

#define TMEM_LD_32(r, addr)                                                                                              \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                               \
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,"   \
                 "%27,%28,%29,%30,%31}, [%32];"                                                                          \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),       \
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), \
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),            \
                   "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),            \
                   "=r"(r[30]), "=r"(r[31])                                                                              \
                 : "r"(addr)                                                                                             \
                 : "memory")

#define TMEM_ST_32(addr, r)                                                                                              \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                         \
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"  \
                 "%28,%29,%30,%31,%32};"                                                                                 \
                 ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),    \
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),         \
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),       \
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])        \
                 : "memory")

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- packed fp32 pairs (one instruction, two lanes) ----
__device__ __forceinline__ uint64_t pk64(float a, float b)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void up64(uint64_t v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2p(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2p(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add2p_rm(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rm.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2p(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t sub2p(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// exp2 of a pair on the FMA pipe: x = n + f with n = floor(x) taken by a magic-number add that rounds down, a cubic
// in f on [0, 1) (max relative error 1.6e-4, below half a unit of either 16-bit format P is rounded to), n added
// into the exponent field.  x <= 0 up to the lazy-max slack, clamped at -120 so that the exponent cannot wrap.
__device__ __forceinline__ void exp2_fma_pair(uint64_t x, float &e0, float &e1)
{
    const uint64_t magic = pk64(12582912.f, 12582912.f);   // 1.5 * 2^23
    float x0, x1;
    up64(x, x0, x1);
    x = pk64(fmaxf(x0, -120.f), fmaxf(x1, -120.f));
    const uint64_t r = add2p_rm(x, magic);
    const uint64_t f = sub2p(x, sub2p(r, magic));
    uint64_t q = fma2p(pk64(0.0790210f, 0.0790210f), f, pk64(0.2249302f, 0.2249302f));
    q = fma2p(q, f, pk64(0.6960656f, 0.6960656f));
    q = fma2p(q, f, pk64(1.0f, 1.0f));
    float q0, q1, r0, r1;
    up64(q, q0, q1);
    up64(r, r0, r1);
    e0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(r0) << 23));
    e1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(r1) << 23));
}

// packed fp16 pair -> packed bf16 pair (the MMA wants A and B in one format)
__device__ __forceinline__ uint32_t f16x2_to_bf16x2(uint32_t v)
{
    const float2 f = __half22float2(*reinterpret_cast<__half2 *>(&v));
    __nv_bfloat162 o = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<uint32_t *>(&o);
}
// (a0, a1) * b + c on the packed fp32 pipe
__device__ __forceinline__ void fma2(float &d0, float &d1, float a0, float a1, float b, float c)
{
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %4};\n\t"
        "mov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int is_bf16)
{
    if (is_bf16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

#define TMEM_LD_16(r, addr)                                                                                          \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];" \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),   \
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) \
                 : "r"(addr)                                                                                         \
                 : "memory")
#define TMEM_ST_16(addr, r)                                                                                          \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" \
                 ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), \
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])      \
                 : "memory")

// Builds the union of the key blocks of block-rows 2*pair and 2*pair+1 in shared memory: the upper row's
// blocks in LUT order, then the blocks only the lower row has.  All threads of the CTA call it (it contains
// __syncthreads); the result is complete after the caller's next __syncthreads.  cand is kMaxUnion words of
// scratch.  Returns through *n_out; 0 with *abort_flag set if a row does not fit.  Two dependent global reads
// deep (row headers, then both rows' entries at once); everything after that works from shared memory.
__device__ __forceinline__ void build_union(const uint2 *nn, uint32_t pair, uint32_t nb, UnionEntry *entries,
                                            uint2 *cand, uint32_t *n_out, uint32_t *abort_flag)
{
    const uint32_t row0 = pair * 2, row1 = pair * 2 + 1;
    const uint2 head0 = nn[row0];
    const uint2 head1 = row1 < nb ? nn[row1] : make_uint2(0, 0);
    const uint32_t n0 = head0.y, n1 = head1.y;
    const bool fits = n0 <= kMaxUnion && n1 <= kMaxUnion;
    if (fits) {
        for (uint32_t i = threadIdx.x; i < n0 + n1; i += blockDim.x) {
            if (i < n0) {
                const uint2 ent = nn[head0.x + i];
                entries[i].col = ent.y;
                entries[i].flags = 1;
                entries[i].blk[0] = ent.x;
                entries[i].blk[1] = 0;
            } else {
                cand[i - n0] = nn[head1.x + (i - n0)];
            }
        }
    }
    __syncthreads();
    if (fits) {
        // lower-row blocks the upper row has too: tag the existing entry, mark the candidate as placed
        for (uint32_t e = threadIdx.x; e < n1; e += blockDim.x) {
            const uint2 ent = cand[e];
            for (uint32_t u = 0; u < n0; u++)
                if (entries[u].col == ent.y) {
                    entries[u].flags |= 2;
                    entries[u].blk[1] = ent.x;
                    cand[e].y = 0xffffffffu;
                    break;
                }
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        // the rest are appended in order: ballot + prefix count per group of 32 candidates
        uint32_t n = n0;
        bool ok = fits;
        for (uint32_t base = 0; ok && base < n1; base += 32) {
            const uint32_t e = base + threadIdx.x;
            const uint2 ent = e < n1 ? cand[e] : make_uint2(0, 0xffffffffu);
            const bool fresh = ent.y != 0xffffffffu;
            const uint32_t votes = __ballot_sync(0xffffffffu, fresh);
            const uint32_t at = n + __popc(votes & ((1u << threadIdx.x) - 1u));
            ok = n + __popc(votes) <= kMaxUnion;
            if (ok && fresh) {
                entries[at].col = ent.y;
                entries[at].flags = 2;
                entries[at].blk[0] = 0;
                entries[at].blk[1] = ent.x;
            }
            n += __popc(votes);
        }
        if (threadIdx.x == 0) {
            if (!ok) {
                n = 0;
                *abort_flag = 1;
                atomicCAS(&g_status, 0u, (9u << 24) | (blockIdx.x & 0xffffffu));  // row pair too long for these kernels
            }
            *n_out = n;
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// [rows, H*64] 16-bit row-major tensor, boxes of box_rows x 64 elements (one head's slice), 128-byte swizzle; pitch =
// elements between consecutive rows (0 = H*64; larger when the H heads are a slice of a wider tensor)
inline int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint32_t H, int is_bf16, uint32_t box_rows, uint64_t pitch = 0)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)H * 64, rows};
    cuuint64_t strides[1] = {(cuuint64_t)(pitch ? pitch : (uint64_t)H * 64) * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}


}  // namespace tc
}  // namespace sfb
