// Fused block-sparse attention on the 5th-generation tensor cores (tcgen05) for 16-bit operands,
// block_size 64, head size 64.
//
// One CTA owns a PAIR of adjacent block-rows (128 queries = one M=128 MMA tile) and walks the union of
// the two rows' key blocks.  Nothing is exchanged between CTAs: no flags, no scratch, no waiting on
// other CTAs.  Per key block:
//     S  = Q . K^T            tcgen05.mma, A and B from shared memory, accumulator in TMEM (two S buffers)
//     P  = exp2(S*c - m)      128 threads, one query row each, straight out of TMEM (two exponentials per
//                             MUFU instruction on packed fp16); P is written back over S as 16-bit pairs
//     O += P . [V | 1]        tcgen05.mma, P as the A operand from TMEM, V from shared memory as an
//                             MN-major operand, followed by a tile of ones: 16 extra accumulator
//                             columns receive the row sums of P, so the softmax denominator comes out
//                             of the tensor core and is rescaled together with O
// Warp roles: warp 0 issues the TMA loads, warp 1 issues the MMAs, warps 2-5 do the softmax and the
// epilogue.  Every wait on an mbarrier is bounded; on a timeout the CTA records a status word and
// leaves through the common teardown (TMEM freed, loads in flight drained).
#include "attn.cuh"
#include <cuda.h>

namespace sfb {

namespace tc {

constexpr int kStages = 4;                      // K/V ring depth
constexpr int kMaxUnion = 512;                  // key blocks a row pair may touch
constexpr uint32_t kTileBytes = 64 * 64 * 2;    // one 64x64 16-bit tile
constexpr uint32_t kQBytes = 128 * 64 * 2;
constexpr uint32_t kTmemCols = 256;             // S0 | S1 | O (64 + 16 row-sum columns); P reuses S's first 32 columns
constexpr uint32_t kOnesBytes = 64 * 128;       // the tile of ones behind V
constexpr uint32_t kWaitLimit = 1u << 24;
constexpr float kRescaleThreshold = 8.0f;       // log2 units: P stays below 2^8

struct UnionEntry {
    uint32_t col;      // key block column
    uint32_t flags;    // bit 0: upper block-row has it, bit 1: lower block-row has it
    uint32_t blk[2];   // block ids (for the element masks)
};

struct SharedState {
    uint64_t q_full, kv_full[kStages], kv_empty[kStages];
    uint64_t s_full[2], p_full[2], pv_done, o_final, drained;
    uint32_t tmem_base, n_union, abort_flag, pad;
    UnionEntry entries[kMaxUnion];
    uint8_t found[kMaxUnion];
};

constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + kQBytes + kStages * 2 * kTileBytes + kOnesBytes + sizeof(SharedState);

struct Params {
    const uint2 *nn_lut;
    const uint64_t *mask;
    void *O;
    uint32_t B, H, nb, blocks, lut_stride, mask_stride;
    float scale_log2e;
    int is_bf16;
};

__device__ uint32_t g_status = 0;

#ifdef SFB_TC_TIMING
// per-phase cycle counts of one softmax lane and the MMA lane of one CTA (profiling builds only)
__device__ unsigned long long g_timing[32];
#define TIC(var) const long long var = clock64()
#define TOC(slot, var) do { if (timing_on) atomicAdd(&g_timing[slot], (unsigned long long)(clock64() - var)); } while (0)
#else
#define TIC(var)
#define TOC(slot, var)
#endif  // 0 = ok; otherwise (code << 24 | detail) of the first CTA that gave up

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

// exp2 of two values at once: fp32 pair -> packed fp16 pair -> MUFU on both halves (lo = first value)
__device__ __forceinline__ uint32_t ex2_pair_f16(float lo, float hi)
{
    __half2 h = __floats2half2_rn(lo, hi);
    uint32_t x = *reinterpret_cast<uint32_t *>(&h), y;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
    return y;
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

// ---- the kernel ---------------------------------------------------------------------------------
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

template <bool HAS_MASK, bool BF16>
__global__ void __launch_bounds__(192, 2)
fused_attention_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                          const __grid_constant__ CUtensorMap vmap, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *q_tile = smem;
    uint8_t *kv_tiles = q_tile + kQBytes;                      // stage s: K at s*2*kTileBytes, V right after
    uint8_t *ones_tile = kv_tiles + kStages * 2 * kTileBytes;
    SharedState *st = (SharedState *)(ones_tile + kOnesBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t pair = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const uint32_t row0 = pair * 2, row1 = pair * 2 + 1;
    const bool has_row1 = row1 < p.nb;
    const uint32_t L = p.nb * 64;
    const uint2 *nn = p.nn_lut + (size_t)h * p.lut_stride;
    volatile uint32_t *abort_flag = &st->abort_flag;
    const uint32_t fmt = BF16 ? 1u : 0u;

    // ---- set-up: barriers, the tile of ones, TMEM, the union of the two rows' key blocks ----
    if (threadIdx.x == 0) {
        mbar_init(&st->q_full, 1);
        for (int s = 0; s < kStages; s++) {
            mbar_init(&st->kv_full[s], 1);
            mbar_init(&st->kv_empty[s], 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(&st->s_full[s], 1);
            mbar_init(&st->p_full[s], 128);
        }
        mbar_init(&st->pv_done, 1);
        mbar_init(&st->o_final, 1);
        mbar_init(&st->drained, 1);
        st->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {
        // 1.0 in the operand type of V, everywhere: the swizzle cannot matter
        const uint32_t one2 = BF16 ? 0x3f803f80u : 0x3c003c00u;
        for (uint32_t i = threadIdx.x; i < kOnesBytes / 16; i += blockDim.x)
            ((uint4 *)ones_tile)[i] = make_uint4(one2, one2, one2, one2);
        fence_proxy_async();
    }
    const uint2 head0 = nn[row0];
    const uint2 head1 = has_row1 ? nn[row1] : make_uint2(0, 0);
    const uint32_t n0 = head0.y, n1 = head1.y;
    const bool fits = n0 <= kMaxUnion && n1 <= kMaxUnion;
    if (fits) {
        for (uint32_t e = threadIdx.x; e < n0; e += blockDim.x) {
            uint2 ent = nn[head0.x + e];
            st->entries[e].col = ent.y;
            st->entries[e].flags = 1;
            st->entries[e].blk[0] = ent.x;
            st->entries[e].blk[1] = 0;
        }
    }
    __syncthreads();
    if (fits) {
        for (uint32_t e = threadIdx.x; e < n1; e += blockDim.x) {
            uint2 ent = nn[head1.x + e];
            uint8_t f = 0;
            for (uint32_t u = 0; u < n0; u++)
                if (st->entries[u].col == ent.y) {
                    st->entries[u].flags |= 2;
                    st->entries[u].blk[1] = ent.x;
                    f = 1;
                    break;
                }
            st->found[e] = f;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t n = n0;
        bool ok = fits;
        for (uint32_t e = 0; ok && e < n1; e++)
            if (!st->found[e]) {
                if (n >= kMaxUnion) { ok = false; break; }
                uint2 ent = nn[head1.x + e];
                st->entries[n].col = ent.y;
                st->entries[n].flags = 2;
                st->entries[n].blk[0] = 0;
                st->entries[n].blk[1] = ent.x;
                n++;
            }
        if (!ok) {
            n = 0;
            st->abort_flag = 1;
            atomicCAS(&g_status, 0u, (9u << 24) | (blockIdx.x & 0xffffffu));  // row pair too long for this kernel
        }
        st->n_union = n;
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&st->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();

#ifdef SFB_TC_TIMING
    const bool timing_on = blockIdx.x == 7 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp == 1 || warp == 2);
#endif
    const uint32_t T = st->n_union;
    const uint32_t tmem = st->tmem_base;
    const uint32_t tmem_s[2] = {tmem, tmem + 64};
    const uint32_t tmem_o = tmem + 128;          // 64 columns of O, then 16 columns that all hold the row sum
    const int32_t xq = (int32_t)(h * 64);

    if (warp == 0) {
        // ===== TMA producer: a stage (K and V of one key block) is released when its P.V has completed =====
        if (lane == 0 && T > 0) {
            mbar_expect_tx(&st->q_full, kQBytes);
            tma_load_2d(smem_u32(q_tile), &qmap, &st->q_full, xq, (int32_t)(b * L + pair * 128));
            for (uint32_t t = 0; t < T; t++) {
                const uint32_t s = t % kStages;
                const int32_t y = (int32_t)(b * L + st->entries[t].col * 64);
                if (t >= kStages && !mbar_wait(&st->kv_empty[s], ((t / kStages) - 1) & 1, abort_flag, 1)) break;
                mbar_expect_tx(&st->kv_full[s], 2 * kTileBytes);
                tma_load_2d(smem_u32(kv_tiles + s * 2 * kTileBytes), &kmap, &st->kv_full[s], xq, y);
                tma_load_2d(smem_u32(kv_tiles + s * 2 * kTileBytes + kTileBytes), &vmap, &st->kv_full[s], xq, y);
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: S(0) | S(1) O(0) | S(2) O(1) | ...  S(t+1) lands in the buffer that held P(t-1); the
        // tensor core runs this thread's MMAs in order, so P(t-1) has been consumed by then =====
        if (lane == 0 && T > 0) {
            const uint32_t idesc_qk = instr_desc(fmt, fmt, 128, 64, 0);
            const uint32_t idesc_pv = instr_desc(fmt, fmt, 128, 80, 1);   // A and B must share a format
            const uint64_t q_desc = smem_desc_sw128(smem_u32(q_tile));
            bool alive = mbar_wait(&st->q_full, 0, abort_flag, 2);
            auto issue_qk = [&](uint32_t t) -> bool {
                const uint32_t s = t % kStages;
                TIC(c0);
                if (!mbar_wait(&st->kv_full[s], (t / kStages) & 1, abort_flag, 3)) return false;
                TOC(10, c0);
                tcgen05_fence_after();
                const uint64_t k_desc = smem_desc_sw128(smem_u32(kv_tiles + s * 2 * kTileBytes));
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++)   // 16 of the 64 head elements per MMA: +32 bytes inside the swizzled row
                    umma_f16(tmem_s[t & 1], q_desc + 2 * kk, k_desc + 2 * kk, idesc_qk, kk);
                umma_commit(&st->s_full[t & 1]);
                return true;
            };
            if (alive) alive = issue_qk(0);
            for (uint32_t t = 0; alive && t < T; t++) {
                const uint32_t s = t % kStages;
                if (t + 1 < T && !issue_qk(t + 1)) { alive = false; break; }
                TIC(c2);
                if (!mbar_wait(&st->p_full[t & 1], (t >> 1) & 1, abort_flag, 5)) { alive = false; break; }
                TOC(12, c2);
                tcgen05_fence_after();
                // B = [V | ones]: 64 columns from the V tile, the next group of columns from the tile of ones
                const uint32_t v_addr = smem_u32(kv_tiles + s * 2 * kTileBytes + kTileBytes);
                const uint64_t v_desc = smem_desc_sw128(v_addr, smem_u32(ones_tile) - v_addr);
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++)   // 16 keys per MMA: 8 TMEM columns of P, 16 rows (2048 bytes) of V
                    umma_f16_ts(tmem_o, tmem_s[t & 1] + 8 * kk, v_desc + 128 * kk, idesc_pv, (t | kk) ? 1u : 0u);
                umma_commit(&st->kv_empty[s]);
                umma_commit(&st->pv_done);
                // the epilogue may be two completions ahead of pv_done, which a parity wait cannot tell apart
                if (t + 1 == T) umma_commit(&st->o_final);
            }
        }
    } else {
        // ===== softmax + epilogue: one query row per thread =====
        const uint32_t quarter = warp & 3;                 // TMEM lanes this warp may touch
        const uint32_t r = quarter * 32 + lane;            // row inside the 128-query tile
        const uint32_t half = r >> 6;                      // which of the two block-rows
        const uint32_t lane_field = (quarter * 32) << 16;
        const bool row_valid = half == 0 || has_row1;
        const float sl = p.scale_log2e;
        float m_used = -INFINITY;
        bool alive = true;

        TIC(c_loop);
        for (uint32_t t = 0; t < T; t++) {
            TIC(c0);
            if (!mbar_wait_warp(&st->s_full[t & 1], (t >> 1) & 1, abort_flag, 6)) { alive = false; break; }
            TOC(0, c0);
            TIC(c1);
            tcgen05_fence_after();
            uint32_t sr[64];
            TMEM_LD_32((sr), tmem_s[t & 1] + lane_field);
            TMEM_LD_32((sr + 32), tmem_s[t & 1] + lane_field + 32);
            tmem_wait_ld();
            TOC(1, c1);
            TIC(c2);

            const UnionEntry ent = st->entries[t];
            const bool mine = (ent.flags >> half) & 1;
            float mx = -INFINITY;
            if (mine) {
                if (HAS_MASK) {
                    const uint64_t w = p.mask[(size_t)h * p.mask_stride + (size_t)ent.blk[half] * 64 + (r & 63)];
#pragma unroll
                    for (int c = 0; c < 64; c++)
                        if (!((w >> c) & 1)) sr[c] = 0xff800000u;
                }
                float m4[4];
#pragma unroll
                for (int c = 0; c < 4; c++) m4[c] = __uint_as_float(sr[c]);
#pragma unroll
                for (int c = 4; c < 64; c += 8) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (c + 2 * j + 1 < 64)
                            m4[j] = max3(m4[j], __uint_as_float(sr[c + 2 * j]), __uint_as_float(sr[c + 2 * j + 1]));
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl;
            }
            // move the reference max only when the row max outgrew it by 2^8: rescaling O stays rare
            const bool grow = mx > m_used + kRescaleThreshold || (m_used == -INFINITY && mx > -INFINITY);
            const bool fix_o = grow && m_used > -INFINITY;
            float alpha = 1.f;
            if (grow) {
                alpha = fix_o ? ex2_approx(m_used - mx) : 0.f;
                m_used = mx;
            }
            if (t > 0 && __any_sync(0xffffffffu, fix_o)) {
                // O (and the row sums next to it) must be complete before they are rescaled
                if (!mbar_wait_warp(&st->pv_done, (t - 1) & 1, abort_flag, 7)) { alive = false; break; }
                tcgen05_fence_after();
                const float a = fix_o ? alpha : 1.f;
#pragma unroll
                for (int c0 = 0; c0 < 80; c0 += 16) {
                    uint32_t oc[16];
                    TMEM_LD_16((oc), tmem_o + lane_field + c0);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 16; c++) oc[c] = __float_as_uint(__uint_as_float(oc[c]) * a);
                    TMEM_ST_16(tmem_o + lane_field + c0, (oc));
                }
                tmem_wait_st();
            }
            TOC(2, c2);
            TIC(c3);
            const float neg_m = m_used > -INFINITY ? -m_used : 0.f;
            uint32_t pk[32];
            if (mine) {
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    float x0, x1;
                    fma2(x0, x1, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]), sl, neg_m);
                    const uint32_t e2 = ex2_pair_f16(x0, x1);
                    pk[c >> 1] = BF16 ? f16x2_to_bf16x2(e2) : e2;
                }
            } else {
#pragma unroll
                for (int c = 0; c < 32; c++) pk[c] = 0u;
            }
            TOC(3, c3);
            TIC(c5);
            // P (16-bit pairs) takes the place of the first 32 columns of this row of S
            TMEM_ST_32(tmem_s[t & 1] + lane_field, (pk));
            tmem_wait_st();
            tcgen05_fence_before();
            mbar_arrive(&st->p_full[t & 1]);
            TOC(5, c5);
        }
        TOC(6, c_loop);
#ifdef SFB_TC_TIMING
        if (timing_on) atomicAdd(&g_timing[7], (unsigned long long)T);
#endif

        // ---- epilogue: O / row sum -> global ----
        if (T > 0 && alive) alive = mbar_wait_warp(&st->o_final, 0, abort_flag, 10);
        if (alive && row_valid) {
            tcgen05_fence_after();
            float inv = 0.f;
            if (T > 0) {
                uint32_t lc[16];
                TMEM_LD_16((lc), tmem_o + lane_field + 64);
                tmem_wait_ld();
                const float lsum = __uint_as_float(lc[0]);
                inv = lsum > 0.f ? 1.f / lsum : 0.f;
            }
            uint16_t *dst = (uint16_t *)p.O + ((size_t)b * L + (size_t)pair * 128 + r) * ((size_t)p.H * 64) + (size_t)h * 64;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t oc[16], w[8];
                if (T > 0) {
                    TMEM_LD_16((oc), tmem_o + lane_field + c0);
                    tmem_wait_ld();
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float a0 = T > 0 ? __uint_as_float(oc[2 * j]) * inv : 0.f;
                    const float a1 = T > 0 ? __uint_as_float(oc[2 * j + 1]) * inv : 0.f;
                    w[j] = pack2(a0, a1, BF16);
                }
                *(uint4 *)(dst + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                *(uint4 *)(dst + c0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
            }
        } else if (!row_valid) {
            // lanes of the absent lower block-row still take part in the aligned TMEM loads above: nothing to do
        }
    }

    // ---- teardown (also the way out after a timeout) ----
    tcgen05_fence_before();
    __syncthreads();
    if (st->abort_flag) {
        // give loads and MMAs in flight a bounded time to land before shared memory and TMEM are released
        if (warp == 1 && lane == 0) {
            umma_commit(&st->drained);
            for (uint32_t i = 0; i < kWaitLimit && !mbar_try_wait(&st->drained, 0); i++) {}
        }
        if (warp == 0 && lane == 0) {
            const uint64_t t0 = clock64();
            while (clock64() - t0 < 2000000ull) {}
        }
        __syncthreads();
    }
    if (warp == 0) {
        __syncwarp();
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
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

// [rows, H*64] 16-bit row-major tensor, boxes of box_rows x 64 elements (one head's slice), 128-byte swizzle
static int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint32_t H, int is_bf16, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)H * 64, rows};
    cuuint64_t strides[1] = {(cuuint64_t)H * 64 * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

}  // namespace tc

bool tc_fused_attention_supported(int dtype, uint32_t bs, const AttnDims &p, float scale, uint32_t max_lut)
{
    return (dtype == SFB_BF16 || dtype == SFB_F16) && bs == 64 && p.d == 64 && scale > 0.f && p.nb_a == p.nb_b &&
           2 * (uint64_t)max_lut <= tc::kMaxUnion && (uint64_t)p.B * p.nb_a * 64 < (1ull << 31);
}

int tc_fused_attention(cudaStream_t s, const void *nn_lut, const void *q, const void *k, const void *v, void *o,
                       const void *mask, int dtype, const AttnDims &p, float scale)
{
    using namespace tc;
    const uintptr_t al = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o;
    SFB_REQUIRE((al & 15) == 0, "sfb_fused_attention: q, k, v, o must be 16-byte aligned");
    const int is_bf16 = dtype == SFB_BF16;
    const uint64_t rows = (uint64_t)p.B * p.nb_a * 64;
    CUtensorMap qm, km, vm;
    if (make_map(&qm, q, rows, p.H, is_bf16, 128) || make_map(&km, k, rows, p.H, is_bf16, 64) ||
        make_map(&vm, v, rows, p.H, is_bf16, 64))
        return 1;
    Params prm = {(const uint2 *)nn_lut, (const uint64_t *)mask, o, p.B, p.H, p.nb_a, p.blocks, p.lut_stride, p.mask_stride,
                  scale * 1.4426950408889634f, is_bf16};
    dim3 grid((p.nb_a + 1) / 2, p.B, p.H);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(fused_attention_tc_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fused_attention_tc_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fused_attention_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fused_attention_tc_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return fail("sfb_fused_attention: cannot reserve %zu bytes of shared memory", kSmemBytes);
        configured = true;
    }
    if (mask && is_bf16) fused_attention_tc_kernel<true, true><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, prm);
    else if (mask) fused_attention_tc_kernel<true, false><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, prm);
    else if (is_bf16) fused_attention_tc_kernel<false, true><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, prm);
    else fused_attention_tc_kernel<false, false><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, prm);
    return check_launch("sfb_fused_attention");
}

#ifdef SFB_TC_TIMING
extern "C" int sfb_debug_timing(unsigned long long *out, int reset)
{
    cudaMemcpyFromSymbol(out, tc::g_timing, sizeof(unsigned long long) * 32);
    if (reset) {
        unsigned long long z[32] = {0};
        cudaMemcpyToSymbol(tc::g_timing, z, sizeof(z));
    }
    return 0;
}
#endif

int tc_status(uint32_t *out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, tc::g_status, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace sfb
