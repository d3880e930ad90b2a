// Dense projection on the 5th-generation tensor cores: out[m, n] = act(x[m, k] . w[k, n] + bias[n]) for 16-bit
// x, w and out (fp32 accumulation, fp32 bias).  This is the product the encoder layer makes six times around the
// block-sparse attention (Q/K/V/output projections, the two FFN matrices), with the bias add and the GELU that
// the reference launches as separate kernels folded into the epilogue.
//
// Persistent, one CTA per SM.  A CTA tile is 128 rows x 256 columns: x arrives by TMA as a K-major A operand
// (128 x 64 per stage), w -- row-major [k, n], so n is the contiguous direction -- as an MN-major B operand
// (four 64 x 64 boxes per stage, one 128-byte swizzle span each; the descriptor's leading-dimension offset
// steps from one to the next), four stages of 48 KB.  One thread issues M128 N256 K16 tcgen05.mma into one of
// two 256-column accumulators in TMEM; eight epilogue warps drain the other one (tcgen05.ld, bias, activation,
// 32-byte stores), so the epilogue of a tile runs under the MMAs of the next.
// Every wait on an mbarrier is bounded; on a timeout the CTA records a status word and leaves through the
// common teardown.
#include "tc_common.cuh"
#include <cstdlib>

namespace sfb {
namespace tc {

constexpr uint32_t kGBM = 128, kGBN = 256, kGBK = 64;
constexpr uint32_t kGABytes = kGBM * kGBK * 2;           // 16 KB per 128 rows
constexpr uint32_t kGBBytes = kGBK * kGBN * 2;           // 32 KB: four 64 x 64 boxes
// MT = row sub-tiles of 128 per CTA tile.  MT = 1: 128 x 256 tiles, two accumulators, the epilogue of a tile runs
// under the MMAs of the next.  MT = 2: 256 x 256 tiles -- both sub-tiles multiply the same w boxes, so a third less
// travels from L2 per flop, which is what long-k products are bound by -- at the price of a single accumulator set.
template <int MT> struct GCfg {
    static constexpr int stages = MT == 1 ? 4 : 3;
    static constexpr int acc_bufs = MT == 1 ? 2 : 1;
    static constexpr uint32_t stage_bytes = MT * kGABytes + kGBBytes;
    static constexpr size_t smem = 1024 + stages * stage_bytes + 256;
};
constexpr int kGMaxStages = 4;

struct GShared {
    uint64_t full[kGMaxStages], empty[kGMaxStages], acc_full[2], acc_empty[2], drained;
    uint32_t tmem_base, abort_flag;
};
static_assert(sizeof(GShared) <= 256, "GShared outgrew its slot");

struct GParams {
    void *out;
    const float *bias;
    uint32_t M, N, K, tiles_m, tiles_n;
    int is_bf16, act;
    int w_transposed;   // w is [n, k] row-major (out = x . w^T, the tied-embedding logits): its tile is a K-major B operand
    uint32_t band;      // CTA-pair kernel: column tiles per band of the tile order (tile_coords)
};

// Tile t of the CTA-pair kernel -> (row tile, column tile).  The tiles run band by band, a band being `band` column
// tiles wide, row tile by row tile inside it: the pairs that work at the same time then spread over `band` different
// w tiles and a stripe of x tiles, instead of all asking the same few L2 slices for one w tile at once (eight wide: the
// 74 pairs of a B200 then cover about nine row tiles by eight column tiles; measured against 1, 2 and 4).
__device__ __forceinline__ void tile_coords(const GParams &p, uint32_t t, uint32_t &tm, uint32_t &tn)
{
    const uint32_t per_band = p.tiles_m * p.band;
    const uint32_t b = t / per_band, rem = t - b * per_band;
    const uint32_t width = min(p.band, p.tiles_n - b * p.band);    // the last band may be narrower
    tm = rem / width;
    tn = b * p.band + (rem - tm * width);
}

__device__ __forceinline__ float gelu_ref(float t)
{
    // x * sigmoid(1.702 x), the reference's GELU (gelu_gpu_v2, cuda_kernels.h:561-581), as
    // 0.5 x tanh(0.851 x) + 0.5 x: one MUFU operation per element instead of an exponential and a reciprocal
    // (tanh.approx: relative error about 2^-11, below half a unit of the 16-bit output)
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.851f * t));
    const float h = 0.5f * t;
    return fmaf(h, th, h);
}

// One thread's share of a 128-row accumulator: row `row` of the output, 128 columns from n0 on, read from TMEM at
// tcol 32 columns at a time (the next 32 travel while these are written), bias and activation applied, 32-byte stores.
__device__ __forceinline__ void drain_rows(const GParams &p, uint32_t tcol, uint32_t row, uint32_t n0)
{
    const bool row_ok = row < p.M;
    const size_t off = (size_t)row * p.N + n0;
    uint32_t v[2][32];
    TMEM_LD_32((v[0]), tcol);
#pragma unroll
    for (uint32_t c = 0; c < 4; c++) {
        const uint32_t c0 = c * 32;
        tmem_wait_ld();
        if (c + 1 < 4) TMEM_LD_32((v[(c + 1) & 1]), tcol + c0 + 32);
        uint32_t(&cur)[32] = v[c & 1];
#pragma unroll
        for (uint32_t q = 0; q < 2; q++) {
            const uint32_t col = n0 + c0 + q * 16;
            if (row_ok && col < p.N) {      // N is a multiple of 16: a group of 16 is inside or outside as a whole
                float x[16];
#pragma unroll
                for (int j = 0; j < 16; j++) x[j] = __uint_as_float(cur[q * 16 + j]);
                if (p.bias) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float4 bb = __ldg((const float4 *)(p.bias + col) + j);   // the same address in every lane: one broadcast
                        x[4 * j] += bb.x; x[4 * j + 1] += bb.y; x[4 * j + 2] += bb.z; x[4 * j + 3] += bb.w;
                    }
                }
                if (p.act == 1) {
#pragma unroll
                    for (int j = 0; j < 16; j++) x[j] = gelu_ref(x[j]);
                }
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 8; j++) w[j] = pack2(x[2 * j], x[2 * j + 1], p.is_bf16);
                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"((uint16_t *)p.out + off + c0 + q * 16),
                             "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                             : "memory");
            }
        }
    }
}

// The same share of an accumulator, leaving through shared memory: the warp's 32 rows x 64 columns are packed into a
// staging tile in the tensor map's 128-byte swizzle (16-byte chunk c of row r at chunk c ^ (r % 8)) and one lane hands
// the tile to the TMA, twice per 128 columns.  The writes reach memory as whole 128-byte rows instead of 32 bytes per
// thread and instruction, and the storing threads are free as soon as the tile is in shared memory.
// row0 = first of the warp's 32 rows, n0 = first of its 128 columns.
__device__ __forceinline__ void drain_rows_staged(const GParams &p, const CUtensorMap *omap, uint32_t tcol, uint8_t *stage, uint32_t row0,
                                                  uint32_t n0, uint32_t lane)
{
    uint8_t *srow = stage + lane * 128;
    uint32_t v[2][32];
    TMEM_LD_32((v[0]), tcol);
#pragma unroll
    for (uint32_t c = 0; c < 4; c++) {
        const uint32_t c0 = c * 32;
        tmem_wait_ld();
        if (c + 1 < 4) TMEM_LD_32((v[(c + 1) & 1]), tcol + c0 + 32);
        if ((c & 1) == 0) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the store that used the tile has read it
            __syncwarp();
        }
        uint32_t(&cur)[32] = v[c & 1];
#pragma unroll
        for (uint32_t q = 0; q < 2; q++) {
            const uint32_t col = n0 + c0 + q * 16;
            float x[16];
#pragma unroll
            for (int j = 0; j < 16; j++) x[j] = __uint_as_float(cur[q * 16 + j]);
            if (p.bias && col < p.N) {      // N is a multiple of 16: a group of 16 is inside or outside as a whole
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float4 bb = __ldg((const float4 *)(p.bias + col) + j);
                    x[4 * j] += bb.x; x[4 * j + 1] += bb.y; x[4 * j + 2] += bb.z; x[4 * j + 3] += bb.w;
                }
            }
            if (p.act == 1) {
#pragma unroll
                for (int j = 0; j < 16; j++) x[j] = gelu_ref(x[j]);
            }
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; j++) w[j] = pack2(x[2 * j], x[2 * j + 1], p.is_bf16);
            const uint32_t ch = ((c & 1) * 32 + q * 16) >> 3;     // 16-byte chunk of the 128-byte row
            *(uint4 *)(srow + ((ch ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            *(uint4 *)(srow + (((ch + 1) ^ (lane & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
        }
        if (c & 1) {
            fence_proxy_async();
            __syncwarp();
            const uint32_t col0 = n0 + (c0 - 32);
            if (lane == 0 && col0 < p.N && row0 < p.M) {      // rows and columns of the box beyond the tensor are not written
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                             ::"l"((uint64_t)omap), "r"(smem_u32(stage)), "r"((int32_t)col0), "r"((int32_t)row0) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
    }
}

template <int MT>
__global__ void __launch_bounds__(320, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, const GParams p)
{
    constexpr int kGStages = GCfg<MT>::stages, kBufs = GCfg<MT>::acc_bufs;
    constexpr uint32_t kGStageBytes = GCfg<MT>::stage_bytes, kBBase = MT * kGABytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *tiles = smem;                                   // stage s: A (16 KB) then B (32 KB)
    GShared *st = (GShared *)(tiles + kGStages * kGStageBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile uint32_t *abort_flag = &st->abort_flag;
    const uint32_t fmt = p.is_bf16 ? 1u : 0u;
    const uint32_t n_tiles = p.tiles_m * p.tiles_n;
    const uint32_t kblocks = (p.K + kGBK - 1) / kGBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGStages; s++) { mbar_init(&st->full[s], 1); mbar_init(&st->empty[s], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&st->acc_full[s], 1); mbar_init(&st->acc_empty[s], 256); }
        mbar_init(&st->drained, 1);
        st->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&st->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = st->tmem_base;
    grid_dependency_wait();        // set-up done; x (and a w or bias written on the device) come from kernels before this one
    grid_launch_dependents();

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            uint32_t g = 0;   // k-blocks loaded so far (ring position)
            for (uint32_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
                const int32_t m0 = (int32_t)((t % p.tiles_m) * (MT * kGBM)), n0 = (int32_t)((t / p.tiles_m) * kGBN);
                bool alive = true;
                for (uint32_t kb = 0; kb < kblocks; kb++, g++) {
                    const uint32_t s = g % kGStages;
                    if (g >= kGStages && !mbar_wait(&st->empty[s], ((g / kGStages) - 1) & 1, abort_flag, 41)) { alive = false; break; }
                    const uint32_t base = smem_u32(tiles + s * kGStageBytes);
                    mbar_expect_tx(&st->full[s], kGStageBytes);   // boxes beyond the tensor arrive as zeros and still count
#pragma unroll
                    for (uint32_t mt = 0; mt < MT; mt++)
                        tma_load_2d(base + mt * kGABytes, &amap, &st->full[s], (int32_t)(kb * kGBK), m0 + (int32_t)(mt * kGBM));
                    if (p.w_transposed) {
                        // 256 rows of w, 64 of k: one box
                        tma_load_2d(base + kBBase, &bmap, &st->full[s], (int32_t)(kb * kGBK), n0);
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < 4; j++)
                            tma_load_2d(base + kBBase + j * kTileBytes, &bmap, &st->full[s], n0 + (int32_t)(j * 64), (int32_t)(kb * kGBK));
                    }
                }
                if (!alive) break;
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            const uint32_t idesc = instr_desc(fmt, fmt, kGBM, kGBN, p.w_transposed ? 0 : 1);
            const uint32_t b_step = p.w_transposed ? 2u : 128u;   // descriptor units of 16 bytes per 16 of K
            uint32_t g = 0, i = 0;
            for (uint32_t t = blockIdx.x; t < n_tiles; t += gridDim.x, i++) {
                const uint32_t buf = i % kBufs;
                bool alive = true;
                if (i >= (uint32_t)kBufs && !mbar_wait(&st->acc_empty[buf], ((i / kBufs) - 1) & 1, abort_flag, 42)) break;
                tcgen05_fence_after();
                for (uint32_t kb = 0; kb < kblocks; kb++, g++) {
                    const uint32_t s = g % kGStages;
                    if (!mbar_wait(&st->full[s], (g / kGStages) & 1, abort_flag, 43)) { alive = false; break; }
                    tcgen05_fence_after();
                    const uint32_t base = smem_u32(tiles + s * kGStageBytes);
                    // MN-major: the next 64 columns are one box further on; K-major: 256 rows of 128 bytes
                    const uint64_t b_desc = p.w_transposed ? smem_desc_sw128(base + kBBase) : smem_desc_sw128(base + kBBase, kTileBytes);
#pragma unroll
                    for (uint32_t mt = 0; mt < MT; mt++) {
                        const uint64_t a_desc = smem_desc_sw128(base + mt * kGABytes);
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; kk++)   // 16 of K per MMA: +32 bytes in A's swizzled rows, +16 rows (2048 bytes) in B
                            umma_f16(tmem + (buf * MT + mt) * kGBN, a_desc + 2 * kk, b_desc + b_step * kk, idesc, (kb | kk) ? 1u : 0u);
                    }
                    umma_commit(&st->empty[s]);
                }
                if (!alive) break;
                umma_commit(&st->acc_full[buf]);
            }
        }
    } else {
        // ===== epilogue: eight warps; a thread takes one output row and half of the tile's 256 columns, 32 at a time =====
        const uint32_t quarter = warp & 3;                 // TMEM lanes this warp may touch
        const uint32_t chalf = (warp - 2) >> 2;            // which 128 columns
        const uint32_t r = quarter * 32 + lane;
        const uint32_t lane_field = (quarter * 32) << 16;
        uint32_t i = 0;
        for (uint32_t t = blockIdx.x; t < n_tiles; t += gridDim.x, i++) {
            const uint32_t buf = i % kBufs;
            const uint32_t n0 = (t / p.tiles_m) * kGBN + chalf * 128;
            if (!mbar_wait_warp(&st->acc_full[buf], (i / kBufs) & 1, abort_flag, 44)) break;
            tcgen05_fence_after();
#pragma unroll 1
            for (uint32_t mt = 0; mt < MT; mt++) {
            const uint32_t m0 = (t % p.tiles_m) * (MT * kGBM) + mt * kGBM;
            drain_rows(p, tmem + (buf * MT + mt) * kGBN + chalf * 128 + lane_field, m0 + r, n0);
            }
            tcgen05_fence_before();
            mbar_arrive(&st->acc_empty[buf]);
        }
    }

    // ---- teardown (also the way out after a timeout) ----
    tcgen05_fence_before();
    __syncthreads();
    if (st->abort_flag) {
        if (warp == 1 && lane == 0) {
            umma_commit(&st->drained);
            for (uint32_t k = 0; k < kWaitLimit && !mbar_try_wait(&st->drained, 0); k++) {}
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---- the same product on CTA pairs ------------------------------------------------------------------------
// With one CTA per tile the kernel above is bound by shared-memory bandwidth: an M128 N256 K16 MMA reads 4 KB of A and
// 8 KB of B from shared memory in its 128 cycles while the TMA writes the next stage at the same rate -- more than
// the 128 bytes per clock an SM's shared memory moves, which is where its 61 % tensor-pipe activity comes from.
// Here the two CTAs of a cluster (the two SMs of a TPC) share a 256 x 256 tile: each loads its own 128 rows of x and
// only HALF of the w tile (128 of the 256 columns), and one thread of the even CTA issues tcgen05.mma.cta_group::2
// (M 256), which reads A and its half of B from each CTA's own shared memory and writes each CTA's 128 rows of the
// accumulator into that CTA's TMEM.  Per CTA and MMA: 4 KB + 4 KB read, and stages of 32 KB instead of 48.
//   * Both producers signal the even CTA's `full` barrier (it expects the bytes of both); the commit after a stage's
//     MMAs arrives on the `empty` barrier of both CTAs, the commit after a tile on both `acc_full` barriers.
//   * Each CTA drains its own 128 rows (through per-warp staging tiles and TMA stores); its epilogue warps arrive on
//     the even CTA's `acc_empty` barrier.
//   * No load is a multicast: each CTA fetches what it multiplies.
#ifndef SFB_GEMM_PAIRS
#define SFB_GEMM_PAIRS 1
#endif
constexpr bool kUsePairs = SFB_GEMM_PAIRS != 0;
#ifndef SFB_GEMM_BAND
#define SFB_GEMM_BAND 8
#endif
constexpr uint32_t kPBand = SFB_GEMM_BAND;
constexpr uint32_t kPStages = 6;
constexpr uint32_t kPStagingBytes = 8 * 32 * 128;     // one 32-row x 64-column tile per epilogue warp
constexpr uint32_t kPABytes = kGBM * kGBK * 2;            // 16 KB: this CTA's 128 rows of x
constexpr uint32_t kPBBytes = kGBK * (kGBN / 2) * 2;      // 16 KB: this CTA's 128 columns of w
constexpr uint32_t kPStageBytes = kPABytes + kPBBytes;
constexpr size_t kPSmem = 1024 + kPStages * kPStageBytes + kPStagingBytes + 256;

struct PShared {
    uint64_t full[kPStages], empty[kPStages], acc_full[2], acc_empty[2], drained;
    uint32_t tmem_base, abort_flag;
};
static_assert(sizeof(PShared) <= 256, "PShared outgrew its slot");

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of this CTA's shared-memory address `addr` in CTA `rank`
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t rank)
{
    uint32_t d;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(d) : "r"(addr), "r"(rank));
    return d;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// a tile into this CTA's shared memory, its bytes counted on a barrier that may live in the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster_addr, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar)
{
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"(both)
                 : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
linear_tc_pair_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
                      const __grid_constant__ CUtensorMap omap, const GParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *tiles = smem;                                   // stage s: A (16 KB) then this CTA's half of B (16 KB)
    uint8_t *staging = tiles + kPStages * kPStageBytes;      // the epilogue warps' output tiles (4 KB each)
    PShared *st = (PShared *)(staging + kPStagingBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0: issues the MMAs of the pair
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    volatile uint32_t *abort_flag = &st->abort_flag;
    const uint32_t fmt = p.is_bf16 ? 1u : 0u;
    const uint32_t n_tiles = p.tiles_m * p.tiles_n;          // tiles of 256 x 256
    const uint32_t kblocks = (p.K + kGBK - 1) / kGBK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kPStages; s++) { mbar_init(&st->full[s], 1); mbar_init(&st->empty[s], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&st->acc_full[s], 1); mbar_init(&st->acc_empty[s], 16); }   // 8 epilogue warps of each CTA
        mbar_init(&st->drained, 1);
        st->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&st->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                      // both CTAs' barriers exist before anything signals across
    tcgen05_fence_after();
    const uint32_t tmem = st->tmem_base;
    grid_dependency_wait();        // set-up done; nothing of global memory has been read yet
    grid_launch_dependents();

    if (warp == 0) {
        // ===== TMA producer (both CTAs): own rows of x, own half of the w tile; bytes counted on the even CTA's barrier =====
        if (lane == 0) {
            uint32_t g = 0;
            for (uint32_t t = pair; t < n_tiles; t += pairs) {
                uint32_t tm, tn;
                tile_coords(p, t, tm, tn);
                const int32_t m0 = (int32_t)(tm * 256 + rank * kGBM);
                const int32_t n0 = (int32_t)(tn * kGBN + rank * (kGBN / 2));
                bool alive = true;
                for (uint32_t kb = 0; kb < kblocks; kb++, g++) {
                    const uint32_t s = g % kPStages;
                    if (g >= kPStages && !mbar_wait(&st->empty[s], ((g / kPStages) - 1) & 1, abort_flag, 51)) { alive = false; break; }
                    const uint32_t base = smem_u32(tiles + s * kPStageBytes);
                    const uint32_t bar = mapa_rank(smem_u32(&st->full[s]), 0);
                    if (rank == 0) mbar_expect_tx(&st->full[s], 2 * kPStageBytes);   // both CTAs' bytes; boxes beyond the tensor arrive as zeros and still count
                    tma_load_2d_pair(base, &amap, bar, (int32_t)(kb * kGBK), m0);
                    if (p.w_transposed) {
                        tma_load_2d_pair(base + kPABytes, &bmap, bar, (int32_t)(kb * kGBK), n0);      // 128 rows of w, 64 of k
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < 2; j++)
                            tma_load_2d_pair(base + kPABytes + j * kTileBytes, &bmap, bar, n0 + (int32_t)(j * 64), (int32_t)(kb * kGBK));
                    }
                }
                if (!alive) break;
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: one thread of the even CTA for the pair =====
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc(fmt, fmt, 256, kGBN, p.w_transposed ? 0 : 1);
            const uint32_t b_step = p.w_transposed ? 2u : 128u;
            uint32_t g = 0, i = 0;
            for (uint32_t t = pair; t < n_tiles; t += pairs, i++) {
                const uint32_t buf = i & 1;
                bool alive = true;
                if (i >= 2 && !mbar_wait(&st->acc_empty[buf], ((i >> 1) - 1) & 1, abort_flag, 52)) break;
                tcgen05_fence_after();
                for (uint32_t kb = 0; kb < kblocks; kb++, g++) {
                    const uint32_t s = g % kPStages;
                    if (!mbar_wait(&st->full[s], (g / kPStages) & 1, abort_flag, 53)) { alive = false; break; }
                    tcgen05_fence_after();
                    const uint32_t base = smem_u32(tiles + s * kPStageBytes);
                    const uint64_t a_desc = smem_desc_sw128(base);
                    const uint64_t b_desc = p.w_transposed ? smem_desc_sw128(base + kPABytes) : smem_desc_sw128(base + kPABytes, kTileBytes);
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; kk++)
                        umma_f16_pair(tmem + buf * kGBN, a_desc + 2 * kk, b_desc + b_step * kk, idesc, (kb | kk) ? 1u : 0u);
                    umma_commit_pair(&st->empty[s]);
                }
                if (!alive) break;
                umma_commit_pair(&st->acc_full[buf]);
            }
        }
    } else {
        // ===== epilogue (both CTAs): this CTA's 128 rows of the tile; a warp takes 32 rows and 128 columns and stores them
        // through its own staging tile =====
        const uint32_t quarter = warp & 3;
        const uint32_t chalf = (warp - 2) >> 2;
        const uint32_t lane_field = (quarter * 32) << 16;
        const uint32_t acc_empty0[2] = {mapa_rank(smem_u32(&st->acc_empty[0]), 0), mapa_rank(smem_u32(&st->acc_empty[1]), 0)};
        uint32_t i = 0;
        for (uint32_t t = pair; t < n_tiles; t += pairs, i++) {
            const uint32_t buf = i & 1;
            uint32_t tm, tn;
            tile_coords(p, t, tm, tn);
            const uint32_t n0 = tn * kGBN + chalf * 128;
            const uint32_t m0 = tm * 256 + rank * kGBM;
            if (!mbar_wait_warp(&st->acc_full[buf], (i >> 1) & 1, abort_flag, 54)) break;
            tcgen05_fence_after();
            drain_rows_staged(p, &omap, tmem + buf * kGBN + chalf * 128 + lane_field, staging + (warp - 2) * 4096, m0 + quarter * 32, n0, lane);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(buf ? acc_empty0[1] : acc_empty0[0]);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the last tile has left shared memory
    }

    // ---- teardown (also the way out after a timeout) ----
    tcgen05_fence_before();
    __syncthreads();
    if (st->abort_flag) {
        if (warp == 1 && lane == 0 && rank == 0) {
            asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&st->drained)) : "memory");
            for (uint32_t k = 0; k < kWaitLimit && !mbar_try_wait(&st->drained, 0); k++) {}
        }
        if (warp == 0 && lane == 0) {
            const uint64_t t0 = clock64();
            while (clock64() - t0 < 2000000ull) {}
        }
        __syncthreads();
    }
    cluster_sync_all();      // neither CTA leaves, nor frees its TMEM, while the other may still read its shared memory or signal it
    if (warp == 0) {
        __syncwarp();
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// [rows, cols] 16-bit row-major tensor, boxes of box_rows x 64 elements, 128-byte swizzle
static int make_map_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, int is_bf16, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

}  // namespace tc

int tc_linear(cudaStream_t s, void *out, const void *x, const void *w, const float *bias, uint32_t m, uint32_t n, uint32_t k,
              int dtype, int act, bool w_transposed)
{
    using namespace tc;
    const int is_bf16 = dtype == SFB_BF16;
    CUtensorMap am, bm;
    if (make_map_2d(&am, x, m, k, is_bf16, kGBM)) return 1;
    if (w_transposed ? make_map_2d(&bm, w, n, k, is_bf16, kGBN) : make_map_2d(&bm, w, k, n, is_bf16, kGBK)) return 1;
    static DeviceOnce once;
    const int dev = current_device();
    const int sms = device_sm_count(dev);
    if (sms <= 0) return fail("sfb_linear: cannot read the SM count");
    if (!once.done(dev)) {
        if (cudaFuncSetAttribute(linear_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GCfg<1>::smem) != cudaSuccess ||
            cudaFuncSetAttribute(linear_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GCfg<2>::smem) != cudaSuccess)
            return fail("sfb_linear: cannot reserve %zu bytes of shared memory", GCfg<1>::smem);
        once.mark(dev);
    }
    const uint32_t tiles_n = (n + kGBN - 1) / kGBN;
    // CTA pairs on 256 x 256 tiles whenever there is at least one tile per pair of SMs
    const uint32_t pair_tiles = ((m + 255) / 256) * tiles_n;
    if (kUsePairs && sms >= 2 && pair_tiles >= (uint32_t)(sms / 2)) {
        CUtensorMap bp;
        if (w_transposed ? make_map_2d(&bp, w, n, k, is_bf16, kGBN / 2) : make_map_2d(&bp, w, k, n, is_bf16, kGBK)) return 1;
        static DeviceOnce once_pair;
        if (!once_pair.done(dev)) {
            if (cudaFuncSetAttribute(linear_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPSmem) != cudaSuccess)
                return fail("sfb_linear: cannot reserve %zu bytes of shared memory", kPSmem);
            once_pair.mark(dev);
        }
        CUtensorMap om;      // out as [m, n], boxes of 32 rows x 64 columns for the epilogue's stores
        if (make_map_2d(&om, out, m, n, is_bf16, 32)) return 1;
        GParams prm = {out, bias, m, n, k, (m + 255) / 256, tiles_n, is_bf16, act, w_transposed ? 1 : 0, tiles_n < kPBand ? tiles_n : kPBand};
        const uint32_t pairs = pair_tiles < (uint32_t)(sms / 2) ? pair_tiles : (uint32_t)(sms / 2);
        launch_overlapped(linear_tc_pair_kernel, dim3(2 * pairs), dim3(320), kPSmem, s, am, bp, om, prm);
        // a device or a partition that cannot place the clusters refuses the launch: the single-CTA kernel takes over
        if (cudaGetLastError() == cudaSuccess) { clear_error(); return 0; }
    }
    // long-k products are bound by what travels from L2: 256-row tiles, as long as they still fill the SMs twice over
    const int mt = (k >= 2048 && (uint64_t)((m + 255) / 256) * tiles_n >= 2ull * sms) ? 2 : 1;
    GParams prm = {out, bias, m, n, k, (m + mt * kGBM - 1) / (mt * kGBM), tiles_n, is_bf16, act, w_transposed ? 1 : 0, 1};
    const uint32_t tiles = prm.tiles_m * prm.tiles_n;
    const uint32_t grid = tiles < (uint32_t)sms ? tiles : (uint32_t)sms;
    if (mt == 2) launch_overlapped(linear_tc_kernel<2>, dim3(grid), dim3(320), GCfg<2>::smem, s, am, bm, prm);
    else launch_overlapped(linear_tc_kernel<1>, dim3(grid), dim3(320), GCfg<1>::smem, s, am, bm, prm);
    return check_launch("sfb_linear");
}

int tc_status_clear_gemm()
{
    const uint32_t zero = 0;
    cudaError_t e = cudaMemcpyToSymbol(tc::g_status, &zero, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status_clear: %s", cudaGetErrorString(e));
    return 0;
}

int tc_status_gemm(uint32_t *out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, tc::g_status, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace sfb
