// The unfused operators on the tensor cores (tcgen05) for 16-bit operands, block_size 64, head size 64:
//   sddmm_tc_kernel   S(block) = Q_i . K_j^T for every kept block          (bst_sgemm_nt,  blocksparse.h:425)
//   spmm_tc_kernel    O_i = sum over the row's blocks of P(block) . V_j     (bst_sgemm_xn,  blocksparse.h:965)
// Same tiling as the fused kernel: a CTA owns a pair of adjacent block-rows (128 queries, one M=128 MMA
// tile) and walks the union of their key blocks; operands arrive by TMA into 128-byte-swizzled shared
// memory, accumulators live in TMEM.  Both operators are HBM-bound (8 KB of S or P per 1 MFLOP), so the
// point of the tensor cores here is to get the arithmetic out of the way of the memory system.
#include "tc_common.cuh"

namespace sfb {
namespace tc {

constexpr int kUStages = 4;

static int make_p_map(CUtensorMap *map, const void *base, uint64_t rows, int is_bf16);

struct UShared {
    uint64_t q_full, in_full[kUStages], in_empty[kUStages], s_full[2], s_empty[2], o_final, drained;
    uint32_t tmem_base, n_union, abort_flag, pad;
    UnionEntry entries[kMaxUnion];
    uint2 cand[kMaxUnion];
};

struct UParams {
    const uint2 *nn_lut;
    void *out;                 // S blocks (sddmm) or O (spmm)
    uint32_t B, H, nb, blocks, lut_stride;
    int out_dtype;             // SFB_F32 / SFB_BF16 / SFB_F16
    int is_bf16;               // operand format
    uint32_t p_rows;           // spmm: rows of the 2-D view of P (= B*H*blocks*64); a coordinate beyond it reads zeros
    int trans;                 // spmm: 1 = the blocks are used transposed and the LUT walks block columns (TN_OP)
    const float *delta;        // sddmm, gradient mode: [B, L, H] row sums of dO * O
    float scale;               // sddmm, gradient mode
};

constexpr int kSdStagesMax = 5;                 // key stages: five without the P tile, four with it (shared memory per CTA)
constexpr uint32_t kChunk = 32;                 // consecutive LUT entries one CTA takes
struct SdShared {
    uint64_t in_full[kSdStagesMax], in_empty[kSdStagesMax], s_full[2], s_empty[2], drained, q_full[2], q_empty[2];
    uint32_t tmem_base, abort_flag;
    uint2 ent[kChunk];                          // this CTA's LUT entries
};
// two query-row tiles (kept while consecutive blocks share their block-row), the key stages, two output staging tiles
constexpr size_t kSddmmSmem = 1024 + 2 * kTileBytes + 5 * 1 * kTileBytes + 2 * kTileBytes + sizeof(SdShared);
constexpr size_t kSddmmGradSmem = 1024 + 2 * kTileBytes + 4 * 2 * kTileBytes + 2 * kTileBytes + sizeof(SdShared);
constexpr size_t kSpmmSmem = 1024 + kUStages * (kQBytes + kTileBytes) + sizeof(UShared);

__device__ __forceinline__ void store_row16(void *dst_base, size_t elem_off, const uint32_t (&v)[16], int out_dtype, int c0)
{
    // 16 consecutive fp32 accumulator values of one row -> the output type
    if (out_dtype == SFB_F32) {
        float4 *d = (float4 *)((float *)dst_base + elem_off + c0);
#pragma unroll
        for (int j = 0; j < 4; j++)
            d[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                               __uint_as_float(v[4 * j + 3]));
    } else {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; j++) w[j] = pack2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]), out_dtype == SFB_BF16);
        // one 32-byte store: a whole sector per thread
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"((uint16_t *)dst_base + elem_off + c0), "r"(w[0]),
                     "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                     : "memory");
    }
}

// ---- SDDMM ----------------------------------------------------------------------------------------
// The operator only receives the nt_lut (one (row, column) pair per kept block, in any order), so a CTA takes
// a run of kChunk consecutive blocks.  The 64 query rows sit in one of two tiles that are loaded only when the
// block-row changes (the LUT is in row-major scan order, so a run shares its rows: without this every block pulled
// 16 KB through L2 for the 8 KB it writes); per block a stage holds the 64 key rows.  The M=128 MMA reads the query
// tile and whatever follows it as its A operand, so accumulator lanes 0-63 hold Q.K^T and lanes 64-127 a by-product
// that is never read -- the operator is bound by the bytes it moves, not by tensor work.  warp 0: TMA; warp 1: MMA; warps 4-5 and 8-9: TMEM lanes 0-63 -> global, half a score row (32
// columns) per thread.
//
// GRAD: the same kernel as the first half of a fused backward.  With a = dO and b = V the accumulator is dP = dO.V^T;
// a third tile per stage brings the block of P, and the drain writes dS = P * (dP - delta) * scale, where
// delta[row] = sum over the head of dO * O.  That row constant equals the sum over the row's blocks of dP * P which the
// unfused softmax gradient has to reduce first, so dS needs no pass over the row and dP never reaches memory.
template <bool GRAD>
__global__ void __launch_bounds__(320, GRAD ? 2 : 4)
sddmm_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                const __grid_constant__ CUtensorMap omap, const __grid_constant__ CUtensorMap pmap, const UParams p)
{
    constexpr uint32_t kStage = (GRAD ? 2 : 1) * kTileBytes;
    constexpr uint32_t kSdStages = GRAD ? 4 : 5;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *q_tiles = smem;                                 // two tiles of query rows
    uint8_t *tiles = q_tiles + 2 * kTileBytes;               // stage s: K rows (8 KB), GRAD: the block of P (8 KB)
    uint8_t *stage_out = tiles + kSdStages * kStage;         // two 8 KB tiles of 16-bit scores on their way out
    SdShared *st = (SdShared *)(stage_out + 2 * kTileBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b = blockIdx.y, h = blockIdx.z;
    const uint32_t k0 = blockIdx.x * kChunk;
    const uint32_t T = min(kChunk, p.blocks - k0);
    const uint32_t L = p.nb * 64;
    const uint2 *lut = p.nn_lut + (size_t)h * p.lut_stride + k0;   // here: the nt_lut
    volatile uint32_t *abort_flag = &st->abort_flag;
    const uint32_t fmt = p.is_bf16 ? 1u : 0u;

    if (threadIdx.x == 0) {
        // GRAD: a stage is free when the MMA has read Q and K AND the 128 drain threads have read P
        for (uint32_t s = 0; s < kSdStages; s++) { mbar_init(&st->in_full[s], 1); mbar_init(&st->in_empty[s], GRAD ? 129 : 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&st->s_full[s], 1); mbar_init(&st->s_empty[s], 128); }
        for (int s = 0; s < 2; s++) { mbar_init(&st->q_full[s], 1); mbar_init(&st->q_empty[s], 1); }
        mbar_init(&st->drained, 1);
        st->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + T) st->ent[threadIdx.x - 64] = lut[threadIdx.x - 64];
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&st->tmem_base)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = st->tmem_base;
    const int32_t xq = (int32_t)(h * 64);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t n_q = 0;                                  // query tiles requested so far
            for (uint32_t t = 0; t < T; t++) {
                const uint32_t s = t % kSdStages;
                if (t >= kSdStages && !mbar_wait(&st->in_empty[s], ((t / kSdStages) - 1) & 1, abort_flag, 21)) break;
                const uint2 ent = st->ent[t];
                if (ent.x >= p.nb || ent.y >= p.nb) {   // a LUT entry outside the block grid: report, do not fetch
                    st->abort_flag = 1;
                    atomicCAS(&g_status, 0u, (20u << 24) | (blockIdx.x & 0xffffffu));
                    break;
                }
                if (t == 0 || ent.x != st->ent[t - 1].x) {
                    // a new block-row: its query rows go into the tile the row before last used, once the MMAs that read it are done
                    const uint32_t qi = n_q & 1;
                    if (n_q >= 2 && !mbar_wait(&st->q_empty[qi], ((n_q >> 1) - 1) & 1, abort_flag, 27)) break;
                    mbar_expect_tx(&st->q_full[qi], kTileBytes);
                    tma_load_2d(smem_u32(q_tiles + qi * kTileBytes), &qmap, &st->q_full[qi], xq, (int32_t)(b * L + ent.x * 64));
                    n_q++;
                }
                mbar_expect_tx(&st->in_full[s], kStage);
                tma_load_2d(smem_u32(tiles + s * kStage), &kmap, &st->in_full[s], xq, (int32_t)(b * L + ent.y * 64));
                if (GRAD)
                    tma_load_2d(smem_u32(tiles + s * kStage + kTileBytes), &pmap, &st->in_full[s], 0,
                                (int32_t)((((size_t)b * p.H + h) * p.blocks + k0 + t) * 64));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(fmt, fmt, 128, 64, 0);
            uint32_t n_q = 0, qi = 0;
            for (uint32_t t = 0; t < T; t++) {
                const uint32_t s = t % kSdStages;
                const uint32_t row = st->ent[t].x;
                if (t == 0 || row != st->ent[t - 1].x) {
                    qi = n_q & 1;
                    if (!mbar_wait(&st->q_full[qi], (n_q >> 1) & 1, abort_flag, 28)) break;
                    n_q++;
                }
                if (!mbar_wait(&st->in_full[s], (t / kSdStages) & 1, abort_flag, 23)) break;
                if (t >= 2 && !mbar_wait(&st->s_empty[t & 1], ((t >> 1) - 1) & 1, abort_flag, 24)) break;
                tcgen05_fence_after();
                const uint64_t a_desc = smem_desc_sw128(smem_u32(q_tiles + qi * kTileBytes));
                const uint64_t b_desc = smem_desc_sw128(smem_u32(tiles + s * kStage));
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++) umma_f16(tmem + 64 * (t & 1), a_desc + 2 * kk, b_desc + 2 * kk, idesc, kk);
                umma_commit(&st->s_full[t & 1]);
                umma_commit(&st->in_empty[s]);
                if (t + 1 == T || st->ent[t + 1].x != row) umma_commit(&st->q_empty[qi]);   // last block of this block-row
            }
        }
    } else if (warp == 4 || warp == 5 || warp == 8 || warp == 9) {
        const uint32_t quarter = warp & 3;                 // 0 and 1: TMEM lanes 0-63
        const int cbase = warp >= 8 ? 32 : 0;              // which half of the 64 columns
        const uint32_t r = quarter * 32 + lane;
        const uint32_t lane_field = (quarter * 32) << 16;
        for (uint32_t t = 0; t < T; t++) {
            // the four drain warps leave together or not at all: they meet at named barriers below
            const bool ok = mbar_wait_warp(&st->s_full[t & 1], (t >> 1) & 1, abort_flag, 25);
            uint32_t all_ok;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.red.and.pred p, 2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
            if (!all_ok) break;
            tcgen05_fence_after();
            const size_t off = ((((size_t)b * p.H + h) * p.blocks + k0 + t) * 64 + r) * 64;
            if (p.out_dtype == SFB_F32) {
#pragma unroll
                for (int c0 = cbase; c0 < cbase + 32; c0 += 16) {
                    uint32_t v[16];
                    TMEM_LD_16((v), tmem + 64 * (t & 1) + lane_field + c0);
                    tmem_wait_ld();
                    store_row16(p.out, off, v, p.out_dtype, c0);
                }
            } else {
                // 16-bit scores leave through shared memory and one TMA store per tile: rows of 128 bytes, 16-byte
                // chunk c of row r at chunk c ^ (r % 8) (the tensor map's 128-byte swizzle)
                const bool leader = warp == 4 && lane == 0;
                if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the store that used this buffer has read it
                asm volatile("bar.sync 4, 128;" ::: "memory");
                uint8_t *orow = stage_out + (t & 1) * kTileBytes + r * 128;
                const uint32_t sg = t % kSdStages;
                const uint8_t *prow = tiles + sg * kStage + kTileBytes + r * 128;
                float dl = 0.f;
                bool p_ok = true;
                if (GRAD) {
                    // P arrived with the same transaction barrier the MMA waited for; observing it here makes the tile visible
                    p_ok = mbar_wait_warp(&st->in_full[sg], (t / kSdStages) & 1, abort_flag, 26);
                    dl = __ldg(p.delta + ((size_t)b * L + (size_t)st->ent[t].x * 64 + r) * p.H + h);
                }
#pragma unroll
                for (int c0 = cbase; c0 < cbase + 32; c0 += 16) {
                    uint32_t v[16], w[8];
                    TMEM_LD_16((v), tmem + 64 * (t & 1) + lane_field + c0);
                    tmem_wait_ld();
                    if (GRAD) {
                        const uint32_t chp = c0 >> 3;
                        const uint4 pa = *(const uint4 *)(prow + ((chp ^ (r & 7)) << 4)), pb = *(const uint4 *)(prow + (((chp + 1) ^ (r & 7)) << 4));
                        const uint32_t pw[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            float p0, p1;
                            if (p.out_dtype == SFB_BF16) {
                                p0 = __uint_as_float(pw[j] << 16);
                                p1 = __uint_as_float(pw[j] & 0xffff0000u);
                            } else {
                                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&pw[j]));
                                p0 = f.x;
                                p1 = f.y;
                            }
                            v[2 * j] = __float_as_uint(p_ok ? p0 * (__uint_as_float(v[2 * j]) - dl) * p.scale : 0.f);
                            v[2 * j + 1] = __float_as_uint(p_ok ? p1 * (__uint_as_float(v[2 * j + 1]) - dl) * p.scale : 0.f);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++) w[j] = pack2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]), p.out_dtype == SFB_BF16);
                    const uint32_t ch = c0 >> 3;
                    *(uint4 *)(orow + ((ch ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *(uint4 *)(orow + (((ch + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
                }
                fence_proxy_async();
                asm volatile("bar.sync 3, 128;" ::: "memory");
                if (leader) {
                    const int32_t y = (int32_t)((((size_t)b * p.H + h) * p.blocks + k0 + t) * 64);
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                 ::"l"((uint64_t)&omap), "r"(smem_u32(stage_out + (t & 1) * kTileBytes)), "r"(0), "r"(y) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                if (GRAD) mbar_arrive(&st->in_empty[sg]);   // this thread is done with the stage's P tile
            }
            tcgen05_fence_before();
            mbar_arrive(&st->s_empty[t & 1]);
        }
        // shared memory must outlive the stores that read it
        if (warp == 4 && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }

    tcgen05_fence_before();
    __syncthreads();
    if (st->abort_flag) {
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

// ---- SpMM -----------------------------------------------------------------------------------------
// warp 0: TMA (per key block: the two 64-row halves of the P tile -- a half whose block-row does not keep the
// block is fetched from beyond the tensor and arrives as zeros -- and the V tile); warp 1: MMA; warps 2-5: epilogue.
// With p.trans the same kernel does the backward products C = A^T . B: the CTA owns two block COLUMNS, the LUT is
// the tn_lut, and the two blocks of a step are read as ONE MN-major A operand (M = the 2 x 64 key positions,
// contiguous inside a shared-memory row; K = the 64 query rows, 2048 bytes per 16) instead of a K-major one.
__global__ void __launch_bounds__(192, 2)
spmm_tc_kernel(const __grid_constant__ CUtensorMap pmap, const __grid_constant__ CUtensorMap vmap, const UParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *tiles = smem;                                   // stage s: P (16 KB) then V (8 KB)
    constexpr uint32_t kStageBytes = kQBytes + kTileBytes;
    UShared *st = (UShared *)(tiles + kUStages * kStageBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t pair = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const bool has_row1 = pair * 2 + 1 < p.nb;
    const uint32_t L = p.nb * 64;
    const uint2 *nn = p.nn_lut + (size_t)h * p.lut_stride;
    volatile uint32_t *abort_flag = &st->abort_flag;
    const uint32_t fmt = p.is_bf16 ? 1u : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kUStages; s++) { mbar_init(&st->in_full[s], 1); mbar_init(&st->in_empty[s], 1); }
        mbar_init(&st->o_final, 1);
        mbar_init(&st->drained, 1);
        st->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    build_union(nn, pair, p.nb, st->entries, st->cand, &st->n_union, &st->abort_flag);
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&st->tmem_base)), "r"(64u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();

    const uint32_t T = st->n_union;
    const uint32_t tmem = st->tmem_base;

    if (warp == 0) {
        if (lane == 0 && T > 0) {
            const uint32_t bh_rows = ((b * p.H + h) * p.blocks) * 64;    // first row of this (b,h) in the 2-D view of P
            for (uint32_t t = 0; t < T; t++) {
                const uint32_t s = t % kUStages;
                if (t >= kUStages && !mbar_wait(&st->in_empty[s], ((t / kUStages) - 1) & 1, abort_flag, 31)) break;
                const UnionEntry ent = st->entries[t];
                uint8_t *ptile = tiles + s * kStageBytes;
                mbar_expect_tx(&st->in_full[s], kStageBytes);
                const int32_t y0 = (ent.flags & 1) ? (int32_t)(bh_rows + ent.blk[0] * 64) : (int32_t)p.p_rows;
                const int32_t y1 = (ent.flags & 2) ? (int32_t)(bh_rows + ent.blk[1] * 64) : (int32_t)p.p_rows;
                tma_load_2d(smem_u32(ptile), &pmap, &st->in_full[s], 0, y0);
                tma_load_2d(smem_u32(ptile + kTileBytes), &pmap, &st->in_full[s], 0, y1);
                tma_load_2d(smem_u32(ptile + kQBytes), &vmap, &st->in_full[s], (int32_t)(h * 64), (int32_t)(b * L + ent.col * 64));
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && T > 0) {
            const uint32_t idesc = instr_desc(fmt, fmt, 128, 64, 1) | (p.trans ? 1u << 15 : 0u);   // bit 15: A is MN-major
            const uint32_t a_step = p.trans ? 128u : 2u;   // descriptor units of 16 bytes per 16 of K
            for (uint32_t t = 0; t < T; t++) {
                const uint32_t s = t % kUStages;
                if (!mbar_wait(&st->in_full[s], (t / kUStages) & 1, abort_flag, 33)) break;
                tcgen05_fence_after();
                const uint32_t p_addr = smem_u32(tiles + s * kStageBytes);
                // transposed: the second block is the next group of 64 along M, one tile further on
                const uint64_t p_desc = p.trans ? smem_desc_sw128(p_addr, kTileBytes) : smem_desc_sw128(p_addr);
                const uint64_t v_desc = smem_desc_sw128(smem_u32(tiles + s * kStageBytes + kQBytes));
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++) umma_f16(tmem, p_desc + a_step * kk, v_desc + 128 * kk, idesc, (t | kk) ? 1u : 0u);
                umma_commit(&st->in_empty[s]);
                if (t + 1 == T) umma_commit(&st->o_final);
            }
        }
    } else {
        const uint32_t quarter = warp & 3;
        const uint32_t r = quarter * 32 + lane;
        const uint32_t lane_field = (quarter * 32) << 16;
        const bool row_valid = (r >> 6) == 0 || has_row1;
        bool alive = true;
        if (T > 0) alive = mbar_wait_warp(&st->o_final, 0, abort_flag, 35);
        if (alive) {
            tcgen05_fence_after();
            const size_t off = ((size_t)b * L + (size_t)pair * 128 + r) * ((size_t)p.H * 64) + (size_t)h * 64;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t v[16];
                if (T > 0) {
                    TMEM_LD_16((v), tmem + lane_field + c0);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = 0u;    // rows without blocks are written as zeros (blocksparse.h:949-962)
                }
                if (row_valid) store_row16(p.out, off, v, p.out_dtype, c0);
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (st->abort_flag) {
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64u) : "memory");
    }
}

// ---- fused SDDMM + softmax, probabilities out ----------------------------------------------------------
// Row-pair tiling as the three-stage kernel.  The row's scores are produced twice by the tensor core instead of
// making a round trip through memory: sweep 1 over the row pair's key blocks keeps the running row max and sum,
// sweep 2 recomputes S and writes exp2(s*c - max) / sum.  warp 0: TMA (Q once, the K tiles twice); warp 1: MMA;
// warps 2-9: two threads per query row, 32 score columns each.  The two threads of a row keep their own running
// (max, sum) through sweep 1 and combine them once, between the sweeps, through shared memory: no exchange per step,
// and twice the warps to hide the TMEM-load -> exponentials -> store chain of a step.
struct FpParams {
    const uint2 *nn_lut;
    const uint64_t *mask;      // mask_np order, or NULL
    void *Y;
    uint32_t B, H, nb, blocks, lut_stride, mask_stride;
    float scale_log2e;
    int out_dtype, is_bf16;
};

constexpr size_t kFpSmem = 1024 + kQBytes + kUStages * kTileBytes + sizeof(UShared) + 256 * sizeof(float2);
constexpr int kFpThreads = 64 + 256;
#ifndef SFB_FP_POLY
#define SFB_FP_POLY 2
#endif
constexpr int kFpPoly = SFB_FP_POLY;        // sweep 1: every kFpPoly-th pair of exponentials on the FMA pipe (0 = none)

__global__ void __launch_bounds__(kFpThreads, 3)
fused_p_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap, const FpParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *q_tile = smem;
    uint8_t *k_tiles = q_tile + kQBytes;
    UShared *st = (UShared *)(k_tiles + kUStages * kTileBytes);
    float2 *comb = (float2 *)(st + 1);         // [column half][row]: (max, sum) after sweep 1

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t pair = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const uint32_t L = p.nb * 64;
    const uint2 *nn = p.nn_lut + (size_t)h * p.lut_stride;
    volatile uint32_t *abort_flag = &st->abort_flag;
    const uint32_t fmt = p.is_bf16 ? 1u : 0u;

    if (threadIdx.x == 0) {
        mbar_init(&st->q_full, 1);
        for (int s = 0; s < kUStages; s++) { mbar_init(&st->in_full[s], 1); mbar_init(&st->in_empty[s], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&st->s_full[s], 1); mbar_init(&st->s_empty[s], 256); }
        mbar_init(&st->o_final, 256);          // here: both halves of every row have published their (max, sum)
        mbar_init(&st->drained, 1);
        st->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    build_union(nn, pair, p.nb, st->entries, st->cand, &st->n_union, &st->abort_flag);
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&st->tmem_base)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();

    const uint32_t T = st->n_union;
    const uint32_t T2 = 2 * T;                 // every key block is visited twice
    const uint32_t tmem = st->tmem_base;
    const int32_t xq = (int32_t)(h * 64);

    if (warp == 0) {
        if (lane == 0 && T > 0) {
            mbar_expect_tx(&st->q_full, kQBytes);
            tma_load_2d(smem_u32(q_tile), &qmap, &st->q_full, xq, (int32_t)(b * L + pair * 128));
            for (uint32_t t = 0; t < T2; t++) {
                const uint32_t s = t % kUStages;
                if (t >= kUStages && !mbar_wait(&st->in_empty[s], ((t / kUStages) - 1) & 1, abort_flag, 41)) break;
                mbar_expect_tx(&st->in_full[s], kTileBytes);
                tma_load_2d(smem_u32(k_tiles + s * kTileBytes), &kmap, &st->in_full[s], xq,
                            (int32_t)(b * L + st->entries[t < T ? t : t - T].col * 64));
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && T > 0) {
            const uint32_t idesc = instr_desc(fmt, fmt, 128, 64, 0);
            const uint64_t q_desc = smem_desc_sw128(smem_u32(q_tile));
            bool alive = mbar_wait(&st->q_full, 0, abort_flag, 42);
            for (uint32_t t = 0; alive && t < T2; t++) {
                const uint32_t s = t % kUStages;
                if (!mbar_wait(&st->in_full[s], (t / kUStages) & 1, abort_flag, 43)) break;
                if (t >= 2 && !mbar_wait(&st->s_empty[t & 1], ((t >> 1) - 1) & 1, abort_flag, 44)) break;
                tcgen05_fence_after();
                const uint64_t k_desc = smem_desc_sw128(smem_u32(k_tiles + s * kTileBytes));
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++) umma_f16(tmem + 64 * (t & 1), q_desc + 2 * kk, k_desc + 2 * kk, idesc, kk);
                umma_commit(&st->s_full[t & 1]);
                umma_commit(&st->in_empty[s]);
            }
        }
    } else {
        const uint32_t quarter = warp & 3;         // the TMEM lanes a warp may read: 32 * (warp % 4)
        const uint32_t ch = (warp - 2) >> 2;       // which 32 of the 64 score columns
        const uint32_t cb = ch * 32;
        const uint32_t r = quarter * 32 + lane;
        const uint32_t half = r >> 6;
        const uint32_t lane_field = (quarter * 32) << 16;
        const float sl = p.scale_log2e;
        float m = -INFINITY, l = 0.f, inv = 0.f;
        for (uint32_t t = 0; t < T2; t++) {
            if (!mbar_wait_warp(&st->s_full[t & 1], (t >> 1) & 1, abort_flag, 45)) break;
            tcgen05_fence_after();
            uint32_t sr[32];
            TMEM_LD_32((sr), tmem + 64 * (t & 1) + lane_field + cb);
            tmem_wait_ld();
            tcgen05_fence_before();
            mbar_arrive(&st->s_empty[t & 1]);

            if (t == T) {
                // sweep 1 is over, whichever block-row owns the union's first and last entries: the row's two threads
                // merge their (max, sum).  A bounded wait on a barrier, not bar.sync: a warp that gave up never arrives.
                comb[ch * 128 + r] = make_float2(m, l);
                mbar_arrive(&st->o_final);
                if (!mbar_wait_warp(&st->o_final, 0, abort_flag, 46)) break;
                const float2 o = comb[(ch ^ 1) * 128 + r];
                const float mf = fmaxf(m, o.x);
                l = (m > -INFINITY ? l * ex2_approx(m - mf) : 0.f) + (o.x > -INFINITY ? o.y * ex2_approx(o.x - mf) : 0.f);
                m = mf;
                inv = l > 0.f ? 1.f / l : 0.f;
            }
            const UnionEntry *ent = &st->entries[t < T ? t : t - T];     // read in place: a copy indexed by `half` would live in local memory
            if (!((ent->flags >> half) & 1)) continue;
            if (p.mask) {
                const uint32_t w = (uint32_t)(p.mask[(size_t)h * p.mask_stride + (size_t)ent->blk[half] * 64 + (r & 63)] >> cb);
#pragma unroll
                for (int c = 0; c < 32; c++)
                    if (!((w >> c) & 1)) sr[c] = 0xff800000u;
            }
            if (t < T) {
                // sweep 1: running max and sum of this thread's columns
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < 32; c++) mx = fmaxf(mx, __uint_as_float(sr[c]));
                mx *= sl;
                if (mx > m) {
                    l *= ex2_approx(m - mx);     // 0 while m is still -inf
                    m = mx;
                }
                if (m > -INFINITY) {
                    // only the sum of these exponentials is kept: every kFpPoly-th pair is a cubic on the FMA pipe
                    // (relative error 1.6e-4), which takes that share of sweep 1 off the MUFU
                    uint64_t acc0 = 0ull, acc1 = 0ull;          // four partial sums as two packed pairs
                    const uint64_t sl2 = pk64(sl, sl), nm2 = pk64(-m, -m);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const uint64_t x = fma2p(pk64(__uint_as_float(sr[2 * j]), __uint_as_float(sr[2 * j + 1])), sl2, nm2);
                        float e0, e1;
                        if (kFpPoly > 0 && j % (kFpPoly > 0 ? kFpPoly : 1) == 0) {
                            exp2_fma_pair(x, e0, e1);
                        } else {
                            float x0, x1;
                            up64(x, x0, x1);
                            e0 = ex2_approx(x0);
                            e1 = ex2_approx(x1);
                        }
                        if (j & 1) acc1 = add2p(acc1, pk64(e0, e1));
                        else acc0 = add2p(acc0, pk64(e0, e1));
                    }
                    float ps4[4];
                    up64(acc0, ps4[0], ps4[1]);
                    up64(acc1, ps4[2], ps4[3]);
                    l += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
                }
            } else {
                // sweep 2: probabilities out
                const float neg_m = m > -INFINITY ? -m : 0.f;
                const size_t off = ((((size_t)b * p.H + h) * p.blocks + ent->blk[half]) * 64 + (r & 63)) * 64 + cb;
                // a row with nothing visible has only -inf scores: every exponential is 0 and so is 0 * inv
                const uint64_t sl2 = pk64(sl, sl), nm2 = pk64(neg_m, neg_m), inv2 = pk64(inv, inv);
#pragma unroll
                for (int c0 = 0; c0 < 32; c0 += 16) {
                    uint32_t v[16];
#pragma unroll
                    for (int c = 0; c < 16; c += 2) {
                        const uint64_t x = fma2p(pk64(__uint_as_float(sr[c0 + c]), __uint_as_float(sr[c0 + c + 1])), sl2, nm2);
                        float x0, x1;
                        up64(x, x0, x1);
                        const uint64_t y = mul2p(pk64(ex2_approx(x0), ex2_approx(x1)), inv2);
                        float y0, y1;
                        up64(y, y0, y1);
                        v[c] = __float_as_uint(y0);
                        v[c + 1] = __float_as_uint(y1);
                    }
                    store_row16(p.Y, off, v, p.out_dtype, c0);
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (st->abort_flag) {
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

// P viewed as [rows, 64] 16-bit row-major, boxes of 64 x 64, 128-byte swizzle, zero fill outside
static int make_p_map(CUtensorMap *map, const void *base, uint64_t rows, int is_bf16)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {64, rows};
    cuuint64_t strides[1] = {128};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

}  // namespace tc

static bool tc_shape_ok(uint32_t bs, const AttnDims &p, uint32_t max_lut)
{
    return bs == 64 && p.d == 64 && p.nb_a == p.nb_b && max_lut != 0 && 2 * (uint64_t)max_lut <= tc::kMaxUnion &&
           (uint64_t)p.B * p.nb_a * 64 < (1ull << 31) && (uint64_t)p.B * p.H * p.blocks * 64 < (1ull << 31) - 64;
}

bool tc_sddmm_supported(int ab_dtype, uint32_t bs, const AttnDims &p, const void *a, const void *b, const void *c)
{
    // what the kernel cannot take goes to the CUDA-core kernel instead of failing: unequal block grids, operands the TMA
    // cannot address (16-byte aligned a, b; 32-byte aligned c)
    if ((((uintptr_t)a | (uintptr_t)b) & 15) != 0 || ((uintptr_t)c & 31) != 0 || p.nb_a != p.nb_b) return false;
    return (ab_dtype == SFB_BF16 || ab_dtype == SFB_F16) && bs == 64 && p.d == 64 && p.blocks > 0 &&
           (uint64_t)p.B * (p.nb_a > p.nb_b ? p.nb_a : p.nb_b) * 64 < (1ull << 31);
}

int tc_sddmm(cudaStream_t s, const void *nt_lut, const void *a, const void *b, void *c, int ab_dtype, int c_dtype, const AttnDims &p)
{
    using namespace tc;
    SFB_REQUIRE((((uintptr_t)a | (uintptr_t)b) & 15) == 0 && ((uintptr_t)c & 31) == 0, "sfb_bst_sgemm_nt: a, b must be 16-byte and c 32-byte aligned");
    SFB_REQUIRE(p.nb_a == p.nb_b, "sfb_bst_sgemm_nt: ctx_blks_a != ctx_blks_b is not supported for 16-bit operands");
    const int is_bf16 = ab_dtype == SFB_BF16;
    const uint64_t rows = (uint64_t)p.B * p.nb_a * 64;
    CUtensorMap qm, km, om;
    if (make_map(&qm, a, rows, p.H, is_bf16, 64) || make_map(&km, b, rows, p.H, is_bf16, 64)) return 1;
    // the scores as [B*H*blocks*64 rows, 64] for the TMA stores of 16-bit outputs (unused for fp32 outputs)
    if (make_p_map(&om, c, (uint64_t)p.B * p.H * p.blocks * 64, c_dtype != SFB_F16)) return 1;
    SFB_REQUIRE((uint64_t)p.B * p.H * p.blocks * 64 < (1ull << 31), "sfb_bst_sgemm_nt: too many blocks for one launch");
    UParams prm = {(const uint2 *)nt_lut, c, p.B, p.H, p.nb_a, p.blocks, p.lut_stride, c_dtype, is_bf16, 0};
    static DeviceOnce once;
    const int dev = current_device();
    if (!once.done(dev)) {
        if (cudaFuncSetAttribute(sddmm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSddmmSmem) != cudaSuccess ||
            cudaFuncSetAttribute(sddmm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSddmmGradSmem) != cudaSuccess)
            return fail("sfb_bst_sgemm_nt: cannot reserve %zu bytes of shared memory", kSddmmGradSmem);
        once.mark(dev);
    }
    sddmm_tc_kernel<false><<<dim3((p.blocks + kChunk - 1) / kChunk, p.B, p.H), 320, kSddmmSmem, s>>>(qm, km, om, om, prm);
    return check_launch("sfb_bst_sgemm_nt");
}

// dS = P * (dO.V^T - delta) * scale on the kept blocks: 16-bit dO, V, P and dS of one type
int tc_sddmm_softmax_grad(cudaStream_t s, const void *nt_lut, const void *dout, const void *v, const void *pblk, const float *delta,
                          void *ds, int dtype, const AttnDims &p, float scale)
{
    using namespace tc;
    SFB_REQUIRE((((uintptr_t)dout | (uintptr_t)v | (uintptr_t)pblk) & 15) == 0 && ((uintptr_t)ds & 31) == 0,
                "sfb_fused_sddmm_softmax_grad: dO, V, P must be 16-byte and dS 32-byte aligned");
    const int is_bf16 = dtype == SFB_BF16;
    const uint64_t rows = (uint64_t)p.B * p.nb_a * 64, prow = (uint64_t)p.B * p.H * p.blocks * 64;
    SFB_REQUIRE(prow < (1ull << 31), "sfb_fused_sddmm_softmax_grad: too many blocks for one launch");
    CUtensorMap qm, km, om, pm;
    if (make_map(&qm, dout, rows, p.H, is_bf16, 64) || make_map(&km, v, rows, p.H, is_bf16, 64) || make_p_map(&om, ds, prow, is_bf16) ||
        make_p_map(&pm, pblk, prow, is_bf16))
        return 1;
    UParams prm = {(const uint2 *)nt_lut, ds, p.B, p.H, p.nb_a, p.blocks, p.lut_stride, dtype, is_bf16, 0, 0, delta, scale};
    static DeviceOnce once;
    const int dev = current_device();
    if (!once.done(dev)) {
        if (cudaFuncSetAttribute(sddmm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSddmmGradSmem) != cudaSuccess)
            return fail("sfb_fused_sddmm_softmax_grad: cannot reserve %zu bytes of shared memory", kSddmmGradSmem);
        once.mark(dev);
    }
    sddmm_tc_kernel<true><<<dim3((p.blocks + kChunk - 1) / kChunk, p.B, p.H), 320, kSddmmGradSmem, s>>>(qm, km, om, pm, prm);
    return check_launch("sfb_fused_sddmm_softmax_grad");
}

bool tc_fused_p_supported(int ab_dtype, uint32_t bs, const AttnDims &p, float scale, const void *a, const void *b, const void *y)
{
    if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)y) & 31) != 0) return false;     // the CUDA-core kernel takes any alignment
    // the longest row is not an argument of the fused entry points: any row of the block grid must fit the union list
    return (ab_dtype == SFB_BF16 || ab_dtype == SFB_F16) && scale > 0.f && p.blocks > 0 &&
           tc_shape_ok(bs, p, p.nb_a <= tc::kMaxUnion / 2 ? p.nb_a : 0);
}

int tc_fused_p(cudaStream_t s, const void *nn_lut, const void *a, const void *b, const void *mask, void *y, int ab_dtype,
               int y_dtype, const AttnDims &p, float scale)
{
    using namespace tc;
    SFB_REQUIRE((((uintptr_t)a | (uintptr_t)b | (uintptr_t)y) & 31) == 0, "sfb_fused_sddmm_softmax: a, b, y must be 32-byte aligned");
    const int is_bf16 = ab_dtype == SFB_BF16;
    const uint64_t rows = (uint64_t)p.B * p.nb_a * 64;
    CUtensorMap qm, km;
    if (make_map(&qm, a, rows, p.H, is_bf16, 128) || make_map(&km, b, rows, p.H, is_bf16, 64)) return 1;
    FpParams prm = {(const uint2 *)nn_lut, (const uint64_t *)mask, y, p.B, p.H, p.nb_a, p.blocks, p.lut_stride, p.mask_stride,
                    scale * 1.4426950408889634f, y_dtype, is_bf16};
    static DeviceOnce once;
    const int dev = current_device();
    if (!once.done(dev)) {
        if (cudaFuncSetAttribute(fused_p_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFpSmem) != cudaSuccess)
            return fail("sfb_fused_sddmm_softmax: cannot reserve %zu bytes of shared memory", kFpSmem);
        once.mark(dev);
    }
    fused_p_tc_kernel<<<dim3((p.nb_a + 1) / 2, p.B, p.H), kFpThreads, kFpSmem, s>>>(qm, km, prm);
    return check_launch("sfb_fused_sddmm_softmax");
}

bool tc_spmm_supported(int a_dtype, int bc_dtype, uint32_t bs, const AttnDims &p, uint32_t max_lut, const void *a, const void *b,
                       const void *c)
{
    if ((((uintptr_t)a | (uintptr_t)b) & 15) != 0 || ((uintptr_t)c & 31) != 0) return false;    // the CUDA-core kernel takes any alignment
    return a_dtype == bc_dtype && (a_dtype == SFB_BF16 || a_dtype == SFB_F16) && p.blocks > 0 && tc_shape_ok(bs, p, max_lut);
}

int tc_spmm(cudaStream_t s, const void *nn_lut, const void *a, const void *b, void *c, int dtype, const AttnDims &p, bool trans)
{
    using namespace tc;
    SFB_REQUIRE((((uintptr_t)a | (uintptr_t)b) & 15) == 0 && ((uintptr_t)c & 31) == 0, "sfb_bst_sgemm_xn: a, b must be 16-byte and c 32-byte aligned");
    const int is_bf16 = dtype == SFB_BF16;
    const uint64_t prow = (uint64_t)p.B * p.H * p.blocks * 64;
    CUtensorMap pm, vm;
    if (make_p_map(&pm, a, prow, is_bf16) || make_map(&vm, b, (uint64_t)p.B * p.nb_b * 64, p.H, is_bf16, 64)) return 1;
    UParams prm = {(const uint2 *)nn_lut, c, p.B, p.H, p.nb_a, p.blocks, p.lut_stride, dtype, is_bf16, (uint32_t)prow, trans ? 1 : 0};
    static DeviceOnce once;
    const int dev = current_device();
    if (!once.done(dev)) {
        if (cudaFuncSetAttribute(spmm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSpmmSmem) != cudaSuccess)
            return fail("sfb_bst_sgemm_xn: cannot reserve %zu bytes of shared memory", kSpmmSmem);
        once.mark(dev);
    }
    spmm_tc_kernel<<<dim3((p.nb_a + 1) / 2, p.B, p.H), 192, kSpmmSmem, s>>>(pm, vm, prm);
    return check_launch("sfb_bst_sgemm_xn");
}

int tc_status_clear_unfused()
{
    const uint32_t zero = 0;
    cudaError_t e = cudaMemcpyToSymbol(tc::g_status, &zero, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status_clear: %s", cudaGetErrorString(e));
    return 0;
}

int tc_status_unfused(uint32_t *out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, tc::g_status, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace sfb
