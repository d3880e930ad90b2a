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
#include "tc_common.cuh"

namespace sfb {

namespace tc {

constexpr int kStages = 4;                      // K/V ring depth
constexpr uint32_t kTmemCols = 256;             // S0 | S1 | O (64 + 16 row-sum columns); P reuses S's first 32 columns
constexpr uint32_t kOnesBytes = 64 * 128;       // the tile of ones behind V
constexpr float kRescaleThreshold = 8.0f;       // log2 units: P stays below 2^8

struct SharedState {
    uint64_t q_full, kv_full[kStages], kv_empty[kStages];
    uint64_t s_full[2], p_full[2], pv_done, o_final, drained;
    uint32_t tmem_base, n_union, abort_flag, pad;
    UnionEntry entries[kMaxUnion];
    uint2 cand[kMaxUnion];
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



// ---- the kernel ---------------------------------------------------------------------------------
template <bool HAS_MASK, bool BF16>
__global__ void __launch_bounds__(192, 2)
fused_attention_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                          const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap omap, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *q_tile = smem;
    uint8_t *kv_tiles = q_tile + kQBytes;                      // stage s: K at s*2*kTileBytes, V right after
    uint8_t *ones_tile = kv_tiles + kStages * 2 * kTileBytes;
    SharedState *st = (SharedState *)(ones_tile + kOnesBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t pair = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const bool has_row1 = pair * 2 + 1 < p.nb;
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
        // Q does not depend on the LUT: it travels while the union is built
        mbar_expect_tx(&st->q_full, kQBytes);
        tma_load_2d(smem_u32(q_tile), &qmap, &st->q_full, (int32_t)(h * 64), (int32_t)(b * L + pair * 128));
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&st->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        // 1.0 in the operand type of V, everywhere: the swizzle cannot matter
        const uint32_t one2 = BF16 ? 0x3f803f80u : 0x3c003c00u;
        for (uint32_t i = threadIdx.x; i < kOnesBytes / 16; i += blockDim.x)
            ((uint4 *)ones_tile)[i] = make_uint4(one2, one2, one2, one2);
        fence_proxy_async();
    }
    build_union(nn, pair, p.nb, st->entries, st->cand, &st->n_union, &st->abort_flag);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();

    const uint32_t T = st->n_union;
    const uint32_t tmem = st->tmem_base;
    const uint32_t tmem_s[2] = {tmem, tmem + 64};
    const uint32_t tmem_o = tmem + 128;          // 64 columns of O, then 16 columns that all hold the row sum
    const int32_t xq = (int32_t)(h * 64);

    if (warp == 0) {
        // ===== TMA producer: a stage (K and V of one key block) is released when its P.V has completed =====
        if (lane == 0) {
            for (uint32_t t = 0; t < T; t++) {
                const uint32_t s = t % kStages;
                const int32_t y = (int32_t)(b * L + st->entries[t].col * 64);
                if (t >= kStages && !mbar_wait(&st->kv_empty[s], ((t / kStages) - 1) & 1, abort_flag, 1)) break;
                mbar_expect_tx(&st->kv_full[s], 2 * kTileBytes);
                tma_load_2d(smem_u32(kv_tiles + s * 2 * kTileBytes), &kmap, &st->kv_full[s], xq, y);
                tma_load_2d(smem_u32(kv_tiles + s * 2 * kTileBytes + kTileBytes), &vmap, &st->kv_full[s], xq, y);
            }
            if (T == 0) mbar_wait(&st->q_full, 0, abort_flag, 2);   // nobody else waits for the Q tile then
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
                if (!mbar_wait(&st->kv_full[s], (t / kStages) & 1, abort_flag, 3)) return false;
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
                if (!mbar_wait(&st->p_full[t & 1], (t >> 1) & 1, abort_flag, 5)) { alive = false; break; }
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
        uint32_t sr[64];                                   // this row of S(t), fp32 bits
        if (T > 0) {
            alive = mbar_wait_warp(&st->s_full[0], 0, abort_flag, 6);
            if (alive) {
                tcgen05_fence_after();
                TMEM_LD_32((sr), tmem_s[0] + lane_field);
                TMEM_LD_32((sr + 32), tmem_s[0] + lane_field + 32);
            }
        }
        for (uint32_t t = 0; alive && t < T; t++) {
            tmem_wait_ld();
            const UnionEntry ent = st->entries[t];
            const bool mine = (ent.flags >> half) & 1;     // the same for the whole warp
            if (HAS_MASK && mine) {
                const uint64_t w = p.mask[(size_t)h * p.mask_stride + (size_t)ent.blk[half] * 64 + (r & 63)];
#pragma unroll
                for (int c = 0; c < 64; c++)
                    if (!((w >> c) & 1)) sr[c] = 0xff800000u;
            }
            uint32_t pk[32];
            float mx = -INFINITY;
            bool settle = true;
            if (t > 0) {
                // Speculate that the reference max still holds (it moves only when a row max outgrows it by
                // 2^8): exponentials and the row max come out of ONE pass over the registers, so the max no
                // longer sits in front of the MUFU work.  A warp that guessed wrong repeats the tile below.
                if (mine) {
                    const float neg_m = m_used > -INFINITY ? -m_used : 0.f;
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int c = 0; c < 64; c += 2) {
                        float x0, x1;
                        m4[(c >> 1) & 3] = max3(m4[(c >> 1) & 3], __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
                        fma2(x0, x1, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]), sl, neg_m);
                        const uint32_t e2 = ex2_pair_f16(x0, x1);
                        pk[c >> 1] = BF16 ? f16x2_to_bf16x2(e2) : e2;
                    }
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl;
                } else {
#pragma unroll
                    for (int c = 0; c < 32; c++) pk[c] = 0u;
                }
                const bool grow = mx > m_used + kRescaleThreshold || (m_used == -INFINITY && mx > -INFINITY);
                settle = __any_sync(0xffffffffu, grow);
            }
            if (settle) {
                if (t == 0 && mine) {
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
                const float neg_m = m_used > -INFINITY ? -m_used : 0.f;
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
            }
            // P (16-bit pairs) takes the place of the first 32 columns of this row of S; while that store is in
            // flight the next tile's scores start their way into the registers
            TMEM_ST_32(tmem_s[t & 1] + lane_field, (pk));
            // if S(t+1) is there already its load overlaps the store; P(t) is never held back waiting for it
            const bool early = t + 1 < T && __all_sync(0xffffffffu, mbar_try_wait(&st->s_full[(t + 1) & 1], ((t + 1) >> 1) & 1));
            if (early) {
                tcgen05_fence_after();
                TMEM_LD_32((sr), tmem_s[(t + 1) & 1] + lane_field);
                TMEM_LD_32((sr + 32), tmem_s[(t + 1) & 1] + lane_field + 32);
            }
            tmem_wait_st();
            tcgen05_fence_before();
            mbar_arrive(&st->p_full[t & 1]);
            if (t + 1 < T && !early) {
                if (!mbar_wait_warp(&st->s_full[(t + 1) & 1], ((t + 1) >> 1) & 1, abort_flag, 6)) { alive = false; break; }
                tcgen05_fence_after();
                TMEM_LD_32((sr), tmem_s[(t + 1) & 1] + lane_field);
                TMEM_LD_32((sr + 32), tmem_s[(t + 1) & 1] + lane_field + 32);
            }
        }
        tmem_wait_ld();

        // ---- epilogue: O / row sum -> global.  The four softmax warps agree first on whether all of them got here
        // in good order (they meet at a named barrier below, so they take that road together or not at all) ----
        if (T > 0 && alive) alive = mbar_wait_warp(&st->o_final, 0, abort_flag, 10);
        // a row pair without key blocks never multiplied: its Q load may still be on its way into the buffer O is staged in
        if (T == 0 && alive) alive = mbar_wait_warp(&st->q_full, 0, abort_flag, 2);
        uint32_t all_ok;
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.red.and.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(all_ok) : "r"((uint32_t)alive) : "memory");
        if (all_ok) {
            tcgen05_fence_after();
            uint32_t oc[64];
            float inv = 0.f;
            if (T > 0) {
                uint32_t lc[16];
                TMEM_LD_16((lc), tmem_o + lane_field + 64);
                TMEM_LD_32((oc), tmem_o + lane_field);
                TMEM_LD_32((oc + 32), tmem_o + lane_field + 32);
                tmem_wait_ld();
                const float lsum = __uint_as_float(lc[0]);
                inv = lsum > 0.f ? 1.f / lsum : 0.f;
            }
            uint32_t w[32];
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float a0 = T > 0 ? __uint_as_float(oc[2 * j]) * inv : 0.f;
                const float a1 = T > 0 ? __uint_as_float(oc[2 * j + 1]) * inv : 0.f;
                w[j] = pack2(a0, a1, BF16);
            }
            if (has_row1) {
                // the 128 x 64 tile leaves through the Q tile's shared memory (every MMA that read Q has completed) and one
                // TMA store: whole 128-byte lines instead of 128 scattered rows.  16-byte chunk c of row r sits at chunk
                // c ^ (r % 8), the tensor map's 128-byte swizzle.
                uint8_t *orow = q_tile + r * 128;
#pragma unroll
                for (int ch = 0; ch < 8; ch++)
                    *(uint4 *)(orow + ((ch ^ (r & 7)) << 4)) = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
                fence_proxy_async();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                 ::"l"((uint64_t)&omap), "r"(smem_u32(q_tile)), "r"(xq), "r"((int32_t)(b * L + pair * 128)) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the store's reads
                }
            } else if (row_valid) {
                // an odd number of block-rows: the last CTA owns 64 rows only and writes them directly
                uint16_t *dst = (uint16_t *)p.O + ((size_t)b * L + (size_t)pair * 128 + r) * ((size_t)p.H * 64) + (size_t)h * 64;
#pragma unroll
                for (int ch = 0; ch < 8; ch++) *(uint4 *)(dst + 8 * ch) = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
            }
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
    CUtensorMap qm, km, vm, om;
    if (make_map(&qm, q, rows, p.H, is_bf16, 128) || make_map(&km, k, rows, p.H, is_bf16, 64) ||
        make_map(&vm, v, rows, p.H, is_bf16, 64) || make_map(&om, o, rows, p.H, is_bf16, 128))
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
    if (mask && is_bf16) fused_attention_tc_kernel<true, true><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, om, prm);
    else if (mask) fused_attention_tc_kernel<true, false><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, om, prm);
    else if (is_bf16) fused_attention_tc_kernel<false, true><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, om, prm);
    else fused_attention_tc_kernel<false, false><<<grid, 192, kSmemBytes, s>>>(qm, km, vm, om, prm);
    return check_launch("sfb_fused_attention");
}

int tc_status_fused(uint32_t *out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, tc::g_status, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace sfb
