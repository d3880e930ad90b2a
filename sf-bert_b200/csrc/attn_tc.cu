// Fused block-sparse attention on the 5th-generation tensor cores (tcgen05) for 16-bit operands,
// block_size 64, head size 64.
//
// One persistent CTA per SM runs THREE independent streams.  A stream owns one work item at a time: a PAIR of
// adjacent block-rows of one (batch, head) = 128 queries = one M=128 MMA tile, and walks the union of the two
// rows' key blocks.  Nothing is exchanged between CTAs or between streams: no flags, no scratch in global
// memory, no waiting on other CTAs (the reference's fused kernels spin on counters in global memory,
// fusion_blocksparse.h:224-366).  Per key block of a stream:
//     S  = Q . K^T            tcgen05.mma, A and B from shared memory (TMA, 128-byte swizzle), accumulator in TMEM
//     P  = exp2(S*c - m)      128 threads, one query row each, straight out of TMEM (fp32 ex2.approx; the packed
//                             fp16 form measured slower); the row sum is kept in fp32 registers; P goes back to
//                             TMEM as 16-bit pairs
//     O += P . V              tcgen05.mma, P as the A operand from TMEM, V from shared memory as an MN-major operand
// TMEM per stream (160 columns): two score buffers that overlap by half, S_even = [0,64) and S_odd = [32,96), with
// P_even = [0,32) and P_odd = [64,96): S(t+1) never touches P(t), so the next scores are produced while the
// softmax of the current ones runs, and a buffer is handed back as soon as its scores are in registers.  O = [96,160).
// Why three streams and one MMA-issuing warp per stream: a tcgen05.mma costs its issuing thread 120-145 cycles
// whatever its N (measured), issuers in different warps overlap, and the softmax pass only reaches the MUFU's
// rate with three warps per SM sub-partition.
// Warps: 0-11 softmax + epilogue (stream = warp / 4, TMEM lane quarter = warp % 4), 12-14 MMA issuers, 15 TMA
// producer of the query and key tiles (lane = stream), 16 the same for the value tiles and the output stores, 17-19
// planners (each builds the unions of its stream's coming items while the current one runs).  The control warpgroups hand registers to the softmax warpgroups (setmaxnreg): the pool is what
// the CTA was launched with (640 threads x 96); the softmax warps take 12 x 32 x 32 = 12288 more, exactly what the
// control warps give back (8 x 32 x 48).  An increase that the pool cannot cover would wait for ever.
// Every wait is bounded; on a timeout the CTA records a status word and leaves through the common teardown.
#include "tc_common.cuh"

// every SFB_TC_POLY-th pair of exponentials runs as a cubic on the FMA pipe (0 = all on the MUFU, the default: with
// every fourth pair moved the kernel was no faster, the MUFU is not what holds it back)
#ifndef SFB_TC_POLY
#define SFB_TC_POLY 0
#endif

namespace sfb {

namespace tc {

constexpr int kStreams = 3;
constexpr int kMaxU = 256;                      // key blocks a row pair may touch in this kernel
constexpr uint32_t kThreads = 20 * 32;       // five warpgroups: three of softmax warps, two of control warps
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kStreamCols = 160;
constexpr float kRescaleThreshold = 8.0f;       // log2 units: P stays below 2^8

struct UEntry {
    uint32_t col_flags;   // key block column | bit 30: upper block-row has it | bit 31: lower block-row has it
    uint32_t blk[2];      // block ids (for the element masks)
    uint32_t pad;
};

struct StreamState {
    uint64_t q_full, q_free;
    uint64_t k_full[2], v_full[2];
    uint64_t qk_done[2];    // S(t) is complete: the softmax threads read it, the producer refills the key tile's buffer
    uint64_t pv_done[2];    // O += P(t).V(t) is complete: O may be rescaled, the producer refills the value tile's buffer
    uint64_t s_free, p_full[2], o_final, o_free;
    uint64_t list_ready[2], list_free[2];
    uint64_t stage_full, stage_free;
    uint32_t list_n[2];
    int32_t store_x, store_y;   // where the staged output tile goes (y < 0: the rows were written directly)
};

struct SharedState {
    StreamState st[kStreams];
    uint64_t drained[kStreams];
    uint32_t tmem_base, abort_flag;
};

constexpr uint32_t kOffQ = 0;                                        // 3 x 16 KB query tiles
constexpr uint32_t kOffK = kOffQ + kStreams * kQBytes;               // 3 x 2 x 8 KB key tiles
constexpr uint32_t kOffV = kOffK + kStreams * 2 * kTileBytes;        // 3 x 2 x 8 KB value tiles
constexpr uint32_t kOffO = kOffV + kStreams * 2 * kTileBytes;        // 3 x 16 KB output staging
constexpr uint32_t kOffList = kOffO + kStreams * kQBytes;            // 3 x 2 union lists
constexpr uint32_t kOffState = kOffList + kStreams * 2 * kMaxU * (uint32_t)sizeof(UEntry);
constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + kOffState + sizeof(SharedState);
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

struct Params {
    const uint2 *nn_lut;
    const uint64_t *mask;
    void *O;
    uint32_t B, H, nb, npairs, n_items, lut_stride, mask_stride;
    uint32_t o_pitch;      // elements between consecutive rows of O
    uint32_t cta_first;    // order in which a round's items are dealt to the CTAs' streams (item_id)
    float scale_log2e;
};

struct Item {
    uint32_t pair, b, h;
};

// item ids run over (batch, head) slowest and the row pair fastest, so that CTAs working at the same time share
// K and V in L2; inside one (batch, head) the pairs are dealt from both ends inwards: the long rows of the
// layouts at hand sit at the ends (causal: the last rows; BigBird: the global first and last rows), and they
// go first (the reference's heuristic, blocksparse.h:747-748)
__device__ __forceinline__ Item decode_item(uint32_t id, const Params &p)
{
    const uint32_t bh = id / p.npairs, pr = id % p.npairs;
    Item it;
    it.pair = (pr & 1u) ? p.npairs - 1u - (pr >> 1) : (pr >> 1);
    it.b = bh / p.H;
    it.h = bh % p.H;
    return it;
}
// round k, stream s of this CTA.  Long launches: a CTA's three streams take neighbouring items (neighbouring row pairs
// of one head).  Launches of only a few rounds (p.cta_first): within a round the items go to stream 0 of every CTA
// first, then to stream 1, ...: in the last, partial round a CTA then runs fewer streams at once instead of some CTAs
// running three and others none, and a stream with the SM to itself finishes its item sooner (the 24-layer stack with
// 512 items per launch: 973 -> 1036 sequences/s).  On long launches with items of very different length (BigBird)
// that order measured 8 % slower, so it is kept to the launches that are all tail.
__device__ __forceinline__ uint32_t item_id(uint32_t k, uint32_t s, const Params &p)
{
    return p.cta_first ? (k * kStreams + s) * gridDim.x + blockIdx.x : (k * gridDim.x + blockIdx.x) * kStreams + s;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi)
{
    uint32_t y;
    if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(y) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(y) : "f"(hi), "f"(lo));
    return y;
}
__device__ __forceinline__ void give_up(volatile uint32_t *abort_flag, uint32_t code)
{
    *abort_flag = 1;
    atomicCAS(&g_status, 0u, (code << 24) | (blockIdx.x & 0xffffffu));
}

#ifndef SFB_TC_HINT_NS
#define SFB_TC_HINT_NS 2000
#endif
constexpr uint32_t kSleepPolls = kWaitLimit >> 8;    // polls of up to SFB_TC_HINT_NS each before a wait gives up

// bounded wait that sleeps in the barrier unit between polls
__device__ __forceinline__ bool bar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
{
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < kSleepPolls; i++) {
        if (mbar_try_wait_sleep(bar, parity, SFB_TC_HINT_NS)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    give_up(abort_flag, code);
    return false;
}
__device__ __forceinline__ bool bar_wait_warp(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
{
    const bool ok = bar_wait(bar, parity, abort_flag, code);
    return __all_sync(0xffffffffu, ok);
}

// bounded wait on two barriers at once (one dependent chain instead of two)
__device__ __forceinline__ bool mbar_wait2(uint64_t *bar_a, uint32_t par_a, uint64_t *bar_b, uint32_t par_b, volatile uint32_t *abort_flag,
                                           uint32_t code)
{
    const bool a = mbar_try_wait(bar_a, par_a), b = mbar_try_wait(bar_b, par_b);
    if (a && b) return true;
    return (a || bar_wait(bar_a, par_a, abort_flag, code)) && (b || bar_wait(bar_b, par_b, abort_flag, code));
}

// The union of the key blocks of block-rows 2*pair and 2*pair+1, built by ONE warp: the upper row's blocks in LUT
// order, then the blocks only the lower row has.  Returns the number of entries, or 0xffffffff when a row or the
// union does not fit kMaxU.
__device__ __forceinline__ uint32_t plan_union(const uint2 *nn, uint32_t pair, uint32_t nb, UEntry *ent, uint32_t lane)
{
    const uint32_t row0 = pair * 2, row1 = pair * 2 + 1;
    const uint2 head0 = nn[row0];
    const uint2 head1 = row1 < nb ? nn[row1] : make_uint2(0, 0);
    const uint32_t n0 = head0.y, n1 = head1.y;
    if (n0 > (uint32_t)kMaxU || n1 > (uint32_t)kMaxU) return 0xffffffffu;
    for (uint32_t i = lane; i < n0; i += 32) {
        const uint2 e = nn[head0.x + i];
        ent[i].col_flags = (e.y & 0x3fffffffu) | (1u << 30);
        ent[i].blk[0] = e.x;
        ent[i].blk[1] = 0;
    }
    __syncwarp();
    uint32_t n = n0;
    for (uint32_t base = 0; base < n1; base += 32) {
        const uint32_t i = base + lane;
        const bool valid = i < n1;
        const uint2 e = valid ? nn[head1.x + i] : make_uint2(0, 0);
        bool fresh = valid;
        if (valid)
            for (uint32_t u = 0; u < n0; u++)
                if ((ent[u].col_flags & 0x3fffffffu) == (e.y & 0x3fffffffu)) {
                    ent[u].col_flags |= 1u << 31;
                    ent[u].blk[1] = e.x;
                    fresh = false;
                    break;
                }
        const uint32_t votes = __ballot_sync(0xffffffffu, fresh);
        const uint32_t at = n + __popc(votes & ((1u << lane) - 1u));
        if (n + __popc(votes) > (uint32_t)kMaxU) return 0xffffffffu;
        if (fresh) {
            ent[at].col_flags = (e.y & 0x3fffffffu) | (1u << 31);
            ent[at].blk[0] = 0;
            ent[at].blk[1] = e.x;
        }
        n += __popc(votes);
    }
    __syncwarp();
    return n;
}

// A TMA producer: IS_K = true loads every item's query tile and key tiles, IS_K = false its value tiles (the two run
// in different warps: a value tile's buffer is released late, by the P.V product two steps back, and must not hold up
// the key tile of the next step); the value producer also issues the TMA stores of the staged output tiles (qmap is
// the output's map there).  Lane s of the producer warp serves stream s: the three cursors sit in the lanes' own
// registers and advance side by side (a single thread walking three cursors kept them in local or shared memory and
// needed thousands of cycles per round, measured).  Nothing here suspends the thread, so one slow stream never
// holds up another for longer than a divergent branch.
template <bool IS_K>
__device__ __forceinline__ void tma_producer(uint32_t s, uint8_t *smem, SharedState *sh, const UEntry *lists, const CUtensorMap &qmap,
                                             const CUtensorMap &tmap, const Params &p, uint32_t L, volatile uint32_t *abort_flag)
{
    StreamState *st = &sh->st[s];
    uint32_t k = 0, t = 0, T = 0, g = 0, kq = 0, stage = 0, stored = 0, age = 0, idle = 0;
    int32_t xq = 0, row0 = 0, pair128 = 0;
    bool pending = false, done = false;
    uint64_t *blocked_on = &st->list_ready[0];     // what this lane waits for when a round makes no progress
    uint32_t blocked_par = 0;
    while (!done) {
        bool progress = false;
        if (!IS_K) {
            // the value producer also sends the stream's staged output tiles on their way (every item has one)
            if (mbar_test_wait(&st->stage_full, stored & 1)) {
                if (pending) {
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    mbar_arrive(&st->stage_free);
                }
                if (st->store_y >= 0) {
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                 ::"l"((uint64_t)&qmap), "r"(smem_u32(smem + kOffO + s * kQBytes)), "r"(st->store_x), "r"(st->store_y) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                // the tile is handed back a little later, when the store has surely read it (a wait here would hold up the loads)
                pending = true;
                age = 0;
                stored++;
                progress = true;
            } else if (pending && (++age >= 8 || stage == 4)) {
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the store's reads
                mbar_arrive(&st->stage_free);
                pending = false;
            }
            if (stage == 4 && stored == k && !pending) break;
        }
        bool again = stage != 4;
        while (again) {
            again = false;
            if (stage == 0) {
                const uint32_t id = item_id(k, s, p);
                if (id >= p.n_items) {
                    if (IS_K) done = true;
                    else stage = 4;            // loads done; the stores of the last items are still to come
                    progress = true;
                    break;
                }
                if (!mbar_test_wait(&st->list_ready[k & 1], (k >> 1) & 1)) {
                    blocked_on = &st->list_ready[k & 1];
                    blocked_par = (k >> 1) & 1;
                    break;
                }
                T = st->list_n[k & 1];
                progress = again = true;
                if (T == 0) {
                    mbar_arrive(&st->list_free[k & 1]);
                    k++;
                    continue;
                }
                const Item it = decode_item(id, p);
                xq = (int32_t)(it.h * 64);
                row0 = (int32_t)(it.b * L);
                pair128 = (int32_t)(it.pair * 128);
                t = 0;
                stage = IS_K ? 1 : 2;
            } else if (stage == 1) {
                // the query tile is free once the previous item's last S product has completed
                if (kq >= 1 && !mbar_test_wait(&st->q_free, (kq - 1) & 1)) {
                    blocked_on = &st->q_free;
                    blocked_par = (kq - 1) & 1;
                    break;
                }
                mbar_expect_tx(&st->q_full, kQBytes);
                tma_load_2d(smem_u32(smem + kOffQ + s * kQBytes), &qmap, &st->q_full, xq, row0 + pair128);
                stage = 2;
                progress = again = true;
            } else {
                const uint32_t gg = g + t, b2 = gg & 1;
                const UEntry *list = lists + (s * 2 + (k & 1)) * kMaxU;
                uint64_t *empty = IS_K ? &st->qk_done[b2] : &st->pv_done[b2];
                uint64_t *full = IS_K ? &st->k_full[b2] : &st->v_full[b2];
                if (gg >= 2 && !mbar_test_wait(empty, ((gg >> 1) - 1) & 1)) {
                    blocked_on = empty;
                    blocked_par = ((gg >> 1) - 1) & 1;
                    break;
                }
                mbar_expect_tx(full, kTileBytes);
                tma_load_2d(smem_u32(smem + (IS_K ? kOffK : kOffV) + (s * 2 + b2) * kTileBytes), &tmap, full, xq,
                            row0 + (int32_t)((list[t].col_flags & 0x3fffffffu) * 64));
                progress = again = true;
                if (++t == T) {
                    g += T;
                    kq++;
                    mbar_arrive(&st->list_free[k & 1]);
                    k++;
                    stage = 0;
                }
            }
        }
        if (progress) {
            idle = 0;
        } else {
            // Nothing to do: sleep in the barrier unit on what this lane is waiting for, a quarter of a microsecond at most (the
            // tiles are asked for a step ahead, the value lanes' stores can wait that long too).  A lane that polls flat
            // out takes a third of its sub-partition's issue slots from the softmax warps (measured); __nanosleep is no
            // alternative: a request of 20 ns came back after about a microsecond.
            if (stage != 4) mbar_try_wait_sleep(blocked_on, blocked_par, 256);
            if ((++idle & 63u) == 0 && *abort_flag) break;
            if (idle > (kWaitLimit >> 2)) {
                give_up(abort_flag, IS_K ? 1 : 15);
                break;
            }
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------------------
// POLY: every POLY-th pair of exponentials runs on the FMA pipe (0 = none)
template <bool HAS_MASK, bool BF16, int POLY>
__global__ void __launch_bounds__(kThreads, 1)
fused_attention_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                          const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap omap, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    SharedState *sh = (SharedState *)(smem + kOffState);
    UEntry *lists = (UEntry *)(smem + kOffList);

    const uint32_t hw_warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t warp = hw_warp;
    const uint32_t L = p.nb * 64;
    volatile uint32_t *abort_flag = &sh->abort_flag;
    const uint32_t fmt = BF16 ? 1u : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStreams; s++) {
            StreamState *st = &sh->st[s];
            mbar_init(&st->q_full, 1);
            mbar_init(&st->q_free, 1);
            for (int i = 0; i < 2; i++) {
                mbar_init(&st->k_full[i], 1);
                mbar_init(&st->v_full[i], 1);
                mbar_init(&st->qk_done[i], 1);
                mbar_init(&st->pv_done[i], 1);
                mbar_init(&st->p_full[i], 128);
                mbar_init(&st->list_ready[i], 1);
                mbar_init(&st->list_free[i], 7);   // two producers, issuer, four softmax warps
            }
            mbar_init(&st->s_free, 128);
            mbar_init(&st->o_final, 1);
            mbar_init(&st->o_free, 128);
            mbar_init(&st->stage_full, 128);
            mbar_init(&st->stage_free, 1);
            mbar_init(&sh->drained[s], 1);
        }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (hw_warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = sh->tmem_base;
    // barriers and TMEM are set up; nothing of global memory has been read yet.  Launched as a programmatic dependent,
    // the kernel waits here for the kernel before it (the projection that writes Q, K, V) to complete
    grid_dependency_wait();
    grid_launch_dependents();

    if (warp >= 16) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
        // ===== planner of stream s: the unions of the coming items, up to two ahead =====
        if (warp == 16) {
            if (lane < (uint32_t)kStreams) tma_producer<false>(lane, smem, sh, lists, omap, vmap, p, L, abort_flag);
        } else {
            const uint32_t s = warp - 17;
            StreamState *st = &sh->st[s];
            for (uint32_t k = 0;; k++) {
                const uint32_t id = item_id(k, s, p);
                if (id >= p.n_items) break;
                const uint32_t slot = k & 1;
                if (k >= 2 && !bar_wait_warp(&st->list_free[slot], ((k >> 1) - 1) & 1, abort_flag, 20)) break;
                const Item it = decode_item(id, p);
                uint32_t n = plan_union(p.nn_lut + (size_t)it.h * p.lut_stride, it.pair, p.nb, lists + (s * 2 + slot) * kMaxU, lane);
                if (n == 0xffffffffu) {
                    // a row pair that is too long for this kernel: recorded, and the pair's rows are written as zeros
                    if (lane == 0) atomicCAS(&g_status, 0u, (9u << 24) | (blockIdx.x & 0xffffffu));
                    n = 0;
                }
                if (lane == 0) {
                    st->list_n[slot] = n;
                    mbar_arrive(&st->list_ready[slot]);
                }
            }
        }
    } else if (warp >= 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
        if (warp == 15) {
            if (lane < (uint32_t)kStreams) tma_producer<true>(lane, smem, sh, lists, qmap, kmap, p, L, abort_flag);
        } else {
        // ===== MMA issuer of stream s:  S(0) | S(1) O(0) | S(2) O(1) | ...  =====
        const uint32_t s = warp - 12;
        if (lane == 0) {
            StreamState *st = &sh->st[s];
            const uint32_t tbase = tmem + s * kStreamCols;
            const uint32_t t_o = tbase + 96;     // S(even) = tbase, S(odd) = tbase + 32, P(even) = tbase, P(odd) = tbase + 64
            const uint32_t idesc_qk = instr_desc(fmt, fmt, 128, 64, 0);
            const uint32_t idesc_pv = instr_desc(fmt, fmt, 128, 64, 1);   // A and B must share a format
            const uint64_t q_desc = smem_desc_sw128(smem_u32(smem + kOffQ + s * kQBytes));
            uint32_t g = 0, kq = 0;
            bool alive = true;
            auto issue_qk = [&](uint32_t gg) -> bool {
                const uint32_t b2 = gg & 1;
                // S(gg) overlaps half of S(gg-1): that one must be in the softmax threads' registers
                if (gg >= 1 ? !mbar_wait2(&st->s_free, (gg - 1) & 1, &st->k_full[b2], (gg >> 1) & 1, abort_flag, 4)
                            : !bar_wait(&st->k_full[b2], (gg >> 1) & 1, abort_flag, 3))
                    return false;
                tcgen05_fence_after();
                const uint64_t k_desc = smem_desc_sw128(smem_u32(smem + kOffK + (s * 2 + b2) * kTileBytes));
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++)   // 16 of the 64 head elements per MMA: +32 bytes inside the swizzled row
                    umma_f16(tbase + 32 * b2, q_desc + 2 * kk, k_desc + 2 * kk, idesc_qk, kk);
                umma_commit(&st->qk_done[b2]);
                return true;
            };
            for (uint32_t k = 0; alive; k++) {
                const uint32_t id = item_id(k, s, p);
                if (id >= p.n_items) break;
                if (!bar_wait(&st->list_ready[k & 1], (k >> 1) & 1, abort_flag, 8)) break;
                const uint32_t T = st->list_n[k & 1];
                if (T > 0) {
                    if (!bar_wait(&st->q_full, kq & 1, abort_flag, 2)) break;
                    alive = issue_qk(g);
                    if (alive && T == 1) umma_commit(&st->q_free);
                    for (uint32_t t = 0; alive && t < T; t++) {
                        const uint32_t gg = g + t, b2 = gg & 1;
                        if (t + 1 < T) {
                            if (!issue_qk(gg + 1)) { alive = false; break; }
                            if (t + 2 == T) umma_commit(&st->q_free);
                        }
                        // the accumulator still holds the previous item's O until its epilogue has read it
                        if (t == 0 && kq >= 1 && !bar_wait(&st->o_free, (kq - 1) & 1, abort_flag, 11)) { alive = false; break; }
                        if (!mbar_wait2(&st->p_full[b2], (gg >> 1) & 1, &st->v_full[b2], (gg >> 1) & 1, abort_flag, 5)) { alive = false; break; }
                        tcgen05_fence_after();
                        const uint64_t v_desc = smem_desc_sw128(smem_u32(smem + kOffV + (s * 2 + b2) * kTileBytes));
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; kk++)   // 16 keys per MMA: 8 TMEM columns of P, 16 rows (2048 bytes) of V
                            umma_f16_ts(t_o, tbase + 64 * b2 + 8 * kk, v_desc + 128 * kk, idesc_pv, (t | kk) ? 1u : 0u);
                        umma_commit(&st->pv_done[b2]);
                        if (t + 1 == T) umma_commit(&st->o_final);
                    }
                    g += T;
                    kq++;
                }
                if (alive) mbar_arrive(&st->list_free[k & 1]);
            }
        }
        }
    } else {
        // ===== softmax + epilogue: one query row per thread =====
        asm volatile("setmaxnreg.inc.sync.aligned.u32 128;");
        const uint32_t s = warp >> 2, quarter = warp & 3;
        StreamState *st = &sh->st[s];
        const uint32_t r = quarter * 32 + lane;            // row inside the 128-query tile
        const uint32_t half = r >> 6;                      // which of the two block-rows
        const uint32_t lane_field = (quarter * 32) << 16;
        const uint32_t tbase = tmem + s * kStreamCols + lane_field;
        const uint32_t t_o = tbase + 96;         // S(even) = tbase, S(odd) = tbase + 32, P(even) = tbase, P(odd) = tbase + 64
        uint8_t *ostage = smem + kOffO + s * kQBytes;
        const float sl = p.scale_log2e;
        const uint64_t sl2 = pk64(sl, sl);
        uint32_t g = 0, kq = 0, n_epi = 0;
        bool alive = true;

        // The epilogue of an item: O / row sum -> the stream's staging tile -> (value producer) one TMA store per row pair,
        // 16 accumulator columns at a time.  (Running it behind the next item's first softmax step, so that nothing waits
        // for the item's last O product, was built and measured: slower.)
        auto epilogue = [&](bool has_data, uint32_t e_id, uint64_t l0, uint64_t l1) -> bool {
            const Item e_it = decode_item(e_id, p);
            const uint32_t e_pair = e_it.pair, e_b = e_it.b, e_h = e_it.h;
            const bool has_row1 = e_pair * 2 + 1 < p.nb;
            float inv = 0.f;
            if (has_data) {
                if (!bar_wait_warp(&st->o_final, kq & 1, abort_flag, 10)) return false;
                tcgen05_fence_after();
                float a0, a1, a2, a3;
                up64(l0, a0, a1);
                up64(l1, a2, a3);
                const float lsum = (a0 + a1) + (a2 + a3);
                inv = lsum > 0.f ? 1.f / lsum : 0.f;
            }
            // the previous store out of the staging tile has been read out of shared memory
            if (n_epi >= 1 && !bar_wait_warp(&st->stage_free, (n_epi - 1) & 1, abort_flag, 13)) return false;
            uint8_t *orow = ostage + r * 128;
            uint16_t *dst = (uint16_t *)p.O + ((size_t)e_b * L + (size_t)e_pair * 128 + r) * (size_t)p.o_pitch + (size_t)e_h * 64;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t oc[16];
                if (has_data) {
                    TMEM_LD_16((oc), t_o + c0);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int c = 0; c < 16; c++) oc[c] = 0u;      // a row pair without key blocks gives zeros (blocksparse.h:949-962)
                }
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 8; j++) w[j] = pack_pair<BF16>(__uint_as_float(oc[2 * j]) * inv, __uint_as_float(oc[2 * j + 1]) * inv);
                if (has_row1) {
                    // 16-byte chunk c of row r sits at chunk c ^ (r % 8): the tensor map's 128-byte swizzle
                    const int ch = c0 >> 3;
                    *(uint4 *)(orow + (((ch) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *(uint4 *)(orow + (((ch + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
                } else if (half == 0) {
                    // an odd number of block-rows: the last pair has 64 rows only, written directly
                    *(uint4 *)(dst + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                    *(uint4 *)(dst + c0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
            if (has_data) {
                tcgen05_fence_before();
                mbar_arrive(&st->o_free);              // the next item's first O product may overwrite the accumulator
                kq++;
            }
            if (has_row1) fence_proxy_async();
            if (r == 0) {
                st->store_x = (int32_t)(e_h * 64);
                st->store_y = has_row1 ? (int32_t)(e_b * L + e_pair * 128) : -1;
            }
            mbar_arrive(&st->stage_full);      // the value producer issues the store and hands the tile back
            n_epi++;
            return true;
        };

        uint32_t sr[64];                                   // this row of S(t), fp32 bits
        for (uint32_t k = 0; alive; k++) {
            const uint32_t id = item_id(k, s, p);
            if (id >= p.n_items) break;
            if (!bar_wait_warp(&st->list_ready[k & 1], (k >> 1) & 1, abort_flag, 8)) break;
            const uint32_t T = st->list_n[k & 1];
            const UEntry *list = lists + (s * 2 + (k & 1)) * kMaxU;
            const uint32_t item_h = HAS_MASK ? decode_item(id, p).h : 0u;
            float m_used = -INFINITY;
            uint64_t lacc0 = 0, lacc1 = 0;                 // four partial row sums (two packed pairs)
            for (uint32_t t = 0; t < T; t++) {
                const uint32_t gg = g + t, b2 = gg & 1;
                const uint32_t t_s = tbase + 32 * b2, t_p = tbase + 64 * b2;
                if (!bar_wait_warp(&st->qk_done[b2], (gg >> 1) & 1, abort_flag, 6)) { alive = false; break; }
                tcgen05_fence_after();
                TMEM_LD_32((sr), t_s);
                TMEM_LD_32((sr + 32), t_s + 32);
                tmem_wait_ld();
                tcgen05_fence_before();
                mbar_arrive(&st->s_free);                  // the buffer may be overwritten from here on
                const bool mine = (list[t].col_flags >> (30 + half)) & 1;     // the same for the whole warp
                if (mine) {
                    if (HAS_MASK) {
                        const uint64_t mw = p.mask[(size_t)item_h * p.mask_stride + (size_t)list[t].blk[half] * 64 + (r & 63)];
#pragma unroll
                        for (int c = 0; c < 64; c++)
                            if (!((mw >> c) & 1)) sr[c] = 0xff800000u;
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
                    const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl;
                    // the reference max moves only when a row max outgrows it by 2^8, so O is rescaled rarely
                    const bool grow = mx > m_used + kRescaleThreshold || (m_used == -INFINITY && mx > -INFINITY);
                    if (__any_sync(0xffffffffu, grow)) {
                        const bool fix_o = grow && m_used > -INFINITY;
                        float alpha = 1.f;
                        if (grow) {
                            alpha = fix_o ? ex2_approx(m_used - mx) : 0.f;
                            m_used = mx;
                            const uint64_t a2 = pk64(alpha, alpha);
                            lacc0 = fma2p(lacc0, a2, 0ull);
                            lacc1 = fma2p(lacc1, a2, 0ull);
                        }
                        if (t > 0 && __any_sync(0xffffffffu, fix_o)) {
                            // O must be complete before it is rescaled, and P(t) is only handed over afterwards
                            if (!bar_wait_warp(&st->pv_done[(gg - 1) & 1], ((gg - 1) >> 1) & 1, abort_flag, 7)) { alive = false; break; }
                            tcgen05_fence_after();
#pragma unroll
                            for (int c0 = 0; c0 < 64; c0 += 16) {
                                uint32_t oc[16];
                                TMEM_LD_16((oc), t_o + c0);
                                tmem_wait_ld();
#pragma unroll
                                for (int c = 0; c < 16; c++) oc[c] = __float_as_uint(__uint_as_float(oc[c]) * alpha);
                                TMEM_ST_16(t_o + c0, (oc));
                            }
                        }
                    }
                    const float neg_m = m_used > -INFINITY ? -m_used : 0.f;
                    const uint64_t nm2 = pk64(neg_m, neg_m);
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        uint32_t pk[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int c = hh * 32 + 2 * j;
                            const uint64_t x = fma2p(pk64(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), sl2, nm2);
                            float e0, e1;
                            if (POLY > 0 && (j % (POLY > 0 ? POLY : 1)) == (POLY > 0 ? POLY : 1) - 1) {
                                exp2_fma_pair(x, e0, e1);
                            } else {
                                float x0, x1;
                                up64(x, x0, x1);
                                e0 = ex2_approx(x0);
                                e1 = ex2_approx(x1);
                            }
                            if (j & 1) lacc1 = add2p(lacc1, pk64(e0, e1));
                            else lacc0 = add2p(lacc0, pk64(e0, e1));
                            pk[j] = pack_pair<BF16>(e0, e1);
                        }
                        TMEM_ST_16(t_p + hh * 16, (pk));
                    }
                } else {
                    uint32_t pk[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) pk[j] = 0u;
                    TMEM_ST_16(t_p, (pk));
                    TMEM_ST_16(t_p + 16, (pk));
                }
                tmem_wait_st();
                tcgen05_fence_before();
                mbar_arrive(&st->p_full[b2]);
            }
            if (!alive) break;
            g += T;
            if (!epilogue(T > 0, id, lacc0, lacc1)) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&st->list_free[k & 1]);
        }
    }

    // ---- teardown (also the way out after a timeout) ----
    tcgen05_fence_before();
    __syncthreads();
    if (sh->abort_flag) {
        // give loads and MMAs in flight a bounded time to land before shared memory and TMEM are released
        if (warp >= 12 && warp < 15 && lane == 0) {
            umma_commit(&sh->drained[warp - 12]);
            for (uint32_t i = 0; i < kWaitLimit && !mbar_try_wait(&sh->drained[warp - 12], 0); i++) {}
        }
        if (warp == 15 && lane == 0) {
            const uint64_t t0 = clock64();
            while (clock64() - t0 < 2000000ull) {}
        }
        __syncthreads();
    }
    if (hw_warp == 0) {
        __syncwarp();
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sh->tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace tc

bool tc_fused_attention_supported(int dtype, uint32_t bs, const AttnDims &p, float scale, uint32_t max_lut)
{
    // a row pair's union of key blocks must fit the kernel's list: known from max_lut, or from the width of the block grid
    const uint64_t longest = max_lut ? (2 * (uint64_t)max_lut < p.nb_b ? 2 * (uint64_t)max_lut : p.nb_b) : p.nb_b;
    return (dtype == SFB_BF16 || dtype == SFB_F16) && bs == 64 && p.d == 64 && scale > 0.f && p.nb_a == p.nb_b &&
           longest <= (uint64_t)tc::kMaxU && (uint64_t)p.B * p.nb_a * 64 < (1ull << 31) && p.nb_a < (1u << 30);
}

int tc_fused_attention(cudaStream_t s, const void *nn_lut, const void *q, const void *k, const void *v, void *o,
                       const void *mask, int dtype, const AttnDims &p, float scale)
{
    using namespace tc;
    const int is_bf16 = dtype == SFB_BF16;
    const uint64_t rows = (uint64_t)p.B * p.nb_a * 64;
    CUtensorMap qm, km, vm, om;
    if (make_map(&qm, q, rows, p.H, is_bf16, 128, p.in_pitch) || make_map(&km, k, rows, p.H, is_bf16, 64, p.in_pitch) ||
        make_map(&vm, v, rows, p.H, is_bf16, 64, p.in_pitch) || make_map(&om, o, rows, p.H, is_bf16, 128, p.out_pitch))
        return 1;
    const uint32_t npairs = (p.nb_a + 1) / 2;
    const uint64_t n_items = (uint64_t)npairs * p.B * p.H;
    SFB_REQUIRE(n_items < (1ull << 31), "sfb_fused_attention: too many row pairs for one launch");
    Params prm = {(const uint2 *)nn_lut, (const uint64_t *)mask, o, p.B, p.H, p.nb_a, npairs, (uint32_t)n_items, p.lut_stride,
                  p.mask_stride, (uint32_t)(p.out_pitch ? p.out_pitch : (uint64_t)p.H * 64), 0u, scale * 1.4426950408889634f};
    const int dev = current_device();
    const int sms = device_sm_count(dev);
    prm.cta_first = sms > 0 && n_items < 4ull * kStreams * (uint64_t)sms ? 1u : 0u;     // fewer than four rounds
    if (sms <= 0) return fail("sfb_fused_attention: cannot read the SM count");
    static DeviceOnce once;
    if (!once.done(dev)) {
        cudaError_t e = cudaFuncSetAttribute(fused_attention_tc_kernel<false, false, SFB_TC_POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fused_attention_tc_kernel<false, true, SFB_TC_POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fused_attention_tc_kernel<true, false, SFB_TC_POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fused_attention_tc_kernel<true, true, SFB_TC_POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return fail("sfb_fused_attention: cannot reserve %zu bytes of shared memory", kSmemBytes);
        once.mark(dev);
    }
    // one CTA per SM, three streams each; fewer CTAs only when there are fewer items than SMs (few rounds) or than streams
    const uint64_t want = prm.cta_first ? n_items : (n_items + kStreams - 1) / kStreams;
    const dim3 grid((unsigned)(want < (uint64_t)sms ? want : (uint64_t)sms));
    const dim3 block(kThreads);
    if (mask && is_bf16) launch_overlapped(fused_attention_tc_kernel<true, true, SFB_TC_POLY>, grid, block, kSmemBytes, s, qm, km, vm, om, prm);
    else if (mask) launch_overlapped(fused_attention_tc_kernel<true, false, SFB_TC_POLY>, grid, block, kSmemBytes, s, qm, km, vm, om, prm);
    else if (is_bf16) launch_overlapped(fused_attention_tc_kernel<false, true, SFB_TC_POLY>, grid, block, kSmemBytes, s, qm, km, vm, om, prm);
    else launch_overlapped(fused_attention_tc_kernel<false, false, SFB_TC_POLY>, grid, block, kSmemBytes, s, qm, km, vm, om, prm);
    return check_launch("sfb_fused_attention");
}

int tc_status_clear_fused()
{
    const uint32_t zero = 0;
    cudaError_t e = cudaMemcpyToSymbol(tc::g_status, &zero, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status_clear: %s", cudaGetErrorString(e));
    return 0;
}

int tc_status_fused(uint32_t *out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, tc::g_status, sizeof(uint32_t));
    if (e != cudaSuccess) return fail("sfb_device_status: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace sfb
