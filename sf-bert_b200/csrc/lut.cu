// Layout generation, layout -> LUT construction and element-mask packing on the device.
// Integer work only; results are bit-identical to the reference's host loops
// (stride_fusion_test.cu:48-227 and its siblings).
#include "common.cuh"

namespace sfb {

__device__ __forceinline__ uint64_t hash64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// one CTA per (head, row); threads stride over the columns
__global__ void layout_kernel(uint8_t *layout, uint32_t nb, int kind, uint32_t p0, uint32_t p1,
                              uint32_t p2, uint32_t p3, int causal, uint64_t seed)
{
    const uint32_t h = blockIdx.y, i = blockIdx.x;
    uint8_t *row = layout + ((size_t)h * nb + i) * nb;
    for (uint32_t j = threadIdx.x; j < nb; j += blockDim.x) {
        bool keep = false;
        switch (kind) {
        case SFB_LAYOUT_FULL:
            keep = true;
            break;
        case SFB_LAYOUT_FIXED: {
            // summary columns stride-(h+1) + n*stride, plus the row's own group of `stride` blocks
            int first = (int)p0 - (int)(h + 1);
            bool summary = p0 && (int)j >= first && (((int)j - first) % (int)p0) == 0;
            bool group = p0 && (j / p0) == (i / p0);
            keep = summary || group;
            break;
        }
        case SFB_LAYOUT_STRIDE:
            keep = (j <= i && j + p0 > i) || (p1 && (j % p1) == 0);
            break;
        case SFB_LAYOUT_SAWTOOTH: {
            uint32_t off = p0 ? i % p0 : 0;
            keep = (j + off >= i) && (j <= i);
            break;
        }
        case SFB_LAYOUT_LOCAL:
            keep = (j + p0 >= i) && (j <= i + p1);
            break;
        case SFB_LAYOUT_BIGBIRD: {
            uint32_t dist = i > j ? i - j : j - i;
            bool rg = (i < p1) || (i + p2 >= nb);
            bool cg = (j < p1) || (j + p2 >= nb);
            keep = dist <= p0 || rg || cg;
            break;
        }
        }
        if (causal && kind != SFB_LAYOUT_BIGBIRD && j > i) keep = false;
        row[j] = keep ? 1 : 0;
    }
    if (kind == SFB_LAYOUT_BIGBIRD) {
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t nrand = p3 > nb ? nb : p3;
            uint32_t drawn[64];
            uint32_t nd = 0;
            uint64_t ctr = 0;
            while (nd < nrand && nd < 64) {
                uint64_t key = (seed << 32) ^ ((uint64_t)h << 48) ^ ((uint64_t)i << 20) ^ ctr;
                uint32_t c = (uint32_t)(hash64(key) % nb);
                ctr++;
                bool dup = false;
                for (uint32_t t = 0; t < nd; t++) dup |= (drawn[t] == c);
                if (dup) continue;
                drawn[nd++] = c;
                row[c] = 1;
            }
        }
    }
}

__global__ void lut_count_kernel(const uint8_t *layout, uint32_t nb, uint32_t *head_blocks)
{
    __shared__ uint32_t total;
    if (threadIdx.x == 0) total = 0;
    __syncthreads();
    const uint8_t *lay = layout + (size_t)blockIdx.x * nb * nb;
    uint32_t cnt = 0;
    for (size_t e = threadIdx.x; e < (size_t)nb * nb; e += blockDim.x) cnt += lay[e] != 0;
    cnt = (uint32_t)__reduce_add_sync(0xffffffffu, cnt);
    if ((threadIdx.x & 31) == 0) atomicAdd(&total, cnt);
    __syncthreads();
    if (threadIdx.x == 0) head_blocks[blockIdx.x] = total;
}

// one CTA per head; dynamic smem: uint32 count[nb], offset[nb]
__global__ void lut_build_kernel(const uint8_t *layout, uint32_t nb, uint32_t blocks, uint2 *nt_lut,
                                 uint2 *nn_lut, uint2 *rblk_lut, uint32_t *nn_max, uint32_t *status)
{
    extern __shared__ uint32_t sh[];
    uint32_t *count = sh, *offset = sh + nb;
    __shared__ uint32_t total;
    const uint32_t h = blockIdx.x;
    const uint8_t *lay = layout + (size_t)h * nb * nb;

    for (uint32_t i = threadIdx.x; i < nb; i += blockDim.x) {
        uint32_t c = 0;
        for (uint32_t j = 0; j < nb; j++) c += lay[(size_t)i * nb + j] != 0;
        count[i] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t i = 0; i < nb; i++) {
            offset[i] = run;
            run += count[i];
        }
        total = run;
    }
    __syncthreads();
    if (total != blocks) {
        if (threadIdx.x == 0 && status) atomicExch(status, 1u);
        return;
    }
    uint2 *nt = nt_lut + (size_t)h * blocks;
    uint2 *nn = nn_lut + (size_t)h * (nb + blocks);
    uint2 *rb = rblk_lut ? rblk_lut + (size_t)h * blocks : nullptr;
    uint32_t mx = 0;
    for (uint32_t i = threadIdx.x; i < nb; i += blockDim.x) {
        uint32_t k = offset[i];
        nn[i] = make_uint2(nb + k, count[i]);          // header: offsets start at nb
        mx = max(mx, count[i]);
        for (uint32_t j = 0; j < nb; j++)
            if (lay[(size_t)i * nb + j]) {
                nt[k] = make_uint2(i, j);              // (row block, column block), scan order
                nn[nb + k] = make_uint2(k, j);         // (block id, column block)
                if (rb) rb[k] = make_uint2(k, i);      // (block id, row block)
                k++;
            }
    }
    if (nn_max) {
        mx = __reduce_max_sync(0xffffffffu, mx);
        if ((threadIdx.x & 31) == 0) atomicMax(nn_max, mx);
    }
}

// The column-major twin for the backward matmuls; one CTA of 256 threads per head; dynamic smem: uint32
// cursor[nb].  Block ids are positions in the row-major scan, so the rows are walked in order by the whole CTA
// (a ballot scan gives every kept block of the row its id) while each thread appends to its own columns.
__global__ void lut_build_tn_kernel(const uint8_t *layout, uint32_t nb, uint32_t blocks, uint2 *tn_lut, uint32_t *tn_max,
                                    uint32_t *status)
{
    extern __shared__ uint32_t cursor[];
    __shared__ uint32_t total, warp_sum[8];
    const uint32_t h = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint8_t *lay = layout + (size_t)h * nb * nb;

    for (uint32_t j = threadIdx.x; j < nb; j += blockDim.x) {
        uint32_t c = 0;
        for (uint32_t i = 0; i < nb; i++) c += lay[(size_t)i * nb + j] != 0;
        cursor[j] = c;
    }
    __syncthreads();
    uint2 *tn = tn_lut + (size_t)h * (nb + blocks);
    if (threadIdx.x == 0) {
        uint32_t run = 0, mx = 0;
        for (uint32_t j = 0; j < nb; j++) {
            const uint32_t c = cursor[j];
            if (run + c <= blocks) tn[j] = make_uint2(nb + run, c);   // header: offsets start at nb
            cursor[j] = nb + run;
            run += c;
            mx = max(mx, c);
        }
        total = run;
        if (run == blocks && tn_max) atomicMax(tn_max, mx);
    }
    __syncthreads();
    if (total != blocks) {
        if (threadIdx.x == 0 && status) atomicExch(status, 1u);
        return;
    }
    uint32_t id_base = 0;
    for (uint32_t i = 0; i < nb; i++)
        for (uint32_t c0 = 0; c0 < nb; c0 += blockDim.x) {
            const uint32_t j = c0 + threadIdx.x;
            const bool kept = j < nb && lay[(size_t)i * nb + j] != 0;
            const uint32_t votes = __ballot_sync(0xffffffffu, kept);
            if (lane == 0) warp_sum[wid] = __popc(votes);
            __syncthreads();
            uint32_t before = 0, all = 0;
            for (uint32_t w2 = 0; w2 < blockDim.x / 32; w2++) {
                before += w2 < wid ? warp_sum[w2] : 0;
                all += warp_sum[w2];
            }
            if (kept) tn[cursor[j]++] = make_uint2(id_base + before + __popc(votes & ((1u << lane) - 1u)), i);   // (block id, row block)
            id_base += all;
            __syncthreads();
        }
}

template <typename W>
__global__ void mask_pack_kernel(const uint2 *nt_lut, uint32_t blocks, uint32_t bs, int pred, uint32_t ctx,
                                 W *mask_np, W *mask_t)
{
    const uint32_t k = blockIdx.x, h = blockIdx.y, r = threadIdx.x;
    if (r >= bs) return;
    uint2 e = nt_lut[(size_t)h * blocks + k];
    W w = 0;
    for (uint32_t c = 0; c < bs; c++) {
        bool keep = true;
        if (pred == SFB_MASK_CAUSAL_DIAG) keep = e.x != e.y || r >= c;
        else if (pred == SFB_MASK_CAUSAL_ALL) keep = r >= c;
        else if (pred == SFB_MASK_LOCAL) {
            uint32_t row = e.x * bs + r, col = e.y * bs + c;
            keep = !(e.x == e.y && c > r) && !(col > row || col + ctx <= row);
        }
        w |= (W)(keep ? 1 : 0) << c;
    }
    if (mask_np) mask_np[((size_t)h * blocks + k) * bs + r] = w;
    if (mask_t) mask_t[((size_t)h * bs + r) * blocks + k] = w;
}

}  // namespace sfb

using namespace sfb;

extern "C" int sfb_layout_generate(sfb_stream_t stream, uint8_t *layout, uint32_t heads, uint32_t nb, int kind,
                                   uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3, int causal, uint64_t seed)
{
    SFB_REQUIRE(layout, "sfb_layout_generate: layout is NULL");
    SFB_REQUIRE(heads >= 1 && heads <= 65535 && nb >= 1, "sfb_layout_generate: bad heads=%u nb=%u", heads, nb);
    SFB_REQUIRE(kind >= SFB_LAYOUT_FULL && kind <= SFB_LAYOUT_BIGBIRD, "sfb_layout_generate: unknown kind %d", kind);
    SFB_REQUIRE(kind != SFB_LAYOUT_FIXED || p0 >= 1, "sfb_layout_generate: fixed layout needs stride >= 1");
    SFB_REQUIRE(kind != SFB_LAYOUT_BIGBIRD || p3 <= 64, "sfb_layout_generate: at most 64 random blocks per row");
    layout_kernel<<<dim3(nb, heads), 128, 0, as_stream(stream)>>>(layout, nb, kind, p0, p1, p2, p3, causal, seed);
    return check_launch("sfb_layout_generate");
}

extern "C" int sfb_lut_count(sfb_stream_t stream, const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t *head_blocks)
{
    SFB_REQUIRE(layout && head_blocks, "sfb_lut_count: NULL pointer");
    SFB_REQUIRE(heads >= 1 && nb >= 1, "sfb_lut_count: bad heads=%u nb=%u", heads, nb);
    lut_count_kernel<<<heads, 256, 0, as_stream(stream)>>>(layout, nb, head_blocks);
    return check_launch("sfb_lut_count");
}

extern "C" int sfb_lut_build(sfb_stream_t stream, const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t blocks,
                             void *nt_lut, void *nn_lut, void *rblk_lut, uint32_t *nn_max, uint32_t *status)
{
    SFB_REQUIRE(layout && nt_lut && nn_lut, "sfb_lut_build: NULL pointer");
    SFB_REQUIRE(heads >= 1 && nb >= 1 && nb <= 4096, "sfb_lut_build: bad heads=%u nb=%u (nb <= 4096)", heads, nb);
    cudaStream_t s = as_stream(stream);
    if (nn_max) cudaMemsetAsync(nn_max, 0, sizeof(uint32_t), s);
    if (status) cudaMemsetAsync(status, 0, sizeof(uint32_t), s);
    lut_build_kernel<<<heads, 256, 2 * nb * sizeof(uint32_t), s>>>(layout, nb, blocks, (uint2 *)nt_lut, (uint2 *)nn_lut,
                                                                 (uint2 *)rblk_lut, nn_max, status);
    return check_launch("sfb_lut_build");
}

extern "C" int sfb_lut_build_tn(sfb_stream_t stream, const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t blocks,
                                void *tn_lut, uint32_t *tn_max, uint32_t *status)
{
    SFB_REQUIRE(layout && tn_lut, "sfb_lut_build_tn: NULL pointer");
    SFB_REQUIRE(heads >= 1 && nb >= 1 && nb <= 4096, "sfb_lut_build_tn: bad heads=%u nb=%u (nb <= 4096)", heads, nb);
    cudaStream_t s = as_stream(stream);
    if (tn_max) cudaMemsetAsync(tn_max, 0, sizeof(uint32_t), s);
    if (status) cudaMemsetAsync(status, 0, sizeof(uint32_t), s);
    lut_build_tn_kernel<<<heads, 256, nb * sizeof(uint32_t), s>>>(layout, nb, blocks, (uint2 *)tn_lut, tn_max, status);
    return check_launch("sfb_lut_build_tn");
}

extern "C" int sfb_mask_pack(sfb_stream_t stream, const void *nt_lut, uint32_t heads, uint32_t blocks,
                             uint32_t block_size, int pred, uint32_t ctx, void *mask_np, void *mask_t)
{
    SFB_REQUIRE(nt_lut, "sfb_mask_pack: nt_lut is NULL");
    SFB_REQUIRE(block_size == 32 || block_size == 64, "sfb_mask_pack: block_size %u not supported (32 or 64)", block_size);
    SFB_REQUIRE(pred >= SFB_MASK_ALL && pred <= SFB_MASK_LOCAL, "sfb_mask_pack: unknown predicate %d", pred);
    SFB_REQUIRE(heads >= 1 && heads <= 65535, "sfb_mask_pack: bad heads=%u", heads);
    if (blocks == 0) { clear_error(); return 0; }
    dim3 grid(blocks, heads);
    if (block_size == 32)
        mask_pack_kernel<uint32_t><<<grid, 32, 0, as_stream(stream)>>>((const uint2 *)nt_lut, blocks, 32, pred, ctx,
                                                                      (uint32_t *)mask_np, (uint32_t *)mask_t);
    else
        mask_pack_kernel<uint64_t><<<grid, 64, 0, as_stream(stream)>>>((const uint2 *)nt_lut, blocks, 64, pred, ctx,
                                                                      (uint64_t *)mask_np, (uint64_t *)mask_t);
    return check_launch("sfb_mask_pack");
}

extern "C" void sfb_magicu64(uint32_t d, uint32_t *magic, uint32_t *shift)
{
    // smallest p with 2^p > nc * (d - 1 - (2^p - 1) mod d)   (blocksparse.h:1016-1043)
    if (d == 1 || d == 2 || d == 4 || d == 8) {
        *magic = 1;
        *shift = d == 1 ? 0 : d == 2 ? 1 : d == 4 ? 2 : 3;
        return;
    }
    *magic = 0;
    *shift = 0;
    if (d == 0) return;
    const uint32_t nbits = d == 3 ? 64 : 63;
    const uint64_t nmax = d == 3 ? 0xffffffffull : 0x7fffffffull;
    const uint64_t d64 = d;
    const uint64_t nc = ((nmax + 1ull) / d64) * d64 - 1ull;
    for (uint32_t p = 0; p < nbits; p++) {
        const uint64_t two_p = 1ull << p;
        const uint64_t rem = d64 - 1ull - (two_p - 1ull) % d64;
        if (two_p > nc * rem) {
            const uint32_t mg = (uint32_t)((two_p + rem) / d64);
            *magic = mg;
            *shift = mg == 1 ? p : p - 32;
            return;
        }
    }
}
