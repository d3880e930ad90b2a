// Element-sparse (CSR) attention: the alternative sparse format the reference prototypes with one thread per query row
// (csr_sddmm / csr_softmax / csr_spmm and fused_attention, cuda_kernels.h:976-1075; mask generators ewops.h:430-459).
// One CSR pattern (rowptr [L+1], colidx [nnz], int32) is shared by every (batch, head).
//
//   csr_from_layout_kernel   block layout -> the CSR pattern of all elements of its kept blocks
//   csr_attention_*_kernel   O_i = sum_j softmax_j(q_i . k_j) v_j over the row's columns, one WARP per query row.
//                            In use: four lanes per key, each with a quarter of q_i and of the accumulators in
//                            registers (eight keys per warp and step, partial scores joined by two shuffles, K and V
//                            pieces requested together); every group of four runs its own online softmax, merged by
//                            shuffles at the end.  Measured on the BERT-base stride pattern: 5.7 ms, against 9.0 ms with
//                            two lanes per key, 17.7 ms with one (whole q_i per lane, 8 resident warps per SM), 6.8 ms with eight,
//                            7.0 ms with four and two keys per group and step.
// The format has no reuse of K/V between query rows (every row gathers its own keys through L2), which is why the
// block-sparse path exists; these kernels are the correct, coalesced-per-key version of the prototype, not a fast path.
#include "attn.cuh"

namespace sfb {

// one CTA per block-row; dynamic smem: uint32 cols[nb] (kept column blocks of this row)
__global__ void csr_from_layout_kernel(const uint8_t *__restrict__ layout, uint32_t nb, uint32_t bs, int32_t *__restrict__ rowptr,
                                       int32_t *__restrict__ colidx)
{
    extern __shared__ uint32_t cols[];
    __shared__ uint32_t before, mine;
    const uint32_t bi = blockIdx.x;
    if (threadIdx.x == 0) {
        uint32_t b = 0, m = 0;
        for (uint32_t r = 0; r < bi; r++)
            for (uint32_t j = 0; j < nb; j++) b += layout[(size_t)r * nb + j] != 0;
        for (uint32_t j = 0; j < nb; j++)
            if (layout[(size_t)bi * nb + j]) cols[m++] = j;
        before = b;
        mine = m;
    }
    __syncthreads();
    const size_t base = (size_t)before * bs * bs;           // nonzeros of all earlier block-rows
    const uint32_t per_row = mine * bs;
    for (uint32_t r = threadIdx.x; r < bs; r += blockDim.x) rowptr[(size_t)bi * bs + r + 1] = (int32_t)(base + (size_t)(r + 1) * per_row);
    if (bi == 0 && threadIdx.x == 0) rowptr[0] = 0;
    for (size_t e = threadIdx.x; e < (size_t)bs * per_row; e += blockDim.x) {
        const uint32_t within = (uint32_t)(e % per_row);
        colidx[base + e] = (int32_t)(cols[within / bs] * bs + within % bs);
    }
}

template <int DT> struct Row;   // loads D consecutive elements of a [.., d] row as floats, 16 bytes at a time
template <> struct Row<SFB_F32> {
    template <int D> static __device__ __forceinline__ void load(float (&v)[D], const void *p, size_t off)
    {
        const float4 *s = (const float4 *)((const float *)p + off);
#pragma unroll
        for (int i = 0; i < D / 4; i++) { const float4 t = __ldg(s + i); v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w; }
    }
};
template <> struct Row<SFB_BF16> {
    template <int D> static __device__ __forceinline__ void load(float (&v)[D], const void *p, size_t off)
    {
        const uint4 *s = (const uint4 *)((const uint16_t *)p + off);
#pragma unroll
        for (int i = 0; i < D / 8; i++) {
            const uint4 t = __ldg(s + i);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int j = 0; j < 4; j++) { v[8 * i + 2 * j] = __uint_as_float(w[j] << 16); v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
        }
    }
};
template <> struct Row<SFB_F16> {
    template <int D> static __device__ __forceinline__ void load(float (&v)[D], const void *p, size_t off)
    {
        const uint4 *s = (const uint4 *)((const uint16_t *)p + off);
#pragma unroll
        for (int i = 0; i < D / 8; i++) {
            const uint4 t = __ldg(s + i);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int j = 0; j < 4; j++) { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j])); v[8 * i + 2 * j] = f.x; v[8 * i + 2 * j + 1] = f.y; }
        }
    }
};

// D = head size rounded up to 32/64/128 by the dispatcher only when it is exactly that value
template <int DT, int D>
__global__ void __launch_bounds__(128) csr_attention_kernel(const int32_t *__restrict__ rowptr, const int32_t *__restrict__ colidx,
                                                           const void *__restrict__ Q, const void *__restrict__ K,
                                                           const void *__restrict__ V, void *__restrict__ O, uint32_t L, uint32_t H,
                                                           float scale_log2e, uint32_t *bad)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t i = blockIdx.x * 4 + (threadIdx.x >> 5), b = blockIdx.y, h = blockIdx.z;
    if (i >= L) return;
    const size_t HD = (size_t)H * D;
    const size_t row_off = ((size_t)b * L + i) * HD + (size_t)h * D;
    const int32_t lo = rowptr[i], hi = rowptr[i + 1];
    float q[D], acc[D];
    Row<DT>::template load<D>(q, Q, row_off);
#pragma unroll
    for (int x = 0; x < D; x++) acc[x] = 0.f;
    float m = -INFINITY, l = 0.f;          // m: running max of the unscaled scores of this lane's keys
    for (int32_t e = lo + (int32_t)lane; e < hi; e += 32) {
        const int32_t j = __ldg(colidx + e);
        if (j < 0 || (uint32_t)j >= L) {   // a column outside the sequence: counted, not read
            if (bad) atomicAdd(bad, 1u);
            continue;
        }
        const size_t key_off = ((size_t)b * L + (uint32_t)j) * HD + (size_t)h * D;
        float t[D];
        Row<DT>::template load<D>(t, K, key_off);
        float s = 0.f;
#pragma unroll
        for (int x = 0; x < D; x++) s = fmaf(q[x], t[x], s);
        if (s > m) {
            const float f = exp2f((m - s) * scale_log2e);   // 0 on the first key
            l *= f;
#pragma unroll
            for (int x = 0; x < D; x++) acc[x] *= f;
            m = s;
        }
        const float p = exp2f((s - m) * scale_log2e);
        l += p;
        Row<DT>::template load<D>(t, V, key_off);
#pragma unroll
        for (int x = 0; x < D; x++) acc[x] = fmaf(p, t[x], acc[x]);
    }
    // merge the 32 lanes' softmaxes
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float f = m > -INFINITY ? exp2f((m - M) * scale_log2e) : 0.f;
    l *= f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    const float inv = l > 0.f ? 1.f / (l + 1e-6f) : 0.f;   // the reference's denominator (ewops.h:93, cuda_kernels.h:1022)
    // transpose-reduce: after step k lane holds sums over lane groups; finally lane x owns elements x, x+32, ...
#pragma unroll
    for (int x = 0; x < D; x++) {
        float a = acc[x] * f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        acc[x] = a * inv;
    }
    // every lane holds the whole row now; each writes its share
#pragma unroll
    for (int x = 0; x < D; x++)
        if ((x & 31) == (int)lane) Elem<DT>::store(O, row_off + x, acc[x]);
}


// 16-byte pieces -> floats, by element type
template <int DT> struct Piece;
template <> struct Piece<SFB_F32> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(float *v, const uint4 &t)
    {
        v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y); v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
    }
};
template <> struct Piece<SFB_BF16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(float *v, const uint4 &t)
    {
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; j++) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
    }
};
template <> struct Piece<SFB_F16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(float *v, const uint4 &t)
    {
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; j++) { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j])); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    }
};

// The same attention with TWO lanes per key, each owning half of the head dimension: half the registers per lane
// (q and the accumulators are D/2 wide), so twice the warps are resident, and the key's K and V pieces are all
// requested before the first is used (one memory round trip per key instead of two).  The two lanes exchange their
// partial scores with one shuffle; both then carry the same running max and sum.
template <int DT, int D, int LPK>
__global__ void __launch_bounds__(128) csr_attention_split_kernel(const int32_t *__restrict__ rowptr, const int32_t *__restrict__ colidx,
                                                                 const void *__restrict__ Q, const void *__restrict__ K,
                                                                 const void *__restrict__ V, void *__restrict__ O, uint32_t L,
                                                                 uint32_t H, float scale_log2e, uint32_t *bad)
{
    constexpr int HD2 = D / LPK;                     // elements per lane
    constexpr int KPI = 32 / LPK;                    // keys per warp and step
    constexpr int NP = HD2 / Piece<DT>::N;           // 16-byte pieces per lane and operand
    constexpr int ESZ = 16 / Piece<DT>::N;
    const uint32_t lane = threadIdx.x & 31, hp = lane % LPK, pi = lane / LPK;
    const uint32_t i = blockIdx.x * 4 + (threadIdx.x >> 5), b = blockIdx.y, h = blockIdx.z;
    if (i >= L) return;
    const size_t HD = (size_t)H * D;
    const size_t row_off = ((size_t)b * L + i) * HD + (size_t)h * D + hp * HD2;
    const int32_t lo = rowptr[i], hi = rowptr[i + 1];
    float q[HD2], acc[HD2];
    {
        const uint4 *src = (const uint4 *)((const uint8_t *)Q + row_off * ESZ);
#pragma unroll
        for (int n = 0; n < NP; n++) Piece<DT>::unpack(q + n * Piece<DT>::N, __ldg(src + n));
    }
#pragma unroll
    for (int x = 0; x < HD2; x++) acc[x] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int32_t base = lo; base < hi; base += KPI) {          // the same trip count for every lane: the shuffle below is full-warp
        const int32_t e = base + (int32_t)pi;
        bool valid = e < hi;
        int32_t j = 0;
        if (valid) {
            j = __ldg(colidx + e);
            if (j < 0 || (uint32_t)j >= L) {                   // a column outside the sequence: counted once, not read
                if (bad && hp == 0) atomicAdd(bad, 1u);
                valid = false;
            }
        }
        uint4 kr[NP], vr[NP];
        if (valid) {
            const size_t key_off = (((size_t)b * L + (uint32_t)j) * HD + (size_t)h * D + hp * HD2) * ESZ;
            const uint4 *ks = (const uint4 *)((const uint8_t *)K + key_off), *vs = (const uint4 *)((const uint8_t *)V + key_off);
#pragma unroll
            for (int n = 0; n < NP; n++) kr[n] = __ldg(ks + n);
#pragma unroll
            for (int n = 0; n < NP; n++) vr[n] = __ldg(vs + n);
        }
        float part = 0.f;
        if (valid) {
#pragma unroll
            for (int n = 0; n < NP; n++) {
                float t[Piece<DT>::N];
                Piece<DT>::unpack(t, kr[n]);
#pragma unroll
                for (int x = 0; x < Piece<DT>::N; x++) part = fmaf(q[n * Piece<DT>::N + x], t[x], part);
            }
        }
        float sc = part;
#pragma unroll
        for (int o = 1; o < LPK; o <<= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
        if (valid) {
            if (sc > m) {
                const float f = exp2f((m - sc) * scale_log2e);   // 0 on the first key
                l *= f;
#pragma unroll
                for (int x = 0; x < HD2; x++) acc[x] *= f;
                m = sc;
            }
            const float p = exp2f((sc - m) * scale_log2e);
            l += p;
#pragma unroll
            for (int n = 0; n < NP; n++) {
                float t[Piece<DT>::N];
                Piece<DT>::unpack(t, vr[n]);
#pragma unroll
                for (int x = 0; x < Piece<DT>::N; x++) acc[n * Piece<DT>::N + x] = fmaf(p, t[x], acc[n * Piece<DT>::N + x]);
            }
        }
    }
    // merge the 16 pairs' softmaxes (the two lanes of a pair hold the same max and sum: offsets 16..2 only)
    float M = m;
#pragma unroll
    for (int o = 16; o >= LPK; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float f = m > -INFINITY ? exp2f((m - M) * scale_log2e) : 0.f;
    l *= f;
#pragma unroll
    for (int o = 16; o >= LPK; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    const float inv = l > 0.f ? 1.f / (l + 1e-6f) : 0.f;   // the reference's denominator (ewops.h:93, cuda_kernels.h:1022)
#pragma unroll
    for (int x = 0; x < HD2; x++) {
        float a = acc[x] * f;
#pragma unroll
        for (int o = 16; o >= LPK; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        // every lane of this parity holds the element now; pair x % 16 writes it
        if ((x % KPI) == (int)pi) Elem<DT>::store(O, row_off + x, a * inv);
    }
}

int csr_from_layout(cudaStream_t s, const uint8_t *layout, uint32_t nb, uint32_t bs, int32_t *rowptr, int32_t *colidx)
{
    csr_from_layout_kernel<<<nb, 256, nb * sizeof(uint32_t), s>>>(layout, nb, bs, rowptr, colidx);
    return check_launch("sfb_csr_from_layout");
}

int csr_attention(cudaStream_t s, const int32_t *rowptr, const int32_t *colidx, const void *q, const void *k, const void *v, void *o,
                  int dtype, uint32_t B, uint32_t L, uint32_t H, uint32_t d, float scale, uint32_t *bad)
{
    if (bad) cudaMemsetAsync(bad, 0, sizeof(uint32_t), s);
    const dim3 grid((L + 3) / 4, B, H);
    const float sl = scale * 1.4426950408889634f;
    const int lanes = 4;   // lanes per key; the one- and two-lane kernels are kept for comparison
#define CSR_LAUNCH(DTV, DV)                                                                                            \
    do {                                                                                                               \
        if (lanes == 4) csr_attention_split_kernel<DTV, DV, 4><<<grid, 128, 0, s>>>(rowptr, colidx, q, k, v, o, L, H, sl, bad); \
        else if (lanes == 2) csr_attention_split_kernel<DTV, DV, 2><<<grid, 128, 0, s>>>(rowptr, colidx, q, k, v, o, L, H, sl, bad); \
        else csr_attention_kernel<DTV, DV><<<grid, 128, 0, s>>>(rowptr, colidx, q, k, v, o, L, H, sl, bad);             \
    } while (0)
#define CSR_BY_D(DTV) if (d == 32) CSR_LAUNCH(DTV, 32); else if (d == 64) CSR_LAUNCH(DTV, 64); else CSR_LAUNCH(DTV, 128)
    if (dtype == SFB_F32) { CSR_BY_D(SFB_F32); } else if (dtype == SFB_BF16) { CSR_BY_D(SFB_BF16); } else { CSR_BY_D(SFB_F16); }
#undef CSR_BY_D
#undef CSR_LAUNCH
    return check_launch("sfb_csr_attention");
}

}  // namespace sfb

extern "C" int sfb_csr_from_layout(sfb_stream_t stream, const uint8_t *layout, uint32_t nb, uint32_t block_size, int32_t *rowptr,
                                   int32_t *colidx)
{
    SFB_REQUIRE(layout && rowptr && colidx, "sfb_csr_from_layout: NULL pointer");
    SFB_REQUIRE(nb >= 1 && nb <= 4096 && block_size >= 1 && block_size <= 128, "sfb_csr_from_layout: bad nb=%u block_size=%u", nb, block_size);
    SFB_REQUIRE((uint64_t)nb * nb * block_size * block_size < (1ull << 31), "sfb_csr_from_layout: the pattern may exceed 2^31 entries");
    return sfb::csr_from_layout((cudaStream_t)stream, layout, nb, block_size, rowptr, colidx);
}

extern "C" int sfb_csr_attention(sfb_stream_t stream, const int32_t *rowptr, const int32_t *colidx, const void *q, const void *k,
                                 const void *v, void *o, int dtype, uint32_t batch_dim, uint32_t seq_len, uint32_t head_dim,
                                 uint32_t state_dim, float scale, uint32_t *bad_columns)
{
    const char *who = "sfb_csr_attention";
    SFB_REQUIRE(rowptr && colidx && q && k && v && o, "%s: NULL pointer", who);
    SFB_REQUIRE(dtype == SFB_F32 || dtype == SFB_BF16 || dtype == SFB_F16, "%s: unknown dtype", who);
    SFB_REQUIRE(state_dim == 32 || state_dim == 64 || state_dim == 128, "%s: state_dim %u not supported (32, 64 or 128)", who, state_dim);
    SFB_REQUIRE(batch_dim >= 1 && batch_dim <= 65535 && head_dim >= 1 && head_dim <= 65535, "%s: bad batch_dim=%u head_dim=%u", who, batch_dim, head_dim);
    SFB_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) == 0, "%s: q, k, v, o must be 16-byte aligned", who);
    if (seq_len == 0) { sfb::clear_error(); return 0; }
    return sfb::csr_attention((cudaStream_t)stream, rowptr, colidx, q, k, v, o, dtype, batch_dim, seq_len, head_dim, state_dim, scale,
                              bad_columns);
}
