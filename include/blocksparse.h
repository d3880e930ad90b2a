/*
 * Drop-in replacement for the reference's blocksparse.h (HeyHaoh/SF-Bert): the same free functions
 * with the same signatures, forwarding to the C ABI of libsfbert_b200.so (sfbert_b200.h).  Include
 * it where the reference header was included and link with -lsfbert_b200.
 *
 * Differences a caller can observe:
 *   - the functions return false (and sfb_last_error() has a message) on rejected arguments or a
 *     failed launch, where the reference always returned true (blocksparse.h:455);
 *   - block_size 64 works everywhere; the reference's matmuls silently did nothing unless
 *     block_size == 32 (blocksparse.h:448,996);
 *   - rows without blocks get probabilities / outputs of zero.
 */
#ifndef SFB_DROPIN_BLOCKSPARSE_H
#define SFB_DROPIN_BLOCKSPARSE_H

#include "gpu_types.h"
#include "sfbert_b200.h"

namespace sfb_dropin {
template <typename T> struct dtype_of;
template <> struct dtype_of<float> { static const int value = SFB_F32; };
template <> struct dtype_of<bhalf> { static const int value = SFB_BF16; };
template <> struct dtype_of<ehalf> { static const int value = SFB_F16; };
}  // namespace sfb_dropin

/* blocksparse.h:425-432 */
inline bool bst_sgemm_nt(CUstream stream, const uint2 *lut, const float *a, const float *b, bhalf *c,
                         uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a, uint ctx_blks_b,
                         uint head_dim, uint state_dim, uint lut_heads, uint lut_dim)
{
    return sfb_bst_sgemm_nt(stream, lut, a, b, c, SFB_F32, SFB_BF16, block_size, blocks, batch_dim, ctx_blks_a,
                            ctx_blks_b, head_dim, state_dim, lut_heads, lut_dim) == 0;
}

/* blocksparse.h:202-209 */
inline bool bst_sgemm_nt_float(CUstream stream, const uint2 *lut, const float *a, const float *b, float *c,
                               uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a, uint ctx_blks_b,
                               uint head_dim, uint state_dim, uint lut_heads, uint lut_dim)
{
    return sfb_bst_sgemm_nt(stream, lut, a, b, c, SFB_F32, SFB_F32, block_size, blocks, batch_dim, ctx_blks_a,
                            ctx_blks_b, head_dim, state_dim, lut_heads, lut_dim) == 0;
}

/* blocksparse.h:1420-1427: the reference's timing ablation without the global store; same result here */
inline bool bst_sgemm_nt_nosl(CUstream stream, const uint2 *lut, const float *a, const float *b, bhalf *c,
                              uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a, uint ctx_blks_b,
                              uint head_dim, uint state_dim, uint lut_heads, uint lut_dim)
{
    return bst_sgemm_nt(stream, lut, a, b, c, block_size, blocks, batch_dim, ctx_blks_a, ctx_blks_b, head_dim, state_dim,
                        lut_heads, lut_dim);
}

/* blocksparse.h:649-658; V is the reference's vector type of T and plays no role here.
 * mask is the transposed mask [block_size][blocks] per head, or NULL. */
template <typename T, typename V>
bool BlocksparseMaskedSoftmax(CUstream stream, const uint2 *lut, const uint *mask, const bhalf *x, T *y,
                              uint block_size, uint blocks, uint batch_dim, uint head_dim, uint ctx_blks,
                              uint lut_heads, uint lut_dim, uint max_lut, uint mask_heads, float scale)
{
    return sfb_masked_softmax(stream, lut, mask, x, y, SFB_BF16, sfb_dropin::dtype_of<T>::value, block_size, blocks,
                              batch_dim, head_dim, ctx_blks, lut_heads, lut_dim, max_lut, mask_heads, scale) == 0;
}

/* blocksparse.h:1645-1654 */
template <typename T, typename V>
bool BlocksparseMaskedSoftmax_nosl(CUstream stream, const uint2 *lut, const uint *mask, const bhalf *x, T *y,
                                   uint block_size, uint blocks, uint batch_dim, uint head_dim, uint ctx_blks,
                                   uint lut_heads, uint lut_dim, uint max_lut, uint mask_heads, float scale)
{
    return BlocksparseMaskedSoftmax<T, V>(stream, lut, mask, x, y, block_size, blocks, batch_dim, head_dim, ctx_blks,
                                          lut_heads, lut_dim, max_lut, mask_heads, scale);
}

/* blocksparse.h:965-972 (op = NN_OP with the nn_lut, or TN_OP with the tn_lut for the backward products) */
inline bool bst_sgemm_xn(CUstream stream, const uint2 *lut, const bhalf *a, const float *b, float *c,
                         uint block_size, uint blocks, uint batch_dim, uint ctx_blks_b, uint ctx_blks_c,
                         uint head_dim, uint state_dim, uint lut_heads, uint lut_dim, uint op, uint magic,
                         uint shift, uint max_lut)
{
    return sfb_bst_sgemm_xn(stream, lut, a, b, c, SFB_BF16, SFB_F32, block_size, blocks, batch_dim, ctx_blks_b,
                            ctx_blks_c, head_dim, state_dim, lut_heads, lut_dim, op, magic, shift, max_lut) == 0;
}

/* blocksparse.h:1164-1173; V is the reference's vector type of T and plays no role here.  lut is the nn_lut. */
template <typename T, typename V>
bool BlocksparseMaskedSoftmaxGrad(CUstream stream, const uint2 *lut, const T *dy, const T *y, T *dx, uint block_size,
                                  uint blocks, uint batch_dim, uint head_dim, uint ctx_blks, uint lut_heads,
                                  uint lut_dim, uint max_lut, float scale)
{
    return sfb_masked_softmax_grad(stream, lut, dy, y, dx, sfb_dropin::dtype_of<T>::value, block_size, blocks, batch_dim,
                                   head_dim, ctx_blks, lut_heads, lut_dim, max_lut, scale) == 0;
}

/* blocksparse.h:1016 */
inline void magicu64(uint d, uint &magic, uint &shift)
{
    uint32_t m = 0, s = 0;
    sfb_magicu64(d, &m, &s);
    magic = m;
    shift = s;
}

/* ---- Additions: 16-bit activations (no counterpart in the reference, whose Q, K, V, O are fp32) ---------------
 * The same operators with Q, K, V, O as bhalf (bf16) or ehalf (fp16): with block_size 64 and state_dim 64 they run on
 * the tensor cores.  QT is deduced from the pointers. */
template <typename QT>
inline bool bst_sgemm_nt(CUstream stream, const uint2 *lut, const QT *a, const QT *b, bhalf *c, uint block_size, uint blocks,
                         uint batch_dim, uint ctx_blks_a, uint ctx_blks_b, uint head_dim, uint state_dim, uint lut_heads,
                         uint lut_dim)
{
    return sfb_bst_sgemm_nt(stream, lut, a, b, c, sfb_dropin::dtype_of<QT>::value, SFB_BF16, block_size, blocks, batch_dim,
                            ctx_blks_a, ctx_blks_b, head_dim, state_dim, lut_heads, lut_dim) == 0;
}

template <typename PT, typename QT>
inline bool bst_sgemm_xn(CUstream stream, const uint2 *lut, const PT *a, const QT *b, QT *c, uint block_size, uint blocks,
                         uint batch_dim, uint ctx_blks_b, uint ctx_blks_c, uint head_dim, uint state_dim, uint lut_heads,
                         uint lut_dim, uint op, uint magic, uint shift, uint max_lut)
{
    return sfb_bst_sgemm_xn(stream, lut, a, b, c, sfb_dropin::dtype_of<PT>::value, sfb_dropin::dtype_of<QT>::value, block_size,
                            blocks, batch_dim, ctx_blks_b, ctx_blks_c, head_dim, state_dim, lut_heads, lut_dim, op, magic, shift,
                            max_lut) == 0;
}

/* One call for what the reference's test programs do inline (stride_fusion_test.cu:77-227): nt_lut, nn_lut, rblk_lut,
 * nn_max and, when pred >= 0, the element masks in both orders.  Any output pointer may be NULL. */
inline bool sfb_build_lut(CUstream stream, const uchar *layout, uint heads, uint ctx_blks, uint block_size, uint blocks,
                          uint2 *nt_lut, uint2 *nn_lut, uint2 *rblk_lut, uint *nn_max, uint *status, int pred, uint ctx,
                          void *mask_np, void *mask_t)
{
    if (sfb_lut_build(stream, layout, heads, ctx_blks, blocks, nt_lut, nn_lut, rblk_lut, nn_max, status) != 0) return false;
    if (pred >= 0 && (mask_np || mask_t))
        return sfb_mask_pack(stream, nt_lut, heads, blocks, block_size, pred, ctx, mask_np, mask_t) == 0;
    return true;
}

#endif
