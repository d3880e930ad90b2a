/*
 * Drop-in replacement for the reference's fusion_blocksparse.h (HeyHaoh/SF-Bert): the fused
 * SDDMM + softmax entry points and the three-stage fusion, with the reference's signatures,
 * forwarding to the C ABI of libsfbert_b200.so.
 *
 * The reference's kernels exchange row maxima and sums between CTAs through the caller's
 * Max / Sum buffers and spin on the rblk_flag counters (fusion_blocksparse.h:224-366), which the
 * caller has to zero before every call.  Here a CTA owns a whole block-row, so those arguments
 * (c, rblk_flag, rblk_flag1, rblk_lut, Max, Sum, d_id_extractor) are accepted and never touched.
 * lut_dim is the nt_lut stride; the nn_lut stride is lut_dim + ctx_blks_a, as at
 * fusion_blocksparse.h:1245.  Mask is in mask_np order [blocks][block_size].
 */
#ifndef SFB_DROPIN_FUSION_BLOCKSPARSE_H
#define SFB_DROPIN_FUSION_BLOCKSPARSE_H

#include "blocksparse.h"

namespace sfb_dropin {
template <typename T>
inline bool fused_p(CUstream stream, const float *a, const float *b, const uint2 *nn_lut, const void *mask, T *y,
                    uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a, uint ctx_blks_b, uint head_dim,
                    uint state_dim, uint lut_heads, uint lut_dim, uint mask_heads, float scale)
{
    return sfb_fused_sddmm_softmax(stream, nn_lut, a, b, mask, y, SFB_F32, dtype_of<T>::value, block_size, blocks,
                                   batch_dim, ctx_blks_a, ctx_blks_b, head_dim, state_dim, lut_heads, lut_dim,
                                   mask_heads, scale) == 0;
}
}  // namespace sfb_dropin

/* fusion_blocksparse.h:400-416 */
template <typename T, typename V>
bool fusion_attention1(CUstream stream, const uint2 *nt_lut, const float *a, const float *b, bhalf *c,
                       const uint2 *nn_lut, int *rblk_flag, int *rblk_flag1, uint2 *rblk_lut, const uint *Mask,
                       float *Max, float *Sum, T *Y, uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a,
                       uint ctx_blks_b, uint head_dim, uint state_dim, uint lut_heads, uint lut_dim, uint mask_heads,
                       float scale)
{
    (void)nt_lut; (void)c; (void)rblk_flag; (void)rblk_flag1; (void)rblk_lut; (void)Max; (void)Sum;
    return sfb_dropin::fused_p<T>(stream, a, b, nn_lut, Mask, Y, block_size, blocks, batch_dim, ctx_blks_a, ctx_blks_b,
                                  head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale);
}

/* fusion_blocksparse.h:1212-1227 */
template <typename T, typename V>
bool fusion_attention2(CUstream stream, const uint2 *nt_lut, const float *a, const float *b, bhalf *c,
                       const uint2 *nn_lut, int *rblk_flag, int *rblk_flag1, const uint *Mask, float *Max, float *Sum,
                       T *Y, uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a, uint ctx_blks_b,
                       uint head_dim, uint state_dim, uint lut_heads, uint lut_dim, uint mask_heads, float scale)
{
    (void)nt_lut; (void)c; (void)rblk_flag; (void)rblk_flag1; (void)Max; (void)Sum;
    return sfb_dropin::fused_p<T>(stream, a, b, nn_lut, Mask, Y, block_size, blocks, batch_dim, ctx_blks_a, ctx_blks_b,
                                  head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale);
}

/* fusion_blocksparse.h:1636-1652 */
template <typename T, typename V>
bool fusion_attention_full(CUstream stream, const uint2 *nt_lut, const float *a, const float *b, bhalf *c,
                           const uint2 *nn_lut, int *rblk_flag, int *rblk_flag1, int *d_id_extractor, const uint *Mask,
                           float *Max, float *Sum, T *Y, uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a,
                           uint ctx_blks_b, uint head_dim, uint state_dim, uint lut_heads, uint lut_dim,
                           uint mask_heads, float scale)
{
    (void)nt_lut; (void)c; (void)rblk_flag; (void)rblk_flag1; (void)d_id_extractor; (void)Max; (void)Sum;
    return sfb_dropin::fused_p<T>(stream, a, b, nn_lut, Mask, Y, block_size, blocks, batch_dim, ctx_blks_a, ctx_blks_b,
                                  head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale);
}

/* fusion_blocksparse.h:2030-2045 */
template <typename T, typename V>
bool fusion_attention_local(CUstream stream, const uint2 *nt_lut, const float *a, const float *b, bhalf *c,
                            const uint2 *nn_lut, int *rblk_flag, int *rblk_flag1, const uint *Mask, float *Max,
                            float *Sum, T *Y, uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a,
                            uint ctx_blks_b, uint head_dim, uint state_dim, uint lut_heads, uint lut_dim,
                            uint mask_heads, float scale)
{
    (void)nt_lut; (void)c; (void)rblk_flag; (void)rblk_flag1; (void)Max; (void)Sum;
    return sfb_dropin::fused_p<T>(stream, a, b, nn_lut, Mask, Y, block_size, blocks, batch_dim, ctx_blks_a, ctx_blks_b,
                                  head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale);
}

/* fusion_blocksparse.h:2456-2471: the block_size 64 entry point (64-bit mask words) */
template <typename T, typename V>
bool fusion_attention2_64(CUstream stream, const uint2 *nt_lut, const float *a, const float *b, bhalf *c,
                          const uint2 *nn_lut, int *rblk_flag, int *rblk_flag1, const uint64 *Mask, float *Max,
                          float *Sum, T *Y, uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a,
                          uint ctx_blks_b, uint head_dim, uint state_dim, uint lut_heads, uint lut_dim,
                          uint mask_heads, float scale)
{
    (void)nt_lut; (void)c; (void)rblk_flag; (void)rblk_flag1; (void)Max; (void)Sum;
    return sfb_dropin::fused_p<T>(stream, a, b, nn_lut, Mask, Y, block_size, blocks, batch_dim, ctx_blks_a, ctx_blks_b,
                                  head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale);
}

/* fusion_blocksparse.h:2990-3007: SDDMM + softmax + SpMM; e is V, f receives O, Y is not written */
template <typename T, typename V>
bool fusion_attention(CUstream stream, const uint2 *nt_lut, const float *a, const float *b, bhalf *c,
                      const uint2 *nn_lut, int *rblk_flag, int *rblk_flag1, const uint *Mask, float *Max, float *Sum,
                      T *Y, float *e, float *f, uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a,
                      uint ctx_blks_b, uint ctx_blks_c, uint head_dim, uint state_dim, uint lut_heads, uint lut_dim,
                      uint mask_heads, float scale, uint max_lut)
{
    (void)nt_lut; (void)c; (void)rblk_flag; (void)rblk_flag1; (void)Max; (void)Sum; (void)Y; (void)ctx_blks_b; (void)ctx_blks_c;
    return sfb_fused_attention(stream, nn_lut, a, b, e, f, Mask, SFB_F32, block_size, blocks, batch_dim, ctx_blks_a,
                               head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale, max_lut) == 0;
}

/* ---- Additions: 16-bit activations (no counterpart in the reference) ------------------------------------------
 * fusion_attention with Q, K, V, O as bhalf (bf16) or ehalf (fp16); with block_size 64 and state_dim 64 this is the
 * tensor-core kernel.  Mask words are 64-bit for block_size 64 (as fusion_attention2_64 takes them). */
template <typename T, typename V, typename QT>
bool fusion_attention(CUstream stream, const uint2 *nt_lut, const QT *a, const QT *b, bhalf *c, const uint2 *nn_lut,
                      int *rblk_flag, int *rblk_flag1, const void *Mask, float *Max, float *Sum, T *Y, const QT *e, QT *f,
                      uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a, uint ctx_blks_b, uint ctx_blks_c,
                      uint head_dim, uint state_dim, uint lut_heads, uint lut_dim, uint mask_heads, float scale, uint max_lut)
{
    (void)nt_lut; (void)c; (void)rblk_flag; (void)rblk_flag1; (void)Max; (void)Sum; (void)Y; (void)ctx_blks_b; (void)ctx_blks_c;
    return sfb_fused_attention(stream, nn_lut, a, b, e, f, Mask, sfb_dropin::dtype_of<QT>::value, block_size, blocks, batch_dim,
                               ctx_blks_a, head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale, max_lut) == 0;
}

#endif
