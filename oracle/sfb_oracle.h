/*
 * CPU oracle for the block-sparse attention path of SF-BERT.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing here is on the product path: the shipped
 * library never links, loads or calls this file.  It restates, in plain C, the
 * algorithms of the reference so that the CUDA kernels can be checked against
 * them, and it is timed as the CPU baseline.
 *
 * Parity pins (see tests/test_oracle_pins.py):
 *   - LUT / mask builders: bit-exact against the arrays that the reference's own
 *     test programs upload (captured by oracle/ref_capture, committed under
 *     tests/golden/).
 *   - attention math: against the reference's own CPU operators compiled from
 *     its headers (oracle/_ref/libsfb_ref.so) on the dense-causal layout, and
 *     against the all-ones known answer of the reference test programs.
 *
 * Every function cites the reference file:line it follows.
 */
#ifndef SFB_ORACLE_H
#define SFB_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- layouts: uint8 [heads][nb][nb], 1 = block kept ------------------------------ */

/* all blocks, or the lower triangle when causal (no_fusion_test.cu:47-63). */
void orc_layout_full(uint8_t *layout, uint32_t heads, uint32_t nb, int causal);

/* "fixed" pattern of fixed_fusion_test.cu:52-107: head h keeps the summary columns
 * j = stride-(h+1), +stride, ... of every row plus the row's own group of `stride`
 * blocks; causal != 0 applies the j<=i cut of lines 95-107. */
void orc_layout_fixed(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t stride, int causal);

/* strided pattern: band (i-band < j <= i) plus every `every`-th column; the causal
 * cut is optional.  band=4, every=8, causal=0 is the BERT-base stride config. */
void orc_layout_stride(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t band, uint32_t every, int causal);

/* the sawtooth rule of stride_fusion_test.cu:57-70: keep j in [i - i%chunks, i]. */
void orc_layout_stride_sawtooth(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t chunks);

/* sliding window i-left <= j <= i+right (local_fusion_test.cu:46-66 is left=extra_diag, right=0). */
void orc_layout_local(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t left, uint32_t right);

/* BigBird: window |i-j| <= window, the first g_first and last g_last block rows and
 * columns dense, plus nrand distinct random columns per row (big_bird_fusion_test.cu:50-99
 * has the structure; its rand() draw is replaced by the counter hash below so that host
 * and device agree bit for bit). */
void orc_layout_bigbird(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t window,
                        uint32_t g_first, uint32_t g_last, uint32_t nrand, uint64_t seed);

/* the counter-based generator used for the random BigBird columns and the synthetic data */
uint64_t orc_hash64(uint64_t x);

/* ---- layout -> LUT (stride_fusion_test.cu:77-134,215-223; fixed_fusion_test.cu:126-187) ---- */

/* blocks per head; returns 0 and sets *blocks when every head has the same count
 * (the reference's per-head stride is one number, blocksparse.h:442), else -1. */
int orc_lut_count(const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t *blocks);

/* nt_lut   [heads][blocks][2]      (x = row block, y = column block), row-major scan order
 * nn_lut   [heads][nb+blocks][2]   header (x = offset, y = count), entries (x = block id, y = column)
 * rblk_lut [heads][blocks][2]      (x = block id within the head, y = row block)
 * nn_max   largest row count over all heads */
int orc_lut_build(const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t blocks,
                  uint32_t *nt_lut, uint32_t *nn_lut, uint32_t *rblk_lut, uint32_t *nn_max);

/* tn_lut [heads][nb+blocks][2]: the same structure walked by block COLUMN -- header (x = offset, y = count),
 * entries (x = block id, y = row block), rows ascending (generate_tn_lut, ewops.h:675-701, which covers the
 * dense causal layout only).  tn_max = largest column count over all heads. */
int orc_lut_build_tn(const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t blocks,
                     uint32_t *tn_lut, uint32_t *tn_max);

/* ---- element masks (stride_fusion_test.cu:142-179, no_fusion_test.cu:124-165,
 *      local_fusion_test.cu:146-202) ------------------------------------------------ */
enum {
    ORC_MASK_ALL        = 0, /* every element kept */
    ORC_MASK_CAUSAL_DIAG = 1, /* r >= c on blocks with row == column                    */
    ORC_MASK_CAUSAL_ALL  = 2, /* r >= c on every block (stride_fusion_test.cu:149-160)  */
    ORC_MASK_LOCAL       = 3  /* col <= row && col + ctx > row in absolute positions     */
};
/* mask_np [heads][blocks][bs] words, bit c of word r = keep(r,c)  (fused kernels);
 * mask_t  [heads][bs][blocks] the transposed copy                 (unfused softmax).
 * Words are 32-bit for bs <= 32 and 64-bit for bs == 64 (blocksparse.h:688). Either may be NULL. */
void orc_mask_pack(const uint32_t *nt_lut, uint32_t heads, uint32_t blocks, uint32_t bs,
                   int pred, uint32_t ctx, void *mask_np, void *mask_t);

/* ---- arithmetic ---------------------------------------------------------------- */

/* fp32 -> bf16 bits with the reference's rounding (ew_op_gpu.h:241-253): add half an
 * ulp of the magnitude, truncate. */
uint16_t orc_to_bhalf(float v);
float    orc_from_bhalf(uint16_t v);

/* Block-sparse attention on [B,L,H,d] fp32 operands (transformer_attention_optimize.cu:719-748
 * fixes the layout).  Follows matmul.h:53-78 (scores, float accumulation over d in order),
 * ewops.h:64-98 (max of the unscaled kept scores, exp((x-max)*scale), divide by sum+eps)
 * and matmul.h:6-20 (P.V accumulated over keys in ascending order), with the causal
 * predicate k>=m replaced by the block layout and the element mask.
 *   mask_np   NULL = all kept; else as orc_mask_pack writes it
 *   s_out     NULL or [B][H][blocks][bs][bs] scores (unscaled)
 *   p_out     NULL or same shape, probabilities
 *   o_out     NULL or [B,L,H,d]
 *   eps       1e-6f reproduces ewops.h:93; 0 reproduces the GPU kernels (blocksparse.h:633)
 *   round_s_bf16 != 0 rounds the scores to bf16 before the softmax as the GPU path
 *   stores them (blocksparse.h:402). */
void orc_attention(const float *q, const float *k, const float *v,
                   const uint32_t *nt_lut, const uint32_t *nn_lut, const void *mask_np,
                   uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t d,
                   uint32_t blocks, uint32_t lut_heads, uint32_t mask_heads,
                   float scale, float eps, int round_s_bf16,
                   float *s_out, float *p_out, float *o_out);

/* y = LayerNorm(resid + (x + bias)) * gain + beta, also mean and rstd per row
 * (ewops.h:10-17 bias, ewops.h:296-301 residual add, layernorm.h:13-38: double sums,
 * var = E[x^2] - mean^2, eps 1e-5 inside the square root).  bias/resid may be NULL. */
void orc_bias_residual_layernorm(float *out, float *sum_out, float *mean, float *rstd,
                                 const float *x, const float *bias, const float *resid,
                                 const float *gain, const float *beta,
                                 uint32_t m, uint32_t hidden);

/* out = t * (1 / (exp(-1.702 t) + 1)), t = x + bias (ewops.h:10-17 then ewops.h:32-43: the exponential in
 * double of the float product, the reciprocal and the result in float).  bias may be NULL. */
void orc_bias_gelu(float *out, const float *x, const float *bias, uint32_t m, uint32_t n);

/* ---- backward of the block-sparse path (call order transformer_attention_optimize.cu:924-964) ---- */

/* dx = (dy - sum_row(dy*y)) * y * scale over the concatenated blocks of every query row; dy, y, dx are
 * [B][H][blocks][bs][bs] (bst_masked_softmax_grad, blocksparse.h:1045-1157; softmax_grad, ewops.h:103-122). */
void orc_softmax_grad(const float *dy, const float *y, const uint32_t *nn_lut,
                      uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t blocks,
                      uint32_t lut_heads, float scale, float *dx);

/* C = A^T . B walked by block column with the tn_lut (bst_sgemm_xn TN_OP, blocksparse.h:1005-1010;
 * multiheadmatmulTN, matmul.h:81-99): dV = P^T dO and dK = dS^T Q. */
void orc_spmm_tn(const float *a, const float *b, const uint32_t *tn_lut,
                 uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t d, uint32_t blocks,
                 uint32_t lut_heads, float *c);

/* C = A . B walked by block row with the nn_lut (bst_sgemm_xn NN_OP; multiheadmatmulNN, matmul.h:6-20):
 * O = P V and dQ = dS K. */
void orc_spmm_nn(const float *a, const float *b, const uint32_t *nn_lut,
                 uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t d, uint32_t blocks,
                 uint32_t lut_heads, float *c);

/* out = act(x . w + bias), x [m,k], w [k,n], out [m,n] row-major, act 0 = none, 1 = the reference's GELU
 * (matrixMulNNCPU matmul.h:101-118, bias ewops.h:10-17, gelu ewops.h:32-43).  bias may be NULL. */
void orc_linear(float *out, const float *x, const float *w, const float *bias, uint32_t m, uint32_t n, uint32_t k, int act);

/* out = act(x . wt^T + bias), wt [n,k] row-major (matrixMulNTCPU, matmul.h:121-132; the tied-embedding logits,
 * transformer_inference_part.cpp:241). */
void orc_linear_nt(float *out, const float *x, const float *wt, const float *bias, uint32_t m, uint32_t n, uint32_t k, int act);

/* out[b,l,:] = table[ids[b,l],:] + pos[l,:] (embedding.h:5-12, ewops.h:276-282); pos may be NULL; ids outside
 * [0, vocab) give zero rows. */
void orc_embedding(float *out, const float *table, const int32_t *ids, const float *pos, uint32_t batch, uint32_t seq_len,
                   uint32_t hidden, uint32_t vocab);

/* ---- element-sparse (CSR) attention, the alternative format the reference prototypes (cuda_kernels.h:976-1075,
 *      mask generators ewops.h:430-459) ---- */
void orc_csr_full_mask(int32_t *rowptr, int32_t *colidx, uint32_t L);
uint32_t orc_csr_from_layout(const uint8_t *layout, uint32_t nb, uint32_t bs, int32_t *rowptr, int32_t *colidx);
void orc_csr_attention(const float *q, const float *k, const float *v, const int32_t *rowptr, const int32_t *colidx,
                       uint32_t B, uint32_t H, uint32_t L, uint32_t d, float scale, float *o);

/* magic-number division constants (blocksparse.h:1016-1043) */
void orc_magicu64(uint32_t d, uint32_t *magic, uint32_t *shift);

/* deterministic N(0,1) data: element i of stream `seed` (Box-Muller on orc_hash64). */
void orc_fill_normal(float *dst, size_t n, uint64_t seed, float stddev);

int orc_num_threads(void);
/* overrides OMP_NUM_THREADS (launchers such as torchrun set it to 1 for their children) */
void orc_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
