/*
 * libsfbert_b200.so -- C ABI of the B200 (sm_100a) block-sparse attention path.
 *
 * Every entry point takes plain pointers and sizes.  Unless a comment says otherwise all
 * pointers are DEVICE pointers owned by the caller, nothing is allocated or freed, the
 * work is queued on `stream` (a cudaStream_t / CUstream) and the call returns without
 * synchronising.  Return value: 0 on success, non-zero on a rejected argument or a failed
 * launch; sfb_last_error() then holds a message (thread local).  No entry point has a CPU
 * fallback.
 *
 * Each declaration names the interface of the reference (HeyHaoh/SF-Bert) it replaces.
 * Parameter names follow the reference, including its misleading ones:
 *   head_dim  = number of heads H          state_dim = size of one head d
 *   batch_dim = B                          ctx_blks_* = sequence length / block_size
 *   blocks    = non-zero blocks of ONE head's layout
 *   lut_heads = 1 (one LUT for all heads) or H;  lut_dim = per-head LUT stride in uint2
 * Tensors Q, K, V, O are [B, L, H, d] (no head transpose, transformer_attention_optimize.cu:719-748);
 * S and P are [B, H, blocks, block_size, block_size], row-major inside a block.
 */
#ifndef SFBERT_B200_H
#define SFBERT_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *sfb_stream_t;

/* element types of operand buffers */
enum { SFB_F32 = 0, SFB_BF16 = 1, SFB_F16 = 2 };

/* layout kinds for sfb_layout_generate */
enum {
    SFB_LAYOUT_FULL = 0,     /* p0 unused                                   (no_fusion_test.cu:47-63)       */
    SFB_LAYOUT_FIXED = 1,    /* p0 = stride                                 (fixed_fusion_test.cu:52-107)   */
    SFB_LAYOUT_STRIDE = 2,   /* p0 = band, p1 = every                       (BERT-base stride config)       */
    SFB_LAYOUT_SAWTOOTH = 3, /* p0 = chunks                                 (stride_fusion_test.cu:57-70)   */
    SFB_LAYOUT_LOCAL = 4,    /* p0 = left, p1 = right                       (local_fusion_test.cu:46-66)    */
    SFB_LAYOUT_BIGBIRD = 5   /* p0 = window, p1 = g_first, p2 = g_last, p3 = nrand (big_bird_fusion_test.cu:50-99) */
};

/* element-mask predicates for sfb_mask_pack */
enum { SFB_MASK_ALL = 0, SFB_MASK_CAUSAL_DIAG = 1, SFB_MASK_CAUSAL_ALL = 2, SFB_MASK_LOCAL = 3 };

/* activations of sfb_linear */
enum { SFB_ACT_NONE = 0, SFB_ACT_GELU = 1 };

/* block-sparse matmul variants (gpu_types.h:135-137) */
enum { SFB_NT_OP = 0, SFB_NN_OP = 1, SFB_TN_OP = 2 };

/* message of the last failed call on this thread ("" if none) */
const char *sfb_last_error(void);
int sfb_version(void);

/* ---- layout -> LUT ------------------------------------------------------------------ */

/* Writes a block layout, uint8 [heads][nb][nb] (1 = kept), into device memory.
 * Replaces the inline layout loops of the reference test programs (see the enum). */
int sfb_layout_generate(sfb_stream_t stream, uint8_t *layout, uint32_t heads, uint32_t nb,
                        int kind, uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3,
                        int causal, uint64_t seed);

/* Counts the kept blocks: head_blocks[h] (device, uint32 [heads]).  The caller reads it
 * back to size the LUTs; every head must have the same count (blocksparse.h:442 has one
 * per-head stride).  Replaces stride_fusion_test.cu:57-70 (the counting half). */
int sfb_lut_count(sfb_stream_t stream, const uint8_t *layout, uint32_t heads, uint32_t nb,
                  uint32_t *head_blocks);

/* Builds, in device memory,
 *   nt_lut   uint2 [heads][blocks]       (x = row block, y = column block), row-major scan order
 *   nn_lut   uint2 [heads][nb + blocks]  header (x = offset, y = count), then (x = block id, y = column)
 *   rblk_lut uint2 [heads][blocks]       (x = block id, y = row block)            (may be NULL)
 *   nn_max   uint32 [1]                  longest row over all heads               (may be NULL)
 * Replaces stride_fusion_test.cu:77-134,215-223 / fixed_fusion_test.cu:126-187,296-312.
 * A head whose count differs from `blocks` makes status[0] non-zero (uint32 [1], may be NULL)
 * and that head's LUTs are left untouched. */
int sfb_lut_build(sfb_stream_t stream, const uint8_t *layout, uint32_t heads, uint32_t nb,
                  uint32_t blocks, void *nt_lut, void *nn_lut, void *rblk_lut,
                  uint32_t *nn_max, uint32_t *status);

/* Builds, in device memory, the LUT the backward matmuls walk (sfb_bst_sgemm_xn with SFB_TN_OP):
 *   tn_lut   uint2 [heads][nb + blocks]  header per block COLUMN (x = offset, y = count), then
 *                                        (x = block id, y = row block), rows ascending
 *   tn_max   uint32 [1]                  longest column over all heads            (may be NULL)
 * Block ids are those of sfb_lut_build (row-major scan).  Replaces generate_tn_lut (ewops.h:675-701,
 * inlined in test.cu:139-170), which the reference has for the dense causal layout only.  status as in
 * sfb_lut_build. */
int sfb_lut_build_tn(sfb_stream_t stream, const uint8_t *layout, uint32_t heads, uint32_t nb,
                     uint32_t blocks, void *tn_lut, uint32_t *tn_max, uint32_t *status);

/* Packs element masks: bit c of word r of block k = keep(r, c).
 *   mask_np [heads][blocks][block_size]  (the fused kernels' order, fusion_blocksparse.h:690)
 *   mask_t  [heads][block_size][blocks]  (the unfused softmax's order, blocksparse.h:482)
 * Words are uint32 for block_size 32 and uint64 for 64 (blocksparse.h:688).  Either may be NULL.
 * Replaces stride_fusion_test.cu:142-187, no_fusion_test.cu:124-171, local_fusion_test.cu:146-202. */
int sfb_mask_pack(sfb_stream_t stream, const void *nt_lut, uint32_t heads, uint32_t blocks,
                  uint32_t block_size, int pred, uint32_t ctx, void *mask_np, void *mask_t);

/* Host-only: magic-number division constants.  Replaces magicu64 (blocksparse.h:1016-1043). */
void sfb_magicu64(uint32_t d, uint32_t *magic, uint32_t *shift);

/* ---- unfused operators ---------------------------------------------------------------- */

/* SDDMM: S[b,h,k] = Q[b, rows of block x, h, :] . K[b, rows of block y, h, :]^T for (x,y) = lut[k],
 * unscaled.  Replaces bst_sgemm_nt (blocksparse.h:425-456, openai_blocksparse.h:202-233; c_dtype
 * SFB_BF16) and bst_sgemm_nt_float (blocksparse.h:202-233; c_dtype SFB_F32).  ab_dtype is the type
 * of a and b (the reference has SFB_F32 only).  block_size 32 or 64. */
int sfb_bst_sgemm_nt(sfb_stream_t stream, const void *lut, const void *a, const void *b, void *c,
                     int ab_dtype, int c_dtype, uint32_t block_size, uint32_t blocks,
                     uint32_t batch_dim, uint32_t ctx_blks_a, uint32_t ctx_blks_b,
                     uint32_t head_dim, uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim);

/* P = softmax over the concatenated blocks of every query row of scale*S, with the optional
 * transposed bit mask (NULL = keep all).  lut is the nn_lut; lut_dim its per-head stride
 * (blocks + ctx_blks).  x is bf16 (x_dtype SFB_BF16) as in the reference, or SFB_F32.
 * Replaces BlocksparseMaskedSoftmax<T,V> (blocksparse.h:649-722). */
int sfb_masked_softmax(sfb_stream_t stream, const void *lut, const void *mask, const void *x, void *y,
                       int x_dtype, int y_dtype, uint32_t block_size, uint32_t blocks,
                       uint32_t batch_dim, uint32_t head_dim, uint32_t ctx_blks,
                       uint32_t lut_heads, uint32_t lut_dim, uint32_t max_lut,
                       uint32_t mask_heads, float scale);

/* SpMM.  op = SFB_NN_OP (forward, lut = nn_lut): O[b, rows of block-row i, h, :] = sum over the row's
 * blocks k of P[b,h,k] . V[b, rows of column block of k, h, :]; also dQ = dS K.
 * op = SFB_TN_OP (backward, lut = tn_lut of sfb_lut_build_tn): C[b, rows of block COLUMN j, h, :] = sum over
 * the column's blocks k of A[b,h,k]^T . B[b, rows of row block of k, h, :]: dV = P^T dO, dK = dS^T Q
 * (call sites transformer_attention_optimize.cu:924,954,964).  magic/shift are accepted and ignored.
 * Replaces bst_sgemm_xn (blocksparse.h:965-1014). */
int sfb_bst_sgemm_xn(sfb_stream_t stream, const void *lut, const void *a, const void *b, void *c,
                     int a_dtype, int bc_dtype, uint32_t block_size, uint32_t blocks,
                     uint32_t batch_dim, uint32_t ctx_blks_b, uint32_t ctx_blks_c,
                     uint32_t head_dim, uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim,
                     uint32_t op, uint32_t magic, uint32_t shift, uint32_t max_lut);

/* dx = (dy - sum over the query row of dy*y) * y * scale on the concatenated blocks of every query row;
 * dy, y and dx are [B, H, blocks, block_size, block_size] of one type (the reference has bf16 and fp32).
 * lut is the nn_lut, lut_dim its per-head stride; max_lut as for sfb_masked_softmax (0 = unknown).
 * Replaces BlocksparseMaskedSoftmaxGrad<T,V> (blocksparse.h:1164-1227; call site
 * transformer_attention_optimize.cu:944); CPU twin softmax_grad, ewops.h:103-122. */
int sfb_masked_softmax_grad(sfb_stream_t stream, const void *lut, const void *dy, const void *y, void *dx,
                            int dtype, uint32_t block_size, uint32_t blocks, uint32_t batch_dim,
                            uint32_t head_dim, uint32_t ctx_blks, uint32_t lut_heads, uint32_t lut_dim,
                            uint32_t max_lut, float scale);

/* out[row] = sum over the row of a * b, rows of d elements (d a multiple of 8) of type dtype, out fp32.
 * delta = sfb_rowdot(dO, O) over the B*L*H head rows is the row constant of the softmax gradient below.
 * No counterpart in the reference. */
int sfb_rowdot(sfb_stream_t stream, float *out, const void *a, const void *b, uint64_t rows, uint32_t d, int dtype);

/* dS = P * (dO . V^T - delta) * scale on the kept blocks in ONE launch, in place of sfb_bst_sgemm_nt(dO, V) followed by
 * sfb_masked_softmax_grad (transformer_attention_optimize.cu:934-944): delta [B, L, H] (fp32, sfb_rowdot(dO, O))
 * equals the sum over a query row of dP * P that the unfused gradient reduces first, so no pass over the row is
 * needed and dP is never written.  lut is the nt_lut; dO, V are [B, L, H, d]; P and dS are [B, H, blocks, 64, 64];
 * all four of type dtype (SFB_BF16 or SFB_F16); block_size 64, state_dim 64.  No counterpart in the reference. */
int sfb_fused_sddmm_softmax_grad(sfb_stream_t stream, const void *nt_lut, const void *dout, const void *v,
                                 const void *p_blocks, const float *delta, void *ds, int dtype, uint32_t block_size,
                                 uint32_t blocks, uint32_t batch_dim, uint32_t ctx_blks, uint32_t head_dim,
                                 uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim, float scale);

/* ---- fused, synchronisation-free operators -------------------------------------------- */

/* SDDMM + masked softmax in one launch: each CTA owns a block-row, so there are no flags, no
 * Max/Sum scratch and no waiting between CTAs.  mask is mask_np order (NULL = keep all);
 * lut_dim is the nt_lut stride (`blocks`), the nn_lut stride is lut_dim + ctx_blks_a as in
 * fusion_blocksparse.h:1245.  Replaces fusion_attention1 (fusion_blocksparse.h:400-455),
 * fusion_attention2 (:1212-1268), fusion_attention_full (:1636-1694), fusion_attention_local
 * (:2030-2086) and fusion_attention2_64 (:2456-2514). */
int sfb_fused_sddmm_softmax(sfb_stream_t stream, const void *nn_lut, const void *a, const void *b,
                            const void *mask, void *y, int ab_dtype, int y_dtype,
                            uint32_t block_size, uint32_t blocks, uint32_t batch_dim,
                            uint32_t ctx_blks_a, uint32_t ctx_blks_b, uint32_t head_dim,
                            uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim,
                            uint32_t mask_heads, float scale);

/* SDDMM + softmax + SpMM in one launch: O = softmax(scale * Q K^T on the kept blocks) V with S
 * and P never leaving the chip.  dtype is the type of q, k, v and o.  Replaces fusion_attention
 * (fusion_blocksparse.h:2990-3050), whose kernel the reference left unfinished. */
int sfb_fused_attention(sfb_stream_t stream, const void *nn_lut, const void *q, const void *k,
                        const void *v, void *o, const void *mask, int dtype,
                        uint32_t block_size, uint32_t blocks, uint32_t batch_dim,
                        uint32_t ctx_blks, uint32_t head_dim, uint32_t state_dim,
                        uint32_t lut_heads, uint32_t lut_dim, uint32_t mask_heads,
                        float scale, uint32_t max_lut);

/* The same operator on a SLICE of the heads of wider tensors, in place: q, k, v point at the slice's first head inside
 * [B, L, H_total, d] tensors whose rows (one sequence position) lie in_pitch elements apart (H_total * d), o likewise
 * with out_pitch; head_dim counts the heads of the slice, lut_heads / mask_heads are 1 or that count.  0 for a pitch
 * means head_dim * state_dim, i.e. sfb_fused_attention.  This is how one GPU of several takes its share of the
 * (batch, head) pairs without packing them first: the reference addresses a pair by offsets off the tensor base with
 * the full row stride (blocksparse.h:250-266), but derives that stride from head_dim (blocksparse.h:434-437), so its
 * own entry points cannot be handed a slice.  The tensor cores are used when the pitches are multiples of 8 elements. */
int sfb_fused_attention_slice(sfb_stream_t stream, const void *nn_lut, const void *q, const void *k,
                              const void *v, void *o, const void *mask, int dtype,
                              uint32_t block_size, uint32_t blocks, uint32_t batch_dim,
                              uint32_t ctx_blks, uint32_t head_dim, uint32_t state_dim,
                              uint32_t lut_heads, uint32_t lut_dim, uint32_t mask_heads,
                              float scale, uint32_t max_lut, uint64_t in_pitch, uint64_t out_pitch);

/* Synchronises with the device and reads the library's status word into *status (HOST pointer):
 * 0 while no kernel has given up on a bounded wait, otherwise (code << 24 | CTA index) of the
 * first one that did.  Code 9 is not a wait: a row pair of sfb_fused_attention touched more key blocks than the
 * tensor-core kernel's list holds (256) although max_lut promised otherwise; that pair's output rows are written
 * as zeros, all other rows are correct.  No counterpart in the reference, whose fused kernels spin without a
 * bound (fusion_blocksparse.h:246-289). */
int sfb_device_status(uint32_t *status);

/* Synchronises with the device and sets the status word back to 0 (it keeps the first code it was given until then). */
int sfb_device_status_clear(void);

/* ---- epilogue -------------------------------------------------------------------------- */

/* out = LayerNorm(resid + (x + bias)) * gain + beta over rows of `hidden` elements; also writes
 * the pre-norm sum (sum_out), mean and rstd when those are not NULL.  bias and resid may be NULL.
 * dtype is the type of x, resid, out and sum_out; bias, gain, beta, mean, rstd are fp32.
 * out (or sum_out) may be x or resid: a row is read completely before it is written.
 * Replaces tensor_add_vector_gpu + tensor_add_tensor_gpu + layernorm_gpu
 * (cuda_kernels.h:459-469, :449-457, :334-372; call site transformer_attention_optimize.cu:763-771). */
int sfb_bias_residual_layernorm(sfb_stream_t stream, void *out, void *sum_out, float *mean,
                                float *rstd, const void *x, const float *bias, const void *resid,
                                const float *gain, const float *beta, uint32_t m, uint32_t hidden,
                                int dtype);

/* out = t * sigmoid(1.702 t), t = x + bias, over m rows of n elements (bias fp32 [n], may be NULL; out may
 * alias x).  Replaces tensor_add_vector_gpu_2048 + gelu_gpu_v2 (cuda_kernels.h:471-489, :561-581; call site
 * transformer_attention_optimize.cu:781-785); CPU twin gelu, ewops.h:32-43. */
int sfb_bias_gelu(sfb_stream_t stream, void *out, const void *x, const float *bias, uint32_t m,
                  uint32_t n, int dtype);

/* ---- dense projections around the attention --------------------------------------------- */

/* out[m, n] = act(x[m, k] . w[k, n] + bias[n]) on the tensor cores: x, w, out row-major 16-bit (dtype SFB_BF16 or
 * SFB_F16), fp32 accumulation, bias fp32 [n] (may be NULL), act SFB_ACT_NONE or SFB_ACT_GELU (t * sigmoid(1.702 t),
 * gelu_gpu_v2).  n must be a multiple of 16, k of 8.  w is laid out as the reference keeps its weights: its
 * cublasSgemm(OP_N, OP_N, n, m, k, W, n, X, k, C, n) calls are out = x . w with w row-major [k, n].
 * Replaces cublasSgemm + tensor_add_vector_gpu (transformer_attention_optimize.cu:693-716, 755-763) and
 * cublasSgemm + tensor_add_vector_gpu_2048 + gelu_gpu_v2 (:773-785) for 16-bit operands; fp32 products are
 * rejected (they stay with the GEMM library: tensor-core arithmetic cannot meet fp32 parity). */
int sfb_linear(sfb_stream_t stream, void *out, const void *x, const void *w, const float *bias, uint32_t m,
               uint32_t n, uint32_t k, int dtype, int act);

/* out[m, n] = act(x[m, k] . wt[n, k]^T + bias[n]): the same kernel with the weights stored row-major [n, k] -- the
 * logits over the tied embedding table, cblas_sgemm(RowMajor, NoTrans, Trans, m, vocab, n, x, n, x_embed, n, logits, vocab)
 * (transformer_inference_part.cpp:241); CPU twin matrixMulNTCPU, matmul.h:121-132.  n must be a multiple of 16 (pad the
 * vocabulary), k of 8. */
int sfb_linear_nt(sfb_stream_t stream, void *out, const void *x, const void *wt, const float *bias, uint32_t m,
                  uint32_t n, uint32_t k, int dtype, int act);

/* out[b, l, :] = table[ids[b, l], :] + pos[l, :]: the front of the encoder stack.  table [vocab, hidden], pos
 * [seq_len, hidden] (may be NULL) and out [batch, seq_len, hidden] are of type dtype; ids are int32 in device memory.
 * An id outside [0, vocab) gives a row of zeros and is counted in *bad_ids (device uint32, may be NULL) instead of
 * being read out of bounds.  hidden must be a multiple of 8 (4 for fp32).
 * Replaces embedding_lookup_gpu + tensor_add_matrix_gpu (cuda_kernels.h:210-221, 526-535); CPU twins embedding_lookup
 * (embedding.h:5-12) and tensor_add_matrix (ewops.h:276-282); call site transformer_inference_part.cpp:201-209. */
int sfb_embedding(sfb_stream_t stream, void *out, const void *table, const int32_t *ids, const void *pos,
                  uint32_t batch, uint32_t seq_len, uint32_t hidden, uint32_t vocab, int dtype, uint32_t *bad_ids);

/* ---- element-sparse (CSR) attention: the alternative format the reference prototypes ------------------ */

/* The CSR pattern of a block layout (ONE head, uint8 [nb][nb]): every element of every kept block, columns ascending.
 * rowptr int32 [nb*block_size + 1], colidx int32 [blocks*block_size^2], both in device memory.  The host-side
 * generators it stands beside: generate_csr_full_mask / generate_csr_fixed_mask (ewops.h:430-443, 616-659). */
int sfb_csr_from_layout(sfb_stream_t stream, const uint8_t *layout, uint32_t nb, uint32_t block_size, int32_t *rowptr,
                        int32_t *colidx);

/* O[b,i,h,:] = sum over the columns j of row i of softmax_j(scale * q_i . k_j) v_j, one CSR pattern (rowptr [seq_len+1],
 * colidx [nnz]) for every (batch, head); q, k, v, o are [B, L, H, d] of type dtype, d = 32, 64 or 128.  Rows without
 * entries give zeros; a column outside [0, seq_len) is skipped and counted in *bad_columns (device uint32, may be NULL).
 * Replaces csr_sddmm + csr_softmax + csr_spmm and their one-kernel form fused_attention (cuda_kernels.h:976-1075). */
int sfb_csr_attention(sfb_stream_t stream, const int32_t *rowptr, const int32_t *colidx, const void *q, const void *k,
                      const void *v, void *o, int dtype, uint32_t batch_dim, uint32_t seq_len, uint32_t head_dim,
                      uint32_t state_dim, float scale, uint32_t *bad_columns);

#ifdef __cplusplus
}
#endif
#endif
