/*
 * C-ABI wrappers around the reference's own UNFUSED GPU operators (SDDMM, masked softmax, SpMM),
 * compiled for sm_100a from the reference header where it lies (never copied).
 * TEST INFRASTRUCTURE ONLY: a second pin for the parity tests (the reference's GPU arithmetic on
 * the same B200) and a timed "reference on the same GPU" figure for bench.py's reference arm.
 * Built by oracle/Makefile into oracle/_ref/libsfb_ref_gpu.so.
 *
 * Only these operators (forward: SDDMM, softmax, SpMM; backward: softmax gradient, transposed SpMM) are
 * wrapped.  They launch plain kernels without cross-CTA waits.
 * The reference's fused kernels (fusion_blocksparse.h) spin on global flags without a bound and are
 * deliberately not wrapped: nothing here can launch them.
 *
 * The reference implements the two matmuls for block_size 32 only (blocksparse.h:448, :996; any other
 * size launches nothing), so their wrappers refuse another block size instead of returning garbage; the
 * softmax wrapper also takes 64.
 */
#include "blocksparse.h"

namespace {

int check_common(uint block_size, uint blocks, uint batch_dim, uint ctx_blks, uint heads, uint state_dim)
{
    if (block_size != 32) return -1;
    if (!blocks || !batch_dim || !ctx_blks || !heads || !state_dim) return -2;
    if (state_dim % 4) return -3;                     /* float4 loads along the head size */
    /* all offsets inside the kernels are 32-bit */
    unsigned long long act = 1ull * batch_dim * ctx_blks * block_size * heads * state_dim;
    unsigned long long blk = 1ull * batch_dim * heads * blocks * block_size * block_size;
    if (act >= (1ull << 32) || blk >= (1ull << 32)) return -4;
    return 0;
}

int launched() { return cudaGetLastError() == cudaSuccess ? 0 : -9; }

}  // namespace

extern "C" {

/* blocksparse.h:425-456  S[b,h,k] = Q-rows(nt_lut[k].x) . K-rows(nt_lut[k].y)^T, fp32 in, bf16 out, unscaled */
int ref_gpu_bst_sgemm_nt(void *stream, const void *nt_lut, const float *a, const float *b, void *c,
                         uint block_size, uint blocks, uint batch_dim, uint ctx_blks_a, uint ctx_blks_b,
                         uint head_dim, uint state_dim, uint lut_heads, uint lut_dim)
{
    int rc = check_common(block_size, blocks, batch_dim, ctx_blks_a, head_dim, state_dim);
    if (rc) return rc;
    if (ctx_blks_a != ctx_blks_b) return -5;
    bst_sgemm_nt((CUstream)stream, (const uint2 *)nt_lut, a, b, (bhalf *)c, block_size, blocks, batch_dim,
                 ctx_blks_a, ctx_blks_b, head_dim, state_dim, lut_heads, lut_dim);
    return launched();
}

/* blocksparse.h:649-722  P = softmax over each query row's concatenated blocks of scale*S.
 * y_is_float: 0 → <bhalf,bhalf2> (no_fusion_test.cu:221), 1 → <float,float2> (fixed_fusion_test.cu:435).
 * mask = NULL keeps everything. */
int ref_gpu_masked_softmax(void *stream, const void *nn_lut, const void *mask, const void *x, void *y,
                           int y_is_float, uint block_size, uint blocks, uint batch_dim, uint head_dim,
                           uint ctx_blks, uint lut_heads, uint lut_dim, uint max_lut, uint mask_heads,
                           float scale)
{
    /* the softmax, unlike the two matmuls, is also implemented for block size 64 (blocksparse.h:684-693, uint64 masks) */
    int rc = check_common(block_size == 64 ? 32 : block_size, blocks, batch_dim, ctx_blks, head_dim, 4);
    if (rc) return rc;
    if (1ull * batch_dim * head_dim * blocks * block_size * block_size >= (1ull << 32)) return -4;
    if (!max_lut || max_lut * block_size > 16 * 1024) return -6;   /* keeps the launch at <= 1024 threads, unroll 4..8 */
    if (y_is_float)
        BlocksparseMaskedSoftmax<float, float2>((CUstream)stream, (const uint2 *)nn_lut, (const uint *)mask,
            (const bhalf *)x, (float *)y, block_size, blocks, batch_dim, head_dim, ctx_blks, lut_heads,
            lut_dim, max_lut, mask_heads, scale);
    else
        BlocksparseMaskedSoftmax<bhalf, bhalf2>((CUstream)stream, (const uint2 *)nn_lut, (const uint *)mask,
            (const bhalf *)x, (bhalf *)y, block_size, blocks, batch_dim, head_dim, ctx_blks, lut_heads,
            lut_dim, max_lut, mask_heads, scale);
    return launched();
}

/* blocksparse.h:965-1014 with NN_OP  O-rows(i) = sum over row i's blocks of P[b,h,k] . V-rows(col k);
 * P bf16, V and O fp32.  magic/shift from the reference's own magicu64 (blocksparse.h:1016-1043), as at
 * transformer_attention_optimize.cu:135-137. */
int ref_gpu_bst_sgemm_nn(void *stream, const void *nn_lut, const void *a, const float *b, float *c,
                         uint block_size, uint blocks, uint batch_dim, uint ctx_blks_b, uint ctx_blks_c,
                         uint head_dim, uint state_dim, uint lut_heads, uint lut_dim, uint max_lut)
{
    int rc = check_common(block_size, blocks, batch_dim, ctx_blks_c, head_dim, state_dim);
    if (rc) return rc;
    if (ctx_blks_b != ctx_blks_c) return -5;
    if (!max_lut || ((max_lut + 1) / 2) * 2 * 8 > 32 * 1024) return -6;   /* dynamic shared memory */
    uint magic = 0, shift = 0;
    magicu64(CEIL_DIV(state_dim, 64), magic, shift);
    bst_sgemm_xn((CUstream)stream, (const uint2 *)nn_lut, (const bhalf *)a, b, c, block_size, blocks,
                 batch_dim, ctx_blks_b, ctx_blks_c, head_dim, state_dim, lut_heads, lut_dim, NN_OP,
                 magic, shift, max_lut);
    return launched();
}

/* blocksparse.h:1164-1227  dx = (dy - sum over the query row of dy*y) * y * scale, <bhalf,bhalf2> as at
 * no_fusion_test.cu:460 / transformer_attention_optimize.cu:944; block size 32 or 64. */
int ref_gpu_masked_softmax_grad(void *stream, const void *nn_lut, const void *dy, const void *y, void *dx,
                                uint block_size, uint blocks, uint batch_dim, uint head_dim, uint ctx_blks,
                                uint lut_heads, uint lut_dim, uint max_lut, float scale)
{
    int rc = check_common(block_size == 64 ? 32 : block_size, blocks, batch_dim, ctx_blks, head_dim, 4);
    if (rc) return rc;
    if (1ull * batch_dim * head_dim * blocks * block_size * block_size >= (1ull << 32)) return -4;
    if (!max_lut || max_lut * block_size > 16 * 1024) return -6;
    BlocksparseMaskedSoftmaxGrad<bhalf, bhalf2>((CUstream)stream, (const uint2 *)nn_lut, (const bhalf *)dy,
        (const bhalf *)y, (bhalf *)dx, block_size, blocks, batch_dim, head_dim, ctx_blks, lut_heads, lut_dim,
        max_lut, scale);
    return launched();
}

/* blocksparse.h:965-1014 with TN_OP  C-rows(block column j) = sum over the column's blocks of A[b,h,k]^T .
 * B-rows(row of k); lut = tn_lut (header per block column), max_lut its longest column.  dV = P^T dO and
 * dK = dS^T Q at transformer_attention_optimize.cu:924,954. */
int ref_gpu_bst_sgemm_tn(void *stream, const void *tn_lut, const void *a, const float *b, float *c,
                         uint block_size, uint blocks, uint batch_dim, uint ctx_blks_b, uint ctx_blks_c,
                         uint head_dim, uint state_dim, uint lut_heads, uint lut_dim, uint max_lut)
{
    int rc = check_common(block_size, blocks, batch_dim, ctx_blks_c, head_dim, state_dim);
    if (rc) return rc;
    if (ctx_blks_b != ctx_blks_c) return -5;
    if (!max_lut || ((max_lut + 1) / 2) * 2 * 8 > 32 * 1024) return -6;
    uint magic = 0, shift = 0;
    magicu64(CEIL_DIV(state_dim, 64), magic, shift);
    bst_sgemm_xn((CUstream)stream, (const uint2 *)tn_lut, (const bhalf *)a, b, c, block_size, blocks,
                 batch_dim, ctx_blks_b, ctx_blks_c, head_dim, state_dim, lut_heads, lut_dim, TN_OP,
                 magic, shift, max_lut);
    return launched();
}

}  // extern "C"
