/*
 * C-ABI wrappers around the reference's own CPU operators, compiled from the reference
 * headers where they lie (never copied).  TEST INFRASTRUCTURE ONLY: used to pin the
 * oracle restatement (tests/) and as the timed CPU baseline (bench.py).
 * Built by oracle/Makefile into oracle/_ref/libsfb_ref.so.
 */
#include "matmul.h"
#include "ewops.h"
#include "layernorm.h"
#include "embedding.h"
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

/* matmul.h:53-78  C[B,H,mA,mB] = A[B,H,mA,nA] . B[B,H,mB,nA]^T, entries with column > row zeroed */
void ref_multiheadmatmulNT(float *C, float *A, float *B, int batch, int heads, int mA, int nA, int mB)
{
    multiheadmatmulNT<float, float, float>(C, A, B, batch, heads, mA, nA, mB);
}

/* matmul.h:6-20  C[B,H,mA,nB] = A[B,H,mA,nA] . B[B,H,nA,nB] */
void ref_multiheadmatmulNN(float *C, float *A, float *B, int batch, int heads, int mA, int nA, int nB)
{
    multiheadmatmulNN<float, float, float>(C, A, B, batch, heads, mA, nA, nB);
}

/* ewops.h:64-98  causal row softmax of the unscaled scores */
void ref_softmax(float *C, float *A, float scaler, int seq_len, int batch, int heads)
{
    softmax<float, float>(C, A, scaler, seq_len, batch, heads);
}

/* ewops.h:103-122  dx = (dy - sum_row(dy*y)) * y * scaler, dense rows */
void ref_softmax_grad(float *out, float *dy, float *y, float scaler, int batch, int heads, int seq_len)
{
    softmax_grad<float, float, float>(out, dy, y, scaler, batch, heads, seq_len);
}

/* matmul.h:81-99  C[b,h] = A[b,h]^T . B[b,h], A [mA,nA], B [mA,nB] */
void ref_multiheadmatmulTN(float *C, float *A, float *B, int batch, int heads, int mA, int nA, int nB)
{
    multiheadmatmulTN<float, float, float>(C, A, B, batch, heads, mA, nA, nB);
}

/* ewops.h:314-331  [d0,d1,d2,d3] -> [d0,d2,d1,d3] */
void ref_transpose_0123to0213(float *src, float *des, int d0, int d1, int d2, int d3)
{
    transpose_0123to0213(src, des, d0, d1, d2, d3);
}

/* ewops.h:10-17 */
void ref_bias(float *out, const float *in, const float *b, int n, int m) { bias(out, in, b, n, m); }

/* ewops.h:296-301 */
void ref_tensor_add_tensor(float *C, float *A, float *B, int d0, int d1, int d2)
{
    tensor_add_tensor(C, A, B, d0, d1, d2);
}

/* ewops.h:32-43 */
void ref_gelu(float *C, float *A, int batch, int seq_len, int state) { gelu(C, A, batch, seq_len, state); }

/* layernorm.h:13-38 */
void ref_layernorm(float *out, float *mean, float *rstd, const float *in, const float *gain,
                   const float *b, int batch, int seq_len, int state)
{
    layernorm(out, mean, rstd, in, gain, b, batch, seq_len, state);
}

/* matmul.h:101-118 */
void ref_matrixMulNNCPU(float *C, const float *A, const float *B, int mA, int nA, int nB)
{
    matrixMulNNCPU(C, A, B, mA, nA, nB);
}

/* matmul.h:121-132 */
void ref_matrixMulNTCPU(float *C, const float *A, const float *B, int mA, int nA, int mB) { matrixMulNTCPU(C, A, B, mA, nA, mB); }

/* embedding.h:5-12 */
void ref_embedding_lookup(float *C, float *A, int *B, int batch, int seq_len, int heads, int per_head)
{
    embedding_lookup(C, A, B, batch, seq_len, heads, per_head);
}

/* ewops.h:276-282 */
void ref_tensor_add_matrix(float *C, float *A, float *B, int d0, int d1, int d2) { tensor_add_matrix(C, A, B, d0, d1, d2); }

/* ewops.h:430-443 */
void ref_generate_csr_full_mask(int *rowptr, int *colidx, int batch, int heads, int seq_len)
{
    generate_csr_full_mask(rowptr, colidx, batch, heads, seq_len);
}

void ref_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}

int ref_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}
