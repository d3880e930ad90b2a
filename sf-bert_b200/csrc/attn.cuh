// Internal interface between the C ABI (ops.cu) and the kernel files.
#pragma once
#include "common.cuh"

namespace sfb {

struct AttnDims {
    uint32_t B, H, d, nb_a, nb_b, blocks;
    uint32_t lut_stride;   // uint2 per head in the LUT handed to the kernel (0 = shared by all heads)
    uint32_t mask_stride;  // words per head in the mask (0 = shared)
    uint64_t in_pitch;     // elements between consecutive rows of q, k, v (0 = H * d: the tensors hold these heads only)
    uint64_t out_pitch;    // the same for o
};

// CUDA-core kernels (attn_simt.cu)
int simt_sddmm_nt(cudaStream_t s, const void *lut, const void *a, const void *b, void *c, int ab_dtype, int c_dtype,
                  uint32_t bs, const AttnDims &p);
int simt_softmax(cudaStream_t s, const void *lut, const void *mask, const void *x, void *y, int x_dtype, int y_dtype,
                 uint32_t bs, const AttnDims &p, float scale, uint32_t max_lut);
int simt_spmm_nn(cudaStream_t s, const void *lut, const void *a, const void *b, void *c, int a_dtype, int bc_dtype,
                 uint32_t bs, const AttnDims &p, bool trans);
int simt_softmax_grad(cudaStream_t s, const void *lut, const void *dy, const void *y, void *dx, int dtype, uint32_t bs,
                      const AttnDims &p, float scale, uint32_t max_lut);
int simt_fused_sddmm_softmax(cudaStream_t s, const void *nn_lut, const void *a, const void *b, const void *mask, void *y,
                             int ab_dtype, int y_dtype, uint32_t bs, const AttnDims &p, float scale);
int simt_fused_attention(cudaStream_t s, const void *nn_lut, const void *q, const void *k, const void *v, void *o,
                         const void *mask, int dtype, uint32_t bs, const AttnDims &p, float scale);

// tcgen05 kernels (attn_tc.cu)
bool tc_fused_attention_supported(int dtype, uint32_t bs, const AttnDims &p, float scale, uint32_t max_lut);
int tc_fused_attention(cudaStream_t s, const void *nn_lut, const void *q, const void *k, const void *v, void *o,
                       const void *mask, int dtype, const AttnDims &p, float scale);
int tc_status_fused(uint32_t *out);
int tc_status_clear_fused();
bool tc_sddmm_supported(int ab_dtype, uint32_t bs, const AttnDims &p, const void *a, const void *b, const void *c);
int tc_sddmm(cudaStream_t s, const void *nt_lut, const void *a, const void *b, void *c, int ab_dtype, int c_dtype, const AttnDims &p);
bool tc_spmm_supported(int a_dtype, int bc_dtype, uint32_t bs, const AttnDims &p, uint32_t max_lut, const void *a, const void *b,
                       const void *c);
int tc_spmm(cudaStream_t s, const void *lut, const void *a, const void *b, void *c, int dtype, const AttnDims &p, bool trans);
bool tc_fused_p_supported(int ab_dtype, uint32_t bs, const AttnDims &p, float scale, const void *a, const void *b, const void *y);
int tc_fused_p(cudaStream_t s, const void *nn_lut, const void *a, const void *b, const void *mask, void *y, int ab_dtype,
               int y_dtype, const AttnDims &p, float scale);
int tc_sddmm_softmax_grad(cudaStream_t s, const void *nt_lut, const void *dout, const void *v, const void *pblk, const float *delta,
                          void *ds, int dtype, const AttnDims &p, float scale);
int rowdot(cudaStream_t s, float *out, const void *a, const void *b, size_t rows, uint32_t d, int dtype);
int tc_status_unfused(uint32_t *out);
int tc_status_clear_unfused();

// tcgen05 dense projection (gemm_tc.cu)
int tc_linear(cudaStream_t s, void *out, const void *x, const void *w, const float *bias, uint32_t m, uint32_t n, uint32_t k,
              int dtype, int act, bool w_transposed);
int embedding_lookup(cudaStream_t s, void *out, const void *table, const int32_t *ids, const void *pos, uint32_t batch,
                     uint32_t seq_len, uint32_t hidden, uint32_t vocab, int dtype, uint32_t *bad_ids);
int tc_status_gemm(uint32_t *out);
int tc_status_clear_gemm();

}  // namespace sfb
