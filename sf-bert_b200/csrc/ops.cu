// C ABI of the attention operators: argument checks and the choice between the tensor-core
// (tcgen05) kernels and the CUDA-core kernels.  No path leaves the GPU.
#include "attn.cuh"

using namespace sfb;

static int check_common(const char *who, uint32_t bs, uint32_t B, uint32_t H, uint32_t d, uint32_t lut_heads)
{
    SFB_REQUIRE(bs == 32 || bs == 64, "%s: block_size %u not supported (32 or 64)", who, bs);
    SFB_REQUIRE(B >= 1 && B <= 65535 && H >= 1 && H <= 65535, "%s: batch_dim=%u / head_dim=%u out of range", who, B, H);
    SFB_REQUIRE(d >= 1, "%s: state_dim is 0", who);
    SFB_REQUIRE(lut_heads == 1 || lut_heads == H, "%s: lut_heads=%u must be 1 or head_dim=%u", who, lut_heads, H);
    return 0;
}

static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

extern "C" int sfb_bst_sgemm_nt(sfb_stream_t stream, const void *lut, const void *a, const void *b, void *c, int ab_dtype,
                                int c_dtype, uint32_t block_size, uint32_t blocks, uint32_t batch_dim, uint32_t ctx_blks_a,
                                uint32_t ctx_blks_b, uint32_t head_dim, uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim)
{
    const char *who = "sfb_bst_sgemm_nt";
    SFB_REQUIRE(lut && a && b && c, "%s: NULL pointer", who);
    SFB_REQUIRE(valid_dtype(ab_dtype) && valid_dtype(c_dtype), "%s: unknown dtype", who);
    if (check_common(who, block_size, batch_dim, head_dim, state_dim, lut_heads)) return 1;
    SFB_REQUIRE(lut_heads == 1 || lut_dim >= blocks, "%s: lut_dim %u smaller than blocks %u", who, lut_dim, blocks);
    if (blocks == 0) { clear_error(); return 0; }
    AttnDims p = {batch_dim, head_dim, state_dim, ctx_blks_a, ctx_blks_b, blocks, lut_heads > 1 ? lut_dim : 0, 0};
    if (tc_sddmm_supported(ab_dtype, block_size, p, a, b, c)) return tc_sddmm(as_stream(stream), lut, a, b, c, ab_dtype, c_dtype, p);
    return simt_sddmm_nt(as_stream(stream), lut, a, b, c, ab_dtype, c_dtype, block_size, p);
}

extern "C" int sfb_masked_softmax(sfb_stream_t stream, const void *lut, const void *mask, const void *x, void *y, int x_dtype,
                                  int y_dtype, uint32_t block_size, uint32_t blocks, uint32_t batch_dim, uint32_t head_dim,
                                  uint32_t ctx_blks, uint32_t lut_heads, uint32_t lut_dim, uint32_t max_lut, uint32_t mask_heads,
                                  float scale)
{
    const char *who = "sfb_masked_softmax";
    SFB_REQUIRE(lut && x && y, "%s: NULL pointer", who);
    SFB_REQUIRE(x_dtype == SFB_BF16 || x_dtype == SFB_F32, "%s: x must be bf16 or fp32", who);
    SFB_REQUIRE(valid_dtype(y_dtype), "%s: unknown y dtype", who);
    if (check_common(who, block_size, batch_dim, head_dim, 1, lut_heads)) return 1;
    SFB_REQUIRE(mask_heads == 1 || mask_heads == head_dim, "%s: mask_heads=%u must be 1 or head_dim", who, mask_heads);
    SFB_REQUIRE(lut_heads == 1 || lut_dim >= blocks + ctx_blks, "%s: lut_dim %u smaller than blocks+ctx_blks", who, lut_dim);
    SFB_REQUIRE(aligned16(x) && aligned16(y), "%s: x and y must be 16-byte aligned", who);
    if (blocks == 0 || ctx_blks == 0) { clear_error(); return 0; }
    AttnDims p = {batch_dim, head_dim, 0, ctx_blks, ctx_blks, blocks, lut_heads > 1 ? lut_dim : 0,
                  mask_heads > 1 ? blocks * block_size : 0};
    // max_lut (the reference sizes its CTA from it, blocksparse.h:665-680) picks the register-resident variant;
    // a value smaller than the longest row would drop blocks, so 0 (= unknown) is always safe
    return simt_softmax(as_stream(stream), lut, mask, x, y, x_dtype, y_dtype, block_size, p, scale, max_lut);
}

extern "C" int sfb_bst_sgemm_xn(sfb_stream_t stream, const void *lut, const void *a, const void *b, void *c, int a_dtype,
                                int bc_dtype, uint32_t block_size, uint32_t blocks, uint32_t batch_dim, uint32_t ctx_blks_b,
                                uint32_t ctx_blks_c, uint32_t head_dim, uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim,
                                uint32_t op, uint32_t magic, uint32_t shift, uint32_t max_lut)
{
    const char *who = "sfb_bst_sgemm_xn";
    (void)magic; (void)shift;
    SFB_REQUIRE(lut && a && b && c, "%s: NULL pointer", who);
    SFB_REQUIRE(op == SFB_NN_OP || op == SFB_TN_OP, "%s: op %u not supported (NN_OP or TN_OP)", who, op);
    SFB_REQUIRE(valid_dtype(a_dtype) && valid_dtype(bc_dtype), "%s: unknown dtype", who);
    if (check_common(who, block_size, batch_dim, head_dim, state_dim, lut_heads)) return 1;
    SFB_REQUIRE(lut_heads == 1 || lut_dim >= blocks + ctx_blks_c, "%s: lut_dim %u smaller than blocks+ctx_blks", who, lut_dim);
    if (ctx_blks_c == 0) { clear_error(); return 0; }
    AttnDims p = {batch_dim, head_dim, state_dim, ctx_blks_c, ctx_blks_b, blocks, lut_heads > 1 ? lut_dim : 0, 0};
    const bool trans = op == SFB_TN_OP;
    if (tc_spmm_supported(a_dtype, bc_dtype, block_size, p, max_lut, a, b, c)) return tc_spmm(as_stream(stream), lut, a, b, c, a_dtype, p, trans);
    return simt_spmm_nn(as_stream(stream), lut, a, b, c, a_dtype, bc_dtype, block_size, p, trans);
}

extern "C" int sfb_masked_softmax_grad(sfb_stream_t stream, const void *lut, const void *dy, const void *y, void *dx, int dtype,
                                       uint32_t block_size, uint32_t blocks, uint32_t batch_dim, uint32_t head_dim,
                                       uint32_t ctx_blks, uint32_t lut_heads, uint32_t lut_dim, uint32_t max_lut, float scale)
{
    const char *who = "sfb_masked_softmax_grad";
    SFB_REQUIRE(lut && dy && y && dx, "%s: NULL pointer", who);
    SFB_REQUIRE(valid_dtype(dtype), "%s: unknown dtype", who);
    if (check_common(who, block_size, batch_dim, head_dim, 1, lut_heads)) return 1;
    SFB_REQUIRE(lut_heads == 1 || lut_dim >= blocks + ctx_blks, "%s: lut_dim %u smaller than blocks+ctx_blks", who, lut_dim);
    SFB_REQUIRE(aligned16(dy) && aligned16(y) && aligned16(dx), "%s: dy, y and dx must be 16-byte aligned", who);
    if (blocks == 0 || ctx_blks == 0) { clear_error(); return 0; }
    AttnDims p = {batch_dim, head_dim, 0, ctx_blks, ctx_blks, blocks, lut_heads > 1 ? lut_dim : 0, 0};
    return simt_softmax_grad(as_stream(stream), lut, dy, y, dx, dtype, block_size, p, scale, max_lut);
}

extern "C" int sfb_fused_sddmm_softmax(sfb_stream_t stream, const void *nn_lut, const void *a, const void *b, const void *mask,
                                       void *y, int ab_dtype, int y_dtype, uint32_t block_size, uint32_t blocks,
                                       uint32_t batch_dim, uint32_t ctx_blks_a, uint32_t ctx_blks_b, uint32_t head_dim,
                                       uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim, uint32_t mask_heads, float scale)
{
    const char *who = "sfb_fused_sddmm_softmax";
    SFB_REQUIRE(nn_lut && a && b && y, "%s: NULL pointer", who);
    SFB_REQUIRE(valid_dtype(ab_dtype) && valid_dtype(y_dtype), "%s: unknown dtype", who);
    if (check_common(who, block_size, batch_dim, head_dim, state_dim, lut_heads)) return 1;
    SFB_REQUIRE(mask_heads == 1 || mask_heads == head_dim, "%s: mask_heads=%u must be 1 or head_dim", who, mask_heads);
    SFB_REQUIRE(lut_heads == 1 || lut_dim >= blocks, "%s: lut_dim %u smaller than blocks %u", who, lut_dim, blocks);
    if (blocks == 0 || ctx_blks_a == 0) { clear_error(); return 0; }
    // the nn_lut of head h starts at h * (lut_dim + ctx_blks_a)  (fusion_blocksparse.h:1245)
    AttnDims p = {batch_dim, head_dim, state_dim, ctx_blks_a, ctx_blks_b, blocks, lut_heads > 1 ? lut_dim + ctx_blks_a : 0,
                  mask_heads > 1 ? blocks * block_size : 0};
    if (ctx_blks_a == ctx_blks_b && tc_fused_p_supported(ab_dtype, block_size, p, scale, a, b, y))
        return tc_fused_p(as_stream(stream), nn_lut, a, b, mask, y, ab_dtype, y_dtype, p, scale);
    return simt_fused_sddmm_softmax(as_stream(stream), nn_lut, a, b, mask, y, ab_dtype, y_dtype, block_size, p, scale);
}

static int fused_attention_common(const char *who, sfb_stream_t stream, const void *nn_lut, const void *q, const void *k, const void *v,
                                  void *o, const void *mask, int dtype, uint32_t block_size, uint32_t blocks, uint32_t batch_dim,
                                  uint32_t ctx_blks, uint32_t head_dim, uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim,
                                  uint32_t mask_heads, float scale, uint32_t max_lut, uint64_t in_pitch, uint64_t out_pitch)
{
    SFB_REQUIRE(nn_lut && q && k && v && o, "%s: NULL pointer", who);
    SFB_REQUIRE(valid_dtype(dtype), "%s: unknown dtype %d", who, dtype);
    if (check_common(who, block_size, batch_dim, head_dim, state_dim, lut_heads)) return 1;
    SFB_REQUIRE(mask_heads == 1 || mask_heads == head_dim, "%s: mask_heads=%u must be 1 or head_dim", who, mask_heads);
    SFB_REQUIRE(lut_heads == 1 || lut_dim >= blocks, "%s: lut_dim %u smaller than blocks %u", who, lut_dim, blocks);
    const uint64_t width = (uint64_t)head_dim * state_dim;
    SFB_REQUIRE((in_pitch == 0 || in_pitch >= width) && (out_pitch == 0 || out_pitch >= width),
                "%s: a row pitch smaller than head_dim * state_dim = %llu elements", who, (unsigned long long)width);
    SFB_REQUIRE(in_pitch < (1ull << 31) && out_pitch < (1ull << 31), "%s: row pitch too large", who);
    if (ctx_blks == 0) { clear_error(); return 0; }
    AttnDims p = {batch_dim, head_dim, state_dim, ctx_blks, ctx_blks, blocks, lut_heads > 1 ? lut_dim + ctx_blks : 0,
                  mask_heads > 1 ? blocks * block_size : 0, in_pitch, out_pitch};
    // 16-bit operands with 64x64 blocks and 64-wide heads run on the tensor cores, when the TMA can address them
    // (16-byte aligned bases and row pitches); everything else runs on the CUDA cores
    const bool tma_ok = ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) == 0) && in_pitch % 8 == 0 && out_pitch % 8 == 0;
    if (tma_ok && tc_fused_attention_supported(dtype, block_size, p, scale, max_lut))
        return tc_fused_attention(as_stream(stream), nn_lut, q, k, v, o, mask, dtype, p, scale);
    return simt_fused_attention(as_stream(stream), nn_lut, q, k, v, o, mask, dtype, block_size, p, scale);
}

extern "C" int sfb_fused_attention(sfb_stream_t stream, const void *nn_lut, const void *q, const void *k, const void *v, void *o,
                                   const void *mask, int dtype, uint32_t block_size, uint32_t blocks, uint32_t batch_dim,
                                   uint32_t ctx_blks, uint32_t head_dim, uint32_t state_dim, uint32_t lut_heads, uint32_t lut_dim,
                                   uint32_t mask_heads, float scale, uint32_t max_lut)
{
    return fused_attention_common("sfb_fused_attention", stream, nn_lut, q, k, v, o, mask, dtype, block_size, blocks, batch_dim, ctx_blks,
                                  head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale, max_lut, 0, 0);
}

extern "C" int sfb_fused_attention_slice(sfb_stream_t stream, const void *nn_lut, const void *q, const void *k, const void *v, void *o,
                                         const void *mask, int dtype, uint32_t block_size, uint32_t blocks, uint32_t batch_dim,
                                         uint32_t ctx_blks, uint32_t head_dim, uint32_t state_dim, uint32_t lut_heads,
                                         uint32_t lut_dim, uint32_t mask_heads, float scale, uint32_t max_lut, uint64_t in_pitch,
                                         uint64_t out_pitch)
{
    return fused_attention_common("sfb_fused_attention_slice", stream, nn_lut, q, k, v, o, mask, dtype, block_size, blocks, batch_dim,
                                  ctx_blks, head_dim, state_dim, lut_heads, lut_dim, mask_heads, scale, max_lut, in_pitch, out_pitch);
}

static int linear_common(const char *who, sfb_stream_t stream, void *out, const void *x, const void *w, const float *bias, uint32_t m,
                         uint32_t n, uint32_t k, int dtype, int act, bool w_transposed);

extern "C" int sfb_linear(sfb_stream_t stream, void *out, const void *x, const void *w, const float *bias, uint32_t m, uint32_t n,
                          uint32_t k, int dtype, int act)
{
    return linear_common("sfb_linear", stream, out, x, w, bias, m, n, k, dtype, act, false);
}

extern "C" int sfb_linear_nt(sfb_stream_t stream, void *out, const void *x, const void *wt, const float *bias, uint32_t m, uint32_t n,
                             uint32_t k, int dtype, int act)
{
    return linear_common("sfb_linear_nt", stream, out, x, wt, bias, m, n, k, dtype, act, true);
}

extern "C" int sfb_embedding(sfb_stream_t stream, void *out, const void *table, const int32_t *ids, const void *pos, uint32_t batch,
                             uint32_t seq_len, uint32_t hidden, uint32_t vocab, int dtype, uint32_t *bad_ids)
{
    const char *who = "sfb_embedding";
    SFB_REQUIRE(out && table && ids, "%s: NULL pointer", who);
    SFB_REQUIRE(valid_dtype(dtype), "%s: unknown dtype", who);
    SFB_REQUIRE(hidden % 8 == 0, "%s: hidden=%u must be a multiple of 8", who, hidden);
    SFB_REQUIRE(aligned16(out) && aligned16(table) && (!pos || aligned16(pos)), "%s: out, table and pos must be 16-byte aligned", who);
    SFB_REQUIRE((uint64_t)batch * seq_len < (1ull << 31), "%s: too many tokens", who);
    if (batch == 0 || seq_len == 0 || hidden == 0) { clear_error(); return 0; }
    return embedding_lookup(as_stream(stream), out, table, ids, pos, batch, seq_len, hidden, vocab, dtype, bad_ids);
}

static int linear_common(const char *who, sfb_stream_t stream, void *out, const void *x, const void *w, const float *bias, uint32_t m,
                         uint32_t n, uint32_t k, int dtype, int act, bool w_transposed)
{
    SFB_REQUIRE(out && x && w, "%s: NULL pointer", who);
    SFB_REQUIRE(dtype == SFB_BF16 || dtype == SFB_F16, "%s: x, w and out must be bf16 or fp16 (fp32 products stay with the GEMM library)", who);
    SFB_REQUIRE(act == SFB_ACT_NONE || act == SFB_ACT_GELU, "%s: unknown activation %d", who, act);
    SFB_REQUIRE(n % 16 == 0 && k % 8 == 0, "%s: n=%u must be a multiple of 16 and k=%u of 8", who, n, k);
    SFB_REQUIRE(aligned16(x) && aligned16(w) && (!bias || aligned16(bias)) && ((uintptr_t)out & 31) == 0,
                "%s: x, w, bias must be 16-byte and out 32-byte aligned", who);
    SFB_REQUIRE((uint64_t)m < (1ull << 31) && (uint64_t)n < (1ull << 31) && (uint64_t)k < (1ull << 31), "%s: dimension too large", who);
    if (m == 0 || n == 0) { clear_error(); return 0; }
    SFB_REQUIRE(k > 0, "%s: k is 0", who);
    return tc_linear(as_stream(stream), out, x, w, bias, m, n, k, dtype, act, w_transposed);
}

extern "C" int sfb_rowdot(sfb_stream_t stream, float *out, const void *a, const void *b, uint64_t rows, uint32_t d, int dtype)
{
    const char *who = "sfb_rowdot";
    SFB_REQUIRE(out && a && b, "%s: NULL pointer", who);
    SFB_REQUIRE(valid_dtype(dtype), "%s: unknown dtype", who);
    SFB_REQUIRE(d % 8 == 0 && d > 0, "%s: row length %u must be a positive multiple of 8", who, d);
    SFB_REQUIRE(aligned16(a) && aligned16(b), "%s: a and b must be 16-byte aligned", who);
    SFB_REQUIRE(rows < (1ull << 40), "%s: too many rows", who);
    if (rows == 0) { clear_error(); return 0; }
    return rowdot(as_stream(stream), out, a, b, (size_t)rows, d, dtype);
}

extern "C" int sfb_fused_sddmm_softmax_grad(sfb_stream_t stream, const void *nt_lut, const void *dout, const void *v, const void *p_blocks,
                                            const float *delta, void *ds, int dtype, uint32_t block_size, uint32_t blocks,
                                            uint32_t batch_dim, uint32_t ctx_blks, uint32_t head_dim, uint32_t state_dim,
                                            uint32_t lut_heads, uint32_t lut_dim, float scale)
{
    const char *who = "sfb_fused_sddmm_softmax_grad";
    SFB_REQUIRE(nt_lut && dout && v && p_blocks && delta && ds, "%s: NULL pointer", who);
    SFB_REQUIRE(dtype == SFB_BF16 || dtype == SFB_F16, "%s: dO, V, P and dS must be bf16 or fp16", who);
    SFB_REQUIRE(block_size == 64 && state_dim == 64, "%s: block_size %u / state_dim %u not supported (64 / 64)", who, block_size, state_dim);
    if (check_common(who, block_size, batch_dim, head_dim, state_dim, lut_heads)) return 1;
    SFB_REQUIRE(lut_heads == 1 || lut_dim >= blocks, "%s: lut_dim %u smaller than blocks %u", who, lut_dim, blocks);
    if (blocks == 0 || ctx_blks == 0) { clear_error(); return 0; }
    AttnDims p = {batch_dim, head_dim, state_dim, ctx_blks, ctx_blks, blocks, lut_heads > 1 ? lut_dim : 0, 0};
    SFB_REQUIRE((uint64_t)batch_dim * ctx_blks * 64 < (1ull << 31), "%s: sequence too long for one launch", who);
    return tc_sddmm_softmax_grad(as_stream(stream), nt_lut, dout, v, p_blocks, delta, ds, dtype, p, scale);
}

extern "C" int sfb_device_status_clear(void)
{
    if (tc_status_clear_fused() || tc_status_clear_unfused() || tc_status_clear_gemm()) return 1;
    clear_error();
    return 0;
}

extern "C" int sfb_device_status(uint32_t *status)
{
    SFB_REQUIRE(status, "sfb_device_status: NULL pointer");
    uint32_t a = 0, b = 0, c = 0;
    if (tc_status_fused(&a) || tc_status_unfused(&b) || tc_status_gemm(&c)) return 1;
    *status = a ? a : b ? b : c;
    clear_error();
    return 0;
}
