// A driver shaped like the reference's *_fusion_test.cu programs: it builds the look-up tables on the
// host the way those programs do, uploads them, and calls the operators through the drop-in headers
// (include/blocksparse.h, include/fusion_blocksparse.h) with the reference's argument order.  Inputs are
// all ones, the reference's own known answer (fixed_fusion_test.cu:263-268, test.cu:382-386): every score
// equals d, every probability 1 / (kept keys of the row), every output 1.
// The backward follows with the reference's call order (transformer_attention_optimize.cu:924-964) and dO = 1:
// dV[key j] = sum over the rows r >= j of 1/(r+1), dP = d everywhere, and dS, dQ, dK vanish up to the bf16
// rounding of P (a softmax whose upstream gradient is constant along the row has none).
// Prints "PASS" and returns 0 when all of that holds on the GPU.
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <vector>
#include "blocksparse.h"
#include "fusion_blocksparse.h"

static float bf(ushort v) { unsigned u = (unsigned)v << 16; float f; memcpy(&f, &u, 4); return f; }

// The additions below the reference's surface: sfb_build_lut (LUTs + masks in one call, on the device) and the 16-bit
// overload of fusion_attention (bf16 Q, K, V, O; 64x64 blocks, 64-wide heads: the tensor-core kernel), on the all-ones
// known answer with the causal element mask on the diagonal blocks: every output 1.
static size_t sixteen_bit_additions()
{
    const uint B = 2, H = 3, d = 64, bs = 64, nb = 6, L = nb * bs;
    std::vector<uchar> lay(nb * nb, 0);
    uint blocks = 0;
    for (uint i = 0; i < nb; i++)
        for (uint j = 0; j <= i; j++) { lay[i * nb + j] = 1; blocks++; }
    uchar *d_lay;
    uint2 *nt, *nn, *rblk;
    uint *nn_max, *status;
    uint64 *mask_np, *mask_t;
    cudaMalloc(&d_lay, nb * nb);
    cudaMemcpy(d_lay, lay.data(), nb * nb, cudaMemcpyHostToDevice);
    cudaMalloc(&nt, sizeof(uint2) * blocks);
    cudaMalloc(&nn, sizeof(uint2) * (nb + blocks));
    cudaMalloc(&rblk, sizeof(uint2) * blocks);
    cudaMalloc(&nn_max, sizeof(uint));
    cudaMalloc(&status, sizeof(uint));
    cudaMemset(status, 0, sizeof(uint));
    cudaMalloc(&mask_np, sizeof(uint64) * blocks * bs);
    cudaMalloc(&mask_t, sizeof(uint64) * blocks * bs);
    bool ok = sfb_build_lut(0, d_lay, 1, nb, bs, blocks, nt, nn, rblk, nn_max, status, SFB_MASK_CAUSAL_DIAG, 0, mask_np, mask_t);
    uint h_max = 0, h_status = 1;
    cudaMemcpy(&h_max, nn_max, sizeof(uint), cudaMemcpyDeviceToHost);
    cudaMemcpy(&h_status, status, sizeof(uint), cudaMemcpyDeviceToHost);
    const size_t n = (size_t)B * L * H * d;
    std::vector<bhalf> one(n, bhalf((ushort)0x3f80));    // 1.0 in bf16
    bhalf *q, *o;
    cudaMalloc(&q, sizeof(bhalf) * n);
    cudaMalloc(&o, sizeof(bhalf) * n);
    cudaMemcpy(q, one.data(), sizeof(bhalf) * n, cudaMemcpyHostToDevice);
    cudaMemset(o, 0, sizeof(bhalf) * n);
    ok = ok && fusion_attention<float, float2>(0, nt, q, q, (bhalf *)0, nn, (int *)0, (int *)0, mask_np, (float *)0, (float *)0,
                                               (float *)0, q, o, bs, blocks, B, nb, nb, nb, H, d, 1, blocks, 1, 0.125f, h_max);
    uint word = 1;
    ok = ok && sfb_device_status(&word) == 0;
    std::vector<bhalf> o_h(n);
    cudaMemcpy(o_h.data(), o, sizeof(bhalf) * n, cudaMemcpyDeviceToHost);
    size_t bad = (ok && h_max == nb && h_status == 0 && word == 0) ? 0 : 1;
    if (bad) printf("16-bit additions: call failed (%s), nn_max %u status %u word %u\n", sfb_last_error(), h_max, h_status, word);
    for (size_t i = 0; i < n; i++) bad += fabsf(bf(o_h[i].x) - 1.0f) > 1.0f / 128;
    return bad;
}

int main()
{
    const uint batch_dim = 2, heads_ = 4, head_state_ = 128, blk_size_ = 32, seq_len = 320;
    const uint ctx_blks_ = seq_len / blk_size_;
    const float scale = 1.0f / sqrtf((float)head_state_);
    const uint lut_heads = 1, mask_heads = 1;

    // causal block layout, as no_fusion_test.cu builds it
    std::vector<uint2> nt;
    for (uint i = 0; i < ctx_blks_; i++)
        for (uint j = 0; j <= i; j++) nt.push_back(make_uint2(i, j));
    const uint blocks = (uint)nt.size();
    std::vector<uint2> nn(ctx_blks_ + blocks, make_uint2(0, 0));
    for (uint k = 0; k < blocks; k++) {
        nn[ctx_blks_ + k] = make_uint2(k, nt[k].y);
        nn[nt[k].x].y++;
    }
    nn[0].x = ctx_blks_;
    for (uint i = 1; i < ctx_blks_; i++) nn[i].x = nn[i - 1].x + nn[i - 1].y;
    uint nn_max = 0;
    for (uint i = 0; i < ctx_blks_; i++) nn_max = nn[i].y > nn_max ? nn[i].y : nn_max;
    // causal element mask on the diagonal blocks: mask_np [blocks][32] and its transpose [32][blocks]
    std::vector<uint> mask_np(blocks * blk_size_), mask_t(blocks * blk_size_);
    for (uint k = 0; k < blocks; k++)
        for (uint r = 0; r < blk_size_; r++) {
            uint w = 0;
            for (uint c = 0; c < blk_size_; c++)
                if (nt[k].x != nt[k].y || r >= c) w |= 1u << c;
            mask_np[k * blk_size_ + r] = w;
            mask_t[r * blocks + k] = w;
        }

    const size_t n_in = (size_t)batch_dim * seq_len * heads_ * head_state_;
    const size_t n_blk = (size_t)batch_dim * heads_ * blocks * blk_size_ * blk_size_;
    std::vector<float> ones(n_in, 1.0f);
    uint2 *d_nt, *d_nn;
    uint *d_mask_np, *d_mask_t;
    float *a_ptr, *b_ptr, *v_ptr, *o_ptr, *o2_ptr, *y_ptr, *Max, *Sum;
    bhalf *c_ptr, *y2_ptr;
    int *flag, *flag1;
    cudaMalloc(&d_nt, sizeof(uint2) * blocks);
    cudaMalloc(&d_nn, sizeof(uint2) * nn.size());
    cudaMalloc(&d_mask_np, sizeof(uint) * mask_np.size());
    cudaMalloc(&d_mask_t, sizeof(uint) * mask_t.size());
    cudaMalloc(&a_ptr, sizeof(float) * n_in);
    cudaMalloc(&b_ptr, sizeof(float) * n_in);
    cudaMalloc(&v_ptr, sizeof(float) * n_in);
    cudaMalloc(&o_ptr, sizeof(float) * n_in);
    cudaMalloc(&o2_ptr, sizeof(float) * n_in);
    cudaMalloc(&y_ptr, sizeof(float) * n_blk);
    cudaMalloc(&c_ptr, sizeof(bhalf) * n_blk);
    cudaMalloc(&y2_ptr, sizeof(bhalf) * n_blk);
    cudaMalloc(&Max, sizeof(float) * batch_dim * heads_ * blocks * blk_size_);
    cudaMalloc(&Sum, sizeof(float) * batch_dim * heads_ * blocks * blk_size_);
    cudaMalloc(&flag, sizeof(int) * ctx_blks_ * batch_dim * heads_);
    cudaMalloc(&flag1, sizeof(int) * ctx_blks_ * batch_dim * heads_);
    cudaMemcpy(d_nt, nt.data(), sizeof(uint2) * blocks, cudaMemcpyHostToDevice);
    cudaMemcpy(d_nn, nn.data(), sizeof(uint2) * nn.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_mask_np, mask_np.data(), sizeof(uint) * mask_np.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_mask_t, mask_t.data(), sizeof(uint) * mask_t.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(a_ptr, ones.data(), sizeof(float) * n_in, cudaMemcpyHostToDevice);
    cudaMemcpy(b_ptr, ones.data(), sizeof(float) * n_in, cudaMemcpyHostToDevice);
    cudaMemcpy(v_ptr, ones.data(), sizeof(float) * n_in, cudaMemcpyHostToDevice);

    CUstream custream;
    cudaStreamCreate(&custream);
    uint magic_, shift_;
    magicu64(CEIL_DIV(head_state_, 64), magic_, shift_);

    // the unfused path, as transformer_attention_optimize.cu:728-748 calls it
    bool ok = bst_sgemm_nt(custream, d_nt, a_ptr, b_ptr, c_ptr, blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_,
                           head_state_, lut_heads, blocks);
    ok = ok && BlocksparseMaskedSoftmax<bhalf, bhalf2>(custream, d_nn, d_mask_t, c_ptr, y2_ptr, blk_size_, blocks, batch_dim,
                                                       heads_, ctx_blks_, lut_heads, blocks + ctx_blks_, nn_max, mask_heads, scale);
    ok = ok && bst_sgemm_xn(custream, d_nn, y2_ptr, v_ptr, o_ptr, blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_,
                            head_state_, lut_heads, blocks + ctx_blks_, NN_OP, magic_, shift_, nn_max);
    // the fused paths, as the *_fusion_test.cu programs call them
    ok = ok && fusion_attention2<float, float2>(custream, d_nt, a_ptr, b_ptr, c_ptr, d_nn, flag, flag1, d_mask_np, Max, Sum, y_ptr,
                                                blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_, head_state_,
                                                lut_heads, blocks, mask_heads, scale);
    ok = ok && fusion_attention<float, float2>(custream, d_nt, a_ptr, b_ptr, c_ptr, d_nn, flag, flag1, d_mask_np, Max, Sum, y_ptr,
                                               v_ptr, o2_ptr, blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, ctx_blks_, heads_,
                                               head_state_, lut_heads, blocks, mask_heads, scale, nn_max);
    // the backward, as transformer_attention_optimize.cu:924-964 calls it; tn_lut as generate_tn_lut builds it (ewops.h:675-701)
    std::vector<uint2> tn(ctx_blks_ + blocks, make_uint2(0, 0));
    {
        uint sum = ctx_blks_, cnt = ctx_blks_, at = ctx_blks_;
        for (uint c = 0; c < ctx_blks_; c++) {
            tn[c] = make_uint2(sum, cnt);
            sum += cnt;
            cnt--;
        }
        for (uint col = 0; col < ctx_blks_; col++)
            for (uint row = col; row < ctx_blks_; row++) tn[at++] = make_uint2(row * (row + 1) / 2 + col, row);
    }
    uint2 *d_tn;
    float *dv_ptr, *dk_ptr, *dq_ptr;
    bhalf *dw_ptr, *dx_ptr;
    cudaMalloc(&d_tn, sizeof(uint2) * tn.size());
    cudaMalloc(&dv_ptr, sizeof(float) * n_in);
    cudaMalloc(&dk_ptr, sizeof(float) * n_in);
    cudaMalloc(&dq_ptr, sizeof(float) * n_in);
    cudaMalloc(&dw_ptr, sizeof(bhalf) * n_blk);
    cudaMalloc(&dx_ptr, sizeof(bhalf) * n_blk);
    cudaMemcpy(d_tn, tn.data(), sizeof(uint2) * tn.size(), cudaMemcpyHostToDevice);
    const uint tn_max = ctx_blks_;
    float *do_ptr = v_ptr;   // all ones
    ok = ok && bst_sgemm_xn(custream, d_tn, y2_ptr, do_ptr, dv_ptr, blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_,
                            head_state_, lut_heads, blocks + ctx_blks_, TN_OP, magic_, shift_, tn_max);
    ok = ok && bst_sgemm_nt(custream, d_nt, do_ptr, v_ptr, dw_ptr, blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_,
                            head_state_, lut_heads, blocks);
    ok = ok && BlocksparseMaskedSoftmaxGrad<bhalf, bhalf2>(custream, d_nn, dw_ptr, y2_ptr, dx_ptr, blk_size_, blocks, batch_dim,
                                                           heads_, ctx_blks_, lut_heads, blocks + ctx_blks_, nn_max, scale);
    ok = ok && bst_sgemm_xn(custream, d_tn, dx_ptr, a_ptr, dk_ptr, blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_,
                            head_state_, lut_heads, blocks + ctx_blks_, TN_OP, magic_, shift_, tn_max);
    ok = ok && bst_sgemm_xn(custream, d_nn, dx_ptr, b_ptr, dq_ptr, blk_size_, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_,
                            head_state_, lut_heads, blocks + ctx_blks_, NN_OP, magic_, shift_, nn_max);
    // an unsupported block size is reported, not silently ignored
    const bool rejected = !bst_sgemm_nt(custream, d_nt, a_ptr, b_ptr, c_ptr, 16, blocks, batch_dim, ctx_blks_, ctx_blks_, heads_,
                                        head_state_, lut_heads, blocks);
    if (cudaDeviceSynchronize() != cudaSuccess || !ok || !rejected) {
        printf("FAIL: call failed (%s)\n", sfb_last_error());
        return 1;
    }

    std::vector<bhalf> s_h(n_blk);
    std::vector<float> y_h(n_blk), o_h(n_in), o2_h(n_in);
    cudaMemcpy(s_h.data(), c_ptr, sizeof(bhalf) * n_blk, cudaMemcpyDeviceToHost);
    cudaMemcpy(y_h.data(), y_ptr, sizeof(float) * n_blk, cudaMemcpyDeviceToHost);
    cudaMemcpy(o_h.data(), o_ptr, sizeof(float) * n_in, cudaMemcpyDeviceToHost);
    cudaMemcpy(o2_h.data(), o2_ptr, sizeof(float) * n_in, cudaMemcpyDeviceToHost);
    size_t bad = 0;
    for (size_t i = 0; i < n_blk; i++) bad += bf(s_h[i].x) != (float)head_state_;
    for (uint bh = 0; bh < batch_dim * heads_; bh++)
        for (uint k = 0; k < blocks; k++)
            for (uint r = 0; r < blk_size_; r++) {
                const uint kept = nt[k].x * blk_size_ + r + 1;   // causal: keys 0 .. row
                for (uint c = 0; c < blk_size_; c++) {
                    const bool keep = nt[k].x != nt[k].y || r >= c;
                    const float want = keep ? 1.0f / kept : 0.0f;
                    const float got = y_h[(((size_t)bh * blocks + k) * blk_size_ + r) * blk_size_ + c];
                    bad += fabsf(got - want) > 1e-6f;
                }
            }
    for (size_t i = 0; i < n_in; i++) bad += fabsf(o_h[i] - 1.0f) > 1e-2f;   // bf16 probabilities on this path
    for (size_t i = 0; i < n_in; i++) bad += fabsf(o2_h[i] - 1.0f) > 1e-5f;
    std::vector<float> dv_h(n_in), dk_h(n_in), dq_h(n_in);
    std::vector<bhalf> dw_h(n_blk);
    cudaMemcpy(dv_h.data(), dv_ptr, sizeof(float) * n_in, cudaMemcpyDeviceToHost);
    cudaMemcpy(dk_h.data(), dk_ptr, sizeof(float) * n_in, cudaMemcpyDeviceToHost);
    cudaMemcpy(dq_h.data(), dq_ptr, sizeof(float) * n_in, cudaMemcpyDeviceToHost);
    cudaMemcpy(dw_h.data(), dw_ptr, sizeof(bhalf) * n_blk, cudaMemcpyDeviceToHost);
    for (size_t i = 0; i < n_blk; i++) bad += bf(dw_h[i].x) != (float)head_state_;
    std::vector<double> tail(seq_len + 1, 0.0);   // tail[j] = sum over r >= j of 1/(r+1)
    for (int r = (int)seq_len - 1; r >= 0; r--) tail[r] = tail[r + 1] + 1.0 / (r + 1);
    const size_t row_elems = (size_t)heads_ * head_state_;
    for (size_t i = 0; i < n_in; i++) {
        const size_t key = (i / row_elems) % seq_len;
        bad += fabs(dv_h[i] - tail[key]) > 2e-2 * tail[key];
        bad += fabsf(dk_h[i]) > 0.5f;
        bad += fabsf(dq_h[i]) > 0.5f;
    }
    bad += sixteen_bit_additions();
    printf(bad ? "FAIL: %zu wrong values\n" : "PASS\n", bad);
    return bad ? 1 : 0;
}
