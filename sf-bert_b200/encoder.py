"""One transformer encoder layer around the block-sparse attention path, in the operation order of the
reference's driver (transformer_attention_optimize.cu:688-801 / transformer_inference_part.cpp:210-239):

    pre-LN  (the reference):  h = LN(x); a = Attn(hWq+bq, hWk+bk, hWv+bv); x1 = x + aWo + bo;
                              h2 = LN(x1); x2 = x1 + GELU(h2 W1 + b1) W2 + b2
    post-LN (BERT):           x1 = LN(x + Attn(...)Wo + bo); x2 = LN(x1 + GELU(x1 W1 + b1) W2 + b2)

The dense projections are either plain library GEMMs (projections="library": torch.matmul -> cuBLAS; the
reference calls cublasSgemm there) or this library's tcgen05 kernel with the bias add / GELU in its epilogue
(projections="tensor", 16-bit operands).  Everything else -- attention, bias + residual + LayerNorm, bias +
GELU -- is this library's kernels.  Dropout is off (keep probability 1), as in every parity run."""
import math

import torch


class EncoderLayerWeights:
    def __init__(self, hidden, ffn, dtype, device="cuda", seed=0, std=0.02):
        g = torch.Generator(device=device).manual_seed(seed)
        rn = lambda *s: (torch.randn(*s, device=device, generator=g) * std).to(dtype)
        self.wq, self.wk, self.wv, self.wo = (rn(hidden, hidden) for _ in range(4))
        self.w1, self.w2 = rn(hidden, ffn), rn(ffn, hidden)
        z = lambda n: torch.zeros(n, device=device, dtype=torch.float32)
        self.bq, self.bk, self.bv, self.bo, self.b2 = (z(hidden) for _ in range(5))
        self.b1 = z(ffn)
        self.g1, self.g2 = (torch.ones(hidden, device=device, dtype=torch.float32) for _ in range(2))
        self.be1, self.be2 = z(hidden), z(hidden)
        self._qkv = None

    def fused_qkv(self):
        """[hidden, 3 * hidden] weight and [3 * hidden] bias of the three projections side by side (built on first use
        from wq, wk, wv, which stay the layer's parameters)."""
        if self._qkv is None:
            self._qkv = (torch.cat([self.wq, self.wk, self.wv], dim=1).contiguous(), torch.cat([self.bq, self.bk, self.bv]).contiguous())
        return self._qkv


def encoder_layer(sfb, x, w, lay, heads, ln_order="post", projections="library"):
    """x [B, L, hidden] -> [B, L, hidden].  `sfb` is the loaded package, `lay` a BlockLayout."""
    B, L, hidden = x.shape
    d = hidden // heads
    m = B * L
    x2d = x.reshape(m, hidden)
    scale = 1.0 / math.sqrt(d)
    if projections == "tensor":
        return _encoder_layer_tensor(sfb, x2d, w, lay, heads, ln_order, scale).view(B, L, hidden)

    def attn(h2d):
        q = torch.addmm(w.bq.to(h2d.dtype), h2d, w.wq).view(B, L, heads, d)
        k = torch.addmm(w.bk.to(h2d.dtype), h2d, w.wk).view(B, L, heads, d)
        v = torch.addmm(w.bv.to(h2d.dtype), h2d, w.wv).view(B, L, heads, d)
        return sfb.fused_attention(q, k, v, lay, scale).view(m, hidden)

    if ln_order == "pre":
        h, _, _, _ = sfb.bias_residual_layernorm(x2d, None, None, w.g1, w.be1)
        a = torch.mm(attn(h), w.wo)
        h2, x1, _, _ = sfb.bias_residual_layernorm(a, w.bo, x2d, w.g2, w.be2, want_sum=True)
        f = sfb.bias_gelu(torch.mm(h2, w.w1), w.b1)
        y = torch.addmm(w.b2.to(x.dtype), f, w.w2)
        return (x1 + y).view(B, L, hidden)
    a = torch.mm(attn(x2d), w.wo)
    x1, _, _, _ = sfb.bias_residual_layernorm(a, w.bo, x2d, w.g1, w.be1)
    f = sfb.bias_gelu(torch.mm(x1, w.w1), w.b1)
    y = torch.mm(f, w.w2)
    out, _, _, _ = sfb.bias_residual_layernorm(y, w.b2, x1, w.g2, w.be2)
    return out.view(B, L, hidden)


def _encoder_layer_tensor(sfb, x2d, w, lay, heads, ln_order, scale):
    """The same layer with every projection on sfb.linear: biases and the GELU ride in the GEMM epilogues, so the
    layer is 1 + 1 + 2 projections, the attention and two LayerNorm launches."""
    m, hidden = x2d.shape
    d = hidden // heads
    L = lay.nb * lay.block_size
    B = m // L

    def attn(h2d):
        # one product for the three projections (the activations are read once, and three times the column tiles fill
        # the last wave of the GEMM's grid better); the attention reads Q, K and V in place as column slices of the
        # [m, 3 * hidden] result, rows 3 * hidden elements apart
        wqkv, bqkv = w.fused_qkv()
        qkv = sfb.linear(h2d, wqkv, bqkv).view(B, L, 3, heads, d)
        return sfb.fused_attention_slice(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], lay, scale).view(m, hidden)

    if ln_order == "pre":
        h, _, _, _ = sfb.bias_residual_layernorm(x2d, None, None, w.g1, w.be1)
        a = sfb.linear(attn(h), w.wo)
        h2, x1, _, _ = sfb.bias_residual_layernorm(a, w.bo, x2d, w.g2, w.be2, want_sum=True)
        f = sfb.linear(h2, w.w1, w.b1, sfb.ACT_GELU)
        return x1 + sfb.linear(f, w.w2, w.b2)
    a = sfb.linear(attn(x2d), w.wo)
    x1, _, _, _ = sfb.bias_residual_layernorm(a, w.bo, x2d, w.g1, w.be1)
    f = sfb.linear(x1, w.w1, w.b1, sfb.ACT_GELU)
    y = sfb.linear(f, w.w2)
    out, _, _, _ = sfb.bias_residual_layernorm(y, w.b2, x1, w.g2, w.be2)
    return out

