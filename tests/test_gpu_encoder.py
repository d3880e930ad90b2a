"""The encoder layer built around the path (attention + bias/residual/LayerNorm + bias/GELU from this
library, projections from the GEMM library or from this library's tcgen05 kernel) against the CPU oracle: the reference's operator order
(transformer_inference_part.cpp:210-239) with its matrixMulNNCPU standing in for cblas_sgemm."""
import importlib.util
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _encoder():
    spec = importlib.util.spec_from_file_location("sfb_encoder", os.path.join(ROOT, "sf-bert_b200", "encoder.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _cpu_layer(O, x, w, luts, heads, bs, order):
    B, L, hidden = x.shape
    d = hidden // heads
    m = B * L
    f32 = lambda t: t.float().cpu().numpy()
    mm = lambda a, b: (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)   # matmul.h:101-118 accumulates in double
    x2 = x.reshape(m, hidden)

    def attn(h):
        q, k, v = ((mm(h, f32(W)) + f32(b)).reshape(B, L, heads, d) for W, b in ((w.wq, w.bq), (w.wk, w.bk), (w.wv, w.bv)))
        return O.attention(q, k, v, luts, bs, np.float32(1 / np.sqrt(d)), want=("o",))["o"].reshape(m, hidden)

    if order == "pre":
        h = O.bias_residual_layernorm(x2, None, None, f32(w.g1), f32(w.be1))[0]
        a = mm(attn(h), f32(w.wo))
        h2, x1, _, _ = O.bias_residual_layernorm(a, f32(w.bo), x2, f32(w.g2), f32(w.be2))
        f = O.bias_gelu(mm(h2, f32(w.w1)), f32(w.b1))
        return (x1 + mm(f, f32(w.w2)) + f32(w.b2)).reshape(B, L, hidden)
    a = mm(attn(x2), f32(w.wo))
    x1 = O.bias_residual_layernorm(a, f32(w.bo), x2, f32(w.g1), f32(w.be1))[0]
    f = O.bias_gelu(mm(x1, f32(w.w1)), f32(w.b1))
    return O.bias_residual_layernorm(mm(f, f32(w.w2)), f32(w.b2), x1, f32(w.g2), f32(w.be2))[0].reshape(B, L, hidden)


@pytest.mark.parametrize("order", ["pre", "post"])
@pytest.mark.parametrize("dtype,bs,tol,proj", [("f32", 32, 2e-4, "library"), ("bf16", 64, 3e-2, "library"), ("bf16", 64, 3e-2, "tensor"),
                                               ("f16", 64, 3e-2, "tensor")])
def test_encoder_layer(sfb, oracle, order, dtype, bs, tol, proj):
    enc = _encoder()
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    B, L, heads, hidden, ffn = 2, 256, 4, 256, 512
    nb = L // bs
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, nb, bs, p0=2, p1=4)
    luts = oracle.lut_build(oracle.layout("stride", 1, nb, band=2, every=4))
    w = enc.EncoderLayerWeights(hidden, ffn, tdt, seed=5, std=0.05)
    for name in ("bq", "bk", "bv", "bo", "b1", "b2", "be1", "be2"):
        getattr(w, name).copy_(torch.from_numpy(oracle.fill_normal(tuple(getattr(w, name).shape), hash(name) % 1000, 0.1)))
    x = torch.from_numpy(oracle.fill_normal((B, L, hidden), 77)).cuda().to(tdt)
    y = enc.encoder_layer(sfb, x, w, lay, heads, order, proj).float().cpu().numpy()
    assert sfb.device_status() == 0
    want = _cpu_layer(oracle, x.float().cpu().numpy(), w, luts, heads, bs, order)
    assert np.abs(y - want).max() <= tol * max(1.0, np.abs(want).max())


def _fill_small_params(oracle, w):
    for name in ("bq", "bk", "bv", "bo", "b1", "b2", "be1", "be2"):
        getattr(w, name).copy_(torch.from_numpy(oracle.fill_normal(tuple(getattr(w, name).shape), hash(name) % 1000, 0.1)))


@pytest.mark.parametrize("name,dtype,L,heads,ffn,kind,kw,dev", [
    ("bert_base_stride", "f16", 4096, 12, 3072, "stride", dict(band=4, every=8), ("LAYOUT_STRIDE", dict(p0=4, p1=8))),
    ("bert_large_full", "bf16", 1024, 16, 4096, "full", dict(), ("LAYOUT_FULL", dict())),
])
def test_encoder_layer_at_the_benchmark_shapes(sfb, oracle, name, dtype, L, heads, ffn, kind, kw, dev):
    """One post-LN encoder layer at the two shapes the metric names (hidden 768 / FFN 3072 / L 4096 on the stride layout,
    hidden 1024 / FFN 4096 / L 1024 on the full layout), every kernel from this library, one sequence, every row checked
    against the oracle chain in the reference's operator order (transformer_inference_part.cpp:210-239).  The bar is
    element-wise: 3e-2 of the element plus 3e-2 of the output's root mean square (two 16-bit projections, the attention
    and two LayerNorms compound their roundings; the LayerNorm output has unit scale)."""
    enc = _encoder()
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    hidden, nb = heads * 64, L // 64
    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), 1, nb, 64, **dev[1])
    luts = oracle.lut_build(oracle.layout(kind, 1, nb, **kw))
    w = enc.EncoderLayerWeights(hidden, ffn, tdt, seed=11, std=0.03)
    _fill_small_params(oracle, w)
    x = torch.from_numpy(oracle.fill_normal((1, L, hidden), 78)).cuda().to(tdt)
    y = enc.encoder_layer(sfb, x, w, lay, heads, "post", "tensor").float().cpu().numpy()
    assert sfb.device_status() == 0
    want = _cpu_layer(oracle, x.float().cpu().numpy(), w, luts, heads, 64, "post")
    oracle.assert_close_16bit(y, want, rel=3e-2, floor_of_rms=1.0)


def test_embedding_two_layers_logits_at_the_bert_large_shape(sfb, oracle):
    """The stack either side of the attention at the BERT-large shape on one sequence: embedding lookup + positions
    (embedding.h:5-12, ewops.h:276-282), two post-LN layers, logits over the tied embedding table
    (transformer_inference_part.cpp:201-209, 241), against the oracle chain."""
    enc = _encoder()
    tdt = torch.bfloat16
    L, heads, hidden, ffn, vocab = 1024, 16, 1024, 4096, 30522
    vpad = (vocab + 15) // 16 * 16
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_FULL, 1, L // 64, 64)
    luts = oracle.lut_build(oracle.layout("full", 1, L // 64))
    g = torch.Generator(device="cuda").manual_seed(21)
    table = torch.zeros(vpad, hidden, device="cuda", dtype=tdt)
    table[:vocab] = (0.05 * torch.randn(vocab, hidden, device="cuda", generator=g)).to(tdt)
    pos = (0.05 * torch.randn(L, hidden, device="cuda", generator=g)).to(tdt)
    ids = torch.randint(0, vocab, (1, L), device="cuda", dtype=torch.int32, generator=g)
    ws = [enc.EncoderLayerWeights(hidden, ffn, tdt, seed=30 + i, std=0.03) for i in range(2)]
    for w in ws:
        _fill_small_params(oracle, w)
    x, bad = sfb.embedding(table, ids, pos)
    assert int(bad.item()) == 0
    x0 = x.clone()
    for w in ws:
        x = enc.encoder_layer(sfb, x, w, lay, heads, "post", "tensor")
    logits = sfb.linear_nt(x.view(L, hidden), table).float().cpu().numpy()
    assert sfb.device_status() == 0
    f32 = lambda t: t.float().cpu().numpy()
    h = oracle.embedding(f32(table), ids.cpu().numpy(), f32(pos))
    np.testing.assert_allclose(f32(x0), h, atol=1e-3, rtol=2.0 ** -8)   # one bf16 rounding of the sum
    h = f32(x0)
    for w in ws:
        h = _cpu_layer(oracle, h, w, luts, heads, 64, "post")
    oracle.assert_close_16bit(f32(x), h, rel=3e-2, floor_of_rms=1.0)
    want = (h.reshape(L, hidden).astype(np.float64) @ f32(table).astype(np.float64).T).astype(np.float32)
    oracle.assert_close_16bit(logits[:, :vocab], want[:, :vocab], rel=3e-2, floor_of_rms=1.0)
