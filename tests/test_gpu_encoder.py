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
