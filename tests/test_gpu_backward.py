"""GPU parity of the backward operators of the block-sparse path (tn_lut builder, softmax gradient,
bst_sgemm_xn with TN_OP, and the reference's backward call sequence), called through the C ABI and
compared with the CPU oracle on the same seeded inputs.
Tolerances: LUT bit-exact; fp32 products max-abs 2e-5 * sqrt(contraction length); fp32 softmax
gradient 2e-6 absolute; 16-bit operands 2e-2 relative to the largest reference value."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from test_gpu_parity import LAYOUTS, CASES, TD, _u32, _make   # noqa: E402


@pytest.mark.parametrize("kind,kw,dev", LAYOUTS)
@pytest.mark.parametrize("heads,nb", [(1, 16), (4, 16), (1, 64), (2, 256), (1, 300)])
def test_tn_lut_bit_exact(sfb, oracle, kind, kw, dev, heads, nb):
    if kind == "bigbird" and heads > 1:
        pytest.skip("per-head random blocks give the heads different counts, which the LUT format cannot hold")
    lay, ref_layout, _ = _make(sfb, oracle, kind, kw, dev, heads, nb, 32)
    want = oracle.lut_build_tn(ref_layout)
    assert lay.tn_max == want["tn_max"]
    assert np.array_equal(_u32(lay.tn_lut), want["tn"])


def test_tn_lut_rejects_wrong_block_count(sfb):
    layout = torch.ones(1, 4, 4, dtype=torch.uint8, device="cuda")
    tn = torch.zeros(1, 4 + 15, 2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = sfb.lib.sfb_lut_build_tn(None, layout.data_ptr(), 1, 4, 15, tn.data_ptr(), None, status.data_ptr())
    assert rc == 0 and int(status.item()) == 1


def _blocks(oracle, shape, seed, dtype):
    a = torch.from_numpy(oracle.fill_normal(shape, seed)).cuda().to(TD[dtype])
    return a, a.float().cpu().numpy()


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "%s-bs%d" % (c[0], c[8]))
def test_softmax_grad(sfb, oracle, case, dtype):
    kind, kw, dev, hl, B, H, L, d, bs = case
    lay, _, luts = _make(sfb, oracle, kind, kw, dev, hl, L // bs, bs)
    shape = (B, H, luts["blocks"], bs, bs)
    dy, dyn = _blocks(oracle, shape, 300, dtype)
    # y: a probability-like tensor (positive, rows of the right scale)
    y = torch.from_numpy(np.abs(oracle.fill_normal(shape, 301)) / (bs * luts["nn_max"])).cuda().to(TD[dtype])
    yn = y.float().cpu().numpy()
    want = oracle.softmax_grad(dyn, yn, luts, bs, np.float32(0.125))
    got = sfb.masked_softmax_grad(dy, y, lay, 0.125).float().cpu().numpy()
    if dtype == "f32":
        np.testing.assert_allclose(got, want, rtol=0, atol=2e-6)
    else:
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "%s-bs%d-d%d" % (c[0], c[8], c[7]))
def test_spmm_tn(sfb, oracle, case, dtype):
    """C = A^T.B by block column with the reference's operand types: A in bf16 (or fp32), B and C in fp32."""
    kind, kw, dev, hl, B, H, L, d, bs = case
    lay, ref_layout, luts = _make(sfb, oracle, kind, kw, dev, hl, L // bs, bs)
    tn = oracle.lut_build_tn(ref_layout)["tn"]
    a, an = _blocks(oracle, (B, H, luts["blocks"], bs, bs), 310, dtype)
    b, bn = _blocks(oracle, (B, L, H, d), 311, "f32")
    want = oracle.spmm_tn(an, bn, tn, bs)
    got = sfb.bst_sgemm_tn(a, b, lay).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5 * np.sqrt(bs * tn[..., :L // bs, 1].max()) * 4)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("H_lut,nb,kind,kw,dev", [
    (1, 16, "stride", dict(band=4, every=8), ("LAYOUT_STRIDE", dict(p0=4, p1=8))),
    (1, 5, "full", dict(causal=1), ("LAYOUT_FULL", dict(causal=1))),            # odd number of block columns
    (1, 9, "local", dict(left=1, right=2), ("LAYOUT_LOCAL", dict(p0=1, p1=2))),
    (4, 16, "fixed", dict(stride=4), ("LAYOUT_FIXED", dict(p0=4))),             # per-head LUTs
    (1, 16, "bigbird", dict(window=1, g_first=1, g_last=1, nrand=3, seed=3), ("LAYOUT_BIGBIRD", dict(p0=1, p1=1, p2=1, p3=3, seed=3))),
    (1, 64, "full", dict(), ("LAYOUT_FULL", dict())),                           # columns of 64 blocks
])
def test_spmm_tn_on_tensor_cores(sfb, oracle, dtype, H_lut, nb, kind, kw, dev):
    """16-bit operands, 64x64 blocks, 64-wide heads: the tcgen05 kernel with the blocks as an MN-major A operand."""
    B, H, bs, d = 2, 4, 64, 64
    lay, ref_layout, luts = _make(sfb, oracle, kind, kw, dev, H_lut, nb, bs)
    tn = oracle.lut_build_tn(ref_layout)["tn"]
    a, an = _blocks(oracle, (B, H, luts["blocks"], bs, bs), 350, dtype)
    b, bn = _blocks(oracle, (B, nb * bs, H, d), 351, dtype)
    want = oracle.spmm_tn(an, bn, tn, bs)
    got = sfb.bst_sgemm_tn(a, b, lay)
    assert sfb.device_status() == 0
    assert got.dtype == TD[dtype]
    assert np.abs(got.float().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max()


def test_spmm_tn_empty_columns_on_tensor_cores(sfb, oracle):
    bs, nb = 64, 6
    layout = np.zeros((1, nb, nb), np.uint8)
    layout[0, :, 0] = 1
    layout[0, 2, 3] = 1                       # columns 1, 2, 4, 5 have no block; the pair (2, 3) is half empty
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), bs)
    a, an = _blocks(oracle, (1, 2, lay.blocks, bs, bs), 360, "bf16")
    b, bn = _blocks(oracle, (1, nb * bs, 2, 64), 361, "bf16")
    got = sfb.bst_sgemm_tn(a, b, lay).float().cpu().numpy()
    want = oracle.spmm_tn(an, bn, oracle.lut_build_tn(layout)["tn"], bs)
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    for c in (1, 2, 4, 5):
        assert float(np.abs(got[:, c * bs:(c + 1) * bs]).max()) == 0.0


def test_spmm_tn_empty_columns_give_zeros(sfb, oracle):
    bs, nb = 32, 6
    layout = np.zeros((1, nb, nb), np.uint8)
    layout[0, :, 0] = 1
    layout[0, 2, 3] = 1                       # columns 1, 2, 4, 5 have no block
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), bs)
    a, an = _blocks(oracle, (1, 2, lay.blocks, bs, bs), 320, "f32")
    b, bn = _blocks(oracle, (1, nb * bs, 2, 64), 321, "f32")
    got = sfb.bst_sgemm_tn(a, b, lay).cpu().numpy()
    want = oracle.spmm_tn(an, bn, oracle.lut_build_tn(layout)["tn"], bs)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-4)
    for c in (1, 2, 4, 5):
        assert float(np.abs(got[:, c * bs:(c + 1) * bs]).max()) == 0.0


@pytest.mark.parametrize("case", CASES[:4], ids=lambda c: "%s-bs%d-d%d" % (c[0], c[8], c[7]))
def test_backward_sequence_fp32(sfb, oracle, case):
    """The reference's backward call order (transformer_attention_optimize.cu:924-964) in fp32 against the
    oracle's chain; then against a finite-difference check of the forward oracle in one direction."""
    kind, kw, dev, hl, B, H, L, d, bs = case
    lay, ref_layout, luts = _make(sfb, oracle, kind, kw, dev, hl, L // bs, bs)
    tn = oracle.lut_build_tn(ref_layout)["tn"]
    scale = np.float32(1.0 / np.sqrt(d))
    q, k, v, do = (oracle.fill_normal((B, L, H, d), 330 + i) for i in range(4))
    tq, tk, tv, tdo = (torch.from_numpy(t).cuda() for t in (q, k, v, do))
    fwd = oracle.attention(q, k, v, luts, bs, scale, eps=0.0, want=("p", "o"))
    p = torch.from_numpy(fwd["p"]).cuda()
    dq, dk, dv = sfb.attention_backward(tq, tk, tv, p, tdo, lay, float(scale), s_dtype=torch.float32)

    w_dp = oracle.attention(do, v, v, luts, bs, scale, want=("s",))["s"]
    w_ds = oracle.softmax_grad(w_dp, fwd["p"], luts, bs, scale)
    w_dv = oracle.spmm_tn(fwd["p"], do, tn, bs)
    w_dk = oracle.spmm_tn(w_ds, q, tn, bs)
    w_dq = oracle.spmm_nn(w_ds, k, luts["nn"], bs)
    for got, want in ((dv, w_dv), (dk, w_dk), (dq, w_dq)):
        assert np.abs(got.cpu().numpy() - want).max() <= 1e-4 * max(1.0, np.abs(want).max())

    # directional derivative of <O, dO> along a random direction in Q, K, V (central difference in float64 terms)
    eps = 1e-2
    dirs = [oracle.fill_normal((B, L, H, d), 340 + i) for i in range(3)]
    lp = oracle.attention(q + eps * dirs[0], k + eps * dirs[1], v + eps * dirs[2], luts, bs, scale, eps=0.0, want=("o",))["o"]
    lm = oracle.attention(q - eps * dirs[0], k - eps * dirs[1], v - eps * dirs[2], luts, bs, scale, eps=0.0, want=("o",))["o"]
    num = float(((lp.astype(np.float64) - lm) * do).sum() / (2 * eps))
    ana = float((dq.cpu().numpy().astype(np.float64) * dirs[0]).sum() + (dk.cpu().numpy().astype(np.float64) * dirs[1]).sum() +
                (dv.cpu().numpy().astype(np.float64) * dirs[2]).sum())
    assert abs(num - ana) <= 2e-2 * max(1.0, abs(ana))


def test_backward_at_benchmark_size_properties(sfb, oracle):
    """BERT-base stride configuration at full size in bf16 blocks: properties that need no CPU pass over the
    whole tensor, and the oracle on one (batch, head) slice."""
    B, H, L, d, bs = 8, 12, 4096, 64, 64
    nb = L // bs
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, nb, bs, p0=4, p1=8)
    ref_layout = oracle.layout("stride", 1, nb, band=4, every=8)
    luts = oracle.lut_build(ref_layout)
    tn = oracle.lut_build_tn(ref_layout)["tn"]
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v, do = (torch.randn(B, L, H, d, device="cuda", generator=g) for _ in range(4))
    p = sfb.fused_sddmm_softmax(q.to(torch.bfloat16), k.to(torch.bfloat16), lay, 0.125, torch.bfloat16)
    # rows of dS sum to zero (up to the rounding of P): sum_j (dy_j - s) y_j = s (1 - sum_j y_j)
    dp = sfb.bst_sgemm_nt(do, v, lay, torch.bfloat16)
    ds = sfb.masked_softmax_grad(dp, p, lay, 0.125)
    b0, h0 = 3, 7
    dsn = ds[b0:b0 + 1, h0:h0 + 1].float().cpu().numpy()
    rows = oracle.blocks_to_dense(dsn, luts["nt"], nb, bs).sum(-1)
    scale_ref = np.abs(dsn).max()
    assert np.abs(rows).max() <= 0.05 * scale_ref * np.sqrt(12 * bs)
    want_ds = oracle.softmax_grad(dp[b0:b0 + 1, h0:h0 + 1].float().cpu().numpy(), p[b0:b0 + 1, h0:h0 + 1].float().cpu().numpy(),
                                  luts, bs, np.float32(0.125))
    assert np.abs(dsn - want_ds).max() <= 2e-2 * np.abs(want_ds).max()
    # dV with P := all ones / all-ones dO: every entry of a block column's rows is the column's number of kept query rows
    ones_p = torch.ones_like(p)
    ones_o = torch.ones_like(do)
    dv1 = sfb.bst_sgemm_tn(ones_p, ones_o, lay)
    counts = ref_layout[0].sum(axis=0).astype(np.float32) * bs
    got = dv1[b0, :, h0, 0].cpu().numpy().reshape(nb, bs)
    assert np.array_equal(got, np.repeat(counts[:, None], bs, axis=1))
    # the same product on the tensor cores (16-bit B and C): exact for ones
    dv1h = sfb.bst_sgemm_tn(ones_p, ones_o.to(torch.bfloat16), lay)
    assert np.array_equal(dv1h[b0, :, h0, 5].float().cpu().numpy().reshape(nb, bs), np.repeat(counts[:, None], bs, axis=1))
    dkh = sfb.bst_sgemm_tn(ds, q.to(torch.bfloat16), lay)
    want_dkh = oracle.spmm_tn(dsn, q.to(torch.bfloat16)[b0:b0 + 1, :, h0:h0 + 1].float().cpu().numpy(), tn, bs)
    assert np.abs(dkh[b0:b0 + 1, :, h0:h0 + 1].float().cpu().numpy() - want_dkh).max() <= 2e-2 * np.abs(want_dkh).max()
    assert sfb.device_status() == 0
    # one slice of dK = dS^T Q against the oracle
    dk = sfb.bst_sgemm_tn(ds, q, lay)
    want_dk = oracle.spmm_tn(dsn, q[b0:b0 + 1, :, h0:h0 + 1].cpu().numpy(), tn, bs)
    got_dk = dk[b0:b0 + 1, :, h0:h0 + 1].cpu().numpy()
    assert np.abs(got_dk - want_dk).max() <= 1e-4 * max(1.0, np.abs(want_dk).max())


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("H_lut,nb,kind,kw,dev", [
    (1, 16, "stride", dict(band=4, every=8), ("LAYOUT_STRIDE", dict(p0=4, p1=8))),
    (1, 5, "full", dict(causal=1), ("LAYOUT_FULL", dict(causal=1))),
    (4, 16, "fixed", dict(stride=4), ("LAYOUT_FIXED", dict(p0=4))),             # per-head LUTs
    (1, 40, "local", dict(left=1, right=2), ("LAYOUT_LOCAL", dict(p0=1, p1=2))),  # more blocks than one CTA's chunk
])
def test_fused_sddmm_softmax_grad(sfb, oracle, dtype, H_lut, nb, kind, kw, dev):
    """dS = P*(dO.V^T - rowdot(dO, O))*scale in one launch against the oracle's unfused chain on the same P."""
    B, H, bs, d = 2, 4, 64, 64
    lay, ref_layout, luts = _make(sfb, oracle, kind, kw, dev, H_lut, nb, bs)
    scale = np.float32(0.125)
    q, k, v, do = (torch.from_numpy(oracle.fill_normal((B, nb * bs, H, d), 370 + i)).cuda().to(TD[dtype]) for i in range(4))
    fwd = oracle.attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), luts, bs, scale, eps=0.0, want=("p",))
    p = torch.from_numpy(fwd["p"]).cuda().to(TD[dtype])
    pn, von, don = p.float().cpu().numpy(), v.float().cpu().numpy(), do.float().cpu().numpy()
    o = oracle.spmm_nn(pn, von, luts["nn"], bs)                              # the forward output that belongs to this (rounded) P
    delta = sfb.rowdot(do, torch.from_numpy(o).cuda().to(TD[dtype]))
    want_delta = (don * torch.from_numpy(o).to(TD[dtype]).float().numpy()).sum(-1)
    np.testing.assert_allclose(delta.cpu().numpy(), want_delta, rtol=0, atol=1e-4 * max(1.0, np.abs(want_delta).max()))
    ds = sfb.fused_sddmm_softmax_grad(do, v, p, delta, lay, float(scale)).float().cpu().numpy()
    assert sfb.device_status() == 0
    dp = oracle.attention(don, von, von, luts, bs, scale, want=("s",))["s"]
    want = oracle.softmax_grad(dp, pn, luts, bs, scale)
    assert np.abs(ds - want).max() <= 3e-2 * np.abs(want).max()
    # and the whole fused backward against the unfused one
    dq1, dk1, dv1 = sfb.attention_backward_fused(q, k, v, p, torch.from_numpy(o).cuda().to(TD[dtype]), do, lay, float(scale))
    dq0, dk0, dv0 = sfb.attention_backward(q, k, v, p, do, lay, float(scale), s_dtype=TD[dtype])
    for a, b in ((dq1, dq0), (dk1, dk0), (dv1, dv0)):
        assert float((a.float() - b.float()).abs().max()) <= 5e-2 * float(b.float().abs().max())

