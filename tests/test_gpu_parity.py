"""GPU parity tests: every operator is called through the C ABI (via the package's ctypes binding)
and compared with the CPU oracle on the same seeded inputs.
Tolerances: LUT / mask arrays bit-exact; fp32 attention outputs max-abs 1e-5; 16-bit outputs
2e-2 relative; softmax row sums within 1e-3 of 1."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TD = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def _u32(t):
    return t.cpu().numpy().astype(np.int64).astype(np.uint32) if t.dtype == torch.int32 else t.cpu().numpy()


def _words(t, bs):
    a = t.cpu().numpy()
    return a.view(np.uint32) if bs == 32 else a.view(np.uint64)


LAYOUTS = [
    ("full", dict(causal=0), ("LAYOUT_FULL", dict())),
    ("full", dict(causal=1), ("LAYOUT_FULL", dict(causal=1))),
    ("fixed", dict(stride=4), ("LAYOUT_FIXED", dict(p0=4))),
    ("fixed", dict(stride=4, causal=1), ("LAYOUT_FIXED", dict(p0=4, causal=1))),
    ("stride", dict(band=4, every=8), ("LAYOUT_STRIDE", dict(p0=4, p1=8))),
    ("sawtooth", dict(chunks=4), ("LAYOUT_SAWTOOTH", dict(p0=4))),
    ("local", dict(left=8, right=8), ("LAYOUT_LOCAL", dict(p0=8, p1=8))),
    ("local", dict(left=1, right=0), ("LAYOUT_LOCAL", dict(p0=1, p1=0))),
    ("bigbird", dict(window=1, g_first=1, g_last=1, nrand=3, seed=1236),
     ("LAYOUT_BIGBIRD", dict(p0=1, p1=1, p2=1, p3=3, seed=1236))),
]


def _make(sfb, oracle, kind, kw, dev, heads, nb, bs):
    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), heads, nb, bs, **dev[1])
    ref_layout = oracle.layout(kind, heads, nb, **kw)
    return lay, ref_layout, oracle.lut_build(ref_layout)


@pytest.mark.parametrize("kind,kw,dev", LAYOUTS)
@pytest.mark.parametrize("heads,nb", [(1, 16), (4, 16), (1, 64), (2, 256)])
def test_layout_and_lut_bit_exact(sfb, oracle, kind, kw, dev, heads, nb):
    if kind == "bigbird" and heads > 1:
        pytest.skip("per-head random blocks give the heads different counts, which the LUT format cannot hold")
    lay, ref_layout, luts = _make(sfb, oracle, kind, kw, dev, heads, nb, 32)
    assert np.array_equal(lay.layout.cpu().numpy(), ref_layout)
    assert lay.blocks == luts["blocks"] and lay.nn_max == luts["nn_max"]
    assert np.array_equal(_u32(lay.nt_lut), luts["nt"])
    assert np.array_equal(_u32(lay.nn_lut), luts["nn"])
    assert np.array_equal(_u32(lay.rblk_lut), luts["rblk"])


@pytest.mark.parametrize("prog,nb,pred,ctx", [("stride_fusion_test", 32, "MASK_CAUSAL_ALL", 0),
                                               ("local_fusion_test", 32, "MASK_LOCAL", 32),
                                               ("no_fusion_test", 10, "MASK_CAUSAL_DIAG", 0),
                                               ("big_bird_fusion_test", 10, None, 0)])
def test_lut_and_mask_match_reference_uploads(sfb, prog, nb, pred, ctx):
    """Device builder against the arrays the reference's own test programs upload."""
    g = np.load(os.path.join(GOLD, "ref_uploads.npz"))
    nt_ref = g[prog + "/nt_lut"].reshape(-1, 2)
    layout = np.zeros((1, nb, nb), np.uint8)
    layout[0, nt_ref[:, 0], nt_ref[:, 1]] = 1
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), 32)
    assert np.array_equal(_u32(lay.nt_lut)[0], nt_ref)
    assert np.array_equal(_u32(lay.nn_lut)[0], g[prog + "/nn_lut"].reshape(-1, 2))
    if prog + "/rblk_lut" in g:
        assert np.array_equal(_u32(lay.rblk_lut)[0], g[prog + "/rblk_lut"].reshape(-1, 2))
    if pred:
        lay.pack_mask(getattr(sfb, pred), ctx)
        assert np.array_equal(_words(lay.mask_np, 32).ravel(), g[prog + "/mask_np"])
        assert np.array_equal(_words(lay.mask_t, 32).ravel(), g[prog + "/mask_t"])


@pytest.mark.parametrize("bs", [32, 64])
@pytest.mark.parametrize("pred,ctx", [("MASK_ALL", 0), ("MASK_CAUSAL_DIAG", 0), ("MASK_CAUSAL_ALL", 0), ("MASK_LOCAL", 96)])
def test_mask_pack_bit_exact(sfb, oracle, bs, pred, ctx):
    lay, _, luts = _make(sfb, oracle, "local", dict(left=2, right=1), ("LAYOUT_LOCAL", dict(p0=2, p1=1)), 2, 12, bs)
    lay.pack_mask(getattr(sfb, pred), ctx)
    m_np, m_t = oracle.mask_pack(luts["nt"], bs, getattr(oracle, pred), ctx)
    assert np.array_equal(_words(lay.mask_np, bs), m_np)
    assert np.array_equal(_words(lay.mask_t, bs), m_t)


def test_unequal_head_counts_are_rejected(sfb):
    layout = torch.zeros(2, 4, 4, dtype=torch.uint8, device="cuda")
    layout[0, 0, 0] = 1
    layout[1, 0, :2] = 1
    with pytest.raises(sfb.SfbError):
        sfb.BlockLayout(layout, 32)


# --------------------------------------------------------------------------------------------
def _inputs(oracle, B, L, H, d, seed, dtype):
    q, k, v = (oracle.fill_normal((B, L, H, d), seed + i) for i in range(3))
    tq, tk, tv = (torch.from_numpy(t).cuda().to(TD[dtype]) for t in (q, k, v))
    # the oracle sees the rounded operands
    return (tq, tk, tv), tuple(t.float().cpu().numpy() for t in (tq, tk, tv))


CASES = [
    # kind, kw, dev, H_lut, B, H, L, d, bs
    ("fixed", dict(stride=4), ("LAYOUT_FIXED", dict(p0=4)), 4, 1, 4, 512, 64, 32),       # benchmark config 1
    ("stride", dict(band=4, every=8), ("LAYOUT_STRIDE", dict(p0=4, p1=8)), 1, 2, 3, 1024, 64, 64),
    ("bigbird", dict(window=1, g_first=1, g_last=1, nrand=3, seed=7),
     ("LAYOUT_BIGBIRD", dict(p0=1, p1=1, p2=1, p3=3, seed=7)), 1, 1, 2, 1024, 64, 64),
    ("local", dict(left=2, right=2), ("LAYOUT_LOCAL", dict(p0=2, p1=2)), 1, 1, 2, 512, 128, 32),
    ("full", dict(), ("LAYOUT_FULL", dict()), 1, 2, 2, 256, 40, 32),                       # d not a multiple of 32
    ("sawtooth", dict(chunks=3), ("LAYOUT_SAWTOOTH", dict(p0=3)), 1, 1, 1, 384, 128, 64),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "%s-bs%d-d%d" % (c[0], c[8], c[7]))
def test_unfused_pipeline_fp32(sfb, oracle, case):
    """bst_sgemm_nt -> BlocksparseMaskedSoftmax -> bst_sgemm_xn with the reference's types:
    fp32 operands, bf16 scores and probabilities."""
    kind, kw, dev, hl, B, H, L, d, bs = case
    lay, _, luts = _make(sfb, oracle, kind, kw, dev, hl, L // bs, bs)
    (q, k, v), (qn, kn, vn) = _inputs(oracle, B, L, H, d, 100, "f32")
    scale = float(1.0 / np.sqrt(d))
    ref = oracle.attention(qn, kn, vn, luts, bs, np.float32(scale), eps=0.0, round_s_bf16=True)

    s = sfb.bst_sgemm_nt(q, k, lay, torch.bfloat16)
    s_f = s.float().cpu().numpy()
    assert np.abs(s_f - ref["s"]).max() <= np.abs(ref["s"]).max() * 2.0 ** -7   # one bf16 step
    s32 = sfb.bst_sgemm_nt(q, k, lay, torch.float32).cpu().numpy()
    full = oracle.attention(qn, kn, vn, luts, bs, np.float32(scale), eps=0.0, want=("s",))["s"]
    np.testing.assert_allclose(s32, full, rtol=0, atol=2e-5 * np.sqrt(d))

    # softmax on exactly the oracle's rounded scores
    s_in = torch.from_numpy(oracle.to_bhalf(ref["s"]).view(np.int16)).cuda().view(torch.bfloat16)
    p32 = sfb.masked_softmax(s_in, lay, scale, torch.float32).cpu().numpy()
    np.testing.assert_allclose(p32, ref["p"], rtol=0, atol=2e-6)
    dense = oracle.blocks_to_dense(p32, luts["nt"], L // bs, bs)
    np.testing.assert_allclose(dense.sum(-1), 1.0, atol=1e-3)
    p16 = sfb.masked_softmax(s_in, lay, scale, torch.bfloat16)
    assert np.abs(p16.float().cpu().numpy() - ref["p"]).max() <= ref["p"].max() * 2.0 ** -7

    o = sfb.bst_sgemm_xn(p16, v, lay).cpu().numpy()
    p16n = p16.float().cpu().numpy()
    want = np.zeros_like(vn)
    nb = L // bs
    for h in range(H):
        nt = luts["nt"][h if hl > 1 else 0]
        for kk in range(luts["blocks"]):
            i, j = int(nt[kk, 0]), int(nt[kk, 1])
            want[:, i * bs:(i + 1) * bs, h] += np.einsum("brc,bcd->brd", p16n[:, h, kk], vn[:, j * bs:(j + 1) * bs, h])
    np.testing.assert_allclose(o, want, rtol=0, atol=2e-5)
    np.testing.assert_allclose(o, ref["o"], rtol=0, atol=2e-2 * np.abs(ref["o"]).max())


@pytest.mark.parametrize("case", CASES, ids=lambda c: "%s-bs%d-d%d" % (c[0], c[8], c[7]))
def test_fused_fp32(sfb, oracle, case):
    kind, kw, dev, hl, B, H, L, d, bs = case
    lay, _, luts = _make(sfb, oracle, kind, kw, dev, hl, L // bs, bs)
    (q, k, v), (qn, kn, vn) = _inputs(oracle, B, L, H, d, 200, "f32")
    scale = float(1.0 / np.sqrt(d))
    ref = oracle.attention(qn, kn, vn, luts, bs, np.float32(scale))          # the CPU reference semantics (eps 1e-6)
    p = sfb.fused_sddmm_softmax(q, k, lay, scale, torch.float32).cpu().numpy()
    assert np.abs(p - ref["p"]).max() < 1e-5
    np.testing.assert_allclose(oracle.blocks_to_dense(p, luts["nt"], L // bs, bs).sum(-1), 1.0, atol=1e-3)
    o = sfb.fused_attention(q, k, v, lay, scale).cpu().numpy()
    assert np.abs(o - ref["o"]).max() < 1e-5


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "%s-bs%d-d%d" % (c[0], c[8], c[7]))
def test_fused_16bit(sfb, oracle, case, dtype):
    kind, kw, dev, hl, B, H, L, d, bs = case
    lay, _, luts = _make(sfb, oracle, kind, kw, dev, hl, L // bs, bs)
    (q, k, v), (qn, kn, vn) = _inputs(oracle, B, L, H, d, 300, dtype)
    scale = float(1.0 / np.sqrt(d))
    ref = oracle.attention(qn, kn, vn, luts, bs, np.float32(scale))
    o = sfb.fused_attention(q, k, v, lay, scale).float().cpu().numpy()
    oracle.assert_close_16bit(o, ref["o"], 2e-2)
    p = sfb.fused_sddmm_softmax(q, k, lay, scale, TD[dtype]).float().cpu().numpy()
    # probabilities: 2e-2 relative per element, with a floor of 2e-2 of their root mean square
    oracle.assert_close_16bit(p, ref["p"], 2e-2, floor_of_rms=1.0)
    np.testing.assert_allclose(oracle.blocks_to_dense(p, luts["nt"], L // bs, bs).sum(-1), 1.0, atol=2e-2)
    s = sfb.bst_sgemm_nt(q, k, lay, torch.float32).cpu().numpy()
    np.testing.assert_allclose(s, ref["s"], rtol=0, atol=1e-3 * np.sqrt(d))


@pytest.mark.parametrize("bs,pred,ctx", [(32, "MASK_CAUSAL_DIAG", 0), (64, "MASK_CAUSAL_DIAG", 0),
                                          (32, "MASK_LOCAL", 48), (64, "MASK_CAUSAL_ALL", 0)])
def test_element_masks(sfb, oracle, bs, pred, ctx):
    B, H, L, d = 2, 2, 8 * bs, 64
    lay, _, luts = _make(sfb, oracle, "full", dict(causal=1), ("LAYOUT_FULL", dict(causal=1)), 1, L // bs, bs)
    lay.pack_mask(getattr(sfb, pred), ctx)
    m_np, _ = oracle.mask_pack(luts["nt"], bs, getattr(oracle, pred), ctx)
    (q, k, v), (qn, kn, vn) = _inputs(oracle, B, L, H, d, 400, "f32")
    scale = float(1.0 / np.sqrt(d))
    ref = oracle.attention(qn, kn, vn, luts, bs, np.float32(scale), mask_np=m_np)
    o = sfb.fused_attention(q, k, v, lay, scale, use_mask=True).cpu().numpy()
    assert np.abs(o - ref["o"]).max() < 1e-5
    p = sfb.fused_sddmm_softmax(q, k, lay, scale, torch.float32, use_mask=True).cpu().numpy()
    assert np.abs(p - ref["p"]).max() < 1e-5
    s = sfb.bst_sgemm_nt(q, k, lay, torch.float32)
    p2 = sfb.masked_softmax(s, lay, scale, torch.float32, use_mask=True).cpu().numpy()
    assert np.abs(p2 - ref["p"]).max() < 1e-5


def test_causal_dense_matches_reference_cpu_golden(sfb, oracle):
    """GPU against outputs of the reference's own CPU operators (tests/golden/ref_cpu_attention.npz)."""
    g = np.load(os.path.join(GOLD, "ref_cpu_attention.npz"))
    B, L, H, d = (int(x) for x in g["attn/shape"])
    bs = 32
    (q, k, v) = (torch.from_numpy(oracle.fill_normal((B, L, H, d), int(s))).cuda() for s in g["attn/seeds"])
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_FULL, 1, L // bs, bs, causal=1).pack_mask(sfb.MASK_CAUSAL_DIAG)
    o = sfb.fused_attention(q, k, v, lay, float(1 / np.sqrt(d)), use_mask=True).cpu().numpy()
    assert np.abs(o - g["attn/o"]).max() < 1e-5


def test_all_ones_known_answer(sfb, oracle):
    """Q = K = 1 gives every score d and uniform rows (fixed_fusion_test.cu:263-268, test.cu:382-386)."""
    B, H, L, d, bs = 2, 4, 320, 128, 32
    lay, _, luts = _make(sfb, oracle, "fixed", dict(stride=4, causal=1), ("LAYOUT_FIXED", dict(p0=4, causal=1)), 4, L // bs, bs)
    ones = torch.ones(B, L, H, d, device="cuda")
    s = sfb.bst_sgemm_nt(ones, ones, lay, torch.bfloat16).float()
    assert bool((s == d).all())
    p = sfb.fused_sddmm_softmax(ones, ones, lay, float(1 / np.sqrt(d)), torch.float32).cpu().numpy()
    for h in range(H):
        nn = luts["nn"][h]
        for i in range(L // bs):
            cnt = int(nn[i, 1])
            blk = int(nn[int(nn[i, 0]), 0])
            np.testing.assert_allclose(p[:, h, blk], 1.0 / (cnt * bs), rtol=1e-5)
    o = sfb.fused_attention(ones, ones, ones, lay).cpu().numpy()
    np.testing.assert_allclose(o, 1.0, rtol=1e-5)


def test_empty_block_rows_give_zero_output(sfb, oracle):
    bs, nb, B, H, d = 32, 6, 1, 2, 64
    layout = np.zeros((1, nb, nb), np.uint8)
    layout[0, 0, 0] = layout[0, 2, 1] = layout[0, 2, 5] = layout[0, 5, 3] = 1   # rows 1, 3, 4 are empty
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), bs)
    luts = oracle.lut_build(layout)
    (q, k, v), (qn, kn, vn) = _inputs(oracle, B, nb * bs, H, d, 500, "f32")
    ref = oracle.attention(qn, kn, vn, luts, bs, np.float32(0.125))
    o = torch.full_like(q, 7.0)
    sfb.fused_attention(q, k, v, lay, 0.125, out=o)
    assert np.abs(o.cpu().numpy() - ref["o"]).max() < 1e-5
    assert float(o[:, bs:2 * bs].abs().max()) == 0.0
    p = sfb.fused_sddmm_softmax(q, k, lay, 0.125, torch.bfloat16)
    o2 = sfb.bst_sgemm_xn(p, v, lay)
    assert float(o2[:, 3 * bs:5 * bs].abs().max()) == 0.0


@pytest.mark.parametrize("dtype,m,hidden", [("f32", 300, 768), ("f32", 64, 1024), ("bf16", 257, 1024), ("f16", 128, 768),
                                             ("f32", 33, 320), ("bf16", 16, 4096)])
def test_bias_residual_layernorm(sfb, oracle, dtype, m, hidden):
    x = torch.from_numpy(oracle.fill_normal((m, hidden), 31)).cuda().to(TD[dtype])
    r = torch.from_numpy(oracle.fill_normal((m, hidden), 32)).cuda().to(TD[dtype])
    b = torch.from_numpy(oracle.fill_normal((hidden,), 33, 0.02)).cuda()
    g = torch.from_numpy(1.0 + oracle.fill_normal((hidden,), 34, 0.1)).cuda()
    be = torch.from_numpy(oracle.fill_normal((hidden,), 35, 0.1)).cuda()
    y, summed, mean, rstd = sfb.bias_residual_layernorm(x, b, r, g, be, want_sum=True)
    wy, ws, wm, wr = oracle.bias_residual_layernorm(x.float().cpu().numpy(), b.cpu().numpy(), r.float().cpu().numpy(),
                                                    g.cpu().numpy(), be.cpu().numpy())
    tol = 1e-5 if dtype == "f32" else 2e-2
    np.testing.assert_allclose(mean.cpu().numpy(), wm, atol=1e-5)
    np.testing.assert_allclose(rstd.cpu().numpy(), wr, rtol=1e-5)
    assert np.abs(summed.float().cpu().numpy() - ws).max() <= tol * max(1.0, np.abs(ws).max())
    assert np.abs(y.float().cpu().numpy() - wy).max() <= tol * max(1.0, np.abs(wy).max())
    y2, _, _, _ = sfb.bias_residual_layernorm(x, None, None, g, be)
    wy2 = oracle.bias_residual_layernorm(x.float().cpu().numpy(), None, None, g.cpu().numpy(), be.cpu().numpy())[0]
    assert np.abs(y2.float().cpu().numpy() - wy2).max() <= tol * max(1.0, np.abs(wy2).max())


@pytest.mark.parametrize("dtype,m,hidden", [("f16", 5000, 768), ("bf16", 4736, 1024), ("f32", 6001, 768),
                                             ("bf16", 9473, 320), ("f16", 4741, 2048), ("bf16", 20003, 8)])
def test_layernorm_many_rows(sfb, oracle, dtype, m, hidden):
    """More rows than the fixed grid has warps (the warps loop), ragged last round, rows narrower than a warp."""
    x = torch.from_numpy(oracle.fill_normal((m, hidden), 41)).cuda().to(TD[dtype])
    r = torch.from_numpy(oracle.fill_normal((m, hidden), 42)).cuda().to(TD[dtype])
    b = torch.from_numpy(oracle.fill_normal((hidden,), 43, 0.02)).cuda()
    g = torch.from_numpy(1.0 + oracle.fill_normal((hidden,), 44, 0.1)).cuda()
    be = torch.from_numpy(oracle.fill_normal((hidden,), 45, 0.1)).cuda()
    y, summed, mean, rstd = sfb.bias_residual_layernorm(x, b, r, g, be, want_sum=True)
    wy, ws, wm, wr = oracle.bias_residual_layernorm(x.float().cpu().numpy(), b.cpu().numpy(), r.float().cpu().numpy(),
                                                    g.cpu().numpy(), be.cpu().numpy())
    tol = 1e-5 if dtype == "f32" else 2e-2
    np.testing.assert_allclose(mean.cpu().numpy(), wm, atol=1e-5)
    np.testing.assert_allclose(rstd.cpu().numpy(), wr, rtol=1e-5)
    assert np.abs(summed.float().cpu().numpy() - ws).max() <= tol * max(1.0, np.abs(ws).max())
    assert np.abs(y.float().cpu().numpy() - wy).max() <= tol * max(1.0, np.abs(wy).max())


def test_layernorm_matches_reference_cpu_golden(sfb, oracle):
    g = np.load(os.path.join(GOLD, "ref_cpu_attention.npz"))
    m, hidden = (int(x) for x in g["ln/shape"])
    sx, sr, sb, sg, sbe = (int(x) for x in g["ln/seeds"])
    x = torch.from_numpy(oracle.fill_normal((m, hidden), sx)).cuda()
    r = torch.from_numpy(oracle.fill_normal((m, hidden), sr)).cuda()
    b = torch.from_numpy(oracle.fill_normal((hidden,), sb, 0.02)).cuda()
    gain = torch.from_numpy(1.0 + oracle.fill_normal((hidden,), sg, 0.1)).cuda()
    beta = torch.from_numpy(oracle.fill_normal((hidden,), sbe, 0.1)).cuda()
    y, _, mean, rstd = sfb.bias_residual_layernorm(x, b, r, gain, beta)
    np.testing.assert_allclose(y.cpu().numpy(), g["ln/y"], atol=1e-5)
    np.testing.assert_allclose(mean.cpu().numpy(), g["ln/mean"], atol=1e-6)
    np.testing.assert_allclose(rstd.cpu().numpy(), g["ln/rstd"], rtol=1e-5)


@pytest.mark.parametrize("dtype,m,n", [("f32", 100, 3072), ("bf16", 64, 4096), ("f16", 33, 768)])
def test_bias_gelu(sfb, oracle, dtype, m, n):
    x = torch.from_numpy(oracle.fill_normal((m, n), 61, 2.0)).cuda().to(TD[dtype])
    b = torch.from_numpy(oracle.fill_normal((n,), 62, 0.5)).cuda()
    want = oracle.bias_gelu(x.float().cpu().numpy(), b.cpu().numpy())
    got = sfb.bias_gelu(x, b).float().cpu().numpy()
    tol = 2e-6 if dtype == "f32" else 2e-2
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("bs", [32, 64])
@pytest.mark.parametrize("longest", [1, 4, 5, 8, 9, 12, 13, 16, 17, 18, 19, 20, 21, 33])
def test_masked_softmax_every_row_length_variant(sfb, oracle, bs, longest):
    """Rows of 1 .. `longest` kept blocks in one layout: the caller's max_lut picks the softmax variant (rows held in
    registers in 4, 8, 12, 16, 18 or 20 block slots, whole or quarter block-rows per CTA, or streamed beyond that), and
    every variant must give the same probabilities: bf16 scores against a float64 softmax of the same values, bf16 and
    fp32 outputs, with and without an element mask."""
    nb = 36
    rng = np.random.default_rng(700 + longest)
    layout = np.zeros((1, nb, nb), np.uint8)
    for i in range(nb):
        n = longest if i == nb // 2 else 1 + (i * 7) % longest
        layout[0, i, rng.choice(nb, size=n, replace=False)] = 1
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), bs)
    luts = oracle.lut_build(layout)
    assert int(lay.nn_max) == longest
    B, H = 2, 3
    gen = torch.Generator(device="cuda").manual_seed(41)
    s = (3.0 * torch.randn(B, H, luts["blocks"], bs, bs, device="cuda", generator=gen)).to(torch.bfloat16)
    sn = s.float().cpu().numpy().astype(np.float64)
    nt = luts["nt"][0]
    for use_mask in (False, True):
        keep = np.ones((luts["blocks"], bs, bs), bool)
        if use_mask:
            lay.pack_mask(sfb.MASK_CAUSAL_DIAG, 0)
            for kblk in range(luts["blocks"]):
                if nt[kblk][0] == nt[kblk][1]:
                    keep[kblk] = np.tril(np.ones((bs, bs), bool))
        ref = np.zeros_like(sn)
        for i in range(nb):
            ids = [kblk for kblk in range(luts["blocks"]) if nt[kblk][0] == i]
            x = np.concatenate([np.where(keep[kblk], sn[:, :, kblk] * 0.125, -np.inf) for kblk in ids], axis=-1)
            mx = x.max(-1, keepdims=True)
            e = np.exp(x - np.where(np.isfinite(mx), mx, 0.0))
            den = e.sum(-1, keepdims=True)
            pr = np.where(den > 0, e / np.where(den > 0, den, 1.0), 0.0)
            for j, kblk in enumerate(ids):
                ref[:, :, kblk] = pr[..., j * bs:(j + 1) * bs]
        p32 = sfb.masked_softmax(s, lay, 0.125, torch.float32, use_mask=use_mask).cpu().numpy()
        np.testing.assert_allclose(p32, ref, rtol=0, atol=3e-6)
        p16 = sfb.masked_softmax(s, lay, 0.125, torch.bfloat16, use_mask=use_mask).float().cpu().numpy()
        assert np.abs(p16 - ref).max() <= 2.0 ** -8

