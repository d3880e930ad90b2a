"""Parity of the tcgen05 fused attention kernel (16-bit operands, 64x64 blocks, 64-wide heads),
called through the C ABI, against the CPU oracle -- small cases element by element, the five
benchmark configurations at full size through slices and size-independent properties."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TD = {"bf16": torch.bfloat16, "f16": torch.float16}
REL = 2e-2   # 16-bit operands, fp32 accumulation


def _rand(oracle, shape, seed, dtype):
    return torch.from_numpy(oracle.fill_normal(shape, seed)).cuda().to(TD[dtype])


def _check_slice(sfb, oracle, lay, luts, q, k, v, o, b, h, scale, mask_np=None):
    """Oracle on one (batch, head) slice of the full-size problem."""
    sl = lambda t: t[b:b + 1, :, h:h + 1].float().cpu().numpy()
    one = dict(luts)
    if luts["nt"].shape[0] > 1:
        one = dict(nt=luts["nt"][h:h + 1], nn=luts["nn"][h:h + 1], blocks=luts["blocks"])
        if mask_np is not None:
            mask_np = mask_np[h:h + 1]
    ref = oracle.attention(sl(q), sl(k), sl(v), one, 64, np.float32(scale), mask_np=mask_np, want=("o",))["o"]
    got = o[b:b + 1, :, h:h + 1].float().cpu().numpy()
    oracle.assert_close_16bit(got, ref, REL)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("nb,kind,kw,dev", [
    (1, "full", dict(), ("LAYOUT_FULL", dict())),
    (2, "full", dict(), ("LAYOUT_FULL", dict())),
    (5, "full", dict(causal=1), ("LAYOUT_FULL", dict(causal=1))),       # odd number of block-rows
    (9, "local", dict(left=1, right=2), ("LAYOUT_LOCAL", dict(p0=1, p1=2))),
    (16, "bigbird", dict(window=1, g_first=1, g_last=1, nrand=3, seed=3),
     ("LAYOUT_BIGBIRD", dict(p0=1, p1=1, p2=1, p3=3, seed=3))),
    (64, "full", dict(), ("LAYOUT_FULL", dict())),                       # rows of 64 blocks
])
def test_small_cases_elementwise(sfb, oracle, dtype, nb, kind, kw, dev):
    B, H, L, d = 2, 2, nb * 64, 64
    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), 1, nb, 64, **dev[1])
    luts = oracle.lut_build(oracle.layout(kind, 1, nb, **kw))
    q, k, v = (_rand(oracle, (B, L, H, d), 600 + i, dtype) for i in range(3))
    o = sfb.fused_attention(q, k, v, lay, 0.125)
    assert sfb.device_status() == 0
    ref = oracle.attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), luts, 64,
                           np.float32(0.125), want=("o",))["o"]
    oracle.assert_close_16bit(o.float().cpu().numpy(), ref, REL)


@pytest.mark.parametrize("pred,ctx", [("MASK_CAUSAL_DIAG", 0), ("MASK_LOCAL", 100)])
def test_element_masks_on_tensor_cores(sfb, oracle, pred, ctx):
    B, H, nb, d = 1, 3, 7, 64
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_FULL, 1, nb, 64, causal=1).pack_mask(getattr(sfb, pred), ctx)
    luts = oracle.lut_build(oracle.layout("full", 1, nb, causal=1))
    m_np, _ = oracle.mask_pack(luts["nt"], 64, getattr(oracle, pred), ctx)
    q, k, v = (_rand(oracle, (B, nb * 64, H, d), 700 + i, "bf16") for i in range(3))
    o = sfb.fused_attention(q, k, v, lay, 0.125, use_mask=True)
    assert sfb.device_status() == 0
    ref = oracle.attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), luts, 64,
                           np.float32(0.125), mask_np=m_np, want=("o",))["o"]
    assert np.abs(o.float().cpu().numpy() - ref).max() <= REL * np.abs(ref).max()


def test_per_head_luts_and_empty_rows(sfb, oracle):
    H, nb, d = 3, 6, 64
    layout = np.zeros((H, nb, nb), np.uint8)
    rng = np.random.RandomState(0)
    for h in range(H):
        # 9 blocks per head, rows 1 and 4 left empty
        cells = [(i, j) for i in (0, 2, 3, 5) for j in range(nb)]
        for idx in rng.choice(len(cells), 9, replace=False):
            layout[h][cells[idx]] = 1
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), 64)
    luts = oracle.lut_build(layout)
    q, k, v = (_rand(oracle, (2, nb * 64, H, d), 800 + i, "bf16") for i in range(3))
    o = torch.full_like(q, 3.0)
    sfb.fused_attention(q, k, v, lay, 0.125, out=o)
    assert sfb.device_status() == 0
    ref = oracle.attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), luts, 64,
                           np.float32(0.125), want=("o",))["o"]
    assert np.abs(o.float().cpu().numpy() - ref).max() <= REL * np.abs(ref).max()
    assert float(o[:, 64:128].abs().max()) == 0.0 and float(o[:, 256:320].abs().max()) == 0.0


def test_all_ones_known_answer_16bit(sfb):
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, 16, 64, p0=4, p1=8)
    ones = torch.ones(1, 1024, 2, 64, device="cuda", dtype=torch.float16)
    o = sfb.fused_attention(ones, ones, ones, lay).float()
    assert float((o - 1.0).abs().max()) < 2e-3


FULL = [
    # name, dtype, B, H, L, layout
    ("stride_bertbase", "f16", 8, 12, 4096, ("stride", dict(band=4, every=8)), ("LAYOUT_STRIDE", dict(p0=4, p1=8))),
    ("bigbird", "bf16", 16, 12, 4096, ("bigbird", dict(window=1, g_first=1, g_last=1, nrand=3, seed=1236)),
     ("LAYOUT_BIGBIRD", dict(p0=1, p1=1, p2=1, p3=3, seed=1236))),
    ("local_bertlarge", "bf16", 4, 16, 16384, ("local", dict(left=8, right=8)), ("LAYOUT_LOCAL", dict(p0=8, p1=8))),
    ("full_bertlarge", "bf16", 32, 16, 1024, ("full", dict()), ("LAYOUT_FULL", dict())),
]


@pytest.mark.parametrize("name,dtype,B,H,L,orc,dev", FULL, ids=[c[0] for c in FULL])
def test_benchmark_configs_full_size(sfb, oracle, name, dtype, B, H, L, orc, dev):
    """Full-size runs of benchmark configurations 2-5: oracle parity on (batch, head) slices, and
    properties that do not need the oracle at full size -- rows of P sum to 1 (V = 1 gives O = 1),
    linearity in V, and agreement of the fused kernel with the unfused three-kernel pipeline."""
    nb, d = L // 64, 64
    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), 1, nb, 64, **dev[1])
    luts = oracle.lut_build(oracle.layout(orc[0], 1, nb, **orc[1]))
    assert np.array_equal(lay.nn_lut.cpu().numpy().astype(np.uint32), luts["nn"])
    gen = torch.Generator(device="cuda").manual_seed(99)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=gen).to(TD[dtype]) for _ in range(3))
    scale = 0.125
    o = sfb.fused_attention(q, k, v, lay, scale)
    assert sfb.device_status() == 0
    assert bool(torch.isfinite(o.float()).all())
    for (b, h) in [(0, 0), (B - 1, H - 1), (B // 2, 5)]:
        _check_slice(sfb, oracle, lay, luts, q, k, v, o, b, h, scale)
    # softmax rows sum to 1
    ones = torch.ones_like(v)
    o1 = sfb.fused_attention(q, k, ones, lay, scale).float()
    assert float((o1 - 1.0).abs().max()) < 1e-3 + 2 ** -8
    # the same bar without the 16-bit pack of O in the way: fp32 probabilities of the tensor-core SDDMM + softmax kernel on the
    # same operands, one batch element at full length, every row summed over its kept blocks
    pf = sfb.fused_sddmm_softmax(q[:1].contiguous(), k[:1].contiguous(), lay, scale, torch.float32)
    row_sums = torch.zeros(H, L, device="cuda", dtype=torch.float32)
    rows_of = (lay.nt_lut[0, :, 0].long() * 64).view(-1, 1) + torch.arange(64, device="cuda").view(1, -1)
    row_sums.index_add_(1, rows_of.reshape(-1), pf[0].sum(-1).reshape(H, -1))
    assert float((row_sums - 1.0).abs().max()) < 1e-3
    del pf, row_sums
    # linearity in V
    v2 = torch.randn(B, L, H, d, device="cuda", generator=gen).to(TD[dtype])
    o2 = sfb.fused_attention(q, k, v2, lay, scale).float()
    o12 = sfb.fused_attention(q, k, (v.float() + v2.float()).to(TD[dtype]), lay, scale).float()
    assert float((o12 - (o.float() + o2)).abs().max()) <= 3 * REL * float(o12.abs().max())
    del o1, o2, o12, v2, ones
    # fused against unfused on one batch element (S and P make the round trip through HBM there)
    qb, kb, vb = q[:1].contiguous(), k[:1].contiguous(), v[:1].contiguous()
    s = sfb.bst_sgemm_nt(qb, kb, lay, torch.bfloat16)
    p = sfb.masked_softmax(s, lay, scale, torch.bfloat16)
    ou = sfb.bst_sgemm_xn(p, vb, lay).float()
    assert float((ou - o[:1].float()).abs().max()) <= 2 * REL * float(ou.abs().max())


# --------------------------------------------------------------------------------------------
# the unfused operators on the tensor cores (16-bit operands, 64x64 blocks, 64-wide heads)
def _random_layout(H, nb, per_head, seed, empty_rows=()):
    rng = np.random.RandomState(seed)
    layout = np.zeros((H, nb, nb), np.uint8)
    rows = [i for i in range(nb) if i not in empty_rows]
    cells = [(i, j) for i in rows for j in range(nb)]
    for h in range(H):
        for idx in rng.choice(len(cells), per_head, replace=False):
            layout[h][cells[idx]] = 1
    return layout


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("out", ["f32", "bf16"])
@pytest.mark.parametrize("H_lut,nb,per_head,empty", [(1, 5, 11, ()), (3, 6, 9, (1, 4)), (1, 40, 70, ())])
def test_sddmm_on_tensor_cores(sfb, oracle, dtype, out, H_lut, nb, per_head, empty):
    B, H, d = 2, 3, 64
    layout = _random_layout(H_lut, nb, per_head, 5, empty)
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), 64)
    luts = oracle.lut_build(layout)
    q, k, v = (_rand(oracle, (B, nb * 64, H, d), 900 + i, dtype) for i in range(3))
    ref = oracle.attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), luts, 64,
                           np.float32(0.125), want=("s",))["s"]
    s = sfb.bst_sgemm_nt(q, k, lay, {"f32": torch.float32, "bf16": torch.bfloat16}[out])
    assert sfb.device_status() == 0
    tol = 1e-3 * np.sqrt(d) if out == "f32" else np.abs(ref).max() * 2.0 ** -7
    assert np.abs(s.float().cpu().numpy() - ref).max() <= tol


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("H_lut,nb,per_head,empty", [(1, 5, 11, ()), (3, 6, 9, (1, 4)), (1, 40, 70, ()), (1, 1, 1, ())])
def test_spmm_on_tensor_cores(sfb, oracle, dtype, H_lut, nb, per_head, empty):
    B, H, d = 2, 3, 64
    layout = _random_layout(H_lut, nb, per_head, 6, empty)
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), 64)
    luts = oracle.lut_build(layout)
    v = _rand(oracle, (B, nb * 64, H, d), 950, dtype)
    gen = torch.Generator(device="cuda").manual_seed(3)
    p = torch.rand(B, H, lay.blocks, 64, 64, device="cuda", generator=gen).to(TD[dtype])
    o = torch.full_like(v, 5.0)
    o = sfb.bst_sgemm_xn(p, v, lay)
    assert sfb.device_status() == 0
    pn, vn = p.float().cpu().numpy(), v.float().cpu().numpy()
    want = np.zeros_like(vn)
    for h in range(H):
        nt = luts["nt"][h if H_lut > 1 else 0]
        for kk in range(luts["blocks"]):
            i, j = int(nt[kk, 0]), int(nt[kk, 1])
            want[:, i * 64:(i + 1) * 64, h] += np.einsum("brc,bcd->brd", pn[:, h, kk], vn[:, j * 64:(j + 1) * 64, h])
    assert np.abs(o.float().cpu().numpy() - want).max() <= REL * max(1.0, np.abs(want).max())
    for i in empty:
        assert float(o[:, i * 64:(i + 1) * 64].abs().max()) == 0.0


def test_unfused_pipeline_16bit_full_size(sfb, oracle):
    """SDDMM -> softmax -> SpMM, all 16-bit, at the BigBird configuration's full size, against the fused kernel."""
    B, H, L, d = 16, 12, 4096, 64
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_BIGBIRD, 1, L // 64, 64, p0=1, p1=1, p2=1, p3=3, seed=1236)
    gen = torch.Generator(device="cuda").manual_seed(11)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(3))
    s = sfb.bst_sgemm_nt(q, k, lay, torch.bfloat16)
    p = sfb.masked_softmax(s, lay, 0.125, torch.bfloat16)
    o = sfb.bst_sgemm_xn(p, v, lay).float()
    assert sfb.device_status() == 0
    fused = sfb.fused_attention(q, k, v, lay, 0.125).float()
    assert float((o - fused).abs().max()) <= 2 * REL * float(fused.abs().max())


@pytest.mark.parametrize("heads", [1, 37, 148, 213, 226, 300])
def test_fused_attention_item_dealing(sfb, heads):
    """Every row pair of every (batch, head) is computed exactly once whichever way the launch deals its items to the
    CTAs' streams: fewer items than SMs, fewer than streams, just under and just over four rounds of items (where the
    order of dealing changes), and more.  Against the three unfused operators on the same inputs."""
    B, L, d = 1, 1024, 64                 # 8 row pairs per head
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, L // 64, 64, p0=3, p1=4)
    gen = torch.Generator(device="cuda").manual_seed(500 + heads)
    q, k, v = (torch.randn(B, L, heads, d, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(3))
    o = torch.full((B, L, heads, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    sfb.fused_attention(q, k, v, lay, 0.125, out=o)
    assert sfb.device_status() == 0
    s = sfb.bst_sgemm_nt(q, k, lay, torch.bfloat16)
    p = sfb.masked_softmax(s, lay, 0.125, torch.bfloat16)
    ref = sfb.bst_sgemm_xn(p, v, lay).float()
    assert bool(torch.isfinite(o.float()).all())
    assert float((o.float() - ref).abs().max()) <= 2 * REL * float(ref.abs().max())


@pytest.mark.parametrize("dtype,out", [("bf16", "f32"), ("f16", "f16"), ("bf16", "bf16")])
@pytest.mark.parametrize("pred,ctx", [(None, 0), ("MASK_CAUSAL_DIAG", 0), ("MASK_LOCAL", 100)])
def test_fused_sddmm_softmax_on_tensor_cores(sfb, oracle, dtype, out, pred, ctx):
    """fusion_attention1/2/_full/_local/2_64 for 16-bit operands: probabilities against the oracle, rows sum to 1."""
    B, H, nb, d = 2, 3, 9, 64
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_FULL, 1, nb, 64, causal=1)
    luts = oracle.lut_build(oracle.layout("full", 1, nb, causal=1))
    m_np = None
    if pred:
        lay.pack_mask(getattr(sfb, pred), ctx)
        m_np, _ = oracle.mask_pack(luts["nt"], 64, getattr(oracle, pred), ctx)
    q, k, v = (_rand(oracle, (B, nb * 64, H, d), 1000 + i, dtype) for i in range(3))
    ref = oracle.attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), luts, 64,
                           np.float32(0.125), mask_np=m_np, want=("p",))["p"]
    odt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[out]
    p = sfb.fused_sddmm_softmax(q, k, lay, 0.125, odt, use_mask=pred is not None).float().cpu().numpy()
    assert sfb.device_status() == 0
    tol = 2e-3 if out == "f32" else REL
    assert np.abs(p - ref).max() <= tol * ref.max()
    sums = oracle.blocks_to_dense(p, luts["nt"], nb, 64).sum(-1)
    np.testing.assert_allclose(sums, 1.0, atol=1e-3 if out == "f32" else 2e-2)


@pytest.mark.parametrize("nb", [9, 40, 41, 48])
@pytest.mark.parametrize("out", ["f32", "f16", "bf16"])
def test_fused_sddmm_softmax_row_maximum_grows_along_the_row(sfb, oracle, nb, out):
    """Keys whose magnitude grows with position: the running row maximum moves at nearly every key block, so the
    probabilities written early are rescaled by large factors.  Unions of up to 40 key blocks take the single sweep
    that rescales what it wrote, longer ones the double sweep; both sides of that boundary against the oracle."""
    B, H, d = 1, 2, 64
    L = nb * 64
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_FULL, 1, nb, 64)
    luts = oracle.lut_build(oracle.layout("full", 1, nb))
    q, k = (_rand(oracle, (B, L, H, d), 1300 + i, "bf16") for i in range(2))
    ramp = (0.25 + 3.0 * torch.arange(L, device=k.device, dtype=torch.float32) / L).view(1, L, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    qn, kn = q.float().cpu().numpy(), k.float().cpu().numpy()
    ref = oracle.attention(qn, kn, kn, luts, 64, np.float32(0.125), want=("p",))["p"]
    odt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[out]
    p = sfb.fused_sddmm_softmax(q, k, lay, 0.125, odt).float().cpu().numpy()
    assert sfb.device_status() == 0
    tol = 2e-3 if out == "f32" else REL
    assert np.abs(p - ref).max() <= tol * ref.max()
    sums = oracle.blocks_to_dense(p, luts["nt"], nb, 64).sum(-1)
    np.testing.assert_allclose(sums, 1.0, atol=1e-3 if out == "f32" else 2e-2)


@pytest.mark.parametrize("case", ["lower_interior_subset", "upper_empty", "lower_in_the_middle_only"])
@pytest.mark.parametrize("op", ["probabilities", "attention"])
def test_row_pair_ownership_of_union_entries(sfb, oracle, case, op):
    """A block-row of a pair that owns neither the first nor the last entry of the pair's union of key blocks
    (or no entry at all) still gets its softmax denominator: the tensor-core kernels walk the union, not the row."""
    nb, B, H, d = 4, 2, 2, 64
    layout = np.zeros((1, nb, nb), np.uint8)
    if case == "lower_interior_subset":
        rows = {0: (0, 1, 2), 1: (1,), 2: (0, 3), 3: (2,)}
    elif case == "upper_empty":
        rows = {0: (), 1: (0, 2), 2: (1,), 3: (0, 1, 2, 3)}
    else:
        rows = {0: (0, 1, 2, 3), 1: (2,), 2: (0, 1, 3), 3: (1,)}
    for i, cols in rows.items():
        layout[0, i, list(cols)] = 1
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), 64)
    luts = oracle.lut_build(layout)
    q, k, v = (_rand(oracle, (B, nb * 64, H, d), 1100 + i, "bf16") for i in range(3))
    ref = oracle.attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), luts, 64,
                           np.float32(0.125), want=("p", "o"))
    if op == "probabilities":
        p = sfb.fused_sddmm_softmax(q, k, lay, 0.125, torch.float32).float().cpu().numpy()
        assert sfb.device_status() == 0
        assert np.abs(p - ref["p"]).max() <= 2e-3 * ref["p"].max()
        sums = oracle.blocks_to_dense(p, luts["nt"], nb, 64).sum(-1)
        for i, cols in rows.items():
            np.testing.assert_allclose(sums[:, :, i * 64:(i + 1) * 64], 1.0 if cols else 0.0, atol=1e-3)
    else:
        o = sfb.fused_attention(q, k, v, lay, 0.125).float().cpu().numpy()
        assert sfb.device_status() == 0
        assert np.abs(o - ref["o"]).max() <= REL * np.abs(ref["o"]).max()


def test_host_pipeline_matches_resident_call(sfb):
    """Pinned host operands through the chunked, overlapped pipeline give the result of the resident call."""
    B, L, H, d = 4, 1024, 3, 64
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, L // 64, 64, p0=4, p1=8)
    gen = torch.Generator(device="cuda").manual_seed(21)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(3))
    want = sfb.fused_attention(q, k, v, lay, 0.125)
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq).pin_memory()
    pipe = sfb.HostPipeline(tuple(q.shape), torch.bfloat16, lay, chunks=4)
    for _ in range(2):
        pipe(hq, hk, hv, ho, 0.125)
        torch.cuda.synchronize()
        assert torch.equal(ho, want.cpu())
