"""GPU parity of the element-sparse (CSR) attention path against the CPU oracle, and against the block-sparse path on
patterns both can express.  Tolerances: pattern arrays bit-exact; fp32 outputs max-abs 1e-5; 16-bit 2e-2 relative."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TD = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


@pytest.mark.parametrize("kind,kw,dev,nb,bs", [
    ("stride", dict(band=2, every=4), ("LAYOUT_STRIDE", dict(p0=2, p1=4)), 8, 32),
    ("local", dict(left=1, right=1), ("LAYOUT_LOCAL", dict(p0=1, p1=1)), 5, 64),
    ("full", dict(causal=1), ("LAYOUT_FULL", dict(causal=1)), 4, 32),
])
def test_csr_pattern_from_layout_bit_exact(sfb, oracle, kind, kw, dev, nb, bs):
    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), 1, nb, bs, **dev[1])
    rowptr, colidx = sfb.csr_from_layout(lay)
    wr, wc = oracle.csr_from_layout(oracle.layout(kind, 1, nb, **kw)[0], bs)
    assert np.array_equal(rowptr.cpu().numpy(), wr) and np.array_equal(colidx.cpu().numpy(), wc)


@pytest.mark.parametrize("dtype,d", [("f32", 64), ("f32", 32), ("bf16", 64), ("f16", 128)])
def test_csr_attention_against_oracle_on_an_irregular_pattern(sfb, oracle, dtype, d):
    """Rows of very different lengths, one empty row, unsorted columns."""
    B, L, H = 2, 200, 3
    rng = np.random.RandomState(5)
    rows = []
    for i in range(L):
        n = 0 if i == 7 else int(rng.randint(1, 90 if i % 5 else 200))
        rows.append(rng.choice(L, size=n, replace=False).astype(np.int32))
    rowptr = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
    colidx = np.concatenate(rows).astype(np.int32)
    q, k, v = (torch.from_numpy(oracle.fill_normal((B, L, H, d), 500 + i)).cuda().to(TD[dtype]) for i in range(3))
    o, bad = sfb.csr_attention(q, k, v, torch.from_numpy(rowptr).cuda(), torch.from_numpy(colidx).cuda(), 0.125)
    assert int(bad.item()) == 0
    want = oracle.csr_attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), rowptr, colidx, np.float32(0.125))
    got = o.float().cpu().numpy()
    if dtype == "f32":
        assert np.abs(got - want).max() < 1e-5
    else:
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    assert float(np.abs(got[:, 7]).max()) == 0.0


def test_csr_attention_equals_block_sparse_attention(sfb, oracle):
    """The same pattern through both formats: CSR of a block layout against the fused block-sparse kernel."""
    B, H, d, bs, nb = 2, 4, 64, 64, 16
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, nb, bs, p0=4, p1=8)
    rowptr, colidx = sfb.csr_from_layout(lay)
    q, k, v = (torch.from_numpy(oracle.fill_normal((B, nb * bs, H, d), 510 + i)).cuda() for i in range(3))
    a, _ = sfb.csr_attention(q, k, v, rowptr, colidx, 0.125)
    b = sfb.fused_attention(q, k, v, lay, 0.125)
    assert float((a - b).abs().max()) < 2e-5


def test_csr_columns_outside_the_sequence_are_counted_not_read(sfb):
    L, d = 8, 32
    q = torch.ones(1, L, 1, d, device="cuda")
    rowptr = torch.arange(0, 2 * L + 1, 2, dtype=torch.int32, device="cuda")
    colidx = torch.tensor([0, 1] * L, dtype=torch.int32, device="cuda")
    colidx[3], colidx[10] = -5, L
    o, bad = sfb.csr_attention(q, q, q, rowptr, colidx, 1.0)
    assert int(bad.item()) == 2
    assert torch.allclose(o, torch.ones_like(o), atol=1e-4)
